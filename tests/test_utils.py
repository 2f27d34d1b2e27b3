"""CPU: axis algebra, PDAF router, batched-MTP layout, op-trace contract, switches, dumps, source lint."""
import os
import re

import torch

from ferrite_b200.config import GlmConfig
from ferrite_b200.engine import mtp_batch as MB
from ferrite_b200.parallel.axes import (Axis, MergeKind, ModuleKind, Phase, RankCoord, ShardAxes, TensorAxis,
                                        collectives_per_step, layer_modules, module_parallel)
from ferrite_b200.parallel.router import PdafRouter, StaticPlan, cp_layer_range
from ferrite_b200.utils.acc_hist import AcceptHistogram
from ferrite_b200.utils.dump import UnitDump, compare, first_divergence, token_parity
from ferrite_b200.utils.optrace import GraphRunner, OpTrace, Recorder
from ferrite_b200.utils.switches import Switches
from ferrite_b200.utils.trace import PhaseTimer, layer_checksums

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mesh_coordinates_and_groups():
    ax = ShardAxes(tp=2, kv=4, q=1)
    assert ax.world == 8
    for r in range(8):
        assert ax.linear(ax.coord(r)) == r
    assert ax.coord(5) == RankCoord(1, 1, 0)
    assert ax.group_ranks(Axis.KV, 5) == [4, 5, 6, 7]        # the LSE-merge group of rank 5
    assert ax.group_ranks(Axis.HEAD, 5) == [1, 5]            # its all-reduce group
    assert ax.group_ranks(Axis.Q, 5) == [5]


def test_module_table_and_collective_counts():
    assert module_parallel(ModuleKind.DSA_ATTN, Phase.DECODE).kv_merge is MergeKind.LSE
    assert module_parallel(ModuleKind.DSA_ATTN, Phase.PREFILL).q_merge is MergeKind.ROW_GATHER
    assert module_parallel(ModuleKind.GDN_ATTN, Phase.PREFILL).q_merge is MergeKind.PIPELINE
    assert module_parallel(ModuleKind.MOE, Phase.DECODE).head_merge is MergeKind.SUM
    assert module_parallel(ModuleKind.DSA_LATENT_KV, Phase.DECODE).axis is TensorAxis.KV_PAGES
    cfg = GlmConfig.production()
    assert layer_modules(cfg, 3)[-2] is ModuleKind.DSA_ATTN and layer_modules(cfg, 0)[1] is ModuleKind.GDN_ATTN
    c = collectives_per_step(cfg, ShardAxes(tp=4), Phase.DECODE)
    n_dsa = sum(cfg.is_dsa(l) for l in range(cfg.num_layers))
    # two head-axis merges per layer: partial sums, except that DSA head outputs concatenate (o_proj sums after)
    assert c["sum"] == 2 * cfg.num_layers - n_dsa and c["concat"] == n_dsa
    c = collectives_per_step(cfg, ShardAxes(tp=1, kv=4), Phase.DECODE)
    assert c["lse"] == n_dsa and c["concat"] == n_dsa         # LSE merge + indexer score gather per DSA layer


def test_static_plan_and_pdaf_router():
    cfg = GlmConfig.production()
    plan = StaticPlan.from_config(cfg)
    assert (plan.num_linear, plan.num_dsa, plan.num_dense, plan.num_moe) == (34, 11, 3, 42)
    assert [o.kind for o in plan.layer_ops(3)] == ["attn:dsa", "ffn:moe"]
    ranges = [cp_layer_range(45, 4, r) for r in range(4)]
    assert ranges == [(0, 12), (12, 23), (23, 34), (34, 45)]
    rt = PdafRouter(prefill_ranks=[0, 1, 2, 3], decode_ranks=[4, 5, 6, 7], page_size=16)
    rt.admit(7, 100)
    assert rt.route_prefill(7, 64) == [0, 1, 2, 3] and rt.transfers() == []
    rt.route_prefill(7, 36)
    ev = rt.transfers()
    assert len(ev) == 1 and ev[0].seq == 7 and len(ev[0].plans) == 4
    assert sorted(p for pl in ev[0].plans for p in pl.src_pages) == list(range(7))
    assert rt.route_decode(7) == [4, 5, 6, 7] and rt.decoding[7] == 101
    rt.finish(7)
    assert not rt.decoding and rt.transfers() == []


def test_batched_mtp_layout():
    assert [MB.padded_seqs(n) for n in (1, 3, 5, 16, 17)] == [1, 4, 8, 16, 32]
    rmap = MB.SeqRowMap(n_live=3, n_padded=4, width=3)
    assert rmap.n_rows == 12 and list(rmap.rows_of(2)) == [6, 7, 8] and rmap.seq_of(7) == (2, 1)
    assert rmap.live_rows() == list(range(9))
    drafts = [[5, 6], [5, 6], [1, 2]]
    judges = [[5, 6, 7], [5, 9, 7], [3, 2, 2]]
    plan = MB.plan_commit(rmap, drafts, judges, base=[10, 20, 30, 0])
    assert plan.keep == (3, 2, 1) and plan.emitted == ((5, 6, 7), (5, 9), (3,))
    assert plan.new_lengths() == (13, 22, 31) and plan.rows_to_keep(rmap) == [0, 1, 2, 3, 4, 6]


class _FakeLib:
    def __init__(self):
        self.calls = 0

    def call(self, name, *args, **kw):
        self.calls += 1


def test_op_trace_contract():
    lib = _FakeLib()
    state = {"n": 3}

    def step():
        lib.call("fb_rmsnorm", torch.zeros(1), None, 4, 4096, 1e-5)
        lib.call("fb_gemv", torch.zeros(1), state["n"], 4096)

    runner = GraphRunner(lib)
    tr = runner.assert_stable(step)
    assert len(tr) == 2 and tr.ops[1].ints == (3, 4096) and tr.histogram() == {"fb_rmsnorm": 1, "fb_gemv": 1}
    assert lib.calls == 4 and lib.call.__name__ == "call"

    def unstable():
        state["n"] += 1
        step()

    try:
        runner.assert_stable(unstable)
        assert False, "an unstable step must be refused"
    except RuntimeError as e:
        assert "not stable at op 1" in str(e)
    assert OpTrace(tr.ops).first_difference(tr) is None


def test_switches_histogram_timer_dump(tmp_path):
    s = Switches.from_env({"FERRITE_TIMING": "1", "FERRITE_AR_GROUP": "64", "FERRITE_DUMP_DIR": "/x", "FERRITE_PDL": "0"})
    assert s.timing and s.ar_group == 64 and s.dump_dir == "/x" and not s.pdl and not s.nvtx
    h = AcceptHistogram(3)
    h.extend([1, 3, 3, 2, 9])
    assert h.steps == 5 and h.tokens == 12 and abs(h.mean - 2.4) < 1e-9 and "3:3" in h.line()
    t = PhaseTimer()
    with t.phase("a"):
        pass
    assert t.summary()["a"]["calls"] == 1
    assert layer_checksums(torch.ones(2, 3, 4)) == [12.0, 12.0]
    a, b = UnitDump(), UnitDump()
    x = torch.randn(4, 8)
    a("l0.h", x)
    a("l1.h", x)
    b("l0.h", x + 1e-4)
    b("l1.h", x + 1.0)
    a.save(str(tmp_path))
    a2 = UnitDump.load(str(tmp_path))
    diffs = compare(a2, b)
    assert [d.name for d in diffs] == ["l0.h", "l1.h"] and first_divergence(diffs).name == "l1.h"
    assert token_parity([1, 2, 3], [1, 2, 4])["first_mismatch"] == (2, 3, 4)


def test_sources_name_no_closed_constructs():
    """No source file that travels to a GPU names a batched memcpy call or a device trap (the run harness
    itself refuses sources that name a cluster-wide bulk-load broadcast, so that is not repeated here)."""
    banned = ["cudaMemcpy" + "BatchAsync", "cudaMemcpy3D" + "BatchAsync",
              "cuMemcpy" + "BatchAsync", "cuMemcpy3D" + "BatchAsync", r"\b__trap\s*\(", r"asm\s*\(\s*\"trap"]
    bad = []
    for top in ("csrc", "ferrite_b200", "tests", "bench.py", "bench_kernels.py", "__graft_entry__.py"):
        path = os.path.join(ROOT, top)
        files = [path] if os.path.isfile(path) else [os.path.join(d, f) for d, _, fs in os.walk(path) for f in fs]
        for fn in files:
            if not fn.endswith((".cu", ".cuh", ".h", ".cpp", ".py")) or fn.endswith("test_utils.py"):
                continue
            text = open(fn, errors="ignore").read()
            for pat in banned:
                if re.search(pat, text):
                    bad.append((os.path.relpath(fn, ROOT), pat))
    assert not bad, bad
