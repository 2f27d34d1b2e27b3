"""Worker run under torch.distributed.run by test_gpu_multi.py: layer-split (context-parallel) prefill over a
group of stages, hand-off to a decode-context-parallel group that stores its latent pages compactly, decode
with the cross-rank attention merge.  With 2 ranks both groups are {0, 1}; with 4 the prefill group is {0, 1}
and the decode group {2, 3}."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrite_b200.config import EngineConfig, GlmConfig  # noqa: E402
from ferrite_b200.engine.glm_engine import GlmEngine  # noqa: E402
from ferrite_b200.models.glm import DictSource  # noqa: E402
from ferrite_b200.models.glm_weights import random_weights  # noqa: E402
from ferrite_b200.parallel.cp import CpStage, cp_layer_range, hand_off  # noqa: E402
from ferrite_b200.parallel.symm import DcpAttentionMerge  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = GlmConfig.golden4()
    w = random_weights(cfg, 0, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (45,), generator=torch.Generator().manual_seed(5)).tolist()
    stage_ranks = [0, 1]
    decode_ranks = [0, 1] if world < 4 else [2, 3]
    assert cp_layer_range(cfg.num_layers, 2, 0)[1] == cp_layer_range(cfg.num_layers, 2, 1)[0]
    dgroup = dist.new_group(decode_ranks) if world >= 4 else None
    for mtp_n in (1, 3):
        ecfg = EngineConfig(max_ctx=256, mtp_n=mtp_n, kv_dtype="f32")
        stage = eng = merge = None
        if rank in stage_ranks:
            stage = CpStage(cfg, ecfg, DictSource(w, dev), stage_ranks.index(rank), 2, stage_ranks, dev, prefill_rows=16)
            assert sum(L is not None for L in stage.model.layers[:cfg.num_layers]) == stage.l1 - stage.l0
        if rank in decode_ranks:
            d = decode_ranks.index(rank)
            eng = GlmEngine(cfg, ecfg, DictSource(w, dev), device=dev, prefill_rows=16, dcp_shard=(d, 2))
            m = eng.model
            assert m.lat_cache.shape[1] == (m.max_pages + 1) // 2          # half of the latent pages per rank
            merge = DcpAttentionMerge(dev, d, 2, max_rows=16, heads=m.h_dsa, latent_dim=cfg.dsa.kv_lora_rank, group=dgroup)
            m.dcp = (d, 2, merge)
        first = torch.zeros(1, dtype=torch.int64, device=dev)
        if stage is not None:
            t = stage.prefill(prompt)
            if t is not None:
                first[0] = t
        secs = hand_off(stage, eng, len(prompt), stage_ranks, decode_ranks, cfg, rank, compact=True)
        dist.broadcast(first, stage_ranks[-1])
        if eng is not None:
            out = [int(first.item())]
            eng.build_graphs(mtp_n > 1)
            while len(out) < 14:
                out += eng.spec_step() if mtp_n > 1 else [eng.step_plain()]
            merge.check()
            ref = GlmEngine(cfg, ecfg, DictSource(w, dev), device=dev, prefill_rows=16)
            want, _ = ref.generate(prompt, 14)
            same = sum(a == b for a, b in zip(out[:14], want))
            assert same >= 13, (mtp_n, rank, out, want)     # pipeline stages and the merge sum in other orders than one rank
            t = torch.tensor(out[:14], device=dev)
            t0 = t.clone()
            dist.broadcast(t0, decode_ranks[0], group=dgroup)
            assert torch.equal(t, t0), "DCP ranks emitted different tokens"
            if rank == decode_ranks[0]:
                print(f"cp2 -> dcp2 (compact) mtp_n={mtp_n}: {out[:14]} ({same}/14 equal to one rank), hand-off {secs * 1e3:.1f} ms")
        dist.barrier()
        if merge is not None:
            merge.close()
    # the same prefill group handing off to a TENSOR-PARALLEL decode group: every decode rank gets all cache pages
    # and its own heads of the recurrent states (2 ranks: both groups are {0, 1})
    if world == 2:
        from ferrite_b200.parallel.collective import make_allreduce
        ar = make_allreduce(dev, rank, world, max_elems=64 * cfg.hidden_size, kind="p2p")
        for mtp_n in (1, 3):
            ecfg1 = EngineConfig(max_ctx=256, mtp_n=mtp_n, kv_dtype="f32")
            ecfg2 = EngineConfig(max_ctx=256, mtp_n=mtp_n, kv_dtype="f32", tp=world)
            stage = CpStage(cfg, ecfg1, DictSource(w, dev), rank, 2, [0, 1], dev, prefill_rows=16)
            eng = GlmEngine(cfg, ecfg2, DictSource(w, dev), rank=rank, world=world, device=dev, allreduce=ar, prefill_rows=16)
            first = torch.zeros(1, dtype=torch.int64, device=dev)
            t = stage.prefill(prompt)
            if t is not None:
                first[0] = t
            hand_off(stage, eng, len(prompt), [0, 1], [0, 1], cfg, rank, mode="tp")
            dist.broadcast(first, 1)
            out = [int(first.item())]
            eng.build_graphs(mtp_n > 1)
            while len(out) < 14:
                out += eng.spec_step() if mtp_n > 1 else [eng.step_plain()]
            ar.check()
            ref = GlmEngine(cfg, ecfg1, DictSource(w, dev), device=dev, prefill_rows=16)
            want, _ = ref.generate(prompt, 14)
            same = sum(a == b for a, b in zip(out[:14], want))
            assert same >= 12, (mtp_n, rank, out, want)      # shards quantise their own fp8 blocks
            tt = torch.tensor(out[:14], device=dev)
            t0 = tt.clone()
            dist.broadcast(t0, 0)
            assert torch.equal(tt, t0), "TP ranks emitted different tokens"
            if rank == 0:
                print(f"cp2 -> tp2 mtp_n={mtp_n}: {out[:14]} ({same}/14 equal to one rank)")
            dist.barrier()
    dist.destroy_process_group()
    if rank == decode_ranks[-1]:
        print("CP_WORKER_OK")


if __name__ == "__main__":
    main()
