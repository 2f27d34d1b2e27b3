"""Worker run under torch.distributed.run by test_gpu_multi.py (one process per GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrite_b200.config import EngineConfig, GlmConfig  # noqa: E402
from ferrite_b200.engine.glm_engine import GlmEngine  # noqa: E402
from ferrite_b200.models.glm import DictSource  # noqa: E402
from ferrite_b200.models.glm_weights import random_weights  # noqa: E402
from ferrite_b200.parallel.symm import CrossRankArgmax, FusedGemmAllReduce, FusedGemvAllReduce, P2PAllReduce  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ar = P2PAllReduce(dev, rank, world, max_elems=64 * 4096)
    ar.fused = FusedGemvAllReduce(dev, rank, world)
    ar.argmax = CrossRankArgmax(dev, rank, world)
    # 1. one-shot all-reduce == NCCL all-reduce, bit-identical across ranks, eager and in a graph
    for n in (4096, 3 * 4096, 16 * 4096 + 8, 64 * 4096):
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        for it in range(3):
            x = torch.randn(n, device=dev, generator=g)
            want = x.clone()
            dist.all_reduce(want)
            got = x.clone()
            ar(got)
            torch.cuda.synchronize()
            ar.check()
            assert torch.allclose(got, want, atol=1e-4, rtol=1e-5), (n, it, (got - want).abs().max().item())
            ref = got.clone()
            dist.broadcast(ref, 0)
            assert torch.equal(ref, got), "ranks disagree bitwise"
    buf = torch.ones(4096, device=dev) * (rank + 1)
    ar(buf)  # warm-up outside capture
    buf.fill_(rank + 1)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ar(buf)
    total = world * (world + 1) / 2
    for it in range(4):
        buf.fill_(rank + 1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.all(buf == total), (it, buf[:4])
    ar.check()
    # 1b. fused GEMV + all-reduce == GEMV then NCCL all-reduce (eager and replayed in a graph)
    from ferrite_b200 import _lib
    from ferrite_b200.models.glm import Act
    K = _lib.lib()
    for (N, Kd, m) in ((4096, 4096, 3), (4096, 1024, 8), (5120, 512, 1)):
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        W = (torch.randn(N, Kd, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        x = Act(dev, 8, Kd)
        x.f.copy_(torch.randn(8, Kd, device=dev, generator=g))
        K.call("fb_split_rows", x.f, Kd, *x.sp(3), 8, Kd)
        want = (x.f[:m].double() @ W.double().t()).float()
        dist.all_reduce(want)
        y = torch.zeros(8, N, device=dev)
        ar.fused(W, None, x.s, Kd, x.plane, y, N, m, N, Kd, False, True, None)
        torch.cuda.synchronize()
        ar.check()
        err = (y[:m] - want).abs().max().item()
        assert err < 2e-2 * max(1.0, want.abs().max().item()), (N, Kd, m, err)
        ref = y.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, y), "fused all-reduce: ranks disagree bitwise"
        graph = torch.cuda.CUDAGraph()
        y2 = torch.zeros(8, N, device=dev)
        with torch.cuda.graph(graph):
            ar.fused(W, None, x.s, Kd, x.plane, y2, N, m, N, Kd, False, True, None)
        for it in range(3):
            y2.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y2, y), (N, Kd, m, it)
        ar.check()
    # 1b'. fused prefill GEMM (tcgen05) + two-shot all-reduce == GEMM then NCCL all-reduce, bitwise equal on all
    # ranks, eager and replayed in a graph, with and without a local addend
    for mode, (N, Kd, m, acc) in [(md, c) for md in (1, 2) for c in ((4096, 1024, 256, False), (4096, 512, 100, True),
                                                                    (1024, 256, 37, False), (512, 128, 16, False))]:
        gar = FusedGemmAllReduce(dev, rank, world, max_rows=256, n_max=4096, mode=mode)   # one-shot, then two-shot
        assert gar.fits(m, N), (m, N, gar.plan(m, N))
        g = torch.Generator(device=dev).manual_seed(31 + rank)
        W = (torch.randn(N, Kd, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        xb = torch.randn(m, Kd, device=dev, generator=g).to(torch.bfloat16)
        add = torch.randn(m, N, device=dev, generator=g) if acc else torch.zeros(m, N, device=dev)
        want = (xb.double() @ W.double().t()).float() + add
        dist.all_reduce(want)
        y = add.clone()
        gar(W, xb, Kd, y, N, m, N, Kd, acc)
        torch.cuda.synchronize()
        gar.check()
        err = (y - want).abs().max().item()
        assert err < 2e-3 * max(1.0, want.abs().max().item()), ("gemm_ar", N, Kd, m, err)
        ref = y.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(ref, y), "fused GEMM all-reduce: ranks disagree bitwise"
        graph = torch.cuda.CUDAGraph()
        y2 = add.clone()
        gar(W, xb, Kd, y2, N, m, N, Kd, acc)      # warm-up outside capture (keeps the epochs of all ranks aligned)
        with torch.cuda.graph(graph):
            gar(W, xb, Kd, y2, N, m, N, Kd, acc)
        for it in range(3):
            y2.copy_(add)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y2, y), ("gemm_ar graph", mode, N, Kd, m, it)
        gar.check()
        gar.close()
    # 1c. vocab-sliced argmax merged across ranks == argmax of the full row (first maximum wins)
    V, n = 4096 * world, 5
    full = torch.randn(n, V, device=dev, generator=torch.Generator(device=dev).manual_seed(11))
    full[1, 17] = full[1, V - 3] = 60.0      # a tie across slices: the lower index wins
    full[2, V - 1] = 70.0
    vl = V // world
    mine = full[:, rank * vl:(rank + 1) * vl].contiguous()
    part = torch.zeros(n * 64, dtype=torch.int64, device=dev)
    ids = torch.zeros(n, dtype=torch.int32, device=dev)
    vals = torch.zeros(n, device=dev)
    for it in range(3):
        ar.argmax(mine, vl, part, n, vl, rank * vl, ids, 1, vals)
        torch.cuda.synchronize()
        ar.check()
        from ferrite_b200.ops.reference import argmax_first
        assert ids.tolist() == argmax_first(full.cpu()).tolist(), (it, ids.tolist())
        assert torch.equal(vals.cpu(), full.max(-1).values.cpu())
    # 1d. expert-parallel MoE (all-to-all dispatch / combine) == all experts applied to this rank's own rows
    from ferrite_b200.ops import reference as R
    from ferrite_b200.parallel.ep import EpMoE
    H_, I_, E_, topk_ = 256, 128, 4 * world, 2
    gw = torch.Generator().manual_seed(21)
    w13f = torch.randn(E_, 2 * I_, H_, generator=gw) * 0.05
    w2f = torch.randn(E_, H_, I_, generator=gw) * 0.05
    q13 = [R.quant_fp8_block(w13f[e]) for e in range(E_)]
    q2 = [R.quant_fp8_block(w2f[e]) for e in range(E_)]
    el = E_ // world
    mine = range(rank * el, (rank + 1) * el)
    w13 = torch.stack([q13[e][0] for e in mine]).to(dev)
    s13 = torch.stack([q13[e][1] for e in mine]).to(dev)
    w2 = torch.stack([q2[e][0] for e in mine]).to(dev)
    s2 = torch.stack([q2[e][1] for e in mine]).to(dev)
    # few rows: per-pair tensor-core kernels between dispatch and combine; 40 rows per rank: the gathered pairs are
    # sorted by local expert and run through the grouped tcgen05 GEMM
    for n_max_, cases in ((4, (3, 4, 1)), (40, (40, 17))):
        ep = EpMoE(dev, rank, world, n_max_, H_, topk_, I_)
        assert (world * n_max_ * topk_ >= ep.tc_pairs) == (n_max_ == 40)
        for it, n_loc in enumerate(cases):
            gx = torch.Generator().manual_seed(100 * it + rank)
            xa = Act(dev, n_max_, H_)
            xa.f[:n_loc].copy_(torch.randn(n_loc, H_, generator=gx))
            K.call("fb_split_rows", xa.f, H_, *xa.sp(3), n_max_, H_)
            ids = torch.stack([torch.randperm(E_, generator=gx)[:topk_] for _ in range(n_loc)]).to(torch.int32).to(dev)
            wts = torch.rand(n_loc, topk_, generator=gx).to(dev)
            add = torch.randn(n_max_, H_, generator=gx).to(dev)
            y = torch.zeros(n_max_, H_, device=dev)
            ep.forward(xa.s, xa.plane, ids, wts, n_loc, w13, s13, w2, s2, el, 7.0, y, add)
            torch.cuda.synchronize()
            ep.check()
            want = add[:n_loc].cpu().clone()
            xc = xa.f[:n_loc].cpu()
            for r in range(n_loc):
                for s_ in range(topk_):
                    e = int(ids[r, s_])
                    gu = xc[r] @ R.dequant_fp8_block(*q13[e]).t()
                    h = R.swiglu_limited(gu[:I_], gu[I_:], 7.0) * float(wts[r, s_])
                    want[r] += h @ R.dequant_fp8_block(*q2[e]).t()
            err = (y[:n_loc].cpu() - want).abs().max().item()
            assert err < 3e-2 * max(1.0, want.abs().max().item()), (it, n_loc, err)
        ep.close()
    # 2. tensor-parallel engine == single-rank engine, token for token (greedy and MTP).  At more than two ranks the
    # slices of these toy models are a few columns wide: every shard quantises its own fp8 blocks, the logits of a
    # random model sit close together, and greedy tokens part early although each engine is right (the production
    # shapes are compared token by token at every rank count by bench.py, "tokens_match_tp1").  There the check is
    # greedy == speculative, all ranks bitwise equal, and the first token after the 29-token prefill.
    agree = 10 if world == 2 else 1
    for name in ("tiny", "golden4"):
        cfg = getattr(GlmConfig, name)()
        w = random_weights(cfg, 0, std=0.05)
        prompt = torch.randint(0, cfg.vocab_size, (29,), generator=torch.Generator().manual_seed(1)).tolist()
        outs = {}
        for mtp_n in (1, 3):
            ecfg = EngineConfig(max_ctx=256, mtp_n=mtp_n, kv_dtype="f32", tp=world)
            eng = GlmEngine(cfg, ecfg, DictSource(w, dev), rank=rank, world=world, device=dev, allreduce=ar,
                            prefill_rows=16)
            outs[mtp_n], _ = eng.generate(prompt, 14)
            ar.check()
        assert outs[1] == outs[3], (name, outs)
        # routed experts split by expert instead of by intermediate columns: whole experts per rank are quantised
        # exactly like the single-rank engine's, so the tokens agree with the column-split run up to fp8 block effects
        if cfg.n_routed_experts % world == 0:
            ecfg = EngineConfig(max_ctx=256, mtp_n=3, kv_dtype="f32", tp=world, moe_shard="expert")
            eng = GlmEngine(cfg, ecfg, DictSource(w, dev), rank=rank, world=world, device=dev, allreduce=ar,
                            prefill_rows=16)
            by_expert, _ = eng.generate(prompt, 14)
            ar.check()
            same = sum(a == b for a, b in zip(by_expert, outs[1]))
            assert same >= agree and by_expert[0] == outs[1][0], (name, "expert-sharded", by_expert, outs[1])
        t = torch.tensor(outs[1], device=dev)
        t0 = t.clone()
        dist.broadcast(t0, 0)
        assert torch.equal(t, t0), "ranks emitted different tokens"
        if rank == 0:
            e1 = GlmEngine(cfg, EngineConfig(max_ctx=256, mtp_n=1, kv_dtype="f32"), DictSource(w, dev), device=dev,
                           prefill_rows=16)
            single, _ = e1.generate(prompt, 14)
            # shards quantise their own fp8 blocks, so a rare late divergence is tolerated:
            same = sum(a == b for a, b in zip(single, outs[1]))
            assert same >= agree and single[0] == outs[1][0], (name, single, outs[1])
            print(f"{name}: tp{world} tokens {outs[1]} (tp1 agreement {same}/14)")
    # 3. DSV41: tensor-parallel engine (heads / groups / expert-inter / engram rows split) == single rank
    from ferrite_b200.engine.dsv41_engine import Dsv41Engine
    from ferrite_b200.models.dsv41 import DictWeights
    from ferrite_b200.models.dsv41_config import Dsv41Config
    from ferrite_b200.models.dsv41_weights import random_weights as d4_weights
    if world == 2:
        cfg = Dsv41Config.tiny()
        w = d4_weights(cfg, 2)
        prompt = [3, 17, 99, 250, 4, 8, 15, 16, 23, 42, 77]
        outs = {}
        for spec in (False, True):
            eng = Dsv41Engine(cfg, DictWeights(w), rank=rank, world=world, device=dev, allreduce=ar, max_ctx=128)
            outs[spec] = eng.generate(prompt, 12, spec=spec)
            ar.check()
        assert outs[False] == outs[True], outs
        t = torch.tensor(outs[False], device=dev)
        t0 = t.clone()
        dist.broadcast(t0, 0)
        assert torch.equal(t, t0), "DSV41 ranks emitted different tokens"
        if rank == 0:
            single = Dsv41Engine(cfg, DictWeights(w), device=dev, max_ctx=128).generate(prompt, 12)
            same = sum(a == b for a, b in zip(single, outs[False]))
            assert same >= 9, (single, outs)
            print(f"dsv41 tiny: tp{world} tokens {outs[False]} (tp1 agreement {same}/12)")
    dist.barrier()
    ar.close()
    # A peer that does not join a launch (it left between steps, with nothing of its own in flight): the waiting
    # rank's bounded poll runs out after a few milliseconds, the kernel returns, the status word names the peer,
    # and the engine-level check raises.  No kernel is made to spin, trap or fault.
    from ferrite_b200.parallel.status import CollectiveTimeout
    ar2 = P2PAllReduce(dev, rank, world, max_elems=4 * 4096, max_spins=400000)   # a wait budget of a few hundred ms
    buf = torch.ones(1, 4096, device=dev)
    torch.cuda.synchronize()
    dist.barrier()                    # the joint launch below must not pay for start-up skew out of that budget
    ar2(buf)
    torch.cuda.synchronize()
    ar2.arena.verify()
    assert float(buf[0, 0]) == world
    dist.barrier()
    if rank == 0:
        ar2(buf)                      # nobody else launches this one
        torch.cuda.synchronize()
        try:
            ar2.arena.verify()
            raise AssertionError("the missing peers went unnoticed")
        except CollectiveTimeout as e:
            assert e.peer == 1 and e.name.startswith("allreduce"), (e.peer, e.name)
            print(f"missing peer detected: {e}")
    dist.barrier()
    ar2.close()
    dist.destroy_process_group()
    if rank == 0:
        print("TP_WORKER_OK")


if __name__ == "__main__":
    main()
