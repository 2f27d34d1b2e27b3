"""Microbenchmarks of the peer-memory collective kernels (run with 2, 4 or 8 ranks):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 bench_collectives.py

Every case is timed with CUDA events around a CUDA graph of `--iters` launches, after warm-up, and
reported as the MAXIMUM over ranks.  For each fused kernel the roofline time is the slower of
(bytes streamed from HBM / measured HBM bandwidth) and (bytes that cross NVLink per GPU / 770 GB/s,
the measured peer-copy bandwidth of this pool); `frac` = roofline / achieved.

Cases
  ar_oneshot.<rows>x4096      one-shot all-reduce (baseline for the fused kernels) vs NCCL all-reduce
  gemv_ar.<site>              GEMV + all-reduce (+ fold) in one kernel vs GEMV, all-reduce, hc_post_mix separately
  gemm_ar.<site>.m<rows>      prefill rows: tcgen05 GEMM + two-shot all-reduce in one kernel vs GEMM, then all-reduce
  argmax_xchg                 vocab-sliced argmax merge
  dcp_merge                   cross-rank LSE merge of attention partials
  ep_moe                      dispatch -> grouped experts -> combine
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def hbm_gbs() -> float:
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def timed(fn, iters: int, warmup: int = 5) -> float:
    """us per call, graph-timed, max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ferrite_b200 import _lib
    from ferrite_b200.models.glm import Act
    from ferrite_b200.parallel.ep import EpMoE
    from ferrite_b200.parallel.symm import (CrossRankArgmax, DcpAttentionMerge, FusedGemmAllReduce, FusedGemvAllReduce,
                                            P2PAllReduce)
    K = _lib.lib()
    hbm = hbm_gbs()
    rows = []

    def add(name, us, hbm_bytes=0, link_bytes=0, note=""):
        roof = max(hbm_bytes / hbm / 1e3, link_bytes / NVLINK_GBS / 1e3)
        rows.append({"case": name, "us": round(us, 2), "roofline_us": round(roof, 2),
                     "frac": round(roof / us, 3) if us > 0 else None, "note": note})

    # ---- all-reduce baselines -------------------------------------------------------------------
    ar = P2PAllReduce(dev, rank, world, max_elems=64 * 4096)
    for m in (1, 3, 16):
        buf = torch.randn(m, 4096, device=dev)
        us = timed(lambda: ar(buf), args.iters)
        link = (world - 1) * m * 4096 * 4          # bytes each GPU pushes to its peers
        add(f"ar_oneshot.{m}x4096", us, 0, link, "peer stores + flag + local reduce")
    for m in (3,):   # NCCL cannot be captured here reliably: eager, event-timed
        buf = torch.randn(m, 4096, device=dev)
        for _ in range(5):
            dist.all_reduce(buf)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            dist.all_reduce(buf)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        add(f"nccl_allreduce.{m}x4096.eager", float(t.item()), 0, (world - 1) * m * 4096 * 4, "library baseline, eager launches")

    # ---- GEMV + all-reduce (+ fold) -----------------------------------------------------------------
    fused = FusedGemvAllReduce(dev, rank, world)
    H, m = 4096, 3
    for site, Kfull in (("gdn_o_proj", 8192), ("dsa_o_proj", 16384), ("shared_down", 2048)):
        Kl = Kfull // world
        reps = max(2, int(300e6 // (H * Kl * 2)) + 1)
        ws = [torch.randn(H, Kl, device=dev, dtype=torch.bfloat16) for _ in range(reps)]
        x = Act(dev, 8, Kl)
        x.f.normal_()
        K.call("fb_split_rows", x.f, Kl, *x.sp(3), 8, Kl)
        y = torch.zeros(8, H, device=dev)
        R0, R1 = torch.randn(8, 4, H, device=dev), torch.zeros(8, 4, H, device=dev)
        post, comb = torch.rand(8, 4, device=dev), torch.rand(8, 16, device=dev)
        fn = torch.randn(24, 4 * H, device=dev) * 0.02
        acc = torch.zeros(8, 25, device=dev)
        st = {"i": 0}

        def fused_fold():
            w = ws[st["i"] % reps]; st["i"] += 1
            fused(w, None, x.s, Kl, x.plane, y, H, m, H, Kl, False, False, (R0, R1, post, comb, fn, acc, 24))

        def fused_ar():
            w = ws[st["i"] % reps]; st["i"] += 1
            fused(w, None, x.s, Kl, x.plane, y, H, m, H, Kl, False, True, None)

        def separate():
            w = ws[st["i"] % reps]; st["i"] += 1
            K.call("fb_gemv_mma_bf16", w, x.s, Kl, x.plane, y, H, m, H, Kl, 0, 0, None, 0, 0, 0)
            ar(y[:m])
            K.call("fb_hc_post_mix", R0, R1, y, post, comb, fn, acc, m, H, 24)
            acc.zero_()

        wbytes = H * Kl * 2
        link = (world - 1) * m * H * 4
        add(f"gemv_ar.{site}.fold", timed(fused_fold, args.iters), wbytes + 24 * 4 * H * 4, link, f"K/rank={Kl}")
        add(f"gemv_ar.{site}.ar_only", timed(fused_ar, args.iters), wbytes, link, "")
        add(f"separate.{site}", timed(separate, args.iters), wbytes + 24 * 4 * H * 4, link, "gemv + all-reduce + hc_post_mix")
    fused.check()

    # ---- prefill GEMM + two-shot all-reduce -----------------------------------------------------------
    gar = FusedGemmAllReduce(dev, rank, world, max_rows=256, n_max=4096, mode=2)    # two-shot
    gar1 = FusedGemmAllReduce(dev, rank, world, max_rows=256, n_max=4096, mode=1)   # one-shot (needs world x the staging)
    tc_status = torch.zeros(4, dtype=torch.int32, device=dev)
    for site, Kfull, M in (("gdn_o_proj", 8192, 256), ("dsa_o_proj", 16384, 256), ("gdn_o_proj", 8192, 64)):
        Kl = Kfull // world
        reps = max(2, int(300e6 // (H * Kl * 2)) + 1)
        ws = [torch.randn(H, Kl, device=dev, dtype=torch.bfloat16) for _ in range(reps)]
        xb = torch.randn(M, Kl, device=dev).to(torch.bfloat16)
        yg = torch.zeros(M, H, device=dev)
        st = {"i": 0}

        def fused_gemm():
            w = ws[st["i"] % reps]; st["i"] += 1
            gar(w, xb, Kl, yg, H, M, H, Kl, False)

        def fused_gemm1():
            w = ws[st["i"] % reps]; st["i"] += 1
            gar1(w, xb, Kl, yg, H, M, H, Kl, False)

        def separate_gemm():
            w = ws[st["i"] % reps]; st["i"] += 1
            K.call("fb_gemm_tc_bf16", w, xb, Kl, yg, H, M, H, Kl, 0, tc_status)
            step = ar.max_elems // H
            for r0 in range(0, M, step):
                ar(yg[r0:min(M, r0 + step)])

        flops_us = 2.0 * M * H * Kl / 1611e12 * 1e6
        link = 2 * (world - 1) * M * H * 4 // world       # reduce-scatter + all-gather volume per GPU
        us_f = timed(fused_gemm, args.iters)
        us_s = timed(separate_gemm, args.iters)
        roof = max(H * Kl * 2 / hbm / 1e3, link / NVLINK_GBS / 1e3, flops_us)
        rows.append({"case": f"gemm_ar.{site}.m{M}.twoshot", "us": round(us_f, 2), "roofline_us": round(roof, 2),
                     "frac": round(roof / us_f, 3), "note": f"K/rank={Kl}; tcgen05 GEMM + two-shot all-reduce, one launch"})
        if world == 2 or (world - 1) * M * H * 4 <= (8 << 20):
            us_1 = timed(fused_gemm1, args.iters)
            roof1 = max(H * Kl * 2 / hbm / 1e3, (world - 1) * M * H * 4 / NVLINK_GBS / 1e3, flops_us)
            rows.append({"case": f"gemm_ar.{site}.m{M}.oneshot", "us": round(us_1, 2), "roofline_us": round(roof1, 2),
                         "frac": round(roof1 / us_1, 3), "note": "every tile pushed to every rank, one publish / wait round"})
        rows.append({"case": f"separate_gemm.{site}.m{M}", "us": round(us_s, 2), "roofline_us": round(roof, 2),
                     "frac": round(roof / us_s, 3), "note": "tcgen05 GEMM, then one-shot all-reduce in 64-row chunks"})
    gar.check()
    gar1.check()

    # ---- cross-rank argmax --------------------------------------------------------------------------
    xa = CrossRankArgmax(dev, rank, world)
    V = 154880 // world
    logits = torch.randn(3, V, device=dev)
    part = torch.zeros(3 * 64, dtype=torch.int64, device=dev)
    ids = torch.zeros(3, dtype=torch.int32, device=dev)
    add("argmax_xchg.3rows", timed(lambda: xa(logits, V, part, 3, V, rank * V, ids), args.iters), 3 * V * 4, (world - 1) * 3 * 8,
        "partial argmax of the vocab slice + exchange")

    # ---- DCP merge -----------------------------------------------------------------------------------
    hl, DL, nsplit, n = 64, 512, 16, 3
    dm = DcpAttentionMerge(dev, rank, world, max_rows=8, heads=hl, latent_dim=DL)
    o_part = torch.randn(n, nsplit, hl, DL, device=dev)
    ml = torch.rand(n, nsplit, hl, 2, device=dev)
    ctx = torch.zeros(n, hl, DL, device=dev)
    add("dcp_merge.64h.3rows", timed(lambda: dm(o_part, ml, ctx, n, hl, DL, nsplit), args.iters),
        n * nsplit * hl * DL * 4, (world - 1) * n * hl * (DL + 4) * 4, "split-K merge + cross-rank LSE merge")
    dm.check()

    # ---- EP MoE ---------------------------------------------------------------------------------------
    Hh, I, E, topk, n_max = 4096, 2048, 8 * world, 8, 4
    el = E // world
    w13 = torch.randint(0, 255, (el, 2 * I, Hh), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    w2 = torch.randint(0, 255, (el, Hh, I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    s13 = torch.rand(el, 2 * I // 128, Hh // 128, device=dev) * 1e-3
    s2 = torch.rand(el, Hh // 128, I // 128, device=dev) * 1e-3
    ep = EpMoE(dev, rank, world, n_max, Hh, topk, I)
    xr = Act(dev, n_max, Hh)
    xr.f.normal_()
    K.call("fb_split_rows", xr.f, Hh, *xr.sp(3), n_max, Hh)
    g = torch.Generator().manual_seed(rank)
    idsr = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(n_max)]).to(torch.int32).to(dev)
    wts = torch.rand(n_max, topk, device=dev)
    yo = torch.zeros(n_max, Hh, device=dev)
    us = timed(lambda: ep.forward(xr.s, xr.plane, idsr, wts, n_max, w13, s13, w2, s2, el, 10.0, yo), max(10, args.iters // 5))
    pairs_here = n_max * topk   # expected (row, slot) pairs served per rank
    add("ep_moe.4rows_per_rank", us, pairs_here * 3 * I * Hh, (world - 1) * n_max * Hh * (2 * 4 + 4),
        "dispatch + gate/up + down + combine; HBM bytes = expected expert weights per rank")
    ep.check()

    if rank == 0:
        print(f"{'case':40s} {'us':>9s} {'roofline':>9s} {'frac':>6s}  note   (world {world}, HBM {hbm:.0f} GB/s, NVLink {NVLINK_GBS:.0f} GB/s)")
        for r in rows:
            print(f"{r['case']:40s} {r['us']:9.2f} {r['roofline_us']:9.2f} {r['frac']!s:>6s}  {r['note']}")
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"world": world, "rows": rows}, f, indent=1)
    dist.barrier()
    for o in (ar, fused, gar, gar1, xa, dm, ep):
        o.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
