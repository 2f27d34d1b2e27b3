#!/usr/bin/env python
"""Per-kernel micro-benchmarks at GLM-5.3-Flash decode shapes, against the HBM roofline.

Each case runs one kernel entry point on weights that rotate through enough distinct
copies to exceed the 126 MB L2, is timed with CUDA events after warm-up, and is reported as
algorithmic bytes / time and as a fraction of the measured copy bandwidth
(MEASURED_PEAKS.json `hbm_gbs`, fallback 6650 GB/s).

  python bench_kernels.py                 # all cases, one table
  python bench_kernels.py --only moe_down # one case (the form used under ncu)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

from ferrite_b200 import _lib  # noqa: E402


def hbm_peak_gbs() -> tuple:
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "of measured"
    return 6650.0, "of fallback"


def split_buf(x: torch.Tensor) -> torch.Tensor:
    M, K = x.shape
    sp = torch.zeros(4, M, K, dtype=torch.int16, device=x.device)
    bh = x.bfloat16(); bl = (x - bh.float()).bfloat16()
    hh = x.half(); hl = (x - hh.float()).half()
    for i, t in enumerate((bh, bl, hh, hl)):
        sp[i] = t.view(torch.int16)
    return sp


def fp8_rand(*shape):
    return (torch.randn(*shape, device="cuda", dtype=torch.bfloat16) * 100).to(torch.float8_e4m3fn)


class Case:
    def __init__(self, name, nbytes, fn, note=""):
        self.name, self.nbytes, self.fn, self.note = name, nbytes, fn, note


def make_cases(K, only):
    cases = []
    dev = "cuda"

    def want(name):
        return only is None or only in name or name in only

    def gemv_case(name, N, Kd, m, fp8=False, mma=True):
        if not want(name):
            return
        esz = 1 if fp8 else 2
        reps = max(2, int(300e6 // (N * Kd * esz)) + 1)
        x = torch.randn(m, Kd, device=dev)
        xs = split_buf(x)
        out = torch.zeros(m, N, device=dev)
        if fp8:
            ws = [fp8_rand(N, Kd) for _ in range(reps)]
            sc = torch.rand((N + 127) // 128, (Kd + 127) // 128, device=dev) * 1e-3
        else:
            ws = [torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) for _ in range(reps)]
        state = {"i": 0}

        def fn():
            w = ws[state["i"] % reps]
            state["i"] += 1
            if mma:
                if fp8:
                    K.call("fb_gemv_mma_fp8", w, sc, xs, Kd, m * Kd, out, N, m, N, Kd, 0, None, 0, 0, 0)
                else:
                    K.call("fb_gemv_mma_bf16", w, xs, Kd, m * Kd, out, N, m, N, Kd, 0, 0, None, 0, 0, 0)
            else:
                if fp8:
                    K.call("fb_gemv_fp8", w, sc, x, Kd, out, N, m, N, Kd, 0, 0)
                else:
                    K.call("fb_gemv_bf16", w, x, Kd, out, N, m, N, Kd, 0, 0)
        cases.append(Case(name, N * Kd * esz, fn, f"N={N} K={Kd} m={m}"))

    def fused_case(name, N, Kd, m, fold, fp8=False):
        """GEMV + (world 1: no collective) + hyper-connection fold in one launch."""
        if not want(name):
            return
        from ferrite_b200.parallel.symm import FusedGemvAllReduce
        esz = 1 if fp8 else 2
        reps = max(2, int(300e6 // (N * Kd * esz)) + 1)
        x = torch.randn(m, Kd, device=dev)
        xs = split_buf(x)
        out = torch.zeros(m, N, device=dev)
        if fp8:
            ws = [fp8_rand(N, Kd) for _ in range(reps)]
            sc = torch.rand((N + 127) // 128, (Kd + 127) // 128, device=dev) * 1e-3
        else:
            ws = [torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) for _ in range(reps)]
            sc = None
        R0, R1 = torch.randn(8, 4, N, device=dev), torch.zeros(8, 4, N, device=dev)
        fns = [torch.randn(24, 4 * N, device=dev) * 0.02 for _ in range(40)]
        acc = torch.zeros(8, 25, device=dev)
        post, comb = torch.rand(8, 4, device=dev), torch.rand(8, 16, device=dev)
        f = FusedGemvAllReduce(torch.device(dev), 0, 1)
        state = {"i": 0}

        def fn():
            i = state["i"]
            state["i"] += 1
            fd = (R0, R1, post, comb, fns[i % 40], acc, 24) if fold else None
            f(ws[i % reps], sc, xs, Kd, m * Kd, out, N, m, N, Kd, False, True, fd)
        cases.append(Case(name, N * Kd * esz + (24 * 4 * N * 4 if fold else 0), fn, f"N={N} K={Kd} m={m} fold={fold}"))

    def tc_gemv_case(name, N, Kd, m, nsplit):
        """TMA + tcgen05 split-K GEMV (decode rows), hi + lo activation planes."""
        if not want(name):
            return
        reps = max(2, int(300e6 // (N * Kd * 2)) + 1)
        x = torch.randn(16, Kd, device=dev)
        xs = split_buf(x)
        out = torch.zeros(m, N, device=dev)
        ws = [torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) for _ in range(reps)]
        tiles = (N + 127) // 128
        part = torch.zeros(tiles * nsplit * 16 * 128, device=dev)
        ticket = torch.zeros(tiles, dtype=torch.int32, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        state = {"i": 0}

        def fn():
            w = ws[state["i"] % reps]
            state["i"] += 1
            K.call("fb_gemv_tc_bf16", w, xs, Kd, 16 * Kd, out, N, m, N, Kd, 0, nsplit, part, ticket, status)
        cases.append(Case(name, N * Kd * 2, fn, f"N={N} K={Kd} m={m} splits={nsplit} CTAs={tiles * nsplit}"))

    for ns in (4, 8, 16):
        tc_gemv_case(f"gemv_tc.gdn_o_proj.m3.s{ns}", 4096, 8192, 3, ns)
    for ns in (1, 2, 3):
        tc_gemv_case(f"gemv_tc.gdn_in.m3.s{ns}", 24896, 4096, 3, ns)
    tc_gemv_case("gemv_tc.lm_head.m3.s1", 154880, 4096, 3, 1)
    tc_gemv_case("gemv_tc.router_shared.m3.s8", 4384, 4096, 3, 8)
    fused_case("gemv_ar.gdn_o_proj.m3.nofold", 4096, 8192, 3, False)
    fused_case("gemv_ar.gdn_o_proj.m3.fold", 4096, 8192, 3, True)
    fused_case("gemv_ar.shared_down.m3.fold", 4096, 2048, 3, True)
    fused_case("gemv_ar.dense_down.m3.fold", 4096, 12288, 3, True, fp8=True)
    gemv_case("gemv_mma_bf16.lm_head.m1", 154880, 4096, 1)
    gemv_case("gemv_mma_bf16.lm_head.m3", 154880, 4096, 3)
    gemv_case("gemv_simt_bf16.lm_head.m3", 154880, 4096, 3, mma=False)
    gemv_case("gemv_mma_bf16.gdn_in.m3", 24896, 4096, 3)
    gemv_case("gemv_mma_bf16.gdn_o_proj.m3", 4096, 8192, 3)
    gemv_case("gemv_simt_bf16.gdn_o_proj.m3", 4096, 8192, 3, mma=False)
    gemv_case("gemv_mma_bf16.dsa_o_proj.m3", 4096, 16384, 3)
    gemv_case("gemv_mma_bf16.dsa_q.m3", 20480, 1536, 3)
    gemv_case("gemv_mma_bf16.router_shared.m3", 4384, 4096, 3)
    gemv_case("gemv_mma_bf16.shared_down.m3", 4096, 2048, 3)
    gemv_case("gemv_mma_fp8.dense_gate_up.m3", 24576, 4096, 3, fp8=True)
    gemv_case("gemv_mma_fp8.dense_down.m3", 4096, 12288, 3, fp8=True)
    gemv_case("gemv_simt_fp8.dense_down.m3", 4096, 12288, 3, fp8=True, mma=False)

    # ---- MoE experts: 3 rows x 8 slots, experts drawn from a pool larger than L2 ----------
    for tag, I, H in (("tp1", 2048, 4096), ("tp8", 256, 4096)):
        if not (want("moe_gate_up") or want("moe_down")):
            break
        E, n, topk = (40 if I == 2048 else 320), 3, 8
        w13 = fp8_rand(E, 2 * I, H)
        s13 = torch.rand(E, 2 * I // 128, H // 128, device=dev) * 1e-3
        w2 = fp8_rand(E, H, I)
        s2 = torch.rand(E, H // 128, I // 128, device=dev) * 1e-3
        x = torch.randn(n, H, device=dev)
        xs = split_buf(x)
        asp = torch.zeros(4, n * topk, I, dtype=torch.int16, device=dev)
        act = torch.zeros(n, topk, I, device=dev)
        out = torch.zeros(n, H, device=dev)
        wts = torch.rand(n, topk, device=dev)
        idsets = [torch.randperm(E, device=dev)[:n * topk].int().view(n, topk).contiguous() for _ in range(8)]
        st = {"i": 0}

        def gu(I=I, H=H, w13=w13, s13=s13, xs=xs, asp=asp, idsets=idsets, st=st, wts=wts):
            ids = idsets[st["i"] % 8]; st["i"] += 1
            K.call("fb_moe_gate_up_mma", w13, s13, xs, H, n * H, ids, wts, asp, I, n * topk * I, n, topk, I, H, 0, E, 10.0)

        def dn(I=I, H=H, w2=w2, s2=s2, asp=asp, idsets=idsets, st=st, out=out):
            ids = idsets[st["i"] % 8]; st["i"] += 1
            K.call("fb_moe_down_mma", w2, s2, asp, I, n * topk * I, ids, out, H, n, topk, I, H, 0, E, 0, None, 0, 0, 0)

        def gu_simt(I=I, H=H, w13=w13, s13=s13, x=x, act=act, idsets=idsets, st=st):
            ids = idsets[st["i"] % 8]; st["i"] += 1
            K.call("fb_moe_gate_up_fp8", w13, s13, x, H, ids, act, n, topk, I, H, 0, E, 10.0)

        def dn_simt(I=I, H=H, w2=w2, s2=s2, act=act, idsets=idsets, st=st, out=out, wts=wts):
            ids = idsets[st["i"] % 8]; st["i"] += 1
            K.call("fb_moe_down_fp8", w2, s2, act, ids, wts, out, H, n, topk, I, H, 0, E, 0)

        if want("moe_gate_up"):
            cases.append(Case(f"moe_gate_up_mma.{tag}", n * topk * 2 * I * H, gu, f"24 experts I={I}"))
            cases.append(Case(f"moe_gate_up_simt.{tag}", n * topk * 2 * I * H, gu_simt, f"24 experts I={I}"))
        if want("moe_down"):
            cases.append(Case(f"moe_down_mma.{tag}", n * topk * I * H, dn, f"24 experts I={I}"))
            cases.append(Case(f"moe_down_simt.{tag}", n * topk * I * H, dn_simt, f"24 experts I={I}"))

    # ---- tcgen05 prefill GEMM (reported in TFLOP/s through the note; bytes = weights once) -------
    for tag, M, N, Kd in (("qkv_in.m1024", 1024, 24896, 4096), ("o_proj.m1024", 1024, 4096, 8192), ("lm_head.m256", 256, 154880, 4096),
                          ("o_proj.m64", 64, 4096, 8192)):
        name = f"gemm_tc_bf16.{tag}"
        if not want(name):
            continue
        w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16)
        x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(M, N, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)

        def tcfn(w=w, x=x, out=out, status=status, M=M, N=N, Kd=Kd):
            K.call("fb_gemm_tc_bf16", w, x, Kd, out, N, M, N, Kd, 0, status)
        cases.append(Case(name, N * Kd * 2, tcfn, f"M={M} N={N} K={Kd} FLOP={2 * M * N * Kd}"))

    # ---- the fused GEMM + all-reduce kernel with one rank: its tcgen05 / TMA pipeline without the collective --------
    if want("gemm_tc_ar"):
        from ferrite_b200.parallel.symm import FusedGemmAllReduce
        gar = FusedGemmAllReduce(torch.device("cuda"), 0, 1, max_rows=256, n_max=4096)
        for tag, M, N, Kd in (("o_proj.m256", 256, 4096, 8192), ("o_proj.m64", 64, 4096, 8192)):
            ws_ = [torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) for _ in range(4)]   # 4 x 67 MB > L2
            x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
            out = torch.zeros(M, N, device=dev)
            stg = {"i": 0}

            def garfn(ws_=ws_, x=x, out=out, stg=stg, M=M, N=N, Kd=Kd):
                w = ws_[stg["i"] % 4]; stg["i"] += 1
                gar(w, x, Kd, out, N, M, N, Kd, False)
            cases.append(Case(f"gemm_tc_ar.world1.{tag}", N * Kd * 2, garfn, f"M={M} N={N} K={Kd} FLOP={2 * M * N * Kd}"))

    # ---- DSV41: fp4 experts (TP8 slice), sparse attention with sink, indexer scoring -----------------
    if want("d4_expert"):
        E, n, topk, I, D = 384, 1, 6, 320, 5120
        w13 = torch.randint(0, 256, (E, 2, I, D // 2), dtype=torch.uint8, device=dev)
        s13 = torch.full((E, 2, I, D // 32), 120, dtype=torch.uint8, device=dev)
        w2 = torch.randint(0, 256, (E, D, I // 2), dtype=torch.uint8, device=dev)
        s2 = torch.full((E, D, I // 32), 120, dtype=torch.uint8, device=dev)
        x = torch.randn(n, D, device=dev)
        hbuf = torch.zeros(n * topk, I, device=dev)
        y = torch.zeros(n, D, device=dev)
        wts = torch.rand(n, topk, device=dev)
        idsets = [torch.randperm(E, device=dev)[:n * topk].to(torch.int32).view(n, topk).contiguous() for _ in range(64)]
        st4 = {"i": 0}

        def d4gu():
            ids = idsets[st4["i"] % 64]; st4["i"] += 1
            K.call("fb_d4_expert_gate_up", x, D, ids, wts, w13, s13, hbuf, n, topk, I, D, 10.0)

        def d4dn():
            ids = idsets[st4["i"] % 64]; st4["i"] += 1
            K.call("fb_d4_expert_down", hbuf, ids, w2, s2, y, D, n, topk, I, D, 0)
        cases.append(Case("d4_expert_gate_up.tp8.m1", topk * 2 * I * (D // 2 + D // 32), d4gu, f"6 experts x 2 x {I} x {D} e2m1"))
        cases.append(Case("d4_expert_down.tp8.m1", topk * D * (I // 2 + I // 32), d4dn, f"6 experts x {D} x {I} e2m1"))
        # tensor-core variants (quad-interleaved bytes; random bytes need no repack), TP8 slice and the whole expert
        from ferrite_b200.models.glm import Act
        for tag, Im, Em in (("tp8", 320, 384), ("tp1", 2304, 48)):
            w13m = torch.randint(0, 256, (Em, 2, Im, D // 2), dtype=torch.uint8, device=dev)
            s13m = torch.full((Em, 2, Im, D // 32), 120, dtype=torch.uint8, device=dev)
            w2m = torch.randint(0, 256, (Em, D, Im // 2), dtype=torch.uint8, device=dev)
            s2m = torch.full((Em, D, Im // 32), 120, dtype=torch.uint8, device=dev)
            xa, ha = Act(dev, 8, D), Act(dev, 8 * topk, Im)
            xa.f.normal_()
            K.call("fb_d4_quant_rows", xa.f, D, xa.f, D, 8, D, *xa.sp(2))
            ha.f.normal_()
            K.call("fb_d4_quant_rows", ha.f, Im, ha.f, Im, 8 * topk, Im, *ha.sp(2))
            hout = torch.zeros(8 * topk, Im, device=dev)
            ym = torch.zeros(8, D, device=dev)
            for m in (1, 6):
                sets = [torch.stack([torch.randperm(Em, device=dev)[:topk] for _ in range(m)]).to(torch.int32).contiguous()
                        for _ in range(8)]
                wm = torch.rand(m, topk, device=dev)
                stm = {"i": 0}

                def gu(m=m, sets=sets, wm=wm, stm=stm, w13m=w13m, s13m=s13m, xa=xa, hout=hout, Im=Im):
                    ids = sets[stm["i"] % 8]; stm["i"] += 1
                    K.call("fb_d4_expert_gate_up_mma", _lib.ctypes.c_void_p(xa.s.data_ptr() + 4 * xa.plane), D, ids, wm, w13m, s13m,
                           hout, m, topk, Im, D, 10.0)

                def dn(m=m, sets=sets, stm=stm, w2m=w2m, s2m=s2m, ha=ha, ym=ym, Im=Im):
                    ids = sets[stm["i"] % 8]; stm["i"] += 1
                    K.call("fb_d4_expert_down_mma", _lib.ctypes.c_void_p(ha.s.data_ptr() + 4 * ha.plane), ids, w2m, s2m, ym, D, m, topk,
                           Im, D, 0)
                cases.append(Case(f"d4_expert_gate_up_mma.{tag}.m{m}", m * topk * 2 * Im * (D // 2 + D // 32), gu,
                                  f"{m * topk} pairs x 2 x {Im} x {D} e2m1 (bytes if all pairs differ)"))
                cases.append(Case(f"d4_expert_down_mma.{tag}.m{m}", m * topk * D * (Im // 2 + Im // 32), dn,
                                  f"{m * topk} pairs x {D} x {Im} e2m1"))
    # ---- DSV41: block-scaled tcgen05 grouped GEMM (e2m1 weights x e4m3 rows, ue8m0 scales), prefill / batched sizes ----
    if want("mx_gemm"):
        from ferrite_b200.ops import mx
        D = 5120
        for tag, Em, Nm, rows_per in (("gate_up.tp8.96e", 96, 2 * 384, 64), ("gate_up.tp1.16e", 16, 2 * 2304, 64),
                                      ("gate_up.tp1.16e.r256", 16, 2 * 2304, 256)):
            wp = torch.randint(0, 256, (Em, Nm, D // 2), dtype=torch.uint8, device=dev)
            sfa = mx.pack_weight_scales(torch.full((Em, Nm, D // 32), 120, dtype=torch.uint8, device=dev))
            Mr = Em * rows_per
            x8 = (torch.randn(Mr, D, device=dev) * 2).to(torch.float8_e4m3fn)
            xsf = torch.full((Mr, D // 32), 124, dtype=torch.uint8, device=dev)
            bn = mx.pick_bn(rows_per)
            tiles, n_tiles, _ = mx.make_tiles(torch.full((Em,), rows_per, dtype=torch.int32, device=dev), bn)
            outm = torch.zeros(Mr, Nm, device=dev)
            stat = torch.zeros(4, dtype=torch.int32, device=dev)

            def mxfn(wp=wp, sfa=sfa, x8=x8, xsf=xsf, tiles=tiles, n_tiles=n_tiles, outm=outm, bn=bn, stat=stat):
                mx.mx_gemm_grouped(wp, sfa, x8, xsf, tiles, n_tiles, outm, bn, stat)
            wbytes = Em * Nm * (D // 2 + D // 32)
            cases.append(Case(f"mx_gemm.{tag}", wbytes + Mr * D + Mr * Nm * 4, mxfn,
                              f"{Em} experts x {Nm} x {D} e2m1 ({wbytes / 1e6:.0f} MB), {rows_per} rows each (bn {bn}) "
                              f"FLOP={2 * Mr * Nm * D}"))
    # ---- GLM: W8A16 grouped tcgen05 GEMM (e4m3 weights + 128x128 f32 scales, f16 rows), prefill sizes ----
    if want("fp8w_gemm"):
        for tag, Em, Nm, Km, rows_per in (("gate_up.128e.r64", 128, 4096, 4096, 64), ("down.128e.r64", 128, 4096, 2048, 64),
                                          ("gate_up.36e.r228", 36, 4096, 4096, 228), ("gate_up.128e.r24", 128, 4096, 4096, 24),
                                          ("gate_up.16e.r64", 16, 4096, 4096, 64)):
            wq = torch.randint(0, 120, (Em * Nm, Km), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
            sc = torch.rand(Em, Nm // 128, Km // 128, device=dev) * 0.01
            Mr = Em * rows_per
            xh = torch.randn(Mr, Km, device=dev).half()
            bn = 32 if rows_per <= 32 else 64 if rows_per <= 64 else 128
            mt = Em * ((rows_per + bn - 1) // bn) + 8
            tiles = torch.zeros(mt, 4, dtype=torch.int32, device=dev)
            n_tiles = torch.zeros(1, dtype=torch.int32, device=dev)
            offs = torch.zeros(Em + 1, dtype=torch.int32, device=dev)
            K.call("fb_mx_tiles", torch.full((Em,), rows_per, dtype=torch.int32, device=dev), Em, bn, tiles, n_tiles, offs, mt)
            outw = torch.zeros(Mr, Nm, device=dev)
            stat = torch.zeros(4, dtype=torch.int32, device=dev)

            def fwfn(wq=wq, sc=sc, xh=xh, tiles=tiles, n_tiles=n_tiles, mt=mt, outw=outw, Mr=Mr, Em=Em, Nm=Nm, Km=Km, bn=bn, stat=stat):
                K.call("fb_fp8w_gemm_grouped", wq, sc, xh, tiles, n_tiles, mt, outw, Nm, Mr, Em, Nm, Km, bn, stat)
            wbytes = Em * Nm * Km
            cases.append(Case(f"fp8w_gemm.{tag}", wbytes + Mr * Km * 2 + Mr * Nm * 4, fwfn,
                              f"{Em} experts x {Nm} x {Km} e4m3 ({wbytes / 1e6:.0f} MB), {rows_per} rows each (bn {bn}) "
                              f"FLOP={2 * Mr * Nm * Km}"))
    if want("d4_sparse_attn"):
        n, Hl, hd, W, cap, ktop, ccap = 1, 8, 512, 128, 136, 512, 8192
        ring = torch.randn(1, cap, hd, device=dev).to(torch.bfloat16)
        comp = torch.randn(1, ccap, hd, device=dev).to(torch.bfloat16)
        q = torch.randn(n, Hl * hd, device=dev)
        idx = torch.randperm(ccap, device=dev)[:ktop].sort().values.to(torch.int32).view(n, ktop).contiguous()
        sink = torch.zeros(Hl, device=dev)
        freqs = torch.rand(32, device=dev)
        meta = torch.zeros(n, 8, dtype=torch.int32, device=dev)
        meta[:, 1] = 5000
        out = torch.zeros(n, Hl * hd, device=dev)
        at_o, at_ml = torch.zeros(n * Hl * 16 * hd, device=dev), torch.zeros(n * Hl * 16 * 2, device=dev)

        def d4at():
            K.call("fb_d4_sparse_attn", q, Hl * hd, ring, cap, W, comp, ccap, idx, ktop, ktop, None, 0, sink, freqs, 64, meta, 0, 0,
                   float(hd ** -0.5), Hl, hd, out, Hl * hd, n, 16, at_o, at_ml, None, 0, 0, 0, None)
        at_tk = torch.zeros(n * ((Hl + 7) // 8), dtype=torch.int32, device=dev)

        def d4at1():
            K.call("fb_d4_sparse_attn", q, Hl * hd, ring, cap, W, comp, ccap, idx, ktop, ktop, None, 0, sink, freqs, 64, meta, 0, 0,
                   float(hd ** -0.5), Hl, hd, out, Hl * hd, n, 16, at_o, at_ml, None, 0, 0, 0, at_tk)
        cases.append(Case("d4_sparse_attn.tp8.m1", (W + ktop) * hd * 2, d4at, f"{Hl} heads, {W}+{ktop} keys x {hd} bf16 (L2-resident), two kernels"))
        cases.append(Case("d4_sparse_attn_1k.tp8.m1", (W + ktop) * hd * 2, d4at1, "same, the last CTA of a head tile merges the splits"))
        def d4attc():
            K.call("fb_d4_sparse_attn_tc", q, Hl * hd, ring, cap, W, comp, ccap, idx, ktop, ktop, sink, freqs, 64, meta, 0, 0,
                   float(hd ** -0.5), Hl, out, Hl * hd, n, 10, at_o, at_ml, None, 0, 0, 0)
        cases.append(Case("d4_sparse_attn_tc.tp8.m1", (W + ktop) * hd * 2, d4attc, "tensor-core form, 10 splits of 64 keys + merge kernel"))
        for ns in (32, 40, 80):
            bo, bm = torch.zeros(n * Hl * ns * hd, device=dev), torch.zeros(n * Hl * ns * 2, device=dev)
            # one-kernel form: the merging warp keeps a split per lane (<= 32 splits); multiples of 8 merge by clusters
            for tk, tag in ((None, "2k"), (at_tk, "1k")) if ns <= 32 else ((None, "2k"),):
                def f(ns=ns, bo=bo, bm=bm, tk=tk):
                    K.call("fb_d4_sparse_attn", q, Hl * hd, ring, cap, W, comp, ccap, idx, ktop, ktop, None, 0, sink, freqs, 64, meta,
                           0, 0, float(hd ** -0.5), Hl, hd, out, Hl * hd, n, ns, bo, bm, None, 0, 0, 0, tk)
                cases.append(Case(f"d4_sparse_attn_{tag}.split{ns}.tp8.m1", (W + ktop) * hd * 2, f, f"{ns} splits"))
    if want("d4_route_swiglu"):
        # DSV41 decode, one row: routing over 384 experts (block-parallel scores, one-warp picks) and the shared
        # expert's SwiGLU + quantiser as two roles of one launch
        n, E, topk, I = 1, 384, 6, 512
        lg = torch.randn(n, E, device=dev) * 3
        bias = torch.randn(E, device=dev) * 0.1
        gu = torch.randn(n, 2 * I, device=dev) * 4
        ridx = torch.zeros(n, topk, dtype=torch.int32, device=dev)
        rw = torch.zeros(n, topk, device=dev)
        hs = torch.zeros(n, I, device=dev)

        def d4rs():
            K.call("fb_d4_route_swiglu", lg, E, bias, None, None, n, E, topk, 2.5, ridx, rw, gu, 2 * I, hs, I, I, 7.0, None, 0, 0, 0)

        def d4r():
            K.call("fb_d4_route", lg, E, bias, None, None, n, E, topk, 2.5, ridx, rw)
        cases.append(Case("d4_route_swiglu.m1", E * 8 + 3 * I * 4, d4rs, "one launch: route (384 experts, top 6) + SwiGLU/quantiser of 512 channels"))
        cases.append(Case("d4_route_block.m1", E * 8, d4r, "the block-wide router alone (six barriers per pick)"))
    if want("hc_pre_wide_offset"):
        # DSV41 decode, one row: the column-parallel hyper-connection front fed by 320 tiles of partials
        n, H, tiles, ld = 1, 5120, 320, 512
        Rm = torch.randn(n, 4, H, device=dev)
        part = torch.randn(8, 25, ld, device=dev) * 0.1
        part[:, 24] = part[:, 24].abs() * 50 + 1.0          # sums of squares
        gram = torch.randn(8, 10, ld, device=dev).abs() + 0.5
        part_n = torch.full((8,), tiles, dtype=torch.int32, device=dev)
        scale, base = torch.ones(3, device=dev), torch.zeros(24, device=dev)
        ln_w = torch.ones(H, device=dev)
        pre_in, pre_out = torch.rand(n, 4, device=dev) + 0.1, torch.zeros(n, 4, device=dev)
        post, comb = torch.zeros(n, 4, device=dev), torch.zeros(n, 16, device=dev)
        xo, xq = torch.zeros(n, H, device=dev), torch.zeros(n, H, device=dev)
        acc = torch.zeros(n, 25, device=dev)

        def hcw():
            K.call("fb_hc_pre_wide_offset", Rm, part, gram, part_n, ld, scale, base, ln_w, pre_in, pre_out, xo, post, comb, n, H,
                   24, 1e-6, 1e-6, 20, None, 0, 0, 0, xq, None, 0, 0, 0)

        def hc1():
            acc.copy_(part[:1, :, 0])
            K.call("fb_d4_hc_pre", Rm, acc, scale, base, ln_w, pre_in, pre_out, post, comb, xo, None, n, H, 4, 1e-6, 1e-6, 20,
                   None, 0, 0, 0, None, None, 0, None, None, 0, 0, 0)
        cases.append(Case("hc_pre_wide_offset.m1", 4 * H * 4 + 2 * H * 4 + 35 * tiles * 4, hcw,
                          "11 CTAs per row: contraction + RMSNorm + e4m3 round trip per 512 columns, coefficients in their own CTA"))
        cases.append(Case("hc_pre_offset_one_cta.m1", 4 * H * 4 + H * 4, hc1, "one CTA per row (plus a 100-byte copy that refills its accumulator)"))
    if want("d4_index_score"):
        n, IHl, ID, ccap = 1, 4, 128, 65536
        kc = torch.randn(1, ccap, ID, device=dev).to(torch.bfloat16)
        q = torch.randn(n, IHl * ID, device=dev)
        wv = torch.rand(n, 8, device=dev)
        meta = torch.zeros(n, 8, dtype=torch.int32, device=dev)
        meta[:, 1] = ccap - 1
        score = torch.zeros(n, ccap, device=dev)

        def d4is():
            K.call("fb_d4_index_score", q, IHl * ID, wv, 8, kc, ccap, meta, score, ccap, n, IHl, ID, 1, 0.01)
        cases.append(Case("d4_index_score.tp8.m1.ctx64k", ccap * ID * 2, d4is, f"{IHl} heads x {ID}, {ccap} keys bf16"))

    # ---- MHC site -----------------------------------------------------------------------
    if want("hc_"):
        n, H, mix = 3, 4096, 24
        R0, R1 = torch.randn(n, 4, H, device=dev), torch.zeros(n, 4, H, device=dev)
        fns = [torch.randn(mix, 4 * H, device=dev) * 0.02 for _ in range(100)]
        acc = torch.zeros(n, 25, device=dev)
        y = torch.randn(n, H, device=dev)
        post, comb = torch.rand(n, 4, device=dev), torch.rand(n, 16, device=dev)
        scale, base, ln = torch.ones(3, device=dev), torch.zeros(mix, device=dev), torch.ones(H, device=dev)
        xn = torch.zeros(n, H, device=dev)
        sp = torch.zeros(4, n, H, dtype=torch.int16, device=dev)
        st = {"i": 0}

        def pm():
            f = fns[st["i"] % 100]; st["i"] += 1
            K.call("fb_hc_post_mix", R0, R1, y, post, comb, f, acc, n, H, mix)

        def pa():
            K.call("fb_hc_pre_apply", R1, acc, scale, base, ln, None, xn, post, comb, n, H, 4, 1e-5, 1e-6, 20, sp, H, n * H, 3, None, None, 0)
        cases.append(Case("hc_post_mix.m3", mix * 4 * H * 4 + 2 * n * 4 * H * 4, pm, "fn 1.5 MB f32"))
        cases.append(Case("hc_pre_apply.m3", n * 4 * H * 4, pa, "latency-bound"))
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default=None)
    ap.add_argument("--no-graph", action="store_true", help="eager launches (use under ncu)")
    args = ap.parse_args()
    K = _lib.lib()
    peak, tag = hbm_peak_gbs()
    rows = []
    cases = make_cases(K, args.only)
    exact = [c for c in cases if c.name == args.only]   # a full case name runs that case alone
    for c in exact or cases:
        for _ in range(args.warmup):
            c.fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.no_graph:
            e0.record()
            for _ in range(args.iters):
                c.fn()
            e1.record()
        else:  # one graph of `iters` launches: no per-launch host time in the measurement
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(args.iters):
                    c.fn()
            g.replay()
            torch.cuda.synchronize()
            e0.record()
            g.replay()
            e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.iters
        gbs = c.nbytes / us / 1e3
        rows.append({"kernel": c.name, "us": round(us, 2), "MB": round(c.nbytes / 1e6, 1), "GB/s": round(gbs, 0),
                     "frac": round(gbs / peak, 3), "note": c.note})
        extra = ""
        if "FLOP=" in c.note:
            tf = float(c.note.split("FLOP=")[1]) / us / 1e6
            rows[-1]["TFLOPs"] = round(tf, 1)
            extra = f"  {tf:7.1f} TFLOP/s"
        print(f"{c.name:38s} {us:9.2f} us  {c.nbytes / 1e6:8.1f} MB  {gbs:7.0f} GB/s  {gbs / peak:5.2f} {tag}  {c.note}{extra}")
    if args.json:
        json.dump({"hbm_peak_gbs": peak, "peak_kind": tag, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
