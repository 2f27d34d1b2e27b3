"""GPU: DSV41 kernels one at a time against plain fp32 statements of the same op (``ops/quant.py`` codecs,
``models/dsv41_ref.py`` helpers, fp32 matmuls of dequantised weights)."""
import math

import pytest
import torch
import torch.nn.functional as F

from ferrite_b200.models import dsv41_ref as G
from ferrite_b200.ops import quant as Q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from ferrite_b200 import _lib
    return _lib.lib()


def gen(seed):
    return torch.Generator().manual_seed(seed)


def meta_for(pos):
    m = torch.zeros(len(pos), 8, dtype=torch.int32)
    m[:, 1] = torch.tensor(pos, dtype=torch.int32)
    return m.cuda()


def close(name, got, want, tol):
    err = (got.float().cpu() - want.float()).abs().max().item()
    assert err <= tol, f"{name}: max abs err {err} > {tol}"


@pytest.mark.parametrize("inverse,fp4_rt", [(0, 0), (1, 0), (0, 1)])
def test_rope_heads(K, inverse, fp4_rt):
    n, heads, hd, rd = 4, 3, 128, 64
    x = torch.randn(n, heads * hd, generator=gen(1))
    freqs = torch.rand(rd // 2, generator=gen(2)) * 0.1
    pos = [0, 7, 1234, 99999]
    xd = x.clone().cuda()
    K.call("fb_d4_rope_heads", xd, heads * hd, n, heads, hd, rd, freqs.cuda(), meta_for(pos), 0, inverse, fp4_rt, None, 0, 0, 0)
    want = G.apply_rope(x.view(n, heads, hd), torch.tensor(pos), freqs, inverse=bool(inverse))
    if fp4_rt:
        # the device computes sin / cos in f32 of an f32 angle, the statement too; a value within one ulp of an e2m1
        # rounding boundary may still land on the other side, so the comparison is on the un-quantised rotation
        got_rt = xd.cpu().view(n, heads, hd)
        want_rt = Q.fp4_act_roundtrip(want, 32)
        frac = ((got_rt - want_rt).abs() > 1e-6).float().mean().item()
        assert frac < 0.01, frac
    else:
        close("rope", xd.view(n, heads, hd), want, 2e-3)     # angles up to 1e4 rad in f32


def test_rmsnorm_quant(K):
    n, Kd = 5, 1536
    x = torch.randn(n, Kd, generator=gen(3)) * torch.logspace(-2, 1, n).unsqueeze(1)
    w = 1 + 0.1 * torch.randn(Kd, generator=gen(4))
    out = torch.zeros(n, Kd, device="cuda")
    K.call("fb_d4_rmsnorm_quant", x.cuda(), Kd, w.cuda(), out, Kd, n, Kd, 1e-6, None, 0, 0, 0)
    normed = G.rmsnorm(x, w, 1e-6)
    want = Q.fp8_act_roundtrip(normed, 32)
    # identical up to elements whose un-quantised value sits on an e4m3 rounding boundary (the two sides sum the
    # squares in different orders): such an element moves by one e4m3 step = 1/8 of its magnitude at most
    diff = (out.cpu() - want).abs()
    assert (diff > 1e-6).float().mean().item() < 0.002
    assert (diff <= 0.126 * normed.abs() + 1e-6).all()


@pytest.mark.parametrize("lim", [0.0, 7.0])
def test_swiglu_clamp_and_quant(K, lim):
    n, I = 3, 384
    gu = torch.randn(n, 2 * I, generator=gen(5)) * 6
    g, u = gu[:, :I], gu[:, I:]
    if lim > 0:
        g, u = g.clamp(max=lim), u.clamp(-lim, lim)
    want = F.silu(g) * u
    out = torch.zeros(n, I, device="cuda")
    K.call("fb_d4_swiglu_clamp", gu.cuda(), 2 * I, out, I, n, I, lim)
    close("swiglu", out, want, 1e-5 * want.abs().max().item())
    outq = torch.zeros(n, I, device="cuda")
    K.call("fb_d4_swiglu_clamp_quant", gu.cuda(), 2 * I, outq, I, n, I, lim, None, 0, 0, 0)
    wq = Q.fp8_act_roundtrip(want, 32)
    diff = (outq.cpu() - wq).abs()
    assert (diff > 1e-6).float().mean().item() < 0.005 and (diff <= 0.126 * want.abs() + 1e-6).all()


@pytest.mark.parametrize("E,topk,image", [(64, 6, False), (256, 8, True), (16, 1, False)])
def test_route_sqrt_softplus(K, E, topk, image):
    n = 6
    logits = torch.randn(n, E, generator=gen(6)) * 3
    logits[0, 3] = logits[0, 9]                       # a tie: the lower index wins
    bias = torch.randn(E, generator=gen(7)) * 0.1
    bias_vl = torch.randn(E, generator=gen(8)) * 0.1
    is_img = torch.tensor([0, 1, 0, 1, 1, 0], dtype=torch.uint8)
    idx = torch.zeros(n, topk, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n, topk, device="cuda")
    K.call("fb_d4_route", logits.cuda(), E, bias.cuda(), bias_vl.cuda() if image else None, is_img.cuda() if image else None,
           n, E, topk, 2.5, idx, wts)
    scores = F.softplus(logits).sqrt()
    b = bias.expand(n, E)
    if image:
        b = torch.where(is_img.bool().unsqueeze(-1), bias_vl.expand(n, E), b)
    widx = G.topk_stable(scores + b, topk)
    ww = scores.gather(1, widx)
    if topk > 1:
        ww = ww / (ww.sum(-1, keepdim=True) + 1e-20)
    assert idx.cpu().tolist() == widx.tolist()
    close("route weights", wts, ww * 2.5, 1e-5)


def _fp4_experts(E, N, Kd, seed):
    w = torch.randn(E, N, Kd, generator=gen(seed)) * 0.05
    packed, scales, deq = [], [], []
    for e in range(E):
        p, s = Q.quant_fp4_weight(w[e], 32)
        packed.append(p); scales.append(s); deq.append(Q.dequant_fp4_weight(p, s, 32))
    return torch.stack(packed), torch.stack(scales), torch.stack(deq)


@pytest.mark.parametrize("n,topk,E,I,D", [(2, 2, 4, 64, 128), (3, 4, 8, 192, 512)])
def test_fp4_expert_gate_up_and_down(K, n, topk, E, I, D):
    w13p, w13s, w13 = _fp4_experts(E, 2 * I, D, 9)          # [E][gate I | up I][D]
    w2p, w2s, w2 = _fp4_experts(E, D, I, 10)
    x = Q.fp8_act_roundtrip(torch.randn(n, D, generator=gen(11)), 32)
    idx = torch.stack([torch.randperm(E, generator=gen(12 + r))[:topk] for r in range(n)]).to(torch.int32)
    wts = torch.rand(n, topk, generator=gen(20)) + 0.1
    lim = 7.0
    h = torch.zeros(n, topk, I, device="cuda")
    K.call("fb_d4_expert_gate_up", x.cuda(), D, idx.cuda(), wts.cuda(), w13p.cuda(), w13s.cuda(), h, n, topk, I, D, lim)
    want_h = torch.zeros(n, topk, I)
    for r in range(n):
        for s in range(topk):
            gu = w13[idx[r, s]] @ x[r]
            g, u = gu[:I].clamp(max=lim), gu[I:].clamp(-lim, lim)
            want_h[r, s] = F.silu(g) * u * wts[r, s]
    close("expert gate/up", h, want_h, 2e-5 * max(1.0, want_h.abs().max().item()))
    hq = Q.fp8_act_roundtrip(want_h, 32)
    y = torch.full((n, D), 0.5, device="cuda")
    K.call("fb_d4_expert_down", hq.cuda(), idx.cuda(), w2p.cuda(), w2s.cuda(), y, D, n, topk, I, D, 1)
    want_y = torch.full((n, D), 0.5)
    for r in range(n):
        for s in range(topk):
            want_y[r] += w2[idx[r, s]] @ hq[r, s]
    close("expert down", y, want_y, 2e-5 * max(1.0, want_y.abs().max().item()))


def test_gemv_f32_weights(K):
    m, N, Kd = 5, 70, 1024
    W = torch.randn(N, Kd, generator=gen(30))
    x = torch.randn(m, Kd + 4, generator=gen(31))
    out = torch.zeros(m, N, device="cuda")
    K.call("fb_d4_gemv_f32w", W.cuda(), x.cuda(), Kd + 4, out, N, m, N, Kd)
    close("gemv f32w", out, x[:, :Kd].double() @ W.double().t(), 1e-3)


@pytest.mark.parametrize("nsplit,own_merge", [(4, False), (4, True), (7, True), (8, True), (16, True), (32, True)])
def test_sparse_attention_with_sink_matches_rows_statement(K, nsplit, own_merge):
    """Window ring + compressed rows + sink against models/dsv41_ref.py::sparse_attn_rows on the gathered keys; the
    split partials merged by a second kernel or by the last CTA of each (row, head tile)."""
    n, Hl, hd, W, cap, ccap, ktop = 2, 4, 128, 16, 24, 64, 8
    pos = [40, 9]                                       # row 1: fewer positions than the window holds
    ring = (torch.randn(1, cap, hd, generator=gen(40)) * 0.5).to(torch.bfloat16)
    comp = (torch.randn(1, ccap, hd, generator=gen(41)) * 0.5).to(torch.bfloat16)
    q = torch.randn(n, Hl * hd, generator=gen(42))
    idx = torch.stack([torch.randperm(ccap, generator=gen(43 + r))[:ktop].sort().values for r in range(n)]).to(torch.int32)
    idx[1, 5:] = -1                                     # a short candidate list
    sink = torch.randn(Hl, generator=gen(50))
    freqs = torch.zeros(32)                             # no output rotation: rd = 64 dims with zero angles
    meta = meta_for(pos)
    out = torch.zeros(n, Hl * hd, device="cuda")
    ticket = torch.zeros(n, dtype=torch.int32, device="cuda") if own_merge else None
    o_part = torch.zeros(n * Hl * nsplit * hd, device="cuda")
    ml_part = torch.zeros(n * Hl * nsplit * 2, device="cuda")
    scale = hd ** -0.5
    K.call("fb_d4_sparse_attn", q.cuda(), Hl * hd, ring.cuda(), cap, W, comp.cuda(), ccap, idx.cuda(), ktop, ktop, None, 0,
           sink.cuda(), freqs.cuda(), 64, meta, 0, 0, float(scale), Hl, hd, out, Hl * hd, n, nsplit, o_part, ml_part,
           None, 0, 0, 0, ticket)
    if own_merge:
        assert int(ticket.abs().sum()) == 0        # left at zero for the next launch
    for r in range(n):
        win = [p % cap for p in G.window_positions(pos[r], W)]
        keys = [ring[0, p].float() for p in win] + [comp[0, int(j)].float() for j in idx[r] if j >= 0]
        kv = torch.stack(keys)                                        # [keys, hd]
        want = G.sparse_attn_rows(q[r].view(Hl, hd), kv, sink, scale)  # [Hl, hd]
        close(f"sparse attention row {r}", out[r].view(Hl, hd), want, 3e-3)


def test_hc_front_column_parallel_offset_form(K):
    """fb_hc_pre_wide_offset (partial tiles of the mix dots, the sum of squares and the Gram of R in; x, its e4m3 round
    trip and this site's coefficients out) against the fp32 statement of the offset hyper-connection front."""
    from ferrite_b200.ops import reference as R
    n, H, m, tiles, ld = 3, 1536, 4, 5, 8
    Rm = torch.randn(n, m, H, generator=gen(60)) * torch.tensor([0.5, 1.0, 3.0]).view(n, 1, 1)
    fn = torch.randn(24, m * H, generator=gen(61)) * 0.05
    scale = torch.tensor([0.7, 1.3, 0.9])
    base = torch.randn(24, generator=gen(62)) * 0.3
    ln_w = 1 + 0.1 * torch.randn(H, generator=gen(63))
    pre_in = torch.rand(n, m, generator=gen(64)) + 0.1
    rms_eps, hc_eps, iters = 1e-6, 1e-6, 20
    flat = Rm.reshape(n, -1)
    # per-tile partials: column tiles of unequal width, each tile's share of every sum
    edges = [0, 100, 612, 613, 1400, H]
    part = torch.zeros(8, 25, ld)
    gram = torch.zeros(8, 10, ld)
    for t in range(tiles):
        sl = Rm[:, :, edges[t]:edges[t + 1]]                                   # [n, m, w]
        fl = fn.view(24, m, H)[:, :, edges[t]:edges[t + 1]]
        part[:n, :24, t] = torch.einsum("nmw,qmw->nq", sl, fl)
        part[:n, 24, t] = sl.square().sum((1, 2))
        p = 0
        for i in range(m):
            for k in range(i, m):
                gram[:n, p, t] = (sl[:, i] * sl[:, k]).sum(-1)
                p += 1
    part[:, :, tiles:] = 7.0                                                   # beyond the tile count: never read
    part_n = torch.full((8,), tiles, dtype=torch.int32)
    x_out, xq_out = torch.zeros(n, H, device="cuda"), torch.zeros(n, H, device="cuda")
    pre_out, post, comb = torch.zeros(n, m, device="cuda"), torch.zeros(n, m, device="cuda"), torch.zeros(n, m * m, device="cuda")
    K.call("fb_hc_pre_wide_offset", Rm.cuda(), part.cuda(), gram.cuda(), part_n.cuda(), ld, scale.cuda(), base.cuda(),
           ln_w.cuda(), pre_in.cuda(), pre_out, x_out, post, comb, n, H, 24, rms_eps, hc_eps, iters, None, 0, 0, 0,
           xq_out, None, 0, 0, 0)
    r = torch.rsqrt(flat.square().mean(-1, keepdim=True) + rms_eps)
    wpre, wpost, wcomb = R.hc_coeffs((flat @ fn.t()) * r, scale, base, m, hc_eps, iters)
    close("pre", pre_out, wpre, 1e-5)
    close("post", post, wpost, 1e-5)
    close("comb", comb, wcomb.reshape(n, -1), 1e-5)
    want = G.rmsnorm((pre_in.unsqueeze(-1) * Rm).sum(1), ln_w, rms_eps)
    close("x", x_out, want, 2e-5 * want.abs().max().item())
    wq = Q.fp8_act_roundtrip(want, 32)
    diff = (xq_out.cpu() - wq).abs()
    assert (diff > 1e-6).float().mean().item() < 0.005 and (diff <= 0.126 * want.abs() + 1e-6).all()


def test_qnorm_and_kv_append_in_one_launch_match_the_two_kernels(K):
    n, ql, hd, rd, cap = 3, 192, 128, 64, 16
    qa = torch.randn(n, ql + hd, generator=gen(70)).cuda()
    q_w = (1 + 0.1 * torch.randn(ql, generator=gen(71))).cuda()
    kv_w = (1 + 0.1 * torch.randn(hd, generator=gen(72))).cuda()
    freqs = (torch.rand(rd // 2, generator=gen(73)) * 0.1).cuda()
    meta = meta_for([5, 77, 1000])
    outs = []
    for fused in (False, True):
        q_out = torch.zeros(n, ql, device="cuda")
        ring = torch.zeros(1, cap, hd, dtype=torch.bfloat16, device="cuda")
        rows = torch.zeros(n, hd, device="cuda")
        if fused:
            K.call("fb_d4_qnorm_kv_append", qa, ql + hd, ql, q_w, q_out, ql, 1e-6, None, 0, 0, 0, kv_w, freqs, meta, ring, cap,
                   rows, n, hd, rd, 0)
        else:
            K.call("fb_d4_rmsnorm_quant", qa, ql + hd, q_w, q_out, ql, n, ql, 1e-6, None, 0, 0, 0)
            K.call("fb_d4_kv_append", _lib_view(qa, ql), ql + hd, kv_w, freqs, meta, ring, cap, rows, n, hd, rd, 1e-6, 0)
        outs.append((q_out.cpu(), ring.float().cpu(), rows.cpu()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    want = Q.fp8_act_roundtrip(G.rmsnorm(qa[:, :ql].cpu(), q_w.cpu(), 1e-6), 32)
    diff = (outs[1][0] - want).abs()
    assert (diff > 1e-6).float().mean().item() < 0.005


def _lib_view(t, elems):
    import ctypes
    return ctypes.c_void_p(t.data_ptr() + elems * t.element_size())


@pytest.mark.parametrize("E,topk,n", [(384, 6, 1), (256, 8, 11), (40, 1, 3)])
def test_route_and_swiglu_in_one_launch_match_the_two_kernels(K, E, topk, n):
    I = 96
    logits = torch.randn(n, E, generator=gen(80)) * 3
    logits[0, 3] = logits[0, 9]                       # a tie: the lower index wins
    logits[n - 1, :5] = float("-inf")
    bias = (torch.randn(E, generator=gen(81)) * 0.1).cuda()
    bias_vl = (torch.randn(E, generator=gen(82)) * 0.1).cuda()
    is_img = (torch.arange(n) % 2).to(torch.uint8).cuda()
    gu = (torch.randn(n, 2 * I, generator=gen(83)) * 4).cuda()
    lg = logits.cuda()
    idx0, w0 = torch.zeros(n, topk, dtype=torch.int32, device="cuda"), torch.zeros(n, topk, device="cuda")
    out0 = torch.zeros(n, I, device="cuda")
    K.call("fb_d4_route", lg, E, bias, bias_vl, is_img, n, E, topk, 2.5, idx0, w0)
    K.call("fb_d4_swiglu_clamp_quant", gu, 2 * I, out0, I, n, I, 7.0, None, 0, 0, 0)
    idx1, w1, out1 = torch.zeros_like(idx0), torch.zeros_like(w0), torch.zeros_like(out0)
    K.call("fb_d4_route_swiglu", lg, E, bias, bias_vl, is_img, n, E, topk, 2.5, idx1, w1, gu, 2 * I, out1, I, I, 7.0,
           None, 0, 0, 0)
    assert torch.equal(idx0, idx1) and torch.equal(w0, w1) and torch.equal(out0, out1)


def test_two_problem_gemv_matches_two_launches(K):
    from ferrite_b200.models.glm import Act
    m, Kd, Na, Nb = 3, 1024, 40, 200
    dev = torch.device("cuda")
    xa, xb = Act(dev, m, Kd), Act(dev, m, Kd)
    xa.f.copy_(torch.randn(m, Kd, generator=gen(90)))
    xb.f.copy_(torch.randn(m, Kd, generator=gen(91)))
    for a in (xa, xb):
        K.call("fb_split_rows", a.f, Kd, *a.sp(1), m, Kd)
    Wa = torch.randn(Na, Kd, generator=gen(92)).to(torch.bfloat16).cuda()
    Wb = torch.randn(Nb, Kd, generator=gen(93)).to(torch.bfloat16).cuda()
    oa, ob = torch.zeros(m, Na + 8, device="cuda"), torch.zeros(m, Nb, device="cuda")
    K.call("fb_gemv_mma_bf16_dual", Wa, xa.s, xa.ld, xa.plane, oa, Na + 8, Na, Kd, Wb, xb.s, xb.ld, xb.plane, ob, Nb, Nb, Kd, m)
    close("problem a", oa[:, :Na], xa.f.cpu().double() @ Wa.float().cpu().double().t(), 2e-3)
    close("problem b", ob, xb.f.cpu().double() @ Wb.float().cpu().double().t(), 2e-3)
    assert float(oa[:, Na:].abs().sum()) == 0.0


def test_index_score_relu_weighted_heads(K):
    """score[r][j] = sum_h relu(q_h . k_j) w_h over the visible compressed rows, -inf beyond."""
    n, IH, ID, ratio, cap, lds = 3, 8, 64, 2, 40, 48
    pos = [9, 40, 79]                                  # visible rows: 5, 20, 40 (= cap)
    q = torch.randn(n, IH * ID, generator=gen(100))
    w = torch.randn(n, IH, generator=gen(101))
    kc = torch.randn(1, cap, ID, generator=gen(102)).to(torch.bfloat16)
    score = torch.full((n, lds), 7.0, device="cuda")
    K.call("fb_d4_index_score", q.cuda(), IH * ID, w.cuda(), IH, kc.cuda(), cap, meta_for(pos), score, lds, n, IH, ID, ratio, 0.25)
    want = (torch.einsum("shd,td->sht", q.view(n, IH, ID), kc[0].float()).relu() * (w * 0.25).unsqueeze(-1)).sum(1)
    got = score.cpu()
    for r in range(n):
        clen = (pos[r] + 1) // ratio
        close(f"index score row {r}", got[r, :clen], want[r, :clen], 2e-4 * max(1.0, want[r].abs().max().item()))
        assert torch.isinf(got[r, clen:cap]).all() and (got[r, clen:cap] < 0).all()


@pytest.mark.parametrize("ratio", [1, 4])
def test_compressor_pools_groups_with_channel_softmax(K, ratio):
    """A row whose position completes a group pools the group's positions with a per-channel softmax over the scores
    and RMS-normalises (ratio 1: plain RMSNorm); other rows only store into the ring."""
    hd, depth, n = 64, 16, 6
    pos = list(range(5, 5 + n))                        # positions 5..10: groups complete at 7 (ratio 4) / everywhere (1)
    kv = torch.randn(n, 2 * hd, generator=gen(110))    # [kv | score] per row
    w = 1 + 0.1 * torch.randn(hd, generator=gen(111))
    ring_kv = torch.zeros(1, depth, hd, device="cuda")
    ring_sc = torch.zeros(1, depth, hd, device="cuda")
    hist_kv = torch.randn(5, hd, generator=gen(112))   # positions 0..4, already in the ring
    hist_sc = torch.randn(5, hd, generator=gen(113))
    ring_kv[0, :5] = hist_kv.cuda()
    ring_sc[0, :5] = hist_sc.cuda()
    lat = torch.zeros(n, hd, device="cuda")
    flag = torch.full((n,), -1, dtype=torch.int32, device="cuda")
    kvd = kv.cuda()
    import ctypes
    K.call("fb_d4_compress", kvd, ctypes.c_void_p(kvd.data_ptr() + 4 * hd), 2 * hd, meta_for(pos),
           ring_kv if ratio > 1 else None, ring_sc if ratio > 1 else None, depth, w.cuda(), lat, flag, n, hd, ratio, 1e-6)
    all_kv = torch.cat([hist_kv, kv[:, :hd]])
    all_sc = torch.cat([hist_sc, kv[:, hd:]])
    for r, p in enumerate(pos):
        done = (p + 1) % ratio == 0
        assert int(flag[r]) == int(done)
        if not done:
            continue
        if ratio == 1:
            pooled = kv[r, :hd]
        else:
            g = slice(p - ratio + 1, p + 1)
            pooled = (all_kv[g] * all_sc[g].softmax(0)).sum(0)
        close(f"latent of position {p}", lat[r], G.rmsnorm(pooled, w, 1e-6), 1e-4)


def test_engram_apply_gates_the_value_into_every_stream(K):
    n, hc, D = 3, 4, 256
    Rm = torch.randn(n, hc, D, generator=gen(120))
    kv = torch.randn(n, (hc + 1) * D, generator=gen(121))
    qk = torch.randn(hc, D, generator=gen(122))
    dead = torch.tensor([0, 1, 0], dtype=torch.uint8)
    Rd = Rm.clone().cuda()
    K.call("fb_d4_engram_apply", Rd, kv.cuda(), qk.cuda(), dead.cuda(), n, hc, D, 1e-6)
    key, value = kv[:, :hc * D].view(n, hc, D), kv[:, hc * D:]
    rstd = torch.rsqrt(Rm.square().mean(-1) + 1e-6) * torch.rsqrt(key.square().mean(-1) + 1e-6)
    dot = (Rm * qk * key).sum(-1) * rstd * D ** -0.5
    gate = torch.sigmoid(torch.copysign(dot.abs().clamp_min(1e-6).sqrt(), dot))
    gate = gate.masked_fill(dead.bool().unsqueeze(-1), 0)
    close("engram", Rd, Rm + gate.unsqueeze(-1) * value.unsqueeze(-2), 1e-4)


def test_hc_front_one_cta_per_row_and_post_mix(K):
    """fb_hc_post_mix (R' = post y + comb^T R, mix dots of R' into acc) followed by fb_d4_hc_pre (coefficients of the
    site from acc, contraction with the previous site's pre) against the fp32 statement."""
    from ferrite_b200.ops import reference as R
    n, m, H = 2, 4, 512
    Rm = torch.randn(n, m, H, generator=gen(130))
    y = torch.randn(n, H, generator=gen(131))
    post = torch.rand(n, m, generator=gen(132)) * 2
    comb = torch.rand(n, m, m, generator=gen(133))
    fn = torch.randn(24, m * H, generator=gen(134)) * 0.05
    scale = torch.tensor([0.7, 1.3, 0.9])
    base = torch.randn(24, generator=gen(135)) * 0.3
    ln_w = 1 + 0.1 * torch.randn(H, generator=gen(136))
    pre_in = torch.rand(n, m, generator=gen(137)) + 0.1
    Rout = torch.zeros(n, m, H, device="cuda")
    acc = torch.zeros(n, 25, device="cuda")
    K.call("fb_hc_post_mix", Rm.cuda(), Rout, y.cuda(), post.cuda(), comb.reshape(n, -1).cuda(), fn.cuda(), acc, n, H, 24)
    want_R = R.hc_post(y, Rm, post, comb)
    close("hc_post", Rout, want_R, 1e-4)
    flat = want_R.reshape(n, -1)
    close("mix dots", acc[:, :24], flat @ fn.t(), 2e-3)
    close("sum of squares", acc[:, 24], flat.square().sum(-1), 1e-2)
    x = torch.zeros(n, H, device="cuda")
    pre_out, post_o, comb_o = torch.zeros(n, m, device="cuda"), torch.zeros(n, m, device="cuda"), torch.zeros(n, 16, device="cuda")
    K.call("fb_d4_hc_pre", Rout, acc, scale.cuda(), base.cuda(), ln_w.cuda(), pre_in.cuda(), pre_out, post_o, comb_o, x, None,
           n, H, m, 1e-6, 1e-6, 20, None, 0, 0, 0, None, None, 0, None, None, 0, 0, 0)
    r = torch.rsqrt(flat.square().mean(-1, keepdim=True) + 1e-6)
    wpre, wpost, wcomb = R.hc_coeffs((flat @ fn.t()) * r, scale, base, m, 1e-6, 20)
    close("pre", pre_out, wpre, 2e-5)
    close("post", post_o, wpost, 2e-5)
    close("comb", comb_o, wcomb.reshape(n, -1), 2e-5)
    want = G.rmsnorm((pre_in.unsqueeze(-1) * want_R).sum(1), ln_w, 1e-6)
    close("x", x, want, 2e-5 * want.abs().max().item())
    assert float(acc.abs().sum()) == 0.0               # cleared for the next site
