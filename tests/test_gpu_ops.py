"""GPU: every CUDA op against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

from ferrite_b200.ops import reference as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from ferrite_b200 import _lib
    return _lib.lib()


def dev(t):
    return t.cuda()


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def check(name, got, want, atol, rtol=1e-3):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs().max().item()
    ref = want.abs().max().item()
    assert torch.allclose(got, want, atol=atol, rtol=rtol), f"{name}: max err {err:.3e} (ref max {ref:.3e})"


def unsplit(sp, kind):
    """Rebuild f32 values from a [4, M, ld] int16 split buffer (kind 0 = bf16 pair, 1 = f16 pair)."""
    dt = torch.bfloat16 if kind == 0 else torch.float16
    hi = sp[2 * kind].view(dt).float()
    lo = sp[2 * kind + 1].view(dt).float()
    return hi + lo


def check_split(name, sp, want, n, K_):
    for kind in (0, 1):
        got = unsplit(sp.cpu(), kind)[:n, :K_]
        err = (got - want.float().cpu()).abs().max().item()
        ref = want.abs().max().item() + 1e-9
        assert err / ref < 2e-4, f"{name} kind {kind}: rel err {err / ref:.2e}"


def to_split(x, ld=None):
    """Host-side split of an f32 [M, K] tensor into the [4, M, ld] int16 layout."""
    M, K_ = x.shape
    ld = ld or K_
    sp = torch.zeros(4, M, ld, dtype=torch.int16)
    bh = x.bfloat16()
    bl = (x - bh.float()).bfloat16()
    hh = x.half()
    hl = (x - hh.float()).half()
    for i, t in enumerate((bh, bl, hh, hl)):
        sp[i, :, :K_] = t.view(torch.int16)
    return sp


def make_meta(K, slots, gsizes, seq_len):
    """Row tables + RowMeta for groups (slot, size); seq_len: per-slot start positions."""
    rs, ro, rg, gf = [], [], [], []
    for s, g in zip(slots, gsizes):
        gf.append(len(rs))
        for o in range(g):
            rs.append(s); ro.append(o); rg.append(g)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    n = len(rs)
    meta = torch.zeros(n * 32, dtype=torch.uint8, device="cuda")
    sl = t(seq_len)
    K.call("fb_prep_rows", t(rs), t(ro), t(rg), sl, meta, n, 0, None)
    return meta, t(gf), n, sl


def test_prep_rows_clamps_at_the_context_limit(K):
    """Row metadata is the single source of positions: a group that would pass the limit is moved back
    below it and the status word names the slot.  Only metadata is computed here; no cache is touched."""
    import struct
    t = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    meta = torch.zeros(5 * 32, dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    # slot 0: 3 rows from 10 (fine); slot 1: 2 rows from 63 with a limit of 64 (one too many)
    K.call("fb_prep_rows", t([0, 0, 0, 1, 1]), t([0, 1, 2, 0, 1]), t([3, 3, 3, 2, 2]), t([10, 63]), meta, 5, 64, status)
    torch.cuda.synchronize()
    rows = [struct.unpack("8i", bytes(meta[i * 32:(i + 1) * 32].tolist())) for i in range(5)]
    assert [r[1] for r in rows] == [10, 11, 12, 62, 63]            # positions
    assert [r[3] for r in rows] == [13, 13, 13, 64, 64]            # totals stay <= limit
    assert status.tolist() == [3, 1, 63, 2]                         # FB_BAD_ARG, slot, length, rows


@pytest.mark.parametrize("m,N,K_,group", [(1, 300, 256, 0), (3, 4100, 512, 0), (8, 9600, 128, 0),
                                          (2, 16 * 64, 32, 64), (5, 777, 4096, 0)])
def test_gemv_bf16(K, m, N, K_, group):
    G = N // group if group else 1
    w = rnd(N, K_, seed=1, scale=0.1).bfloat16()
    x = rnd(m, G * K_, seed=2)
    out = torch.full((m, N), 7.0)
    wd, xd, od = dev(w), dev(x), dev(out)
    K.call("fb_gemv_bf16", wd, xd, G * K_, od, N, m, N, K_, group, 0)
    if group:
        want = torch.einsum("mgk,gnk->mgn", x.view(m, G, K_), w.float().view(G, group, K_)).reshape(m, N)
    else:
        want = x @ w.float().t()
    check("gemv", od, want, 2e-3)
    K.call("fb_gemv_bf16", wd, xd, G * K_, od, N, m, N, K_, group, 1)
    check("gemv-acc", od, 2 * want, 4e-3)


@pytest.mark.parametrize("m,N,K_", [(1, 256, 256), (3, 512, 4096), (8, 10240, 384), (2, 200, 128)])
def test_gemv_fp8(K, m, N, K_):
    w = rnd(N, K_, seed=3, scale=0.05)
    q, s = R.quant_fp8_block(w)
    x = rnd(m, K_, seed=4)
    od = torch.zeros(m, N, device="cuda")
    K.call("fb_gemv_fp8", dev(q), dev(s), dev(x), K_, od, N, m, N, K_, 0, 0)
    want = x @ R.dequant_fp8_block(q, s).t()
    check("gemv_fp8", od, want, 2e-3)


def test_rmsnorm_and_add(K):
    n, d = 5, 384
    a, b, w = rnd(n, d, seed=1), rnd(n, d, seed=2), rnd(d, seed=3)
    out, s = torch.zeros(n, d, device="cuda"), torch.zeros(n, d, device="cuda")
    K.call("fb_rmsnorm", dev(a), dev(b), s, dev(w), out, n, d, d, d, 1e-5, None, 0, 0, 0)
    check("sum", s, a + b, 1e-6)
    check("rmsnorm", out, R.rmsnorm(a + b, w, 1e-5), 1e-5)
    K.call("fb_rmsnorm", dev(a), None, None, dev(w), out, n, d, d, d, 1e-5, None, 0, 0, 0)
    check("rmsnorm1", out, R.rmsnorm(a, w, 1e-5), 1e-5)


@pytest.mark.parametrize("H", [128, 4096])
def test_hc_chain(K, H):
    n, mult, mix = 3, 4, 24
    Rr = rnd(n, mult, H, seed=1)
    fn = rnd(mix, mult * H, seed=2, scale=0.05)
    scale = torch.tensor([0.7, 1.3, 0.9])
    base = rnd(mix, seed=3, scale=0.3)
    ln = rnd(H, seed=4).abs() + 0.5
    y = rnd(n, H, seed=5)
    Rd = dev(Rr.clone())
    acc = torch.zeros(n, 25, device="cuda")
    x, xn = torch.zeros(n, H, device="cuda"), torch.zeros(n, H, device="cuda")
    sp = torch.zeros(4, n, H, dtype=torch.int16, device="cuda")
    post, comb = torch.zeros(n, 4, device="cuda"), torch.zeros(n, 16, device="cuda")
    K.call("fb_hc_mix", Rd, dev(fn), acc, n, mult * H, mix)
    K.call("fb_hc_pre_apply", Rd, acc, dev(scale), dev(base), dev(ln), x, xn, post, comb, n, H, mult, 1e-5, 1e-6, 20, sp, H, n * H, 3, None, None, 0)
    check_split("hc xn split", sp, xn, n, H)
    xr, pr, cr = R.hc_pre(Rr, fn, scale, base, 1e-5, 1e-6, 20)
    check("hc x", x, xr, 1e-4)
    check("hc post", post, pr, 1e-5)
    check("hc comb", comb.view(n, 4, 4), cr, 1e-5)
    check("hc xn", xn, R.rmsnorm(xr, ln, 1e-5), 1e-4)
    assert acc.abs().max().item() == 0.0, "accumulator must be cleared for reuse"
    # fused hc_post + next-site mix into a second buffer, then the in-place stand-alone form
    R2 = torch.zeros_like(Rd)
    fn2 = rnd(mix, mult * H, seed=12, scale=0.05)
    K.call("fb_hc_post_mix", Rd, R2, dev(y), post, comb, dev(fn2), acc, n, H, mix)
    Rn = R.hc_post(y, Rr, pr, cr)
    check("hc_post fused", R2, Rn, 1e-4)
    flat = Rn.reshape(n, -1)
    check("mix fused", acc[:, :mix], flat @ fn2.t(), 2e-3)
    check("sumsq fused", acc[:, 24], flat.pow(2).sum(-1), 1e-2, rtol=1e-4)
    acc.zero_()
    K.call("fb_hc_post", Rd, dev(y), post, comb, n, H)
    check("hc_post", Rd, Rn, 1e-4)
    hf, xh = torch.zeros(n, H, device="cuda"), torch.zeros(n, H, device="cuda")
    K.call("fb_hc_head", dev(Rr), dev(ln), hf, xh, n, H, mult, 1e-5, None, 0, 0, 0)
    check("hc_head", hf, Rr.mean(1), 1e-5)
    check("hc_head norm", xh, R.rmsnorm(Rr.mean(1), ln, 1e-5), 1e-5)


def test_embed_and_mtp_prep(K):
    V, H, n = 50, 96, 4
    emb = rnd(V, H, seed=1).bfloat16()
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32)
    out = torch.zeros(n, 4, H, device="cuda")
    K.call("fb_embed_expand", dev(ids), dev(emb), out, n, H, 4, V)
    check("embed", out, emb.float()[ids.long()].unsqueeze(1).repeat(1, 4, 1), 0)
    hp, en, hn = rnd(n, H, seed=2), rnd(H, seed=3), rnd(H, seed=4)
    o2 = torch.zeros(n, 2 * H, device="cuda")
    K.call("fb_mtp_prep", dev(ids), dev(emb), dev(hp), dev(en), dev(hn), o2, n, H, V, 1e-5, None, 0, 0, 0)
    want = torch.cat([R.rmsnorm(emb.float()[ids.long()], en, 1e-5), R.rmsnorm(hp, hn, 1e-5)], -1)
    check("mtp_prep", o2, want, 1e-5)


@pytest.mark.parametrize("dk,H,groups,nbuf,snap", [(32, 2, [3], 4, 1), (64, 3, [1, 2], 1, 0), (128, 2, [5], 4, 0),
                                                   (128, 1, [3, 3], 4, 1)])
def test_gdn_fused(K, dk, H, groups, nbuf, snap):
    r_lr, P = 16, H * dk
    slots = list(range(len(groups)))
    S = len(groups)
    n = sum(groups)
    ld = 3 * P + 2 * r_lr + H
    ld += (-ld) % 4
    b_off = 3 * P + 2 * r_lr
    proj = rnd(n, ld, seed=1)
    fb, gb = rnd(n, P, seed=2), rnd(n, P, seed=3)
    conv_w = rnd(3 * P, 4, seed=4, scale=0.5)
    a_log, dt_bias, o_norm = rnd(H, seed=5, scale=0.3), rnd(P, seed=6, scale=0.3), rnd(dk, seed=7).abs() + 0.5
    state = rnd(S, nbuf, H, dk, dk, seed=8, scale=0.2)
    conv_state = rnd(S, nbuf, 3 * P, 3, seed=9)
    cur = torch.tensor([1 % nbuf] * S, dtype=torch.int32)
    meta, gf, n_, _ = make_meta(K, slots, groups, [10] * S)
    sd, cd = dev(state.clone()), dev(conv_state.clone())
    out = torch.zeros(n, P, device="cuda")
    K.call("fb_gdn_fused", dev(proj), ld, dev(fb), dev(gb), P, dev(conv_w), dev(a_log), dev(dt_bias), dev(o_norm),
           sd, cd, dev(cur), meta, gf, len(groups), out, P, H, dk, b_off, nbuf, snap, -5.0, 1e-5, None, 0, 0, 0,
           None, 0, 0, 0)
    r0 = 0
    for gi, g in enumerate(groups):
        c = int(cur[gi])
        rows = slice(r0, r0 + g)
        co, tail = R.causal_conv1d(proj[rows, :3 * P], conv_w, conv_state[gi, c])
        co = torch.nn.functional.silu(co)
        q, k, v = (co[:, i * P:(i + 1) * P].reshape(g, H, dk) for i in range(3))
        q, k = R.l2norm_heads(q) * dk ** -0.5, R.l2norm_heads(k)
        beta = torch.sigmoid(proj[rows, b_off:b_off + H])
        gl = R.gdn_log_decay(fb[rows], dt_bias, a_log, -5.0, H)
        core, s_new = R.gdn_recurrent(q, k, v, beta, gl, state[gi, c])
        want = R.gated_rmsnorm(core, gb[rows].view(g, H, dk), o_norm, 1e-5).reshape(g, P)
        check(f"gdn out g{gi}", out[rows], want, 2e-4)
        wb = (c + g) % nbuf if (snap and nbuf > 1) else c
        check(f"gdn state g{gi}", sd[gi, wb], s_new, 2e-4)
        check(f"gdn conv g{gi}", cd[gi, wb], tail, 1e-6)
        if snap and nbuf > 1:
            _, s1 = R.gdn_recurrent(q[:1], k[:1], v[:1], beta[:1], gl[:1], state[gi, c])
            check(f"gdn snap0 g{gi}", sd[gi, (c + 1) % nbuf], s1, 2e-4)
            check(f"gdn untouched g{gi}", sd[gi, c], state[gi, c], 0)
        r0 += g


@pytest.mark.parametrize("dk,H,groups", [(128, 2, [70]), (64, 3, [33, 5, 64]), (128, 1, [16, 1])])
def test_gdn_chunk_wy_matches_recurrence(K, dk, H, groups):
    """WY-chunked scan (32 tokens per step) against the fp32 step recurrence, with strong decays (gate floor -5)."""
    r_lr, P, S, n = 16, H * dk, len(groups), sum(groups)
    ld = 3 * P + 2 * r_lr + H
    ld += (-ld) % 4
    b_off = 3 * P + 2 * r_lr
    proj = rnd(n, ld, seed=1)
    fb, gb = rnd(n, P, seed=2, scale=3.0), rnd(n, P, seed=3)        # wide range of decays, down to e^-5 per token
    conv_w = rnd(3 * P, 4, seed=4, scale=0.5)
    a_log, dt_bias, o_norm = rnd(H, seed=5, scale=0.3), rnd(P, seed=6, scale=0.3), rnd(dk, seed=7).abs() + 0.5
    state, conv_state = rnd(S, 1, H, dk, dk, seed=8, scale=0.2), rnd(S, 1, 3 * P, 3, seed=9)
    cur = torch.zeros(S, dtype=torch.int32)
    meta, gf, _, _ = make_meta(K, list(range(S)), groups, [10] * S)
    sd, cd = dev(state.clone()), dev(conv_state.clone())
    out = torch.zeros(n, P, device="cuda")
    K.call("fb_gdn_chunk", dev(proj), ld, dev(fb), dev(gb), P, dev(conv_w), dev(a_log), dev(dt_bias), dev(o_norm),
           sd, cd, dev(cur), meta, gf, S, out, P, H, dk, b_off, 1, -5.0, 1e-5, None, 0, 0, 0)
    torch.cuda.synchronize()
    r0 = 0
    for gi, g in enumerate(groups):
        rows = slice(r0, r0 + g)
        co, tail = R.causal_conv1d(proj[rows, :3 * P], conv_w, conv_state[gi, 0])
        co = torch.nn.functional.silu(co)
        q, k, v = (co[:, i * P:(i + 1) * P].reshape(g, H, dk) for i in range(3))
        q, k = R.l2norm_heads(q) * dk ** -0.5, R.l2norm_heads(k)
        beta = torch.sigmoid(proj[rows, b_off:b_off + H])
        gl = R.gdn_log_decay(fb[rows], dt_bias, a_log, -5.0, H)
        core, s_new = R.gdn_recurrent(q, k, v, beta, gl, state[gi, 0])
        want = R.gated_rmsnorm(core, gb[rows].view(g, H, dk), o_norm, 1e-5).reshape(g, P)
        check(f"wy out g{gi}", out[rows], want, 5e-4)
        check(f"wy state g{gi}", sd[gi, 0], s_new, 5e-4)
        check(f"wy conv g{gi}", cd[gi, 0], tail, 1e-6)
        r0 += g


@pytest.mark.parametrize("E,topk", [(8, 2), (288, 8)])
def test_moe_route(K, E, topk):
    n = 6
    logits = rnd(n, E, seed=1)
    logits[0, 3] = logits[0, 5]  # a tie resolves to the lower index
    bias = rnd(E, seed=2, scale=0.1)
    ids = torch.zeros(n, topk, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n, topk, device="cuda")
    K.call("fb_moe_route", dev(logits), E, dev(bias), ids, wts, n, E, topk, 2.5)
    w_ref, i_ref = R.moe_route(logits, bias, topk, 2.5)
    assert torch.equal(ids.cpu().long(), i_ref), (ids.cpu(), i_ref)
    check("route w", wts, w_ref, 1e-5)


@pytest.mark.parametrize("n,E,topk,I,H", [(1, 8, 2, 128, 256), (3, 16, 8, 256, 4096), (2, 6, 3, 2048, 512)])
def test_moe_experts_fp8(K, n, E, topk, I, H):
    g = torch.Generator().manual_seed(7)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
    w2 = torch.randn(E, H, I, generator=g) * 0.05
    q13, s13 = zip(*[R.quant_fp8_block(w13[e]) for e in range(E)])
    q2, s2 = zip(*[R.quant_fp8_block(w2[e]) for e in range(E)])
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13), torch.stack(q2), torch.stack(s2)
    x = torch.randn(n, H, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(n)]).int()
    wts = torch.rand(n, topk, generator=g)
    act = torch.zeros(n, topk, I, device="cuda")
    out = torch.ones(n, H, device="cuda")
    K.call("fb_moe_gate_up_fp8", dev(q13), dev(s13), dev(x), H, dev(ids), act, n, topk, I, H, 0, E, 10.0)
    K.call("fb_moe_down_fp8", dev(q2), dev(s2), act, dev(ids), dev(wts), out, H, n, topk, I, H, 0, E, 1)
    want = torch.ones(n, H)
    act_ref = torch.zeros(n, topk, I)
    for r in range(n):
        for s in range(topk):
            e = int(ids[r, s])
            W13 = R.dequant_fp8_block(q13[e], s13[e])
            a = R.swiglu_limited(x[r] @ W13[:I].t(), x[r] @ W13[I:].t(), 10.0)
            act_ref[r, s] = a
            want[r] += wts[r, s] * (a @ R.dequant_fp8_block(q2[e], s2[e]).t())
    check("moe act", act, act_ref, 2e-3)
    check("moe out", out, want, 5e-3)
    # expert-parallel masking: experts outside [e_lo, e_lo+cnt) contribute nothing
    lo, cnt = E // 2, E - E // 2
    out2 = torch.zeros(n, H, device="cuda")
    K.call("fb_moe_gate_up_fp8", dev(q13[lo:]), dev(s13[lo:]), dev(x), H, dev(ids), act, n, topk, I, H, lo, cnt, 10.0)
    K.call("fb_moe_down_fp8", dev(q2[lo:]), dev(s2[lo:]), act, dev(ids), dev(wts), out2, H, n, topk, I, H, lo, cnt, 0)
    want2 = torch.zeros(n, H)
    for r in range(n):
        for s in range(topk):
            e = int(ids[r, s])
            if e >= lo:
                want2[r] += wts[r, s] * (act_ref[r, s] @ R.dequant_fp8_block(q2[e], s2[e]).t())
    check("moe ep", out2, want2, 5e-3)


def test_swiglu(K):
    n, I = 3, 300
    gu = rnd(n, 2 * I, seed=1, scale=8.0)
    act = torch.zeros(n, I, device="cuda")
    K.call("fb_swiglu", dev(gu), 2 * I, act, n, I, 10.0)
    check("swiglu", act, R.swiglu_limited(gu[:, :I], gu[:, I:], 10.0), 1e-5)


def test_argmax_and_accept(K):
    n, V = 4, 154880
    logits = rnd(n, V, seed=1)
    logits[1, 77] = logits[1, 9000] = 50.0
    ids = torch.zeros(n, dtype=torch.int32, device="cuda")
    vals = torch.zeros(n, device="cuda")
    part = torch.zeros(n * 64, dtype=torch.int64, device="cuda")
    K.call("fb_argmax", dev(logits), V, part, ids, vals, n, V, 1, 0)
    assert ids.cpu().tolist() == R.argmax_first(logits).tolist()
    check("argmax vals", vals, logits.max(-1).values, 0)
    H, nv, nbuf = 64, 3, 4
    for drafts, judges, k in (([5, 6], [5, 6, 7], 3), ([5, 6], [5, 9, 7], 2), ([5, 6], [1, 6, 7], 1)):
        blk = torch.tensor([11] + drafts, dtype=torch.int32, device="cuda")
        jd = torch.tensor(judges, dtype=torch.int32, device="cuda")
        out = torch.zeros(nv + 1, dtype=torch.int32, device="cuda")
        hf = dev(rnd(nv, H, seed=2))
        mtp_ids = torch.zeros(2, dtype=torch.int32, device="cuda")
        mtp_h = dev(rnd(2, H, seed=3))
        old1 = mtp_h[1].clone()
        gslot = torch.zeros(1, dtype=torch.int32, device="cuda")
        main_len = torch.tensor([100], dtype=torch.int32, device="cuda")
        mtp_len = torch.tensor([101], dtype=torch.int32, device="cuda")
        cur = torch.tensor([3], dtype=torch.int32, device="cuda")
        K.call("fb_mtp_accept", blk, jd, out, hf, mtp_ids, mtp_h, gslot, main_len, mtp_len, cur, 1, nv, H, nbuf)
        torch.cuda.synchronize()
        assert out.tolist() == [k] + judges[:k] + [-1] * (nv - k)
        assert main_len.item() == 100 + k and mtp_len.item() == 98 + k and cur.item() == (3 + k) % nbuf
        assert blk[0].item() == judges[k - 1]
        assert mtp_ids.tolist() == [([11] + drafts)[k - 1], judges[k - 1]]
        check("mtp_h1", mtp_h[1], hf[k - 1], 0)
        check("mtp_h0", mtp_h[0], old1 if k == 1 else hf[k - 2], 0)


def _dsa_setup(K, n_groups_rows, ctx0, kpool, page, ID, IH, DL, max_pages, kv_f32, seed=0):
    """Fill a paged cache for one slot with `ctx0` tokens then append the group's rows."""
    g = torch.Generator().manual_seed(seed)
    total = ctx0 + n_groups_rows
    lat = torch.randn(total, DL, generator=g)
    kidx = torch.randn(total, ID, generator=g)
    kgate = torch.randn(total, ID, generator=g)
    num_pages = max_pages
    perm = torch.randperm(num_pages, generator=g).int()  # scattered physical pages
    pt = perm.view(1, max_pages).contiguous()
    return lat, kidx, kgate, pt, total


@pytest.mark.parametrize("ctx0,n,kpool,select_max", [(0, 7, 4, 8), (37, 3, 4, 4), (200, 1, 4, 16), (41, 2, 2, 64),
                                                      (5000, 3, 4, 512)])
def test_dsa_pool_scores_select(K, ctx0, n, kpool, select_max):
    page, ID, IH, DL = 16, 32, 4, 64
    total = ctx0 + n
    max_pages = (total + page - 1) // page + 2
    lat, kidx, kgate, pt, _ = _dsa_setup(K, n, ctx0, kpool, page, ID, IH, DL, max_pages, True, seed=ctx0 + n)
    g = torch.Generator().manual_seed(99)
    ape = torch.randn(kpool, ID, generator=g)
    qi = torch.randn(n, IH, ID, generator=g)
    wi = torch.rand(n, IH, generator=g)
    # physical caches
    kidx_c = torch.zeros(max_pages, page, ID)
    kgate_c = torch.zeros(max_pages, page, ID)
    for t in range(total):
        pg = int(pt[0, t // page])
        kidx_c[pg, t % page] = kidx[t]
        kgate_c[pg, t % page] = kgate[t]
    pool_c = torch.zeros(max_pages, page // kpool, ID, device="cuda")
    ptd = dev(pt)
    # pools of the cached prefix are filled by "prefill" rows: one forward over all tokens
    meta_all, _, _, _ = make_meta(K, [0], [total], [0])
    K.call("fb_dsa_pool", dev(kidx_c), dev(kgate_c), dev(ape), pool_c, meta_all, ptd, max_pages, page, total, ID, kpool)
    want_pools = R.kpool_compress(kidx, kgate, ape, kpool)
    npools = want_pools.shape[0]
    got_pools = torch.stack([pool_c[int(pt[0, p // (page // kpool)]), p % (page // kpool)] for p in range(npools)])
    check("pool keys", got_pools, want_pools, 1e-5)
    meta, gf, n_, _ = make_meta(K, [0], [n], [ctx0])
    max_pools = npools + 3
    scores = torch.zeros(n, max_pools, device="cuda")
    K.call("fb_dsa_scores", dev(qi.reshape(n, -1)), IH * ID, dev(wi), pool_c, scores, max_pools, meta, ptd, max_pages,
           page, n, IH, ID, kpool, max_pools)
    s_ref = R.indexer_scores(qi, want_pools, wi)
    for i in range(n):
        nvis = min(npools, ctx0 // kpool + i + 1)
        check(f"scores row {i}", scores[i, :nvis], s_ref[i, :nvis], 1e-4)
    # selection is exact on the device's own scores
    W = select_max * kpool + kpool + 3
    idx = torch.full((n, W), -7, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(n, dtype=torch.int32, device="cuda")
    K.call("fb_dsa_select", scores, max_pools, idx, W, cnt, meta, n, kpool, select_max)
    sc = scores.cpu()
    for i in range(n):
        nvis = min(npools, ctx0 // kpool + i + 1)
        select_k = min(select_max, npools)
        s = torch.full((npools,), float("-inf"))
        s[:nvis] = sc[i, :nvis]
        order = torch.sort(s, descending=True, stable=True).indices[:select_k]
        pools = torch.tensor([int(p) if s[p] != float("-inf") else -1 for p in order]).view(1, -1)
        # expand_pool_indices takes ctx0 of row 0; a single row at offset i is ctx0 + i
        ref = R.expand_pool_indices(pools, kpool, ctx0 + i, total, select_k * kpool + kpool - 1)
        want = sorted(set(int(t) for t in ref[0] if t >= 0))
        got = idx[i, :int(cnt[i])].cpu().tolist()
        assert got == want, f"row {i}: got {got[:12]}... ({len(got)}) want {want[:12]}... ({len(want)})"


@pytest.mark.parametrize("hl,DL,kv_f32,ntok,nshard", [(4, 64, 1, 37, 1), (3, 64, 0, 5, 1), (64, 512, 0, 300, 1),
                                                      (8, 512, 1, 70, 1), (4, 64, 1, 90, 2), (16, 512, 0, 130, 4)])
def test_dsa_attention(K, hl, DL, kv_f32, ntok, nshard):
    page, n = 16, 2
    T = 400
    max_pages = T // page
    g = torch.Generator().manual_seed(hl + DL + ntok)
    lat = torch.randn(T, DL, generator=g)
    if not kv_f32:
        lat = lat.bfloat16().float()
    pt = torch.randperm(max_pages, generator=g).int().view(1, max_pages)
    cache = torch.zeros(max_pages, page, DL)
    for t in range(T):
        cache[int(pt[0, t // page]), t % page] = lat[t]
    cache_d = dev(cache if kv_f32 else cache.bfloat16())
    qabs = torch.randn(n, hl, DL, generator=g) * 0.3
    W = ntok + 8
    idx = torch.full((n, W), -1, dtype=torch.int32)
    cnt = torch.tensor([ntok, max(1, ntok // 2)], dtype=torch.int32)
    for i in range(n):
        idx[i, :int(cnt[i])] = torch.randperm(T, generator=g)[:int(cnt[i])].int()
    meta, _, _, _ = make_meta(K, [0], [n], [T - n])
    scale = 0.11
    nsplit = 4
    parts_o, parts_ml = [], []
    for sh in range(nshard):
        o_part = torch.zeros(n, nsplit, hl, DL, device="cuda")
        ml = torch.zeros(n, nsplit, hl, 2, device="cuda")
        K.call("fb_dsa_attn_partial", dev(qabs.reshape(n, -1)), cache_d, dev(idx), W, dev(cnt), o_part, ml, meta,
               dev(pt), max_pages, page, n, hl, DL, nsplit, sh, nshard, scale, kv_f32)
        ctx = torch.zeros(n, hl, DL, device="cuda")
        lse = torch.zeros(n, hl, 2, device="cuda")
        K.call("fb_dsa_attn_merge", o_part, ml, ctx, lse, n, hl, DL, nsplit, 1 if nshard == 1 else 0, None, 0, 0, 0)
        parts_o.append(ctx)
        parts_ml.append(lse)
    if nshard > 1:  # cross-shard merge is the same merge over [n, nshard, hl, *]
        o_all = torch.stack(parts_o, 1).contiguous()
        ml_all = torch.stack(parts_ml, 1).contiguous()
        ctx = torch.zeros(n, hl, DL, device="cuda")
        K.call("fb_dsa_attn_merge", o_all, ml_all, ctx, None, n, hl, DL, nshard, 1, None, 0, 0, 0)
    want = torch.zeros(n, hl, DL)
    for i in range(n):
        ids = idx[i, :int(cnt[i])].long()
        s = torch.einsum("hd,td->ht", qabs[i], lat[ids]) * scale
        p = torch.softmax(s, -1)
        want[i] = p @ lat[ids]
    check("dsa attn", ctx, want, 2e-4)


@pytest.mark.parametrize("hl,ntok,nsplit,nshard", [(64, 300, 4, 1), (64, 1024, 32, 1), (16, 130, 4, 4), (8, 70, 2, 1),
                                                    (32, 2048, 32, 2)])
def test_dsa_attention_tensor_core(K, hl, ntok, nsplit, nshard):
    """mma.sync form of the sparse MLA attention (bf16 latents, DL = 512) against the fp32 statement."""
    page, n, DL = 16, 3, 512
    T = 2304
    max_pages = T // page
    g = torch.Generator().manual_seed(hl + ntok)
    lat = torch.randn(T, DL, generator=g).bfloat16().float()
    pt = torch.randperm(max_pages, generator=g).int().view(1, max_pages)
    cache = torch.zeros(max_pages, page, DL)
    cache[pt[0].long().repeat_interleave(page), torch.arange(T) % page] = lat
    cache_d = dev(cache.bfloat16())
    qabs = torch.randn(n, hl, DL, generator=g) * 0.3
    W = ntok + 8
    idx = torch.full((n, W), -1, dtype=torch.int32)
    cnt = torch.tensor([ntok, max(1, ntok // 2), 1], dtype=torch.int32)
    for i in range(n):
        idx[i, :int(cnt[i])] = torch.randperm(T, generator=g)[:int(cnt[i])].int()
    meta, _, _, _ = make_meta(K, [0], [n], [T - n])
    scale = 0.11
    parts_o, parts_ml = [], []
    for sh in range(nshard):
        o_part = torch.full((n, nsplit, hl, DL), float("nan"), device="cuda")
        ml = torch.full((n, nsplit, hl, 2), float("nan"), device="cuda")
        K.call("fb_dsa_attn_partial_tc", dev(qabs.reshape(n, -1)), cache_d, dev(idx), W, dev(cnt), o_part, ml, meta,
               dev(pt), max_pages, page, n, hl, DL, nsplit, sh, nshard, scale)
        ctx = torch.zeros(n, hl, DL, device="cuda")
        lse = torch.zeros(n, hl, 2, device="cuda")
        K.call("fb_dsa_attn_merge", o_part, ml, ctx, lse, n, hl, DL, nsplit, 1 if nshard == 1 else 0, None, 0, 0, 0)
        parts_o.append(ctx)
        parts_ml.append(lse)
    if nshard > 1:
        o_all = torch.stack(parts_o, 1).contiguous()
        ml_all = torch.stack(parts_ml, 1).contiguous()
        ctx = torch.zeros(n, hl, DL, device="cuda")
        K.call("fb_dsa_attn_merge", o_all, ml_all, ctx, None, n, hl, DL, nshard, 1, None, 0, 0, 0)
    want = torch.zeros(n, hl, DL)
    for i in range(n):
        ids = idx[i, :int(cnt[i])].long()
        s = torch.einsum("hd,td->ht", qabs[i], lat[ids]) * scale
        want[i] = torch.softmax(s, -1) @ lat[ids]
    check("dsa attn tc", ctx, want, 6e-3, rtol=1e-2)   # probabilities are rounded to bf16 for the P.L product


@pytest.mark.parametrize("m,N,K_,group", [(1, 48, 64, 0), (3, 4100, 512, 0), (8, 9600, 128, 0), (2, 16 * 64, 64, 64),
                                          (5, 777, 4096, 0), (3, 24896, 4096, 0)])
def test_gemv_mma_bf16(K, m, N, K_, group):
    G = N // group if group else 1
    w = rnd(N, K_, seed=1, scale=0.1).bfloat16()
    x = rnd(m, G * K_, seed=2)
    xs = dev(to_split(x))
    od = torch.full((m, N), 7.0, device="cuda")
    osp = torch.zeros(4, m, N, dtype=torch.int16, device="cuda")
    K.call("fb_gemv_mma_bf16", dev(w), xs, G * K_, m * G * K_, od, N, m, N, K_, group, 0, osp, N, m * N, 3)
    if group:
        want = torch.einsum("mgk,gnk->mgn", x.view(m, G, K_), w.float().view(G, group, K_)).reshape(m, N)
    else:
        want = x @ w.float().t()
    check("gemv mma", od, want, 2e-3)
    check_split("gemv mma split out", osp, od, m, N)
    K.call("fb_gemv_mma_bf16", dev(w), xs, G * K_, m * G * K_, od, N, m, N, K_, group, 1, None, 0, 0, 0)
    check("gemv mma acc", od, 2 * want, 4e-3)
    # the split conversion kernel agrees with the host-side split
    sp2 = torch.zeros(4, m, G * K_, dtype=torch.int16, device="cuda")
    K.call("fb_split_rows", dev(x), G * K_, sp2, G * K_, m * G * K_, 3, m, G * K_)
    assert torch.equal(sp2.cpu(), to_split(x))


@pytest.mark.parametrize("m,N,K_", [(1, 256, 256), (3, 512, 4096), (8, 10240, 384), (2, 200, 128)])
def test_gemv_mma_fp8(K, m, N, K_):
    w = rnd(N, K_, seed=3, scale=0.05)
    q, s = R.quant_fp8_block(w)
    x = rnd(m, K_, seed=4)
    od = torch.zeros(m, N, device="cuda")
    K.call("fb_gemv_mma_fp8", dev(q), dev(s), dev(to_split(x)), K_, m * K_, od, N, m, N, K_, 0, None, 0, 0, 0)
    # e4m3 weights run with f16 (11-bit) activations: tolerance is relative to the output scale
    want = x @ R.dequant_fp8_block(q, s).t()
    check("gemv mma fp8", od, want, 2e-3 * want.abs().max().item())


@pytest.mark.parametrize("n,E,topk,I,H", [(1, 8, 2, 128, 256), (3, 16, 8, 256, 4096), (2, 6, 3, 2048, 512)])
def test_moe_experts_mma(K, n, E, topk, I, H):
    g = torch.Generator().manual_seed(7)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
    w2 = torch.randn(E, H, I, generator=g) * 0.05
    q13, s13 = zip(*[R.quant_fp8_block(w13[e]) for e in range(E)])
    q2, s2 = zip(*[R.quant_fp8_block(w2[e]) for e in range(E)])
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13), torch.stack(q2), torch.stack(s2)
    x = torch.randn(n, H, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(n)]).int()
    wts = torch.rand(n, topk, generator=g)
    asp = torch.zeros(4, n * topk, I, dtype=torch.int16, device="cuda")
    out = torch.ones(n, H, device="cuda")
    lo, cnt = 0, E
    K.call("fb_moe_gate_up_mma", dev(q13), dev(s13), dev(to_split(x)), H, n * H, dev(ids), dev(wts), asp, I, n * topk * I,
           n, topk, I, H, lo, cnt, 10.0)
    K.call("fb_moe_down_mma", dev(q2), dev(s2), asp, I, n * topk * I, dev(ids), out, H, n, topk, I, H, lo, cnt, 1,
           None, 0, 0, 0)
    want = torch.ones(n, H)
    act_ref = torch.zeros(n * topk, I)
    for r in range(n):
        for s in range(topk):
            e = int(ids[r, s])
            W13 = R.dequant_fp8_block(q13[e], s13[e])
            a = R.swiglu_limited(x[r] @ W13[:I].t(), x[r] @ W13[I:].t(), 10.0) * wts[r, s]
            act_ref[r * topk + s] = a
            want[r] += a @ R.dequant_fp8_block(q2[e], s2[e]).t()
    check("moe mma act", unsplit(asp.cpu(), 1), act_ref, 2e-3 * act_ref.abs().max().item())
    check("moe mma out", out, want, 3e-3 * want.abs().max().item())
    # expert-parallel masking
    lo, cnt = E // 2, E - E // 2
    out2 = torch.zeros(n, H, device="cuda")
    K.call("fb_moe_gate_up_mma", dev(q13[lo:]), dev(s13[lo:]), dev(to_split(x)), H, n * H, dev(ids), dev(wts), asp, I,
           n * topk * I, n, topk, I, H, lo, cnt, 10.0)
    K.call("fb_moe_down_mma", dev(q2[lo:]), dev(s2[lo:]), asp, I, n * topk * I, dev(ids), out2, H, n, topk, I, H, lo,
           cnt, 0, None, 0, 0, 0)
    want2 = torch.zeros(n, H)
    for r in range(n):
        for s in range(topk):
            e = int(ids[r, s])
            if e >= lo:
                want2[r] += act_ref[r * topk + s] @ R.dequant_fp8_block(q2[e], s2[e]).t()
    check("moe mma ep", out2, want2, 3e-3 * want2.abs().max().item())


@pytest.mark.parametrize("n,E,topk,I,H,lo", [(20, 16, 4, 128, 256, 0), (64, 12, 8, 256, 512, 0), (33, 16, 4, 128, 256, 8)])
def test_moe_experts_grouped_equals_per_pair(K, n, E, topk, I, H, lo):
    """Expert-grouped kernels (prefill) give the same rows as the per-pair kernels (decode)."""
    g = torch.Generator().manual_seed(17)
    cnt = E - lo
    q13, s13 = zip(*[R.quant_fp8_block(torch.randn(2 * I, H, generator=g) * 0.05) for _ in range(cnt)])
    q2, s2 = zip(*[R.quant_fp8_block(torch.randn(H, I, generator=g) * 0.05) for _ in range(cnt)])
    q13, s13, q2, s2 = dev(torch.stack(q13)), dev(torch.stack(s13)), dev(torch.stack(q2)), dev(torch.stack(s2))
    x = torch.randn(n, H, generator=g)
    ids = dev(torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(n)]).int())
    wts = dev(torch.rand(n, topk, generator=g))
    xs = dev(to_split(x))
    npair = n * topk
    asp = torch.zeros(4, npair, I, dtype=torch.int16, device="cuda")
    want = torch.full((n, H), 0.5, device="cuda")
    K.call("fb_moe_gate_up_mma", q13, s13, xs, H, n * H, ids, wts, asp, I, npair * I, n, topk, I, H, lo, cnt, 10.0)
    K.call("fb_moe_down_mma", q2, s2, asp, I, npair * I, ids, want, H, n, topk, I, H, lo, cnt, 1, None, 0, 0, 0)
    asp2 = torch.zeros_like(asp)
    gp = torch.zeros(npair * 8, dtype=torch.int32, device="cuda")
    ge = torch.zeros(npair, dtype=torch.int32, device="cuda")
    ng = torch.zeros(1, dtype=torch.int32, device="cuda")
    yp = torch.full((npair, H), float("nan"), device="cuda")
    got = torch.full((n, H), 0.5, device="cuda")
    K.call("fb_moe_group", ids, npair, lo, cnt, gp, ge, ng, npair)
    K.call("fb_moe_gate_up_grp", q13, s13, xs, H, n * H, wts, gp, ge, ng, asp2, I, npair * I, npair, topk, I, H, 10.0)
    K.call("fb_moe_down_grp", q2, s2, asp2, I, npair * I, gp, ge, ng, yp, npair, I, H)
    K.call("fb_moe_sum_pairs", yp, ids, got, H, n, topk, H, lo, cnt, 1)
    torch.cuda.synchronize()
    local = ((ids >= lo) & (ids < lo + cnt)).flatten()
    groups = gp.view(-1, 8)[:int(ng)]
    members = groups[groups >= 0]
    assert sorted(members.tolist()) == local.nonzero().flatten().tolist()      # every local pair in exactly one group
    assert all(len(set(ids.flatten()[gr[gr >= 0]].tolist())) == 1 for gr in groups)   # one expert per group
    check("grouped act", unsplit(asp2.cpu(), 1)[local.cpu()], unsplit(asp.cpu(), 1)[local.cpu()], 1e-6)
    check("grouped out", got, want, 1e-4 * want.abs().max().item())


@pytest.mark.parametrize("M,N,K_", [(5, 300, 256), (16, 128, 64), (64, 4096, 4096), (300, 1000, 512), (1, 129, 1536),
                                    (130, 256, 8192)])
def test_gemm_tcgen05_bf16(K, M, N, K_):
    """TMA + tcgen05 GEMM (weights as the A operand) against fp32 matmul of the same bf16 inputs."""
    w = rnd(N, K_, seed=1, scale=0.1).bfloat16()
    x = rnd(M, K_, seed=2).bfloat16()
    out = torch.full((M, N), 3.0, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    K.call("fb_gemm_tc_bf16", dev(w), dev(x), K_, out, N, M, N, K_, 0, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, f"kernel reported {status.tolist()}"
    want = x.float() @ w.float().t()
    check("gemm tc", out, want, 2e-3 * max(1.0, want.abs().max().item()))
    K.call("fb_gemm_tc_bf16", dev(w), dev(x), K_, out, N, M, N, K_, 1, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    check("gemm tc acc", out, 2 * want, 4e-3 * max(1.0, want.abs().max().item()))


@pytest.mark.parametrize("M,G,gr,K_", [(40, 2, 1024, 128), (300, 8, 512, 192), (17, 4, 256, 512)])
def test_gemm_tcgen05_block_diagonal(K, M, G, gr, K_):
    """Grouped form of the tcgen05 GEMM: rows of group g contract with x columns [g K, (g + 1) K)."""
    w = rnd(G * gr, K_, seed=3, scale=0.1).bfloat16()
    x = rnd(M, G * K_ + 64, seed=4).bfloat16()            # wider rows than the groups use
    out = torch.zeros(M, G * gr, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    K.call("fb_gemm_tc_bf16_grouped", dev(w), dev(x), x.shape[1], out, G * gr, M, G * gr, K_, gr, 0, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, f"kernel reported {status.tolist()}"
    want = torch.cat([x[:, g * K_:(g + 1) * K_].float() @ w[g * gr:(g + 1) * gr].float().t() for g in range(G)], dim=1)
    check("gemm tc grouped", out, want, 2e-3 * max(1.0, want.abs().max().item()))


@pytest.mark.parametrize("fp8", [False, True])
def test_gemv_ar_fold_single_rank(K, fp8):
    """Fused GEMV + hyper-connection fold (world = 1: no collective) against the separate ops."""
    from ferrite_b200.models.glm import Act
    from ferrite_b200.parallel.symm import FusedGemvAllReduce
    m, N, Kd, mix = 5, 4096, 1024, 24
    W = rnd(N, Kd, seed=1, scale=0.05)
    x = Act(torch.device("cuda"), 8, Kd)
    x.f.copy_(dev(rnd(8, Kd, seed=2)))
    K.call("fb_split_rows", x.f, Kd, *x.sp(3), 8, Kd)
    Rin, y0 = dev(rnd(8, 4, N, seed=3)), dev(rnd(8, N, seed=4))
    post, comb = dev(rnd(8, 4, seed=5).abs()), dev(rnd(8, 4, 4, seed=6).abs())
    fn = dev(rnd(mix, 4 * N, seed=7, scale=0.02))
    if fp8:
        wq, ws_ = R.quant_fp8_block(W)
        wdev, sdev, wref = wq.cuda(), ws_.cuda(), R.dequant_fp8_block(wq, ws_)
    else:
        wdev, sdev, wref = W.to(torch.bfloat16).cuda(), None, W.to(torch.bfloat16).float()
    y = y0.clone()
    Rout = torch.zeros_like(Rin)
    acc = torch.zeros(8, 25, device="cuda")
    f = FusedGemvAllReduce(torch.device("cuda"), 0, 1)
    f(wdev, sdev, x.s, Kd, x.plane, y, N, m, N, Kd, True, True, (Rin, Rout, post, comb, fn, acc, mix))
    want_y = x.f[:m].cpu() @ wref.t() + y0[:m].cpu()
    tol = 3e-2 if fp8 else 2e-3
    check("gemv_ar y", y[:m], want_y, tol * want_y.abs().max().item())
    want_R = R.hc_post(want_y, Rin[:m].cpu(), post[:m].cpu(), comb[:m].cpu())
    check("gemv_ar R'", Rout[:m], want_R, tol * want_R.abs().max().item())
    flat = want_R.reshape(m, -1)
    part, part_n, ld = f.partials()
    nt = part_n[:m].cpu().tolist()
    assert len(set(nt)) == 1 and nt[0] in (N // 16, N // 32) and not part_n[m:].any()
    sums = part[:8 * 25 * ld].view(8, 25, ld)[:m, :, :nt[0]].sum(-1)
    check("gemv_ar mix", sums[:, :mix], flat @ fn.cpu().t(), tol * (flat @ fn.cpu().t()).abs().max().item())
    check("gemv_ar sumsq", sums[:, 24], flat.pow(2).sum(-1), tol * flat.pow(2).sum(-1).max().item())
    assert not Rout[m:].any() and not acc.any()
    # the consumer adds the partials to its accumulator and clears the tile count
    Rd = Rout[:m].contiguous()
    xn = torch.zeros(m, N, device="cuda")
    po, co = torch.zeros(m, 4, device="cuda"), torch.zeros(m, 16, device="cuda")
    scale, base, ln = torch.ones(3, device="cuda"), torch.zeros(mix, device="cuda"), torch.ones(N, device="cuda")
    K.call("fb_hc_pre_apply", Rd, acc, scale, base, ln, None, xn, po, co, m, N, 4, 1e-5, 1e-6, 20, None, 0, 0, 0, part, part_n, ld)
    xr, pr, cr = R.hc_pre(want_R, fn.cpu(), scale.cpu(), base.cpu(), 1e-5, 1e-6, 20)
    check("gemv_ar -> hc_pre post", po, pr, 5 * tol)
    check("gemv_ar -> hc_pre comb", co, cr.reshape(m, 16), 5 * tol)
    assert not part_n.any() and not acc.any()


@pytest.mark.parametrize("fp8,N,Kd,m", [(False, 4096, 1024, 3), (True, 4096, 2048, 2), (False, 2048, 4096, 1)])
def test_gemv_ar_swiglu_source_and_front(K, fp8, N, Kd, m):
    """One launch: SwiGLU as the activation source + GEMV + hyper-connection fold + the NEXT site's hc_pre
    (coefficients by the last CTA at a grid barrier, x from the Gram matrix), against the separate fp32 ops."""
    from ferrite_b200.models.glm import Act
    from ferrite_b200.parallel.symm import FusedGemvAllReduce
    mix = 24
    W = rnd(N, Kd, seed=1, scale=0.05)
    gu = dev(rnd(8, 2 * Kd + 8, seed=2, scale=2.0))          # [gate | up] rows with a padded stride
    act = R.swiglu_limited(gu[:m, :Kd].cpu(), gu[:m, Kd:2 * Kd].cpu(), 10.0)
    Rin, y0 = dev(rnd(8, 4, N, seed=3)), dev(rnd(8, N, seed=4))
    post, comb = dev(rnd(8, 4, seed=5).abs()), dev(rnd(8, 4, 4, seed=6).abs())
    fn = dev(rnd(mix, 4 * N, seed=7, scale=0.02))
    scale, base, ln = dev(rnd(3, seed=8).abs() + 0.5), dev(rnd(mix, seed=9, scale=0.3)), dev(rnd(N, seed=10).abs() + 0.5)
    if fp8:
        wq, ws_ = R.quant_fp8_block(W)
        wdev, sdev, wref = wq.cuda(), ws_.cuda(), R.dequant_fp8_block(wq, ws_)
    else:
        wdev, sdev, wref = W.to(torch.bfloat16).cuda(), None, W.to(torch.bfloat16).float()
    y = y0.clone()
    Rout = torch.zeros_like(Rin)
    acc = torch.zeros(8, 25, device="cuda")
    xo = Act(torch.device("cuda"), 8, N)
    npost, ncomb = torch.zeros(8, 4, device="cuda"), torch.zeros(8, 16, device="cuda")
    f = FusedGemvAllReduce(torch.device("cuda"), 0, 1)
    for rep in range(2):      # twice: the barrier's generation and arrival counters must re-arm
        y.copy_(y0)
        f(wdev, sdev, None, Kd, 0, y, N, m, N, Kd, True, True, (Rin, Rout, post, comb, fn, acc, mix),
          swiglu=(gu, 2 * Kd + 8, Kd, 10.0),
          front=(scale, base, ln, npost, ncomb, xo.f, xo.sp(3), 1e-5, 1e-6, 20))
        torch.cuda.synchronize()
        f.check()
    want_y = act @ wref.t() + y0[:m].cpu()
    tol = 3e-2 if fp8 else 2e-3
    check("y", y[:m], want_y, tol * want_y.abs().max().item())
    want_R = R.hc_post(want_y, Rin[:m].cpu(), post[:m].cpu(), comb[:m].cpu())
    check("R'", Rout[:m], want_R, tol * want_R.abs().max().item())
    # the front is checked against the fp32 statement applied to the DEVICE's R' (isolates it from the GEMV error)
    xr, pr, cr = R.hc_pre(Rout[:m].cpu(), fn.cpu(), scale.cpu(), base.cpu(), 1e-5, 1e-6, 20)
    xn = R.rmsnorm(xr, ln.cpu(), 1e-5)
    check("front post", npost[:m], pr, 2e-4)
    check("front comb", ncomb[:m], cr.reshape(m, 16), 2e-4)
    check("front x", xo.f[:m], xn, 5e-4 * max(1.0, xn.abs().max().item()))
    hi = xo.s[0, :m].view(torch.bfloat16).float() + xo.s[1, :m].view(torch.bfloat16).float()
    check("front x split", hi, xn, 5e-4 * max(1.0, xn.abs().max().item()))
    assert not xo.f[m:].any() and not npost[m:].any()


@pytest.mark.parametrize("N,m", [(4096, 3), (2048, 1), (4096, 8)])
def test_hc_pre_wide_from_gram_partials(K, N, m):
    """Column-parallel hyper-connection front fed by the fused GEMV's partials (mix dots, sum of squares, Gram)
    against the fp32 statement applied to the device's R'."""
    from ferrite_b200.models.glm import Act
    from ferrite_b200.parallel.symm import FusedGemvAllReduce
    Kd, mix = 512, 24
    W = rnd(N, Kd, seed=1, scale=0.05).to(torch.bfloat16)
    x = Act(torch.device("cuda"), 8, Kd)
    x.f.copy_(dev(rnd(8, Kd, seed=2)))
    K.call("fb_split_rows", x.f, Kd, *x.sp(3), 8, Kd)
    Rin = dev(rnd(8, 4, N, seed=3))
    post, comb = dev(rnd(8, 4, seed=5).abs()), dev(rnd(8, 4, 4, seed=6).abs())
    fn = dev(rnd(mix, 4 * N, seed=7, scale=0.02))
    scale, base, ln = dev(rnd(3, seed=8).abs() + 0.5), dev(rnd(mix, seed=9, scale=0.3)), dev(rnd(N, seed=10).abs() + 0.5)
    y, Rout, acc = torch.zeros(8, N, device="cuda"), torch.zeros_like(Rin), torch.zeros(8, 25, device="cuda")
    xo = Act(torch.device("cuda"), 8, N)
    npost, ncomb = torch.zeros(8, 4, device="cuda"), torch.zeros(8, 16, device="cuda")
    f = FusedGemvAllReduce(torch.device("cuda"), 0, 1)
    f(dev(W), None, x.s, Kd, x.plane, y, N, m, N, Kd, False, True, (Rin, Rout, post, comb, fn, acc, mix), gram=True)
    part, gram, part_n, ld = f.wide_partials()
    K.call("fb_hc_pre_wide", Rout, part, gram, part_n, ld, scale, base, ln, xo.f, npost, ncomb, m, N, mix, 1e-5, 1e-6, 20,
           *xo.sp(3))
    torch.cuda.synchronize()
    xr, pr, cr = R.hc_pre(Rout[:m].cpu(), fn.cpu(), scale.cpu(), base.cpu(), 1e-5, 1e-6, 20)
    xn = R.rmsnorm(xr, ln.cpu(), 1e-5)
    check("wide post", npost[:m], pr, 2e-4)
    check("wide comb", ncomb[:m], cr.reshape(m, 16), 2e-4)
    check("wide x", xo.f[:m], xn, 5e-4 * max(1.0, xn.abs().max().item()))
    hi = xo.s[0, :m].view(torch.bfloat16).float() + xo.s[1, :m].view(torch.bfloat16).float()
    check("wide x split", hi, xn, 5e-4 * max(1.0, xn.abs().max().item()))
    assert not xo.f[m:].any() and part_n[:m].tolist() == [N // 16] * m


def test_router_gemv_routes_in_its_tail(K):
    """[router | shared gate | shared up] GEMV whose last router CTA also routes: ids / weights equal the
    stand-alone route kernel run on the same logits."""
    from ferrite_b200.models.glm import Act
    n, E, Is, H, topk = 3, 288, 256, 1024, 8
    W = (rnd(E + 2 * Is, H, seed=1, scale=0.05)).to(torch.bfloat16)
    x = Act(torch.device("cuda"), 8, H)
    x.f.copy_(dev(rnd(8, H, seed=2)))
    K.call("fb_split_rows", x.f, H, *x.sp(3), 8, H)
    bias = dev(rnd(E, seed=3, scale=0.1))
    ldl = E + 2 * Is
    lg = torch.zeros(8, ldl, device="cuda")
    ids, wts = torch.zeros(8, topk, dtype=torch.int32, device="cuda"), torch.zeros(8, topk, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    for rep in range(2):
        K.call("fb_gemv_mma_bf16_route", dev(W), x.s, H, x.plane, lg, ldl, n, ldl, H, bias, ids, wts, ticket, E, topk, 2.5)
    torch.cuda.synchronize()
    want = x.f[:n].cpu() @ W.float().t()
    check("router gemv", lg[:n], want, 2e-3 * want.abs().max().item())
    ids2, wts2 = torch.zeros_like(ids), torch.zeros_like(wts)
    K.call("fb_moe_route", lg, ldl, bias, ids2, wts2, n, E, topk, 2.5)
    assert torch.equal(ids[:n], ids2[:n]) and ticket.item() == 0
    check("route w", wts[:n], wts2[:n].cpu(), 1e-6)
    w_ref, i_ref = R.moe_route(lg[:n, :E].cpu(), bias.cpu(), topk, 2.5)
    assert torch.equal(ids[:n].cpu().long(), i_ref)


@pytest.mark.parametrize("dk,H,groups", [(128, 2, [3]), (64, 3, [1, 2])])
def test_gdn_fused_applies_low_rank_projections(K, dk, H, groups):
    """fb / gb computed inside the GatedDeltaNet kernel from f_a | g_a outputs == GEMV first, then the kernel."""
    lr, P, n, S = 64, H * dk, sum(groups), len(groups)
    ld = 3 * P + 2 * lr + H
    ld += (-ld) % 4
    b_off = 3 * P + 2 * lr
    proj = rnd(n, ld, seed=1)
    fgw = (rnd(2 * P, lr, seed=2, scale=0.2)).to(torch.bfloat16)
    fa, ga = proj[:, 3 * P:3 * P + lr], proj[:, 3 * P + lr:3 * P + 2 * lr]
    fb, gb = fa @ fgw[:P].float().t(), ga @ fgw[P:].float().t()
    conv_w = rnd(3 * P, 4, seed=4, scale=0.5)
    a_log, dt_bias, o_norm = rnd(H, seed=5, scale=0.3), rnd(P, seed=6, scale=0.3), rnd(dk, seed=7).abs() + 0.5
    state, conv_state = rnd(S, 1, H, dk, dk, seed=8, scale=0.2), rnd(S, 1, 3 * P, 3, seed=9)
    cur = torch.zeros(S, dtype=torch.int32)
    meta, gf, _, _ = make_meta(K, list(range(S)), groups, [10] * S)
    outs = []
    for own in (False, True):
        sd, cd = dev(state.clone()), dev(conv_state.clone())
        out = torch.zeros(n, P, device="cuda")
        K.call("fb_gdn_fused", dev(proj), ld, dev(fb), dev(gb), P, dev(conv_w), dev(a_log), dev(dt_bias), dev(o_norm),
               sd, cd, dev(cur), meta, gf, S, out, P, H, dk, b_off, 1, 0, -5.0, 1e-5, None, 0, 0, 0,
               dev(fgw) if own else None, 3 * P, lr, max(groups))
        outs.append((out, sd))
    check("gdn own-fg out", outs[1][0], outs[0][0].cpu(), 1e-4)
    check("gdn own-fg state", outs[1][1], outs[0][1].cpu(), 1e-4)


def test_bounded_wait_reports_timeout_and_context_survives(K):
    """Failure detection without a fault: a wait on a flag that nothing sets runs out of polls,
    writes {TIMEOUT, -1, wanted, polls} to the status word and returns; the context stays usable."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.full((4,), -7, dtype=torch.int32, device="cuda")
    K.call("fb_wait_flag", flag, 5, 2000, status)      # wants stamp 5, flag stays 0: gives up after 2000 polls
    torch.cuda.synchronize()
    s = status.tolist()
    assert s[0] == 1 and s[1] == -1 and s[2] == 5 and s[3] > 2000
    flag.fill_(5)
    K.call("fb_wait_flag", flag, 5, 2000, status)      # satisfied at once
    torch.cuda.synchronize()
    assert status[0].item() == 0
    x = torch.arange(8, device="cuda").sum().item()    # the context still runs kernels
    assert x == 28


def test_gumbel_sampling_matches_reference_and_distribution(K):
    n, V = 4, 5000
    logits = rnd(n, V, seed=3) * 2.0
    keys = torch.tensor([17, 18, 900, 5])
    meta = torch.zeros(n, 8, dtype=torch.int32)
    meta[:, 1] = keys
    part = torch.zeros(n * 64, dtype=torch.int64, device="cuda")
    ids = torch.zeros(n, dtype=torch.int32, device="cuda")
    K.call("fb_sample_gumbel", dev(logits), V, part, ids, n, V, 1, 0, 0.7, 1234, dev(meta), 1)
    want = R.sample_gumbel(logits, 0.7, 1234, keys)
    assert ids.cpu().tolist() == want.tolist()
    # vocab-sliced: partial keys of two halves merge to the same draw
    half = V // 2
    p0 = torch.zeros(n * 64, dtype=torch.int64, device="cuda")
    p1 = torch.zeros(n * 64, dtype=torch.int64, device="cuda")
    K.call("fb_sample_gumbel", dev(logits[:, :half].contiguous()), half, p0, None, n, half, 1, 0, 0.7, 1234, dev(meta), 0)
    K.call("fb_sample_gumbel", dev(logits[:, half:].contiguous()), half, p1, None, n, half, 1, half, 0.7, 1234, dev(meta), 0)
    m64 = (1 << 64) - 1
    for r in range(n):
        keys_r = [int(k) & m64 for k in p0.view(n, 64)[r].tolist() + p1.view(n, 64)[r].tolist()]
        assert 0xFFFFFFFF - (max(keys_r) & 0xFFFFFFFF) == int(want[r])
    # draws over many positions follow softmax(logits / T)
    V2, draws = 6, 4000
    lg = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, 1.5]]).repeat(draws, 1)
    meta2 = torch.zeros(draws, 8, dtype=torch.int32)
    meta2[:, 1] = torch.arange(draws)
    part2 = torch.zeros(draws * 64, dtype=torch.int64, device="cuda")
    ids2 = torch.zeros(draws, dtype=torch.int32, device="cuda")
    K.call("fb_sample_gumbel", dev(lg), V2, part2, ids2, draws, V2, 1, 0, 1.0, 7, dev(meta2), 1)
    freq = torch.bincount(ids2.cpu().long(), minlength=V2).float() / draws
    assert (freq - torch.softmax(lg[0], -1)).abs().max().item() < 0.03


def test_device_runtime_fork_join_capture_replay(K):
    """Side-stream fork/join inside a captured step, replayed as a graph, with pinned staging."""
    import ctypes
    from ferrite_b200.utils.devrt import DeviceRuntime
    rt = DeviceRuntime(0, n_side=2)
    a, b = torch.full((4096,), 1.0, device="cuda"), torch.full((4096,), 2.0, device="cuda")
    c, d = torch.zeros(4096, device="cuda"), torch.zeros(4096, device="cuda")
    torch.cuda.synchronize()
    main, side = rt.stream(-1), rt.stream(0)
    assert main and side and main != side

    def step():
        K.call("fb_add", a, b, c, 4096, stream=main)          # c = a + b          (main)
        rt.fork(0)
        K.call("fb_add", c, c, d, 4096, stream=side)          # d = 2c             (side, after c)
        K.call("fb_add", a, a, a, 4096, stream=main)          # a = 2a             (main, concurrent)
        rt.join(0)
        K.call("fb_add", d, a, c, 4096, stream=main)          # c = d + a          (main, after both)

    rt.capture_begin()
    step()
    g = rt.capture_end()
    want_a, want_c = 1.0, 0.0
    for _ in range(3):
        rt.graph_launch(g)
        want_c = 2 * (want_a + 2.0) + 2 * want_a
        want_a *= 2
    rt.sync()
    assert a[0].item() == want_a and c[7].item() == want_c
    host = rt.pinned_alloc(4096 * 4)
    rt.copy(host, c.data_ptr(), 4096 * 4)
    rt.sync()
    got = (ctypes.c_float * 4096).from_address(host)
    assert got[0] == want_c and got[4095] == want_c
    rt.pinned_free(host)
    rt.graph_free(g)
    rt.close()


@pytest.mark.parametrize("m,N,K_,nsplit", [(3, 4096, 8192, 8), (1, 24896, 4096, 2), (16, 300, 256, 3), (5, 129, 1536, 24),
                                           (8, 4384, 4096, 6)])
def test_gemv_tcgen05_splitk(K, m, N, K_, nsplit):
    """Split-K tcgen05 GEMV with hi + lo activation planes against fp32 matmul."""
    from ferrite_b200.models.glm import Act
    W = rnd(N, K_, seed=1, scale=0.05).to(torch.bfloat16)
    x = Act(torch.device("cuda"), 16, K_)
    x.f[:m].copy_(dev(rnd(m, K_, seed=2)))
    K.call("fb_split_rows", x.f, K_, *x.sp(1), 16, K_)
    tiles = (N + 127) // 128
    part = torch.zeros(tiles * nsplit * 16 * 128, device="cuda")
    ticket = torch.zeros(tiles, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.full((m, N), 0.25, device="cuda")
    want = x.f[:m].cpu() @ W.float().t()
    for it, acc in enumerate((0, 1, 0)):
        K.call("fb_gemv_tc_bf16", dev(W), x.s, K_, x.plane, out, N, m, N, K_, acc, nsplit, part, ticket, status)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0, status.tolist()
        exp = want * (2 if acc else 1)
        check(f"gemv tc splitk {it}", out, exp, 2e-3 * max(1.0, exp.abs().max().item()))
        assert not ticket.any()


@pytest.mark.parametrize("M,N,K_", [(256, 4096, 1024), (100, 1000, 512), (16, 512, 128), (300, 4096, 256), (5, 300, 256)])
def test_gemm_tc_ar_single_rank(K, M, N, K_):
    """The fused GEMM + all-reduce kernel with one rank (no collective): a plain tcgen05 GEMM with an
    optional local addend, against fp32 matmul of the same bf16 inputs."""
    from ferrite_b200.parallel.symm import FusedGemmAllReduce
    gar = FusedGemmAllReduce(torch.device("cuda"), 0, 1, max_rows=512, n_max=4096)
    w = dev(rnd(N, K_, seed=1, scale=0.1).bfloat16())
    x = dev(rnd(M, K_, seed=2).bfloat16())
    add = dev(rnd(M, N, seed=3))
    want = x.float() @ w.float().t()
    out = torch.full((M, N), 3.0, device="cuda")
    gar(w, x, K_, out, N, M, N, K_, False)
    torch.cuda.synchronize()
    gar.check()
    check("gemm tc ar", out, want, 2e-3 * max(1.0, want.abs().max().item()))
    out.copy_(add)
    gar(w, x, K_, out, N, M, N, K_, True)
    torch.cuda.synchronize()
    gar.check()
    check("gemm tc ar acc", out, want + add, 2e-3 * max(1.0, want.abs().max().item()))
