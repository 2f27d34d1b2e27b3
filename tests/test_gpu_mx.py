"""GPU: the block-scaled tcgen05 grouped GEMM (MXFP4 weights x e4m3 activations) against the fp32 statement
(dequantised weights x dequantised activations, ops/quant.py)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from ferrite_b200.ops import mx  # noqa: E402
from ferrite_b200.ops import quant as Q  # noqa: E402


def _case(E, N, K, counts, bn, seed=0):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(E, N, K, generator=g) * 0.05
    packed, scales = zip(*[Q.quant_fp4_weight(W[e]) for e in range(E)])
    packed, scales = torch.stack(packed), torch.stack(scales)
    M = sum(counts)
    X = torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 3.0
    xq, xs = Q.fp8_act_quant(X)
    want = torch.zeros(M, N)
    Wdq = torch.stack([Q.dequant_fp4_weight(packed[e], scales[e]) for e in range(E)])
    Xdq = xq.view(M, K // 32, 32) * Q.ue8m0_decode(xs).unsqueeze(-1)
    Xdq = Xdq.reshape(M, K)
    r = 0
    for e, c in enumerate(counts):
        want[r:r + c] = Xdq[r:r + c].double() @ Wdq[e].double().t()
        r += c
    dev = "cuda"
    cnt = torch.tensor(counts, dtype=torch.int32, device=dev)
    tiles, n_tiles, offsets = mx.make_tiles(cnt, bn)
    out = torch.full((M, N), 7.0, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    mx.mx_gemm_grouped(packed.to(dev), mx.pack_weight_scales(scales.to(dev)), xq.to(torch.float8_e4m3fn).to(dev),
                       xs.to(dev), tiles, n_tiles, out, bn, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    assert offsets.tolist()[-1] == M
    return out.cpu(), want.float()


def test_single_k_block_scale_bytes_and_nibbles():
    """K = 128 (one k-block): every scale byte position and nibble position matters exactly once."""
    out, want = _case(E=1, N=128, K=128, counts=[32], bn=32)
    err = (out - want).abs().max().item()
    assert err < 2e-3 * want.abs().max().item(), err


@pytest.mark.parametrize("E,N,K,counts,bn", [(3, 256, 512, [5, 0, 40], 32), (2, 384, 1024, [70, 64], 64),
                                             (4, 128, 256, [1, 130, 2, 17], 128), (2, 256, 4096, [300, 33], 256)])
def test_grouped_shapes(E, N, K, counts, bn):
    out, want = _case(E, N, K, counts, bn, seed=E)
    err = (out - want).abs().max().item()
    assert err < 2e-3 * max(1.0, want.abs().max().item()), (err, want.abs().max().item())


def test_quad_interleaved_weights_and_k_tail():
    """The decode kernels' load-time byte order (quad-interleaved 64-byte groups, 32-byte tail) and a K that is an
    odd multiple of 64 give the same result as plain packed bytes."""
    from ferrite_b200 import _lib
    K_ = _lib.lib()
    g = torch.Generator().manual_seed(5)
    E, N, counts, bn = 2, 256, [40, 9], 32
    for Kd in (320, 256):
        W = torch.randn(E, N, Kd, generator=g) * 0.05
        packed, scales = zip(*[Q.quant_fp4_weight(W[e]) for e in range(E)])
        packed, scales = torch.stack(packed).cuda(), torch.stack(scales).cuda()
        M = sum(counts)
        xq, xs = Q.fp8_act_quant(torch.randn(M, Kd, generator=g))
        xsf = torch.full((M, mx.sf_ld(Kd)), 127, dtype=torch.uint8)
        xsf[:, :Kd // 32] = xs
        tiles, n_tiles, _ = mx.make_tiles(torch.tensor(counts, dtype=torch.int32, device="cuda"), bn)
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        sfa = mx.pack_weight_scales(scales)
        outs = []
        for quad in (False, True):
            wp = packed.clone()
            if quad:
                K_.call("fb_d4_fp4_repack", wp, E * N, Kd // 2, 0)
            out = torch.zeros(M, N, device="cuda")
            mx.mx_gemm_grouped(wp, sfa, xq.to(torch.float8_e4m3fn).cuda(), xsf.cuda(), tiles, n_tiles, out, bn, status, quad=quad)
            outs.append(out)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        Wdq = torch.stack([Q.dequant_fp4_weight(packed[e].cpu(), scales[e].cpu()) for e in range(E)])
        Xdq = (xq.view(M, Kd // 32, 32) * Q.ue8m0_decode(xs).unsqueeze(-1)).reshape(M, Kd)
        want = torch.cat([Xdq[:40].double() @ Wdq[0].double().t(), Xdq[40:].double() @ Wdq[1].double().t()]).float()
        assert (outs[0].cpu() - want).abs().max().item() < 2e-3 * want.abs().max().item(), Kd
        assert torch.equal(outs[0], outs[1]), Kd


def test_sort_quant_swiglu_combine_glue():
    from ferrite_b200 import _lib
    K_ = _lib.lib()
    g = torch.Generator().manual_seed(9)
    n, topk, E, D, I = 20, 3, 7, 256, 96
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(n)]).int().cuda()
    wts = torch.rand(n, topk, generator=g).cuda()
    P = n * topk
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device="cuda")
    pos, counts, offsets, tiles, n_tiles = i32(P), i32(E), i32(E + 1), i32(64, 4), i32(1)
    ws = torch.zeros(P, device="cuda")
    K_.call("fb_mx_sort", ids, wts, P, 0, E, 32, pos, ws, counts, offsets, tiles, n_tiles, 64)
    torch.cuda.synchronize()
    cnt = torch.bincount(ids.flatten().cpu().long(), minlength=E)
    assert counts.cpu().tolist() == cnt.tolist() and offsets.cpu().tolist() == [0] + cnt.cumsum(0).tolist()
    p = pos.cpu().long()
    assert sorted(p.tolist()) == list(range(P))                      # a permutation
    seg = torch.bucketize(p, offsets.cpu()[1:].long(), right=True)   # segment of every pair's position
    assert torch.equal(seg, ids.flatten().cpu().long())              # ... is its expert's
    assert torch.equal(ws.cpu()[p], wts.flatten().cpu())
    assert n_tiles.item() == sum((c + 31) // 32 for c in cnt.tolist())
    x = torch.randn(n, D, generator=g)
    x8, sf = torch.zeros(P, D, dtype=torch.uint8, device="cuda"), torch.zeros(P, mx.sf_ld(D), dtype=torch.uint8, device="cuda")
    K_.call("fb_mx_quant_scatter", x.cuda(), D, pos, topk, n, D, x8, sf, sf.shape[1])
    xq, xs = Q.fp8_act_quant(x)
    rows = torch.arange(n).repeat_interleave(topk)
    assert torch.equal(x8.cpu()[p].view(torch.float8_e4m3fn).float(), xq[rows])
    assert torch.equal(sf.cpu()[p][:, :D // 32], xs[rows]) and (sf.cpu()[:, D // 32:] == 127).all()
    h = torch.randn(P, 2 * I, generator=g) * 4
    a8, asf = torch.zeros(P, I, dtype=torch.uint8, device="cuda"), torch.zeros(P, mx.sf_ld(I), dtype=torch.uint8, device="cuda")
    K_.call("fb_mx_swiglu_quant", h.cuda(), 2 * I, ws, offsets[E:], P, I, 3.0, a8, asf, asf.shape[1])
    act = torch.nn.functional.silu(h[:, :I].clamp(max=3.0)) * h[:, I:].clamp(-3.0, 3.0) * ws.cpu().unsqueeze(-1)
    aq, as_ = Q.fp8_act_quant(act)
    got = a8.cpu().view(torch.float8_e4m3fn).float() * Q.ue8m0_decode(asf.cpu()[:, :I // 32]).repeat_interleave(32, 1)
    want = aq * Q.ue8m0_decode(as_).repeat_interleave(32, 1)
    assert (got - want).abs().max().item() <= 0.07 * want.abs().max().item()      # silu's fast exp can flip a rounding
    assert ((got - want).abs() > 1e-6).float().mean().item() < 0.01
    yp = torch.randn(P, D, generator=g).cuda()
    y = torch.ones(n, D, device="cuda")
    K_.call("fb_mx_combine", yp, D, pos, topk, y, D, n, D, 1)
    want_y = 1.0 + yp.cpu()[p].view(n, topk, D).sum(1)
    assert (y.cpu() - want_y).abs().max().item() < 1e-5


def test_dsv41_prefill_through_block_scaled_experts_matches_decode_kernels():
    """The tiny DSV41 model prefilled in 16-row chunks with the routed experts as block-scaled tcgen05 grouped GEMMs
    (quad-interleaved weights, 64-value k tail) against the same chunks through the weight-streaming kernels: both
    multiply the same e2m1 x e4m3 values, so the logits agree up to summation order."""
    from ferrite_b200.models.dsv41 import DictWeights, Dsv41DeviceModel
    from ferrite_b200.models.dsv41_config import Dsv41Config
    from ferrite_b200.models.dsv41_weights import random_weights
    from ferrite_b200.utils.switches import Switches, set_switches
    cfg = Dsv41Config.tiny()
    w = random_weights(cfg, 4)
    ids = torch.randint(0, cfg.vocab_size - 20, (32,), generator=torch.Generator().manual_seed(3)).tolist()
    logits = {}
    try:
        for mx_rows in (0, 16):
            set_switches(Switches(d4_mx_min_rows=mx_rows, d4_tc_min_rows=16))
            dev = Dsv41DeviceModel(cfg, DictWeights(w), max_rows=16, max_ctx=128)
            assert any(L.get("mx") for L in dev.layers) == (mx_rows > 0)
            # the same router GEMM in both runs (the paired decode launches read the activations' hi + lo planes, the
            # tcgen05 GEMM the hi plane: a router logit that moves in its last bits can pick another expert)
            dev.moe_paired = False
            out = []
            for i in range(0, len(ids), 16):
                c = ids[i:i + 16]
                dev.forward(dev.make_rows([0], [len(c)]), torch.tensor(c, dtype=torch.int32, device="cuda"))
                out.append(dev.ws["logits"][:len(c)].cpu().clone())
            torch.cuda.synchronize()
            assert int(dev.tc_status[0]) == 0
            logits[mx_rows] = torch.cat(out)
    finally:
        set_switches(None)
    a, b = logits[16], logits[0]
    assert (a - b).abs().max().item() < 2e-3 * b.abs().max().item(), (a - b).abs().max().item()
    assert torch.equal(a.argmax(-1), b.argmax(-1))
