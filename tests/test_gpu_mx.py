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
