"""GPU: the expert-grouped W8A16 tcgen05 GEMM (e4m3 weights widened to f16 in shared memory, f16 activation rows, the
128x128 f32 block scales applied to each k-block's accumulator) against fp32 matmuls of the dequantised weights, and
the GLM prefill path through it against the mma.sync grouped kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from ferrite_b200 import _lib  # noqa: E402
from ferrite_b200.ops import reference as R  # noqa: E402


@pytest.mark.parametrize("E,N,K,counts,bn", [(2, 128, 128, [20, 3], 32), (3, 256, 512, [64, 0, 70], 64),
                                             (2, 384, 2048, [130, 40], 128), (1, 256, 4096, [300], 128),
                                             (40, 512, 1024, [7 * (i % 5) for i in range(40)], 32)])
def test_fp8w_grouped_gemm(E, N, K, counts, bn):
    Kl = _lib.lib()
    g = torch.Generator().manual_seed(E + N)
    W = torch.randn(E, N, K, generator=g) * 0.05
    qs = [R.quant_fp8_block(W[e]) for e in range(E)]
    wq = torch.stack([q for q, _ in qs]).cuda()
    sc = torch.stack([s for _, s in qs]).cuda()
    M = sum(counts)
    x = torch.randn(M, K, generator=g).half()
    cnt = torch.tensor(counts, dtype=torch.int32, device="cuda")
    tiles = torch.zeros(64, 4, dtype=torch.int32, device="cuda")          # more tile slots than tiles: the grid is sized by it
    n_tiles = torch.zeros(1, dtype=torch.int32, device="cuda")
    offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    Kl.call("fb_mx_tiles", cnt, E, bn, tiles, n_tiles, offsets, 64)
    out = torch.full((M, N), 7.0, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    Kl.call("fb_fp8w_gemm_grouped", wq, sc, x.cuda(), tiles, n_tiles, 64, out, N, M, E, N, K, bn, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    want = torch.zeros(M, N)
    r = 0
    for e, c in enumerate(counts):
        want[r:r + c] = (x[r:r + c].double() @ R.dequant_fp8_block(*qs[e]).double().t()).float()
        r += c
    err = (out.cpu() - want).abs().max().item()
    assert err < 1e-3 * max(1.0, want.abs().max().item()), (err, want.abs().max().item())   # exact operands, f32 accumulation


def test_glm_prefill_through_tcgen05_experts_matches_grouped_kernels():
    from ferrite_b200.config import EngineConfig, GlmConfig
    from ferrite_b200.engine.glm_engine import GlmEngine
    from ferrite_b200.models.glm import DictSource
    from ferrite_b200.models.glm_weights import random_weights
    from ferrite_b200.utils.switches import Switches, set_switches
    cfg = GlmConfig.golden4()
    w = random_weights(cfg, 0, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (150,), generator=torch.Generator().manual_seed(2)).tolist()
    outs, hid = {}, {}
    try:
        for rows in (0, 64):
            set_switches(Switches(moe_tc_rows=rows))
            eng = GlmEngine(cfg, EngineConfig(max_ctx=256, mtp_n=1), DictSource(w, "cuda"), prefill_rows=64)
            assert ("tc_x" in eng.model.ws) == (rows > 0)
            outs[rows], _ = eng.generate(prompt, 10)
            assert int(eng.model.tc_status[0]) == 0
    finally:
        set_switches(None)
    same = sum(a == b for a, b in zip(outs[0], outs[64]))
    assert same >= 9, outs     # bf16 against f16 activations in the experts: a late near-tie may flip
