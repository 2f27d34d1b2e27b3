"""Low-precision codecs of the DSV41 family, stated in plain PyTorch (CPU or GPU).

Formats (reference ``ref_inference/kernel.py:22-205``, ``crates/ferrite-models/src/dsv41/quant.rs``):

* **e4m3** values with **ue8m0** (power-of-two) scales: dense weights in 32x32 blocks,
  activations and the window KV per 32 consecutive values; ``scale = 2^ceil(log2(amax/448))``
  with ``amax`` floored at 1e-4.
* **e2m1** ("fp4", grid 0, .5, 1, 1.5, 2, 3, 4, 6 with sign; two codes per byte, the even k in
  the low nibble) with ue8m0 scales per 32 values along K (expert weights, indexer q/k) or
  with **e4m3** scales per 16 values (the compressed KV latents; amax floored at 6*2^-9).

Every function here is the reference statement that the CUDA codecs are tested against.
"""
from __future__ import annotations

import torch

E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
FP8_MAX = 448.0
FP4_MAX = 6.0
# the scale of a block is computed as amax * (1/max) in f32, like the reference kernels do
_INV448 = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(448.0, dtype=torch.float32))
_INV6 = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(6.0, dtype=torch.float32))


# ---------------------------------------------------------------------------------------------
# scales
# ---------------------------------------------------------------------------------------------
def pow2_ceil(x: torch.Tensor) -> torch.Tensor:
    """2^ceil(log2(x)) for positive f32 x, exactly (bit manipulation, no transcendental)."""
    bits = x.float().contiguous().view(torch.int32)
    exp = (bits >> 23) & 0xFF
    man = bits & 0x7FFFFF
    e = exp - 127 + (man != 0).to(torch.int32)
    return ((e + 127).clamp(0, 254) << 23).view(torch.float32)


def ue8m0_encode(scale: torch.Tensor) -> torch.Tensor:
    """Power-of-two f32 scale -> its biased exponent byte."""
    return ((scale.float().contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)


def ue8m0_decode(b: torch.Tensor) -> torch.Tensor:
    return (b.to(torch.int32) << 23).view(torch.float32)


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """Round to the e4m3 grid (saturating at +-448), result in f32."""
    return x.float().clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).float()


# ---------------------------------------------------------------------------------------------
# e2m1
# ---------------------------------------------------------------------------------------------
def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (ties to the even code) of f32 values already divided by their scale.
    Returns uint8 codes 0..15 (bit 3 = sign)."""
    a = x.float().abs().clamp(max=FP4_MAX)
    code = torch.zeros_like(a, dtype=torch.int32)
    for c in range(7):
        mid = 0.5 * (E2M1_GRID[c] + E2M1_GRID[c + 1])
        up = (a > mid) if c % 2 == 0 else (a >= mid)  # a tie goes to the even code
        code = code + up.to(torch.int32)
    sign = (x < 0) | ((x == 0) & torch.signbit(x.float()))
    return (code | (sign.to(torch.int32) << 3)).to(torch.uint8)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    grid = torch.tensor(E2M1_GRID, dtype=torch.float32, device=code.device)
    v = grid[(code & 7).long()]
    return torch.where((code & 8) != 0, -v, v)


def e2m1_pack(code: torch.Tensor) -> torch.Tensor:
    """[..., K] codes -> [..., K/2] bytes, even k in the low nibble."""
    c = code.to(torch.uint8)
    return c[..., 0::2] | (c[..., 1::2] << 4)


def e2m1_unpack(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).flatten(-2)


# ---------------------------------------------------------------------------------------------
# activations (round trips: quantise and return the dequantised f32 values)
# ---------------------------------------------------------------------------------------------
def fp8_act_roundtrip(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """e4m3 with a power-of-two scale per `block` consecutive values of the last dim."""
    sh = x.shape
    v = x.float().reshape(-1, sh[-1] // block, block)
    amax = v.abs().amax(-1, keepdim=True).clamp_min(1e-4)
    s = pow2_ceil(amax * _INV448)
    return (e4m3_round(v / s) * s).reshape(sh)


def fp8_act_quant(x: torch.Tensor, block: int = 32):
    """(e4m3 values as f32 on the grid, ue8m0 scale bytes [..., K/block])."""
    sh = x.shape
    v = x.float().reshape(-1, sh[-1] // block, block)
    amax = v.abs().amax(-1, keepdim=True).clamp_min(1e-4)
    s = pow2_ceil(amax * _INV448)
    return e4m3_round(v / s).reshape(sh), ue8m0_encode(s.squeeze(-1)).reshape(*sh[:-1], sh[-1] // block)


def fp4_act_roundtrip(x: torch.Tensor, block: int = 32, scale: str = "ue8m0") -> torch.Tensor:
    """e2m1 with a ue8m0 scale per `block` values, or (scale="e4m3") an e4m3 scale."""
    sh = x.shape
    v = x.float().reshape(-1, sh[-1] // block, block)
    amax = v.abs().amax(-1, keepdim=True)
    if scale == "e4m3":
        s = e4m3_round(amax.clamp_min(6 * 2.0 ** -9) / FP4_MAX)
    else:
        s = pow2_ceil(amax.clamp_min(6 * 2.0 ** -126) * _INV6)
    return (e2m1_decode(e2m1_encode(v / s)) * s).reshape(sh)


# ---------------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------------
def quant_fp4_weight(w: torch.Tensor, block: int = 32):
    """[N, K] f32 -> (packed e2m1 [N, K/2] uint8, ue8m0 scale bytes [N, K/block])."""
    N, K = w.shape
    v = w.float().reshape(N, K // block, block)
    amax = v.abs().amax(-1, keepdim=True).clamp_min(6 * 2.0 ** -126)
    s = pow2_ceil(amax * _INV6)
    code = e2m1_encode(v / s).reshape(N, K)
    return e2m1_pack(code), ue8m0_encode(s.squeeze(-1))


def dequant_fp4_weight(packed: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    N = packed.shape[0]
    v = e2m1_decode(e2m1_unpack(packed)).reshape(N, -1, block)
    return (v * ue8m0_decode(scale).unsqueeze(-1)).reshape(N, -1)


def quant_fp8_weight(w: torch.Tensor, block: int = 32):
    """[N, K] f32 -> (e4m3 [N, K], ue8m0 scale bytes [ceil(N/block), ceil(K/block)])."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    pad = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    pad[:N, :K] = w.float()
    v = pad.reshape(nb, block, kb, block)
    amax = v.abs().amax(dim=(1, 3), keepdim=True).clamp_min(1e-4)
    s = pow2_ceil(amax * _INV448)
    q = (v / s).clamp(-FP8_MAX, FP8_MAX).reshape(nb * block, kb * block)[:N, :K].to(torch.float8_e4m3fn)
    return q, ue8m0_encode(s.reshape(nb, kb))


def dequant_fp8_weight(q: torch.Tensor, scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    N, K = q.shape
    s = ue8m0_decode(scale).repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.float() * s
