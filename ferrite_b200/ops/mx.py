"""Block-scaled (MXFP4 weights x e4m3 activations, ue8m0 scales per 32) grouped GEMM on tcgen05
(``csrc/kernels/mx_gemm.cu``): host-side helpers and the call wrapper.

The fp32 statement it is tested against is ``ops/quant.py``: ``dequant_fp4_weight`` x the dequantised
activation rows of ``fp8_act_quant``.  Counterpart of the reference's tcgen05 expert GEMMs
(``kernels/cuda/dsv41_experts_mxf4.cu:437,5292,7171``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib

TILE_W = 128   # weight rows per CTA
KB = 128       # values per k-block


def pack_weight_scales(scales: torch.Tensor) -> torch.Tensor:
    """ue8m0 scale bytes [E, N, K/32] (N % 128 == 0, K % 128 == 0) -> [E, N/128, K/128, 512]: per (128-row tile,
    128-value k-block) the 512-byte chunk tcgen05.cp reads, byte (i * 16 + g * 4 + s) for row 32 g + i and
    32-value sub-block s.  Done once at load time."""
    E, N, KS = scales.shape
    assert N % TILE_W == 0 and scales.dtype == torch.uint8
    if KS % 4:   # a last k-block past K meets zero values: any valid exponent will do
        scales = torch.nn.functional.pad(scales, (0, 4 - KS % 4), value=127)
        KS = scales.shape[2]
    t = scales.contiguous().view(E, N // TILE_W, 4, 32, KS // 4, 4)          # [E, tile, g, i, kb, s]
    return t.permute(0, 1, 4, 3, 2, 5).contiguous().view(E, N // TILE_W, KS // 4, 512)


def make_tiles(counts: torch.Tensor, bn: int, max_tiles: Optional[int] = None):
    """Tile list (device) of a grouped GEMM over rows sorted by expert: counts [E] int32 rows per expert.
    Returns (tiles [max_tiles, 4] int32, n_tiles [1] int32, offsets [E + 1] int32)."""
    K = _lib.lib()
    E = counts.numel()
    if max_tiles is None:
        max_tiles = E + (int(counts.sum().item()) + bn - 1) // bn
    tiles = torch.zeros(max_tiles, 4, dtype=torch.int32, device=counts.device)
    n_tiles = torch.zeros(1, dtype=torch.int32, device=counts.device)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=counts.device)
    K.call("fb_mx_tiles", counts, E, bn, tiles, n_tiles, offsets, max_tiles)
    return tiles, n_tiles, offsets


def pick_bn(rows_per_expert: float) -> int:
    for bn in (32, 64, 128):
        if rows_per_expert <= bn:
            return bn
    return 256


def sf_ld(K: int) -> int:
    """Row stride (bytes) of an activation scale buffer: whole 128-value k-blocks."""
    return 4 * ((K + KB - 1) // KB)


def mx_gemm_grouped(w_packed: torch.Tensor, sfa: torch.Tensor, x8: torch.Tensor, x_sf: torch.Tensor, tiles: torch.Tensor,
                    n_tiles: torch.Tensor, out: torch.Tensor, bn: int, status: torch.Tensor, quad: bool = False,
                    m_total: Optional[int] = None) -> None:
    """out[p, :] = W[e(p)] . x[p] for the rows of the tile list.  w_packed [E, N, K/2] uint8 (quad: quad-interleaved
    bytes), sfa from :func:`pack_weight_scales`, x8 [M, K] e4m3 rows sorted by expert, x_sf [M, >= sf_ld(K)] uint8
    (bytes past K / 32 must be valid exponents), out [M, >= N] f32."""
    E, N, K2 = w_packed.shape
    M, K = x8.shape
    M = M if m_total is None else m_total
    assert K == 2 * K2 and x_sf.shape[0] >= M and x_sf.stride(0) >= sf_ld(K) and out.shape[0] >= M and out.shape[1] >= N
    _lib.lib().call("fb_mx_gemm_grouped", w_packed, sfa, x8, x_sf, x_sf.stride(0), tiles, n_tiles, tiles.shape[0], out,
                    out.stride(0), M, E, N, K, bn, int(quad), status)
