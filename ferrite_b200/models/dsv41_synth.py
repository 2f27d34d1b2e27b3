"""Synthetic DSV41 weights generated on the device (benchmarks at production dimensions).

``get(name)`` draws the tensor with a per-name seed directly on the GPU (f32, fan-in scaled);
``expert_pack`` fills the packed e2m1 expert tensors and their ue8m0 scales with random bytes, so a
layer with 384 experts is built in milliseconds instead of quantising 13 G values on the host.
Values are not on any checkpoint's grid: use ``random_weights`` + ``DictWeights`` for parity tests.
"""
from __future__ import annotations

import zlib

import torch

from .dsv41_config import Dsv41Config
from .dsv41_weights import tensor_specs


class SyntheticDsv41Source:
    def __init__(self, cfg: Dsv41Config, device, seed: int = 0):
        self.cfg, self.dev, self.seed = cfg, torch.device(device), seed
        self.specs = tensor_specs_lazy(cfg)

    def has(self, name: str) -> bool:
        return name in self.specs

    def _gen(self, name: str) -> torch.Generator:
        g = torch.Generator(device=self.dev)
        g.manual_seed((zlib.crc32(name.encode()) + 7919 * self.seed) & 0x7FFFFFFF)
        return g

    def get(self, name: str) -> torch.Tensor:
        spec = self.specs[name]
        g = self._gen(name)
        shp = spec.shape
        if spec.init == "ones":
            return 1.0 + 0.1 * torch.randn(shp, device=self.dev, generator=g)
        if spec.init in ("small", "bias"):
            return 0.05 * torch.randn(shp, device=self.dev, generator=g)
        if name == "embed.weight":
            return torch.randn(shp, device=self.dev, generator=g)
        return torch.randn(shp, device=self.dev, generator=g) * (shp[-1] ** -0.5)

    def expert_pack(self, prefix: str, E: int, Il: int, rank: int, world: int, dev):
        """(w13 [E,2,Il,d/2], s13 [E,2,Il,d/32], w2 [E,d,Il/2], s2 [E,d,Il/32]) as uint8."""
        d = self.cfg.dim
        g = self._gen(prefix + f"experts@{rank}")
        w13 = torch.randint(0, 256, (E, 2, Il, d // 2), dtype=torch.uint8, device=dev, generator=g)
        w2 = torch.randint(0, 256, (E, d, Il // 2), dtype=torch.uint8, device=dev, generator=g)
        # scales so that dequantised weights have the fan-in scaled magnitude (e2m1 values average ~2)
        e13 = 127 + round(torch.log2(torch.tensor(d ** -0.5 / 2.0)).item())
        e2 = 127 + round(torch.log2(torch.tensor(max(Il * world, 1) ** -0.5 / 2.0)).item())
        s13 = torch.full((E, 2, Il, d // 32), e13, dtype=torch.uint8, device=dev)
        s2 = torch.full((E, d, Il // 32), e2, dtype=torch.uint8, device=dev)
        return w13, s13, w2, s2


    def engram_pack(self, prefix: str, lo: int, hi: int, dev):
        """Rows [lo, hi) of an engram table in its device form: e4m3 bytes [rows, head_dim] (no NaN codes) and one
        ue8m0 scale byte per 32 values, generated in slabs so that a 25 GB shard never needs a second copy."""
        hd = self.cfg.engram_head_dim
        n = max(0, hi - lo)
        g = self._gen(prefix + f"engram@{lo}")
        tab = torch.empty(n, hd, dtype=torch.uint8, device=dev)
        step = 1 << 22
        for r0 in range(0, n, step):
            r1 = min(n, r0 + step)
            mag = torch.randint(0, 0x70, (r1 - r0, hd), dtype=torch.uint8, device=dev, generator=g)     # |v| <= 224
            sgn = torch.randint(0, 2, (r1 - r0, hd), dtype=torch.uint8, device=dev, generator=g) << 7
            tab[r0:r1] = mag | sgn
        scale = torch.full((n, hd // self.cfg.fp8_block), 118, dtype=torch.uint8, device=dev)              # 2^-9
        return tab, scale


def tensor_specs_lazy(cfg: Dsv41Config):
    """Specs without the per-expert entries (the synthetic source packs experts in bulk)."""
    return {k: v for k, v in tensor_specs(cfg).items() if ".experts." not in k and not k.endswith("engram.embed.weight")}
