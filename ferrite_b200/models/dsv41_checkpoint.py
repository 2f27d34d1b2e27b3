"""DSV41 checkpoints: write a model in its storage formats and read it back without changing a bit.

Storage (reference ``ref_inference/model.py:181-259``, ``crates/ferrite-models/src/dsv41/load.rs``):
``dense`` tensors are e4m3 bytes with a ``.scale`` sibling of ue8m0 bytes per 32x32 block,
``expert`` tensors are packed e2m1 (two per byte) with a ``.scale`` sibling per (row, 32), the engram
table is e4m3 with ``.scale`` per (row, 32); the rest is bf16 / f32.  ``Dsv41CheckpointSource.get``
returns the dequantised f32 tensor (exact), which the device model packs again for its kernels.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..ops import quant as Q
from .checkpoint import CheckpointIndex, write_safetensors
from .dsv41_config import Dsv41Config
from .dsv41_weights import Spec, tensor_specs


def _storage_kind(cfg: Dsv41Config, spec: Spec) -> str:
    k = spec.kind
    if k == "expert":
        k = "fp4" if cfg.expert_dtype == "fp4" else "dense"
    if k == "dense":
        k = "fp8" if cfg.dense_dtype == "fp8" else "bf16"
    return k


def save_checkpoint(directory: str, cfg: Dsv41Config, weights: Dict[str, torch.Tensor], shards: int = 2) -> None:
    """Write `weights` (f32, on their storage grids) as `shards` safetensors files."""
    os.makedirs(directory, exist_ok=True)
    specs = tensor_specs(cfg)
    out: Dict[str, torch.Tensor] = {}
    for name, w in weights.items():
        kind = _storage_kind(cfg, specs[name])
        if kind == "fp4":
            p, s = Q.quant_fp4_weight(w.float(), cfg.fp4_block)
            out[name], out[name[:-len("weight")] + "scale"] = p, s
        elif kind == "fp8":
            q, s = Q.quant_fp8_weight(w.float(), cfg.fp8_block)
            out[name], out[name[:-len("weight")] + "scale"] = q, s
        elif kind == "table":
            q, s = Q.fp8_act_quant(w.float(), cfg.fp8_block)
            out[name], out[name[:-len("weight")] + "scale"] = q.to(torch.float8_e4m3fn), s
        elif kind == "bf16":
            out[name] = w.to(torch.bfloat16)
        else:
            out[name] = w.float()
    names = sorted(out)
    per = (len(names) + shards - 1) // shards
    for i in range(shards):
        part = {n: out[n] for n in names[i * per:(i + 1) * per]}
        if part:
            write_safetensors(os.path.join(directory, f"model-{i + 1:05d}-of-{shards:05d}.safetensors"), part)


class Dsv41CheckpointSource:
    """Weight source over a checkpoint directory (``get`` / ``has`` like ``DictWeights``)."""

    def __init__(self, directory: str, cfg: Dsv41Config):
        self.cfg = cfg
        self.index = CheckpointIndex(directory)
        self.specs = tensor_specs(cfg)

    def has(self, name: str) -> bool:
        return name in self.index

    def get(self, name: str) -> torch.Tensor:
        cfg = self.cfg
        kind = _storage_kind(cfg, self.specs[name])
        raw = self.index.view(name)
        if kind in ("fp4", "fp8", "table"):
            scale = self.index.view(name[:-len("weight")] + "scale").view(torch.uint8)
        if kind == "fp4":
            return Q.dequant_fp4_weight(raw.view(torch.uint8), scale, cfg.fp4_block)
        if kind == "fp8":
            return Q.dequant_fp8_weight(raw.view(torch.float8_e4m3fn), scale, cfg.fp8_block)
        if kind == "table":
            v = raw.view(torch.float8_e4m3fn).float().unflatten(-1, (-1, cfg.fp8_block))
            return (v * Q.ue8m0_decode(scale).unsqueeze(-1)).flatten(-2)
        return raw.float()
