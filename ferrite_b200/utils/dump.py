"""Unit dumps: save named tensors of a run and compare two runs (device vs golden, build A vs B).

Reference: ``crates/ferrite-models/src/dsv41/{unit_dump,dump_dev,dspark_parity}.rs`` (per-unit dump and
compare harness, parity checkers).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch


class UnitDump:
    """Collects ``name -> [tensor per call]``; usable as the debug hook of the device and golden models."""

    def __init__(self, keep: Optional[Callable[[str], bool]] = None):
        self.keep = keep
        self.units: Dict[str, List[torch.Tensor]] = {}

    def __call__(self, name: str, t: torch.Tensor) -> None:
        if self.keep is None or self.keep(name):
            self.units.setdefault(name, []).append(t.detach().float().cpu().clone())

    def save(self, directory: str) -> None:
        os.makedirs(directory, exist_ok=True)
        index = {}
        for i, (name, ts) in enumerate(sorted(self.units.items())):
            fn = f"unit_{i:05d}.pt"
            torch.save(ts, os.path.join(directory, fn))
            index[name] = fn
        with open(os.path.join(directory, "index.json"), "w") as f:
            json.dump(index, f, indent=1)

    @staticmethod
    def load(directory: str) -> "UnitDump":
        d = UnitDump()
        with open(os.path.join(directory, "index.json")) as f:
            index = json.load(f)
        for name, fn in index.items():
            d.units[name] = torch.load(os.path.join(directory, fn))
        return d


@dataclass
class UnitDiff:
    name: str
    max_abs: float
    ref_max: float
    frac_over: float       # fraction of elements whose error exceeds rel_tol * ref_max
    shape_ok: bool = True

    @property
    def rel(self) -> float:
        return self.max_abs / max(self.ref_max, 1e-30)


def compare(got: UnitDump, want: UnitDump, rel_tol: float = 1e-2) -> List[UnitDiff]:
    """One record per unit present in both dumps, in name order."""
    out = []
    for name in sorted(set(got.units) & set(want.units)):
        a = torch.cat([t.reshape(t.shape[0], -1) for t in got.units[name]])
        b = torch.cat([t.reshape(t.shape[0], -1) for t in want.units[name]])
        if a.shape != b.shape:
            out.append(UnitDiff(name, float("inf"), float(b.abs().max()), 1.0, False))
            continue
        diff = (a - b).abs()
        ref = float(b.abs().max())
        out.append(UnitDiff(name, float(diff.max()), ref, float((diff > rel_tol * max(ref, 1e-30)).float().mean())))
    return out


def first_divergence(diffs: List[UnitDiff], rel_tol: float = 5e-2, frac_tol: float = 0.01) -> Optional[UnitDiff]:
    """The first unit (in name order) whose bulk error is out of tolerance."""
    for d in diffs:
        if not d.shape_ok or d.frac_over > frac_tol or d.rel > 10 * rel_tol:
            return d
    return None


def token_parity(a: List[int], b: List[int]) -> Dict[str, object]:
    """Draft/verify parity of two token streams: length of the common prefix and the first mismatch."""
    n = 0
    while n < min(len(a), len(b)) and a[n] == b[n]:
        n += 1
    return {"common_prefix": n, "equal": n == len(a) == len(b),
            "first_mismatch": None if n >= min(len(a), len(b)) else (n, a[n], b[n])}
