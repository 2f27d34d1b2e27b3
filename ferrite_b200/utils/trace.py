"""Timing and tracing helpers: NVTX ranges, CUDA-event phase timers (max over ranks), layer
checksums and a torch.profiler wrapper.

Counterparts of the reference's env-gated probes (``FERRITE_TIMING``, ``FERRITE_MTP_TIMING``,
``FERRITE_LAYER_SUM``, ``crates/ferrite-exec/src/tp.rs:1857,3553-3572``) and of its profiler window
(``crates/ferrite-kernel/src/cuda.rs:7248``).
"""
from __future__ import annotations

import contextlib
from collections import defaultdict
from typing import Dict, List, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    if enabled and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimer:
    """Named phases timed with CUDA events on the current stream (host timers without a GPU)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available()
        self._open: Dict[str, object] = {}
        self._pending: List[tuple] = []
        self.total_ms: Dict[str, float] = defaultdict(float)
        self.count: Dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            yield
            b.record()
            self._pending.append((name, a, b))
        else:
            import time
            t0 = time.perf_counter()
            yield
            self.total_ms[name] += (time.perf_counter() - t0) * 1e3
            self.count[name] += 1

    def flush(self) -> None:
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.total_ms[name] += a.elapsed_time(b)
                self.count[name] += 1
            self._pending = []

    def summary(self, group=None) -> Dict[str, dict]:
        """Per phase: total / mean ms; with a process group, the maximum over ranks."""
        self.flush()
        out = {}
        for name in sorted(self.total_ms):
            tot = self.total_ms[name]
            if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
                t = torch.tensor([tot], dtype=torch.float64, device="cuda" if self.cuda else "cpu")
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
                tot = float(t.item())
            out[name] = {"total_ms": tot, "calls": self.count[name], "mean_ms": tot / max(1, self.count[name])}
        return out


def layer_checksums(rows: torch.Tensor) -> List[float]:
    """One number per row of a residual-stream buffer: cheap fingerprint for A/B runs."""
    return rows.detach().float().reshape(rows.shape[0], -1).double().sum(-1).cpu().tolist()


def check_finite(name: str, t: torch.Tensor) -> None:
    if not torch.isfinite(t).all():
        bad = (~torch.isfinite(t)).nonzero()[:4].tolist()
        raise FloatingPointError(f"{name}: non-finite values at {bad}")


@contextlib.contextmanager
def profiler_window(path: Optional[str] = None, activities=None):
    """torch.profiler around a few steps; writes a Chrome trace when `path` is given."""
    from torch.profiler import ProfilerActivity, profile
    acts = activities or [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts) as prof:
        yield prof
    if path:
        prof.export_chrome_trace(path)
