"""Op-trace contract: record the sequence of kernel calls of a step and assert that it is stable
before the step is captured into a CUDA graph.

A graph replays exactly the launches it recorded, so a step whose kernel sequence (names and
integer arguments: shapes, strides, flags) depends on host state cannot be captured.  The recorder
hooks the kernel library's single call path.  Behaviour of the reference's
``crates/ferrite-kernel/src/graph.rs:20-135`` (``OpRecord``, ``OpTrace``, ``Recorder``) and
``crates/ferrite-exec/src/graph.rs:51-160`` (``GraphRunner``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple


@dataclass(frozen=True)
class OpRecord:
    name: str
    ints: Tuple[int, ...]        # integer / float arguments in call order (pointers are not part of the contract)

    def __str__(self) -> str:
        return f"{self.name}{self.ints}"


class OpTrace:
    def __init__(self, ops: Optional[List[OpRecord]] = None):
        self.ops: List[OpRecord] = list(ops or [])

    def __len__(self) -> int:
        return len(self.ops)

    def __eq__(self, other) -> bool:
        return isinstance(other, OpTrace) and self.ops == other.ops

    def first_difference(self, other: "OpTrace") -> Optional[Tuple[int, Optional[OpRecord], Optional[OpRecord]]]:
        for i in range(max(len(self.ops), len(other.ops))):
            a = self.ops[i] if i < len(self.ops) else None
            b = other.ops[i] if i < len(other.ops) else None
            if a != b:
                return i, a, b
        return None

    def histogram(self) -> dict:
        h: dict = {}
        for o in self.ops:
            h[o.name] = h.get(o.name, 0) + 1
        return h


class Recorder:
    """Collects OpRecords; install with ``with Recorder().attach(lib) as rec: ...``."""

    def __init__(self):
        self.trace = OpTrace()
        self._lib = None
        self._orig: Optional[Callable] = None

    def record(self, name: str, args) -> None:
        ints = tuple(a if isinstance(a, (int, float)) and not isinstance(a, bool) else int(a)
                     for a in args if isinstance(a, (int, float, bool)))
        self.trace.ops.append(OpRecord(name, ints))

    def attach(self, lib) -> "Recorder":
        self._lib = lib
        return self

    def __enter__(self) -> "Recorder":
        lib = self._lib
        self._orig = lib.call
        rec = self

        def call(name, *args, **kw):
            rec.record(name, args)
            return rec._orig(name, *args, **kw)

        lib.call = call
        return self

    def __exit__(self, *exc) -> None:
        self._lib.call = self._orig


class GraphRunner:
    """Runs a step function twice under a recorder and refuses capture when the traces differ."""

    def __init__(self, lib):
        self.lib = lib
        self.trace: Optional[OpTrace] = None

    def record(self, step: Callable[[], None]) -> OpTrace:
        with Recorder().attach(self.lib) as rec:
            step()
        return rec.trace

    def assert_stable(self, step: Callable[[], None], runs: int = 2) -> OpTrace:
        first = self.record(step)
        for _ in range(runs - 1):
            other = self.record(step)
            diff = first.first_difference(other)
            if diff is not None:
                i, a, b = diff
                raise RuntimeError(f"op trace is not stable at op {i}: {a} vs {b}; the step cannot be captured")
        self.trace = first
        return first
