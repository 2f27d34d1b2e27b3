"""Accept-length histogram of speculative decoding (reference:
``crates/ferrite-models/src/dsv41/acc_hist.rs``; accept stat line ``crates/ferrite-serve/src/main.rs:486-495``)."""
from __future__ import annotations

from typing import Dict, Iterable


class AcceptHistogram:
    def __init__(self, max_len: int):
        self.max_len = max_len
        self.bins = [0] * (max_len + 1)

    def add(self, k: int) -> None:
        self.bins[min(max(k, 0), self.max_len)] += 1

    def extend(self, ks: Iterable[int]) -> None:
        for k in ks:
            self.add(k)

    @property
    def steps(self) -> int:
        return sum(self.bins)

    @property
    def tokens(self) -> int:
        return sum(k * c for k, c in enumerate(self.bins))

    @property
    def mean(self) -> float:
        return self.tokens / self.steps if self.steps else 0.0

    def as_dict(self) -> Dict[str, object]:
        return {"steps": self.steps, "tokens": self.tokens, "mean_accept": round(self.mean, 4),
                "hist": {str(k): c for k, c in enumerate(self.bins) if c}}

    def line(self) -> str:
        parts = " ".join(f"{k}:{c}" for k, c in enumerate(self.bins) if c)
        return f"[acc-hist] steps={self.steps} tokens={self.tokens} mean={self.mean:.3f} | {parts}"
