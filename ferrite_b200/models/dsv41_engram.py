"""Engram n-gram hashing: bucket layout, hash multipliers and the per-sequence hash state.

For every position the 2-gram .. max-gram ending there are hashed per head into disjoint
prime-sized bucket ranges of the layer's table: the compressed token ids of the look-back
window are multiplied by per-(layer, look-back) odd multipliers, XOR-folded one look-back at
a time, reduced modulo the (layer, n-gram, head) prime and offset into that pair's range.
Look-back stops at the sequence start and at dead tokens (image spans); the pad id stands
in.  Behaviour of ``ref_inference/engram.py:8-190`` (``EngramLayout``, ``NgramHashState``) and
``crates/ferrite-models/src/dsv41/engram.rs``; the token-normalisation map needs the model's
tokenizer and is passed in (identity-modulo map when absent).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    for p in (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37):
        if n % p == 0:
            return n == p
    d, s = n - 1, 0
    while d % 2 == 0:
        d //= 2
        s += 1
    for a in (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37):  # deterministic below 3.3e24
        x = pow(a, d, n)
        if x in (1, n - 1):
            continue
        for _ in range(s - 1):
            x = x * x % n
            if x == n - 1:
                break
        else:
            return False
    return True


def next_unused_prime(start: int, seen: set) -> int:
    c = start + 1
    while not _is_prime(c) or c in seen:
        c += 1
    return c


def hash_multipliers(layer_ids: Sequence[int], max_ngram: int, compressed_vocab: int) -> torch.Tensor:
    """[n_layers, max_ngram] odd int64 multipliers, one RNG stream per layer id."""
    bound = max(1, (np.iinfo(np.int64).max // compressed_vocab) // 2)
    rows = []
    for lid in layer_ids:
        g = np.random.default_rng(10007 * lid)
        rows.append(torch.tensor(g.integers(low=0, high=bound, size=(max_ngram,), dtype=np.int64) * 2 + 1))
    return torch.stack(rows)


@dataclass(frozen=True)
class EngramLayout:
    max_ngram: int
    layer_ids: Tuple[int, ...]
    primes: Tuple[Tuple[Tuple[int, ...], ...], ...]  # [layer][n-gram size - 2][head]
    n_heads: int
    head_dim: int

    @staticmethod
    def from_config(cfg) -> Optional["EngramLayout"]:
        if not cfg.engram_layer_ids:
            return None
        primes, seen = [], set()
        for _ in cfg.engram_layer_ids:
            per_ngram = []
            for _ in range(cfg.engram_max_ngram_size - 1):
                sizes, cur = [], cfg.engram_vocab_size - 1
                for _ in range(cfg.engram_n_heads):
                    cur = next_unused_prime(cur, seen)
                    seen.add(cur)
                    sizes.append(cur)
                per_ngram.append(tuple(sizes))
            primes.append(tuple(per_ngram))
        return EngramLayout(cfg.engram_max_ngram_size, tuple(cfg.engram_layer_ids), tuple(primes),
                            cfg.engram_n_heads, cfg.engram_head_dim)

    @property
    def hash_cols(self) -> int:
        return (self.max_ngram - 1) * self.n_heads

    @property
    def table_rows(self) -> Tuple[int, ...]:
        return tuple(sum(p for per in layer for p in per) for layer in self.primes)

    def flat_primes(self) -> torch.Tensor:
        """[n_layers, hash_cols] (n-gram major, head minor)."""
        return torch.tensor([[p for per in layer for p in per] for layer in self.primes], dtype=torch.int64)

    def offsets(self) -> torch.Tensor:
        fp = self.flat_primes()
        return torch.cumsum(fp, 1) - fp


class NgramHasher:
    """Hash ids of one sequence, carried across prefill chunks and decode steps."""

    DEAD = -1

    def __init__(self, cfg, layout: EngramLayout, token_map: Optional[Sequence[int]] = None):
        self.layout = layout
        cv = cfg.engram_compressed_vocab_size
        if token_map is None:
            token_map = [t % cv for t in range(cfg.vocab_size)]
        self.token_map = torch.tensor(list(token_map), dtype=torch.int64)
        assert int(self.token_map.max()) < cv
        self.pad = int(self.token_map[cfg.engram_pad_id])
        self.mult = hash_multipliers(layout.layer_ids, layout.max_ngram, cv)  # [L, G]
        self.primes = layout.flat_primes().view(len(layout.layer_ids), layout.max_ngram - 1, layout.n_heads)
        self.offs = layout.offsets()
        self.history: List[int] = []  # compressed ids (DEAD for masked tokens) of every position so far

    def truncate(self, n: int) -> None:
        del self.history[n:]

    def extend(self, ids: Sequence[int], alive: Optional[Sequence[bool]] = None) -> torch.Tensor:
        """Append `ids` at the end of the sequence; returns [len(ids), n_layers, hash_cols] int64."""
        start = len(self.history)
        comp = self.token_map[torch.as_tensor(list(ids), dtype=torch.int64)].tolist()
        if alive is not None:
            comp = [c if a else self.DEAD for c, a in zip(comp, alive)]
        self.history += comp
        return self.hash_range(start, len(self.history))

    def hash_range(self, lo: int, hi: int) -> torch.Tensor:
        G = self.layout.max_ngram
        hist = torch.tensor(self.history[:hi], dtype=torch.int64)
        pos = torch.arange(lo, hi)
        toks, blocked = [], torch.zeros(hi - lo, dtype=torch.bool)
        for shift in range(G):
            src = hist[(pos - shift).clamp_min(0)]
            blocked = blocked | (pos < shift) | (src == self.DEAD)
            toks.append(torch.where(blocked, torch.full_like(src, self.pad), src))
        toks = torch.stack(toks, -1)                       # [n, G]
        prod = toks.unsqueeze(1) * self.mult               # [n, L, G]
        rolling, out = prod[..., 0], []
        for i in range(1, G):
            rolling = torch.bitwise_xor(rolling, prod[..., i])
            out.append(rolling.unsqueeze(-1) % self.primes[:, i - 1])   # [n, L, heads]
        return torch.cat(out, -1) + self.offs
