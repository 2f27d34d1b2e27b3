"""Layout math of batched speculative decoding: how the verify rows of several sequences are packed
into one padded forward, how ragged accept lengths map back, and what the commit appends.

Pure functions (no device work); behaviour of the reference's
``crates/ferrite-exec/src/mtp_batch.rs:146-530`` (padded ladder, verify rows, ``SeqRowMap``,
``AppendPlan``, commit layout).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

LADDER = (1, 2, 4, 8, 16, 32)


def padded_seqs(n: int, ladder: Sequence[int] = LADDER) -> int:
    """Smallest ladder bucket that holds n sequences."""
    for b in ladder:
        if n <= b:
            return b
    raise ValueError(f"{n} sequences exceed the largest bucket {ladder[-1]}")


def verify_rows(n_seqs: int, width: int) -> int:
    return n_seqs * width


@dataclass(frozen=True)
class SeqRowMap:
    """Rows of the packed verify forward that belong to each sequence: sequence s owns rows
    [s * width, (s + 1) * width); padding sequences (s >= n_live) own rows that are computed and ignored."""
    n_live: int
    n_padded: int
    width: int

    def rows_of(self, s: int) -> range:
        assert 0 <= s < self.n_padded
        return range(s * self.width, (s + 1) * self.width)

    def seq_of(self, row: int) -> Tuple[int, int]:
        return divmod(row, self.width)

    def live_rows(self) -> List[int]:
        return [r for s in range(self.n_live) for r in self.rows_of(s)]

    @property
    def n_rows(self) -> int:
        return self.n_padded * self.width


@dataclass(frozen=True)
class AppendPlan:
    """What a commit appends: for sequence s, `keep[s]` verify rows stay (1 .. width) and their tokens
    `emitted[s]` are published; cache positions [base[s], base[s] + keep[s]) become valid."""
    keep: Tuple[int, ...]
    base: Tuple[int, ...]
    emitted: Tuple[Tuple[int, ...], ...]

    def new_lengths(self) -> Tuple[int, ...]:
        return tuple(b + k for b, k in zip(self.base, self.keep))

    def rows_to_keep(self, rmap: SeqRowMap) -> List[int]:
        return [rmap.rows_of(s)[i] for s in range(len(self.keep)) for i in range(self.keep[s])]


def plan_commit(rmap: SeqRowMap, drafts: Sequence[Sequence[int]], judges: Sequence[Sequence[int]],
                base: Sequence[int]) -> AppendPlan:
    """drafts[s] = [d1..d_{w-1}], judges[s] = verify argmax of the w rows of sequence s (anchor row in
    the block): accept the longest matching prefix, emit accepted drafts plus the bonus token."""
    keep, emitted = [], []
    for s in range(rmap.n_live):
        m = 0
        while m < rmap.width - 1 and drafts[s][m] == judges[s][m]:
            m += 1
        keep.append(m + 1)
        emitted.append(tuple(judges[s][:m + 1]))
    return AppendPlan(tuple(keep), tuple(base[:rmap.n_live]), tuple(emitted))
