"""The single speculative-accept chain shared by GLM-MTP and the DSpark block draft.

Contract (reference ``crates/ferrite-types/src/spec_step.rs:61-166``): ``drafts[i]`` is the
proposal for the i-th new position, ``judges[i]`` the verify argmax that judges it.  With the
anchor row inside the verify block (GLM ``[t_last, d1..d_nd]``) the result counts EMITTED
tokens, ``1..=len(drafts)+1``; without it (DSpark ``[d1..d5]``, caller prepends the anchor's
argmax to ``judges``) it counts ACCEPTED drafts, ``0..=len(drafts)``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Sequence


def spec_accept(drafts: Sequence[int], judges: Sequence[int], anchor_is_in_block: bool) -> int:
    lim = min(len(drafts), len(judges))
    matched = 0
    while matched < lim and int(drafts[matched]) == int(judges[matched]):
        matched += 1
    return matched + 1 if anchor_is_in_block else matched


class SpecStep(ABC):
    """draft -> verify -> accept -> commit seam; an engine binds its block layout once."""

    ANCHOR_IS_IN_BLOCK: bool = True

    @abstractmethod
    def spec_step(self, *args, **kw):
        ...

    @classmethod
    def accept(cls, drafts: Sequence[int], judges: Sequence[int]) -> int:
        return spec_accept(drafts, judges, cls.ANCHOR_IS_IN_BLOCK)
