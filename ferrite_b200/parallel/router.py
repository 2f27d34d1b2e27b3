"""Static op plan of a model and the PDAF router: prefill work goes to the prefill (CP, layer-split)
group, decode work to the decode (DCP) group, and a sequence that finishes its prefill produces one
transfer event describing where its KV pages and states go.

Behaviour of the reference's ``crates/ferrite-scheduler/src/lib.rs:22-175`` (``StaticPlan``,
``PdafRouter``, ``TransferEvent``) with the layer ranges of ``crates/ferrite-kv/src/shard.rs:60-66``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .pdaf import TransferPlan


@dataclass(frozen=True)
class LayerOp:
    layer: int
    kind: str          # "attn:linear" | "attn:dsa" | "ffn:dense" | "ffn:moe"
    first_half: bool


@dataclass
class StaticPlan:
    ops: List[LayerOp]
    num_layers: int
    num_linear: int
    num_dsa: int
    num_moe: int
    num_dense: int

    @staticmethod
    def from_config(cfg) -> "StaticPlan":
        ops: List[LayerOp] = []
        c = dict(linear=0, dsa=0, moe=0, dense=0)
        for l in range(cfg.num_layers):
            a = "dsa" if cfg.is_dsa(l) else "linear"
            f = "moe" if cfg.is_moe(l) else "dense"
            c[a] += 1
            c[f] += 1
            ops.append(LayerOp(l, f"attn:{a}", True))
            ops.append(LayerOp(l, f"ffn:{f}", False))
        return StaticPlan(ops, cfg.num_layers, c["linear"], c["dsa"], c["moe"], c["dense"])

    def layer_ops(self, layer: int) -> List[LayerOp]:
        return [o for o in self.ops if o.layer == layer]


def cp_layer_range(num_layers: int, n_cp: int, rank: int) -> Tuple[int, int]:
    """Contiguous layer range [lo, hi) of prefill rank `rank`; the remainder goes to the first ranks."""
    base, rem = divmod(num_layers, n_cp)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


@dataclass(frozen=True)
class TransferEvent:
    seq: int
    n_tokens: int
    plans: Tuple[TransferPlan, ...]     # one per decode rank of the DCP group


@dataclass
class PdafRouter:
    """Routes the planner's work items to the two groups and emits transfer events."""
    prefill_ranks: List[int]
    decode_ranks: List[int]
    page_size: int
    prefilling: Dict[int, int] = field(default_factory=dict)    # seq -> prompt tokens still to prefill
    done: Dict[int, int] = field(default_factory=dict)          # seq -> prompt length (prefilled, not yet moved)
    decoding: Dict[int, int] = field(default_factory=dict)      # seq -> context position
    prompt_len: Dict[int, int] = field(default_factory=dict)

    def admit(self, seq: int, prompt_len: int) -> None:
        assert seq not in self.prefilling and seq not in self.decoding
        self.prefilling[seq] = prompt_len
        self.prompt_len[seq] = prompt_len

    def route_prefill(self, seq: int, chunk_tokens: int) -> List[int]:
        """Ranks that run this chunk (every prefill rank: each owns a layer range)."""
        left = self.prefilling[seq]
        assert 0 < chunk_tokens <= left
        self.prefilling[seq] = left - chunk_tokens
        if self.prefilling[seq] == 0:
            del self.prefilling[seq]
            self.done[seq] = self.prompt_len[seq]
        return list(self.prefill_ranks)

    def transfers(self) -> List[TransferEvent]:
        """Sequences whose prefill just finished: their pages split p % n_dcp over the decode group."""
        out = []
        n = len(self.decode_ranks)
        for seq, ntok in sorted(self.done.items()):
            out.append(TransferEvent(seq, ntok, tuple(TransferPlan(ntok, self.page_size, n, d) for d in range(n))))
            self.decoding[seq] = ntok
        self.done.clear()
        return out

    def route_decode(self, seq: int) -> List[int]:
        """Every decode rank takes part in a decode step (each over its own pages)."""
        self.decoding[seq] += 1
        return list(self.decode_ranks)

    def finish(self, seq: int) -> None:
        self.decoding.pop(seq, None)
        self.prompt_len.pop(seq, None)
