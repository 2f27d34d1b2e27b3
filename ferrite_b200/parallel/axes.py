"""Axis algebra of the deployment mesh: which axis a module shards along in each phase and how its
results merge back (sum, LSE, concat, row gather, pipeline).

One table drives three things: the TP weight slicer (head column), the placement of collectives
(merge kinds) and the PDAF reshard (KV column).  Behaviour of the reference's
``crates/ferrite-kv/src/axes.rs:46-300`` (``Axis``, ``ShardAxes``, ``RankCoord``, ``group_along``,
``MergeKind``, ``module_parallel``).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from enum import Enum
from typing import List


class Axis(Enum):
    HEAD = "head"   # head / inter / expert dim: weights slice, projections partial-sum
    KV = "kv"       # KV page dim (context axis): stable LSE merge
    Q = "q"         # query token segments (prefill sequence axis): row gather / state pipeline


class MergeKind(Enum):
    NONE = "none"
    SUM = "sum"
    LSE = "lse"
    CONCAT = "concat"
    ROW_GATHER = "row_gather"
    PIPELINE = "pipeline"


class Phase(Enum):
    PREFILL = "prefill"
    DECODE = "decode"


class TensorAxis(Enum):
    HEAD = "head"
    KV_PAGES = "kv_pages"
    HEAD_AND_KV_PAGES = "head_and_kv_pages"
    Q_SEGMENTS = "q_segments"
    REPLICATED = "replicated"


class ModuleKind(Enum):
    GDN_ATTN = "gdn_attn"
    DSA_INDEXER = "dsa_indexer"
    DSA_ATTN = "dsa_attn"
    DSA_LATENT_KV = "dsa_latent_kv"
    DENSE_MLP = "dense_mlp"
    MOE = "moe"
    REPLICATED = "replicated"


@dataclass(frozen=True)
class RankCoord:
    tp: int
    kv: int
    q: int


@dataclass(frozen=True)
class ShardAxes:
    tp: int = 1
    kv: int = 1
    q: int = 1

    def __post_init__(self):
        assert self.tp >= 1 and self.kv >= 1 and self.q >= 1, "axis sizes must be >= 1 (1 = unsharded)"

    @property
    def world(self) -> int:
        return self.tp * self.kv * self.q

    def size(self, axis: Axis) -> int:
        return {Axis.HEAD: self.tp, Axis.KV: self.kv, Axis.Q: self.q}[axis]

    def coord(self, linear: int) -> RankCoord:
        assert 0 <= linear < self.world, f"rank {linear} out of mesh {self}"
        tp, rest = divmod(linear, self.kv * self.q)
        return RankCoord(tp, rest // self.q, rest % self.q)

    def linear(self, c: RankCoord) -> int:
        return c.tp * self.kv * self.q + c.kv * self.q + c.q

    def group_along(self, axis: Axis, at: RankCoord) -> List[RankCoord]:
        """The communication group of a merge along `axis`, every other coordinate fixed at `at`."""
        field = {Axis.HEAD: "tp", Axis.KV: "kv", Axis.Q: "q"}[axis]
        return [replace(at, **{field: i}) for i in range(self.size(axis))]

    def group_ranks(self, axis: Axis, linear: int) -> List[int]:
        return [self.linear(c) for c in self.group_along(axis, self.coord(linear))]


@dataclass(frozen=True)
class ModuleParallel:
    axis: TensorAxis
    head_merge: MergeKind
    kv_merge: MergeKind
    q_merge: MergeKind


_N, _S, _L, _C, _R, _P = (MergeKind.NONE, MergeKind.SUM, MergeKind.LSE, MergeKind.CONCAT, MergeKind.ROW_GATHER,
                          MergeKind.PIPELINE)


def module_parallel(kind: ModuleKind, phase: Phase) -> ModuleParallel:
    """The GLM module x phase table."""
    if kind is ModuleKind.DSA_ATTN:
        if phase is Phase.PREFILL:
            return ModuleParallel(TensorAxis.Q_SEGMENTS, _C, _L, _R)
        return ModuleParallel(TensorAxis.HEAD_AND_KV_PAGES, _C, _L, _N)
    if kind is ModuleKind.DSA_INDEXER:
        return ModuleParallel(TensorAxis.KV_PAGES, _N, _C, _N)      # page-local scores gathered, one global top-k
    if kind is ModuleKind.DSA_LATENT_KV:
        return ModuleParallel(TensorAxis.KV_PAGES, _N, _N, _N)      # pages disjoint: placement only
    if kind is ModuleKind.GDN_ATTN:
        if phase is Phase.PREFILL:
            return ModuleParallel(TensorAxis.Q_SEGMENTS, _S, _N, _P)  # chunk state chain
        return ModuleParallel(TensorAxis.HEAD, _S, _N, _N)
    if kind in (ModuleKind.DENSE_MLP, ModuleKind.MOE):
        return ModuleParallel(TensorAxis.HEAD, _S, _N, _N)
    return ModuleParallel(TensorAxis.REPLICATED, _N, _N, _N)


def layer_modules(cfg, layer: int) -> List[ModuleKind]:
    """Module kinds of one GLM layer, in execution order."""
    out = [ModuleKind.REPLICATED]
    if cfg.is_dsa(layer):
        out += [ModuleKind.DSA_INDEXER, ModuleKind.DSA_LATENT_KV, ModuleKind.DSA_ATTN]
    else:
        out.append(ModuleKind.GDN_ATTN)
    out.append(ModuleKind.MOE if cfg.is_moe(layer) else ModuleKind.DENSE_MLP)
    return out


def collectives_per_step(cfg, axes: ShardAxes, phase: Phase) -> dict:
    """How many merges of each kind one forward pass issues on this mesh (for planning and tests)."""
    counts = {k: 0 for k in MergeKind}
    for l in range(cfg.num_layers):
        for kind in layer_modules(cfg, l):
            mp = module_parallel(kind, phase)
            for size, merge in ((axes.tp, mp.head_merge), (axes.kv, mp.kv_merge), (axes.q, mp.q_merge)):
                if size > 1 and merge is not MergeKind.NONE:
                    counts[merge] += 1
    return {k.value: v for k, v in counts.items() if v}
