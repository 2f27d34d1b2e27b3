"""Expert-parallel MoE layer: all-to-all dispatch and combine over peer memory around the grouped
tensor-core expert kernels (``csrc/kernels/ep.cu``).

Each rank owns ``E / world`` whole experts and a block of token rows.  ``EpMoE.forward`` takes the
rank's rows (split activation planes) with their routing and returns the routed-expert output
of those rows; three of its five launches are the collective-carrying kernels:

    fb_ep_dispatch -> fb_moe_gate_up_mma -> fb_moe_down_mma -> fb_ep_combine

The reference keeps activations replicated and all-reduces the expert output
(``crates/ferrite-exec/src/lib.rs:1083-1166``); this is the token-sharded alternative that
moves only the rows (and back only their partial sums).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from .status import StatusArena
from .symm import DEFAULT_MAX_SPINS, SymmetricRegion, _Checked


class _Ptr:
    def __init__(self, p: int):
        self.p = p

    def data_ptr(self) -> int:
        return self.p


class EpMoE(_Checked):
    name = "ep_moe"

    def __init__(self, device, rank: int, world: int, n_max: int, hidden: int, topk: int, inter: int,
                 max_spins: int = DEFAULT_MAX_SPINS, group=None, arena=None):
        self.K = _lib.lib()
        self.dev, self.rank, self.world = torch.device(device), rank, world
        self.n_max, self.H, self.topk, self.I, self.max_spins = n_max, hidden, topk, inter, max_spins
        self.n_all = world * n_max
        self.planes = 4
        self.regions = [
            SymmetricRegion(self.planes * self.n_all * hidden * 2, rank, world, group),   # gathered activation planes
            SymmetricRegion(self.n_all * topk * 4, rank, world, group),                   # gathered expert ids
            SymmetricRegion(self.n_all * topk * 4, rank, world, group),                   # gathered routing weights
            SymmetricRegion(world * n_max * hidden * 4, rank, world, group),              # combine staging
            SymmetricRegion(2 * world * 32 * 4, rank, world, group),                      # flags
        ]
        arr = ctypes.c_void_p * (5 * world)
        self._ptrs = arr(*[p for reg in self.regions for p in reg.ptrs])
        self.xs_all, self.ids_all, self.wts_all = (_Ptr(self.regions[i].local) for i in range(3))
        self.arena = arena if arena is not None else StatusArena(self.dev, 256)
        self.epoch = self.arena.take(1, "ep_moe.epoch")
        self.ticket = self.arena.take(1, "ep_moe.ticket")
        self.status = self.arena.status("ep_moe")
        self.act_s = torch.zeros(4, self.n_all * topk, inter, dtype=torch.int16, device=self.dev)
        self.y_all = torch.zeros(self.n_all, hidden, device=self.dev)

    def dispatch(self, xs_local, local_plane: int, ids, wts, n_loc: int):
        self.K.call("fb_ep_dispatch", xs_local, local_plane, ids, wts, n_loc, self.n_max, self.H, self.topk, self.planes,
                    self._ptrs, self.epoch, self.ticket, self.status, self.rank, self.world, self.max_spins)

    def combine(self, y_out, n_loc: int, addend=None):
        self.K.call("fb_ep_combine", self.y_all, addend, y_out, n_loc, self.n_max, self.H, self._ptrs, self.epoch,
                    self.ticket, self.status, self.rank, self.world, self.max_spins)

    def forward(self, xs_local, local_plane: int, ids, wts, n_loc: int, w13, s13, w2, s2, e_per_rank: int,
                limit: float, y_out, addend=None):
        """w13 [El, 2I, H] / w2 [El, H, I]: this rank's experts (e4m3, 128x128 block scales s13 / s2)."""
        H, I, topk = self.H, self.I, self.topk
        self.dispatch(xs_local, local_plane, ids, wts, n_loc)
        plane_all = self.n_all * H
        ld_as, plane_as = I, self.n_all * topk * I
        e_lo = self.rank * e_per_rank
        self.K.call("fb_moe_gate_up_mma", w13, s13, self.xs_all, H, plane_all, self.ids_all, self.wts_all, self.act_s,
                    ld_as, plane_as, self.n_all, topk, I, H, e_lo, e_per_rank, float(limit))
        self.K.call("fb_moe_down_mma", w2, s2, self.act_s, ld_as, plane_as, self.ids_all, self.y_all, H, self.n_all,
                    topk, I, H, e_lo, e_per_rank, 0, None, 0, 0, 0)
        self.combine(y_out, n_loc, addend)

    def close(self):
        for r in self.regions:
            r.close()
