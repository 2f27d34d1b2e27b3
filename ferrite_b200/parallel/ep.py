"""Expert-parallel MoE layer: all-to-all dispatch and combine over peer memory around the grouped
tensor-core expert kernels (``csrc/kernels/ep.cu``).

Each rank owns ``E / world`` whole experts and a block of token rows.  ``EpMoE.forward`` takes the
rank's rows (split activation planes) with their routing and returns the routed-expert output
of those rows.  Dispatch sends a row's planes only to the ranks that own one of its top-k experts.

    decode rows    fb_ep_dispatch -> fb_moe_gate_up_mma -> fb_moe_down_mma -> fb_ep_combine
    >= 64 pairs    fb_ep_dispatch -> fb_mx_sort -> fb_scatter_rows_16 -> fb_fp8w_gemm_grouped (gate | up)
                   -> fb_swiglu_rows_f16 -> fb_fp8w_gemm_grouped (down) -> fb_mx_combine -> fb_ep_combine

The second chain is the expert-grouped tcgen05 GEMM (``csrc/kernels/fp8w_gemm.cu``) between the two collective
kernels: gathered rows are sorted by local expert, every expert's weights stream once.

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
        self.tc_pairs = 64          # gathered (row, slot) pairs from which the grouped tcgen05 GEMM takes over
        self._tc = None

    def dispatch(self, xs_local, local_plane: int, ids, wts, n_loc: int, e_per_rank: int = 0):
        self.K.call("fb_ep_dispatch", xs_local, local_plane, ids, wts, n_loc, self.n_max, self.H, self.topk, self.planes,
                    e_per_rank, self._ptrs, self.epoch, self.ticket, self.status, self.rank, self.world, self.max_spins)

    def _tc_ws(self, El: int):
        if self._tc is None:
            npair, dev = self.n_all * self.topk, self.dev
            i32 = lambda *a: torch.zeros(*a, dtype=torch.int32, device=dev)
            mt = npair // 32 + El + 1
            self._tc = {"pos": i32(npair), "wts": torch.zeros(npair, device=dev), "counts": i32(512), "offsets": i32(513),
                        "tiles": i32(mt, 4), "nt": i32(1), "mt": mt,
                        "x": torch.zeros(npair, self.H, dtype=torch.float16, device=dev),
                        "h": torch.zeros(npair, 2 * self.I, device=dev),
                        "act": torch.zeros(npair, self.I, dtype=torch.float16, device=dev),
                        "ypair": torch.zeros(npair, self.H, device=dev),
                        "status": self.arena.status("ep_moe.tcgen05")}
        return self._tc

    def combine(self, y_out, n_loc: int, addend=None):
        self.K.call("fb_ep_combine", self.y_all, addend, y_out, n_loc, self.n_max, self.H, self._ptrs, self.epoch,
                    self.ticket, self.status, self.rank, self.world, self.max_spins)

    def forward(self, xs_local, local_plane: int, ids, wts, n_loc: int, w13, s13, w2, s2, e_per_rank: int,
                limit: float, y_out, addend=None):
        """w13 [El, 2I, H] / w2 [El, H, I]: this rank's experts (e4m3, 128x128 block scales s13 / s2)."""
        H, I, topk = self.H, self.I, self.topk
        self.dispatch(xs_local, local_plane, ids, wts, n_loc, e_per_rank)
        plane_all = self.n_all * H
        npairs = self.n_all * topk
        if npairs >= self.tc_pairs and H % 128 == 0 and I % 128 == 0 and e_per_rank <= 512:
            t, K = self._tc_ws(e_per_rank), self.K
            bn = 32 if npairs <= 32 * e_per_rank else 64 if npairs <= 64 * e_per_rank else 128
            K.call("fb_mx_sort", self.ids_all, self.wts_all, npairs, self.rank * e_per_rank, e_per_rank, bn, t["pos"], t["wts"],
                   t["counts"], t["offsets"], t["tiles"], t["nt"], t["mt"])
            f16_hi = _Ptr(self.xs_all.p + 2 * plane_all * 2)       # plane 2 of the gathered split activations
            K.call("fb_scatter_rows_16", f16_hi, H, t["pos"], topk, self.n_all, H, t["x"])
            K.call("fb_fp8w_gemm_grouped", w13, s13, t["x"], t["tiles"], t["nt"], t["mt"], t["h"], 2 * I, npairs, e_per_rank,
                   2 * I, H, bn, t["status"])
            m_ptr = _Ptr(t["offsets"].data_ptr() + 4 * e_per_rank)
            K.call("fb_swiglu_rows_f16", t["h"], 2 * I, t["wts"], m_ptr, npairs, I, float(limit), t["act"])
            K.call("fb_fp8w_gemm_grouped", w2, s2, t["act"], t["tiles"], t["nt"], t["mt"], t["ypair"], H, npairs, e_per_rank,
                   H, I, bn, t["status"])
            K.call("fb_mx_combine", t["ypair"], H, t["pos"], topk, self.y_all, H, self.n_all, H, 0)
            self.combine(y_out, n_loc, addend)
            return
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
