"""Symmetric peer memory over CUDA IPC and the one-shot all-reduce built on it.

One process per GPU: every rank allocates its region with ``cudaMalloc``, exports it with
``cudaIpcGetMemHandle``, and opens the peers' handles, so that kernels can store straight
into a peer's HBM over NVLink.  Handles travel through ``torch.distributed`` (any backend).
The reference keeps its ranks as threads of one process and enables peer access directly
(``crates/ferrite-kernel/src/cuda.rs:6607-6762``); the collective itself is described in
``csrc/kernels/collective.cu``.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib

from .status import (FB_BAD_ARG, FB_BAD_CANARY, FB_OK, FB_TIMEOUT, CollectiveTimeout,  # noqa: F401
                     StatusArena)

# Polls of a bounded device wait before it gives up (about two seconds).  Ranks line up on a host barrier
# after their engines are built, so a wait only has to cover the skew inside a step, and a peer that died
# is reported within seconds.  A wait that ran out is sticky until the host clears the status word.
DEFAULT_MAX_SPINS = 2_000_000


class _Checked:
    """Shared ``check()``: read this object's status word on the host (synchronises)."""
    status: torch.Tensor
    name = "collective"

    def check(self):
        s = self.status.tolist()
        if s[0] == FB_TIMEOUT:
            self.status.zero_()
            raise CollectiveTimeout(s[1], s[2], s[3], self.name)


class SymmetricRegion:
    """``nbytes`` of zeroed device memory on every rank, each rank holding pointers to all."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        self.K = _lib.lib()
        self.nbytes, self.rank, self.world = nbytes, rank, world
        p = ctypes.c_void_p()
        self._check(self.K.lib.fb_symm_alloc(ctypes.c_int64(nbytes), ctypes.byref(p)), "fb_symm_alloc")
        self.local = p.value
        handle = ctypes.create_string_buffer(64)
        self._check(self.K.lib.fb_ipc_get_handle(ctypes.c_void_p(self.local), handle), "fb_ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self.local)
                continue
            q = ctypes.c_void_p()
            self._check(self.K.lib.fb_ipc_open(ctypes.c_char_p(handles[r]), ctypes.byref(q)), "fb_ipc_open")
            self.ptrs.append(q.value)
            self._opened.append(q.value)
        dist.barrier(group=group)

    @staticmethod
    def _check(rc: int, what: str):
        if rc != 0:
            raise _lib.KernelError(f"{what} failed with CUDA error {rc}")

    def close(self):
        for q in self._opened:
            self.K.lib.fb_ipc_close(ctypes.c_void_p(q))
        self._opened = []
        if self.local:
            self.K.lib.fb_symm_free(ctypes.c_void_p(self.local))
            self.local = 0


class P2PAllReduce(_Checked):
    """Callable ``f(view)``: in-place sum of a contiguous f32 view across the ranks, one
    kernel launch on the current stream.  ``check()`` reads the status word on the host."""

    name = "allreduce"

    def __init__(self, device, rank: int, world: int, max_elems: int, max_spins: int = DEFAULT_MAX_SPINS, group=None,
                 arena: Optional[StatusArena] = None):
        self.K = _lib.lib()
        self.rank, self.world, self.max_spins = rank, world, max_spins
        self.arena = arena if arena is not None else StatusArena(device)
        mc, ce = ctypes.c_int(), ctypes.c_int()
        self.K.lib.fb_ar_limits(ctypes.byref(mc), ctypes.byref(ce))
        self.max_chunks, self.chunk = mc.value, ce.value
        self.max_elems = min((max_elems + self.chunk - 1) // self.chunk, self.max_chunks) * self.chunk
        self.staging = SymmetricRegion(2 * world * self.max_elems * 8, rank, world, group)   # (value, epoch) pairs
        self.flags = SymmetricRegion(2 * world * self.max_chunks * 4, rank, world, group)
        self.epoch = self.arena.take(self.max_chunks, "allreduce.epoch")
        self.status = self.arena.status("allreduce")
        arr = ctypes.c_void_p * world
        self._sp = arr(*self.staging.ptrs)
        self._fp = arr(*self.flags.ptrs)
        self.calls = 0
        self.fused: Optional["FusedGemvAllReduce"] = None   # attached by make_allreduce
        self.gemm_fused: Optional["FusedGemmAllReduce"] = None   # attached by make_allreduce
        self.argmax: Optional["CrossRankArgmax"] = None      # attached by make_allreduce

    def __call__(self, view: torch.Tensor):
        n = view.numel()
        assert view.is_contiguous() and view.dtype == torch.float32 and n <= self.max_elems and n % 4 == 0
        self.K.call("fb_ar_oneshot", self._sp, self._fp, self.epoch, self.status, view, n, self.rank, self.world,
                    self.max_elems, self.max_spins)
        self.calls += 1

    def check(self):
        """Host-side read of the guards and of every status word of this rank's collectives
        (synchronises the device)."""
        self.arena.verify(snapshot=False)
        _Checked.check(self)
        if self.fused is not None:
            self.fused.check()
        if self.gemm_fused is not None:
            self.gemm_fused.check()
        if self.argmax is not None:
            self.argmax.check()

    def close(self):
        if self.fused is not None:
            self.fused.close()
        if self.gemm_fused is not None:
            self.gemm_fused.close()
        if self.argmax is not None:
            self.argmax.close()
        self.staging.close()
        self.flags.close()


class _GemvArExt(ctypes.Structure):
    """Optional stages of ``fb_gemv_ar`` (``FbGemvArExt`` in csrc/kernels/gemv_ar.cu)."""
    _fields_ = [("gu", ctypes.c_void_p), ("gu_ld", ctypes.c_int64), ("gu_up_off", ctypes.c_int64), ("limit", ctypes.c_float),
                ("pre_scale", ctypes.c_void_p), ("pre_base", ctypes.c_void_p), ("pre_ln_w", ctypes.c_void_p),
                ("pre_post", ctypes.c_void_p), ("pre_comb", ctypes.c_void_p), ("pre_x", ctypes.c_void_p),
                ("xs_base", ctypes.c_void_p), ("xs_ld", ctypes.c_int64), ("xs_plane", ctypes.c_int64),
                ("xs_mask", ctypes.c_int64),
                ("gram", ctypes.c_void_p), ("coef", ctypes.c_void_p), ("bar", ctypes.c_void_p),
                ("rms_eps", ctypes.c_float), ("hc_eps", ctypes.c_float), ("iters", ctypes.c_int64)]


def _p(t):
    return None if t is None else t.data_ptr()


class FusedGemvAllReduce(_Checked):
    """Row-parallel GEMV + all-reduce (+ hyper-connection fold) as one kernel launch
    (``csrc/kernels/gemv_ar.cu``).  With ``world == 1`` it needs no peer memory and only fuses
    the fold epilogue into the GEMV.  ``check()`` reads the status word on the host."""

    name = "gemv_ar"

    def __init__(self, device, rank: int, world: int, max_rows: int = 8, n_max: int = 8192,
                 max_spins: int = DEFAULT_MAX_SPINS, group=None, arena: Optional[StatusArena] = None, ar_group: int = 0):
        self.K = _lib.lib()
        self.rank, self.world, self.max_spins = rank, world, max_spins
        self.arena = arena if arena is not None else StatusArena(device)
        mt, mw, fw = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        self.K.lib.fb_gemv_ar_limits(ctypes.byref(mt), ctypes.byref(mw), ctypes.byref(fw))
        assert world <= mw.value
        self.max_tiles = mt.value
        self.max_elems = max_rows * n_max
        self.epoch = self.arena.take(self.max_tiles, "gemv_ar.epoch")
        self.status = self.arena.status("gemv_ar")
        # mix-dot partials and tile counts for up to `part_rows` rows: a forward of more than 8 rows calls the
        # kernel once per 8-row window, each window with its own slice
        self.part_rows = 64
        self.part = torch.zeros(self.part_rows * 25 * self.max_tiles, dtype=torch.float32, device=device)
        self.part_n = torch.zeros(self.part_rows, dtype=torch.int32, device=device)
        self.ticket = self.arena.take(self.max_tiles, "gemv_ar.ticket")
        # one published group = the whole grid: system-scope fences are the expensive part (measured on 2 GPUs,
        # GLM decode step: groups of 16 tiles 11.99 ms, 64 -> 11.31, 128 -> 11.02, whole grid -> 10.88), and one
        # group means one epoch per launch, so staging parity cannot alias between launches of different widths
        self.group = ar_group if ar_group > 0 else self.max_tiles
        # hyper-connection front computed inside the launch: Gram partials, published coefficients, grid barrier
        self.gram = torch.zeros(8 * 10 * self.max_tiles, dtype=torch.float32, device=device)
        self.coef = torch.zeros(8 * 8, dtype=torch.float32, device=device)
        self.bar = self.arena.take(2, "gemv_ar.front_barrier")
        self.staging = self.flags = None
        self._sp = self._fp = None
        if world > 1:
            self.staging = SymmetricRegion(2 * world * self.max_elems * 8, rank, world, group)   # (value, epoch) pairs
            self.flags = SymmetricRegion(2 * world * self.max_tiles * fw.value * 4, rank, world, group)
            arr = ctypes.c_void_p * world
            self._sp = arr(*self.staging.ptrs)
            self._fp = arr(*self.flags.ptrs)
        self.calls = 0

    def __call__(self, W, scales, xs_ptr, xs_ld: int, xs_plane: int, y, ldo: int, m: int, N: int, K: int,
                 accumulate: bool, store_y: bool, fold=None, swiglu=None, front=None, gram: bool = False):
        """fold = (Rin, Rout, post, comb, fn_or_None, acc, mix) or None.  m may exceed 8 (up to part_rows):
        the kernel then runs once per 8-row window on row-offset pointers.
        swiglu = (gu, ld, up_off, limit): read the activations as SwiGLU of f32 [gate | up] rows instead of split planes.
        front = (scale, base, ln_w, post, comb, x_f32, (xs_base, xs_ld, xs_plane, xs_mask), rms_eps, hc_eps, iters):
        compute the NEXT site's hyper-connection front in the same launch (needs the fold with fn; m <= 8).
        gram: also leave the per-tile Gram partials of R' (for fb_hc_pre_wide; needs the fold with fn; m <= 8)."""
        rin = rout = post = comb = fn = acc = None
        mix = 0
        if fold is not None:
            rin, rout, post, comb, fn, acc, mix = fold
        assert m <= self.part_rows
        ext = None
        if swiglu is not None or front is not None or gram:
            assert m <= 8
            e = _GemvArExt()
            if gram:
                e.gram = self.gram.data_ptr()
            if swiglu is not None:
                gu, ld, up_off, limit = swiglu
                e.gu, e.gu_ld, e.gu_up_off, e.limit = gu.data_ptr(), ld, up_off, limit
            if front is not None:
                scale, base, ln_w, fpost, fcomb, xf, xsp, rms_eps, hc_eps, iters = front
                e.pre_scale, e.pre_base, e.pre_ln_w = scale.data_ptr(), base.data_ptr(), ln_w.data_ptr()
                e.pre_post, e.pre_comb, e.pre_x = fpost.data_ptr(), fcomb.data_ptr(), xf.data_ptr()
                e.xs_base, e.xs_ld, e.xs_plane, e.xs_mask = _p(xsp[0]), xsp[1], xsp[2], xsp[3]
                e.gram, e.coef, e.bar = self.gram.data_ptr(), self.coef.data_ptr(), self.bar.data_ptr()
                e.rms_eps, e.hc_eps, e.iters = rms_eps, hc_eps, iters
            ext = ctypes.pointer(e)   # read by the launcher during the call only

        def off(t, elems, size=4):
            return None if t is None else ctypes.c_void_p(t.data_ptr() + elems * size)

        for r0 in range(0, m, 8):
            mm = min(8, m - r0)
            self.K.call("fb_gemv_ar", W, scales, off(xs_ptr, r0 * xs_ld, 2), xs_ld, xs_plane, off(y, r0 * ldo), ldo, mm, N, K,
                        int(accumulate), int(store_y), self._sp, self._fp, self.epoch, self.ticket, self.status,
                        self.rank, self.world, self.max_elems, self.max_spins, self.group,
                        off(rin, r0 * 4 * N), off(rout, r0 * 4 * N), off(post, r0 * 4), off(comb, r0 * 16), fn,
                        off(acc, r0 * 25), mix, off(self.part, r0 * 25 * self.max_tiles), off(self.part_n, r0), ext)
            self.calls += 1

    def partials(self):
        """(part, part_n, part_ld) arguments for the hc_pre kernel that consumes the mix-dot partials."""
        return (self.part, self.part_n, self.max_tiles)

    def wide_partials(self):
        """(part, gram, part_n, part_ld) arguments for fb_hc_pre_wide."""
        return (self.part, self.gram, self.part_n, self.max_tiles)

    def close(self):
        if self.staging is not None:
            self.staging.close()
            self.flags.close()
            self.staging = self.flags = None


class FusedGemmAllReduce(_Checked):
    """Row-parallel prefill GEMM (TMA + tcgen05) + two-shot all-reduce over peer memory as one kernel
    launch (``csrc/kernels/gemm_tc_ar.cu``): out[m, n] = sum over ranks of x_rank . W_rank^T.  Buffers
    are sized for ``max_rows`` x ``n_max`` outputs; ``fits(m, N)`` says whether a shape can go through
    the fused kernel (co-resident grid, at least one tile per rank)."""

    name = "gemm_ar"

    def __init__(self, device, rank: int, world: int, max_rows: int = 256, n_max: int = 8192,
                 max_spins: int = DEFAULT_MAX_SPINS, group=None, mode: int = 0, arena: Optional[StatusArena] = None):
        self.K = _lib.lib()
        self.rank, self.world, self.max_spins = rank, world, max_spins
        self.arena = arena if arena is not None else StatusArena(device)
        self.max_rows, self.n_max = max_rows, n_max
        self.mode = mode   # 0: the kernel chooses, 1: one-shot, 2: two-shot (all ranks must agree)
        pad_elems = (max_rows + 256) * (n_max + 128)          # whole tiles of any tile height
        self.gather_cap = 2 * pad_elems
        # two-shot: one rounding tile per source slot; two ranks run one-shot and hold both ranks' partials of all tiles
        self.scatter_cap = (2 * world * pad_elems if world == 2 or mode == 1
                            else 2 * pad_elems + 2 * world * 256 * 128)
        self.epoch = self.arena.take(1, "gemm_ar.epoch")
        self.ticket = self.arena.take(2, "gemm_ar.ticket")
        self.status = self.arena.status("gemm_ar")
        self.scatter = self.gather = self.flags = None
        self._sp = self._gp = self._fp = None
        if world > 1:
            self.scatter = SymmetricRegion(self.scatter_cap * 4, rank, world, group)
            self.gather = SymmetricRegion(self.gather_cap * 4, rank, world, group)
            self.flags = SymmetricRegion(4 * world * 32 * 4, rank, world, group)
            arr = ctypes.c_void_p * world
            self._sp = arr(*self.scatter.ptrs)
            self._gp = arr(*self.gather.ptrs)
            self._fp = arr(*self.flags.ptrs)
        self.calls = 0

    def plan(self, m: int, N: int):
        bn, nt = ctypes.c_int(), ctypes.c_int()
        self.K.lib.fb_gemm_tc_ar_plan(ctypes.c_int64(m), ctypes.c_int64(N), ctypes.byref(bn), ctypes.byref(nt))
        return bn.value, nt.value

    def fits(self, m: int, N: int) -> bool:
        bn, nt = self.plan(m, N)
        return 1 <= m <= self.max_rows and N <= self.n_max and N % 4 == 0 and self.world <= nt <= 148

    def __call__(self, W, x_bf16, ldx: int, out, ldo: int, m: int, N: int, K: int, accumulate: bool = False):
        """W [N, K] bf16 (this rank's K slice), x_bf16: pointer/tensor of [m, K] bf16 rows (stride ldx),
        out [m, N] f32 (stride ldo); all ranks must call with the same shape."""
        self.K.call("fb_gemm_tc_ar", W, x_bf16, ldx, out, ldo, m, N, K, int(accumulate), self._sp, self._gp, self._fp,
                    self.scatter_cap, self.gather_cap, self.epoch, self.ticket, self.status, self.rank, self.world,
                    self.max_spins, self.mode)
        self.calls += 1

    def close(self):
        if self.scatter is not None:
            self.scatter.close()
            self.gather.close()
            self.flags.close()
            self.scatter = self.gather = self.flags = None


class CrossRankArgmax(_Checked):
    """Greedy token of a vocab-sliced head: per-rank argmax partials merged over the ranks in one
    small kernel (``fb_argmax_xchg``); every rank gets the same global token id."""

    name = "argmax_xchg"

    def __init__(self, device, rank: int, world: int, max_spins: int = DEFAULT_MAX_SPINS, group=None,
                 arena: Optional[StatusArena] = None):
        self.K = _lib.lib()
        self.rank, self.world, self.max_spins = rank, world, max_spins
        self.arena = arena if arena is not None else StatusArena(device)
        mr = ctypes.c_int()
        self.K.lib.fb_argmax_xchg_limits(ctypes.byref(mr))
        self.max_rows = mr.value
        self.staging = SymmetricRegion(2 * world * self.max_rows * 8, rank, world, group)
        self.flags = SymmetricRegion(max(256, 2 * world * 4), rank, world, group)
        self.epoch = self.arena.take(1, "argmax_xchg.epoch")
        self.status = self.arena.status("argmax_xchg")
        arr = ctypes.c_void_p * world
        self._sp = arr(*self.staging.ptrs)
        self._fp = arr(*self.flags.ptrs)

    def __call__(self, logits, ld: int, part, n: int, v_local: int, vocab_offset: int, out_ids, id_stride: int = 1,
                 vals=None):
        self.K.call("fb_argmax_partial", logits, ld, part, n, v_local, vocab_offset)
        for r0 in range(0, n, self.max_rows):   # the exchange kernel takes up to max_rows rows per launch
            m = min(self.max_rows, n - r0)
            pp = ctypes.c_void_p(part.data_ptr() + r0 * 64 * 8)
            op = ctypes.c_void_p(out_ids.data_ptr() + r0 * id_stride * 4)
            vp = ctypes.c_void_p(vals.data_ptr() + r0 * 4) if vals is not None else None
            self.K.call("fb_argmax_xchg", pp, self._sp, self._fp, self.epoch, self.status, op, vp, id_stride, m,
                        self.rank, self.world, self.max_spins)

    def close(self):
        self.staging.close()
        self.flags.close()


class DcpAttentionMerge(_Checked):
    """Cross-rank LSE merge of sparse-attention partials for a decode-context-parallel group
    (``csrc/kernels/dsa_dcp.cu``): one launch per attention layer."""

    name = "dcp_merge"

    def __init__(self, device, rank: int, world: int, max_rows: int, heads: int, latent_dim: int,
                 max_spins: int = DEFAULT_MAX_SPINS, group=None, arena: Optional[StatusArena] = None):
        self.K = _lib.lib()
        self.rank, self.world, self.max_spins = rank, world, max_spins
        self.arena = arena if arena is not None else StatusArena(device)
        self.slot_elems = max_rows * heads * (latent_dim + 4)
        self.staging = SymmetricRegion(2 * world * self.slot_elems * 4, rank, world, group)
        self.flags = SymmetricRegion(2 * world * 32 * 4, rank, world, group)
        self.epoch = self.arena.take(1, "dcp_merge.epoch")
        self.ticket = self.arena.take(1, "dcp_merge.ticket")
        self.status = self.arena.status("dcp_merge")
        arr = ctypes.c_void_p * world
        self._sp = arr(*self.staging.ptrs)
        self._fp = arr(*self.flags.ptrs)

    def __call__(self, o_part, ml_part, ctx, n: int, heads: int, latent_dim: int, nsplit: int, split=(None, 0, 0, 0)):
        self.K.call("fb_dsa_attn_merge_dcp", o_part, ml_part, ctx, n, heads, latent_dim, nsplit, self._sp, self._fp,
                    self.epoch, self.ticket, self.status, self.rank, self.world, self.slot_elems, self.max_spins, *split)

    def close(self):
        self.staging.close()
        self.flags.close()
