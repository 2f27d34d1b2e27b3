"""All-reduce providers for the tensor-parallel chain.

``make_allreduce`` returns a callable ``f(view)`` that sums a [n, H] f32 buffer across the
ranks in place on the current stream.  ``nccl`` is the library baseline; ``p2p`` is the
one-shot peer-memory all-reduce of :mod:`ferrite_b200.parallel.symm` (bounded waits, status
word), the counterpart of the reference's AR v5 (``kernels/cuda/ferrite_kernels.cu:8968-9524``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def make_allreduce(device, rank: int, world: int, max_elems: int, kind: str = "nccl", fused: bool = True,
                   max_spins: int = 0, group=None):
    """kind "p2p" also carries ``.fused``, the GEMV + all-reduce (+ fold) kernel for decode rows, and
    ``.gemm_fused``, the tcgen05 GEMM + two-shot all-reduce kernel for prefill rows, unless fused=False.
    ``group``: the process group of the ``world`` ranks (``rank`` is the rank inside it); None = all ranks."""
    if kind == "p2p":
        from .status import StatusArena
        from .symm import DEFAULT_MAX_SPINS, CrossRankArgmax, FusedGemmAllReduce, FusedGemvAllReduce, P2PAllReduce
        spins = max_spins or DEFAULT_MAX_SPINS
        arena = StatusArena(device)   # one block of status / epoch / ticket words per rank, read back once per step
        ar = P2PAllReduce(device, rank, world, max_elems, max_spins=spins, arena=arena, group=group)
        ar.group = group
        if fused:
            ar.fused = FusedGemvAllReduce(device, rank, world, max_spins=spins, arena=arena, group=group)
            ar.gemm_fused = FusedGemmAllReduce(device, rank, world, max_rows=256, n_max=8192, max_spins=spins, arena=arena,
                                               group=group)
        ar.argmax = CrossRankArgmax(device, rank, world, max_spins=spins, arena=arena, group=group)   # vocab-sliced head
        return ar

    def nccl_allreduce(view: torch.Tensor):
        dist.all_reduce(view, group=group)

    nccl_allreduce.group = group
    return nccl_allreduce


def startup_barrier(world: int, group=None) -> None:
    """Line the ranks up after an engine is built and before its first peer-memory launch.  Weight loading
    and graph warm-up take seconds to minutes and differ between ranks; the device-side waits are sized for
    the skew inside a step (about two seconds), so the start-up skew is absorbed here, on the host, where a
    missing rank ends in the process group's own timeout instead of in a spinning kernel."""
    if world > 1 and dist.is_available() and dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier(group=group)


def self_test(ar, device, rank: int, world: int) -> dict:
    """Start-up check of the peer-memory collectives against NCCL on small random payloads.  Every rank
    reaches the same verdict (the failure flags are max-reduced); a fused kernel that fails or times out is
    detached (``ar.fused`` / ``ar.gemm_fused`` / ``ar.argmax`` set to None: the engines then fall back to
    separate kernels), a failing base all-reduce raises.  Returns {"allreduce": bool, "gemv_ar": bool,
    "gemm_ar": bool, "argmax": bool}."""
    from .. import _lib
    from ..models.glm import Act
    K = _lib.lib()
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    verdict = {}

    def agree(ok: bool) -> bool:
        t = torch.tensor([0 if ok else 1], device=device, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item()) == 0

    def guarded(fn) -> bool:
        try:
            ok = bool(fn())
            torch.cuda.synchronize()
            ar.check()
            return ok
        except Exception:
            return False

    def t_allreduce():
        x = torch.randn(3 * 4096, device=device, generator=g)
        want = x.clone()
        dist.all_reduce(want)
        ar(x)
        return torch.allclose(x, want, atol=1e-4, rtol=1e-5)

    verdict["allreduce"] = agree(guarded(t_allreduce))
    if not verdict["allreduce"]:
        raise RuntimeError("peer-memory all-reduce failed its start-up check against NCCL")

    def t_gemv():
        N, Kd, m = 4096, 512, 3
        W = (torch.randn(N, Kd, device=device, generator=g) * 0.05).to(torch.bfloat16)
        x = Act(device, 8, Kd)
        x.f.copy_(torch.randn(8, Kd, device=device, generator=g))
        K.call("fb_split_rows", x.f, Kd, *x.sp(3), 8, Kd)
        want = (x.f[:m].double() @ W.double().t()).float()
        dist.all_reduce(want)
        y = torch.zeros(8, N, device=device)
        ar.fused(W, None, x.s, Kd, x.plane, y, N, m, N, Kd, False, True, None)
        torch.cuda.synchronize()
        return (y[:m] - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())

    def t_gemm():
        N, Kd, m = 4096, 256, 64
        W = (torch.randn(N, Kd, device=device, generator=g) * 0.05).to(torch.bfloat16)
        xb = torch.randn(m, Kd, device=device, generator=g).to(torch.bfloat16)
        want = (xb.double() @ W.double().t()).float()
        dist.all_reduce(want)
        ok = True
        for rows in (m, 256):     # a one-shot sized and a two-shot sized launch
            xr = xb if rows == m else xb.repeat(4, 1)
            wr = want if rows == m else want.repeat(4, 1)
            if not ar.gemm_fused.fits(rows, N):
                continue
            y = torch.zeros(rows, N, device=device)
            ar.gemm_fused(W, xr.contiguous(), Kd, y, N, rows, N, Kd, False)
            torch.cuda.synchronize()
            ok = ok and (y - wr).abs().max().item() < 2e-3 * max(1.0, wr.abs().max().item())
        return ok

    def t_argmax():
        V, n = 4096, 3
        full = torch.randn(n, V * world, device=device, generator=torch.Generator(device=device).manual_seed(77))
        mine = full[:, rank * V:(rank + 1) * V].contiguous()
        part = torch.zeros(n * 64, dtype=torch.int64, device=device)
        ids = torch.zeros(n, dtype=torch.int32, device=device)
        ar.argmax(mine, V, part, n, V, rank * V, ids)
        torch.cuda.synchronize()
        return ids.tolist() == full.argmax(-1).tolist()

    for name, attr, fn in (("gemv_ar", "fused", t_gemv), ("gemm_ar", "gemm_fused", t_gemm), ("argmax", "argmax", t_argmax)):
        if getattr(ar, attr, None) is None:
            verdict[name] = False
            continue
        verdict[name] = agree(guarded(fn))
        if not verdict[name]:
            try:
                getattr(ar, attr).status.zero_()
            except Exception:
                pass
            setattr(ar, attr, None)
    return verdict
