"""All-reduce providers for the tensor-parallel chain.

``make_allreduce`` returns a callable ``f(view)`` that sums a [n, H] f32 buffer across the
ranks in place on the current stream.  ``nccl`` is the library baseline; ``p2p`` is the
one-shot peer-memory all-reduce of :mod:`ferrite_b200.parallel.symm` (bounded waits, status
word), the counterpart of the reference's AR v5 (``kernels/cuda/ferrite_kernels.cu:8968-9524``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def make_allreduce(device, rank: int, world: int, max_elems: int, kind: str = "nccl", fused: bool = True):
    """kind "p2p" also carries ``.fused``, the GEMV + all-reduce (+ fold) kernel for decode rows, and
    ``.gemm_fused``, the tcgen05 GEMM + two-shot all-reduce kernel for prefill rows, unless fused=False."""
    if kind == "p2p":
        from .symm import CrossRankArgmax, FusedGemmAllReduce, FusedGemvAllReduce, P2PAllReduce
        ar = P2PAllReduce(device, rank, world, max_elems)
        if fused:
            ar.fused = FusedGemvAllReduce(device, rank, world)
            ar.gemm_fused = FusedGemmAllReduce(device, rank, world, max_rows=256, n_max=8192)
        ar.argmax = CrossRankArgmax(device, rank, world)   # enables the vocab-sliced head
        return ar

    def nccl_allreduce(view: torch.Tensor):
        dist.all_reduce(view)

    return nccl_allreduce
