"""PDAF hand-off: move one prefilled sequence from a prefill rank to a decode rank over NCCL p2p.

What travels is exactly what the reference's CPU ``reshard`` moves
(``crates/ferrite-exec/src/distributed.rs:85-257``, ``crates/ferrite-kv/src/shard.rs:144-212``):

* state layers (GatedDeltaNet): the recurrent state buffers and the conv tail of the slot -
  passed through unchanged to every decode rank;
* paged layers (DSA): the latent / indexer-key / gate / pool pages the sequence uses; with a
  decode-context-parallel group of ``n_dcp`` ranks, rank ``d`` receives page ``p`` iff
  ``p % n_dcp == d`` and stores it at page slot ``p // n_dcp``;
* the sequence bookkeeping (lengths, snapshot cursor, MTP pair).

Pages are gathered into one contiguous staging tensor per cache, so each cache is a single
NCCL send; sends are issued as one batch on a side stream and overlap whatever the compute
stream is doing.  ``TransferPlan`` is the pure layout part (testable without GPUs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class TransferPlan:
    """Which pages of a sequence of ``n_tokens`` go to decode rank ``d`` of ``n_dcp``."""
    n_tokens: int
    page_size: int
    n_dcp: int = 1
    d: int = 0

    @property
    def n_pages(self) -> int:
        return (self.n_tokens + self.page_size - 1) // self.page_size

    @property
    def src_pages(self) -> List[int]:
        return [p for p in range(self.n_pages) if p % self.n_dcp == self.d]

    @property
    def dst_slots(self) -> List[int]:
        return [p // self.n_dcp for p in self.src_pages]

    def bytes_moved(self, bytes_per_page: int, state_bytes: int) -> int:
        return len(self.src_pages) * bytes_per_page + state_bytes


def _paged(model) -> Dict[str, torch.Tensor]:
    return {"lat": model.lat_cache, "kidx": model.kidx_cache, "kgate": model.kgate_cache, "pool": model.pool_cache}


def _state(model) -> Dict[str, torch.Tensor]:
    return {"gdn": model.gdn_state, "conv": model.conv_state}


def _engine_vectors(engine) -> Dict[str, torch.Tensor]:
    return {"block_ids": engine.block_ids, "mtp_ids": engine.mtp_ids, "mtp_h": engine.mtp_h}


def _page_lists(plan: TransferPlan, name: str, compact: bool):
    """(source pages, destination page slots) of one cache.  Only the latent cache is split over a
    DCP group; the indexer caches (keys, gates, pools) are needed whole by every rank because the
    top-k is global.  compact=False keeps every page at its own index on the destination."""
    if name != "lat" or plan.n_dcp == 1:
        pages = list(range(plan.n_pages))
        return pages, pages
    return plan.src_pages, (plan.dst_slots if compact else plan.src_pages)


def send_sequence(engine, dst: int, n_dcp: int = 1, d: int = 0, slot: int = 0, group=None,
                  stream: Optional[torch.cuda.Stream] = None, compact: bool = False) -> TransferPlan:
    """Send slot `slot` of a single-sequence engine (after ``prefill``) to rank `dst`."""
    m = engine.model
    ps = m.cfg.dsa.page_size
    plan = TransferPlan(engine.n_ctx, ps, n_dcp, d)
    dev = m.dev
    side = stream or torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        head = torch.tensor([engine.n_ctx, int(m.main_len[slot]), int(m.mtp_len[slot]), int(m.cur[slot])],
                            dtype=torch.int64, device=dev)
        for r in dist.batch_isend_irecv([dist.P2POp(dist.isend, head, dst, group)]):
            r.wait()
        ops = []
        base = slot * m.max_pages
        keep = []
        for name, cache in _paged(m).items():
            idx = torch.tensor([base + p for p in _page_lists(plan, name, compact)[0]], dtype=torch.long, device=dev)
            if idx.numel():
                buf = cache.index_select(1, idx).contiguous()   # [families, pages, ...]
                keep.append(buf)
                ops.append(dist.P2POp(dist.isend, buf, dst, group))
        for name, st in _state(m).items():
            buf = st[:, slot].contiguous()
            keep.append(buf)
            ops.append(dist.P2POp(dist.isend, buf, dst, group))
        for name, v in _engine_vectors(engine).items():
            ops.append(dist.P2POp(dist.isend, v, dst, group))
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    torch.cuda.current_stream(dev).wait_stream(side)
    return plan


def recv_sequence(engine, src: int, n_dcp: int = 1, d: int = 0, slot: int = 0, group=None,
                  stream: Optional[torch.cuda.Stream] = None, compact: bool = False) -> TransferPlan:
    """Receive a sequence into slot `slot`; afterwards the engine continues as if it had prefilled."""
    m = engine.model
    ps = m.cfg.dsa.page_size
    dev = m.dev
    side = stream or torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        head = torch.zeros(4, dtype=torch.int64, device=dev)
        for r in dist.batch_isend_irecv([dist.P2POp(dist.irecv, head, src, group)]):
            r.wait()
        n_ctx, main_len, mtp_len, cur = (int(v) for v in head.tolist())
        plan = TransferPlan(n_ctx, ps, n_dcp, d)
        ops, fills = [], []
        base = slot * m.max_pages
        for name, cache in _paged(m).items():
            idx = torch.tensor([base + s for s in _page_lists(plan, name, compact)[1]], dtype=torch.long, device=dev)
            if idx.numel():
                buf = torch.empty((cache.shape[0], idx.numel()) + tuple(cache.shape[2:]), dtype=cache.dtype, device=dev)
                ops.append(dist.P2POp(dist.irecv, buf, src, group))
                fills.append((cache, buf, idx))
        for name, st in _state(m).items():
            buf = torch.empty(tuple(st[:, slot].shape), dtype=st.dtype, device=dev)
            ops.append(dist.P2POp(dist.irecv, buf, src, group))
            fills.append((st, buf, None))
        for name, v in _engine_vectors(engine).items():
            ops.append(dist.P2POp(dist.irecv, v, src, group))
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        for dst_t, buf, ix in fills:
            if ix is None:
                dst_t[:, slot].copy_(buf)
            else:
                dst_t.index_copy_(1, ix, buf)
        m.main_len[slot] = main_len
        m.mtp_len[slot] = mtp_len
        m.cur[slot] = cur
    torch.cuda.current_stream(dev).wait_stream(side)
    engine.n_ctx = n_ctx
    return plan
