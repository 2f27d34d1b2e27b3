"""Context-parallel (layer-split) prefill group and its hand-off to a decode group.

A prefill group of ``n_stages`` ranks splits the main layers into contiguous ranges
(``crates/ferrite-kv/src/shard.rs:60-66`` ``cp_layer_range``); stage ``s`` holds ONLY the weights of its
layers (all experts of those layers: no tensor-parallel collectives inside prefill) and the caches /
recurrent states they write.  A prompt streams through the stages chunk by chunk: stage ``s`` receives the
hyper-connection residual streams of a chunk from stage ``s - 1`` over NCCL p2p, runs its layers, and
sends them on, so stage ``s`` works on chunk ``c`` while stage ``s + 1`` works on chunk ``c - 1``
(``crates/ferrite-exec/src/distributed.rs:85-257``).  The last stage owns the head, the first generated
token and the MTP layer (whose cache it fills from the final hidden rows).

When a stage has run its last chunk it exports what its layers wrote to every rank of the decode group
(``hand_off``): the paged caches of its DSA families - with a decode-context-parallel group of
``n_dcp`` ranks, rank ``d`` gets latent page ``p`` iff ``p % n_dcp == d`` (at page slot ``p // n_dcp`` when
``compact``), the indexer caches whole (``crates/ferrite-kv/src/shard.rs:144-212`` ``ReshardPlan``) - and
the GatedDeltaNet / conv states of its linear layers.  Every rank enters ``hand_off`` as soon as its own part
of the prefill is done and the transfers are ordered stage by stage, so the decode ranks receive stage
``s``'s export while the later stages are still prefilling.  The last stage adds the sequence bookkeeping
(lengths, snapshot cursor, first token, MTP pair).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .pdaf import TransferPlan


def cp_layer_range(n_layers: int, n_stages: int, stage: int) -> Tuple[int, int]:
    """Contiguous, balanced split: the first ``n_layers % n_stages`` stages get one layer more."""
    assert 0 <= stage < n_stages <= n_layers
    base, rem = divmod(n_layers, n_stages)
    l0 = stage * base + min(stage, rem)
    return l0, l0 + base + (1 if stage < rem else 0)


def stage_parts(cfg, l0: int, l1: int) -> Tuple[List[int], List[int]]:
    """(DSA cache families, GatedDeltaNet state indices) written by main layers [l0, l1); the last stage also
    owns the MTP layer's family."""
    fams, gidx = [], []
    layers = list(range(l0, l1))
    if l1 == cfg.num_layers:
        layers += list(range(cfg.num_layers, cfg.num_layers + cfg.num_nextn_predict_layers))
    for i in layers:
        if cfg.is_dsa(i):
            fams.append(cfg.dsa_family(i))
        else:
            gidx.append(cfg.linear_layers.index(i))
    return sorted(set(fams)), gidx


@dataclass
class CpTimes:
    prefill_s: float = 0.0
    export_s: float = 0.0


class CpStage:
    """One rank of the prefill group."""

    def __init__(self, cfg, ecfg, src, stage: int, n_stages: int, ranks: Sequence[int], device, prefill_rows: int = 64,
                 group=None):
        from ..models.glm import GlmDeviceModel
        self.cfg, self.ecfg, self.stage, self.n_stages = cfg, ecfg, stage, n_stages
        self.ranks, self.group = list(ranks), group
        self.l0, self.l1 = cp_layer_range(cfg.num_layers, n_stages, stage)
        self.first, self.last = stage == 0, stage == n_stages - 1
        self.rows = max(prefill_rows, 2)
        self.model = GlmDeviceModel(cfg, ecfg, src, 0, 1, device, None, max_rows=self.rows, n_slots=1,
                                    layer_range=(self.l0, self.l1))
        m, dev = self.model, self.model.dev
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
        self.ids, self.pre_ids, self.judges = i32(self.rows), i32(self.rows), i32(self.rows)
        self.use_mtp = ecfg.mtp_n > 1
        H = cfg.hidden_size
        self.mtp_h = torch.zeros(2, H, device=dev)
        self.mtp_ids = i32(2)
        self.block_ids = i32(max(ecfg.mtp_n, 1))
        self.n_ctx = 0
        self.times = CpTimes()
        self._rs: Dict[int, object] = {}

    def _rows(self, g: int):
        if g not in self._rs:
            self._rs[g] = self.model.make_rows([0], [g])
        return self._rs[g]

    def prefill(self, prompt: List[int]) -> Optional[int]:
        """Run this stage's layers over the prompt, chunk by chunk.  Returns the first generated token on the
        last stage, None elsewhere."""
        m, cfg = self.model, self.cfg
        n, C = len(prompt), self.rows
        assert n >= 2
        m.reset_slot(0)
        toks = torch.tensor(prompt, dtype=torch.int32)
        prev = self.ranks[self.stage - 1] if not self.first else None
        nxt = self.ranks[self.stage + 1] if not self.last else None
        t0 = time.perf_counter()
        for c0 in range(0, n, C):
            c1 = min(n, c0 + C)
            g = c1 - c0
            rs = self._rows(g)
            self.ids[:g].copy_(toks[c0:c1])
            if prev is not None:
                dist.recv(m.ws["R0"][:g], prev, group=self.group)
            final = c1 == n
            m.main_forward(rs, self.ids, snapshots=False, advance=True,
                           judges=self.judges if (final and self.last) else None, head_from=g - 1 if final else g)
            if nxt is not None:
                dist.send(m.ws["R"][:g].contiguous(), nxt, group=self.group)
            elif self.use_mtp:
                hf = m.ws["h_final"]
                t_hi = min(c1, n - 2)
                if t_hi > c0:
                    gm = t_hi - c0
                    self.pre_ids[:gm].copy_(toks[c0 + 1:t_hi + 1])
                    m.mtp_forward(self._rows(gm), self.pre_ids, hf, None, advance=True)
                self.mtp_h[0].copy_(hf[g - 2] if g >= 2 else self.mtp_h[1])
                self.mtp_h[1].copy_(hf[g - 1])
        first = None
        if self.last:
            first = int(self.judges[(n - 1) % C].item())
            self.block_ids[0] = first
            if self.use_mtp:
                self.mtp_ids.copy_(torch.tensor([prompt[-1], first], dtype=torch.int32))
                m.mtp_len[0] = n - 2
        torch.cuda.synchronize(m.dev)
        m.arena.verify(snapshot=False)
        self.times.prefill_s = time.perf_counter() - t0
        self.n_ctx = n
        return first


def _page_lists(plan: TransferPlan, name: str, compact: bool):
    if name != "lat" or plan.n_dcp == 1:
        pages = list(range(plan.n_pages))
        return pages, pages
    return plan.src_pages, (plan.dst_slots if compact else plan.src_pages)


def _caches(model):
    return {"lat": model.lat_cache, "kidx": model.kidx_cache, "kgate": model.kgate_cache, "pool": model.pool_cache}


def _parts(src_model, dst_model, plan: TransferPlan, fams, gidx, compact: bool, slot: int, tp=(0, 1)):
    """Matching (source view builder, destination writer) pairs of one stage -> decode-rank transfer, in a
    fixed order.  Either model may be None (the side that is on another rank).  ``tp = (r, n)``: the destination
    is tensor-parallel rank r of n and takes its heads of the recurrent states (the caches are replicated)."""
    td, tn = tp
    items = []
    dev = (src_model or dst_model).dev
    f_idx = torch.tensor(fams, dtype=torch.long, device=dev)
    for name in ("lat", "kidx", "kgate", "pool"):
        sp, dp = _page_lists(plan, name, compact)
        if not fams or not sp:
            continue
        ref = _caches(src_model or dst_model)[name]
        shape = (len(fams), len(sp)) + tuple(ref.shape[2:])
        s_base = slot * (src_model.max_pages if src_model else 0)
        d_base = slot * (dst_model.max_pages if dst_model else 0)
        if name == "lat" and compact and plan.n_dcp > 1 and dst_model is not None:
            d_base = slot * dst_model.lat_pages_slot      # the decode rank stores its latent pages compactly
        s_ix = torch.tensor([s_base + p for p in sp], dtype=torch.long, device=dev)
        d_ix = torch.tensor([d_base + p for p in dp], dtype=torch.long, device=dev)
        items.append((name, shape, ref.dtype, s_ix, d_ix))
    out = []
    for name, shape, dtype, s_ix, d_ix in items:
        def read(name=name, s_ix=s_ix):
            return _caches(src_model)[name].index_select(0, f_idx).index_select(1, s_ix).contiguous()

        def write(buf, name=name, d_ix=d_ix):
            c = _caches(dst_model)[name]
            for j, f in enumerate(fams):
                c[f].index_copy_(0, d_ix, buf[j])
        out.append((shape, dtype, read, write))
    for nm in ("gdn_state", "conv_state"):
        for gi in gidx:
            if src_model is not None:
                full = getattr(src_model, nm)[gi, slot]          # [nbuf, heads, dk, dv] or [nbuf, 3 P, taps]
                per = full.shape[1] // tn if nm == "gdn_state" else full.shape[1] // (3 * tn)
                shape = (full.shape[0], per if nm == "gdn_state" else 3 * per) + tuple(full.shape[2:])
            else:
                shape = tuple(getattr(dst_model, nm)[gi, slot].shape)
            dtype = getattr(src_model or dst_model, nm).dtype

            def read(nm=nm, gi=gi):
                full = getattr(src_model, nm)[gi, slot]
                if tn == 1:
                    return full.contiguous()
                if nm == "gdn_state":
                    hl = full.shape[1] // tn
                    return full[:, td * hl:(td + 1) * hl].contiguous()
                pf = full.shape[1] // 3                          # q | k | v channel thirds, each split by heads
                pl = pf // tn
                return torch.cat([full[:, j * pf + td * pl:j * pf + (td + 1) * pl] for j in range(3)], 1).contiguous()

            def write(buf, nm=nm, gi=gi):
                getattr(dst_model, nm)[gi, slot].copy_(buf)
            out.append((shape, dtype, read, write))
    return out


def hand_off(stage: Optional[CpStage], engine, n_ctx: int, stage_ranks: Sequence[int], decode_ranks: Sequence[int],
             cfg, rank: int, compact: bool = True, group=None, slot: int = 0, mode: str = "dcp") -> float:
    """Move a prefilled sequence from the prefill group to the decode group.  Every rank of either group calls
    this with the same arguments (``stage``: this rank's CpStage or None, ``engine``: this rank's decode engine
    or None).  Transfers run in one global order (stage by stage, decode rank by decode rank); a rank sends,
    receives, copies locally (it is both ends) or skips each of them.  ``mode``: "dcp" - the decode ranks hold
    whole models and split the latent pages; "tp" - the decode ranks are a tensor-parallel group (every rank gets
    all pages and its own heads of the recurrent states).  Returns this rank's wall time."""
    n_stages = len(stage_ranks)
    n_dcp = len(decode_ranks) if mode == "dcp" else 1
    ps = cfg.dsa.page_size
    t0 = time.perf_counter()
    dev = (stage.model if stage is not None else engine.model).dev
    for s, sr in enumerate(stage_ranks):
        l0, l1 = cp_layer_range(cfg.num_layers, n_stages, s)
        fams, gidx = stage_parts(cfg, l0, l1)
        for d, dr in enumerate(decode_ranks):
            if rank != sr and rank != dr:
                continue
            plan = TransferPlan(n_ctx, ps, n_dcp, d if mode == "dcp" else 0)
            src_m = stage.model if rank == sr else None
            dst_m = engine.model if rank == dr else None
            parts = _parts(src_m, dst_m, plan, fams, gidx, compact, slot,
                           tp=(d, len(decode_ranks)) if mode == "tp" else (0, 1))
            last = s == n_stages - 1
            if rank == sr and rank == dr:
                for _, _, read, write in parts:
                    write(read())
            elif rank == sr:
                bufs = [read() for _, _, read, _ in parts]
                ops = [dist.P2POp(dist.isend, b, dr, group) for b in bufs]
                for r in dist.batch_isend_irecv(ops):
                    r.wait()
            else:
                bufs = [torch.empty(shape, dtype=dtype, device=dev) for shape, dtype, _, _ in parts]
                ops = [dist.P2POp(dist.irecv, b, sr, group) for b in bufs]
                for r in dist.batch_isend_irecv(ops):
                    r.wait()
                for b, (_, _, _, write) in zip(bufs, parts):
                    write(b)
            if last:   # sequence bookkeeping and the speculative step's inputs travel with the last stage
                _vectors(stage if rank == sr else None, engine if rank == dr else None, sr, dr, rank, n_ctx, slot, group, dev)
    torch.cuda.synchronize(dev)
    return time.perf_counter() - t0


def _vectors(stage, engine, sr, dr, rank, n_ctx, slot, group, dev):
    if stage is not None:
        m = stage.model
        head = torch.tensor([n_ctx, int(m.main_len[slot]), int(m.mtp_len[slot]), int(m.cur[slot])], dtype=torch.int64, device=dev)
        vec = [head, stage.block_ids, stage.mtp_ids, stage.mtp_h]
    if engine is not None:
        dst = [torch.zeros(4, dtype=torch.int64, device=dev), engine.block_ids, engine.mtp_ids, engine.mtp_h]
    if stage is not None and engine is not None:
        for a, b in zip(dst, vec):
            a[:b.numel()].copy_(b) if a.dim() == 1 else a.copy_(b)
    elif stage is not None:
        for r in dist.batch_isend_irecv([dist.P2POp(dist.isend, v.contiguous(), dr, group) for v in vec]):
            r.wait()
    else:
        tmp = [dst[0], torch.zeros_like(engine.block_ids), dst[2], dst[3]]
        for r in dist.batch_isend_irecv([dist.P2POp(dist.irecv, v, sr, group) for v in tmp]):
            r.wait()
        engine.block_ids.copy_(tmp[1])
    if engine is not None:
        n_ctx_r, main_len, mtp_len, cur = (int(v) for v in dst[0].tolist())
        em = engine.model
        em.main_len[slot] = main_len
        em.mtp_len[slot] = mtp_len
        em.cur[slot] = cur
        engine.n_ctx = n_ctx_r
