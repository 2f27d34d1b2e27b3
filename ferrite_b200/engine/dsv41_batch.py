"""Batched DSV41 serving engine: continuous batching of greedy decode, one row per live sequence.

Every live sequence owns a state slot of the device model (window ring, compressed rows, indexer keys, compressor
ring and engram history are all indexed by slot and position), so a decode tick is ONE row-batched forward over the
live slots, replayed as a CUDA graph per bucket of the ladder: batch membership only changes the device tables of
the bucket's row set (slot of every row), never the graph.  Prompts are admitted FIFO into free slots and prefilled
in chunks of ``prefill_rows`` rows between decode ticks, at most ``prefill_budget`` prompt tokens per tick, so a
long prompt does not stall the sequences that are already decoding.  Routed experts of a decode tick with 32 rows or
more run as the block-scaled tcgen05 grouped GEMMs (every expert's weights stream once per tick, however many rows
routed to it); below that the per-pair tensor-core kernels run (16 rows x 6 picks of 384 experts are nearly all
distinct experts: grouping them buys no reuse).

Counterpart of the reference's batched DSV41 arm (``scripts/batched_400_v2.sh``; serving seam
``crates/ferrite-dsv41/src/serve.rs``) behind the same ``ServeEngine`` protocol as the GLM batched engine
(``engine/gpu_engine.py``).  Speculative decoding stays with the single-sequence engine
(``engine/dsv41_engine.py``); a finished sequence frees its slot by a length reset, nothing is copied.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import torch

from ..models.dsv41 import Dsv41DeviceModel
from ..models.dsv41_config import Dsv41Config
from ..serve.engine import ContextOverflow, ReqEvent, RequestSpec, Usage


@dataclass
class _Seq:
    rid: int
    prompt: List[int]
    max_new: int
    stop: Tuple[int, ...]
    slot: int = -1
    filled: int = 0                 # prompt tokens already in the caches
    out: List[int] = field(default_factory=list)

    @property
    def decoding(self) -> bool:
        return self.slot >= 0 and self.filled == len(self.prompt)


def bucket_for(buckets: Sequence[int], n: int) -> int:
    for b in buckets:
        if b >= n:
            return b
    raise ValueError(f"{n} rows exceed the largest bucket {buckets[-1]}")


class Dsv41BatchEngine:
    def __init__(self, cfg: Dsv41Config, src, rank: int = 0, world: int = 1, device="cuda", allreduce=None,
                 max_ctx: int = 1024, max_seqs: int = 8, prefill_rows: int = 64, prefill_budget: int = 256,
                 buckets: Sequence[int] = (1, 2, 4, 8, 16, 32, 64), use_graphs: bool = True, model=None):
        self.cfg = cfg
        self.max_seqs, self.prefill_rows, self.prefill_budget = max_seqs, prefill_rows, max(prefill_budget, 1)
        # `model`: a ready device model (tests drive the scheduling with a host stand-in of the same interface)
        self.model = m = model if model is not None else Dsv41DeviceModel(
            cfg, src, rank, world, device, allreduce, max_rows=max(prefill_rows, max_seqs), max_ctx=max_ctx,
            n_slots=max_seqs + 1)
        self.dev = dev = m.dev
        self.on_gpu = dev.type == "cuda"
        self.use_graphs = use_graphs and self.on_gpu
        self.buckets = [b for b in buckets if b < max_seqs] + [max_seqs]
        self.dummy_slot = max_seqs                                    # padding rows of a bucket run on this slot
        self.rowsets = {b: m.make_rows(list(range(b)), [1] * b) for b in self.buckets}
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.ids = torch.zeros(max_seqs, dtype=torch.int32, device=dev)          # input token of every graph row
        self.tok_slot = torch.zeros(max_seqs + 1, dtype=torch.int32, device=dev)  # next input token of every slot
        self.pin_out = torch.zeros(max_seqs, dtype=torch.int32)
        if self.on_gpu:
            self.pin_out = self.pin_out.pin_memory()
        self.free: List[int] = list(range(max_seqs - 1, -1, -1))
        self.waiting: Deque[_Seq] = deque()
        self.live: Dict[int, _Seq] = {}                                # by request id, admission order
        self.cancelled: set = set()
        self.next_id = 1
        self.ticks = self.tokens = 0
        self.launches = 0
        if model is None:
            from ..parallel.collective import startup_barrier
            startup_barrier(world, getattr(allreduce, "group", None))

    # ------------------------------------------------------------------ ServeEngine
    def max_prompt(self) -> int:
        return self.model.max_ctx - 4

    def validate(self, spec: RequestSpec) -> None:
        if not spec.prompt_ids or len(spec.prompt_ids) > self.max_prompt():
            raise ContextOverflow(f"prompt of {len(spec.prompt_ids)} tokens does not fit the context limit "
                                  f"(at most {self.max_prompt()})")

    def submit(self, spec: RequestSpec) -> int:
        self.validate(spec)
        rid, self.next_id = self.next_id, self.next_id + 1
        self.waiting.append(_Seq(rid, list(spec.prompt_ids), max(1, spec.max_new_tokens), tuple(spec.stop_ids)))
        return rid

    def cancel(self, req: int) -> None:
        self.cancelled.add(req)

    def idle(self) -> bool:
        return not self.waiting and not self.live

    def stats(self) -> dict:
        # the shape of the GLM engines' stats (this engine keeps no prefix cache and no tiered snapshots)
        return {"engine": {"ticks": self.ticks, "tokens_committed": self.tokens, "live_rows": len(self.live),
                           "queued": len(self.waiting), "free_slots": len(self.free)},
                "radix": {"tree_nodes": 0, "tree_blocks": 0, "evictable_tokens": 0, "protected_tokens": 0,
                          "hits": 0, "misses": 0},
                "hicache": {"tiers": {"device": 0, "host": 0, "disk": 0}, "pages_in_use": len(self.live),
                            "pages_free": len(self.free)}}

    # ------------------------------------------------------------------ one tick
    def _finish(self, s: _Seq, reason: str, out: List[Tuple[int, ReqEvent]]):
        out.append((s.rid, ReqEvent("finished", reason=reason, usage=Usage(len(s.prompt), len(s.out), 0))))
        if s.slot >= 0:
            self.model.reset_slot(s.slot)
            self.free.append(s.slot)
        self.live.pop(s.rid, None)

    def _emit(self, s: _Seq, tok: int, out: List[Tuple[int, ReqEvent]]):
        """Commit one token of a sequence; ends the sequence at a stop id, its budget or the context limit."""
        self.tokens += 1
        if tok in s.stop:
            self._finish(s, "stop", out)
            return
        s.out.append(tok)
        out.append((s.rid, ReqEvent("tokens", ids=[tok])))
        if len(s.out) >= s.max_new:
            self._finish(s, "length", out)
        elif len(s.prompt) + len(s.out) + 2 >= self.model.max_ctx:
            self._finish(s, "context", out)

    def _decode_body(self, bucket: int):
        m = self.model
        m.forward(self.rowsets[bucket], self.ids, advance=True)
        self.ids[:bucket].copy_(m.ws["out_ids"][:bucket])

    def _decode(self, bucket: int):
        g = self.graphs.get(bucket)
        if g is None and self.use_graphs:
            m = self.model
            keep_len, keep_ids = m.seq_len.clone(), self.ids.clone()
            self._decode_body(bucket)              # warm-up on saved lengths: the caches it writes are rewritten below
            m.seq_len.copy_(keep_len)
            self.ids.copy_(keep_ids)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            l0 = m.K.launches
            with torch.cuda.graph(g):
                self._decode_body(bucket)
            self.launches = m.K.launches - l0
            self.graphs[bucket] = g
        if g is not None:
            g.replay()
        else:
            self._decode_body(bucket)

    def tick(self) -> List[Tuple[int, ReqEvent]]:
        m = self.model
        out: List[Tuple[int, ReqEvent]] = []
        self.ticks += 1
        # cancellations: waiting requests are dropped, live ones free their slot
        if self.cancelled:
            self.waiting = deque(s for s in self.waiting if s.rid not in self.cancelled)
            for s in [s for s in self.live.values() if s.rid in self.cancelled]:
                self._finish(s, "cancelled", out)
            self.cancelled.clear()
        # decode: every sequence whose prompt is in the caches advances by one token
        dec = [s for s in self.live.values() if s.decoding]
        if dec:
            bucket = bucket_for(self.buckets, len(dec))
            slots = [s.slot for s in dec] + [self.dummy_slot] * (bucket - len(dec))
            slot_t = torch.tensor(slots, dtype=torch.int32)
            rs = self.rowsets[bucket]
            rs.row_slot.copy_(slot_t)
            rs.group_slot.copy_(slot_t)
            m.reset_slot(self.dummy_slot)
            idx = rs.row_slot.long()
            self.ids[:bucket].copy_(self.tok_slot[idx])
            self._decode(bucket)
            self.tok_slot[idx] = self.ids[:bucket]
            self.pin_out.copy_(self.ids, non_blocking=True)
            m.arena.snapshot_async()
            if self.on_gpu:
                torch.cuda.current_stream().synchronize()
            m.arena.verify()
            for i, s in enumerate(dec):
                self._emit(s, int(self.pin_out[i]), out)
        # admission, then chunked prefill within the tick's token budget (oldest admitted first)
        while self.waiting and self.free:
            s = self.waiting.popleft()
            s.slot = self.free.pop()
            m.reset_slot(s.slot)
            self.live[s.rid] = s
            out.append((s.rid, ReqEvent("admitted", prefix_hit=False, prompt_tokens=len(s.prompt))))
        budget = self.prefill_budget
        for s in [s for s in self.live.values() if not s.decoding]:
            while budget > 0 and s.filled < len(s.prompt):
                n = min(self.prefill_rows, len(s.prompt) - s.filled, budget)
                ids = torch.tensor(s.prompt[s.filled:s.filled + n], dtype=torch.int32, device=self.dev)
                last = s.filled + n == len(s.prompt)
                m.forward(m.make_rows([s.slot], [n]), ids, advance=True, want_logits=last)
                s.filled += n
                budget -= n
                if last:
                    first = int(m.ws["out_ids"][n - 1].item())
                    m.arena.verify(snapshot=False)
                    self.tok_slot[s.slot] = first
                    self._emit(s, first, out)
            if budget <= 0:
                break
        return out

    def run_all(self, specs: List[RequestSpec], max_ticks: int = 100000) -> Dict[int, List[int]]:
        """Convenience for tests and benches: submit everything, tick until idle."""
        ids = [self.submit(s) for s in specs]
        toks: Dict[int, List[int]] = {i: [] for i in ids}
        self.usage: Dict[int, Usage] = {}
        for _ in range(max_ticks):
            for rid, ev in self.tick():
                if ev.kind == "tokens":
                    toks[rid].extend(ev.ids)
                elif ev.kind == "finished":
                    self.usage[rid] = ev.usage
            if self.idle():
                break
        return toks
