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

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..models.dsv41 import Dsv41DeviceModel
from ..models.dsv41_config import Dsv41Config
from ..serve.engine import ContextOverflow, ReqEvent, RequestSpec, Usage


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
        # the planner is native (csrc/runtime/slot_scheduler.h): admission, prefill chunks, decode rows, finish rules
        from .. import build
        build.build_runtime()
        from .. import _runtime as rt
        self.rt = rt
        sc = rt.SlotSchedConfig()
        sc.max_seqs, sc.prefill_rows, sc.prefill_budget, sc.max_ctx = max_seqs, prefill_rows, self.prefill_budget, m.max_ctx
        sc.buckets = [int(b) for b in buckets]
        self.sched = rt.SlotScheduler(sc)
        self.buckets = list(self.sched.buckets())
        self.dummy_slot = max_seqs                                    # padding rows of a bucket run on this slot
        self.rowsets = {b: m.make_rows(list(range(b)), [1] * b) for b in self.buckets}
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.ids = torch.zeros(max_seqs, dtype=torch.int32, device=dev)          # input token of every graph row
        self.tok_slot = torch.zeros(max_seqs + 1, dtype=torch.int32, device=dev)  # next input token of every slot
        self.pin_out = torch.zeros(max_seqs, dtype=torch.int32)
        if self.on_gpu:
            self.pin_out = self.pin_out.pin_memory()
        self.prompts: Dict[int, List[int]] = {}                        # token ids of the live and waiting requests
        self.launches = 0
        if model is None:
            from ..parallel.collective import startup_barrier
            startup_barrier(world, getattr(allreduce, "group", None))

    # ------------------------------------------------------------------ ServeEngine
    def max_prompt(self) -> int:
        return self.sched.max_prompt()

    def validate(self, spec: RequestSpec) -> None:
        if not spec.prompt_ids or len(spec.prompt_ids) > self.max_prompt():
            raise ContextOverflow(f"prompt of {len(spec.prompt_ids)} tokens does not fit the context limit "
                                  f"(at most {self.max_prompt()})")

    def submit(self, spec: RequestSpec) -> int:
        self.validate(spec)
        prompt = [int(t) for t in spec.prompt_ids]
        rid = self.sched.submit(prompt, int(spec.max_new_tokens), [int(t) for t in spec.stop_ids])
        assert rid > 0
        self.prompts[rid] = prompt
        return rid

    def cancel(self, req: int) -> None:
        self.sched.cancel(req)

    def idle(self) -> bool:
        return self.sched.idle()

    @property
    def free(self) -> List[int]:
        return list(self.sched.free_slots())

    def n_decoding(self) -> int:
        """Sequences whose prompt is in the caches (the rows of the next decode tick)."""
        return len(self.sched.plan_decode().slots)

    def stats(self) -> dict:
        st = self.sched.stats()
        # the shape of the GLM engines' stats (this engine keeps no prefix cache and no tiered snapshots)
        return {"engine": {"ticks": st.ticks, "tokens_committed": st.tokens_committed, "live_rows": st.live,
                           "queued": st.queued, "free_slots": st.free_slots},
                "radix": {"tree_nodes": 0, "tree_blocks": 0, "evictable_tokens": 0, "protected_tokens": 0,
                          "hits": 0, "misses": 0},
                "hicache": {"tiers": {"device": 0, "host": 0, "disk": 0}, "pages_in_use": st.live,
                            "pages_free": st.free_slots}}

    # ------------------------------------------------------------------ one tick
    def _convert(self, res, out: List[Tuple[int, ReqEvent]]):
        """(events, released slots) of a planner call -> ReqEvents; released slots get their lengths cleared."""
        evs, released = res
        rt = self.rt
        for e in evs:
            if e.kind == rt.SLOT_EV_ADMITTED:
                out.append((e.req, ReqEvent("admitted", prefix_hit=False, prompt_tokens=e.prompt_tokens)))
            elif e.kind == rt.SLOT_EV_TOKEN:
                out.append((e.req, ReqEvent("tokens", ids=[e.token])))
            else:
                out.append((e.req, ReqEvent("finished", reason=e.reason,
                                            usage=Usage(e.prompt_tokens, e.completion_tokens, 0))))
                self.prompts.pop(e.req, None)
        for slot in released:
            self.model.reset_slot(slot)

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
        self._convert(self.sched.begin_tick(), out)      # cancellations: waiting requests are dropped, live ones free their slot
        # decode: every sequence whose prompt is in the caches advances by one token
        dp = self.sched.plan_decode()
        if dp.bucket:
            bucket, live = dp.bucket, len(dp.slots)
            slots = list(dp.slots) + [self.dummy_slot] * (bucket - live)
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
            self._convert(self.sched.ingest_decode([int(t) for t in self.pin_out[:live]]), out)
        # admission, then chunked prefill within the tick's token budget (oldest admitted first)
        pp = self.sched.plan_prefill()
        for slot in pp.reset_slots:
            m.reset_slot(slot)
        self._convert((pp.events, []), out)
        for ch in pp.chunks:
            prompt = self.prompts[ch.req]
            ids = torch.tensor(prompt[ch.start:ch.start + ch.len], dtype=torch.int32, device=self.dev)
            m.forward(m.make_rows([ch.slot], [ch.len]), ids, advance=True, want_logits=ch.last)
            if ch.last:
                first = int(m.ws["out_ids"][ch.len - 1].item())
                m.arena.verify(snapshot=False)
                self.tok_slot[ch.slot] = first
                self._convert(self.sched.ingest_first(ch.req, first), out)
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
