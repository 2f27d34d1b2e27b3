"""Batched GLM serving engine: the C++ tick planner driving the device model.

A tick replays the planner's decisions: row compaction moves, prefix-cache restores, tiered
snapshot moves, chunked-prefill passes and ONE decode graph for the padded bucket.  Decode
rows are physical: row r = state slot r = graph row r, so batch membership changes only
touch device tables (sequence lengths, page table, token ids, state rows) and never force a
re-capture; there is one CUDA graph per bucket of the ladder.  Counterpart of
``GpuEngine::tick`` (``crates/ferrite-serve/src/gpu_engine.rs:858-1117``) and
``decode_step_batched`` (``crates/ferrite-exec/src/tp.rs:914-1288``).

With ``EngineConfig.mtp_n = nv > 1`` the decode graph of a bucket is a batched speculative step
(``mtp_step_batched``, ``crates/ferrite-exec/src/tp.rs:1327``; layout ``mtp_batch.rs:146-530``):
every live sequence is one GROUP of the row-batched kernels.  Draft pass 0 runs two rows per
sequence on the MTP layer (the pair to repair and the new anchor), passes 1..nv-2 one row each,
the main model verifies nv rows per sequence with GatedDeltaNet state snapshots into the
rotating buffers, and ONE accept kernel walks every sequence's accept chain on the device,
advances its lengths and snapshot cursor (commit without copying state) and stages its next
draft inputs.  Per-sequence draft inputs live per state slot between ticks and are gathered
into / scattered from the bucket's rows around the graph.  After a prefix-cache restore the MTP
layer's cache entry of the last shared position was written by the sequence that published the
block (it pairs that position's hidden state with ITS next token); it is left as it is: drafts
only propose, the main model's verify decides every emitted token.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import build
from ..config import EngineConfig, GlmConfig
from ..models.glm import GlmDeviceModel, RowSet
from ..serve.engine import ContextOverflow, ReqEvent, RequestSpec, Usage
from . import mtp_batch as MB


class GpuEngine:
    def __init__(self, cfg: GlmConfig, ecfg: EngineConfig, src, rank: int = 0, world: int = 1, device="cuda",
                 allreduce=None, max_rows: int = 8, prefill_rows: int = 64, num_pages: Optional[int] = None,
                 device_snapshots: int = 8, host_snapshots: int = 32, prefill_budget: Optional[int] = None):
        build.build_runtime()
        from .. import _runtime as rt
        self.rt, self.cfg = rt, cfg
        self.nv = nv = max(1, ecfg.mtp_n)
        ps = cfg.dsa.page_size
        max_pages_seq = (ecfg.max_ctx + ps - 1) // ps
        num_pages = num_pages or (max_rows * max_pages_seq + 1)
        self.model = GlmDeviceModel(cfg, ecfg, src, rank, world, device, allreduce,
                                    max_rows=max(prefill_rows, MB.verify_rows(max_rows, max(nv, 2))), n_slots=max_rows + 1,
                                    num_pages=num_pages)
        m, dev = self.model, self.model.dev
        sc = rt.SchedConfig()
        sc.max_rows, sc.page_size, sc.num_pages = max_rows, ps, num_pages
        sc.prefill_budget = prefill_budget or ecfg.sched.prefill_budget
        sc.device_slots, sc.host_slots, sc.disk_slots = device_snapshots, host_snapshots, 0
        sc.max_ctx = ecfg.max_ctx
        sc.spec_rows = nv
        sc.buckets = [b for b in ecfg.sched.buckets if b <= max_rows] or [max_rows]
        if sc.buckets[-1] < max_rows:
            sc.buckets = sc.buckets + [max_rows]
        self.buckets = list(sc.buckets)
        self.sched = rt.BatchScheduler(sc)
        assert self.sched.reserve_pages(1) == [0]  # page 0 is the scratch page of inert rows
        self.dummy_slot = max_rows                   # padding rows of a bucket run on this slot
        self.max_rows, self.prefill_rows = max_rows, prefill_rows
        self.ids = torch.zeros(max_rows, dtype=torch.int32, device=dev)       # input token per graph row
        self.out = torch.zeros(max_rows, dtype=torch.int32, device=dev)       # greedy token per graph row
        self.tok_slot = torch.zeros(max_rows + 1, dtype=torch.int32, device=dev)  # next input token per slot
        self.prefill_ids = torch.zeros(prefill_rows, dtype=torch.int32, device=dev)
        self.first_tok = torch.zeros(prefill_rows, dtype=torch.int32, device=dev)
        self.pin_out = torch.zeros(max_rows, dtype=torch.int32).pin_memory()
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.rowsets: Dict[int, RowSet] = {b: m.make_rows(list(range(b)), [1] * b) for b in self.buckets}
        if nv > 1:
            H, S = cfg.hidden_size, max_rows + 1
            i32 = lambda *sh: torch.zeros(*sh, dtype=torch.int32, device=dev)
            self.rs2 = {b: m.make_rows(list(range(b)), [2] * b) for b in self.buckets}
            self.rsv = {b: m.make_rows(list(range(b)), [nv] * b) for b in self.buckets}
            self.mtp_ids_slot, self.mtp_h_slot = i32(S, 2), torch.zeros(S, 2, H, device=dev)   # between ticks
            self.block_ids, self.judges = i32(max_rows, nv), i32(max_rows, nv)
            self.out_tokens = i32(max_rows, nv + 1)
            self.mtp_ids, self.mtp_h = i32(max_rows, 2), torch.zeros(max_rows, 2, H, device=dev)
            self.hchain, self.cur_ids, self.draft_ids = torch.zeros(max_rows, H, device=dev), i32(max_rows), i32(2 * max_rows)
            self.mtp_pre_ids = i32(prefill_rows)
            self.pin_spec = torch.zeros(max_rows, nv + 1, dtype=torch.int32).pin_memory()
        self.prompts: Dict[int, List[int]] = {}
        self.page_count: Dict[int, int] = {}
        # tiered recurrent-state snapshots: device tier on the GPU, host tier in pinned memory
        gs, cs = m.gdn_state[:, 0, 0], m.conv_state[:, 0, 0]
        self.snap_dev = (torch.zeros(device_snapshots, *gs.shape, device=dev), torch.zeros(device_snapshots, *cs.shape, device=dev))
        self.snap_host = (torch.zeros(host_snapshots, *gs.shape).pin_memory(), torch.zeros(host_snapshots, *cs.shape).pin_memory())
        self.launches = 0
        from ..parallel.collective import startup_barrier
        startup_barrier(world, getattr(allreduce, "group", None))

    # ------------------------------------------------------------------ ServeEngine
    def validate(self, spec: RequestSpec) -> None:
        if not spec.prompt_ids or len(spec.prompt_ids) > self.sched.max_prompt():
            raise ContextOverflow(f"prompt of {len(spec.prompt_ids)} tokens does not fit the context limit "
                                  f"(at most {self.sched.max_prompt()})")

    def submit(self, spec: RequestSpec) -> int:
        self.validate(spec)
        prompt = list(spec.prompt_ids)
        if self.nv > 1 and len(prompt) == 1:
            prompt = prompt * 2          # the draft layer pairs every position with its successor: two tokens at least
        rid = self.sched.submit(prompt, spec.max_new_tokens, list(spec.stop_ids))
        self.prompts[rid] = prompt
        return rid

    def cancel(self, req: int) -> None:
        self.sched.cancel(req)
        self.prompts.pop(req, None)

    def idle(self) -> bool:
        return self.sched.idle()

    def stats(self) -> dict:
        s = self.sched.stats()
        r = s.radix
        return {"engine": {"ticks": s.ticks, "tokens_committed": s.tokens_committed, "live_rows": s.live_rows,
                           "queued": s.queued},
                "radix": {"tree_nodes": r.tree_nodes, "tree_blocks": r.tree_blocks,
                          "evictable_tokens": r.evictable_tokens, "protected_tokens": r.protected_tokens,
                          "hits": r.hits, "misses": r.misses},
                "hicache": {"tiers": dict(zip(("device", "host", "disk"), s.tiers)),
                            "pages_in_use": s.pages_in_use, "pages_free": s.pages_free}}

    # ------------------------------------------------------------------ state plumbing
    def _tier_bufs(self, tier: int):
        return self.snap_dev if tier == self.rt.TIER_DEVICE else self.snap_host

    def _apply_state_moves(self, moves):
        rt, m = self.rt, self.model
        for mv in moves:
            if mv.to_tier == rt.TIER_NONE:
                continue  # dropped: nothing to copy
            dst = self._tier_bufs(mv.to_tier)
            if mv.from_tier == rt.TIER_NONE:  # capture from live row (nbuf == 1: buffer 0)
                dst[0][mv.to_slot].copy_(m.gdn_state[:, mv.from_slot, 0], non_blocking=True)
                dst[1][mv.to_slot].copy_(m.conv_state[:, mv.from_slot, 0], non_blocking=True)
            else:
                src = self._tier_bufs(mv.from_tier)
                dst[0][mv.to_slot].copy_(src[0][mv.from_slot], non_blocking=True)
                dst[1][mv.to_slot].copy_(src[1][mv.from_slot], non_blocking=True)
        if moves:
            torch.cuda.current_stream().synchronize()  # host-tier copies must land before slots are reused

    def _move_row(self, src: int, dst: int):
        m = self.model
        m.gdn_state[:, dst].copy_(m.gdn_state[:, src])
        m.conv_state[:, dst].copy_(m.conv_state[:, src])
        for t in (m.main_len, m.mtp_len, m.cur, self.tok_slot):
            t[dst] = t[src]
        if self.nv > 1:
            self.mtp_ids_slot[dst].copy_(self.mtp_ids_slot[src])
            self.mtp_h_slot[dst].copy_(self.mtp_h_slot[src])
        m.page_table[dst].copy_(m.page_table[src])
        m.main_len[src] = 0
        m.page_table[src].zero_()

    def _bind_pages(self, row: int, rid: int):
        req = self.sched.get(rid)
        pages = list(req.pages)
        if self.page_count.get(rid) != len(pages):
            t = torch.zeros(self.model.max_pages, dtype=torch.int32)
            t[:len(pages)] = torch.tensor(pages, dtype=torch.int32)
            self.model.page_table[row].copy_(t)
            self.page_count[rid] = len(pages)

    # ------------------------------------------------------------------ tick
    def _decode_body(self, bucket: int):
        if self.nv > 1:
            return self._spec_body(bucket)
        self.model.main_forward(self.rowsets[bucket], self.ids, snapshots=False, advance=True, judges=self.out)

    def _spec_body(self, G: int):
        """One speculative step of G sequences (groups): draft chain, verify, device accept / commit."""
        m, nv, H = self.model, self.nv, self.cfg.hidden_size
        blk = self.block_ids[:G]
        # draft 0: rows (pair to repair, new anchor) of every sequence; the anchor rows' tokens are draft 1
        m.mtp_forward(self.rs2[G], self.mtp_ids, self.mtp_h, self.draft_ids, head_from=0, advance=True)
        blk[:, 1].copy_(self.draft_ids[:2 * G].view(G, 2)[:, 1])
        hout = m.ws["mtp_hout"]
        for d in range(1, nv - 1):
            self.hchain[:G].copy_(hout[:2 * G].view(G, 2, H)[:, 1] if d == 1 else hout[:G])
            self.cur_ids[:G].copy_(blk[:, d])
            m.mtp_forward(self.rowsets[G], self.cur_ids, self.hchain, self.draft_ids, advance=True)
            blk[:, d + 1].copy_(self.draft_ids[:G])
        rsv = self.rsv[G]
        m.main_forward(rsv, self.block_ids, snapshots=True, advance=False, judges=self.judges)
        m.K.call("fb_mtp_accept", self.block_ids, self.judges, self.out_tokens, m.ws["h_final"], self.mtp_ids, self.mtp_h,
                 rsv.group_slot, m.main_len, m.mtp_len, m.cur, G, nv, H, m.nbuf)

    def _decode(self, bucket: int):
        g = self.graphs.get(bucket)
        if g is None and self.model.ecfg.use_graphs:
            # first use: run once eagerly on a saved copy of the small state, then capture
            m = self.model
            small = (m.main_len, m.mtp_len, m.cur, m.gdn_state, m.conv_state)
            if self.nv > 1:
                small = small + (self.block_ids, self.mtp_ids, self.mtp_h)
            keep = [t.clone() for t in small]
            self._decode_body(bucket)
            for dst, src in zip(small, keep):
                dst.copy_(src)
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
        rt, m = self.rt, self.model
        out: List[Tuple[int, ReqEvent]] = []
        plan = self.sched.plan()
        for mv in plan.row_moves:
            self._move_row(mv.from_row, mv.to_row)
        self._apply_state_moves(plan.state_moves)
        for rs in plan.restores:
            req = self.sched.get([r for r in plan.admitted if self.sched.get(r).row == rs.row][0])
            m.gdn_state[:, rs.row, 0].copy_(self.snap_dev[0][rs.device_slot])
            m.conv_state[:, rs.row, 0].copy_(self.snap_dev[1][rs.device_slot])
            m.main_len[rs.row] = req.cached_tokens
            m.mtp_len[rs.row] = req.cached_tokens
            m.cur[rs.row] = 0
        for rid in plan.admitted:
            req = self.sched.get(rid)
            if req.cached_tokens == 0:
                m.gdn_state[:, req.row].zero_()
                m.conv_state[:, req.row].zero_()
                m.main_len[req.row] = 0
                m.mtp_len[req.row] = 0
                m.cur[req.row] = 0
            if self.nv > 1:
                self.mtp_h_slot[req.row].zero_()
            self.page_count.pop(rid, None)
            self._bind_pages(req.row, rid)
        # decode first: rows of sequences that were already decoding before this tick
        if plan.decode.n_live:
            live = [row for row, r in enumerate(plan.decode.rows) if r >= 0]
            bucket = rt.bucket_for(self.buckets, len(live))
            slots = live + [self.dummy_slot] * (bucket - len(live))
            slot_t = torch.tensor(slots, dtype=torch.int32)
            rs = self.rowsets[bucket]
            rs.row_slot.copy_(slot_t)
            rs.group_slot.copy_(slot_t)
            m.main_len[self.dummy_slot] = 0
            idx = rs.row_slot.long()
            toks = [[] for _ in plan.decode.rows]
            if self.nv > 1:
                for rsx, g in ((self.rs2[bucket], 2), (self.rsv[bucket], self.nv)):
                    rsx.row_slot.copy_(slot_t.repeat_interleave(g))
                    rsx.group_slot.copy_(slot_t)
                m.mtp_len[self.dummy_slot] = 0
                m.cur[self.dummy_slot] = 0
                self.block_ids[:bucket, 0].copy_(self.tok_slot[idx])
                self.mtp_ids[:bucket].copy_(self.mtp_ids_slot[idx])
                self.mtp_h[:bucket].copy_(self.mtp_h_slot[idx])
                self._decode(bucket)
                self.tok_slot[idx] = self.block_ids[:bucket, 0]
                self.mtp_ids_slot[idx] = self.mtp_ids[:bucket]
                self.mtp_h_slot[idx] = self.mtp_h[:bucket]
                self.pin_spec.copy_(self.out_tokens, non_blocking=True)
            else:
                self.ids[:bucket].copy_(self.tok_slot[idx])
                self._decode(bucket)
                self.tok_slot[idx] = self.out[:bucket]
                self.pin_out.copy_(self.out, non_blocking=True)
            m.arena.snapshot_async()
            torch.cuda.current_stream().synchronize()
            m.arena.verify()   # status words and guards of the tick: a timed-out wait or a clamped position raises here
            rmap = MB.SeqRowMap(len(live), bucket, self.nv)     # sequence i of the bucket owns verify rows rmap.rows_of(i)
            for i, row in enumerate(live):
                if self.nv > 1:
                    k = int(self.pin_spec[i, 0])
                    assert 1 <= k <= rmap.width, (i, k)
                    toks[row] = [int(t) for t in self.pin_spec[i, 1:1 + k]]
                else:
                    toks[row] = [int(self.pin_out[i])]
            self._convert(self.sched.ingest_decode(toks), out)
        # chunked prefill
        for ch in plan.prefill:
            prompt = self.prompts[ch.req]
            first = -1
            for s0 in range(ch.start, ch.start + ch.len, self.prefill_rows):
                n = min(self.prefill_rows, ch.start + ch.len - s0)
                self.prefill_ids[:n].copy_(torch.tensor(prompt[s0:s0 + n], dtype=torch.int32))
                last = ch.last and s0 + n == ch.start + ch.len
                rs = m.make_rows([ch.row], [n])
                m.main_forward(rs, self.prefill_ids, snapshots=False, advance=True,
                               judges=self.first_tok if last else None, head_from=n - 1 if last else n)
                if self.nv > 1:
                    # the draft layer's cache: pairs (h_t, tok_{t+1}) for t < N - 2; the last two hidden rows of the
                    # prompt stay with the slot as the first draft pass's inputs
                    N, hf = len(prompt), m.ws["h_final"]
                    t_hi = min(s0 + n, N - 2)
                    if t_hi > s0:
                        gm = t_hi - s0
                        self.mtp_pre_ids[:gm].copy_(torch.tensor(prompt[s0 + 1:t_hi + 1], dtype=torch.int32))
                        m.mtp_forward(m.make_rows([ch.row], [gm]), self.mtp_pre_ids, hf, None, advance=True)
                    hs = self.mtp_h_slot[ch.row]
                    hs[0].copy_(hf[n - 2] if n >= 2 else hs[1])
                    hs[1].copy_(hf[n - 1])
                if last:
                    first = int(self.first_tok[n - 1].item())
                    m.arena.verify(snapshot=False)
                    self.tok_slot[ch.row] = first
                    if self.nv > 1:
                        self.mtp_ids_slot[ch.row].copy_(torch.tensor([prompt[-1], first], dtype=torch.int32))
                        m.mtp_len[ch.row] = len(prompt) - 2
            evs, moves = self.sched.ingest_prefill(ch.req, ch.len, first, ch.snapshot_after)
            self._apply_state_moves(moves)
            self._convert(evs, out)
        return out

    def _convert(self, evs, out):
        rt = self.rt
        for e in evs:
            if e.kind == rt.EV_ADMITTED:
                out.append((e.req, ReqEvent("admitted", prefix_hit=e.prefix_hit, prompt_tokens=e.prompt_tokens)))
            elif e.kind == rt.EV_TOKENS:
                out.append((e.req, ReqEvent("tokens", ids=list(e.tokens))))
            else:
                out.append((e.req, ReqEvent("finished", reason=e.reason,
                                            usage=Usage(e.prompt_tokens, e.completion_tokens, e.cached_tokens))))
                self.prompts.pop(e.req, None)
                self.page_count.pop(e.req, None)
                self.sched.forget(e.req)

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
