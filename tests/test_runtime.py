"""CPU: the C++ host runtime -- golden ops against the PyTorch fp32 statements, the page /
slot pools, reshard plan, radix prefix cache, tiered state store and the tick planner."""
import numpy as np
import pytest
import torch

from ferrite_b200 import build

build.build_runtime()
from ferrite_b200 import _runtime as rt  # noqa: E402
from ferrite_b200.ops import reference as R  # noqa: E402

G = rt.golden


def t(a):
    return torch.from_numpy(np.asarray(a))


def rnd(*s, seed=0):
    return torch.randn(*s, generator=torch.Generator().manual_seed(seed))


def test_golden_ops_match_torch_reference():
    x, w = rnd(5, 24, seed=1), rnd(7, 24, seed=2)
    assert torch.allclose(t(G.matmul(x.numpy(), w.numpy())), R.linear(x, w), atol=1e-5)
    nw = rnd(24, seed=3)
    assert torch.allclose(t(G.rmsnorm(x.numpy(), nw.numpy(), 1e-5)), R.rmsnorm(x, nw, 1e-5), atol=1e-5)
    g = rnd(5, 24, seed=4)
    assert torch.allclose(t(G.gated_rmsnorm(x.numpy(), g.numpy(), nw.numpy(), 1e-5)), R.gated_rmsnorm(x, g, nw, 1e-5), atol=1e-5)
    assert torch.allclose(t(G.swiglu_limited((x * 9).numpy(), (g * 9).numpy(), 10.0)), R.swiglu_limited(x * 9, g * 9, 10.0), atol=1e-5)
    cw, cs = rnd(24, 4, seed=5), rnd(24, 3, seed=6)
    o1, s1 = G.causal_conv1d(x.numpy(), cw.numpy(), cs.numpy())
    o2, s2 = R.causal_conv1d(x, cw, cs)
    assert torch.allclose(t(o1), o2, atol=1e-5) and torch.allclose(t(s1), s2)
    n, h, dk = 6, 2, 8
    q, k, v = (rnd(n, h, dk, seed=i) for i in (7, 8, 9))
    beta, gl, st = torch.rand(n, h), -torch.rand(n, h, dk), rnd(h, dk, dk, seed=10) * 0.1
    o1, s1 = G.gdn_recurrent(q.numpy(), k.numpy(), v.numpy(), beta.numpy(), gl.numpy(), st.numpy())
    o2, s2 = R.gdn_recurrent(q, k, v, beta, gl, st)
    assert torch.allclose(t(o1), o2, atol=1e-5) and torch.allclose(t(s1), s2, atol=1e-5)
    qi, keys, wi = rnd(3, 2, 8, seed=11), rnd(9, 8, seed=12), torch.rand(3, 2)
    assert torch.equal(t(G.indexer_topk(qi.numpy(), keys.numpy(), wi.numpy(), 4, 5)), R.indexer_topk(qi, keys, wi, 4, 5))
    T = 12
    kk, vv = rnd(T, h, dk, seed=13), rnd(T, h, dk, seed=14)
    idx = torch.tensor([[0, 3, 3, -1, 7], [11, 2, -1, -1, 2], [5, 5, 5, 5, 5], [-1, -1, -1, -1, -1], [1, 2, 3, 4, 6], [0, 1, 2, 3, 4]])
    o1, l1 = G.sparse_mla_attn(q.numpy(), kk.numpy(), vv.numpy(), idx.numpy(), True)
    o2, l2 = R.sparse_mla_attn(q, kk, vv, idx, return_lse=True)
    assert torch.allclose(t(o1), o2, atol=1e-5)
    assert torch.allclose(t(l1)[[0, 1, 2, 4, 5]], l2[[0, 1, 2, 4, 5]], atol=1e-5)
    lg, bias = rnd(4, 16, seed=15), rnd(16, seed=16) * 0.1
    w1, i1 = G.moe_route(lg.numpy(), bias.numpy(), 3, 2.5)
    w2, i2 = R.moe_route(lg, bias, 3, 2.5)
    assert torch.equal(t(i1), i2) and torch.allclose(t(w1), w2, atol=1e-6)
    Rr, fn, sc, bs = rnd(3, 4, 16, seed=17), rnd(24, 64, seed=18) * 0.1, torch.tensor([0.7, 1.2, 0.9]), rnd(24, seed=19) * 0.2
    a = G.hc_pre(Rr.numpy(), fn.numpy(), sc.numpy(), bs.numpy(), 1e-5, 1e-6, 20)
    b = R.hc_pre(Rr, fn, sc, bs, 1e-5, 1e-6, 20)
    for u, w_ in zip(a, b):
        assert torch.allclose(t(u), w_, atol=1e-5)
    y = rnd(3, 16, seed=20)
    assert torch.allclose(t(G.hc_post(y.numpy(), Rr.numpy(), a[1], a[2])), R.hc_post(y, Rr, b[1], b[2]), atol=1e-5)
    assert G.argmax_first(np.array([1, 5, 5, 2], dtype=np.float32)) == 1
    assert G.spec_accept([5, 6], [5, 9, 7], True) == 2 and G.spec_accept([5, 6], [5, 6], False) == 2


def test_golden_dcp_merge_equals_full():
    n, h, d, T = 3, 2, 8, 40
    q, k, v = rnd(n, h, d, seed=1), rnd(T, h, d, seed=2), rnd(T, h, d, seed=3)
    idx = torch.stack([torch.randperm(T, generator=torch.Generator().manual_seed(i))[:15] for i in range(n)])
    full = G.sparse_mla_attn(q.numpy(), k.numpy(), v.numpy(), idx.numpy())
    outs, lses = [], []
    for shard in range(4):
        own = torch.where((idx // 4) % 4 == shard, idx, torch.full_like(idx, -1))
        o, l = G.sparse_mla_attn(q.numpy(), k.numpy(), v.numpy(), own.numpy(), True)
        outs.append(o); lses.append(l)
    merged = G.lse_merge(np.stack(outs), np.stack(lses))
    assert np.allclose(merged, full, atol=1e-5)


def test_pools_and_reshard_plan():
    p = rt.PagePool(8)
    a = p.alloc(3)
    assert len(a) == 3 and p.free_pages == 5 and p.alloc(6) == []
    p.retain(a[0]); p.release(a[0]); assert p.refcount(a[0]) == 1
    for pg in a:
        p.release(pg)
    assert p.free_pages == 8
    with pytest.raises(RuntimeError):
        p.release(a[0])
    s = rt.SlotPool(2)
    assert [s.alloc(), s.alloc(), s.alloc()] == [0, 1, -1]
    s.free(0); assert s.alloc() == 0
    assert [rt.cp_layer_range(r, 4, 45) for r in range(4)] == [(0, 12), (12, 23), (23, 34), (34, 45)]
    is_dsa = [1 if i % 4 == 3 else 0 for i in range(8)]
    plan = rt.ReshardPlan.compile(is_dsa, 2, 4, 10)
    assert plan.paged_layers == [3, 7] and plan.state_layers == [0, 1, 2, 4, 5, 6]
    assert plan.layer_owner == [0, 0, 0, 0, 1, 1, 1, 1]
    assert plan.filter_pages(1) == [1, 5, 9]
    m = plan.moves[6]
    assert (m.dst_rank, m.dst_index) == (2, 1)


def test_radix_cache_match_lock_evict():
    c = rt.RadixCache(4)
    toks = list(range(12))
    node, dp, ds = c.insert(toks, [10, 11, 12], [-1, 7, -1])
    assert dp == [] and ds == []
    m = c.match(toks + [99])
    assert m.tokens == 8 and m.pages == [10, 11] and m.snapshot == 7  # deepest node WITH a snapshot
    assert c.match([5, 5, 5, 5]).tokens == 0
    _, dp, _ = c.insert(toks[:8] + [50, 51, 52, 53], [20, 21, 22], [-1, -1, 9])
    assert dp == [20, 21]  # blocks already cached keep their pages
    c.lock(m.node)
    ev = c.evict(10)
    assert sorted(ev.pages) == [12, 22] and ev.snapshots == [9]  # the pinned path survives
    c.unlock(m.node)
    ev = c.evict(10)
    assert sorted(ev.pages) == [10, 11] and ev.snapshots == [7]
    st = c.stats()
    assert st.tree_nodes == 0 and st.hits == 1 and st.misses == 1


def test_tiered_store_demotes_before_dropping():
    s = rt.TieredStore(2, 1, 1)
    ids = []
    for row in range(4):
        i, moves, dropped = s.capture(row)
        ids.append(i)
        assert dropped == []
    assert s.census() == [2, 1, 1]
    assert s.tier_of(ids[0]) == rt.TIER_DISK and s.tier_of(ids[1]) == rt.TIER_HOST
    i5, moves, dropped = s.capture(9)
    assert dropped == [ids[0]]  # every tier was full: the oldest falls off the end
    assert [(m.from_tier, m.to_tier) for m in moves][-1] == (rt.TIER_NONE, rt.TIER_DEVICE)
    slot, moves, dropped = s.promote(ids[1])
    assert slot >= 0 and s.tier_of(ids[1]) == rt.TIER_DEVICE
    s.release(ids[1])
    assert s.tier_of(ids[1]) == rt.TIER_NONE


def _drain(sched, steps=200, tokens_per_row=1):
    """Drive the planner with a fake backend that emits token 7 forever."""
    events = []
    for _ in range(steps):
        plan = sched.plan()
        for ch in plan.prefill:
            ev, _ = sched.ingest_prefill(ch.req, ch.len, 7 if ch.last else -1, ch.snapshot_after)
            events += ev
        if plan.decode.n_live:
            events += sched.ingest_decode([[7] * tokens_per_row if r >= 0 else [] for r in plan.decode.rows])
        if sched.idle():
            break
    return events


def test_tick_planner_continuous_batching():
    cfg = rt.SchedConfig()
    cfg.max_rows, cfg.prefill_budget, cfg.page_size, cfg.num_pages = 4, 32, 16, 64
    s = rt.BatchScheduler(cfg)
    ids = [s.submit(list(range(b, b + n)), 5, []) for b, n in ((100, 40), (1000, 20), (2000, 50))]
    plan = s.plan()
    assert plan.admitted == ids
    assert sum(c.len for c in plan.prefill) == 32 and plan.prefill[0].start == 0  # budget respected
    assert plan.prefill[0].len == 32 and plan.prefill[0].snapshot_after  # chunk ends on the last block boundary
    for ch in plan.prefill:
        s.ingest_prefill(ch.req, ch.len, 7 if ch.last else -1, ch.snapshot_after)
    ev = _drain(s)
    fin = [e for e in ev if e.kind == rt.EV_FINISHED]
    assert sorted(e.req for e in fin) == ids and all(e.reason == "length" and e.completion_tokens == 5 for e in fin)
    st = s.stats()
    assert st.live_rows == 0 and st.tokens_committed == 15
    assert st.radix.tree_blocks == 2 + 1 + 3  # whole prompt blocks published to the prefix cache
    # second round: same prompt -> prefix hit restores state and leases the shared pages
    rid = s.submit(list(range(100, 140)), 3, [])
    plan = s.plan()
    assert plan.restores and plan.restores[0].row == 0
    assert plan.prefill[0].start == 32 and plan.prefill[0].len == 8 and plan.prefill[0].last
    ev = []
    for ch in plan.prefill:
        e, _ = s.ingest_prefill(ch.req, ch.len, 7 if ch.last else -1, ch.snapshot_after)
        ev += e
    assert ev[0].kind == rt.EV_ADMITTED and ev[0].prefix_hit and ev[0].cached_tokens == 32
    _drain(s)
    assert s.get(rid).finish_reason == "length"
    assert s.stats().pages_in_use == s.stats().radix.tree_blocks  # only the cache still holds pages


def test_tick_planner_stop_cancel_buckets_and_row_compaction():
    cfg = rt.SchedConfig()
    cfg.max_rows, cfg.prefill_budget, cfg.page_size, cfg.num_pages = 8, 512, 16, 256
    s = rt.BatchScheduler(cfg)
    ids = [s.submit([1, 2, 3, 4, 5], 50 if i != 1 else 2, [99]) for i in range(5)]
    plan = s.plan()
    for ch in plan.prefill:
        s.ingest_prefill(ch.req, ch.len, 7, False)
    plan = s.plan()
    assert plan.decode.n_live == 5 and plan.decode.bucket == 8 and rt.bucket_for([1, 2, 4, 8], 3) == 4
    ev = s.ingest_decode([[7], [7], [99], [7, 7, 7], [7]])  # row 1 hits max_new, row 2 hits a stop id
    fin = {e.req: e.reason for e in ev if e.kind == rt.EV_FINISHED}
    assert fin == {ids[1]: "length", ids[2]: "stop"}
    assert [e.tokens for e in ev if e.kind == rt.EV_TOKENS and e.req == ids[3]] == [[7, 7, 7]]
    assert s.get(ids[2]).generated == [7]  # the stop token is never emitted
    plan = s.plan()
    assert sorted((m.from_row, m.to_row) for m in plan.row_moves) == [(3, 2), (4, 1)]  # live rows stay a dense prefix
    assert plan.decode.n_live == 3 and plan.decode.bucket == 4
    assert s.cancel(ids[0]) and not s.cancel(ids[0])
    assert s.get(ids[0]).finish_reason == "cancelled"
    _drain(s)
    assert s.idle()


def test_tick_planner_page_pressure_evicts_cache_then_queues():
    cfg = rt.SchedConfig()
    cfg.max_rows, cfg.prefill_budget, cfg.page_size, cfg.num_pages = 4, 512, 16, 12
    s = rt.BatchScheduler(cfg)
    a = s.submit(list(range(64)), 8, [])
    _drain(s)
    assert s.stats().radix.tree_blocks == 4
    b = s.submit(list(range(1000, 1100)), 40, [])  # needs 10 pages: the cache must give way
    c = s.submit(list(range(2000, 2100)), 40, [])  # does not fit next to b: stays queued
    plan = s.plan()
    assert plan.admitted == [b] and s.stats().queued == 1
    _drain(s)
    assert s.get(c).finish_reason == "length"


def test_pdaf_transfer_plan_page_mask():
    from ferrite_b200.parallel.pdaf import TransferPlan
    plan = TransferPlan(n_tokens=70, page_size=16, n_dcp=4, d=1)
    assert plan.n_pages == 5 and plan.src_pages == [1] and plan.dst_slots == [0]
    got = sorted(p for d in range(4) for p in TransferPlan(70, 16, 4, d).src_pages)
    assert got == [0, 1, 2, 3, 4]                       # every page goes to exactly one decode rank
    p0 = TransferPlan(70, 16, 4, 0)
    assert p0.src_pages == [0, 4] and p0.dst_slots == [0, 1]   # page p lands at slot p // n_dcp
    assert TransferPlan(70, 16).src_pages == [0, 1, 2, 3, 4]
    assert p0.bytes_moved(100, 7) == 207


def test_slot_scheduler_plans_admission_budgeted_prefill_and_finish_rules():
    """csrc/runtime/slot_scheduler.h driven directly: FIFO admission into free slots, the per-tick prefill budget cut
    into chunks, decode rows in admission order with a padded bucket, stop / length / context / cancel finishes."""
    from ferrite_b200 import build
    build.build_runtime()
    from ferrite_b200 import _runtime as rt
    c = rt.SlotSchedConfig()
    c.max_seqs, c.prefill_rows, c.prefill_budget, c.max_ctx, c.buckets = 2, 4, 6, 16, [1, 2, 4, 8]
    s = rt.SlotScheduler(c)
    assert s.buckets() == [1, 2] and s.max_prompt() == 12 and s.free_slots() == [1, 0]
    assert s.submit([], 1, []) == -1 and s.submit(list(range(13)), 1, []) == -1
    a = s.submit([1, 2, 3, 4, 5, 6, 7], 3, [99])
    b = s.submit([1], 50, [])
    d = s.submit([5, 5], 2, [])
    assert s.begin_tick() == ([], []) and s.plan_decode().bucket == 0
    pp = s.plan_prefill()
    assert [(e.req, e.kind, e.prompt_tokens) for e in pp.events] == [(a, rt.SLOT_EV_ADMITTED, 7), (b, rt.SLOT_EV_ADMITTED, 1)]
    assert pp.reset_slots == [0, 1]
    assert [(ch.req, ch.slot, ch.start, ch.len, ch.last) for ch in pp.chunks] == [(a, 0, 0, 4, False), (a, 0, 4, 2, False)]
    # tick 2: nobody decodes yet; a's last token and b's prompt fit the budget
    s.begin_tick()
    assert s.plan_decode().bucket == 0
    pp = s.plan_prefill()
    assert [(ch.req, ch.start, ch.len, ch.last) for ch in pp.chunks] == [(a, 6, 1, True), (b, 0, 1, True)]
    ev, rel = s.ingest_first(a, 40)
    assert [(e.req, e.kind, e.token) for e in ev] == [(a, rt.SLOT_EV_TOKEN, 40)] and rel == []
    s.ingest_first(b, 41)
    # tick 3: both decode in one bucket of 2; a hits its stop id (not emitted), its slot goes to d in the same tick
    s.begin_tick()
    dp = s.plan_decode()
    assert (dp.bucket, dp.slots, dp.reqs) == (2, [0, 1], [a, b])
    ev, rel = s.ingest_decode([99, 7])
    assert [(e.req, e.kind, e.reason) for e in ev] == [(a, rt.SLOT_EV_FINISHED, "stop"), (b, rt.SLOT_EV_TOKEN, "")]
    assert ev[0].completion_tokens == 1 and rel == [0]
    pp = s.plan_prefill()
    assert [e.req for e in pp.events] == [d] and pp.reset_slots == [0] and [(ch.req, ch.len, ch.last) for ch in pp.chunks] == [(d, 2, True)]
    ev, _ = s.ingest_first(d, 8)
    # b runs into the context limit: 1 prompt token + n outputs + 2 >= 16
    reasons = {}
    for _ in range(40):
        s.begin_tick()
        dp = s.plan_decode()
        if not dp.bucket:
            break
        ev, rel = s.ingest_decode([3] * len(dp.slots))
        for e in ev:
            if e.kind == rt.SLOT_EV_FINISHED:
                reasons[e.req] = (e.reason, e.completion_tokens)
        s.plan_prefill()
    assert reasons[d] == ("length", 2) and reasons[b] == ("context", 13)
    # cancellation of a queued and of a live request
    x = s.submit([1, 2], 5, [])
    y = s.submit([3], 5, [])
    z = s.submit([4], 5, [])
    s.begin_tick(); s.plan_decode(); s.plan_prefill()
    s.cancel(x); s.cancel(z)
    ev, rel = s.begin_tick()
    assert [(e.req, e.reason) for e in ev] == [(x, "cancelled")] and len(rel) == 1
    st = s.stats()
    assert (st.live, st.queued, st.free_slots) == (1, 0, 1) and not s.idle()
