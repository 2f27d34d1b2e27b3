"""CPU: the context limit (planner, single-flight adapter, HTTP 400), the driver's failure handling
(an engine that raises poisons the server instead of hanging it) and the status arena (guard words,
status words read back with a step's result)."""
import queue
import time

import pytest
import torch

from ferrite_b200 import _runtime as rt
from ferrite_b200.parallel.status import (CANARY, FB_BAD_ARG, FB_TIMEOUT, CanaryError, CollectiveTimeout,
                                          ContextGuard, StatusArena)
from ferrite_b200.serve.api import create_app
from ferrite_b200.serve.engine import (ContextOverflow, EngineDriver, EngineFailed, HostEngine, RequestSpec,
                                       SingleFlight)
from ferrite_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer

try:
    from starlette.testclient import TestClient
    HAVE_CLIENT = True
except Exception:
    HAVE_CLIENT = False


def test_planner_finishes_at_the_context_limit_and_refuses_long_prompts():
    cfg = rt.SchedConfig()
    cfg.max_rows, cfg.prefill_budget, cfg.page_size, cfg.num_pages = 2, 64, 16, 64
    cfg.max_ctx, cfg.spec_rows = 32, 3
    s = rt.BatchScheduler(cfg)
    assert cfg.ctx_headroom() == 5 and s.max_prompt() == 26
    assert s.submit(list(range(27)), 4, []) == -1 and s.submit([], 4, []) == -1      # nothing queued
    assert s.idle()
    rid = s.submit(list(range(20)), 1000, [])
    plan = s.plan()
    ev = []
    for ch in plan.prefill:
        e, _ = s.ingest_prefill(ch.req, ch.len, 7 if ch.last else -1, ch.snapshot_after)
        ev += e
    for _ in range(100):
        plan = s.plan()
        if not plan.decode.n_live:
            break
        ev += s.ingest_decode([[7, 7, 7] if r >= 0 else [] for r in plan.decode.rows])
    fin = [e for e in ev if e.kind == rt.EV_FINISHED]
    assert len(fin) == 1 and fin[0].reason == "length"
    # the sequence stopped while a whole 3-row step (+2) still fit below max_ctx
    assert 20 + fin[0].completion_tokens + cfg.ctx_headroom() >= cfg.max_ctx
    assert 20 + fin[0].completion_tokens < cfg.max_ctx and s.get(rid) is not None


class _Limited:
    """StepEngine with a context limit of 12 positions, one token per step."""
    MAX = 12

    def start(self, prompt):
        self.n = len(prompt)
        return 1, 0

    def step(self):
        assert self.room() > 0, "stepped past the limit"
        self.n += 1
        return [1]

    def max_prompt(self):
        return self.MAX - 4

    def room(self):
        return self.MAX - self.n - 3


def test_single_flight_stops_at_the_limit_and_refuses_long_prompts():
    sf = SingleFlight(_Limited())
    with pytest.raises(ContextOverflow):
        sf.submit(RequestSpec(list(range(9)), 5))
    rid = sf.submit(RequestSpec([3, 4, 5], 100))
    evs = []
    while not sf.idle():
        evs += sf.tick()
    fin = [e for r, e in evs if e.kind == "finished"]
    assert fin[0].reason == "length" and fin[0].usage.completion_tokens == 7 and rid == 1


class _Exploding(HostEngine):
    def __init__(self, after: int):
        super().__init__()
        self.after = after

    def tick(self):
        self.after -= 1
        if self.after < 0:
            raise RuntimeError("device fell over")
        return super().tick()


def test_driver_poisons_instead_of_hanging_when_the_engine_raises():
    d = EngineDriver(_Exploding(after=3))
    rid, sink = d.submit(RequestSpec(list(range(40, 60)), 50))
    evs = []
    deadline = time.time() + 10
    while time.time() < deadline:
        try:
            evs.append(sink.get(timeout=0.5))
        except queue.Empty:
            continue
        if evs[-1].kind == "finished":
            break
    assert evs and evs[-1].kind == "finished" and evs[-1].reason == "error:RuntimeError"
    assert d.poisoned and "device fell over" in d.poisoned
    with pytest.raises(EngineFailed):
        d.submit(RequestSpec([1, 2, 3], 4))
    d.shutdown()


def test_driver_hands_a_refusal_back_to_the_caller():
    d = EngineDriver(HostEngine(max_ctx=64))
    with pytest.raises(ContextOverflow):
        d.submit(RequestSpec(list(range(64)), 4))
    rid, sink = d.submit(RequestSpec(list(range(40, 50)), 100))   # still serving; stops at the limit
    n = 0
    while True:
        ev = sink.get(timeout=5)
        if ev.kind == "tokens":
            n += len(ev.ids)
        if ev.kind == "finished":
            break
    assert ev.reason == "length" and 10 + n < 64 and not d.poisoned
    d.shutdown()


@pytest.mark.skipif(not HAVE_CLIENT, reason="starlette TestClient needs httpx")
def test_http_400_for_a_prompt_past_the_limit_and_503_after_a_failure():
    tok = ChatTokenizer(ByteTokenizer())
    d = EngineDriver(HostEngine(max_ctx=48))
    with TestClient(create_app(d, tok, "m", on_shutdown=lambda: None)) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x" * 100}]})
        assert r.status_code == 400 and "context limit" in r.json()["error"]["message"]
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 500})
        assert r.status_code == 200 and r.json()["choices"][0]["finish_reason"] == "length"
        assert r.json()["usage"]["total_tokens"] < 48
    d.shutdown()
    d = EngineDriver(_Exploding(after=0))
    with TestClient(create_app(d, tok, "m", on_shutdown=lambda: None)) as c:
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]})
        assert r.status_code == 200 and r.json()["choices"][0]["finish_reason"] == "error:RuntimeError"
        assert c.get("/health").status_code == 503
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]})
        assert r.status_code == 503 and r.json()["error"]["type"] == "server_error"
    d.shutdown()


def test_status_arena_guards_and_status_words():
    a = StatusArena("cpu", 256)
    epoch = a.take(5, "ar.epoch")
    st = a.status("ar")
    rows = a.status("rows")
    assert epoch.numel() == 5 and st.data_ptr() % 16 == 0 and rows.data_ptr() % 16 == 0
    epoch += 3                       # ordinary use leaves the guards alone
    a.verify(snapshot=False)
    st.copy_(torch.tensor([FB_TIMEOUT, 2, 17, 5], dtype=torch.int32))
    with pytest.raises(CollectiveTimeout) as e:
        a.verify(snapshot=False)
    assert (e.value.peer, e.value.epoch, e.value.chunk, e.value.name) == (2, 17, 5, "ar")
    assert int(st[0]) == 0           # cleared: the next wait gets a fresh budget
    rows.copy_(torch.tensor([FB_BAD_ARG, 1, 4090, 3], dtype=torch.int32))
    with pytest.raises(ContextGuard) as e:
        a.verify(snapshot=False)
    assert (e.value.slot, e.value.length, e.value.rows) == (1, 4090, 3)
    # a stray store one word past the epoch block lands on a guard word
    off = (epoch.data_ptr() - a.buf.data_ptr()) // 4
    a.buf[off + 8] = 1234
    with pytest.raises(CanaryError) as e:
        a.verify(snapshot=False)
    assert e.value.name == "ar.epoch" and e.value.value == 1234
    assert int(a.buf[off + 8]) == CANARY
    a.verify(snapshot=False)
