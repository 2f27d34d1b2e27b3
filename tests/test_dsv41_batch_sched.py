"""CPU: the continuous-batching logic of the batched DSV41 engine (admission into free slots, chunked prefill within
the tick's token budget, decode buckets with padding rows, stop ids, cancellation, the context limit) driven by a
host stand-in of the device model whose next token is a known function of (token, position)."""
import types

import torch

from ferrite_b200.engine.dsv41_batch import Dsv41BatchEngine, bucket_for
from ferrite_b200.serve.engine import ContextOverflow, RequestSpec

V = 1000


def nxt(tok: int, pos: int) -> int:
    return (tok * 31 + pos * 7 + 3) % V


class FakeRows:
    def __init__(self, slots, gsizes):
        rows = [s for s, g in zip(slots, gsizes) for _ in range(g)]
        self.n = len(rows)
        self.row_slot = torch.tensor(rows, dtype=torch.int32)
        self.group_slot = torch.tensor(list(slots), dtype=torch.int32)
        self.gsizes = list(gsizes)


class FakeModel:
    """out_ids[row] = nxt(input token, position of the row); rows of one group take consecutive positions."""

    def __init__(self, n_slots, max_ctx, max_rows, fn=None):
        self.fn = fn or nxt
        self.dev = torch.device("cpu")
        self.max_ctx, self.max_rows = max_ctx, max_rows
        self.seq_len = torch.zeros(n_slots, dtype=torch.int32)
        self.ws = {"out_ids": torch.zeros(max_rows, dtype=torch.int32)}
        self.arena = types.SimpleNamespace(snapshot_async=lambda: None, verify=lambda snapshot=True: None)
        self.K = types.SimpleNamespace(launches=0)
        self.forwards = []            # (rows, distinct slots) of every forward

    def make_rows(self, slots, gsizes):
        return FakeRows(slots, gsizes)

    def reset_slot(self, slot):
        self.seq_len[slot] = 0

    def forward(self, rs, ids, advance=True, want_logits=True):
        slots = rs.row_slot.tolist()
        assert rs.n <= self.max_rows
        seen = {}
        for r, s in enumerate(slots):
            pos = int(self.seq_len[s]) + seen.get(s, 0)
            assert pos < self.max_ctx, "a row beyond the context limit reached the model"
            seen[s] = seen.get(s, 0) + 1
            self.ws["out_ids"][r] = self.fn(int(ids[r]), pos)
        if advance:
            for s, k in seen.items():
                self.seq_len[s] += k
        self.forwards.append((rs.n, len(seen)))


def expected(prompt, n_new, stop=()):
    out, tok = [], None
    pos = len(prompt) - 1
    tok = nxt(prompt[-1], pos)
    while len(out) < n_new and tok not in stop:
        out.append(tok)
        pos += 1
        tok = nxt(tok, pos)
    return out


def engine(max_seqs=3, max_ctx=64, prefill_rows=4, budget=6):
    model = FakeModel(max_seqs + 1, max_ctx, max(prefill_rows, max_seqs))
    return Dsv41BatchEngine(None, None, max_ctx=max_ctx, max_seqs=max_seqs, prefill_rows=prefill_rows, prefill_budget=budget,
                            model=model), model


def test_more_requests_than_slots_all_finish_with_the_single_sequence_tokens():
    eng, model = engine()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in (5, 1, 13, 2, 9, 7)]
    n_new = [4, 9, 3, 6, 5, 8]
    got = eng.run_all([RequestSpec(p, k) for p, k in zip(prompts, n_new)])
    assert eng.idle() and sorted(eng.free) == [0, 1, 2]
    for rid, (p, k) in enumerate(zip(prompts, n_new), start=1):
        assert got[rid] == expected(p, k), rid
        assert eng.usage[rid].prompt_tokens == len(p) and eng.usage[rid].completion_tokens == k
    # no tick prefilled more than its budget, no prefill chunk was wider than prefill_rows, decode ticks ran buckets
    assert all(rows <= 4 or slots > 1 for rows, slots in model.forwards)
    assert any(slots > 1 for _, slots in model.forwards)            # several sequences shared a decode forward
    assert int(model.seq_len[:3].sum()) == 0                          # every slot was released by a length reset


def test_prefill_budget_keeps_decoding_sequences_moving():
    eng, model = engine(max_seqs=2, prefill_rows=4, budget=4)
    a = eng.submit(RequestSpec([1, 2, 3], 20))
    toks = {a: []}
    for _ in range(2):
        for rid, ev in eng.tick():
            if ev.kind == "tokens":
                toks[rid] += ev.ids
    b = eng.submit(RequestSpec(list(range(40)), 2))                  # ten ticks of prefill at 4 tokens per tick
    toks[b] = []
    before = len(toks[a])
    for _ in range(5):
        for rid, ev in eng.tick():
            if ev.kind == "tokens":
                toks[rid] += ev.ids
    assert len(toks[a]) == before + 5 and not toks[b]                # a advanced every tick while b was still prefilling
    for _ in range(40):
        for rid, ev in eng.tick():
            if ev.kind == "tokens":
                toks[rid] += ev.ids
    assert toks[b] == expected(list(range(40)), 2) and toks[a] == expected([1, 2, 3], 20)


def test_stop_id_cancel_and_context_limit():
    eng, _ = engine(max_seqs=2, max_ctx=24)
    p = [5, 6, 7]
    full = expected(p, 30)
    stop = full[3]
    a = eng.submit(RequestSpec(p, 30, stop_ids=(stop,)))
    b = eng.submit(RequestSpec([9, 9], 100))                          # would run past the context limit
    c = eng.submit(RequestSpec([4], 100))                             # waits for a slot, cancelled while queued
    eng.cancel(c)
    toks, reasons = {a: [], b: [], c: []}, {}
    for _ in range(200):
        for rid, ev in eng.tick():
            if ev.kind == "tokens":
                toks[rid] += ev.ids
            elif ev.kind == "finished":
                reasons[rid] = ev.reason
        if eng.idle():
            break
    assert toks[a] == full[:full.index(stop)] and reasons[a] == "stop"
    assert reasons[b] == "context" and len(toks[b]) + 2 + 2 >= 24 and toks[b] == expected([9, 9], len(toks[b]))
    assert c not in reasons and toks[c] == []
    assert eng.idle() and len(eng.free) == 2


def test_prompt_beyond_the_context_limit_is_refused_and_buckets_pad():
    eng, _ = engine(max_seqs=5, max_ctx=16)
    try:
        eng.submit(RequestSpec(list(range(20)), 4))
        raise AssertionError("a prompt longer than the context was admitted")
    except ContextOverflow:
        pass
    assert eng.buckets == [1, 2, 4, 5] and bucket_for(eng.buckets, 3) == 4 and bucket_for(eng.buckets, 5) == 5


def test_attention_split_count_fits_its_workspace_and_the_kernel_limits():
    from ferrite_b200.models.dsv41 import ATTN_MIN_PARTS, attn_splits
    for heads in (1, 4, 8, 16, 32, 64):
        for n in range(1, 300):
            s = attn_splits(heads, n)
            assert 1 <= s <= 32                                   # the merging warp keeps one split per lane
            assert s < 8 or s % 8 == 0                            # 8 and more: whole clusters of 8
            assert n * heads * s <= max(n * heads, ATTN_MIN_PARTS), (heads, n, s)
    assert attn_splits(16, 1) == 32 and attn_splits(16, 16) == 4 and attn_splits(16, 64) == 1 and attn_splits(64, 1) == 16


def test_batched_engine_behind_the_http_server_streams_two_concurrent_requests():
    """EngineDriver + the OpenAI-style API over the batched engine (host stand-in model that emits printable bytes):
    two streamed requests run in the same decode ticks and both get their own greedy text."""
    import json
    import threading

    from fastapi.testclient import TestClient

    from ferrite_b200.serve.api import create_app
    from ferrite_b200.serve.engine import EngineDriver
    from ferrite_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer
    printable = lambda tok, pos: 97 + (tok * 7 + pos) % 26
    model = FakeModel(3, 512, 8, fn=printable)
    eng = Dsv41BatchEngine(None, None, max_ctx=512, max_seqs=2, prefill_rows=8, prefill_budget=64, model=model)
    tok = ChatTokenizer(ByteTokenizer())
    driver = EngineDriver(eng)
    app = create_app(driver, tok, "dsv41-batch", on_shutdown=lambda: None)
    texts = {}

    def ask(c, name, content):
        body = {"messages": [{"role": "user", "content": content}], "max_tokens": 12, "stream": True}
        with c.stream("POST", "/v1/chat/completions", json=body) as s:
            frames = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: {")]
        texts[name] = "".join(f["choices"][0]["delta"].get("content", "") for f in frames)
        assert frames[-1]["choices"][0]["finish_reason"] == "length"

    with TestClient(app) as c:
        th = [threading.Thread(target=ask, args=(c, n, t)) for n, t in (("a", "first prompt"), ("b", "another, longer prompt"))]
        for t in th:
            t.start()
        for t in th:
            t.join(timeout=60)
        assert set(texts) == {"a", "b"} and all(len(v) == 12 and v.isalpha() for v in texts.values())
        assert texts["a"] != texts["b"]
        st = c.get("/v1/stats").json()
        assert st["engine"]["tokens_committed"] == 24 and st["engine"]["free_slots"] == 2
    driver.shutdown()
    assert any(slots == 2 for _, slots in model.forwards)            # the two requests shared decode forwards


def test_weight_bytes_estimate_matches_the_checkpoint_size_and_shrinks_with_ranks():
    from ferrite_b200.models.dsv41_config import Dsv41Config
    from ferrite_b200.models.dsv41_weights import estimate_device_bytes
    cfg = Dsv41Config()
    gib = [estimate_device_bytes(cfg, w) / 2 ** 30 for w in (1, 2, 4, 8)]
    assert 470 < gib[0] < 480                                  # the production checkpoint is 475 GiB
    assert gib[2] < 0.92 * 180e9 / 2 ** 30 < gib[1]            # fits a 180 GB part from four ranks on, not on two
    assert all(a > b for a, b in zip(gib, gib[1:]))
    assert gib[3] > gib[0] / 8                                 # replicated tensors do not shrink
