"""CPU: the HTTP stack over the deterministic host engine (no model): schema, streaming,
UTF-8 hold-back, stop ids, prefix-cache hits, stats, single-flight adapter."""
import json

import pytest

from ferrite_b200.serve.api import create_app
from ferrite_b200.serve.engine import EngineDriver, HostEngine, RequestSpec, SingleFlight
from ferrite_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer, render_chat_template, utf8_holdback

try:
    from starlette.testclient import TestClient
    HAVE_CLIENT = True
except Exception:  # httpx missing
    HAVE_CLIENT = False


def test_chat_template_and_holdback():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "U"}, {"role": "assistant", "content": "A"}]
    assert render_chat_template(msgs) == "<|user|>\nS</s>\n<|user|>\nU</s>\n<|assistant|>\nA</s>\n<|assistant|>\n"
    s = "añ€😀".encode()
    assert utf8_holdback(s) == 0
    assert utf8_holdback(s[:-1]) == 3 and utf8_holdback(s[:-3]) == 1 and utf8_holdback(s[:2]) == 1
    assert utf8_holdback(b"abc") == 0


def _drive(engine, spec, max_ticks=500):
    rid = engine.submit(spec)
    evs = []
    for _ in range(max_ticks):
        for r, e in engine.tick():
            if r == rid:
                evs.append(e)
        if evs and evs[-1].kind == "finished":
            break
    return evs


def test_host_engine_is_deterministic_and_hits_prefix_cache():
    eng = HostEngine(prefill_budget=32)
    prompt = list(range(40, 90))
    a = _drive(eng, RequestSpec(prompt, 12))
    b = _drive(eng, RequestSpec(prompt, 12))
    toks = lambda evs: [t for e in evs if e.kind == "tokens" for t in e.ids]
    assert toks(a) == toks(b) and len(toks(a)) == 12
    assert a[0].kind == "admitted" and not a[0].prefix_hit
    assert b[0].prefix_hit and b[-1].usage.cached_tokens == 48
    st = eng.stats()
    assert st["radix"]["hits"] == 1 and st["radix"]["tree_blocks"] == 3 and st["engine"]["tokens_committed"] == 24


class _Echo:
    """StepEngine that replays the prompt, two tokens per step."""

    def start(self, prompt):
        self.p, self.i = prompt, 1
        return prompt[0], 0

    def step(self):
        out = self.p[self.i:self.i + 2]
        self.i += 2
        if not out:
            raise RuntimeError("ran past the prompt")
        return out


def test_single_flight_fifo_stop_and_poison():
    sf = SingleFlight(_Echo())
    r1 = sf.submit(RequestSpec([5, 6, 7, 9, 8], 10, stop_ids=(9,)))
    r2 = sf.submit(RequestSpec([1, 2, 3], 2))
    r3 = sf.submit(RequestSpec([4], 5))
    evs = []
    while not sf.idle():
        evs += sf.tick()
    by = lambda r: [e for q, e in evs if q == r]
    assert [t for e in by(r1) if e.kind == "tokens" for t in e.ids] == [5, 6, 7] and by(r1)[-1].reason == "stop"
    assert by(r2)[-1].reason == "length" and by(r2)[-1].usage.completion_tokens == 2
    assert by(r3)[-1].reason.startswith("error:") and sf.poisoned  # only that request is lost
    assert [q for q, e in evs if e.kind == "admitted"] == [r1, r2, r3]


@pytest.mark.skipif(not HAVE_CLIENT, reason="starlette TestClient needs httpx")
def test_http_routes_and_streaming():
    tok = ChatTokenizer(ByteTokenizer())
    driver = EngineDriver(HostEngine())
    stopped = []
    app = create_app(driver, tok, "test-model", on_shutdown=lambda: stopped.append(1))
    with TestClient(app) as c:
        assert c.get("/health").json()["status"] == "ok"
        assert c.get("/v1/models").json()["data"][0] == {"id": "test-model", "object": "model", "created": 0, "owned_by": "ferrite"}
        r = c.post("/v1/chat/completions", json={"messages": []})
        assert r.status_code == 400 and r.json()["error"]["type"] == "invalid_request_error"
        body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 9, "unknown_field": 1, "temperature": 0.7}
        r = c.post("/v1/chat/completions", json=body).json()
        assert r["object"] == "chat.completion" and r["choices"][0]["finish_reason"] == "length"
        assert r["usage"]["completion_tokens"] == 9 and r["usage"]["total_tokens"] == r["usage"]["prompt_tokens"] + 9
        text = r["choices"][0]["message"]["content"]
        assert len(text) == 9
        body.update(stream=True, include_usage=True, max_completion_tokens=9)
        with c.stream("POST", "/v1/chat/completions", json=body) as s:
            lines = [l for l in s.iter_lines() if l]
        assert lines[0].startswith(": ferrite: admitted prefix_hit=") and lines[-1] == "data: [DONE]"
        frames = [json.loads(l[6:]) for l in lines if l.startswith("data: {")]
        assert all(f["object"] == "chat.completion.chunk" for f in frames)
        assert "".join(f["choices"][0]["delta"].get("content", "") for f in frames) == text  # same greedy text
        assert frames[-1]["choices"][0]["finish_reason"] == "length" and frames[-1]["usage"]["completion_tokens"] == 9
        st = c.get("/v1/stats").json()
        assert set(st) == {"engine", "radix", "hicache"} and st["engine"]["tokens_committed"] >= 18
        m = c.get("/metrics")
        assert m.status_code == 200 and m.headers["content-type"].startswith("text/plain")
        vals = {l.split(" ")[0]: float(l.split(" ")[1]) for l in m.text.splitlines() if l and not l.startswith("#")}
        assert vals["ferrite_requests_total"] == 2 and vals["ferrite_completion_tokens_total"] == 18
        assert vals['ferrite_requests_finished_total{reason="length"}'] == 2
        assert vals["ferrite_time_to_first_token_seconds_count"] == 2 and vals['ferrite_time_to_first_token_seconds_bucket{le="+Inf"}'] == 2
        assert vals["ferrite_engine_tokens_committed_total"] >= 18 and vals["ferrite_engine_failed"] == 0
        assert c.post("/shutdown").json() == {"status": "shutting_down"}
    driver.shutdown()


def test_cli_dsv41_cpu_backend_generates(capsys):
    """One-shot generation through the CLI with the DSV41 golden model on CPU (plain and DSpark)."""
    from ferrite_b200.serve.__main__ import main
    outs = []
    for mtp in ("1", "3"):
        assert main(["--model", "dsv41-tiny", "--backend", "cpu", "--prompt", "hi", "--max-tokens", "6", "--mtp", mtp]) == 0
        outs.append(capsys.readouterr().out)
    assert outs[0] == outs[1] and len(outs[0]) > 0       # speculation does not change the text


def test_serving_workload_bench_on_the_mock_engine(capsys):
    """bench_serving.py end to end on the host engine: ragged prompts, more requests than rows, every request gets
    its tokens and a first-token time."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench_serving.py")
    spec = importlib.util.spec_from_file_location("bench_serving", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.main(["--model", "mock", "--requests", "20", "--max-seqs", "4", "--prompt-min", "5", "--prompt-max", "90",
                     "--new-tokens", "12"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["metric"] == "serving_output_tok_s" and line["output_tokens"] == 20 * 12 and line["value"] > 0
    assert line["finish_reasons"] == {"length": 20} and line["p50_ttft_ms"] is not None and line["p95_ttft_ms"] >= line["p50_ttft_ms"]


def test_cli_host_cpu_profile(tmp_path, capsys):
    from ferrite_b200.serve.__main__ import main
    out = tmp_path / "run.pstats"
    assert main(["--model", "mock", "--prompt", "hello", "--max-tokens", "4", "--cpu-profile", str(out)]) == 0
    import pstats
    st = pstats.Stats(str(out))
    assert st.total_calls > 0 and "cumulative" in capsys.readouterr().err
