"""OpenAI-compatible HTTP API (FastAPI): chat completions with SSE streaming, models,
health, stats and shutdown.

Routes and payloads follow the reference server (``crates/ferrite-http/src/api.rs:68-393``,
``sse.rs:1-193``): ``POST /v1/chat/completions`` (``messages`` required and non-empty, else
400 ``invalid_request_error``; ``max_completion_tokens`` wins over ``max_tokens``, default 256;
``temperature`` accepted and ignored -- decoding is greedy; unknown fields ignored),
``GET /v1/models``, ``GET /health``, ``GET /v1/stats``, ``POST /shutdown``.  A stream sends an
optional comment line with the admission result, one ``chat.completion.chunk`` per engine
event (bytes of an incomplete UTF-8 character are held back), a final frame with
``finish_reason`` (and ``usage`` if asked), then ``data: [DONE]``; closing the connection
cancels the request.
"""

import asyncio
import json
import os
import threading
import time
import uuid
from typing import List, Optional

from .engine import ContextOverflow, EngineDriver, EngineFailed, RequestSpec, Usage
from .tokenizer import ChatTokenizer, utf8_holdback


def _err(msg: str, status: int = 400, kind: str = "invalid_request_error"):
    from fastapi.responses import JSONResponse
    return JSONResponse({"error": {"message": msg, "type": kind}}, status_code=status)


class _LoopSink:
    """Event sink of one request: the driver thread calls ``put``, the event loop awaits ``get``.  Events
    cross threads with ``call_soon_threadsafe``, so a waiting request costs nothing and wakes at once."""

    def __init__(self, loop):
        self.loop = loop
        self.q: "asyncio.Queue" = asyncio.Queue()

    def put(self, ev) -> None:
        try:
            self.loop.call_soon_threadsafe(self.q.put_nowait, ev)
        except RuntimeError:      # the loop is closed (server shutting down)
            pass

    async def get(self):
        return await self.q.get()


def _usage(u: Optional[Usage]) -> dict:
    u = u or Usage()
    return {"prompt_tokens": u.prompt_tokens, "completion_tokens": u.completion_tokens,
            "total_tokens": u.total_tokens, "cached_tokens": u.cached_tokens}


def finish_reason(reason: str) -> str:
    return reason if reason in ("stop", "length") else ("stop" if reason == "cancelled" else reason)


class ServerMetrics:
    """Counters of the HTTP layer in the Prometheus text exposition format (``GET /metrics``), next to the JSON of
    ``/v1/stats`` (the reference exposes only the latter, ``crates/ferrite-http/src/driver.rs``): requests, prompt and
    completion tokens, finish reasons, a time-to-first-token histogram, and the engine's gauges."""

    BUCKETS = (0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0)

    def __init__(self):
        self.requests = self.prompt_tokens = self.completion_tokens = 0
        self.reasons: dict = {}
        self.ttft_counts = [0] * (len(self.BUCKETS) + 1)
        self.ttft_sum = 0.0

    def first_token(self, seconds: float) -> None:
        self.ttft_sum += seconds
        for i, b in enumerate(self.BUCKETS):
            if seconds <= b:
                self.ttft_counts[i] += 1
                return
        self.ttft_counts[-1] += 1

    def finished(self, reason: str) -> None:
        key = reason.split(":", 1)[0] or "stop"
        self.reasons[key] = self.reasons.get(key, 0) + 1

    def render(self, stats: dict, poisoned: bool) -> str:
        e = stats.get("engine", {})
        out = ["# TYPE ferrite_requests_total counter", f"ferrite_requests_total {self.requests}",
               "# TYPE ferrite_prompt_tokens_total counter", f"ferrite_prompt_tokens_total {self.prompt_tokens}",
               "# TYPE ferrite_completion_tokens_total counter", f"ferrite_completion_tokens_total {self.completion_tokens}",
               "# TYPE ferrite_requests_finished_total counter"]
        for k in sorted(self.reasons):
            out.append(f'ferrite_requests_finished_total{{reason="{k}"}} {self.reasons[k]}')
        out.append("# TYPE ferrite_time_to_first_token_seconds histogram")
        cum = 0
        for b, c in zip(self.BUCKETS, self.ttft_counts):
            cum += c
            out.append(f'ferrite_time_to_first_token_seconds_bucket{{le="{b}"}} {cum}')
        cum += self.ttft_counts[-1]
        out += [f'ferrite_time_to_first_token_seconds_bucket{{le="+Inf"}} {cum}',
                f"ferrite_time_to_first_token_seconds_sum {self.ttft_sum:.6f}",
                f"ferrite_time_to_first_token_seconds_count {cum}"]
        for name, key in (("ticks_total", "ticks"), ("engine_tokens_committed_total", "tokens_committed")):
            out += [f"# TYPE ferrite_{name} counter", f"ferrite_{name} {int(e.get(key, 0))}"]
        for name, key in (("live_rows", "live_rows"), ("queued_requests", "queued")):
            out += [f"# TYPE ferrite_{name} gauge", f"ferrite_{name} {int(e.get(key, 0))}"]
        out += ["# TYPE ferrite_engine_failed gauge", f"ferrite_engine_failed {int(poisoned)}"]
        return "\n".join(out) + "\n"


def create_app(driver: EngineDriver, tokenizer: ChatTokenizer, model_name: str = "glm-5.3-flash",
               on_shutdown=None):
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    app = FastAPI(title="ferrite_b200")
    metrics = ServerMetrics()

    async def _next_event(sink):
        return await sink.get()

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        try:
            body = await request.json()
        except Exception:
            return _err("request body is not valid JSON")
        msgs = body.get("messages") if isinstance(body, dict) else None
        if not isinstance(msgs, list) or not msgs:
            return _err("`messages` must be a non-empty array")
        for m in msgs:
            if not isinstance(m, dict) or "role" not in m or not isinstance(m.get("content", ""), str):
                return _err("each message needs a `role` and a string `content`")
        max_new = body.get("max_completion_tokens", body.get("max_tokens", 256))
        if not isinstance(max_new, int) or max_new < 1:
            return _err("`max_tokens` must be a positive integer")
        model = body.get("model") or model_name
        stream = bool(body.get("stream", False))
        include_usage = bool(body.get("include_usage", False)) or bool((body.get("stream_options") or {}).get("include_usage"))
        prompt = tokenizer.encode_chat(msgs)
        spec = RequestSpec(prompt, max_new, tuple(tokenizer.stop_ids()))
        loop = asyncio.get_running_loop()
        try:   # the driver admits between ticks: wait for it off the event loop
            rid, sink = await loop.run_in_executor(None, driver.submit, spec, _LoopSink(loop))
        except ContextOverflow as e:
            return _err(str(e), 400)
        except EngineFailed as e:
            return _err(f"engine failed: {e}", 503, "server_error")
        cid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        t_submit = time.perf_counter()
        metrics.requests += 1
        metrics.prompt_tokens += len(prompt)

        if not stream:
            ids: List[int] = []
            usage, reason = None, "stop"
            while True:
                ev = await _next_event(sink)
                if ev.kind == "tokens":
                    if not ids:
                        metrics.first_token(time.perf_counter() - t_submit)
                    ids.extend(ev.ids)
                    metrics.completion_tokens += len(ev.ids)
                elif ev.kind == "finished":
                    usage, reason = ev.usage, ev.reason
                    metrics.finished(reason)
                    break
            return JSONResponse({
                "id": cid, "object": "chat.completion", "created": created, "model": model,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": tokenizer.decode(ids)},
                             "finish_reason": finish_reason(reason)}],
                "usage": _usage(usage)})

        def frame(delta: dict, fin=None, usage=None) -> str:
            obj = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model,
                   "choices": [{"index": 0, "delta": delta, "finish_reason": fin}]}
            if usage is not None:
                obj["usage"] = usage
            return "data: " + json.dumps(obj, ensure_ascii=False) + "\n\n"

        async def gen():
            held = b""
            done = False
            first = True
            try:
                while True:
                    ev = await _next_event(sink)
                    if ev.kind == "admitted":
                        yield f": ferrite: admitted prefix_hit={str(ev.prefix_hit).lower()} prompt_tokens={ev.prompt_tokens}\n\n"
                    elif ev.kind == "tokens":
                        if first:
                            metrics.first_token(time.perf_counter() - t_submit)
                            first = False
                        metrics.completion_tokens += len(ev.ids)
                        data = held + tokenizer.decode_bytes(ev.ids)
                        hb = utf8_holdback(data)
                        held = data[len(data) - hb:] if hb else b""
                        text = data[:len(data) - hb].decode("utf-8", errors="replace")
                        if text:
                            yield frame({"content": text})
                    else:
                        tail = held.decode("utf-8", errors="replace")
                        yield frame({"content": tail} if tail else {}, fin=finish_reason(ev.reason),
                                    usage=_usage(ev.usage) if include_usage else None)
                        yield "data: [DONE]\n\n"
                        done = True
                        metrics.finished(ev.reason)
                        return
            finally:
                if not done:  # the client went away: stop generating for it
                    driver.cancel(rid)
                    metrics.finished("client_gone")

        return StreamingResponse(gen(), media_type="text/event-stream",
                                 headers={"Cache-Control": "no-cache", "Connection": "keep-alive"})

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": 0, "owned_by": "ferrite"}]}

    @app.get("/health")
    async def health():
        if driver.poisoned:
            return _err(f"engine failed: {driver.poisoned}", 503, "server_error")
        e = driver.stats().get("engine", {})
        return {"status": "ok", "engine": {"ticks": e.get("ticks", 0), "tokens_committed": e.get("tokens_committed", 0)}}

    @app.get("/v1/stats")
    async def stats():
        return driver.stats()

    @app.get("/metrics")
    async def prometheus():
        from fastapi.responses import PlainTextResponse
        return PlainTextResponse(metrics.render(driver.stats(), bool(driver.poisoned)), media_type="text/plain; version=0.0.4")

    @app.post("/shutdown")
    async def shutdown():
        def later():
            time.sleep(0.3)  # let the reply (and any profiler) flush first
            if on_shutdown:
                on_shutdown()
            else:
                os._exit(0)
        threading.Thread(target=later, daemon=True).start()
        return {"status": "shutting_down"}

    return app


def serve(engine, tokenizer: ChatTokenizer, host: str = "127.0.0.1", port: int = 8000,
          model_name: str = "glm-5.3-flash"):
    """Blocking: run the HTTP server over ``engine`` until /shutdown."""
    import uvicorn
    driver = EngineDriver(engine)
    app = create_app(driver, tokenizer, model_name)
    uvicorn.run(app, host=host, port=port, log_level="warning")
