"""Engine seam of the HTTP server: request/event types, the ``ServeEngine`` / ``StepEngine``
protocols, the single-flight adapter, a deterministic host engine and the driver thread.

Mirrors the reference's ``ferrite-http`` seams: ``RequestSpec`` -> events ``Admitted``,
``Tokens``, ``Finished`` (``crates/ferrite-http/src/engine.rs:27-216``), ``SingleFlight``
(batch = 1, FIFO; ``single_flight.rs:51-330``), the mock ``HostEngine``
(``host_engine.rs:87-225``) and the ``EngineDriver`` thread that owns the engine and is fed
through a queue (``driver.rs:63-274``).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Protocol, Tuple


@dataclass
class RequestSpec:
    prompt_ids: List[int]
    max_new_tokens: int = 256
    stop_ids: Tuple[int, ...] = ()


@dataclass
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0

    @property
    def total_tokens(self) -> int:
        return self.prompt_tokens + self.completion_tokens


@dataclass
class ReqEvent:
    kind: str  # "admitted" | "tokens" | "finished"
    ids: List[int] = field(default_factory=list)
    reason: str = ""
    usage: Optional[Usage] = None
    prefix_hit: bool = False
    prompt_tokens: int = 0


class ServeEngine(Protocol):
    """What the driver thread needs: admit work, run one tick, report events and stats."""

    def submit(self, spec: RequestSpec) -> int: ...
    def cancel(self, req: int) -> None: ...
    def tick(self) -> List[Tuple[int, ReqEvent]]: ...
    def idle(self) -> bool: ...
    def stats(self) -> dict: ...


class StepEngine(Protocol):
    """A model that serves one sequence at a time: prefill, then step."""

    def start(self, prompt_ids: List[int]) -> Tuple[int, int]: ...  # (first token, cached prefix tokens)
    def step(self) -> List[int]: ...  # 1..n tokens (n > 1 with speculative decoding)


class SingleFlight:
    """Adapts a :class:`StepEngine` to :class:`ServeEngine`: one request in flight, FIFO."""

    def __init__(self, inner: StepEngine):
        self.inner = inner
        self.queue: List[Tuple[int, RequestSpec]] = []
        self.cur: Optional[Tuple[int, RequestSpec]] = None
        self.done = 0
        self.next_id = 1
        self.ticks = 0
        self.tokens_committed = 0
        self.poisoned: Optional[str] = None

    def submit(self, spec: RequestSpec) -> int:
        rid = self.next_id
        self.next_id += 1
        self.queue.append((rid, spec))
        return rid

    def cancel(self, req: int) -> None:
        self.queue = [(r, s) for r, s in self.queue if r != req]
        if self.cur and self.cur[0] == req:
            self.cur = None

    def idle(self) -> bool:
        return self.cur is None and not self.queue

    def _emit(self, rid, spec, toks, out) -> bool:
        keep, reason = [], ""
        for t in toks:
            if t in spec.stop_ids:
                reason = "stop"
                break
            keep.append(t)
            self.done += 1
            if self.done >= spec.max_new_tokens:
                reason = "length"
                break
        if keep:
            self.tokens_committed += len(keep)
            out.append((rid, ReqEvent("tokens", ids=keep)))
        if reason:
            out.append((rid, ReqEvent("finished", reason=reason, usage=Usage(len(spec.prompt_ids), self.done, self._cached))))
            self.cur = None
            return True
        return False

    def tick(self) -> List[Tuple[int, ReqEvent]]:
        out: List[Tuple[int, ReqEvent]] = []
        self.ticks += 1
        try:
            if self.cur is None:
                if not self.queue:
                    return out
                self.cur = self.queue.pop(0)
                rid, spec = self.cur
                self.done = 0
                first, self._cached = self.inner.start(list(spec.prompt_ids))
                out.append((rid, ReqEvent("admitted", prefix_hit=self._cached > 0, prompt_tokens=len(spec.prompt_ids))))
                self._emit(rid, spec, [first], out)
                return out
            rid, spec = self.cur
            self._emit(rid, spec, self.inner.step(), out)
        except Exception as e:  # a failed step poisons only the current request
            if self.cur is not None:
                rid, spec = self.cur
                out.append((rid, ReqEvent("finished", reason="error:" + type(e).__name__,
                                          usage=Usage(len(spec.prompt_ids), self.done, 0))))
                self.poisoned = repr(e)
                self.cur = None
        return out

    def stats(self) -> dict:
        return {"engine": {"ticks": self.ticks, "tokens_committed": self.tokens_committed,
                           "live_rows": int(self.cur is not None), "queued": len(self.queue)},
                "radix": {"tree_nodes": 0, "tree_blocks": 0, "evictable_tokens": 0, "protected_tokens": 0,
                          "hits": 0, "misses": 0},
                "hicache": {"tiers": {"device": 0, "host": 0, "disk": 0}, "pages_in_use": 0, "pages_free": 0}}


def _mock_next(tokens: List[int], vocab: int) -> int:
    """Deterministic fake model: the next token is a hash of the last three."""
    h = 0
    for t in tokens[-3:]:
        h = (h * 1000003 + t + 17) & 0xFFFFFFFF
    return 32 + h % max(1, min(vocab, 127) - 32)  # printable ASCII under the byte tokenizer


class HostEngine:
    """Deterministic batched engine over the C++ tick planner: exercises admission, chunked
    prefill, the radix prefix cache and continuous batching without a model."""

    def __init__(self, vocab: int = 257, max_rows: int = 8, prefill_budget: int = 64, num_pages: int = 4096,
                 page_size: int = 16, next_token: Optional[Callable[[List[int]], int]] = None):
        from .. import build
        build.build_runtime()
        from .. import _runtime as rt
        self.rt = rt
        cfg = rt.SchedConfig()
        cfg.max_rows, cfg.prefill_budget, cfg.num_pages, cfg.page_size = max_rows, prefill_budget, num_pages, page_size
        self.sched = rt.BatchScheduler(cfg)
        self.vocab = vocab
        self.next_token = next_token or (lambda toks: _mock_next(toks, vocab))
        self.ctx: Dict[int, List[int]] = {}

    def submit(self, spec: RequestSpec) -> int:
        rid = self.sched.submit(list(spec.prompt_ids), spec.max_new_tokens, list(spec.stop_ids))
        self.ctx[rid] = list(spec.prompt_ids)
        return rid

    def cancel(self, req: int) -> None:
        self.sched.cancel(req)
        self.ctx.pop(req, None)

    def idle(self) -> bool:
        return self.sched.idle()

    def _convert(self, evs, out):
        rt = self.rt
        for e in evs:
            if e.kind == rt.EV_ADMITTED:
                out.append((e.req, ReqEvent("admitted", prefix_hit=e.prefix_hit, prompt_tokens=e.prompt_tokens)))
            elif e.kind == rt.EV_TOKENS:
                self.ctx.setdefault(e.req, []).extend(e.tokens)
                out.append((e.req, ReqEvent("tokens", ids=list(e.tokens))))
            else:
                out.append((e.req, ReqEvent("finished", reason=e.reason,
                                            usage=Usage(e.prompt_tokens, e.completion_tokens, e.cached_tokens))))
                self.ctx.pop(e.req, None)
                self.sched.forget(e.req)

    def tick(self) -> List[Tuple[int, ReqEvent]]:
        out: List[Tuple[int, ReqEvent]] = []
        plan = self.sched.plan()
        for ch in plan.prefill:
            first = self.next_token(self.ctx[ch.req]) if ch.last else -1
            evs, _ = self.sched.ingest_prefill(ch.req, ch.len, first, ch.snapshot_after)
            self._convert(evs, out)
        if plan.decode.n_live:
            toks = [[self.next_token(self.ctx[r])] if r >= 0 and r in self.ctx else [] for r in plan.decode.rows]
            self._convert(self.sched.ingest_decode(toks), out)
        return out

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


class EngineDriver:
    """One thread owns the engine.  Callers talk to it through a command queue and receive a
    request's events on their own queue; dropping a request cancels it."""

    def __init__(self, engine: ServeEngine, idle_sleep: float = 0.002):
        self.engine = engine
        self.cmds: "queue.Queue" = queue.Queue()
        self.sinks: Dict[int, "queue.Queue"] = {}
        self.idle_sleep = idle_sleep
        self._stop = threading.Event()
        self._stats_lock = threading.Lock()
        self._stats: dict = engine.stats()
        self.thread = threading.Thread(target=self._run, name="engine-driver", daemon=True)
        self.thread.start()

    def submit(self, spec: RequestSpec) -> Tuple[int, "queue.Queue"]:
        reply: "queue.Queue" = queue.Queue()
        sink: "queue.Queue" = queue.Queue()
        self.cmds.put(("submit", spec, sink, reply))
        return reply.get(), sink

    def cancel(self, req: int) -> None:
        self.cmds.put(("cancel", req, None, None))

    def stats(self) -> dict:
        with self._stats_lock:
            return dict(self._stats)

    def shutdown(self) -> None:
        self._stop.set()
        self.thread.join(timeout=5)

    def _run(self):
        while not self._stop.is_set():
            try:
                while True:
                    kind, a, sink, reply = self.cmds.get_nowait()
                    if kind == "submit":
                        rid = self.engine.submit(a)
                        self.sinks[rid] = sink
                        reply.put(rid)
                    elif kind == "cancel":
                        self.engine.cancel(a)
                        self.sinks.pop(a, None)
            except queue.Empty:
                pass
            if self.engine.idle():
                time.sleep(self.idle_sleep)
                continue
            for rid, ev in self.engine.tick():
                sink = self.sinks.get(rid)
                if sink is not None:
                    sink.put(ev)
                    if ev.kind == "finished":
                        self.sinks.pop(rid, None)
            with self._stats_lock:
                self._stats = self.engine.stats()
