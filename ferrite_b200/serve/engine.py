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


class ContextOverflow(ValueError):
    """The prompt leaves no room below the engine's context limit (the HTTP layer answers 400)."""


class EngineFailed(RuntimeError):
    """The engine raised outside a single request's step; the driver is poisoned (HTTP 503)."""


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
    # optional: max_prompt() -> longest prompt that still fits; room() -> steps' worth of tokens left below the
    # context limit (<= 0: the sequence must stop)


class SingleFlight:
    """Adapts a :class:`StepEngine` to :class:`ServeEngine`: one request in flight, FIFO."""

    def __init__(self, inner: StepEngine, swallow_errors: bool = True):
        self.inner = inner
        # False under a ReplicatedEngine: an exception must reach the all-rank acknowledgement so that every
        # rank drops the request together; swallowing it on one rank would desynchronise the planners
        self.swallow_errors = swallow_errors
        self.queue: List[Tuple[int, RequestSpec]] = []
        self.cur: Optional[Tuple[int, RequestSpec]] = None
        self.done = 0
        self.next_id = 1
        self.ticks = 0
        self.tokens_committed = 0
        self.poisoned: Optional[str] = None

    def validate(self, spec: RequestSpec) -> None:
        mp = getattr(self.inner, "max_prompt", None)
        if not spec.prompt_ids or (mp is not None and len(spec.prompt_ids) > mp()):
            raise ContextOverflow(f"prompt of {len(spec.prompt_ids)} tokens does not fit the context limit"
                                  + (f" (at most {mp()})" if mp is not None else ""))

    def submit(self, spec: RequestSpec) -> int:
        self.validate(spec)
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
        room = getattr(self.inner, "room", None)
        if not reason and room is not None and room() <= 0:
            reason = "length"   # the next step would run past the context limit
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
            if not self.swallow_errors:
                self.abort_current("error:" + type(e).__name__, out)
                self.poisoned = repr(e)
                self.pending_events = out
                raise
            if self.cur is not None:
                rid, spec = self.cur
                out.append((rid, ReqEvent("finished", reason="error:" + type(e).__name__,
                                          usage=Usage(len(spec.prompt_ids), self.done, 0))))
                self.poisoned = repr(e)
                self.cur = None
        return out

    def abort_current(self, reason: str, out: list) -> None:
        """Finish the request in flight with `reason` (used when a step failed on some rank)."""
        if self.cur is not None:
            rid, spec = self.cur
            out.append((rid, ReqEvent("finished", reason=reason, usage=Usage(len(spec.prompt_ids), self.done, 0))))
            self.cur = None

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
                 page_size: int = 16, next_token: Optional[Callable[[List[int]], int]] = None,
                 max_ctx: int = 1 << 20):
        from .. import build
        build.build_runtime()
        from .. import _runtime as rt
        self.rt = rt
        cfg = rt.SchedConfig()
        cfg.max_rows, cfg.prefill_budget, cfg.num_pages, cfg.page_size = max_rows, prefill_budget, num_pages, page_size
        cfg.max_ctx = max_ctx
        self.sched = rt.BatchScheduler(cfg)
        self.vocab = vocab
        self.next_token = next_token or (lambda toks: _mock_next(toks, vocab))
        self.ctx: Dict[int, List[int]] = {}

    def validate(self, spec: RequestSpec) -> None:
        if not spec.prompt_ids or len(spec.prompt_ids) > self.sched.max_prompt():
            raise ContextOverflow(f"prompt of {len(spec.prompt_ids)} tokens does not fit the context limit "
                                  f"(at most {self.sched.max_prompt()})")

    def submit(self, spec: RequestSpec) -> int:
        self.validate(spec)
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
    request's events on their own sink (anything with ``put``); dropping a request cancels it.

    The thread never dies silently: a request the engine refuses is answered with the exception
    (``submit`` re-raises it in the caller), and an error out of ``tick`` finishes every open request
    with ``error:<type>``, answers every pending command, and poisons the driver: ``poisoned`` holds
    the message, ``submit`` raises :class:`EngineFailed`, the HTTP layer answers 503.  With a replicated
    (multi-process) engine an idle driver runs an empty heartbeat round every ``heartbeat_s`` seconds so
    that the follower ranks, which block in the command broadcast, never run into the control group's
    timeout while the server simply has nothing to do."""

    def __init__(self, engine: ServeEngine, idle_sleep: float = 0.05, heartbeat_s: float = 5.0):
        self.engine = engine
        self.cmds: "queue.Queue" = queue.Queue()
        self._wake = threading.Event()   # set by submit / cancel: an idle driver wakes at once, not after a sleep
        self.sinks: Dict[int, object] = {}
        self.idle_sleep = idle_sleep
        self.heartbeat_s = heartbeat_s
        self.poisoned: Optional[str] = None
        self._stop = threading.Event()
        self._stats_lock = threading.Lock()
        self._stats: dict = engine.stats()
        self.thread = threading.Thread(target=self._run, name="engine-driver", daemon=True)
        self.thread.start()

    def submit(self, spec: RequestSpec, sink=None, timeout: float = 600.0) -> Tuple[int, object]:
        """Blocks until the driver thread has admitted the request (at most one tick).  Raises what the
        engine raised (:class:`ContextOverflow` for a prompt that does not fit) or :class:`EngineFailed`."""
        if self.poisoned:
            raise EngineFailed(self.poisoned)
        reply: "queue.Queue" = queue.Queue()
        sink = sink if sink is not None else queue.Queue()
        self.cmds.put(("submit", spec, sink, reply))
        self._wake.set()
        try:
            res = reply.get(timeout=timeout)
        except queue.Empty:
            raise EngineFailed("the engine driver did not answer") from None
        if isinstance(res, BaseException):
            raise res
        return res, sink

    def cancel(self, req: int) -> None:
        self.cmds.put(("cancel", req, None, None))
        self._wake.set()

    def stats(self) -> dict:
        with self._stats_lock:
            return dict(self._stats)

    def shutdown(self) -> None:
        self._stop.set()
        self._wake.set()
        self.thread.join(timeout=5)

    def _fail(self, e: BaseException) -> None:
        self.poisoned = f"{type(e).__name__}: {e}"
        reason = "error:" + type(e).__name__
        carried = getattr(self.engine, "take_pending_events", None)
        if carried is not None:   # events produced before the failure (tokens of other requests)
            for rid, ev in carried():
                sink = self.sinks.get(rid)
                if sink is not None:
                    sink.put(ev)
                    if ev.kind == "finished":
                        self.sinks.pop(rid, None)
        for rid, sink in list(self.sinks.items()):
            sink.put(ReqEvent("finished", reason=reason, usage=Usage()))
        self.sinks.clear()

    def _drain_cmds(self) -> None:
        try:
            while True:
                kind, a, sink, reply = self.cmds.get_nowait()
                if kind == "submit":
                    if self.poisoned:
                        reply.put(EngineFailed(self.poisoned))
                        continue
                    try:
                        rid = self.engine.submit(a)
                    except Exception as e:      # refused (too long, malformed): the caller gets the reason
                        reply.put(e)
                        continue
                    self.sinks[rid] = sink
                    reply.put(rid)
                elif kind == "cancel" and not self.poisoned:
                    self.engine.cancel(a)
                    self.sinks.pop(a, None)
        except queue.Empty:
            pass

    def _run(self):
        last_beat = time.monotonic()
        while not self._stop.is_set():
            self._drain_cmds()
            if self.poisoned:
                self._wake.wait(self.idle_sleep)
                self._wake.clear()
                continue
            try:
                if self.engine.idle():
                    beat = getattr(self.engine, "heartbeat", None)
                    if beat is not None and time.monotonic() - last_beat >= self.heartbeat_s:
                        beat()
                        last_beat = time.monotonic()
                    self._wake.wait(self.idle_sleep)
                    self._wake.clear()
                    continue
                events = self.engine.tick()
                last_beat = time.monotonic()
            except Exception as e:
                self._fail(e)
                continue
            for rid, ev in events:
                sink = self.sinks.get(rid)
                if sink is not None:
                    sink.put(ev)
                    if ev.kind == "finished":
                        self.sinks.pop(rid, None)
            with self._stats_lock:
                self._stats = self.engine.stats()
