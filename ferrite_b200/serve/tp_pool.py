"""Replicated engine control for multi-process tensor parallelism.

Every rank owns an identical engine (same planner, same model shard layout).  Rank 0 is the
only one that talks to clients: each tick it broadcasts the commands it received since the
last tick (submit / cancel / stop), every rank applies them in the same order and runs the
same tick, and because the planner is deterministic all ranks launch the same kernels and
meet in the same collectives.  Each tick ends with an all-rank acknowledgement so that a
rank that failed is reported by every rank with its error, and a watchdog timeout bounds the
wait.  This is the process-per-GPU counterpart of the reference's ``TpRankPool`` (command
broadcast + all-rank ack collection + watchdog; ``crates/ferrite-dsv41/src/serve.rs:42-386``).
"""
from __future__ import annotations

from datetime import timedelta
from typing import List, Optional, Tuple

import torch.distributed as dist

from .engine import ReqEvent, RequestSpec


class RankFailure(RuntimeError):
    def __init__(self, errors: List[Optional[str]]):
        self.errors = errors
        bad = {r: e for r, e in enumerate(errors) if e}
        super().__init__(f"tick failed on ranks {sorted(bad)}: {bad}")


class ReplicatedEngine:
    """ServeEngine facade on rank 0; call :meth:`follow` on the other ranks."""

    def __init__(self, engine, rank: int, world: int, control_group=None):
        self.engine, self.rank, self.world = engine, rank, world
        self.group = control_group  # a gloo group keeps control traffic off the GPU streams
        self.pending: List[Tuple[str, object]] = []
        self.local_ids = 0
        self.poisoned: Optional[str] = None

    # ---- rank 0 side (ServeEngine protocol) ---------------------------------------------
    def submit(self, spec: RequestSpec) -> int:
        assert self.rank == 0
        validate = getattr(self.engine, "validate", None)
        if validate is not None:
            validate(spec)   # refuse on rank 0, before the command reaches the other ranks
        self.pending.append(("submit", (list(spec.prompt_ids), spec.max_new_tokens, tuple(spec.stop_ids))))
        # ids are assigned by the deterministic planner in submit order: predict it
        self.local_ids += 1
        return self.local_ids

    def cancel(self, req: int) -> None:
        assert self.rank == 0
        self.pending.append(("cancel", req))

    def idle(self) -> bool:
        return not self.pending and self.engine.idle()

    def stats(self) -> dict:
        return self.engine.stats()

    def tick(self) -> List[Tuple[int, ReqEvent]]:
        cmds, self.pending = self.pending, []
        return self._round(cmds)

    def stop(self) -> None:
        if self.rank == 0:
            self._round([("stop", None)])

    def heartbeat(self) -> None:
        """An empty round: keeps the followers' blocking broadcast (and the control group's watchdog) alive
        while rank 0 has nothing to do."""
        if self.rank == 0 and self.world > 1:
            self._round([("beat", None)])

    def take_pending_events(self):
        """Events the engine produced in the tick that failed (the driver still delivers them)."""
        ev = getattr(self.engine, "pending_events", None) or []
        if hasattr(self.engine, "pending_events"):
            self.engine.pending_events = []
        return ev

    # ---- follower side -------------------------------------------------------------------
    def follow(self) -> None:
        """Run ticks driven by rank 0 until it sends stop."""
        assert self.rank != 0
        while self._round(None) is not None:
            pass

    # ---- one replicated tick -------------------------------------------------------------
    def _round(self, cmds):
        box = [cmds]
        if self.world > 1:
            dist.broadcast_object_list(box, src=0, group=self.group)
        cmds = box[0]
        stop = False
        err: Optional[str] = None
        out: List[Tuple[int, ReqEvent]] = []
        try:
            for kind, arg in cmds:
                if kind == "submit":
                    p, mx, st = arg
                    self.engine.submit(RequestSpec(p, mx, st))
                elif kind == "cancel":
                    self.engine.cancel(arg)
                elif kind == "stop":
                    stop = True
            if not stop and not self.engine.idle():
                out = self.engine.tick()
        except Exception as e:  # report, do not desynchronise the ranks
            err = f"{type(e).__name__}: {e}"
        if self.world > 1:
            errs: List[Optional[str]] = [None] * self.world
            dist.all_gather_object(errs, err, group=self.group)
        else:
            errs = [err]
        if any(errs):
            # every rank saw the same list: all of them drop the request in flight together
            abort = getattr(self.engine, "abort_current", None)
            if abort is not None:
                abort("error:RankFailure", [])
            self.poisoned = str(errs)
            raise RankFailure(errs)
        if stop:
            return None
        return out


def make_control_group(timeout_s: float = 1800.0):
    """A gloo group for the command broadcast / acks with the watchdog timeout."""
    return dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_s))
