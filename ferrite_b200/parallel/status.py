"""One arena per device for the words that device-side protocols report through or count with.

Every kernel with a bounded wait ends in a four-int status word (``FB_TIMEOUT`` + peer, epoch, chunk),
every peer-memory collective keeps epoch and ticket counters, and the row-metadata kernel reports a
sequence that ran into the context limit (``FB_BAD_ARG``).  These words used to be separate small
tensors that only tests read.  Here they are slices of ONE int32 buffer, each slice fenced by guard
words on both sides, so that

* an engine copies the whole arena (a few KB) to pinned host memory in the same stream as the step's
  result and checks it after the synchronise it already pays for: a timed-out wait, a clamped position
  or an overwritten guard raises on the step that caused it instead of yielding wrong tokens;
* a stray store next to an epoch / ticket / status block shows up as ``FB_BAD_CANARY`` (the reference
  keeps canaries around its signal pads for the same reason,
  ``crates/ferrite-models/src/dsv41/tp.rs:306-358``).

``make_allreduce`` creates one arena and hands it to every collective of a rank; the device model takes
its own words from the same arena (or creates a private one when it runs without collectives).  The arena
works on CPU tensors too, which is how the guard logic is tested without a GPU.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

FB_OK, FB_TIMEOUT, FB_BAD_CANARY, FB_BAD_ARG = 0, 1, 2, 3
CANARY = 0x5AFEC0DE
GUARD_WORDS = 4   # keeps every payload 16-byte aligned


class CollectiveTimeout(RuntimeError):
    def __init__(self, peer: int, epoch: int, chunk: int, name: str = ""):
        super().__init__(f"{name or 'collective'}: bounded wait ran out (peer {peer}, epoch {epoch}, chunk {chunk})")
        self.peer, self.epoch, self.chunk, self.name = peer, epoch, chunk, name


class CanaryError(RuntimeError):
    def __init__(self, name: str, word: int, value: int):
        super().__init__(f"guard word {word} next to '{name}' was overwritten (now {value:#x})")
        self.name, self.word, self.value, self.code = name, word, value, FB_BAD_CANARY


class ContextGuard(RuntimeError):
    def __init__(self, slot: int, length: int, rows: int, name: str = ""):
        super().__init__(f"{name or 'rows'}: slot {slot} at length {length} + {rows} rows ran past the context limit; "
                         "positions were clamped on the device")
        self.slot, self.length, self.rows, self.code = slot, length, rows, FB_BAD_ARG


class StatusArena:
    def __init__(self, device, words: int = 16384):
        self.dev = torch.device(device)
        self.buf = torch.zeros(words, dtype=torch.int32, device=self.dev)
        self.used = 0
        self.entries: List[Tuple[str, str, int, int]] = []      # (name, kind, offset, n)
        self.pin: Optional[torch.Tensor] = None
        self._status_rows: Optional[torch.Tensor] = None
        self._guard_idx: Optional[torch.Tensor] = None

    def take(self, n: int, name: str, kind: str = "counter") -> torch.Tensor:
        """A zeroed ``n``-int slice fenced by guard words.  kind "status": a four-int status word that
        :meth:`verify` interprets; "counter": epochs / tickets, only their guards are checked."""
        n4 = (n + 3) // 4 * 4
        need = n4 + 2 * GUARD_WORDS
        if self.used + need > self.buf.numel():
            raise RuntimeError("status arena full")
        o = self.used
        self.buf[o:o + GUARD_WORDS] = CANARY
        self.buf[o + GUARD_WORDS + n4:o + need] = CANARY
        self.used += need
        self.entries.append((name, kind, o + GUARD_WORDS, n))
        self._status_rows = self._guard_idx = None
        return self.buf[o + GUARD_WORDS:o + GUARD_WORDS + n]

    def status(self, name: str) -> torch.Tensor:
        return self.take(4, name, "status")

    # ---- host side --------------------------------------------------------------------------------
    def _index(self):
        if self._guard_idx is None:
            g, s = [], []
            for _, kind, o, n in self.entries:
                n4 = (n + 3) // 4 * 4
                g += [o - 2, o - 1, o + n4, o + n4 + 1]   # the two guard words nearest the payload on each side
                if kind == "status":
                    s.append(o)
            self._guard_idx = torch.tensor(g, dtype=torch.long)
            self._status_rows = torch.tensor(s, dtype=torch.long)
        return self._guard_idx, self._status_rows

    def snapshot_async(self) -> None:
        """Enqueue the copy of the arena to pinned host memory on the current stream (no synchronise)."""
        if self.dev.type != "cuda":
            return
        if self.pin is None or self.pin.numel() != self.buf.numel():
            self.pin = torch.zeros(self.buf.numel(), dtype=torch.int32).pin_memory()
        self.pin[:self.used].copy_(self.buf[:self.used], non_blocking=True)
        self._snap_used = self.used

    def verify(self, snapshot: bool = True, clear: bool = True) -> None:
        """Check guards and status words; raises the first problem found.  With ``snapshot`` the copy
        made by :meth:`snapshot_async` is read (the caller has synchronised the stream since); otherwise
        the device buffer is read now (synchronises)."""
        fresh = snapshot and self.pin is not None and getattr(self, "_snap_used", -1) == self.used
        host = self.pin if fresh else self.buf.cpu()
        gi, si = self._index()
        if gi.numel() and bool((host[gi] != CANARY).any()):
            bad = int((host[gi] != CANARY).nonzero()[0])
            word = int(gi[bad])
            name = self.entries[bad // 4][0]
            value = int(host[word]) & 0xFFFFFFFF
            if clear:
                self.buf[word] = CANARY
            raise CanaryError(name, word, value)
        if si.numel() == 0:
            return
        codes = host[si]
        if not bool(codes.any()):
            return
        k = int(codes.nonzero()[0])
        o = int(si[k])
        name = [e for e in self.entries if e[1] == "status"][k][0]
        code, a, b, c = (int(v) for v in host[o:o + 4])
        if clear:
            self.buf[o:o + 4] = 0
        if code == FB_TIMEOUT:
            raise CollectiveTimeout(a, b, c, name)
        if code == FB_BAD_ARG:
            raise ContextGuard(a, b, c, name)
        raise RuntimeError(f"{name}: device status {code} ({a}, {b}, {c})")

    def clear(self) -> None:
        for _, kind, o, _n in self.entries:
            if kind == "status":
                self.buf[o:o + 4] = 0
