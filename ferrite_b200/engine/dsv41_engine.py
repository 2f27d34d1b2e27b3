"""Single-sequence DSV41 engine: chunked prefill, graph-replayed decode, DSpark speculation.

Counterpart of the reference's ``DevChain::step`` / ``dspark_spec_step``
(``crates/ferrite-models/src/dsv41/chain_dev.rs:8875-9017,11629-11673``):

* ``prefill`` feeds the prompt in chunks of ``max_rows`` rows through the same row-batched
  forward that decode uses (the reference prefills one token per forward);
* ``step_plain`` replays one captured CUDA graph per token - the token id, the sequence
  length and every cache cursor live on the device;
* ``spec_step`` = draft block (DSpark layers over the main model's KV) -> ``B + 1``-row verify
  -> accept on the shared chain (``anchor_is_in_block = False``) -> commit.  Commit is a
  length update: caches are position-indexed and the window ring holds ``window + rows``
  entries, so rejected rows are overwritten by the next forward and nothing is copied back
  (the reference snapshots and restores the KV ring and replays the compressor).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..config import EngineConfig
from ..models.dsv41 import Dsv41DeviceModel
from ..models.dsv41_config import Dsv41Config
from ..serve.engine import ContextOverflow
from ..spec import SpecStep, spec_accept


class Dsv41Engine(SpecStep):
    ANCHOR_IS_IN_BLOCK = False

    def __init__(self, cfg: Dsv41Config, src, rank: int = 0, world: int = 1, device="cuda", allreduce=None,
                 max_ctx: int = 1024, use_graphs: bool = True, max_rows: int = 8):
        self.cfg = cfg
        self.model = Dsv41DeviceModel(cfg, src, rank, world, device, allreduce, max_rows=max_rows, max_ctx=max_ctx)
        self.dev = self.model.dev
        self.use_graphs = use_graphs
        self.tok = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.rs1 = self.model.make_rows([0], [1])
        B = cfg.dspark_block_size
        self.has_spec = bool(self.model.mtp)
        if self.has_spec:
            assert B + 1 <= max_rows
            self.rs_draft = self.model.make_rows([0], [B])
            self.rs_verify = self.model.make_rows([0], [B + 1])
        self.graph_plain: Optional[torch.cuda.CUDAGraph] = None
        self.graph_draft: Optional[torch.cuda.CUDAGraph] = None
        self.graph_verify: Optional[torch.cuda.CUDAGraph] = None
        self.pos = 0
        self.accept_hist: List[int] = []
        from ..parallel.collective import startup_barrier
        startup_barrier(world, getattr(allreduce, "group", None))

    # ---- context limit -----------------------------------------------------------------------------
    def _step_rows(self) -> int:
        return (self.cfg.dspark_block_size + 1) if self.has_spec else 1

    def max_prompt(self) -> int:
        return self.model.max_ctx - self._step_rows() - 3

    def room(self) -> int:
        """Positions left before the next (speculative) step would write past max_ctx."""
        return self.model.max_ctx - self.pos - self._step_rows() - 2

    def _require_room(self):
        if self.room() <= 0:
            raise ContextOverflow(f"sequence of {self.pos} tokens is at the context limit ({self.model.max_ctx})")

    # ---- prefill -----------------------------------------------------------------------------------
    def prefill(self, prompt: Sequence[int], start: int = 0) -> int:
        """Prefill prompt[start:] on top of `start` positions that are already in the caches."""
        if not 1 <= len(prompt) <= self.max_prompt():
            raise ContextOverflow(f"prompt of {len(prompt)} tokens does not fit (1..{self.max_prompt()})")
        m = self.model
        if start == 0:
            m.reset_slot(0)
        self.pos = start
        ids = torch.tensor(list(prompt), dtype=torch.int32, device=self.dev)
        step = m.max_rows
        for i in range(start, len(prompt), step):
            c = ids[i:i + step]
            rs = m.make_rows([0], [c.numel()])
            last = i + step >= len(prompt)
            m.forward(rs, c, advance=True, want_logits=last)
            if self.has_spec:
                m.dspark_seed(rs)
            if last:
                self.tok.copy_(m.ws["out_ids"][c.numel() - 1:c.numel()])
        self.pos = len(prompt)
        first = int(self.tok.item())
        m.arena.verify(snapshot=False)
        return first

    # ---- plain decode ------------------------------------------------------------------------------
    def _plain_body(self):
        m = self.model
        m.forward(self.rs1, self.tok, advance=True)
        if self.has_spec:
            m.dspark_seed(self.rs1)
        self.tok.copy_(m.ws["out_ids"][0:1])

    def step_plain(self) -> int:
        self._require_room()
        if not self.use_graphs:
            self._plain_body()
        elif self.graph_plain is None:
            self._plain_body()   # a real step doubles as the warm-up; the next call captures
            self.graph_plain = False
        elif self.graph_plain is False:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._plain_body()
            self.graph_plain = g
            g.replay()
        else:
            self.graph_plain.replay()
        self.pos += 1
        self.model.arena.snapshot_async()
        tok = int(self.tok.item())
        self.model.arena.verify()
        return tok

    def launch_plain_async(self) -> None:
        """Replay the decode graph without reading the token back (for timing loops)."""
        assert isinstance(self.graph_plain, torch.cuda.CUDAGraph)
        self.graph_plain.replay()
        self.pos += 1

    # ---- speculative decode ------------------------------------------------------------------------
    def _run(self, which: str, body):
        g = getattr(self, which)
        if not self.use_graphs:
            body()
        elif g is None:
            body()
            setattr(self, which, False)
        elif g is False:
            torch.cuda.synchronize()
            ng = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ng):
                body()
            setattr(self, which, ng)
            ng.replay()
        else:
            g.replay()

    def spec_step(self) -> List[int]:
        assert self.has_spec
        self._require_room()
        m, B = self.model, self.cfg.dspark_block_size
        self._run("graph_draft", lambda: m.dspark_draft(self.rs_draft, self.tok))
        self._run("graph_verify", lambda: m.forward(self.rs_verify, m.ws["d_out"], advance=False))
        m.arena.snapshot_async()
        block = m.ws["d_out"].tolist()                   # [t0, d1..dB]   (one sync per step)
        m.arena.verify()
        judges = m.ws["out_ids"][:B + 1].tolist()
        n_acc = spec_accept(block[1:], judges, anchor_is_in_block=False)
        k = n_acc + 1                                    # verify rows that stay: t0 + accepted drafts
        emitted = judges[:k]                             # accepted drafts + the bonus token
        m.dspark_seed(self.rs_verify, 0, k)              # main KV of the kept rows for the next draft
        m.seq_len[0:1] += k
        self.tok.copy_(m.ws["out_ids"][n_acc:n_acc + 1])
        self.pos += k
        self.accept_hist.append(k)
        return emitted

    # ---- generation --------------------------------------------------------------------------------
    def generate(self, prompt: Sequence[int], n_new: int, spec: bool = False) -> List[int]:
        out = [self.prefill(prompt)]
        while len(out) < n_new and self.room() > 0:
            if spec:
                out += self.spec_step()
            else:
                out.append(self.step_plain())
        return out[:n_new]


class Dsv41StepEngine:
    """``StepEngine`` over :class:`Dsv41Engine` with a host-snapshot prefix cache (LRU): a prompt whose
    beginning equals a cached prompt resumes from that snapshot and prefills only the rest
    (reference ``crates/ferrite-dsv41/src/serve.rs:934-1039``, ``prefill_or_resume``)."""

    def __init__(self, engine: Dsv41Engine, spec: bool = True, cache_entries: int = 4):
        self.eng = engine
        self.spec = spec and engine.has_spec
        self.cache_entries = cache_entries
        self.cache: List[tuple] = []     # (prompt tuple, snapshot), most recent last
        self.hits = self.misses = 0

    def _lookup(self, prompt: Sequence[int]):
        best = None
        for key, snap in self.cache:
            if len(key) < len(prompt) and tuple(prompt[:len(key)]) == key and (best is None or len(key) > len(best[0])):
                best = (key, snap)
        return best

    def start(self, prompt: List[int]):
        hit = self._lookup(prompt)
        cached = 0
        if hit is not None:
            self.eng.model.restore_slot(hit[1])
            cached = len(hit[0])
            self.hits += 1
        else:
            self.misses += 1
        first = self.eng.prefill(prompt, start=cached)
        if self.cache_entries:
            self.cache = [(k, s) for k, s in self.cache if k != tuple(prompt)]
            self.cache.append((tuple(prompt), self.eng.model.snapshot_slot()))
            del self.cache[:-self.cache_entries]
        return first, cached

    def step(self) -> List[int]:
        return self.eng.spec_step() if self.spec else [self.eng.step_plain()]

    def max_prompt(self) -> int:
        return self.eng.max_prompt()

    def room(self) -> int:
        return self.eng.room()
