"""Single-sequence GLM engine: chunked prefill, one CUDA graph per decode step, MTP.

One decode step is ONE graph launch.  With MTP the graph holds the whole speculative step
-- draft pass 0 (two rows: the repaired previous pair and the new anchor), draft pass 1,
the N-row verify through the main model with GatedDeltaNet snapshots, and the device-side
accept/commit -- so the host only writes the anchor token (4 bytes) and reads back the
emitted tokens.  The reference drives the same four phases with one graph per phase and a
host accept (``crates/ferrite-exec/src/tp.rs:1839-2199``).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..config import EngineConfig, GlmConfig
from ..models.glm import GlmDeviceModel, RowSet, View
from ..serve.engine import ContextOverflow
from ..spec import SpecStep


class GlmEngine(SpecStep):
    ANCHOR_IS_IN_BLOCK = True

    def __init__(self, cfg: GlmConfig, ecfg: EngineConfig, src, rank: int = 0, world: int = 1,
                 device="cuda", allreduce=None, prefill_rows: int = 64, dcp_shard=None):
        self.cfg, self.ecfg = cfg, ecfg
        self.nv = ecfg.mtp_n if (ecfg.mtp_n > 1 and cfg.num_nextn_predict_layers > 0) else 1
        self.prefill_rows = max(prefill_rows, self.nv, 2)
        self.model = GlmDeviceModel(cfg, ecfg, src, rank, world, device, allreduce,
                                    max_rows=self.prefill_rows, n_slots=1, dcp_shard=dcp_shard)
        m, dev = self.model, self.model.dev
        H = cfg.hidden_size
        self.slot = 0
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        self.block_ids = i32(max(self.nv, 1))       # [t_last, d1..d_nd]
        self.judges = i32(self.prefill_rows)
        self.out_tokens = i32(self.nv + 1)          # [k, emitted...]
        self.mtp_ids = i32(2)
        self.mtp_h = torch.zeros(2, H, device=dev)
        self.hchain = torch.zeros(1, H, device=dev)
        self.prefill_ids = i32(self.prefill_rows)
        self.mtp_pre_ids = i32(self.prefill_rows)
        self.pin_in = torch.zeros(1, dtype=torch.int32).pin_memory() if dev.type == "cuda" else None
        self.pin_out = torch.zeros(self.nv + 1, dtype=torch.int32).pin_memory() if dev.type == "cuda" else None
        self.rs1 = m.make_rows([0], [1])
        self.rs2 = m.make_rows([0], [2])
        self.rsv = m.make_rows([0], [self.nv]) if self.nv > 1 else self.rs1
        self._rs_cache = {}
        self.graph_plain: Optional[torch.cuda.CUDAGraph] = None
        self.graph_mtp: Optional[torch.cuda.CUDAGraph] = None
        self.launches_plain = 0
        self.launches_mtp = 0
        self.n_ctx = 0
        from ..parallel.collective import startup_barrier
        startup_barrier(world, getattr(allreduce, "group", None))

    # ------------------------------------------------------------------ context limit
    def max_prompt(self) -> int:
        """Longest prompt after which one decode step still fits below the context limit."""
        return self.ecfg.max_ctx - self.nv - 3

    def room(self) -> int:
        """Positions left before the next step (nv rows, the MTP cache two ahead) would pass max_ctx."""
        return self.ecfg.max_ctx - self.n_ctx - self.nv - 2

    def _require_room(self):
        if self.room() <= 0:
            raise ContextOverflow(f"sequence of {self.n_ctx} tokens is at the context limit ({self.ecfg.max_ctx})")

    def _check_status(self):
        """Status words and guards read back with the step's tokens (see parallel/status.py)."""
        self.model.arena.verify()

    # ------------------------------------------------------------------ prefill
    def _rows(self, g: int) -> RowSet:
        if g not in self._rs_cache:
            self._rs_cache[g] = self.model.make_rows([0], [g])
        return self._rs_cache[g]

    def prefill(self, prompt: List[int]) -> int:
        """Chunked prefill of one prompt into slot 0; returns the first generated token."""
        m, cfg = self.model, self.cfg
        n = len(prompt)
        if not 2 <= n <= self.max_prompt():
            raise ContextOverflow(f"prompt of {n} tokens does not fit (2..{self.max_prompt()})")
        m.reset_slot(0)
        use_mtp = self.nv > 1
        toks = torch.tensor(prompt, dtype=torch.int32)
        C = self.prefill_rows
        for c0 in range(0, n, C):
            c1 = min(n, c0 + C)
            g = c1 - c0
            rs = self._rows(g)
            self.prefill_ids[:g].copy_(toks[c0:c1])
            last = c1 == n
            m.main_forward(rs, self.prefill_ids, snapshots=False, advance=True,
                           judges=self.judges if last else None, head_from=g - 1 if last else g)
            hf = m.ws["h_final"]
            if use_mtp:
                # MTP cache pairs (h_t, tok_{t+1}) for t < n-2; the pair n-2 is written by the first draft pass
                t_hi = min(c1, n - 2)
                if t_hi > c0:
                    gm = t_hi - c0
                    self.mtp_pre_ids[:gm].copy_(toks[c0 + 1:t_hi + 1])
                    m.mtp_forward(self._rows(gm), self.mtp_pre_ids, hf, None, advance=True)
                if g >= 2:
                    self.mtp_h[0].copy_(hf[g - 2])
                else:
                    self.mtp_h[0].copy_(self.mtp_h[1])
                self.mtp_h[1].copy_(hf[g - 1])
        first = int(self.judges[(n - 1) % C].item())
        m.arena.verify(snapshot=False)
        self.block_ids[0] = first
        if use_mtp:
            self.mtp_ids.copy_(torch.tensor([prompt[-1], first], dtype=torch.int32))
            m.mtp_len[0] = n - 2
        self.n_ctx = n
        return first

    # ------------------------------------------------------------------ graphs
    def _plain_body(self):
        m = self.model
        m.main_forward(self.rs1, self.block_ids, snapshots=False, advance=True, judges=self.out_tokens_view1)
        m.K.call("fb_copy_i32", self.out_tokens_view1, self.block_ids, 1, 1, 1)

    def _mtp_body(self):
        m, nv, H = self.model, self.nv, self.cfg.hidden_size
        # draft 0: rows (pair to repair, new anchor); head only on the anchor row -> d1
        m.mtp_forward(self.rs2, self.mtp_ids, self.mtp_h, View(self.block_ids, 1), head_from=1, advance=True)
        for d in range(1, nv - 1):
            src_row = 1 if d == 1 else 0
            self.hchain.copy_(m.ws["mtp_hout"][src_row:src_row + 1])
            m.mtp_forward(self.rs1, View(self.block_ids, d), self.hchain, View(self.block_ids, d + 1), advance=True)
        m.main_forward(self.rsv, self.block_ids, snapshots=True, advance=False, judges=self.judges)
        m.K.call("fb_mtp_accept", self.block_ids, self.judges, self.out_tokens, m.ws["h_final"], self.mtp_ids,
                 self.mtp_h, self.rsv.group_slot, m.main_len, m.mtp_len, m.cur, 1, nv, H, m.nbuf)

    @property
    def out_tokens_view1(self):
        return View(self.out_tokens, 1)

    def _capture(self, body) -> Tuple[Optional[torch.cuda.CUDAGraph], int]:
        K = self.model.K
        if not self.ecfg.use_graphs:
            return None, 0
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        l0 = K.launches
        with torch.cuda.graph(g):
            body()
        return g, K.launches - l0

    def _snapshot_state(self):
        m = self.model
        return [t.clone() for t in (m.main_len, m.mtp_len, m.cur, self.block_ids, self.mtp_ids, self.mtp_h,
                                    m.gdn_state, m.conv_state)]

    def _restore_state(self, snap):
        m = self.model
        for dst, src in zip((m.main_len, m.mtp_len, m.cur, self.block_ids, self.mtp_ids, self.mtp_h,
                             m.gdn_state, m.conv_state), snap):
            dst.copy_(src)

    def build_graphs(self, mtp: bool):
        """Capture the decode step.  Capture records without executing, so sequence state is
        untouched; kernels that need a raised shared-memory limit are run once eagerly first
        on a saved-and-restored copy of the small state."""
        if mtp and self.graph_mtp is None:
            snap = self._snapshot_state()
            self._mtp_body()
            self._restore_state(snap)
            self.graph_mtp, self.launches_mtp = self._capture(self._mtp_body)
        if not mtp and self.graph_plain is None:
            snap = self._snapshot_state()
            self._plain_body()
            self._restore_state(snap)
            self.graph_plain, self.launches_plain = self._capture(self._plain_body)

    # ------------------------------------------------------------------ stepping
    def step_plain(self, token: Optional[int] = None) -> int:
        """One greedy decode step.  ``token`` (host) overrides the device-resident anchor."""
        self._require_room()
        if token is not None:
            self.pin_in[0] = token
            self.block_ids[:1].copy_(self.pin_in, non_blocking=True)
        if self.graph_plain is not None:
            self.graph_plain.replay()
        else:
            self._plain_body()
        self.pin_out[:2].copy_(self.out_tokens[:2], non_blocking=True)
        self.model.arena.snapshot_async()
        torch.cuda.current_stream().synchronize()
        self._check_status()
        self.n_ctx += 1
        return int(self.pin_out[1])

    def spec_step(self, token: Optional[int] = None) -> List[int]:
        """One speculative step (draft -> verify -> accept -> commit); returns 1..nv tokens."""
        self._require_room()
        if token is not None:
            self.pin_in[0] = token
            self.block_ids[:1].copy_(self.pin_in, non_blocking=True)
        if self.graph_mtp is not None:
            self.graph_mtp.replay()
        else:
            self._mtp_body()
        self.pin_out.copy_(self.out_tokens, non_blocking=True)
        self.model.arena.snapshot_async()
        torch.cuda.current_stream().synchronize()
        self._check_status()
        k = int(self.pin_out[0])
        self.n_ctx += k
        return [int(t) for t in self.pin_out[1:1 + k]]

    def launch_step_async(self, mtp: bool):
        """Enqueue one step without any host round trip (device-resident token feedback)."""
        g = self.graph_mtp if mtp else self.graph_plain
        if g is not None:
            g.replay()
        elif mtp:
            self._mtp_body()
        else:
            self._plain_body()

    def generate(self, prompt: List[int], max_new: int, mtp: Optional[bool] = None,
                 stop_ids: Tuple[int, ...] = ()) -> Tuple[List[int], List[int]]:
        mtp = (self.nv > 1) if mtp is None else (mtp and self.nv > 1)
        first = self.prefill(prompt)
        self.build_graphs(mtp)
        out, accepts = [first], []
        while len(out) < max_new and out[-1] not in stop_ids and self.room() > 0:
            if mtp:
                em = self.spec_step()
                accepts.append(len(em))
                for t in em:
                    out.append(t)
                    if t in stop_ids:
                        break
            else:
                out.append(self.step_plain())
        return out[:max_new], accepts
