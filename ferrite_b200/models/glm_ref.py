"""fp32 PyTorch reference engine for GLM-5.3-Flash (CPU-capable oracle).

It executes the whole model -- MHC residual streams, GatedDeltaNet layers, DSA layers with
the k-pool indexer, dense and MoE FFNs, the MTP layer and the speculative loop -- with the
plain ops of :mod:`ferrite_b200.ops.reference`.  Tensor parallelism is simulated in-process:
``world`` weight shards run one after another and their partial sums are added, which is how
the reference proves ``tpN == tp1`` without a cluster
(``crates/ferrite-exec/src/tp.rs:520-535,4317-4436``).  The layer math follows
``crates/ferrite-exec/src/lib.rs:345-1166`` and the MTP layer ``tp.rs:5320-5500``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import GlmConfig
from ..ops import reference as R
from ..spec import spec_accept
from .glm_weights import Weights, shard_weights_tp


@dataclass
class DsaCache:
    k: List[torch.Tensor] = field(default_factory=list)  # per rank [T,h_loc,dk]
    v: List[torch.Tensor] = field(default_factory=list)
    kidx: Optional[torch.Tensor] = None  # [T,D] replicated
    kgate: Optional[torch.Tensor] = None
    length: int = 0


@dataclass
class SeqState:
    conv: Dict[int, List[torch.Tensor]] = field(default_factory=dict)  # layer -> per rank [ch,k-1]
    gdn: Dict[int, List[torch.Tensor]] = field(default_factory=dict)  # layer -> per rank [h,dk,dv]
    dsa: Dict[int, DsaCache] = field(default_factory=dict)  # family -> cache
    tokens: List[int] = field(default_factory=list)
    n_ctx: int = 0
    h_prev: Optional[torch.Tensor] = None  # [H] MTP seed (pre-norm contracted residual)

    def clone(self) -> "SeqState":
        s = SeqState(tokens=list(self.tokens), n_ctx=self.n_ctx,
                     h_prev=None if self.h_prev is None else self.h_prev.clone())
        s.conv = {k: [t.clone() for t in v] for k, v in self.conv.items()}
        s.gdn = {k: [t.clone() for t in v] for k, v in self.gdn.items()}
        for f, c in self.dsa.items():
            s.dsa[f] = DsaCache([t.clone() for t in c.k], [t.clone() for t in c.v],
                                None if c.kidx is None else c.kidx.clone(),
                                None if c.kgate is None else c.kgate.clone(), c.length)
        return s


class GlmReference:
    def __init__(self, cfg: GlmConfig, weights: Weights, world: int = 1, use_wy: bool = False):
        self.cfg = cfg
        self.world = world
        self.use_wy = use_wy
        self.trace = None  # set to a list to record (layer, site, R, y) after every sublayer
        self.shards = [shard_weights_tp({k: v.float() for k, v in weights.items()}, r, world)
                       for r in range(world)]
        self.full = self.shards[0]  # replicated tensors are read from shard 0

    # ---- helpers -----------------------------------------------------------
    def _sum(self, fn):
        """Simulated all-reduce: sum of the per-rank partial results."""
        out = None
        for r in range(self.world):
            p = fn(r, self.shards[r])
            out = p if out is None else out + p
        return out

    def new_seq(self) -> SeqState:
        return SeqState()

    # ---- linear attention ---------------------------------------------------
    def _linear_attn(self, st: SeqState, layer: int, pfx: str, x: torch.Tensor) -> torch.Tensor:
        cfg, la = self.cfg, self.cfg.linear_attn
        n = x.shape[0]
        a = f"{pfx}.self_attn"

        def rank_fn(r, w):
            h = la.num_heads // self.world
            dk = la.head_dim
            P = h * dk
            qkv = R.linear(x, w[f"{a}.qkv_proj.weight"])
            b = R.linear(x, w[f"{a}.b_proj.weight"])
            fb = R.linear(R.linear(x, w[f"{a}.f_a_proj.weight"]), w[f"{a}.f_b_proj.weight"])
            gb = R.linear(R.linear(x, w[f"{a}.g_a_proj.weight"]), w[f"{a}.g_b_proj.weight"])
            conv_st = st.conv.setdefault(layer, [None] * self.world)
            if conv_st[r] is None:
                conv_st[r] = torch.zeros(3 * P, la.conv_kernel - 1)
            co, conv_st[r] = R.causal_conv1d(qkv, w[f"{a}.qkv_conv1d.weight"], conv_st[r])
            co = torch.nn.functional.silu(co)
            q, k, v = (co[:, i * P:(i + 1) * P].reshape(n, h, dk) for i in range(3))
            q = R.l2norm_heads(q) * dk ** -0.5
            k = R.l2norm_heads(k)
            beta = torch.sigmoid(b)
            g = R.gdn_log_decay(fb, w[f"{a}.dt_bias"], w[f"{a}.A_log"], la.gate_lower_bound, h)
            gs = st.gdn.setdefault(layer, [None] * self.world)
            if gs[r] is None:
                gs[r] = torch.zeros(h, dk, dk)
            if self.use_wy and n > 1:
                core, gs[r] = R.gdn_chunk_wy(q, k, v, beta, g, gs[r], la.chunk)
            else:
                core, gs[r] = R.gdn_recurrent(q, k, v, beta, g, gs[r])
            normed = R.gated_rmsnorm(core, gb.view(n, h, dk), w[f"{a}.o_norm.weight"], cfg.rms_norm_eps)
            return R.linear(normed.reshape(n, P), w[f"{a}.o_proj.weight"])

        return self._sum(rank_fn)

    # ---- DSA attention -------------------------------------------------------
    def _dsa_attn(self, st: SeqState, layer: int, pfx: str, x: torch.Tensor) -> torch.Tensor:
        cfg, ds = self.cfg, self.cfg.dsa
        n = x.shape[0]
        a = f"{pfx}.self_attn"
        w0 = self.full
        fam = cfg.dsa_family(layer)
        cache = st.dsa.setdefault(fam, DsaCache())
        ih, idm, kpool = ds.index_n_heads, ds.index_head_dim, ds.index_kpool
        qa = R.rmsnorm(R.linear(x, w0[f"{a}.q_a_proj.weight"]), w0[f"{a}.q_a_layernorm.weight"], cfg.rms_norm_eps)
        latent = R.rmsnorm(R.linear(x, w0[f"{a}.kv_a_proj_with_mqa.weight"]),
                           w0[f"{a}.kv_a_layernorm.weight"], cfg.rms_norm_eps)
        qi = R.linear(qa, w0[f"{a}.indexer.wq_b.weight"]).view(n, ih, idm)
        ki = R.layernorm_affine(R.linear(x, w0[f"{a}.indexer.wk.weight"]), w0[f"{a}.indexer.k_norm.weight"],
                                w0[f"{a}.indexer.k_norm.bias"], cfg.rms_norm_eps)
        wi = R.linear(x, w0[f"{a}.indexer.weights_proj.weight"]) * ih ** -0.5
        kg = R.linear(x, w0[f"{a}.indexer.index_kpool_compress_gate"])
        cache.kidx = ki if cache.kidx is None else torch.cat([cache.kidx[:cache.length], ki], 0)
        cache.kgate = kg if cache.kgate is None else torch.cat([cache.kgate[:cache.length], kg], 0)
        ctx0 = cache.length
        total = ctx0 + n
        pool_keys = R.kpool_compress(cache.kidx, cache.kgate, w0[f"{a}.indexer.index_kpool_compress_ape"], kpool)
        npools = pool_keys.shape[0]
        select_k = min(ds.index_topk // kpool, npools)
        pool_idx = R.indexer_topk(qi, pool_keys, wi, select_k, ctx0 // kpool)
        width = select_k * kpool + (kpool - 1)
        idx = R.expand_pool_indices(pool_idx, kpool, ctx0, total, width)
        if not cache.k:
            cache.k, cache.v = [None] * self.world, [None] * self.world

        def rank_fn(r, w):
            h = ds.num_heads // self.world
            dk, dv = ds.qk_nope_head_dim, ds.v_head_dim
            q = R.linear(qa, w[f"{a}.q_b_proj.weight"]).view(n, h, dk)
            kvb = R.linear(latent, w[f"{a}.kv_b_proj.weight"]).view(n, h, dk + dv)
            kn, vn = kvb[..., :dk], kvb[..., dk:]
            cache.k[r] = kn if cache.k[r] is None else torch.cat([cache.k[r][:ctx0], kn], 0)
            cache.v[r] = vn if cache.v[r] is None else torch.cat([cache.v[r][:ctx0], vn], 0)
            o = R.sparse_mla_attn(q, cache.k[r], cache.v[r], idx)
            return R.linear(o.reshape(n, h * dv), w[f"{a}.o_proj.weight"])

        out = self._sum(rank_fn)
        cache.length = total
        return out

    # ---- FFN ------------------------------------------------------------------
    def _dense_ffn(self, pfx: str, x: torch.Tensor) -> torch.Tensor:
        lim = self.cfg.swiglu_limit
        return self._sum(lambda r, w: R.expert_ffn(
            x, w[f"{pfx}.mlp.gate_proj.weight"], w[f"{pfx}.mlp.up_proj.weight"],
            w[f"{pfx}.mlp.down_proj.weight"], lim))

    def _moe_ffn(self, pfx: str, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        lim = cfg.swiglu_limit
        w0 = self.full
        wts, ids = R.moe_route(R.linear(x, w0[f"{pfx}.mlp.gate.weight"]),
                               w0[f"{pfx}.mlp.gate.e_score_correction_bias"],
                               cfg.num_experts_per_tok, cfg.routed_scaling_factor)

        def rank_fn(r, w):
            out = R.expert_ffn(x, w[f"{pfx}.mlp.shared_expert.gate_proj.weight"],
                               w[f"{pfx}.mlp.shared_expert.up_proj.weight"],
                               w[f"{pfx}.mlp.shared_expert.down_proj.weight"], lim)
            for e in ids.unique().tolist():
                rows, slots = (ids == e).nonzero(as_tuple=True)
                y = R.expert_ffn(x[rows], w[f"{pfx}.mlp.experts.{e}.gate_proj.weight"],
                                 w[f"{pfx}.mlp.experts.{e}.up_proj.weight"],
                                 w[f"{pfx}.mlp.experts.{e}.down_proj.weight"], lim)
                out.index_add_(0, rows, y * wts[rows, slots].unsqueeze(1))
            return out

        return self._sum(rank_fn)

    # ---- whole model ------------------------------------------------------------
    def _attn(self, st, i, pfx, x):
        return self._dsa_attn(st, i, pfx, x) if self.cfg.is_dsa(i) else self._linear_attn(st, i, pfx, x)

    def _ffn(self, i, pfx, x):
        return self._moe_ffn(pfx, x) if self.cfg.is_moe(i) else self._dense_ffn(pfx, x)

    def forward(self, st: SeqState, tokens: List[int]):
        """Run ``tokens`` through the main model, appending to the sequence state.
        Returns (logits [n,V], h_final [n,H])."""
        cfg, w = self.cfg, self.full
        ids = torch.as_tensor(tokens, dtype=torch.long)
        h0 = w["model.embed_tokens.weight"][ids]
        eps = cfg.rms_norm_eps
        if cfg.mhc:
            Rs = R.hc_expand(h0, cfg.hc_mult)
        else:
            Rs = h0
        for i in range(cfg.num_layers):
            pfx = f"model.layers.{i}"
            if cfg.mhc:
                x, post, comb = R.hc_pre(Rs, w[f"{pfx}.hc_attn_fn"], w[f"{pfx}.hc_attn_scale"],
                                         w[f"{pfx}.hc_attn_base"], eps, cfg.hc_eps, cfg.hc_sinkhorn_iters)
                y = self._attn(st, i, pfx, R.rmsnorm(x, w[f"{pfx}.input_layernorm.weight"], eps))
                Rs = R.hc_post(y, Rs, post, comb)
                if self.trace is not None:
                    self.trace.append((i, "attn", Rs.clone(), y.clone()))
                x, post, comb = R.hc_pre(Rs, w[f"{pfx}.hc_ffn_fn"], w[f"{pfx}.hc_ffn_scale"],
                                         w[f"{pfx}.hc_ffn_base"], eps, cfg.hc_eps, cfg.hc_sinkhorn_iters)
                y = self._ffn(i, pfx, R.rmsnorm(x, w[f"{pfx}.post_attention_layernorm.weight"], eps))
                Rs = R.hc_post(y, Rs, post, comb)
                if self.trace is not None:
                    self.trace.append((i, "ffn", Rs.clone(), y.clone()))
            else:
                Rs = Rs + self._attn(st, i, pfx, R.rmsnorm(Rs, w[f"{pfx}.input_layernorm.weight"], eps))
                Rs = Rs + self._ffn(i, pfx, R.rmsnorm(Rs, w[f"{pfx}.post_attention_layernorm.weight"], eps))
        hf = R.hc_contract(Rs) if cfg.mhc else Rs
        logits = R.linear(R.rmsnorm(hf, w["model.norm.weight"], eps), w["lm_head.weight"])
        st.n_ctx += len(tokens)
        return logits, hf

    def mtp_forward(self, st: SeqState, tokens: List[int], h_prev: torch.Tensor):
        """One pass of the MTP layer over rows (token_i, h_prev_i).  Returns (logits, h_out)."""
        cfg, w = self.cfg, self.full
        L = cfg.num_layers
        pfx = f"model.layers.{L}"
        eps = cfg.rms_norm_eps
        ids = torch.as_tensor(tokens, dtype=torch.long)
        e = R.rmsnorm(w["model.embed_tokens.weight"][ids], w[f"{pfx}.enorm.weight"], eps)
        hp = R.rmsnorm(h_prev.view(len(tokens), -1), w[f"{pfx}.hnorm.weight"], eps)
        z = R.linear(torch.cat([e, hp], -1), w[f"{pfx}.eh_proj.weight"])
        x1 = z + self._dsa_attn(st, L, pfx, R.rmsnorm(z, w[f"{pfx}.input_layernorm.weight"], eps))
        x2 = x1 + self._moe_ffn(pfx, R.rmsnorm(x1, w[f"{pfx}.post_attention_layernorm.weight"], eps))
        logits = R.linear(R.rmsnorm(x2, w[f"{pfx}.shared_head.norm.weight"], eps), w["lm_head.weight"])
        return logits, x2

    # ---- generation --------------------------------------------------------------
    def prefill(self, st: SeqState, prompt: List[int], chunk: int = 0, with_mtp: bool = False) -> int:
        """Chunked prefill; returns the first generated token."""
        chunk = chunk or len(prompt)
        hs = []
        logits = None
        for c0 in range(0, len(prompt), chunk):
            logits, hf = self.forward(st, prompt[c0:c0 + chunk])
            hs.append(hf)
        st.tokens = list(prompt)
        hf = torch.cat(hs, 0)
        st.h_prev = hf[-1].clone()
        if with_mtp and self.cfg.num_nextn_predict_layers and len(prompt) > 1:
            self.mtp_forward(st, prompt[1:], hf[:-1])
        return int(R.argmax_first(logits[-1:])[0])

    def decode_greedy(self, st: SeqState, first: int, steps: int) -> List[int]:
        out = [first]
        for _ in range(steps - 1):
            logits, hf = self.forward(st, [out[-1]])
            st.h_prev = hf[-1]
            out.append(int(R.argmax_first(logits)[0]))
        return out

    def _rollback(self, st: SeqState, snap: SeqState, keep_tokens: List[int]):
        """Restore recurrent state from ``snap`` and replay the accepted tokens (the oracle
        does by replay what the device does with per-token snapshots + one commit kernel)."""
        st.conv, st.gdn = snap.conv, snap.gdn
        nmain = self.cfg.n_dsa_families - self.cfg.num_nextn_predict_layers
        for f, c in st.dsa.items():
            if f < nmain:
                c.length = snap.dsa[f].length
        st.n_ctx = snap.n_ctx
        if keep_tokens:
            return self.forward(st, keep_tokens)
        return None

    def mtp_step(self, st: SeqState, t_last: int, n_verify: int = 3):
        """draft(nd) -> verify(block) -> accept -> commit.  Returns (emitted tokens, accept k)."""
        cfg = self.cfg
        nd = n_verify - 1
        fam = cfg.dsa_family(cfg.num_layers)
        mtp_len0 = st.dsa[fam].length if fam in st.dsa else 0
        drafts, tok, hp = [], t_last, st.h_prev
        for _ in range(nd):
            lg, hp = self.mtp_forward(st, [tok], hp)
            hp = hp[0]
            tok = int(R.argmax_first(lg)[0])
            drafts.append(tok)
        block = [t_last] + drafts
        snap = st.clone()
        logits, hf = self.forward(st, block)
        judges = [int(t) for t in R.argmax_first(logits)]
        k = spec_accept(drafts, judges, anchor_is_in_block=True)
        emitted = judges[:k]
        if k < n_verify:
            _, hf2 = self._rollback(st, snap, block[:k])
            st.h_prev = hf2[-1]
        else:
            st.h_prev = hf[k - 1]
        # MTP cache keeps pairs (h_t, tok_{t+1}) for every main position but the newest
        c = st.dsa[fam]
        want = mtp_len0 + k
        if c.length > want:
            c.length = want
        elif c.length < want:  # every draft accepted: fill the one missing pair
            self.mtp_forward(st, [block[-1]], hf[k - 2])
        return emitted, k

    def generate(self, prompt: List[int], steps: int, chunk: int = 0, mtp: bool = False,
                 n_verify: int = 3):
        st = self.new_seq()
        first = self.prefill(st, prompt, chunk, with_mtp=mtp)
        if not mtp:
            return self.decode_greedy(st, first, steps), None
        out, accepts = [first], []
        while len(out) < steps:
            em, k = self.mtp_step(st, out[-1], n_verify)
            out.extend(em)
            accepts.append(k)
        return out[:steps], accepts
