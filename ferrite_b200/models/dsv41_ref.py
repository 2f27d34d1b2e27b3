"""fp32 golden model of the DSV41 family (CPU, plain PyTorch).

One sequence at a time, any chunking: ``forward(state, ids)`` appends ``len(ids)`` positions
to the sequence and returns the logits of every row, so prefill, chunked prefill, decode and
multi-row verify are the same call.  The golden keeps the *whole* KV history per layer and
derives each row's visible set from its position (sliding window of ``window_size`` rows,
``(pos+1)//ratio`` compressed rows); a ring buffer is a device-side storage choice that must
reproduce the same sets.  Semantics: ``ref_inference/model.py`` (Transformer.forward
``:1242-1272``, Block ``:968-994``, Attention ``:613-789``, Compressor ``:429-485``, Indexer
``:488-580``, candidate blocks ``:583-610``, MoE ``:792-904``, Engram ``:296-365``, DSpark
``:1020-1156``) and ``sparse_attn`` (``ref_inference/kernel.py:311-403``); the speculative
verify/accept loop follows ``crates/ferrite-models/src/dsv41/dspark_dev.rs``.

Structural quantisation round trips are part of the model and are reproduced here: fp8
activations per 32 in front of every quantised weight, the window KV in fp8 per 32, the
compressed KV in fp4 per 16 with e4m3 scales, indexer q/k in fp4 per 32.  bf16 roundings of
the reference's intermediate tensors are not (everything else is f32).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops import quant as Q
from ..ops import reference as R
from ..spec import spec_accept
from .dsv41_config import Dsv41Config
from .dsv41_engram import EngramLayout, NgramHasher
from .dsv41_weights import tensor_specs


def rope_freqs(dim: int, base: float, original_seq_len: int, factor: float, beta_fast: float, beta_slow: float) -> torch.Tensor:
    """Per-pair angular frequencies [dim/2]; YaRN blending when original_seq_len > 0."""
    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if original_seq_len > 0:
        def corrected(rot):
            return dim * math.log(original_seq_len / (rot * 2 * math.pi)) / (2 * math.log(base))
        low = max(math.floor(corrected(beta_fast)), 0)
        high = min(math.ceil(corrected(beta_slow)), dim - 1)
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / max(high - low, 1e-3)).clamp(0, 1)
        smooth = 1 - ramp
        freqs = freqs / factor * (1 - smooth) + freqs * smooth
    return freqs


def apply_rope(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate the last ``2*len(freqs)`` dims of x [s, ..., d] (adjacent pairs) by pos[s] * freqs."""
    rd = 2 * freqs.numel()
    ang = pos.float().unsqueeze(-1) * freqs  # [s, rd/2]
    if inverse:
        ang = -ang
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [rd // 2]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    t = x[..., -rd:].float().unflatten(-1, (-1, 2))
    a, b = t[..., 0], t[..., 1]
    rot = torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)
    return torch.cat([x[..., :-rd].float(), rot], -1)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * w.float()


def window_positions(pos: int, window: int) -> range:
    return range(max(0, pos - window + 1), pos + 1)


def topk_stable(score: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries of each row; ties (including -inf) go to the lower index."""
    order = torch.sort(score, dim=-1, descending=True, stable=True).indices
    return order[..., :k]


def select_candidate_blocks(score: torch.Tensor, clen: torch.Tensor, topk_blocks: int, block: int) -> torch.Tensor:
    """[s, n] masked scores -> [s, n] bool: positions inside the best `topk_blocks` blocks per row;
    the block holding the row's newest visible position is always kept."""
    n = score.shape[-1]
    sc = F.pad(score, (0, -n % block), value=float("-inf")).unflatten(-1, (-1, block)).amax(-1)
    nb = sc.shape[-1]
    last = (clen - 1) // block
    sc = sc.masked_fill(torch.arange(nb).unsqueeze(0) == last.view(-1, 1), float("inf"))
    k = min(topk_blocks, nb)
    idx = topk_stable(sc, k)
    vals = sc.gather(-1, idx)
    keep = torch.zeros_like(sc, dtype=torch.bool).scatter_(-1, idx, vals > float("-inf"))
    return keep.repeat_interleave(block, -1)[..., :n]


def sparse_attn_rows(q: torch.Tensor, kv: torch.Tensor, sink: torch.Tensor, scale: float) -> torch.Tensor:
    """q [H, d] against gathered kv [n, d] (n may be 0) with a per-head sink logit -> [H, d]."""
    if kv.shape[0] == 0:
        return torch.zeros_like(q)
    s = (q @ kv.t()) * scale
    m = s.amax(-1, keepdim=True)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True) + torch.exp(sink.view(-1, 1) - m)
    return (e @ kv) / den


@dataclass
class SeqState:
    pos: int = 0
    win: Dict[int, torch.Tensor] = field(default_factory=dict)        # layer -> [T, head_dim] (all positions)
    comp_kv: Dict[int, torch.Tensor] = field(default_factory=dict)    # kv-source layer -> [n, head_dim]
    index_k: Dict[int, torch.Tensor] = field(default_factory=dict)    # kv-source layer -> [n, index_dim]
    pool_kv: Dict[int, torch.Tensor] = field(default_factory=dict)    # ratio>1 sources: pending group rows [<r, hd]
    pool_score: Dict[int, torch.Tensor] = field(default_factory=dict)
    hasher: Optional[NgramHasher] = None

    def clone(self) -> "SeqState":
        return copy.deepcopy(self)


class Dsv41Reference:
    def __init__(self, cfg: Dsv41Config, weights: Dict[str, torch.Tensor], act_quant: bool = True,
                 token_map: Optional[Sequence[int]] = None):
        self.cfg, self.w, self.act_quant = cfg, weights, act_quant
        self.specs = tensor_specs(cfg)
        self.freq_win = rope_freqs(cfg.rope_head_dim, cfg.rope_theta, 0, 1.0, cfg.beta_fast, cfg.beta_slow)
        self.freq_cmp = rope_freqs(cfg.rope_head_dim, cfg.compress_rope_theta, cfg.original_seq_len, cfg.rope_factor,
                                   cfg.beta_fast, cfg.beta_slow)
        self.layout = EngramLayout.from_config(cfg)
        self.token_map = token_map
        self.trace: Optional[Callable[[str, torch.Tensor], None]] = None

    # ---- helpers -----------------------------------------------------------------------------
    def _t(self, name: str, x: torch.Tensor) -> torch.Tensor:
        if self.trace is not None:
            self.trace(name, x)
        return x

    def lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        spec = self.specs[name]
        kind = spec.kind
        quantised = (kind == "dense" and self.cfg.dense_dtype == "fp8") or kind == "expert"
        if quantised and self.act_quant:
            x = Q.fp8_act_roundtrip(x, self.cfg.fp8_block)
        return x.float() @ self.w[name].float().t()

    def new_seq(self) -> SeqState:
        st = SeqState()
        if self.layout is not None:
            st.hasher = NgramHasher(self.cfg, self.layout, self.token_map)
        return st

    def freqs(self, layer: int) -> torch.Tensor:
        return self.freq_cmp if self.cfg.ratio(layer) > 0 else self.freq_win

    # ---- hyper-connections -----------------------------------------------------------------
    def hc_mixes(self, h: torch.Tensor, p: str, which: str):
        cfg = self.cfg
        s = h.shape[0]
        flat = h.float().reshape(s, -1)
        r = torch.rsqrt(flat.square().mean(-1, keepdim=True) + cfg.norm_eps)
        mixes = (flat @ self.w[p + f"hc_{which}_fn"].float().t()) * r
        return R.hc_coeffs(mixes, self.w[p + f"hc_{which}_scale"].float(), self.w[p + f"hc_{which}_base"].float(),
                           cfg.hc_mult, cfg.hc_eps, cfg.hc_sinkhorn_iters)

    @staticmethod
    def hc_pre(h: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
        return (pre.unsqueeze(-1) * h.float()).sum(1)

    # ---- compressor (kv-source layers) -------------------------------------------------------
    def compress(self, st: SeqState, layer: int, p: str, x: torch.Tensor, pos0: int):
        """Returns (group indices [g], latents [g, hd] normed, pre-RoPE) completed by these rows."""
        cfg, r = self.cfg, self.cfg.ratio(layer)
        c = p + "attn.compressor."
        s = x.shape[0]
        if r == 1:
            lat = rmsnorm(x.float() @ self.w[c + "wkv.weight"].float().t(), self.w[c + "norm.weight"], cfg.norm_eps)
            return torch.arange(pos0, pos0 + s), lat
        kv = x.float() @ self.w[c + "wkv.weight"].float().t()
        sc = x.float() @ self.w[c + "wgate.weight"].float().t()
        if layer in st.pool_kv and st.pool_kv[layer].shape[0]:
            kv = torch.cat([st.pool_kv[layer], kv])
            sc = torch.cat([st.pool_score[layer], sc])
        first = pos0 - (kv.shape[0] - s)       # position of kv[0]; a multiple of r
        assert first % r == 0
        ng = kv.shape[0] // r
        st.pool_kv[layer], st.pool_score[layer] = kv[ng * r:].clone(), sc[ng * r:].clone()
        if ng == 0:
            return torch.zeros(0, dtype=torch.long), torch.zeros(0, cfg.head_dim)
        kvg, scg = kv[:ng * r].unflatten(0, (ng, r)), sc[:ng * r].unflatten(0, (ng, r))
        lat = (kvg * scg.softmax(1)).sum(1)
        lat = rmsnorm(lat, self.w[c + "norm.weight"], cfg.norm_eps)
        return first // r + torch.arange(ng), lat

    # ---- attention ---------------------------------------------------------------------------
    def attention(self, st: SeqState, layer: int, p: str, x: torch.Tensor, pos: torch.Tensor, shared: dict) -> torch.Tensor:
        cfg = self.cfg
        s, H, hd, rd = x.shape[0], cfg.n_heads, cfg.head_dim, cfg.rope_head_dim
        a = p + "attn."
        fr = self.freqs(layer)
        qr = rmsnorm(self.lin(x, a + "wq_a.weight"), self.w[a + "q_norm.weight"], cfg.norm_eps)
        q = apply_rope(self.lin(qr, a + "wq_b.weight").view(s, H, hd), pos, fr)
        kv = rmsnorm(self.lin(x, a + "wkv.weight"), self.w[a + "kv_norm.weight"], cfg.norm_eps)
        kv = Q.fp8_act_roundtrip(apply_rope(kv, pos, fr), cfg.fp8_block)
        self._t(f"{p}q", q)
        self._t(f"{p}kv", kv)
        pos0 = int(pos[0])
        st.win[layer] = torch.cat([st.win.get(layer, torch.zeros(0, hd))[:pos0], kv])
        r = cfg.ratio(layer)
        idxs = None
        if r > 0:
            src = cfg.kv_source_of(layer)
            if cfg.is_kv_source(layer):
                gidx, lat = self.compress(st, layer, p, x, pos0)
                if gidx.numel():
                    ix = a + "indexer."
                    k = rmsnorm(lat @ self.w[ix + "wk.weight"].float().t(), self.w[ix + "k_norm.weight"], cfg.norm_eps)
                    k = Q.fp4_act_roundtrip(apply_rope(k, gidx * r, fr), cfg.fp4_block)
                    g0 = int(gidx[0])
                    st.index_k[layer] = torch.cat([st.index_k.get(layer, torch.zeros(0, cfg.index_head_dim))[:g0], k])
                    lat = Q.fp4_act_roundtrip(apply_rope(lat, gidx * r, fr), 16, "e4m3")
                    st.comp_kv[layer] = torch.cat([st.comp_kv.get(layer, torch.zeros(0, hd))[:g0], lat])
                    self._t(f"{p}latent", lat)
            clen = (pos + 1) // r
            n_max = int(clen[-1])
            if cfg.is_index_source(layer):
                if n_max == 0:
                    idxs = torch.full((s, 0), -1, dtype=torch.long)
                else:
                    idxs = self.indexer(st, layer, p, x, qr, pos, clen, n_max, src, shared)
                shared["topk"] = idxs
            else:
                idxs = shared["topk"]
            self._t(f"{p}topk", idxs.float())
        sink = self.w[a + "attn_sink"].float()
        scale = hd ** -0.5
        o = torch.zeros(s, H, hd)
        for t in range(s):
            wp = window_positions(int(pos[t]), cfg.window_size)
            rows = st.win[layer][wp.start:wp.stop]
            if idxs is not None and idxs.shape[1]:
                sel = idxs[t][idxs[t] >= 0]
                rows = torch.cat([rows, st.comp_kv[cfg.kv_source_of(layer)][sel]])
            o[t] = sparse_attn_rows(q[t], rows, sink, scale)
        o = apply_rope(o, pos, fr, inverse=True)
        self._t(f"{p}attn_o", o)
        return self.out_proj(o, a)

    def out_proj(self, o: torch.Tensor, a: str) -> torch.Tensor:
        cfg = self.cfg
        s = o.shape[0]
        og = o.reshape(s, cfg.o_groups, -1)
        wo_a = self.w[a + "wo_a.weight"].float().view(cfg.o_groups, cfg.o_lora_rank, -1)
        low = torch.einsum("sgd,grd->sgr", og, wo_a).reshape(s, -1)
        return self.lin(low, a + "wo_b.weight")

    def indexer(self, st, layer, p, x, qr, pos, clen, n_max, src, shared) -> torch.Tensor:
        cfg = self.cfg
        ix = p + "attn.indexer."
        s, IH, ID = x.shape[0], cfg.index_n_heads, cfg.index_head_dim
        q = apply_rope(self.lin(qr, ix + "wq_b.weight").view(s, IH, ID), pos, self.freqs(layer))
        q = Q.fp4_act_roundtrip(q, cfg.fp4_block)
        wts = (x.float() @ self.w[ix + "weights_proj.weight"].float().t()) * (ID ** -0.5 * IH ** -0.5)
        K = st.index_k[src][:n_max]
        score = (torch.einsum("shd,td->sht", q, K).relu() * wts.unsqueeze(-1)).sum(1)
        score = score.masked_fill(torch.arange(n_max).unsqueeze(0) >= clen.unsqueeze(1), float("-inf"))
        self._t(f"{p}index_score", score)
        if layer == cfg.candidate_source_layer:
            shared["cand"] = select_candidate_blocks(score, clen, cfg.candidate_topk_blocks, cfg.candidate_block_size)
        elif cfg.uses_candidates(layer):
            score = score.masked_fill(~shared["cand"], float("-inf"))
        k = min(cfg.index_topk, n_max)
        idx = topk_stable(score, k).sort(-1).values
        return torch.where(idx < clen.unsqueeze(1), idx, torch.full_like(idx, -1))

    # ---- MoE ---------------------------------------------------------------------------------
    def route(self, x: torch.Tensor, f: str, topk: int, image_mask: Optional[torch.Tensor]):
        scores = F.softplus(x.float() @ self.w[f + "gate.weight"].float().t()).sqrt()
        bias = self.w[f + "gate.bias"].float().expand_as(scores)
        if image_mask is not None and (f + "gate.bias_vl") in self.w:
            bias = torch.where(image_mask.unsqueeze(-1), self.w[f + "gate.bias_vl"].float(), bias)
        idx = topk_stable(scores + bias, topk)
        wts = scores.gather(1, idx)
        if topk > 1:
            wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
        return wts * self.cfg.route_scale, idx

    def expert(self, x: torch.Tensor, pre: str, wts: Optional[torch.Tensor]) -> torch.Tensor:
        lim = self.cfg.swiglu_limit
        gate, up = self.lin(x, pre + "w1.weight"), self.lin(x, pre + "w3.weight")
        if lim > 0:
            up, gate = up.clamp(-lim, lim), gate.clamp(max=lim)
        h = F.silu(gate) * up
        if wts is not None:
            h = h * wts
        return self.lin(h, pre + "w2.weight")

    def moe(self, x: torch.Tensor, layer: int, p: str, image_mask: Optional[torch.Tensor]) -> torch.Tensor:
        f = p + "ffn."
        E, topk = self.cfg.moe_shape(layer)
        wts, idx = self.route(x, f, topk, image_mask)
        self._t(f"{p}route_idx", idx.float())
        self._t(f"{p}route_w", wts)
        y = torch.zeros(x.shape[0], self.cfg.dim)
        for e in idx.unique().tolist():
            rows, slot = torch.where(idx == e)
            y[rows] += self.expert(x[rows], f + f"experts.{e}.", wts[rows, slot, None])
        return y + self.expert(x, f + "shared_experts.", None)

    # ---- engram ------------------------------------------------------------------------------
    def engram(self, h: torch.Tensor, layer: int, hashes: torch.Tensor, alive: Optional[torch.Tensor]) -> torch.Tensor:
        cfg = self.cfg
        p = f"layers.{layer}.engram."
        rows = self.w[p + "embed.weight"].float()[hashes]             # [s, cols, head_dim]
        kv = self.lin(rows.flatten(-2), p + "wkv.weight")
        key, value = kv.split([cfg.hc_mult * cfg.dim, cfg.dim], -1)
        key = key.unflatten(-1, (cfg.hc_mult, cfg.dim))
        w = self.w[p + "q_weight"].float() * self.w[p + "k_weight"].float()
        hf = h.float()
        rstd = torch.rsqrt(hf.square().mean(-1) + cfg.norm_eps) * torch.rsqrt(key.square().mean(-1) + cfg.norm_eps)
        dot = (hf * w * key).sum(-1) * rstd * cfg.dim ** -0.5
        gate = torch.sigmoid(torch.copysign(dot.abs().clamp_min(1e-6).sqrt(), dot))
        if alive is not None:
            gate = gate.masked_fill(~alive.unsqueeze(-1), 0)
        return hf + gate.unsqueeze(-1) * value.unsqueeze(-2)

    # ---- block -------------------------------------------------------------------------------
    def block(self, st, layer, p, h, pre_mix, pos, shared, image_mask, attn_fn=None):
        cfg = self.cfg
        a_pre, a_post, a_comb = self.hc_mixes(h, p, "attn")
        x = rmsnorm(self.hc_pre(h, pre_mix), self.w[p + "attn_norm.weight"], cfg.norm_eps)
        self._t(f"{p}attn_in", x)
        y = attn_fn(x) if attn_fn is not None else self.attention(st, layer, p, x, pos, shared)
        self._t(f"{p}attn_out", y)
        h = R.hc_post(y, h, a_post, a_comb)
        f_pre, f_post, f_comb = self.hc_mixes(h, p, "ffn")
        x = rmsnorm(self.hc_pre(h, a_pre), self.w[p + "ffn_norm.weight"], cfg.norm_eps)
        y = self.moe(x, layer, p, image_mask)
        self._t(f"{p}ffn_out", y)
        h = R.hc_post(y, h, f_post, f_comb)
        self._t(f"{p}h", h)
        return h, f_pre

    # ---- whole model -------------------------------------------------------------------------
    def forward(self, st: SeqState, ids: Sequence[int], image_mask: Optional[torch.Tensor] = None,
                embeds: Optional[torch.Tensor] = None):
        """Append len(ids) positions.  Returns (logits [s, V], main_hidden [s, dim*targets] or None).
        `embeds` [s, dim] overrides the token embedding where `image_mask` is set."""
        cfg = self.cfg
        ids_t = torch.as_tensor(list(ids), dtype=torch.long)
        s = ids_t.numel()
        pos = torch.arange(st.pos, st.pos + s)
        alive = None if image_mask is None else ~image_mask
        hashes = None
        if st.hasher is not None:
            st.hasher.truncate(st.pos)
            hashes = st.hasher.extend(ids_t.tolist(), None if alive is None else alive.tolist())
        e = self.w["embed.weight"].float()[ids_t]
        if embeds is not None:
            e = torch.where(image_mask.unsqueeze(-1), embeds.float(), e) if image_mask is not None else embeds.float()
        h = e.unsqueeze(1).repeat(1, cfg.hc_mult, 1)
        pre_mix = torch.zeros(s, cfg.hc_mult)
        pre_mix[:, 0] = 1.0
        shared: dict = {}
        mains: List[torch.Tensor] = []
        for l in range(cfg.n_layers):
            p = f"layers.{l}."
            ei = cfg.engram_index(l)
            if ei >= 0:
                h = self.engram(h, l, hashes[:, ei], alive)
                self._t(f"{p}engram_h", h)
            if l in cfg.dspark_target_layer_ids:
                mains.append(h.mean(1))
            h, pre_mix = self.block(st, l, p, h, pre_mix, pos, shared, image_mask)
        x = rmsnorm(self.hc_pre(h, pre_mix), self.w["norm.weight"], cfg.norm_eps)
        logits = x @ self.w["head.weight"].float().t()
        st.pos += s
        return self._t("logits", logits), (torch.cat(mains, -1) if mains else None)

    # ---- DSpark ------------------------------------------------------------------------------
    def dspark_main_x(self, main_hidden: torch.Tensor) -> torch.Tensor:
        return rmsnorm(self.lin(main_hidden, "mtp.0.main_proj.weight"), self.w["mtp.0.main_norm.weight"], self.cfg.norm_eps)

    def dspark_seed(self, st: SeqState, main_hidden: torch.Tensor, pos0: int) -> None:
        """Write the main-model KV of rows pos0.. (from their target-layer hiddens) into every DSpark
        layer's window history."""
        cfg = self.cfg
        main_x = self.dspark_main_x(main_hidden)
        pos = torch.arange(pos0, pos0 + main_x.shape[0])
        for j in range(cfg.n_mtp_layers):
            layer, a = cfg.n_layers + j, f"mtp.{j}.attn."
            kv = rmsnorm(self.lin(main_x, a + "wkv.weight"), self.w[a + "kv_norm.weight"], cfg.norm_eps)
            kv = Q.fp8_act_roundtrip(apply_rope(kv, pos, self.freq_win), cfg.fp8_block)
            st.win[layer] = torch.cat([st.win.get(layer, torch.zeros(0, cfg.head_dim))[:pos0], kv])

    def dspark_draft(self, st: SeqState, t0: int, last_pos: int):
        """Draft block after the main model emitted `t0` from position `last_pos` (whose main KV is
        already seeded).  Returns (drafts [B], logits [B, V], confidence [B])."""
        cfg = self.cfg
        B, H, hd = cfg.dspark_block_size, cfg.n_heads, cfg.head_dim
        ids = torch.full((B,), cfg.dspark_noise_token_id, dtype=torch.long)
        ids[0] = t0
        h = self.w["embed.weight"].float()[ids].unsqueeze(1).repeat(1, cfg.hc_mult, 1)
        pre_mix = torch.zeros(B, cfg.hc_mult)
        pre_mix[:, 0] = 1.0
        pos = torch.arange(last_pos + 1, last_pos + 1 + B)
        for j in range(cfg.n_mtp_layers):
            layer, p = cfg.n_layers + j, f"mtp.{j}."
            a = p + "attn."

            def attn(x, layer=layer, a=a):
                qr = rmsnorm(self.lin(x, a + "wq_a.weight"), self.w[a + "q_norm.weight"], cfg.norm_eps)
                q = apply_rope(self.lin(qr, a + "wq_b.weight").view(B, H, hd), pos, self.freq_win)
                kv = rmsnorm(self.lin(x, a + "wkv.weight"), self.w[a + "kv_norm.weight"], cfg.norm_eps)
                kv = Q.fp8_act_roundtrip(apply_rope(kv, pos, self.freq_win), cfg.fp8_block)
                wp = window_positions(last_pos, cfg.window_size)
                rows = torch.cat([st.win[layer][wp.start:wp.stop], kv])   # every draft row sees the whole block
                sink = self.w[a + "attn_sink"].float()
                o = torch.stack([sparse_attn_rows(q[t], rows, sink, hd ** -0.5) for t in range(B)])
                return self.out_proj(apply_rope(o, pos, self.freq_win, inverse=True), a)

            h, pre_mix = self.block(st, layer, p, h, pre_mix, pos, {}, None, attn_fn=attn)
        last = f"mtp.{cfg.n_mtp_layers - 1}."
        xc = self.hc_pre(h, pre_mix)
        logits = rmsnorm(xc, self.w[last + "norm.weight"], cfg.norm_eps) @ self.w["head.weight"].float().t()
        out, membs = [int(t0)], []
        me, mh = self.w[last + "markov_head.embed.weight"].float(), self.w[last + "markov_head.head.weight"].float()
        for i in range(B):
            emb = me[out[i]]
            logits[i] += mh @ emb
            membs.append(emb)
            out.append(int(R.argmax_first(logits[i:i + 1])[0]))
        conf = torch.cat([xc, torch.stack(membs)], -1) @ self.w[last + "confidence_head.proj.weight"].float().t()
        return out[1:], logits, conf.squeeze(-1)

    # ---- generation --------------------------------------------------------------------------
    def generate(self, prompt: Sequence[int], n_new: int) -> List[int]:
        st = self.new_seq()
        logits, _ = self.forward(st, prompt)
        out = [int(R.argmax_first(logits[-1:])[0])]
        while len(out) < n_new:
            logits, _ = self.forward(st, [out[-1]])
            out.append(int(R.argmax_first(logits[-1:])[0]))
        return out

    def spec_generate(self, prompt: Sequence[int], n_new: int):
        """Greedy generation with the DSpark draft + multi-row verify; returns (tokens, accept
        lengths).  Emits exactly the tokens `generate` does."""
        cfg = self.cfg
        st = self.new_seq()
        logits, mh = self.forward(st, prompt)
        self.dspark_seed(st, mh, 0)
        t0 = int(R.argmax_first(logits[-1:])[0])
        out, ks = [t0], []
        while len(out) < n_new:
            last_pos = st.pos - 1
            drafts, _, _ = self.dspark_draft(st, t0, last_pos)
            snap = st.clone()
            block = [t0] + drafts
            logits, mh = self.forward(st, block)
            judges = R.argmax_first(logits).tolist()
            m = spec_accept(drafts, judges, anchor_is_in_block=False)   # accepted drafts
            emitted = judges[:m + 1]                                    # ... plus the bonus token
            k = m + 1                                                   # verify rows that stay
            ks.append(k)
            # keep rows 0..k-1 of the verify block: replay them on the snapshot (the golden has no
            # partial rollback of the pooled compressor state)
            st = snap
            logits, mh = self.forward(st, block[:k])
            self.dspark_seed(st, mh, last_pos + 1)
            out += emitted
            t0 = emitted[-1]
        return out[:n_new], ks
