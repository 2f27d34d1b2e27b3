"""Plain PyTorch fp32 statements of every GLM-5.3-Flash op.

These are the readable oracle the CUDA kernels are compared against op by op,
and they run on CPU.  The math follows the reference's f32 CPU backend
(``crates/ferrite-kernel/src/cpu.rs:82-808``), its hyper-connection helpers
(``crates/ferrite-exec/src/mhc.rs:19-213``), the decode-context-parallel model
(``crates/ferrite-kernel/src/dcp.rs:49-174``) and the WY chunk algebra
(``crates/ferrite-kernel/src/wyf.rs:10-147``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

F32_EPS = 1.1920929e-07


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[n, out_f] = x[n, in_f] . w[out_f, in_f]^T in fp32."""
    return x.float() @ w.float().t()


def rmsnorm(x, w, eps: float):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def gated_rmsnorm(o, gate, w, eps: float):
    """Per-head ``o * rsqrt(mean o^2 + eps) * w * sigmoid(gate)`` (last dim = head_dim)."""
    o = o.float()
    return o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * w.float() * torch.sigmoid(gate.float())


def layernorm_affine(x, w, b, eps: float):
    x = x.float()
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps) * w.float() + b.float()


def swiglu_limited(gate, up, limit: float):
    """silu(min(gate, limit)) * clamp(up, -limit, limit)."""
    g = gate.float().clamp(max=limit)
    u = up.float().clamp(min=-limit, max=limit)
    return F.silu(g) * u


def causal_conv1d(x, w, state):
    """Depthwise causal conv.  x [n, ch], w [ch, k], state [ch, k-1] (oldest first).
    Returns (out [n, ch], new_state [ch, k-1]); no activation is applied."""
    n, ch = x.shape
    k = w.shape[1]
    stream = torch.cat([state.float().t(), x.float()], 0)  # [k-1+n, ch]
    win = stream.unfold(0, k, 1)  # [n, ch, k]
    out = (win * w.float().unsqueeze(0)).sum(-1)
    return out, stream[n:].t().contiguous()


def l2norm_heads(x):
    """Normalise the last dim; an all-zero vector stays zero."""
    x = x.float()
    nrm = x.pow(2).sum(-1, keepdim=True).sqrt()
    return torch.where(nrm > 0, x / nrm.clamp_min(1e-38), torch.zeros_like(x))


def gdn_log_decay(fb, dt_bias, a_log, lower_bound: float, heads: int):
    """g[t,h,i] = lb * sigmoid(exp(A_log_h) * (fb[t,h,i] + dt_bias[h,i])) (always <= 0)."""
    n = fb.shape[0]
    dk = fb.shape[1] // heads
    a = a_log.float().exp().view(1, heads, 1)
    return lower_bound * torch.sigmoid(a * (fb.float().view(n, heads, dk) + dt_bias.float().view(1, heads, dk)))


def gdn_recurrent(q, k, v, beta, g, state):
    """Token-serial GatedDeltaNet/KDA recurrence.

    q,k [n,h,dk]; v [n,h,dv]; beta [n,h]; g [n,h,dk] log-decay; state [h,dk,dv].
    Per token: S *= exp(g) (rows); u = S^T k; S += beta k (v-u)^T; o = S^T q.
    """
    S = state.float().clone()
    n = q.shape[0]
    outs = []
    for t in range(n):
        S = S * g[t].float().exp().unsqueeze(-1)
        u = torch.einsum("hkv,hk->hv", S, k[t].float())
        S = S + beta[t].float().view(-1, 1, 1) * k[t].float().unsqueeze(-1) * (v[t].float() - u).unsqueeze(1)
        outs.append(torch.einsum("hkv,hk->hv", S, q[t].float()))
    return torch.stack(outs, 0), S


def gdn_chunk_wy(q, k, v, beta, g, state, chunk: int):
    """WY-chunked form of :func:`gdn_recurrent`; equal to it up to fp rounding.

    Within a chunk with inclusive log-decay prefix L_t:
      b_t = S0^T (k_t e^{L_t});  c[t,s] = sum_i k_t k_s e^{L_t-L_s} (s<t)
      w_t = beta_t (v_t - b_t - sum_{s<t} c[t,s] w_s)
      O_t = (q_t e^{L_t})^T S0 + sum_{s<=t} m[t,s] w_s
      S_C = diag(e^{L_last}) S0 + sum_s (k_s e^{L_last-L_s}) w_s^T
    """
    n, h, dk = q.shape
    S = state.float().clone()
    outs = []
    for c0 in range(0, n, chunk):
        c1 = min(n, c0 + chunk)
        C = c1 - c0
        qc, kc, vc = (t[c0:c1].float().transpose(0, 1) for t in (q, k, v))  # [h,C,d]
        bc = beta[c0:c1].float().t()  # [h,C]
        L = g[c0:c1].float().transpose(0, 1).cumsum(1)  # [h,C,dk]
        kd = kc * L.exp()  # k_t e^{L_t}
        qd = qc * L.exp()
        # pairwise decay e^{L_t-L_s} is formed per channel so no factor can overflow
        D = (L.unsqueeze(2) - L.unsqueeze(1)).clamp(max=0).exp()  # [h,t,s,dk]
        cmat = torch.einsum("hti,hsi,htsi->hts", kc, kc, D).tril(-1)
        mmat = torch.einsum("hti,hsi,htsi->hts", qc, kc, D).tril(0)
        bvec = torch.einsum("hkv,htk->htv", S, kd)
        rhs = bc.unsqueeze(-1) * (vc - bvec)
        A = torch.eye(C).unsqueeze(0) + bc.unsqueeze(-1) * cmat
        w = torch.linalg.solve_triangular(A, rhs, upper=False)
        o = torch.einsum("htk,hkv->htv", qd, S) + torch.einsum("hts,hsv->htv", mmat, w)
        Llast = L[:, -1]  # [h,dk]
        kend = kc * (Llast.unsqueeze(1) - L).exp()
        S = S * Llast.exp().unsqueeze(-1) + torch.einsum("hsk,hsv->hkv", kend, w)
        outs.append(o.transpose(0, 1))
    return torch.cat(outs, 0), S


def kpool_compress(k_idx, k_gate, ape, kpool: int):
    """Pool consecutive groups of ``kpool`` indexer keys with a per-channel softmax of
    (gate + ape[j]) over the tokens that exist.  k_idx,k_gate [T,D]; ape [kpool,D]."""
    T, D = k_idx.shape
    npools = (T + kpool - 1) // kpool
    pad = npools * kpool - T
    ki = F.pad(k_idx.float(), (0, 0, 0, pad)).view(npools, kpool, D)
    kg = F.pad(k_gate.float(), (0, 0, 0, pad), value=float("-inf")).view(npools, kpool, D)
    wgt = torch.softmax(kg + ape.float().unsqueeze(0), dim=1)
    return (wgt * ki).sum(1)


def indexer_scores(q_idx, pool_keys, w):
    """score[i,p] = D^-0.5 * sum_h w[i,h] relu(q[i,h] . key[p]).  q_idx [n,H,D]."""
    n, H, D = q_idx.shape
    dots = torch.einsum("nhd,pd->nhp", q_idx.float(), pool_keys.float()).clamp_min(0)
    return (dots * w.float().unsqueeze(-1)).sum(1) / math.sqrt(D)


def indexer_topk(q_idx, pool_keys, w, topk: int, ctx0_pools: int):
    """Top-k pools per row, ties to the lower index, invisible (p >= ctx0_pools+i+1) -> -1.
    Returns int64 [n, topk]."""
    n = q_idx.shape[0]
    P = pool_keys.shape[0]
    s = indexer_scores(q_idx, pool_keys, w)
    vis = torch.arange(P).unsqueeze(0) < (ctx0_pools + torch.arange(n) + 1).unsqueeze(1)
    s = torch.where(vis.to(s.device), s, torch.full_like(s, float("-inf")))
    order = torch.sort(s, dim=1, descending=True, stable=True).indices[:, :topk]
    sel = torch.gather(s, 1, order)
    return torch.where(sel == float("-inf"), torch.full_like(order, -1), order)


def expand_pool_indices(pool_idx, kpool: int, ctx0: int, total: int, width: int):
    """Selected pools -> token ids, then the visible tail (tokens past the last full pool).
    Slots that are invisible (t > ctx0+i or t >= total) or unused are -1.  Returns int64 [n,width]."""
    n, sk = pool_idx.shape
    out = torch.full((n, width), -1, dtype=torch.long)
    for i in range(n):
        col = 0
        lim = ctx0 + i
        for r in range(sk):
            p = int(pool_idx[i, r])
            if p < 0:
                continue
            for j in range(kpool):
                t = p * kpool + j
                out[i, col] = t if (t < total and t <= lim) else -1
                col += 1
        vc = lim + 1
        tail = vc % kpool
        start = vc - tail
        for j in range(kpool - 1):
            if col >= width:
                break
            t = start + j
            out[i, col] = t if (j < tail and t <= lim) else -1
            col += 1
    return out


def sparse_mla_attn(q, k, v, idx, return_lse: bool = False):
    """Softmax attention over the gathered token set.

    q [n,h,dk]; k [T,h,dk]; v [T,h,dv]; idx int [n,W] with -1 = skip; repeated ids
    count once.  The denominator carries + f32 epsilon.  Optionally returns the
    max-shifted pair (unnormalised o is NOT returned; lse = m + log(denominator)).
    """
    n, h, dk = q.shape
    T = k.shape[0]
    scale = 1.0 / math.sqrt(dk)
    mask = torch.zeros(n, T, dtype=torch.bool)
    valid = idx >= 0
    rows = torch.arange(n).unsqueeze(1).expand_as(idx)[valid]
    mask[rows, idx[valid]] = True
    s = torch.einsum("nhd,thd->nht", q.float(), k.float()) * scale
    s = s.masked_fill(~mask.unsqueeze(1), float("-inf"))
    m = s.max(-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = (s - m).exp()
    den = e.sum(-1, keepdim=True) + F32_EPS
    o = torch.einsum("nht,thv->nhv", e / den, v.float())
    if return_lse:
        return o, (m + den.log()).squeeze(-1)
    return o


def lse_merge(outs, lses):
    """Merge per-shard normalised partial outputs with their log-sum-exp, max-shifted.
    outs: list of [n,h,dv]; lses: list of [n,h] (-inf = empty shard)."""
    L = torch.stack(lses, 0)
    m = L.max(0).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    wts = (L - m).exp()
    den = wts.sum(0).clamp_min(1e-38)
    O = torch.stack(outs, 0)
    return (O * wts.unsqueeze(-1)).sum(0) / den.unsqueeze(-1)


def moe_route(logits, bias, topk: int, scaling: float):
    """Sigmoid scores; choose top-k of (score + bias) with ties to the lower index; weights
    are the raw scores renormalised (+ f32 eps) times ``scaling``.  Returns (w [n,k], ids [n,k])."""
    s = torch.sigmoid(logits.float())
    choice = s + bias.float()
    ids = torch.sort(choice, dim=1, descending=True, stable=True).indices[:, :topk]
    sel = torch.gather(s, 1, ids)
    return sel / (sel.sum(1, keepdim=True) + F32_EPS) * scaling, ids


def expert_ffn(x, gate_w, up_w, down_w, limit: float):
    return linear(swiglu_limited(linear(x, gate_w), linear(x, up_w), limit), down_w)


def hc_expand(h0, mult: int):
    return h0.float().unsqueeze(1).repeat(1, mult, 1)


def hc_contract(R):
    return R.float().mean(1)


def hc_coeffs(mixes, scale, base, n: int, hc_eps: float, iters: int):
    """pre [T,n], post [T,n], comb [T,n,n] from the 24 mix values of each token."""
    pre = torch.sigmoid(mixes[:, :n] * scale[0] + base[:n]) + hc_eps
    post = 2.0 * torch.sigmoid(mixes[:, n:2 * n] * scale[1] + base[n:2 * n])
    comb = (mixes[:, 2 * n:] * scale[2] + base[2 * n:]).view(-1, n, n)
    comb = torch.softmax(comb, dim=-1) + hc_eps
    comb = comb / (comb.sum(1, keepdim=True) + hc_eps)
    for _ in range(1, iters):
        comb = comb / (comb.sum(2, keepdim=True) + hc_eps)
        comb = comb / (comb.sum(1, keepdim=True) + hc_eps)
    return pre, post, comb


def hc_pre(R, fn, scale, base, rms_eps: float, hc_eps: float, iters: int):
    """R [T,n,H] -> (x [T,H], post [T,n], comb [T,n,n])."""
    T, n, H = R.shape
    flat = R.float().reshape(T, n * H)
    r = torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + rms_eps)
    mixes = (flat @ fn.float().t()) * r
    pre, post, comb = hc_coeffs(mixes, scale.float(), base.float(), n, hc_eps, iters)
    x = (pre.unsqueeze(-1) * R.float()).sum(1)
    return x, post, comb


def hc_post(y, R, post, comb):
    """R'[i] = post_i * y + sum_k comb[k,i] R[k]."""
    return post.unsqueeze(-1) * y.float().unsqueeze(1) + torch.einsum("tki,tkh->tih", comb, R.float())


def argmax_first(logits):
    """First maximum wins."""
    m = logits.max(-1, keepdim=True).values
    V = logits.shape[-1]
    cand = torch.where(logits == m, torch.arange(V, device=logits.device).expand_as(logits),
                       torch.full_like(logits, V, dtype=torch.long))
    return cand.min(-1).values


# ---- fp8 e4m3 block-scaled weights (128x128 blocks) ------------------------------------
def quant_fp8_block(w: torch.Tensor, block: int = 128):
    """Quantise [N,K] to e4m3 with one f32 scale per (block x block) tile.
    Returns (w_fp8 [N,K] float8_e4m3fn, scale [ceil(N/b), ceil(K/b)] f32) with w ~= fp8 * scale."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = F.pad(w.float(), (0, kb * block - K, 0, nb * block - N)).view(nb, block, kb, block)
    amax = wp.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (wp / scale.view(nb, 1, kb, 1)).clamp(-448, 448).view(nb * block, kb * block)[:N, :K]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def dequant_fp8_block(w8: torch.Tensor, scale: torch.Tensor, block: int = 128):
    N, K = w8.shape
    s = scale.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return w8.float() * s


# ---- DCP helpers (reference dcp.rs:179-260) -------------------------------------------
def split_pages_round_robin(total_tokens: int, page: int, n_shards: int):
    """Token ids owned by each shard when page p lives on shard p % n."""
    out = [[] for _ in range(n_shards)]
    for t in range(total_tokens):
        out[(t // page) % n_shards].append(t)
    return out


def sparse_attn_partial(q, k, v, idx, owned: torch.Tensor):
    """Partial attention of one DCP shard: only ids with owned[id] participate."""
    idx2 = torch.where((idx >= 0) & owned[idx.clamp_min(0)], idx, torch.full_like(idx, -1))
    o, lse = sparse_mla_attn(q, k, v, idx2, return_lse=True)
    empty = (idx2 >= 0).sum(1) == 0
    lse = torch.where(empty.unsqueeze(1), torch.full_like(lse, float("-inf")), lse)
    return o, lse


# ---- temperature sampling (Gumbel-max with a counter-based hash) ----------------------------
def _mix32(h: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    h = h ^ (h >> 16)
    h = (h * 0x85EBCA6B) & m
    h = h ^ (h >> 13)
    h = (h * 0xC2B2AE35) & m
    return h ^ (h >> 16)


def gumbel_noise(seed: int, keys: torch.Tensor, V: int, offset: int = 0) -> torch.Tensor:
    """[len(keys), V] noise G = -log(-log u), u from a 32-bit hash of (seed, row key, global index)."""
    m = 0xFFFFFFFF
    idx = (torch.arange(V, dtype=torch.int64) + offset).unsqueeze(0)
    k = (keys.to(torch.int64).unsqueeze(1) * 0x9E3779B1) & m
    h = _mix32(_mix32((seed & m) ^ k) ^ ((idx * 0x85EBCA77) & m))
    u = ((h >> 8).float() + 0.5) * (1.0 / 16777216.0)
    return -torch.log(-torch.log(u))


def sample_gumbel(logits, temperature: float, seed: int, keys: torch.Tensor):
    """argmax(logits / T + G): one draw per row from softmax(logits / T); T = 0 is plain argmax."""
    if temperature == 0:
        return argmax_first(logits)
    z = logits.float() * (1.0 / max(temperature, 1e-5)) + gumbel_noise(seed, keys, logits.shape[-1])
    return argmax_first(z)
