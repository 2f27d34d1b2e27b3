"""GLM-5.3-Flash tensor-name layout, random init, fused-weight aliases, HF name map and
the tensor-parallel shard rules.

Names and shapes follow the reference layout (``crates/ferrite-model/src/weights.rs:44-196``);
the fused aliases accepted on load follow ``weights.rs:327-426``; the checkpoint-side names
follow ``crates/ferrite-model/src/checkpoint.rs:43-90``; the shard rules follow
``crates/ferrite-exec/src/tp.rs:7-20,268-512``.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, Optional, Tuple

import torch

from ..config import GlmConfig

Weights = Dict[str, torch.Tensor]


def _layer_common(d, pfx, cfg: GlmConfig, mhc: bool):
    H = cfg.hidden_size
    d[f"{pfx}.input_layernorm.weight"] = (H,)
    d[f"{pfx}.post_attention_layernorm.weight"] = (H,)
    if mhc:
        for site in ("attn", "ffn"):
            d[f"{pfx}.hc_{site}_base"] = (cfg.hc_mix,)
            d[f"{pfx}.hc_{site}_scale"] = (3,)
            d[f"{pfx}.hc_{site}_fn"] = (cfg.hc_mix, cfg.hc_mult * H)


def _linear_attn(d, pfx, cfg: GlmConfig):
    H, la = cfg.hidden_size, cfg.linear_attn
    P, r = la.proj, la.low_rank
    a = f"{pfx}.self_attn"
    d[f"{a}.qkv_proj.weight"] = (3 * P, H)
    d[f"{a}.f_a_proj.weight"] = (r, H)
    d[f"{a}.f_b_proj.weight"] = (P, r)
    d[f"{a}.b_proj.weight"] = (la.num_heads, H)
    d[f"{a}.g_a_proj.weight"] = (r, H)
    d[f"{a}.g_b_proj.weight"] = (P, r)
    d[f"{a}.A_log"] = (la.num_heads,)
    d[f"{a}.dt_bias"] = (P,)
    d[f"{a}.qkv_conv1d.weight"] = (3 * P, la.conv_kernel)
    d[f"{a}.o_norm.weight"] = (la.head_dim,)
    d[f"{a}.o_proj.weight"] = (H, P)


def _dsa_attn(d, pfx, cfg: GlmConfig):
    H, ds = cfg.hidden_size, cfg.dsa
    a = f"{pfx}.self_attn"
    d[f"{a}.q_a_proj.weight"] = (ds.q_lora_rank, H)
    d[f"{a}.q_a_layernorm.weight"] = (ds.q_lora_rank,)
    d[f"{a}.q_b_proj.weight"] = (ds.num_heads * ds.qk_nope_head_dim, ds.q_lora_rank)
    d[f"{a}.kv_a_proj_with_mqa.weight"] = (ds.kv_lora_rank, H)
    d[f"{a}.kv_a_layernorm.weight"] = (ds.kv_lora_rank,)
    d[f"{a}.kv_b_proj.weight"] = (ds.num_heads * (ds.qk_nope_head_dim + ds.v_head_dim), ds.kv_lora_rank)
    d[f"{a}.indexer.wq_b.weight"] = (ds.index_n_heads * ds.index_head_dim, ds.q_lora_rank)
    d[f"{a}.indexer.wk.weight"] = (ds.index_head_dim, H)
    d[f"{a}.indexer.k_norm.weight"] = (ds.index_head_dim,)
    d[f"{a}.indexer.k_norm.bias"] = (ds.index_head_dim,)
    d[f"{a}.indexer.weights_proj.weight"] = (ds.index_n_heads, H)
    d[f"{a}.indexer.index_kpool_compress_gate"] = (ds.index_head_dim, H)
    d[f"{a}.indexer.index_kpool_compress_ape"] = (ds.index_kpool, ds.index_head_dim)
    d[f"{a}.o_proj.weight"] = (H, ds.num_heads * ds.v_head_dim)


def _dense_mlp(d, pfx, cfg: GlmConfig):
    H, I = cfg.hidden_size, cfg.intermediate_size
    d[f"{pfx}.mlp.gate_proj.weight"] = (I, H)
    d[f"{pfx}.mlp.up_proj.weight"] = (I, H)
    d[f"{pfx}.mlp.down_proj.weight"] = (H, I)


def _moe_mlp(d, pfx, cfg: GlmConfig):
    H, I, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.n_routed_experts
    d[f"{pfx}.mlp.gate.weight"] = (E, H)
    d[f"{pfx}.mlp.gate.e_score_correction_bias"] = (E,)
    Is = I * cfg.n_shared_experts
    for nm, shp in (("gate_proj", (Is, H)), ("up_proj", (Is, H)), ("down_proj", (H, Is))):
        d[f"{pfx}.mlp.shared_expert.{nm}.weight"] = shp
    for e in range(E):
        d[f"{pfx}.mlp.experts.{e}.gate_proj.weight"] = (I, H)
        d[f"{pfx}.mlp.experts.{e}.up_proj.weight"] = (I, H)
        d[f"{pfx}.mlp.experts.{e}.down_proj.weight"] = (H, I)


def weight_layout(cfg: GlmConfig) -> "OrderedDict[str, Tuple[int, ...]]":
    """Every tensor name of the model with its shape, in checkpoint order."""
    d: "OrderedDict[str, Tuple[int, ...]]" = OrderedDict()
    H, V = cfg.hidden_size, cfg.vocab_size
    d["model.embed_tokens.weight"] = (V, H)
    for i in range(cfg.num_layers):
        pfx = f"model.layers.{i}"
        _layer_common(d, pfx, cfg, cfg.mhc)
        (_dsa_attn if cfg.is_dsa(i) else _linear_attn)(d, pfx, cfg)
        (_moe_mlp if cfg.is_moe(i) else _dense_mlp)(d, pfx, cfg)
    for j in range(cfg.num_nextn_predict_layers):
        pfx = f"model.layers.{cfg.num_layers + j}"
        d[f"{pfx}.enorm.weight"] = (H,)
        d[f"{pfx}.hnorm.weight"] = (H,)
        d[f"{pfx}.eh_proj.weight"] = (H, 2 * H)
        _layer_common(d, pfx, cfg, False)
        _dsa_attn(d, pfx, cfg)
        _moe_mlp(d, pfx, cfg)
        d[f"{pfx}.shared_head.norm.weight"] = (H,)
    d["model.norm.weight"] = (H,)
    d["lm_head.weight"] = (V, H)
    return d


_ONES = ("layernorm.weight", "norm.weight", "enorm.weight", "hnorm.weight", "_scale")
_ZEROS = ("A_log", "dt_bias", "k_norm.bias", "e_score_correction_bias", "_base")


def init_kind(name: str) -> str:
    if name.endswith(_ZEROS):
        return "zeros"
    if name.endswith(_ONES):
        return "ones"
    return "normal"


def random_weights(cfg: GlmConfig, seed: int = 0, std: float = 0.02, device="cpu",
                   dtype=torch.float32, names: Optional[Iterable[str]] = None) -> Weights:
    """Deterministic synthetic weights: matrices N(0, std), norm weights and HC scales 1,
    biases / A_log / dt_bias / HC bases 0.  Each tensor has its own generator stream keyed by
    (seed, position in the layout), so a subset draws the same values as the full set."""
    layout = weight_layout(cfg)
    want = set(names) if names is not None else None
    out: Weights = {}
    for pos, (name, shape) in enumerate(layout.items()):
        if want is not None and name not in want:
            continue
        kind = init_kind(name)
        if kind == "zeros":
            t = torch.zeros(shape, dtype=torch.float32)
        elif kind == "ones":
            t = torch.ones(shape, dtype=torch.float32)
        else:
            g = torch.Generator().manual_seed((seed << 20) + pos)
            t = torch.randn(shape, generator=g, dtype=torch.float32) * std
        out[name] = t.to(device=device, dtype=dtype if t.dim() > 1 else torch.float32)
    return out


def apply_fused_aliases(w: Weights, cfg: GlmConfig) -> Weights:
    """Split fused checkpoint tensors into the canonical names (in place; returns ``w``).

    ``fused_qkvbfg_a_proj`` rows = qkv | b | f_a | g_a; ``fused_fg_b_proj`` [2,P,r] = f_b, g_b;
    ``fused_qkv_a_proj_with_mqa`` rows = q_a | kv_a; ``gate_up_proj`` rows = gate | up.
    """
    la, ds = cfg.linear_attn, cfg.dsa
    for name in list(w.keys()):
        t = w[name]
        if name.endswith("self_attn.fused_qkvbfg_a_proj.weight"):
            a = name[: -len("fused_qkvbfg_a_proj.weight")]
            P3, nh, r = 3 * la.proj, la.num_heads, la.low_rank
            assert t.shape[0] == P3 + nh + 2 * r, (name, tuple(t.shape))
            w[a + "qkv_proj.weight"], w[a + "b_proj.weight"], w[a + "f_a_proj.weight"], w[a + "g_a_proj.weight"] = \
                t.split([P3, nh, r, r], 0)
            del w[name]
        elif name.endswith("self_attn.fused_fg_b_proj.weight"):
            a = name[: -len("fused_fg_b_proj.weight")]
            w[a + "f_b_proj.weight"], w[a + "g_b_proj.weight"] = t[0], t[1]
            del w[name]
        elif name.endswith("self_attn.fused_qkv_a_proj_with_mqa.weight"):
            a = name[: -len("fused_qkv_a_proj_with_mqa.weight")]
            w[a + "q_a_proj.weight"], w[a + "kv_a_proj_with_mqa.weight"] = \
                t.split([ds.q_lora_rank, t.shape[0] - ds.q_lora_rank], 0)
            del w[name]
        elif name.endswith("gate_up_proj.weight"):
            a = name[: -len("gate_up_proj.weight")]
            half = t.shape[0] // 2
            w[a + "gate_proj.weight"], w[a + "up_proj.weight"] = t[:half], t[half:]
            del w[name]
    return w


# ---- checkpoint-side names ---------------------------------------------------------------
FUSED_QKV, FUSED_CONV = "__FUSED_QKV__", "__FUSED_CONV__"


def checkpoint_sources(name: str):
    """Internal name -> (marker|None, [checkpoint tensor names]).  ``qkv_proj`` and
    ``qkv_conv1d`` are assembled from separate q/k/v tensors on disk; the shared expert is
    plural on disk; everything but ``lm_head.weight`` lives under ``model.language_model.``."""
    if name == "lm_head.weight":
        return None, [name]
    src = "model.language_model." + name[len("model."):]
    src = src.replace(".shared_expert.", ".shared_experts.")
    if name.endswith("self_attn.qkv_proj.weight"):
        base = src[: -len("qkv_proj.weight")]
        return FUSED_QKV, [base + f"{p}_proj.weight" for p in "qkv"]
    if name.endswith("self_attn.qkv_conv1d.weight"):
        base = src[: -len("qkv_conv1d.weight")]
        return FUSED_CONV, [base + f"{p}_conv1d.weight" for p in "qkv"]
    return None, [src]


# ---- tensor-parallel shard rules ---------------------------------------------------------
def _rows(t, r, n):
    k = t.shape[0] // n
    return t[r * k:(r + 1) * k]


def _cols(t, r, n):
    k = t.shape[1] // n
    return t[:, r * k:(r + 1) * k]


def _thirds_rows(t, r, n):
    """q|k|v thirds, each split by head."""
    return torch.cat([_rows(p, r, n) for p in t.chunk(3, 0)], 0)


def shard_rule(name: str) -> str:
    """One of: rep, rows, cols, thirds, kvb (per-head [K|V] rows)."""
    s = name.split(".")
    leaf = ".".join(s[-2:]) if s[-1] == "weight" else s[-1]
    if "self_attn.indexer" in name:
        return "rep"
    if leaf in ("qkv_proj.weight", "qkv_conv1d.weight"):
        return "thirds"
    if leaf in ("b_proj.weight", "f_b_proj.weight", "g_b_proj.weight", "A_log", "dt_bias",
                "q_b_proj.weight", "kv_b_proj.weight", "gate_proj.weight", "up_proj.weight"):
        return "rows"
    if leaf in ("o_proj.weight", "down_proj.weight"):
        return "cols"
    return "rep"


def shard_weight(name: str, t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    if world == 1:
        return t
    rule = shard_rule(name)
    if rule == "rows":
        return _rows(t, rank, world).contiguous()
    if rule == "cols":
        return _cols(t, rank, world).contiguous()
    if rule == "thirds":
        return _thirds_rows(t, rank, world).contiguous()
    return t


def shard_weights_tp(w: Weights, rank: int, world: int) -> Weights:
    return {k: shard_weight(k, v, rank, world) for k, v in w.items()}


def fp8_row_blocks(rows: int, rank: int, world: int, block: int = 128) -> Tuple[int, int]:
    """Scale-row range of a row shard; cuts must fall on block boundaries."""
    k = rows // world
    assert k % block == 0, f"fp8 row shard {k} is not a multiple of {block}"
    return rank * k // block, (rank + 1) * k // block


def quantize_like_device(cfg: GlmConfig, w: Weights) -> Weights:
    """The weights as a single-rank device model sees them, returned in fp32: matrices are
    rounded to bf16, routed-expert and dense-MLP matrices go through the e4m3 128x128
    block quantiser (gate and up jointly, as they are stored as one [2I, H] matrix).  An
    oracle run on these values differs from the device only by accumulation order."""
    from ..ops.reference import dequant_fp8_block, quant_fp8_block
    out: Weights = {}
    keep_f32 = ("hc_attn_", "hc_ffn_", "A_log", "dt_bias", "conv1d", "e_score_correction_bias", "compress_ape")

    def is_fp8(name: str) -> bool:
        if ".mlp.experts." in name:
            return True
        return ".mlp." in name and ".shared_expert." not in name and ".mlp.gate." not in name \
            and name.endswith(("gate_proj.weight", "up_proj.weight", "down_proj.weight"))

    for name, t in w.items():
        t = t.float()
        if t.dim() < 2 or any(k in name for k in keep_f32):
            out[name] = t.clone()
        elif is_fp8(name):
            if name.endswith("up_proj.weight"):
                continue  # handled with its gate
            if name.endswith("gate_proj.weight"):
                up = name.replace("gate_proj", "up_proj")
                both = torch.cat([t, w[up].float()], 0)
                dq = dequant_fp8_block(*quant_fp8_block(both))
                out[name], out[up] = dq[: t.shape[0]].clone(), dq[t.shape[0]:].clone()
            else:
                out[name] = dequant_fp8_block(*quant_fp8_block(t))
        else:
            out[name] = t.to(torch.bfloat16).float()
    return out
