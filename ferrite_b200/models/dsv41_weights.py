"""DSV41 tensor inventory: names, shapes, storage formats, TP shard rules, random init.

Names follow the checkpoint's module tree (``ref_inference/model.py``: ``layers.N.attn.wq_a``,
``layers.N.ffn.experts.E.w1`` ..., DSpark stages under ``mtp.J``).  Storage kinds:

* ``dense``  - e4m3 with 32x32 ue8m0 block scales (bf16 when ``cfg.dense_dtype == "bf16"``)
* ``expert`` - e2m1 packed two per byte with per-(row, 32) ue8m0 scales (or ``dense`` when
  ``cfg.expert_dtype == "fp8"``)
* ``bf16``, ``f32`` - plain
* ``table``  - the engram table: e4m3 rows with per-(row, 32) ue8m0 scales

Shard rules are those of the reference's TP mapping (``crates/ferrite-models/src/dsv41/
weights.rs:27-330``): ``wq_b`` / ``attn_sink`` / indexer ``wq_b`` + ``weights_proj`` by heads,
``wo_a`` by groups, ``wo_b`` by input columns (all-reduce), routed experts kept on every rank
with the intermediate dim split (zero-padded to a multiple of 64 per rank), shared expert
replicated, engram table by rows (all-reduce), everything else replicated.
"""
from __future__ import annotations

import functools
from dataclasses import dataclass
from typing import Dict, Iterator, Optional, Tuple

import torch

from ..ops import quant as Q
from .dsv41_config import Dsv41Config


@dataclass(frozen=True)
class Spec:
    shape: Tuple[int, ...]
    kind: str                 # dense | expert | bf16 | f32 | table
    shard: Optional[Tuple[str, int]] = None   # ("split", dim) | ("rows_pad", dim) | None = replicated
    init: str = "normal"      # normal | ones | zeros | small | bias


def _block_specs(cfg: Dsv41Config, layer: int, prefix: str) -> Iterator[Tuple[str, Spec]]:
    d, hd, H = cfg.dim, cfg.head_dim, cfg.n_heads
    hc, mix = cfg.hc_mult, (2 + cfg.hc_mult) * cfg.hc_mult
    a = prefix + "attn."
    yield a + "attn_sink", Spec((H,), "f32", ("split", 0), "small")
    yield a + "wq_a.weight", Spec((cfg.q_lora_rank, d), "dense")
    yield a + "q_norm.weight", Spec((cfg.q_lora_rank,), "f32", None, "ones")
    yield a + "wq_b.weight", Spec((H * hd, cfg.q_lora_rank), "dense", ("split", 0))
    yield a + "wkv.weight", Spec((hd, d), "dense")
    yield a + "kv_norm.weight", Spec((hd,), "f32", None, "ones")
    yield a + "wo_a.weight", Spec((cfg.o_groups * cfg.o_lora_rank, H * hd // cfg.o_groups), "bf16", ("split", 0))
    yield a + "wo_b.weight", Spec((d, cfg.o_groups * cfg.o_lora_rank), "dense", ("split", 1))
    r = cfg.ratio(layer)
    if cfg.is_kv_source(layer):
        c = a + "compressor."
        yield c + "wkv.weight", Spec((hd, d), "f32" if r > 1 else "bf16")
        if r > 1:
            yield c + "wgate.weight", Spec((hd, d), "f32")
        yield c + "norm.weight", Spec((hd,), "f32", None, "ones")
    if cfg.is_index_source(layer):
        ix = a + "indexer."
        yield ix + "wq_b.weight", Spec((cfg.index_n_heads * cfg.index_head_dim, cfg.q_lora_rank), "dense", ("split", 0))
        yield ix + "weights_proj.weight", Spec((cfg.index_n_heads, d), "bf16", ("split", 0))
        if cfg.is_kv_source(layer):
            yield ix + "wk.weight", Spec((cfg.index_head_dim, hd), "bf16")
            yield ix + "k_norm.weight", Spec((cfg.index_head_dim,), "f32", None, "ones")
    yield prefix + "attn_norm.weight", Spec((d,), "f32", None, "ones")
    yield prefix + "ffn_norm.weight", Spec((d,), "f32", None, "ones")
    for which in ("attn", "ffn"):
        yield prefix + f"hc_{which}_fn", Spec((mix, hc * d), "f32", None, "small")
        yield prefix + f"hc_{which}_base", Spec((mix,), "f32", None, "small")
        yield prefix + f"hc_{which}_scale", Spec((3,), "f32", None, "ones")
    E, _ = cfg.moe_shape(layer)
    f = prefix + "ffn."
    yield f + "gate.weight", Spec((E, d), "bf16")
    yield f + "gate.bias", Spec((E,), "f32", None, "bias")
    if cfg.vision is not None:
        yield f + "gate.bias_vl", Spec((E,), "f32", None, "bias")
    I = cfg.moe_inter_dim
    for e in range(E):
        yield f + f"experts.{e}.w1.weight", Spec((I, d), "expert", ("rows_pad", 0))
        yield f + f"experts.{e}.w3.weight", Spec((I, d), "expert", ("rows_pad", 0))
        yield f + f"experts.{e}.w2.weight", Spec((d, I), "expert", ("rows_pad", 1))
    for w, shp in (("w1", (I, d)), ("w3", (I, d)), ("w2", (d, I))):
        yield f + f"shared_experts.{w}.weight", Spec(shp, "dense")


def tensor_specs(cfg: Dsv41Config) -> Dict[str, Spec]:
    d = cfg.dim
    out: Dict[str, Spec] = {}
    out["embed.weight"] = Spec((cfg.vocab_size, d), "bf16")
    out["norm.weight"] = Spec((d,), "f32", None, "ones")
    out["head.weight"] = Spec((cfg.vocab_size, d), "bf16", ("split", 0))
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        out.update(_block_specs(cfg, l, p))
        ei = cfg.engram_index(l)
        if ei >= 0:
            rows = cfg.engram_num_embeddings[ei]
            out[p + "engram.embed.weight"] = Spec((rows, cfg.engram_head_dim), "table", ("split", 0))
            out[p + "engram.wkv.weight"] = Spec((d * (cfg.hc_mult + 1), cfg.engram_hash_cols * cfg.engram_head_dim), "dense")
            out[p + "engram.q_weight"] = Spec((cfg.hc_mult, d), "f32", None, "ones")
            out[p + "engram.k_weight"] = Spec((cfg.hc_mult, d), "f32", None, "ones")
    for j in range(cfg.n_mtp_layers):
        p = f"mtp.{j}."
        out.update(_block_specs(cfg, cfg.n_layers + j, p))
        if j == 0:
            out[p + "main_proj.weight"] = Spec((d, d * len(cfg.dspark_target_layer_ids)), "dense")
            out[p + "main_norm.weight"] = Spec((d,), "f32", None, "ones")
        if j == cfg.n_mtp_layers - 1:
            out[p + "norm.weight"] = Spec((d,), "f32", None, "ones")
            out[p + "markov_head.embed.weight"] = Spec((cfg.vocab_size, cfg.dspark_markov_rank), "bf16")
            out[p + "markov_head.head.weight"] = Spec((cfg.vocab_size, cfg.dspark_markov_rank), "bf16", ("split", 0))
            out[p + "confidence_head.proj.weight"] = Spec((1, d + cfg.dspark_markov_rank), "f32")
    if cfg.vision is not None:
        from .dsv41_vision import vision_specs
        out.update(vision_specs(cfg))
    return out


# ---------------------------------------------------------------------------------------------
# sharding
# ---------------------------------------------------------------------------------------------
def padded_inter(cfg: Dsv41Config, world: int) -> int:
    """Per-rank slice of the expert intermediate dim, rounded up to a multiple of 64."""
    per = (cfg.moe_inter_dim + world - 1) // world
    return (per + 63) // 64 * 64


def shard_tensor(cfg: Dsv41Config, name: str, t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The slice of a full (dequantised or plain) tensor that `rank` of `world` keeps."""
    spec = tensor_specs_cached(cfg)[name]
    if world == 1 or spec.shard is None:
        return t
    kind, dim = spec.shard
    if kind == "split":
        n = t.shape[dim]
        if name.endswith("engram.embed.weight"):
            per = (n + world - 1) // world
            return t.narrow(dim, rank * per, max(0, min(per, n - rank * per)))
        assert n % world == 0, f"{name}: dim {dim} of size {n} does not split {world} ways"
        return t.narrow(dim, rank * (n // world), n // world)
    if kind == "rows_pad":
        per = (cfg.moe_inter_dim + world - 1) // world
        pad = padded_inter(cfg, world)
        lo = rank * per
        take = max(0, min(per, cfg.moe_inter_dim - lo))
        shp = list(t.shape)
        shp[dim] = pad
        out = torch.zeros(shp, dtype=t.dtype, device=t.device)
        out.narrow(dim, 0, take).copy_(t.narrow(dim, lo, take))
        return out
    raise ValueError(kind)


@functools.lru_cache(maxsize=8)
def tensor_specs_cached(cfg: Dsv41Config) -> Dict[str, Spec]:
    return tensor_specs(cfg)


def estimate_device_bytes(cfg: Dsv41Config, world: int = 1) -> int:
    """Weight bytes one rank of a `world`-way tensor-parallel device model holds: e2m1 experts with their ue8m0 scales
    (17 / 32 byte per value), engram tables as e4m3 bytes, dense and bf16 tensors as bf16 (dense e4m3 weights are
    expanded at load), f32 vectors; sharded tensors count 1 / world.  Caches and workspaces come on top (a few GB)."""
    import math
    per = {"expert": (17 / 32) if cfg.expert_dtype == "fp4" else 2.0, "table": 1.0, "dense": 2.0, "bf16": 2.0, "f32": 4.0,
           "fp4": 17 / 32, "fp8": 2.0}
    total = 0.0
    for spec in tensor_specs_cached(cfg).values():
        n = math.prod(spec.shape) * per.get(spec.kind, 4.0)
        total += n / world if spec.shard is not None else n
    return int(total)


# ---------------------------------------------------------------------------------------------
# random weights (values already on their storage grid, returned as f32)
# ---------------------------------------------------------------------------------------------
def on_grid(cfg: Dsv41Config, spec: Spec, w: torch.Tensor) -> torch.Tensor:
    """Quantise-dequantise `w` to the storage format of `spec` so that the golden model and a
    device model that re-quantises the same values see identical weights."""
    kind = spec.kind
    if kind == "expert":
        kind = "fp4" if cfg.expert_dtype == "fp4" else "dense"
    if kind == "dense":
        kind = "fp8" if cfg.dense_dtype == "fp8" else "bf16"
    if kind == "fp4":
        return Q.dequant_fp4_weight(*Q.quant_fp4_weight(w, cfg.fp4_block), cfg.fp4_block)
    if kind == "fp8":
        return Q.dequant_fp8_weight(*Q.quant_fp8_weight(w, cfg.fp8_block), cfg.fp8_block)
    if kind == "table":
        return Q.fp8_act_roundtrip(w, cfg.fp8_block)
    if kind == "bf16":
        return w.to(torch.bfloat16).float()
    return w.float()


def random_weights(cfg: Dsv41Config, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in tensor_specs(cfg).items():
        shp = spec.shape
        if spec.init == "ones":
            w = 1.0 + 0.1 * torch.randn(shp, generator=g)
        elif spec.init == "zeros":
            w = torch.zeros(shp)
        elif spec.init == "small":
            w = 0.1 * torch.randn(shp, generator=g)
        elif spec.init == "bias":
            w = 0.05 * torch.randn(shp, generator=g)
        else:
            fan_in = shp[-1]
            w = torch.randn(shp, generator=g) * (fan_in ** -0.5)
            if name.endswith("embed.weight") and "engram" not in name and "markov" not in name:
                w = torch.randn(shp, generator=g)
        out[name] = on_grid(cfg, spec, w)
    return out
