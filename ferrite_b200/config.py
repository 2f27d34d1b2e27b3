"""Typed configuration for the engine and both model families.

One config object is parsed once and handed down; no call site reads the
environment.  The GLM-5.3-Flash dimensions follow the reference's
``crates/ferrite-model/src/config.rs:111-372`` (production values at
``:320-372``, the 4-layer test shape at ``:259-312``); the per-layer role table
follows ``crates/ferrite-model/src/layer.rs:8-61``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from typing import List, Optional

LINEAR = "linear_attention"
DSA = "deepseek_sparse_attention"
DENSE = "dense"
MOE = "sparse"


@dataclass
class LinearAttnConfig:
    num_heads: int = 64
    head_dim: int = 128
    gate_lower_bound: float = -5.0
    conv_kernel: int = 4
    low_rank: int = 128  # rank of the f_a/g_a bottleneck projections
    chunk: int = 64  # WY chunk length used by the prefill scan

    @property
    def proj(self) -> int:
        return self.num_heads * self.head_dim


@dataclass
class DsaConfig:
    num_heads: int = 64
    kv_lora_rank: int = 512
    q_lora_rank: int = 1536
    qk_nope_head_dim: int = 256
    qk_rope_head_dim: int = 0
    v_head_dim: int = 256
    index_n_heads: int = 32
    index_head_dim: int = 128
    index_topk: int = 2048
    index_kpool: int = 4
    page_size: int = 16

    @property
    def select_pools(self) -> int:
        return self.index_topk // self.index_kpool

    @property
    def idx_width(self) -> int:
        """Width of the expanded token-index row: selected pools x kpool + tail."""
        return self.select_pools * self.index_kpool + (self.index_kpool - 1)


@dataclass
class GlmConfig:
    hidden_size: int = 4096
    num_layers: int = 45
    vocab_size: int = 154880
    rms_norm_eps: float = 1e-5
    swiglu_limit: float = 10.0
    max_position_embeddings: int = 1048576
    layer_types: List[str] = field(default_factory=list)
    mlp_types: List[str] = field(default_factory=list)
    intermediate_size: int = 12288
    moe_intermediate_size: int = 2048
    n_routed_experts: int = 288
    n_shared_experts: int = 1
    num_experts_per_tok: int = 8
    routed_scaling_factor: float = 2.5
    linear_attn: LinearAttnConfig = field(default_factory=LinearAttnConfig)
    dsa: DsaConfig = field(default_factory=DsaConfig)
    mhc: bool = True
    hc_mult: int = 4
    hc_eps: float = 1e-6
    hc_sinkhorn_iters: int = 20
    num_nextn_predict_layers: int = 1
    name: str = "glm-5.3-flash"

    # ---- derived -------------------------------------------------------
    @property
    def hc_mix(self) -> int:
        n = self.hc_mult
        return (2 + n) * n

    def is_dsa(self, i: int) -> bool:
        return i >= self.num_layers or self.layer_types[i] == DSA

    def is_moe(self, i: int) -> bool:
        return i >= self.num_layers or self.mlp_types[i] == MOE

    @property
    def dsa_layers(self) -> List[int]:
        return [i for i in range(self.num_layers) if self.layer_types[i] == DSA]

    @property
    def linear_layers(self) -> List[int]:
        return [i for i in range(self.num_layers) if self.layer_types[i] == LINEAR]

    def dsa_family(self, layer: int) -> int:
        """Index of a DSA layer's KV cache; the MTP layer owns the last family."""
        if layer >= self.num_layers:
            return len(self.dsa_layers) + (layer - self.num_layers)
        return self.dsa_layers.index(layer)

    @property
    def n_dsa_families(self) -> int:
        return len(self.dsa_layers) + self.num_nextn_predict_layers

    def validate(self) -> "GlmConfig":
        assert len(self.layer_types) == self.num_layers
        assert len(self.mlp_types) == self.num_layers
        assert self.dsa.qk_rope_head_dim == 0, "GLM DSA is nope-only MLA"
        assert self.dsa.index_topk % self.dsa.index_kpool == 0
        return self

    # ---- constructors ---------------------------------------------------
    @staticmethod
    def production() -> "GlmConfig":
        lt = [DSA if i % 4 == 3 else LINEAR for i in range(45)]
        mt = [DENSE if i < 3 else MOE for i in range(45)]
        return GlmConfig(layer_types=lt, mlp_types=mt).validate()

    @staticmethod
    def tiny() -> "GlmConfig":
        """The reference's 4-layer CPU test shape (hidden 128)."""
        return GlmConfig(
            hidden_size=128, num_layers=4, vocab_size=512, max_position_embeddings=4096,
            layer_types=[LINEAR, DSA, LINEAR, DSA], mlp_types=[DENSE, DENSE, MOE, MOE],
            intermediate_size=256, moe_intermediate_size=64, n_routed_experts=8,
            num_experts_per_tok=2,
            linear_attn=LinearAttnConfig(num_heads=4, head_dim=32, low_rank=16, chunk=16),
            dsa=DsaConfig(num_heads=4, kv_lora_rank=64, q_lora_rank=128, qk_nope_head_dim=32,
                          v_head_dim=32, index_n_heads=2, index_head_dim=16, index_topk=128,
                          index_kpool=2),
            num_nextn_predict_layers=1, name="glm-tiny",
        ).validate()

    @staticmethod
    def golden4() -> "GlmConfig":
        """4-layer GLM-shaped golden config: [GDN+dense, DSA+dense, GDN+MoE, DSA+MoE],
        hidden 256, 4 heads x 64, conv 4, chunk 32, latent 64, indexer top-k 32,
        page 16, 8 experts top-2, expert FFN 512, vocab 4096."""
        return GlmConfig(
            hidden_size=256, num_layers=4, vocab_size=4096, max_position_embeddings=8192,
            layer_types=[LINEAR, DSA, LINEAR, DSA], mlp_types=[DENSE, DENSE, MOE, MOE],
            intermediate_size=512, moe_intermediate_size=512, n_routed_experts=8,
            num_experts_per_tok=2,
            linear_attn=LinearAttnConfig(num_heads=4, head_dim=64, low_rank=32, chunk=32),
            dsa=DsaConfig(num_heads=4, kv_lora_rank=64, q_lora_rank=128, qk_nope_head_dim=64,
                          v_head_dim=64, index_n_heads=2, index_head_dim=32, index_topk=32,
                          index_kpool=4, page_size=16),
            num_nextn_predict_layers=1, name="glm-golden4",
        ).validate()

    @staticmethod
    def scaled(num_layers: int, **kw) -> "GlmConfig":
        """Production dims with fewer layers (for memory-bounded tests)."""
        c = GlmConfig.production()
        c.num_layers = num_layers
        c.layer_types = c.layer_types[:num_layers]
        c.mlp_types = c.mlp_types[:num_layers]
        for k, v in kw.items():
            setattr(c, k, v)
        return c.validate()

    @staticmethod
    def from_hf(path_or_dict) -> "GlmConfig":
        """Parse an HF ``config.json`` (optionally nested under ``text_config``)."""
        raw = path_or_dict
        if not isinstance(raw, dict):
            with open(path_or_dict) as f:
                raw = json.load(f)
        raw = raw.get("text_config", raw)
        g = raw.get
        n = int(g("num_hidden_layers", 45))
        lt = g("layer_types") or [DSA if i % 4 == 3 else LINEAR for i in range(n)]
        mt = g("mlp_layer_types")
        if mt is None:
            k = int(g("first_k_dense_replace", 3))
            mt = [DENSE if i < k else MOE for i in range(n)]
        la = LinearAttnConfig(
            num_heads=int(g("linear_num_heads", g("linear_num_value_heads", 64))),
            head_dim=int(g("linear_head_dim", g("linear_value_head_dim", 128))),
            gate_lower_bound=float(g("gate_lower_bound", -5.0)),
            conv_kernel=int(g("short_conv_kernel_size", g("linear_conv_kernel_dim", 4))),
            low_rank=int(g("linear_gate_low_rank", 128)),
        )
        ds = DsaConfig(
            num_heads=int(g("num_attention_heads", 64)), kv_lora_rank=int(g("kv_lora_rank", 512)),
            q_lora_rank=int(g("q_lora_rank", 1536)), qk_nope_head_dim=int(g("qk_nope_head_dim", 256)),
            qk_rope_head_dim=int(g("qk_rope_head_dim", 0)), v_head_dim=int(g("v_head_dim", 256)),
            index_n_heads=int(g("index_n_heads", 32)), index_head_dim=int(g("index_head_dim", 128)),
            index_topk=int(g("index_topk", 2048)), index_kpool=int(g("index_kpool", 4)),
        )
        return GlmConfig(
            hidden_size=int(g("hidden_size", 4096)), num_layers=n, vocab_size=int(g("vocab_size", 154880)),
            rms_norm_eps=float(g("rms_norm_eps", 1e-5)), swiglu_limit=float(g("swiglu_limit", 10.0)),
            max_position_embeddings=int(g("max_position_embeddings", 1048576)),
            layer_types=list(lt), mlp_types=list(mt), intermediate_size=int(g("intermediate_size", 12288)),
            moe_intermediate_size=int(g("moe_intermediate_size", 2048)),
            n_routed_experts=int(g("n_routed_experts", 288)), n_shared_experts=int(g("n_shared_experts", 1)),
            num_experts_per_tok=int(g("num_experts_per_tok", 8)),
            routed_scaling_factor=float(g("routed_scaling_factor", 2.5)), linear_attn=la, dsa=ds,
            mhc=bool(g("mhc", True)), hc_mult=int(g("hc_mult", 4)), hc_eps=float(g("hc_eps", 1e-6)),
            hc_sinkhorn_iters=int(g("hc_sinkhorn_iters", 20)),
            num_nextn_predict_layers=int(g("num_nextn_predict_layers", 1)),
        ).validate()

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass
class SchedConfig:
    """Planner defaults (reference ``crates/ferrite-dispatch/src/batch.rs:109-146``)."""
    max_rows: int = 32
    prefill_budget: int = 512
    page_size: int = 16
    num_pages: int = 122880
    device_slots: int = 512
    host_slots: int = 4096
    disk_slots: int = 65536
    buckets: tuple = (1, 2, 4, 8, 16, 32)


@dataclass
class EngineConfig:
    """Everything the runtime needs that is not a model dimension."""
    tp: int = 1
    ep: int = 1
    dcp: int = 1
    max_ctx: int = 8192
    max_batch: int = 1
    mtp_n: int = 3  # verify rows; draft depth is mtp_n - 1 (0/1 disables MTP)
    use_graphs: bool = True
    fp8_experts: bool = True
    experts_resident: Optional[int] = None  # None = all routed experts of the shard
    # how the routed experts are split over the tensor-parallel ranks: "inter" = every rank holds a 1/tp slice of
    # every expert's intermediate dim; "expert" = every rank holds E/tp whole experts (activations stay replicated,
    # a rank computes the pairs routed to its experts, the sublayer's all-reduce sums the ranks: expert parallelism
    # without an all-to-all; longer weight rows per expert, load follows the routing)
    moe_shard: str = "inter"
    kv_dtype: str = "bf16"  # latent cache dtype: "bf16" or "fp8"
    # epilogue of a sublayer's last GEMV: "full" = all-reduce + hyper-connection fold in the same kernel,
    # "ar" = all-reduce only, "off" = separate kernels (True / False are accepted for full / off)
    fuse_epilogue: object = "full"
    collective: str = "p2p"  # "p2p" (fused peer-memory kernels) or "nccl"
    ar_max_spins: int = 2_000_000   # polls of a bounded device wait (about two seconds)
    seed: int = 0
    sched: SchedConfig = field(default_factory=SchedConfig)
    debug_sync: bool = False
    prefill_chunk: int = 512
