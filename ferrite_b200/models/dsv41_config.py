"""Configuration of the DeepSeek-V4.1-Flash-style model family ("DSV41").

Field names follow the reference's ``ModelArgs`` (``ref_inference/model.py:45-149``); the
production values are those of ``crates/ferrite-models/configs/dsv41_flash.json`` and
``from_hf`` reads that file's layout (``text_config`` / ``vision_config``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, replace
from typing import Optional, Tuple


@dataclass(frozen=True)
class VisionConfig:
    n_layers: int = 32
    dim: int = 1024
    n_heads: int = 16
    inter_dim: int = 2816
    patch_size: int = 14
    rope_theta: float = 10000.0
    downsample_ratio: int = 3
    max_image_tokens: int = 1024
    norm_eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @staticmethod
    def tiny() -> "VisionConfig":
        return VisionConfig(n_layers=2, dim=128, n_heads=4, inter_dim=192, patch_size=4, downsample_ratio=2,
                            max_image_tokens=16)


@dataclass(frozen=True)
class Dsv41Config:
    vocab_size: int = 129280
    dim: int = 5120
    moe_inter_dim: int = 2304
    n_layers: int = 40
    n_mtp_layers: int = 3
    n_heads: int = 64
    head_dim: int = 512
    rope_head_dim: int = 64
    q_lora_rank: int = 1280
    o_lora_rank: int = 1024
    o_groups: int = 8
    swiglu_limit: float = 10.0
    norm_eps: float = 1e-20
    # MoE
    n_routed_experts: int = 384
    n_shared_experts: int = 1
    n_activated_experts: int = 6
    route_scale: float = 1.5
    dspark_n_routed_experts: int = 128
    dspark_n_activated_experts: int = 3
    # attention: sliding window + compressed KV with an indexer
    window_size: int = 128
    compress_ratios: Tuple[int, ...] = tuple([0, 0] + [2] * 18 + [1] * 20 + [0, 0, 0])
    kv_source_layers: Tuple[int, ...] = (2, 8, 14, 20)
    index_source_layers: Tuple[int, ...] = (2, 8, 14, 20, 24, 28, 32, 36)
    index_n_heads: int = 32
    index_head_dim: int = 128
    index_topk: int = 512
    candidate_source_layer: int = 20
    candidate_topk_blocks: int = 2048
    candidate_block_size: int = 8
    # RoPE / YaRN
    rope_theta: float = 10000.0
    compress_rope_theta: float = 160000.0
    rope_factor: float = 16.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_seq_len: int = 65536
    max_seq_len: int = 1048576
    # hyper-connections
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    # engram (n-gram hash memory)
    engram_layer_ids: Tuple[int, ...] = (1, 14)
    engram_num_embeddings: Tuple[int, ...] = (384006168, 384016682)
    engram_max_ngram_size: int = 4
    engram_vocab_size: int = 16000000
    engram_n_heads: int = 8
    engram_head_dim: int = 256
    engram_pad_id: int = 2
    engram_compressed_vocab_size: int = 99092
    # DSpark speculative draft
    dspark_block_size: int = 5
    dspark_noise_token_id: int = 128799
    dspark_target_layer_ids: Tuple[int, ...] = (37, 38, 39)
    dspark_markov_rank: int = 256
    # formats
    fp8_block: int = 32
    fp4_block: int = 32
    expert_dtype: str = "fp4"   # "fp4" | "fp8"
    dense_dtype: str = "fp8"    # "fp8" | "bf16"
    # multimodal
    image_token_id: int = 129264
    vision: Optional[VisionConfig] = None
    bos_id: int = 0
    eos_id: int = 1
    pad_id: int = 2

    # ---- derived ---------------------------------------------------------------------------
    @property
    def n_total_layers(self) -> int:
        return self.n_layers + self.n_mtp_layers

    @property
    def nope_head_dim(self) -> int:
        return self.head_dim - self.rope_head_dim

    @property
    def heads_per_group(self) -> int:
        return self.n_heads // self.o_groups

    def ratio(self, layer: int) -> int:
        return self.compress_ratios[layer]

    def is_kv_source(self, layer: int) -> bool:
        return layer < self.n_layers and layer in self.kv_source_layers

    def is_index_source(self, layer: int) -> bool:
        return layer < self.n_layers and layer in self.index_source_layers

    def kv_source_of(self, layer: int) -> int:
        """The layer whose compressed KV / index keys `layer` reads (nearest source at or below)."""
        src = [s for s in self.kv_source_layers if s <= layer]
        assert src and self.ratio(layer) > 0, f"layer {layer} reads no compressed KV"
        return src[-1]

    def index_source_of(self, layer: int) -> int:
        src = [s for s in self.index_source_layers if s <= layer]
        assert src and self.ratio(layer) > 0, f"layer {layer} has no index source"
        return src[-1]

    def uses_candidates(self, layer: int) -> bool:
        return 0 <= self.candidate_source_layer < layer and self.is_index_source(layer)

    def moe_shape(self, layer: int) -> Tuple[int, int]:
        """(routed experts, activated experts) of a layer; DSpark layers have their own."""
        if layer >= self.n_layers:
            return self.dspark_n_routed_experts, self.dspark_n_activated_experts
        return self.n_routed_experts, self.n_activated_experts

    def engram_index(self, layer: int) -> int:
        return self.engram_layer_ids.index(layer) if layer in self.engram_layer_ids else -1

    @property
    def engram_hash_cols(self) -> int:
        return (self.engram_max_ngram_size - 1) * self.engram_n_heads

    def validate(self) -> "Dsv41Config":
        assert len(self.compress_ratios) == self.n_total_layers, "one compress ratio per layer (MTP included)"
        assert self.n_heads % self.o_groups == 0 and self.rope_head_dim % 2 == 0
        assert self.head_dim % self.fp8_block == 0 and self.index_head_dim % self.fp4_block == 0
        for l in range(self.n_layers):
            if self.ratio(l) > 0:
                s = self.kv_source_of(l)
                assert self.ratio(s) == self.ratio(l), f"layer {l} and its KV source {s} differ in ratio"
                self.index_source_of(l)
        for l in self.kv_source_layers:
            assert self.ratio(l) > 0 and self.is_index_source(l), "a KV source owns index keys and runs an indexer"
        for l in range(self.n_layers, self.n_total_layers):
            assert self.ratio(l) == 0, "DSpark layers are window-only"
        return self

    # ---- constructors ----------------------------------------------------------------------
    @staticmethod
    def flash() -> "Dsv41Config":
        return Dsv41Config().validate()

    @staticmethod
    def tiny(vision: bool = False, **over) -> "Dsv41Config":
        """A few-layer model that exercises every branch: window-only layers, ratio-2 and ratio-1
        compressed layers, a source and an inheriting layer of each, candidate blocks, an engram
        layer, DSpark with two target layers."""
        cfg = Dsv41Config(
            vocab_size=512, dim=128, moe_inter_dim=64, n_layers=7, n_mtp_layers=2, n_heads=4, head_dim=64,
            rope_head_dim=16, q_lora_rank=64, o_lora_rank=32, o_groups=2,
            n_routed_experts=8, n_activated_experts=2, dspark_n_routed_experts=4, dspark_n_activated_experts=2,
            window_size=8, compress_ratios=(0, 2, 2, 1, 1, 1, 1, 0, 0), kv_source_layers=(1, 3),
            index_source_layers=(1, 3, 5), index_n_heads=4, index_head_dim=32, index_topk=6,
            candidate_source_layer=3, candidate_topk_blocks=3, candidate_block_size=2,
            original_seq_len=64, max_seq_len=512,
            engram_layer_ids=(1,), engram_num_embeddings=(0,), engram_max_ngram_size=3, engram_vocab_size=50,
            engram_n_heads=2, engram_head_dim=32, engram_compressed_vocab_size=512,
            dspark_block_size=3, dspark_noise_token_id=500, dspark_target_layer_ids=(5, 6), dspark_markov_rank=16,
            image_token_id=510, vision=VisionConfig.tiny() if vision else None,
        )
        cfg = replace(cfg, **over)
        if cfg.engram_layer_ids and cfg.engram_num_embeddings == (0,):
            from .dsv41_engram import EngramLayout
            cfg = replace(cfg, engram_num_embeddings=EngramLayout.from_config(cfg).table_rows)
        return cfg.validate()

    @staticmethod
    def from_hf(path: str) -> "Dsv41Config":
        with open(path) as f:
            j = json.load(f)
        t = j.get("text_config", j)
        q = j.get("quantization_config", {})
        rs = t.get("rope_scaling") or {}
        v = j.get("vision_config")
        vision = None
        if v:
            vision = VisionConfig(n_layers=v["num_hidden_layers"], dim=v["hidden_size"], n_heads=v["num_attention_heads"],
                                  inter_dim=v["intermediate_size"], patch_size=v["patch_size"],
                                  rope_theta=float(v.get("rope_theta", 10000.0)),
                                  downsample_ratio=v.get("downsample_ratio", 3),
                                  max_image_tokens=v.get("max_image_tokens", 1024))
        blk = (q.get("weight_block_size") or [32, 32])[0]
        return Dsv41Config(
            vocab_size=t["vocab_size"], dim=t["hidden_size"], moe_inter_dim=t["moe_intermediate_size"],
            n_layers=t["num_hidden_layers"], n_mtp_layers=t.get("num_nextn_predict_layers", 0),
            n_heads=t["num_attention_heads"], head_dim=t["head_dim"], rope_head_dim=t["qk_rope_head_dim"],
            q_lora_rank=t["q_lora_rank"], o_lora_rank=t["o_lora_rank"], o_groups=t["o_groups"],
            swiglu_limit=float(t.get("swiglu_limit", 10.0)), norm_eps=float(t["rms_norm_eps"]),
            n_routed_experts=t["n_routed_experts"], n_shared_experts=t.get("n_shared_experts", 1),
            n_activated_experts=t["num_experts_per_tok"], route_scale=float(t["routed_scaling_factor"]),
            dspark_n_routed_experts=t.get("dspark_n_routed_experts", t["n_routed_experts"]),
            dspark_n_activated_experts=t.get("dspark_num_experts_per_tok", t["num_experts_per_tok"]),
            window_size=t["sliding_window"], compress_ratios=tuple(t["compress_ratios"]),
            kv_source_layers=tuple(t["kv_source_layer_ids"]), index_source_layers=tuple(t["index_source_layer_ids"]),
            index_n_heads=t["index_n_heads"], index_head_dim=t["index_head_dim"], index_topk=t["index_topk"],
            candidate_source_layer=t.get("candidate_source_layer_id", -1),
            candidate_topk_blocks=t.get("candidate_topk_blocks", 0), candidate_block_size=t.get("candidate_block_size", 1),
            rope_theta=float(t["rope_theta"]), compress_rope_theta=float(t.get("compress_rope_theta", t["rope_theta"])),
            rope_factor=float(rs.get("factor", 1.0)), beta_fast=float(rs.get("beta_fast", 32)),
            beta_slow=float(rs.get("beta_slow", 1)), original_seq_len=int(rs.get("original_max_position_embeddings", 0)),
            max_seq_len=t.get("max_position_embeddings", 65536),
            hc_mult=t["hc_mult"], hc_sinkhorn_iters=t["hc_sinkhorn_iters"], hc_eps=float(t["hc_eps"]),
            engram_layer_ids=tuple(t.get("engram_layer_ids", ())), engram_num_embeddings=tuple(t.get("engram_num_embeddings", ())),
            engram_max_ngram_size=t.get("engram_max_ngram_size", 4), engram_vocab_size=t.get("engram_vocab_size", 0),
            engram_n_heads=t.get("engram_n_heads", 8), engram_head_dim=t.get("engram_head_dim", 256),
            engram_pad_id=t.get("engram_pad_token_id", 2),
            engram_compressed_vocab_size=t.get("engram_compressed_vocab_size", t["vocab_size"]),
            dspark_block_size=t.get("dspark_block_size", 0), dspark_noise_token_id=t.get("dspark_noise_token_id", 0),
            dspark_target_layer_ids=tuple(t.get("dspark_target_layer_ids", ())),
            dspark_markov_rank=t.get("dspark_markov_rank", 0),
            fp8_block=blk, fp4_block=32, expert_dtype=q.get("expert_dtype", "fp4"),
            dense_dtype="fp8" if q.get("quant_method") == "fp8" else "bf16",
            image_token_id=j.get("image_token_id", 0), vision=vision,
            bos_id=j.get("bos_token_id", 0), eos_id=j.get("eos_token_id", 1), pad_id=j.get("pad_token_id", 2),
        ).validate()
