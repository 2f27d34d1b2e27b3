"""CPU: safetensors reader (mmap views, byte-range shard copies, fp8 block dequant), name
mapping with fused q/k/v and aliases, corrupted-header detection, checkpoint == in-memory model."""
import os
import struct

import pytest
import torch

from ferrite_b200.config import GlmConfig
from ferrite_b200.models.checkpoint import (CheckpointIndex, CheckpointSource, save_internal_checkpoint,
                                            write_safetensors)
from ferrite_b200.models.glm_ref import GlmReference
from ferrite_b200.models.glm_weights import random_weights
from ferrite_b200.ops.reference import dequant_fp8_block, quant_fp8_block


def test_reader_views_rows_and_fp8(tmp_path):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(300, 260, generator=g)
    q, s = quant_fp8_block(a)
    b = torch.randn(7, 5, generator=g).bfloat16()
    write_safetensors(str(tmp_path / "m.safetensors"), {"a.weight": q, "a.weight_scale_inv": s, "b": b, "i": torch.arange(6)})
    idx = CheckpointIndex(str(tmp_path))
    assert torch.equal(idx.view("b"), b) and torch.equal(idx.view("i"), torch.arange(6))
    assert torch.equal(idx.rows("b", 2, 6, 1, 4), b[2:6, 1:4])
    full = dequant_fp8_block(q, s)
    assert torch.equal(idx.dequant_fp8("a.weight", "a.weight_scale_inv"), full)
    assert torch.equal(idx.dequant_fp8("a.weight", "a.weight_scale_inv", 128, 256), full[128:256])


def test_corrupt_header_is_reported(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(Exception):
        CheckpointIndex(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 9) + b'{"x": [1}' + b"\0" * 16)
    with pytest.raises(ValueError):
        CheckpointIndex(str(tmp_path))


def test_checkpoint_source_equals_in_memory_weights(tmp_path):
    cfg = GlmConfig.tiny()
    w = {k: (v.bfloat16().float() if v.dim() > 1 else v) for k, v in random_weights(cfg, 0, std=0.05).items()}
    save_internal_checkpoint(str(tmp_path / "model.safetensors"), w)
    src = CheckpointSource(str(tmp_path), cfg)
    assert "model.language_model.layers.0.self_attn.q_proj.weight" in src.idx
    assert "model.language_model.layers.2.mlp.shared_experts.up_proj.weight" in src.idx
    loaded = {k: src.get(k).float() for k in w}
    for k in w:
        assert torch.equal(loaded[k], w[k]), k
    prompt = list(range(5, 30))
    a, _ = GlmReference(cfg, w).generate(prompt, 6)
    b, _ = GlmReference(cfg, loaded).generate(prompt, 6)
    assert a == b


def test_fused_aliases_and_fp8_experts_on_disk(tmp_path):
    cfg = GlmConfig.tiny()
    w = {k: (v.bfloat16().float() if v.dim() > 1 else v) for k, v in random_weights(cfg, 0, std=0.05).items()}
    out = {}
    for k, v in w.items():
        out["model.language_model." + k[len("model."):] if k.startswith("model.") else k] = v
    a = "model.language_model.layers.0.self_attn."
    fused = torch.cat([out.pop(a + "qkv_proj.weight"), out.pop(a + "b_proj.weight"), out.pop(a + "f_a_proj.weight"),
                       out.pop(a + "g_a_proj.weight")], 0)
    out[a + "fused_qkvbfg_a_proj.weight"] = fused
    out[a + "fused_fg_b_proj.weight"] = torch.stack([out.pop(a + "f_b_proj.weight"), out.pop(a + "g_b_proj.weight")], 0)
    m = "model.language_model.layers.0.mlp."
    out[m + "gate_up_proj.weight"] = torch.cat([out.pop(m + "gate_proj.weight"), out.pop(m + "up_proj.weight")], 0)
    e = "model.language_model.layers.2.mlp.experts.3.down_proj.weight"
    q, s = quant_fp8_block(out[e])
    out[e], out[e + "_scale_inv"] = q, s
    write_safetensors(str(tmp_path / "model.safetensors"), out)
    src = CheckpointSource(str(tmp_path), cfg)
    for leaf in ("qkv_proj", "b_proj", "f_a_proj", "g_a_proj", "f_b_proj", "g_b_proj"):
        k = f"model.layers.0.self_attn.{leaf}.weight"
        assert torch.equal(src.get(k).float(), w[k]), k
    assert torch.equal(src.get("model.layers.0.mlp.up_proj.weight").float(), w["model.layers.0.mlp.up_proj.weight"])
    k = "model.layers.2.mlp.experts.3.down_proj.weight"
    assert torch.equal(src.get(k), dequant_fp8_block(q, s))
    q2, s2 = src.get_fp8(k)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)
    assert src.get_fp8("model.layers.2.mlp.experts.2.down_proj.weight") is None


def test_bad_scale_tensors_and_sizes_are_refused(tmp_path):
    g = torch.Generator().manual_seed(1)
    a = torch.randn(300, 260, generator=g)
    q, s = quant_fp8_block(a)
    d = tmp_path / "short"
    d.mkdir()
    write_safetensors(str(d / "m.safetensors"), {"a.weight": q, "a.weight_scale_inv": s[:2].contiguous()})
    idx = CheckpointIndex(str(d))
    with pytest.raises(ValueError, match="scale shape"):      # a truncated scale tensor never reaches the reader
        idx.dequant_fp8("a.weight", "a.weight_scale_inv")
    d = tmp_path / "bf16"
    d.mkdir()
    write_safetensors(str(d / "m.safetensors"), {"a.weight": q, "a.weight_scale_inv": s.bfloat16()})
    idx = CheckpointIndex(str(d))
    want = dequant_fp8_block(q, s.bfloat16().float())
    assert torch.equal(idx.dequant_fp8("a.weight", "a.weight_scale_inv"), want)   # bf16 scales: torch path, not a reinterpret
    # an entry whose byte range disagrees with shape x dtype is refused when the index is built
    d = tmp_path / "size"
    d.mkdir()
    import json
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 32]}}).encode()
    (d / "m.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 64)
    with pytest.raises(ValueError, match="bytes for shape"):
        CheckpointIndex(str(d))
    # the C++ reader bounds-checks the scale range itself
    from ferrite_b200 import _runtime as rt
    d = tmp_path / "ok"
    d.mkdir()
    write_safetensors(str(d / "m.safetensors"), {"a.weight": q, "a.weight_scale_inv": s})
    idx = CheckpointIndex(str(d))
    ti, si = idx.tensors["a.weight"], idx.tensors["a.weight_scale_inv"]
    with pytest.raises(Exception):
        ti.file.dequant_e4m3_block(ti.begin, si.end - 8, 300, 260, 128, 0, 300)


def test_flat_fused_fg_b_alias(tmp_path):
    cfg = GlmConfig.tiny()
    w = {k: (v.bfloat16().float() if v.dim() > 1 else v) for k, v in random_weights(cfg, 0, std=0.05).items()}
    out = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v for k, v in w.items()}
    a = "model.language_model.layers.0.self_attn."
    out[a + "fused_fg_b_proj.weight"] = torch.cat([out.pop(a + "f_b_proj.weight"), out.pop(a + "g_b_proj.weight")], 0)
    write_safetensors(str(tmp_path / "model.safetensors"), out)
    src = CheckpointSource(str(tmp_path), cfg)
    for leaf in ("f_b_proj", "g_b_proj"):
        k = f"model.layers.0.self_attn.{leaf}.weight"
        assert torch.equal(src.get(k).float(), w[k]), k
