"""Real-checkpoint checks, skipped unless a checkpoint directory is named by the environment (the counterpart of the
reference's ``DSV41_MODEL_DIR``-gated tests, ``crates/ferrite-dsv41/tests/real_checkpoint.rs``):

    FERRITE_GLM_MODEL_DIR=/ckpt/glm-5.3-flash     python -m pytest tests/test_real_checkpoint.py
    FERRITE_DSV41_MODEL_DIR=/ckpt/dsv41-flash     python -m pytest tests/test_real_checkpoint.py

They read headers and a handful of tensors only (CPU, no GPU): every tensor the model needs is present with the
shape its layout states, block-scaled tensors dequantise to finite values, and the config file agrees with the
built-in production configuration.
"""
import math
import os

import pytest
import torch

GLM_DIR = os.environ.get("FERRITE_GLM_MODEL_DIR", "")
D4_DIR = os.environ.get("FERRITE_DSV41_MODEL_DIR", "")


def one_of_each_kind(names):
    """The first tensor of every name pattern (layer / expert indices aside): every KIND of tensor is read once."""
    import re
    seen, out = set(), []
    for k in names:
        kind = re.sub(r"\d+", "N", k)
        if kind not in seen:
            seen.add(kind)
            out.append(k)
    return out


def test_one_of_each_kind_covers_every_pattern_of_the_tiny_layout():
    from ferrite_b200.config import GlmConfig
    from ferrite_b200.models.glm_weights import weight_layout
    layout = weight_layout(GlmConfig.tiny())
    picks = one_of_each_kind(layout)
    assert 20 < len(picks) < len(layout) and "model.embed_tokens.weight" in picks
    assert any(".experts.0." in k for k in picks) and not any(".experts.1." in k for k in picks)


@pytest.mark.skipif(not GLM_DIR, reason="FERRITE_GLM_MODEL_DIR not set")
def test_glm_checkpoint_has_every_tensor_of_the_layout():
    from ferrite_b200.config import GlmConfig
    from ferrite_b200.models.checkpoint import CheckpointSource
    from ferrite_b200.models.glm_weights import weight_layout
    cfg_path = os.path.join(GLM_DIR, "config.json")
    cfg = GlmConfig.from_hf(cfg_path) if os.path.exists(cfg_path) else GlmConfig.production()
    prod = GlmConfig.production()
    assert (cfg.hidden_size, cfg.num_layers, cfg.n_routed_experts) == (prod.hidden_size, prod.num_layers, prod.n_routed_experts)
    src = CheckpointSource(GLM_DIR, cfg)
    layout = weight_layout(cfg)
    for k in one_of_each_kind(layout):
        t = src.get(k)                          # raises for a tensor the checkpoint (or its name map) does not have
        assert tuple(t.shape) == tuple(layout[k]), (k, tuple(t.shape), layout[k])
        assert torch.isfinite(t.float()).all(), k


@pytest.mark.skipif(not D4_DIR, reason="FERRITE_DSV41_MODEL_DIR not set")
def test_dsv41_checkpoint_has_every_tensor_of_the_specs():
    from ferrite_b200.models.dsv41_checkpoint import Dsv41CheckpointSource
    from ferrite_b200.models.dsv41_config import Dsv41Config
    from ferrite_b200.models.dsv41_weights import tensor_specs
    cfg_path = os.path.join(D4_DIR, "config.json")
    cfg = Dsv41Config.from_hf(cfg_path) if os.path.exists(cfg_path) else Dsv41Config.flash()
    src = Dsv41CheckpointSource(D4_DIR, cfg)
    specs = tensor_specs(cfg)
    missing = [k for k in specs if not src.has(k)]
    assert not missing, missing[:8]
    small = [k for k, s in specs.items() if math.prod(s.shape) <= 64 * 1024 * 1024 and ".layers.0." in k][:16]
    for k in small:
        t = src.get(k)
        assert tuple(t.shape) == tuple(specs[k].shape), (k, tuple(t.shape), specs[k].shape)
        assert torch.isfinite(t.float()).all(), k
