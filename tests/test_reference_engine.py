"""CPU: the fp32 reference engine agrees with itself across execution strategies
(the reference's T3/T4 tiers: chunked == single-shot, tpN == tp1, spec == greedy)."""
import torch

from ferrite_b200.config import GlmConfig
from ferrite_b200.models.glm_ref import GlmReference
from ferrite_b200.models.glm_weights import (apply_fused_aliases, checkpoint_sources, random_weights,
                                             shard_weight, weight_layout)
from ferrite_b200.ops import reference as R
from ferrite_b200.spec import spec_accept


def _prompt(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_chunked_prefill_equals_single_shot():
    cfg = GlmConfig.tiny()
    m = GlmReference(cfg, random_weights(cfg, 0, std=0.05))
    p = _prompt(cfg, 37)
    a, _ = m.generate(p, 10)
    b, _ = m.generate(p, 10, chunk=8)
    assert a == b


def test_tp_equals_single_rank():
    cfg = GlmConfig.tiny()
    w = random_weights(cfg, 0, std=0.05)
    p = _prompt(cfg, 21)
    a, _ = GlmReference(cfg, w).generate(p, 8)
    for world in (2, 4):
        b, _ = GlmReference(cfg, w, world=world).generate(p, 8)
        assert a == b, world


def test_wy_chunk_equals_recurrence():
    g = torch.Generator().manual_seed(3)
    n, h, dk = 70, 3, 16
    q, k, v = (torch.randn(n, h, dk, generator=g) for _ in range(3))
    q, k = R.l2norm_heads(q), R.l2norm_heads(k)
    beta = torch.rand(n, h, generator=g)
    gl = -5 * torch.rand(n, h, dk, generator=g)
    s0 = torch.randn(h, dk, dk, generator=g) * 0.1
    o1, s1 = R.gdn_recurrent(q, k, v, beta, gl, s0)
    o2, s2 = R.gdn_chunk_wy(q, k, v, beta, gl, s0, 32)
    assert torch.allclose(o1, o2, atol=2e-4, rtol=1e-3)
    assert torch.allclose(s1, s2, atol=2e-4, rtol=1e-3)


def test_mtp_equals_greedy():
    cfg = GlmConfig.tiny()
    m = GlmReference(cfg, random_weights(cfg, 0, std=0.05))
    p = _prompt(cfg, 19)
    a, _ = m.generate(p, 12)
    b, acc = m.generate(p, 12, mtp=True)
    assert a == b
    assert all(1 <= k <= 3 for k in acc)


def test_golden4_config_runs():
    cfg = GlmConfig.golden4()
    m = GlmReference(cfg, random_weights(cfg, 0))
    out, _ = m.generate(_prompt(cfg, 128, seed=0), 8, chunk=32)
    assert len(out) == 8 and all(0 <= t < cfg.vocab_size for t in out)


def test_spec_accept_exhaustive():
    import itertools
    for nd in range(0, 4):
        for d in itertools.product(range(2), repeat=nd):
            for j in itertools.product(range(2), repeat=nd + 1):
                want = 0
                while want < nd and d[want] == j[want]:
                    want += 1
                assert spec_accept(d, j, True) == want + 1
                assert spec_accept(d, j[:nd], False) == want
                assert spec_accept(d, j[:nd], False) + 1 == spec_accept(d, list(j[:nd]) + [9], True)


def test_dcp_partial_merge_equals_full():
    g = torch.Generator().manual_seed(5)
    n, h, d, T, page = 3, 2, 8, 50, 4
    q = torch.randn(n, h, d, generator=g)
    k = torch.randn(T, h, d, generator=g)
    v = torch.randn(T, h, d, generator=g)
    idx = torch.stack([torch.randperm(T, generator=g)[:20] for _ in range(n)])
    idx[0, 3] = -1
    idx[1, 5] = idx[1, 6]
    full = R.sparse_mla_attn(q, k, v, idx)
    for shards in (2, 4):
        outs, lses = [], []
        for owned_ids in R.split_pages_round_robin(T, page, shards):
            owned = torch.zeros(T, dtype=torch.bool)
            owned[owned_ids] = True
            o, l = R.sparse_attn_partial(q, k, v, idx, owned)
            outs.append(o)
            lses.append(l)
        assert torch.allclose(R.lse_merge(outs, lses), full, atol=1e-5)


def test_layout_aliases_and_shards():
    cfg = GlmConfig.tiny()
    lay = weight_layout(cfg)
    assert "model.layers.4.eh_proj.weight" in lay and "model.layers.0.hc_attn_fn" in lay
    assert lay["model.layers.0.hc_attn_fn"] == (24, 4 * cfg.hidden_size)
    w = random_weights(cfg, 0)
    a = "model.layers.0.self_attn."
    fused = {a + "fused_qkvbfg_a_proj.weight": torch.cat([w[a + "qkv_proj.weight"], w[a + "b_proj.weight"],
                                                         w[a + "f_a_proj.weight"], w[a + "g_a_proj.weight"]], 0),
             a + "fused_fg_b_proj.weight": torch.stack([w[a + "f_b_proj.weight"], w[a + "g_b_proj.weight"]], 0),
             "model.layers.0.mlp.gate_up_proj.weight": torch.cat([w["model.layers.0.mlp.gate_proj.weight"],
                                                                   w["model.layers.0.mlp.up_proj.weight"]], 0)}
    out = apply_fused_aliases(dict(fused), cfg)
    for nm in ("qkv_proj", "b_proj", "f_a_proj", "g_a_proj", "f_b_proj", "g_b_proj"):
        assert torch.equal(out[a + nm + ".weight"], w[a + nm + ".weight"])
    assert torch.equal(out["model.layers.0.mlp.up_proj.weight"], w["model.layers.0.mlp.up_proj.weight"])
    mk, srcs = checkpoint_sources(a + "qkv_proj.weight")
    assert mk == "__FUSED_QKV__" and srcs[0].startswith("model.language_model.layers.0.self_attn.q_proj")
    assert checkpoint_sources("model.layers.2.mlp.shared_expert.up_proj.weight")[1][0].count("shared_experts") == 1
    q = w[a + "qkv_proj.weight"]
    s = shard_weight(a + "qkv_proj.weight", q, 1, 2)
    P = cfg.linear_attn.proj
    assert torch.equal(s[: P // 2], q[P // 2: P])
