"""CPU: DSV41 codecs, config, engram hashing and the fp32 golden model's invariants."""
import torch

from ferrite_b200.models.dsv41_config import Dsv41Config
from ferrite_b200.models.dsv41_engram import EngramLayout, NgramHasher
from ferrite_b200.models.dsv41_ref import Dsv41Reference, select_candidate_blocks
from ferrite_b200.models.dsv41_weights import padded_inter, random_weights, shard_tensor, tensor_specs
from ferrite_b200.ops import quant as Q


def test_e2m1_codec_grid_and_ties():
    grid = torch.tensor(Q.E2M1_GRID)
    for sign in (1.0, -1.0):
        v = grid * sign
        assert torch.equal(Q.e2m1_decode(Q.e2m1_encode(v)), v)
    # ties go to the even code: .25->0, .75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert Q.e2m1_decode(Q.e2m1_encode(ties)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]
    codes = torch.randint(0, 16, (4, 64), dtype=torch.uint8)
    assert torch.equal(Q.e2m1_unpack(Q.e2m1_pack(codes)), codes)
    assert int(Q.e2m1_pack(torch.tensor([[3, 9]], dtype=torch.uint8))[0, 0]) == 0x93  # even k in the low nibble


def test_scales_are_powers_of_two_and_roundtrips_bound_error():
    x = torch.randn(8, 128, generator=torch.Generator().manual_seed(0)) * 3
    assert Q.pow2_ceil(torch.tensor([1.0, 1.5, 0.3, 4.0])).tolist() == [1.0, 2.0, 0.5, 4.0]
    assert torch.equal(Q.ue8m0_decode(Q.ue8m0_encode(torch.tensor([0.25, 8.0]))), torch.tensor([0.25, 8.0]))
    y = Q.fp8_act_roundtrip(x, 32)
    assert ((y - x).abs() <= x.abs().amax() * 2 ** -3).all() and (y - x).abs().mean() < 0.1
    assert torch.equal(Q.fp8_act_roundtrip(y, 32), y)  # idempotent
    z = Q.fp4_act_roundtrip(x, 32)
    assert torch.equal(Q.fp4_act_roundtrip(z, 32), z)
    z16 = Q.fp4_act_roundtrip(x, 16, "e4m3")
    assert (z16 - x).abs().mean() < 0.5
    w = torch.randn(64, 96, generator=torch.Generator().manual_seed(1))
    p, s = Q.quant_fp4_weight(w)
    assert p.shape == (64, 48) and s.shape == (64, 3)
    wd = Q.dequant_fp4_weight(p, s)
    assert torch.equal(Q.dequant_fp4_weight(*Q.quant_fp4_weight(wd)), wd)   # on-grid values survive a re-quantisation
    q8, s8 = Q.quant_fp8_weight(w)
    assert s8.shape == (2, 3)
    w8 = Q.dequant_fp8_weight(q8, s8)
    assert (w8 - w).abs().max() < 0.3 and torch.equal(Q.dequant_fp8_weight(*Q.quant_fp8_weight(w8)), w8)


def test_production_config_and_specs():
    cfg = Dsv41Config.flash()
    assert cfg.kv_source_of(7) == 2 and cfg.kv_source_of(39) == 20 and cfg.index_source_of(27) == 24
    assert cfg.uses_candidates(24) and not cfg.uses_candidates(20) and not cfg.uses_candidates(25)
    assert cfg.moe_shape(41) == (128, 3) and cfg.engram_hash_cols == 24
    assert padded_inter(cfg, 8) == 320 and padded_inter(cfg, 4) == 576
    import os
    # optional cross-check against an upstream HF-style config file, named by the environment
    ref = os.environ.get("FERRITE_REF_DSV41_CONFIG", "")
    if ref and os.path.exists(ref):
        c2 = Dsv41Config.from_hf(ref)
        assert (c2.dim, c2.n_layers, c2.n_mtp_layers, c2.compress_ratios) == (5120, 40, 3, cfg.compress_ratios)
        assert c2.vision is not None and c2.vision.n_layers == 32


def test_shard_rules_tiny():
    cfg = Dsv41Config.tiny()
    specs = tensor_specs(cfg)
    w = random_weights(cfg, 0)
    assert set(w) == set(specs)
    world = 2
    parts = [shard_tensor(cfg, "layers.2.attn.wq_b.weight", w["layers.2.attn.wq_b.weight"], r, world) for r in range(world)]
    assert torch.equal(torch.cat(parts, 0), w["layers.2.attn.wq_b.weight"])
    parts = [shard_tensor(cfg, "layers.2.attn.wo_b.weight", w["layers.2.attn.wo_b.weight"], r, world) for r in range(world)]
    assert torch.equal(torch.cat(parts, 1), w["layers.2.attn.wo_b.weight"])
    n = "layers.0.ffn.experts.1.w1.weight"
    parts = [shard_tensor(cfg, n, w[n], r, world) for r in range(world)]
    assert parts[0].shape[0] == padded_inter(cfg, world) == 64
    assert torch.equal(parts[0][:32], w[n][:32]) and torch.equal(parts[1][:32], w[n][32:]) and not parts[0][32:].any()
    assert shard_tensor(cfg, "layers.0.attn.wkv.weight", w["layers.0.attn.wkv.weight"], 1, world) is w["layers.0.attn.wkv.weight"]


def test_engram_layout_and_hash_state():
    cfg = Dsv41Config.tiny()
    lay = EngramLayout.from_config(cfg)
    fp = lay.flat_primes()
    assert fp.shape == (1, cfg.engram_hash_cols) and len(set(fp.flatten().tolist())) == fp.numel()
    assert (fp > cfg.engram_vocab_size - 1).all() and lay.table_rows == cfg.engram_num_embeddings
    ids = [5, 9, 200, 7, 7, 3]
    a = NgramHasher(cfg, lay)
    whole = a.extend(ids)
    b = NgramHasher(cfg, lay)
    parts = torch.cat([b.extend(ids[:2]), b.extend(ids[2:3]), b.extend(ids[3:])])
    assert torch.equal(whole, parts)                      # chunking does not change the hashes
    assert (whole >= 0).all() and (whole < lay.table_rows[0]).all()
    offs = lay.offsets()[0]
    col = 1
    assert ((whole[:, 0, col] >= offs[col]) & (whole[:, 0, col] < offs[col] + fp[0, col])).all()
    # a dead token blocks the look-back across it
    c = NgramHasher(cfg, lay)
    dead = c.extend(ids, [True, True, False, True, True, True])
    assert not torch.equal(dead[3], whole[3]) and torch.equal(dead[1], whole[1])


def test_candidate_blocks_pin_newest():
    score = torch.tensor([[0.1, 0.2, 5.0, 4.0, 0.0, 0.3, float("-inf"), float("-inf")]])
    keep = select_candidate_blocks(score, torch.tensor([6]), 2, 2)
    # best block is (5,4); the block of the newest visible position (index 5 -> block 2) is pinned
    assert keep[0].tolist() == [False, False, True, True, True, True, False, False]


def _model(seed=0, **over):
    cfg = Dsv41Config.tiny(**over)
    return cfg, Dsv41Reference(cfg, random_weights(cfg, seed))


def test_chunked_prefill_equals_token_by_token():
    cfg, m = _model()
    ids = torch.randint(0, cfg.vocab_size - 20, (23,), generator=torch.Generator().manual_seed(3)).tolist()
    st = m.new_seq()
    whole, mh = m.forward(st, ids)
    st2 = m.new_seq()
    parts, mhs = [], []
    for chunk in (ids[:5], ids[5:6], ids[6:17], ids[17:]):
        l, h = m.forward(st2, chunk)
        parts.append(l)
        mhs.append(h)
    assert torch.allclose(torch.cat(parts), whole, atol=2e-4, rtol=1e-4)
    assert torch.allclose(torch.cat(mhs), mh, atol=2e-4, rtol=1e-4)
    assert mh.shape == (23, cfg.dim * 2)
    for l in (1, 3):
        assert torch.allclose(st.comp_kv[l], st2.comp_kv[l], atol=1e-5)
    assert st.comp_kv[1].shape[0] == 23 // 2 and st.comp_kv[3].shape[0] == 23


def test_window_and_topk_limit_visibility():
    cfg, m = _model()
    seen = {}
    m.trace = lambda name, x: seen.__setitem__(name, x)
    st = m.new_seq()
    ids = list(range(30, 60))
    m.forward(st, ids)
    tk = seen["layers.5.topk"]
    assert tk.shape == (30, cfg.index_topk)
    last = tk[-1][tk[-1] >= 0]
    assert (last < 30).all() and last.numel() == cfg.index_topk and (last.diff() > 0).all()
    assert (seen["layers.1.topk"][0] == -1).all()      # position 0 of a ratio-2 layer sees no compressed row


def test_spec_generate_matches_greedy():
    cfg, m = _model(seed=2)
    prompt = [3, 17, 99, 250, 4, 8, 15, 16, 23]
    plain = m.generate(prompt, 10)
    spec, ks = m.spec_generate(prompt, 10)
    assert spec == plain
    assert all(1 <= k <= cfg.dspark_block_size + 1 for k in ks)


def test_checkpoint_roundtrip_is_exact(tmp_path):
    from ferrite_b200.models.dsv41_checkpoint import Dsv41CheckpointSource, save_checkpoint
    cfg = Dsv41Config.tiny()
    w = random_weights(cfg, 3)
    save_checkpoint(str(tmp_path), cfg, w, shards=3)
    src = Dsv41CheckpointSource(str(tmp_path), cfg)
    for name in ("layers.1.attn.wq_b.weight", "layers.0.ffn.experts.3.w2.weight", "layers.1.engram.embed.weight",
                 "layers.3.attn.compressor.wkv.weight", "layers.2.hc_attn_fn", "embed.weight", "mtp.1.markov_head.head.weight"):
        assert src.has(name) and torch.equal(src.get(name), w[name]), name
    assert not src.has("layers.0.attn.compressor.wkv.weight")


def test_cpp_golden_matches_python_statement():
    """The C++ golden ops of the DSV41 family against the PyTorch statements."""
    from ferrite_b200 import build
    build.build_runtime()
    from ferrite_b200 import _runtime as rt
    from ferrite_b200.models.dsv41_ref import sparse_attn_rows
    G = rt.golden if hasattr(rt, "golden") else rt
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 128, generator=g) * torch.logspace(-4, 2, 6).unsqueeze(1)
    assert torch.equal(torch.from_numpy(G.d4_e4m3_round(x.numpy())), Q.e4m3_round(x))
    assert torch.equal(torch.from_numpy(G.d4_e2m1_round(x.numpy())), Q.e2m1_decode(Q.e2m1_encode(x)))
    assert torch.equal(torch.from_numpy(G.d4_fp8_act_roundtrip(x.numpy(), 32)), Q.fp8_act_roundtrip(x, 32))
    assert torch.equal(torch.from_numpy(G.d4_fp4_act_roundtrip(x.numpy(), 32, False)), Q.fp4_act_roundtrip(x, 32))
    assert torch.equal(torch.from_numpy(G.d4_fp4_act_roundtrip(x.numpy(), 16, True)), Q.fp4_act_roundtrip(x, 16, "e4m3"))
    q, kv, sink = torch.randn(4, 64, generator=g), torch.randn(9, 64, generator=g), torch.randn(4, generator=g)
    got = torch.from_numpy(G.d4_sparse_attn_sink(q.numpy(), kv.numpy(), sink.numpy(), 0.125))
    assert torch.allclose(got, sparse_attn_rows(q, kv, sink, 0.125), atol=1e-5)
    assert not torch.from_numpy(G.d4_sparse_attn_sink(q.numpy(), kv[:0].numpy(), sink.numpy(), 0.125)).any()
    cfg, m = _model()
    xin = torch.randn(5, cfg.dim, generator=g)
    wts, idx = m.route(xin, "layers.0.ffn.", 2, None)
    logits = xin @ m.w["layers.0.ffn.gate.weight"].t()
    w2, i2 = G.d4_route(logits.numpy(), m.w["layers.0.ffn.gate.bias"].numpy(), 2, cfg.route_scale)
    assert torch.equal(torch.from_numpy(i2), idx) and torch.allclose(torch.from_numpy(w2), wts, atol=1e-5)
    score = torch.tensor([0.1, 0.2, 5.0, 4.0, 0.0, 0.3, -1e30, -1e30])
    keep = torch.from_numpy(G.d4_candidate_blocks(score.numpy(), 6, 2, 2)).bool()
    assert keep.tolist() == select_candidate_blocks(score.masked_fill(torch.arange(8) >= 6, float("-inf")).unsqueeze(0),
                                                    torch.tensor([6]), 2, 2)[0].tolist()


def test_synthetic_source_shapes_and_determinism():
    from ferrite_b200.models.dsv41_synth import SyntheticDsv41Source
    cfg = Dsv41Config.tiny()
    a, b = SyntheticDsv41Source(cfg, "cpu", seed=1), SyntheticDsv41Source(cfg, "cpu", seed=1)
    specs = tensor_specs(cfg)
    for name in ("embed.weight", "layers.1.attn.wq_b.weight", "layers.3.attn.compressor.norm.weight", "mtp.0.main_proj.weight"):
        assert a.has(name) and tuple(a.get(name).shape) == specs[name].shape and torch.equal(a.get(name), b.get(name))
    assert not a.has("layers.0.ffn.experts.0.w1.weight")
    w13, s13, w2, s2 = a.expert_pack("layers.0.ffn.", 8, 64, 0, 1, "cpu")
    assert w13.shape == (8, 2, 64, cfg.dim // 2) and s13.shape == (8, 2, 64, cfg.dim // 32)
    assert w2.shape == (8, cfg.dim, 32) and s2.shape == (8, cfg.dim, 2) and w13.dtype == torch.uint8
