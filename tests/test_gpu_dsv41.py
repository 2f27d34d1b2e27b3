"""GPU: DSV41 kernels and the device forward against the fp32 golden model (tiny config)."""
import pytest
import torch

from ferrite_b200.models.dsv41_config import Dsv41Config
from ferrite_b200.models.dsv41_ref import Dsv41Reference
from ferrite_b200.models.dsv41_weights import random_weights
from ferrite_b200.ops import quant as Q

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from ferrite_b200 import _lib
    return _lib.lib()


def test_quant_rows_matches_codec(K):
    x = torch.randn(5, 256, generator=torch.Generator().manual_seed(0)) * torch.logspace(-3, 2, 5).unsqueeze(1)
    xd = x.cuda()
    out = torch.zeros_like(xd)
    K.call("fb_d4_quant_rows", xd, 256, out, 256, 5, 256, None, 0, 0, 0)
    assert torch.equal(out.cpu(), Q.fp8_act_roundtrip(x, 32))


def test_topk_sorted_ties_and_mask(K):
    from ferrite_b200.models.dsv41_ref import topk_stable
    n, ld, k = 3, 3000, 64
    g = torch.Generator().manual_seed(1)
    score = torch.randn(n, ld, generator=g)
    score[0, 100:400] = 0.5          # a long run of ties straddling the cut
    score[1, ::3] = float("-inf")
    meta = torch.zeros(n, 8, dtype=torch.int32)
    pos = [2999, 1500, 40]           # clen = pos + 1 (ratio 1)
    meta[:, 1] = torch.tensor(pos)
    mask = (torch.rand(n, ld, generator=g) > 0.3).to(torch.uint8)
    out = torch.zeros(n, k, dtype=torch.int32, device="cuda")
    for use_mask in (False, True):
        K.call("fb_d4_topk_sorted", score.cuda(), ld, mask.cuda() if use_mask else None, ld, meta.cuda(), 1, 1, k, out, k, n)
        for r in range(n):
            clen = pos[r] + 1
            s = score[r, :clen].clone()
            if use_mask:
                s[mask[r, :clen] == 0] = float("-inf")
            want = topk_stable(s.unsqueeze(0), min(k, clen))[0].sort().values.tolist()
            want += [-1] * (k - len(want))
            assert out[r].cpu().tolist() == want, (use_mask, r)


def _pair(seed=0, **over):
    cfg = Dsv41Config.tiny(**over)
    w = random_weights(cfg, seed)
    return cfg, w, Dsv41Reference(cfg, w)


def test_device_forward_matches_golden():
    from ferrite_b200.models.dsv41 import DictWeights, Dsv41DeviceModel
    cfg, w, ref = _pair()
    dev = Dsv41DeviceModel(cfg, DictWeights(w), max_rows=8, max_ctx=128)
    ids = torch.randint(0, cfg.vocab_size - 20, (29,), generator=torch.Generator().manual_seed(3)).tolist()
    gold = {}
    ref.trace = lambda name, x: gold.setdefault(name, []).append(x.clone())
    st = ref.new_seq()
    chunks = [ids[:8], ids[8:13], ids[13:21], ids[21:22], ids[22:23], ids[23:29]]
    want = torch.cat([ref.forward(st, c)[0] for c in chunks])
    got_trace = {}
    dev.debug = lambda name, t: got_trace.setdefault(name, []).append(t.detach().float().cpu().clone())
    outs, mhs = [], []
    for c in chunks:
        rs = dev.make_rows([0], [len(c)])
        dev.forward(rs, torch.tensor(c, dtype=torch.int32, device="cuda"))
        outs.append(dev.ws["logits"][:len(c)].cpu().clone())
        mhs.append(dev.ws["mh"][:len(c)].cpu().clone())
    torch.cuda.synchronize()
    assert int(dev.tc_status[0]) == 0
    report = []
    for name in sorted(got_trace, key=lambda s: (int(s.split(".")[1]), s)):
        if name not in gold:
            continue
        a = torch.cat([t.reshape(t.shape[0], -1) for t in got_trace[name]])
        bs = [t.reshape(t.shape[0], -1).float() for t in gold[name]]
        if "topk" in name:   # the golden's list is as wide as the visible range; the device pads with -1
            bs = [torch.nn.functional.pad(t, (0, a.shape[1] - t.shape[1]), value=-1.0) for t in bs]
        b = torch.cat(bs)
        if a.shape != b.shape:
            report.append(f"{name}: shape {tuple(a.shape)} vs {tuple(b.shape)}")
            continue
        if "topk" in name or "route_idx" in name:
            bad = (a != b).any(-1).sum().item()
            if bad:
                report.append(f"{name}: {bad} rows differ")
        else:
            # one flipped e4m3 rounding moves an element by 6 %, and flips compound with depth: bound the
            # bulk of the elements tightly and the outliers loosely
            ref = max(1.0, b.abs().max().item())
            diff = (a - b).abs()
            if (diff > 3e-2 * ref).float().mean().item() > 0.01 or diff.max().item() > 0.25 * ref:
                report.append(f"{name}: max err {diff.max().item():.3e}, p99 {diff.flatten().quantile(0.99).item():.3e} "
                              f"(ref max {b.abs().max().item():.3e})")
    got = torch.cat(outs)
    err = (got - want).abs().max().item()
    assert not report and err < 0.15 * max(1.0, want.abs().max().item()), (report[:12], err)
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.9


def test_engine_plain_and_spec_generation():
    from ferrite_b200.engine.dsv41_engine import Dsv41Engine
    from ferrite_b200.models.dsv41 import DictWeights
    cfg, w, ref = _pair(seed=2)
    prompt = [3, 17, 99, 250, 4, 8, 15, 16, 23, 42, 77]
    n_new = 14
    want = ref.generate(prompt, n_new)
    outs = {}
    for graphs in (False, True):
        eng = Dsv41Engine(cfg, DictWeights(w), max_ctx=128, use_graphs=graphs)
        outs[("plain", graphs)] = eng.generate(prompt, n_new)
        eng2 = Dsv41Engine(cfg, DictWeights(w), max_ctx=128, use_graphs=graphs)
        outs[("spec", graphs)] = eng2.generate(prompt, n_new, spec=True)
        assert all(1 <= k <= cfg.dspark_block_size + 1 for k in eng2.accept_hist)
    torch.cuda.synchronize()
    same = sum(a == b for a, b in zip(want, outs[("plain", False)]))
    assert same >= n_new - 3, (want, outs)          # a flipped e4m3 rounding may move a late argmax
    assert outs[("plain", True)] == outs[("plain", False)], outs
    assert outs[("spec", False)] == outs[("plain", False)], outs
    assert outs[("spec", True)] == outs[("plain", False)], outs


def test_batched_engine_matches_single_sequence_engine():
    """Continuous batching (several sequences of different lengths, more requests than slots, prefill chunks between
    decode ticks, graph per bucket) emits for every request the tokens of the single-sequence engine."""
    from ferrite_b200.engine.dsv41_batch import Dsv41BatchEngine
    from ferrite_b200.engine.dsv41_engine import Dsv41Engine
    from ferrite_b200.models.dsv41 import DictWeights
    from ferrite_b200.serve.engine import RequestSpec
    cfg, w, _ = _pair(seed=2)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (11, 3, 27, 1, 19)]
    n_new = [9, 12, 6, 10, 8]
    single = Dsv41Engine(cfg, DictWeights(w), max_ctx=128)
    want = [single.generate(p, k) for p, k in zip(prompts, n_new)]
    for graphs in (False, True):
        eng = Dsv41BatchEngine(cfg, DictWeights(w), max_ctx=128, max_seqs=3, prefill_rows=8, prefill_budget=12,
                               use_graphs=graphs)
        got = eng.run_all([RequestSpec(p, k) for p, k in zip(prompts, n_new)])
        assert eng.idle() and sorted(eng.free) == [0, 1, 2]
        for rid, (p, k) in enumerate(zip(prompts, n_new), start=1):
            assert got[rid] == want[rid - 1], (graphs, rid, got[rid], want[rid - 1])
            assert eng.usage[rid].prompt_tokens == len(p) and eng.usage[rid].completion_tokens == k
    # more than 8 decode rows, with the sublayers closed by the fused GEMV + fold kernel in two 8-row windows
    from ferrite_b200.utils.switches import Switches, set_switches
    try:
        set_switches(Switches(d4_fused_rows=16))
        many = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (4, 9, 2, 6, 12, 3, 7, 5, 10, 8, 1)]
        want_many = [single.generate(p, 6) for p in many]
        eng = Dsv41BatchEngine(cfg, DictWeights(w), max_ctx=128, max_seqs=11, prefill_rows=16, prefill_budget=200)
        assert eng.model.fused_rows == 16
        got = eng.run_all([RequestSpec(p, 6) for p in many])
        assert max(rows for rows in eng.graphs) == 11                # one tick decoded all eleven sequences
        for rid, wnt in enumerate(want_many, start=1):
            assert got[rid] == wnt, (rid, got[rid], wnt)
    finally:
        set_switches(None)
    # a stop id ends a sequence without emitting it; a cancelled request frees its slot
    eng = Dsv41BatchEngine(cfg, DictWeights(w), max_ctx=128, max_seqs=2, prefill_rows=8)
    stop_at = want[0][4]
    cut = want[0].index(stop_at)
    a = eng.submit(RequestSpec(prompts[0], 9, stop_ids=(stop_at,)))
    b = eng.submit(RequestSpec(prompts[2], 50))
    toks = {a: [], b: []}
    for t in range(200):
        if t == 3:
            eng.cancel(b)
        for rid, ev in eng.tick():
            if ev.kind == "tokens":
                toks[rid] += ev.ids
        if eng.idle():
            break
    assert toks[a] == want[0][:cut] and eng.idle() and len(eng.free) == 2


def test_draft_block_matches_golden():
    from ferrite_b200.models.dsv41 import DictWeights, Dsv41DeviceModel
    cfg, w, ref = _pair(seed=4)
    prompt = [5, 9, 200, 7, 7, 3, 88, 140, 31]
    st = ref.new_seq()
    logits, mh = ref.forward(st, prompt)
    ref.dspark_seed(st, mh, 0)
    t0 = int(logits[-1].argmax())
    drafts, dl, conf = ref.dspark_draft(st, t0, len(prompt) - 1)
    dev = Dsv41DeviceModel(cfg, DictWeights(w), max_rows=8, max_ctx=128)
    for i in range(0, len(prompt), 8):
        c = prompt[i:i + 8]
        rs = dev.make_rows([0], [len(c)])
        dev.forward(rs, torch.tensor(c, dtype=torch.int32, device="cuda"))
        dev.dspark_seed(rs)
    B = cfg.dspark_block_size
    out = dev.dspark_draft(dev.make_rows([0], [B]), torch.tensor([t0], dtype=torch.int32, device="cuda"))
    got = dev.ws["logits"][:B].cpu()
    assert (got - dl).abs().max().item() < 5e-2 * max(1.0, dl.abs().max().item())
    assert out.tolist()[0] == t0 and sum(a == b for a, b in zip(out.tolist()[1:], drafts)) >= B - 1
    assert (dev.dspark_confidence().cpu() - conf).abs().max().item() < 5e-2 * max(1.0, conf.abs().max().item())


def test_step_engine_prefix_cache_resumes_exactly():
    from ferrite_b200.engine.dsv41_engine import Dsv41Engine, Dsv41StepEngine
    from ferrite_b200.models.dsv41 import DictWeights
    cfg, w, ref = _pair(seed=6)
    a = [3, 17, 99, 250, 4, 8, 15, 16, 23, 42, 77, 5, 6]
    b = a + [100, 101, 102, 7]
    for spec in (False, True):
        cold = Dsv41StepEngine(Dsv41Engine(cfg, DictWeights(w), max_ctx=128), spec=spec, cache_entries=0)
        first, cached = cold.start(b)
        want = [first]
        while len(want) < 10:
            want += cold.step()
        warm = Dsv41StepEngine(Dsv41Engine(cfg, DictWeights(w), max_ctx=128), spec=spec)
        f0, c0 = warm.start(a)
        assert c0 == 0
        for _ in range(3):
            warm.step()                      # decode past the prompt: the snapshot must not include this
        f1, c1 = warm.start(b)
        assert c1 == len(a) and warm.hits == 1
        got = [f1]
        while len(got) < 10:
            got += warm.step()
        assert got[:10] == want[:10], (spec, got, want)


def test_vision_tower_and_image_rows():
    from ferrite_b200.models.dsv41 import DictWeights, Dsv41DeviceModel
    from ferrite_b200.models.dsv41_vision import (IMAGE, VisionDevice, VisionReference, expand_image_tokens)
    cfg = Dsv41Config.tiny(vision=True)
    w = random_weights(cfg, 9)
    n_h, n_w = 5, 6
    patches = torch.randn(n_h * n_w, 3 * cfg.vision.patch_size ** 2, generator=torch.Generator().manual_seed(1))
    patches = patches.to(torch.bfloat16).float()
    vref = VisionReference(cfg, w)
    vdev = VisionDevice(cfg, DictWeights(w))
    want_vit = vref.vit(patches, n_h, n_w)
    got_vit = vdev.vit(patches, n_h, n_w).cpu()
    assert (got_vit - want_vit).abs().max().item() < 3e-2 * max(1.0, want_vit.abs().max().item())
    want = vref.encode_image(patches, n_h, n_w)
    got = vdev.encode_image(patches, n_h, n_w).cpu()
    torch.cuda.synchronize()
    assert int(vdev.status[0]) == 0 and got.shape == (9, cfg.dim)
    assert (got - want).abs().max().item() < 3e-2 * max(1.0, want.abs().max().item())
    # a prompt with one image: span rows take the tower's embeddings, no engram, image routing bias
    toks, types, spans = expand_image_tokens([5, 9, cfg.image_token_id, 7, 3], cfg.image_token_id, [(n_h, n_w)],
                                              cfg.vision.downsample_ratio)
    span = spans[0]
    assert len(toks) == 4 + len(span.types) and types.count(IMAGE) == 9 and span.start == 2
    emb_span = vref.span_embeddings(span, patches)
    mask = torch.tensor([t >= 0 for t in types])
    embeds = torch.zeros(len(toks), cfg.dim)
    embeds[mask] = emb_span
    ref = Dsv41Reference(cfg, w)
    st = ref.new_seq()
    want_logits, _ = ref.forward(st, toks, image_mask=mask, embeds=embeds)
    dev = Dsv41DeviceModel(cfg, DictWeights(w), max_rows=8, max_ctx=128)
    outs = []
    for i in range(0, len(toks), 8):
        c = toks[i:i + 8]
        rs = dev.make_rows([0], [len(c)])
        dev.forward(rs, torch.tensor(c, dtype=torch.int32, device="cuda"), image_embeds=embeds[i:i + 8],
                    is_image=mask[i:i + 8])
        outs.append(dev.ws["logits"][:len(c)].cpu().clone())
    got_logits = torch.cat(outs)
    diff = (got_logits - want_logits).abs()
    ref_max = max(1.0, want_logits.abs().max().item())
    assert (diff > 3e-2 * ref_max).float().mean().item() < 0.01 and diff.max().item() < 0.25 * ref_max


@pytest.mark.parametrize("n,topk,E,I,D", [(3, 2, 8, 192, 256), (1, 6, 16, 128, 512), (5, 3, 8, 320, 384)])
def test_fp4_expert_mma_kernels_match_simt(K, n, topk, E, I, D):
    """Tensor-core routed-expert kernels (quad-interleaved weights, f16 activations) against the SIMT kernels
    on the original byte layout; the repack is an involution up to its inverse flag."""
    from ferrite_b200.models.glm import Act
    import ctypes
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    w13 = torch.randint(0, 256, (E, 2, I, D // 2), dtype=torch.uint8, device=dev, generator=g)
    s13 = torch.randint(118, 124, (E, 2, I, D // 32), dtype=torch.uint8, device=dev, generator=g)
    w2 = torch.randint(0, 256, (E, D, I // 2), dtype=torch.uint8, device=dev, generator=g)
    s2 = torch.randint(118, 124, (E, D, I // 32), dtype=torch.uint8, device=dev, generator=g)
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:topk] for _ in range(n)]).to(torch.int32).contiguous()
    wts = torch.rand(n, topk, device=dev, generator=g)
    x = Act(dev, n, D)
    x.f.copy_(torch.randn(n, D, device=dev, generator=g))
    K.call("fb_d4_quant_rows", x.f, D, x.f, D, n, D, *x.sp(2))
    h_ref, h = torch.zeros(n * topk, I, device=dev), Act(dev, n * topk, I)
    y_ref, y = torch.zeros(n, D, device=dev), torch.full((n, D), 0.5, device=dev)
    K.call("fb_d4_expert_gate_up", x.f, D, idx, wts, w13, s13, h_ref, n, topk, I, D, 10.0)
    K.call("fb_d4_quant_rows", h_ref, I, h_ref, I, n * topk, I, None, 0, 0, 0)
    K.call("fb_d4_expert_down", h_ref, idx, w2, s2, y_ref, D, n, topk, I, D, 0)
    w13p, w2p = w13.clone(), w2.clone()
    for t in (w13p, w2p):
        K.call("fb_d4_fp4_repack", t, t.numel() // t.shape[-1], t.shape[-1], 0)
    f16 = lambda a: ctypes.c_void_p(a.s.data_ptr() + 4 * a.plane)
    K.call("fb_d4_expert_gate_up_mma", f16(x), D, idx, wts, w13p, s13, h.f, n, topk, I, D, 10.0)
    torch.cuda.synchronize()
    # compare before the re-quantisation (which can flip a rounding on a last-bit difference)
    h_raw = torch.zeros(n * topk, I, device=dev)
    K.call("fb_d4_expert_gate_up", x.f, D, idx, wts, w13, s13, h_raw, n, topk, I, D, 10.0)
    assert torch.allclose(h.f, h_raw, atol=1e-5 * max(1.0, h_raw.abs().max().item()), rtol=1e-4), (h.f - h_raw).abs().max().item()
    h.f.copy_(h_ref)   # identical quantised input for the down comparison
    K.call("fb_d4_quant_rows", h.f, I, h.f, I, n * topk, I, *h.sp(2))
    K.call("fb_d4_expert_down_mma", f16(h), idx, w2p, s2, y, D, n, topk, I, D, 0)
    torch.cuda.synchronize()
    assert torch.allclose(y, y_ref, atol=1e-5 * max(1.0, y_ref.abs().max().item()), rtol=1e-4), (y - y_ref).abs().max().item()
    K.call("fb_d4_expert_down_mma", f16(h), idx, w2p, s2, y, D, n, topk, I, D, 1)
    torch.cuda.synchronize()
    assert torch.allclose(y, 2 * y_ref, atol=2e-5 * max(1.0, y_ref.abs().max().item()), rtol=1e-4)
    # quantise-on-load form: f32 rows that are not round-tripped yet give the same sums
    y_q = torch.zeros(n, D, device=dev)
    K.call("fb_d4_expert_down_mma_f32", h_raw, idx, w2p, s2, y_q, D, n, topk, I, D, 0)
    torch.cuda.synchronize()
    assert torch.allclose(y_q, y_ref, atol=1e-5 * max(1.0, y_ref.abs().max().item()), rtol=1e-4), (y_q - y_ref).abs().max().item()
    for t, orig in ((w13p, w13), (w2p, w2)):
        K.call("fb_d4_fp4_repack", t, t.numel() // t.shape[-1], t.shape[-1], 1)
        assert torch.equal(t, orig)


@pytest.mark.parametrize("n,heads,pos,ktop", [(1, 8, 5000, 512), (3, 64, 70, 40), (2, 16, 300, 0)])
def test_sparse_attn_tensor_core_matches_simt(K, n, heads, pos, ktop):
    """Tensor-core sparse attention with sink (head_dim 512) against the SIMT kernel on the same ring / compressed rows."""
    dev = torch.device("cuda")
    hd, W, cap, ccap, rd = 512, 128, 136, 2048, 64
    g = torch.Generator(device=dev).manual_seed(9)
    ring = torch.randn(2, cap, hd, device=dev, generator=g).to(torch.bfloat16)
    comp = torch.randn(2, ccap, hd, device=dev, generator=g).to(torch.bfloat16)
    q = torch.randn(n, heads * hd, device=dev, generator=g)
    sink = torch.randn(heads, device=dev, generator=g)
    freqs = torch.rand(rd // 2, device=dev, generator=g)
    meta = torch.zeros(n, 8, dtype=torch.int32, device=dev)
    meta[:, 0] = 1                                     # slot
    meta[:, 1] = torch.arange(n, device=dev) + pos     # pos
    meta[:, 2] = pos                                   # ctx0
    idx = None
    if ktop:
        idx = torch.stack([torch.randperm(ccap, device=dev, generator=g)[:ktop].sort().values for _ in range(n)]).to(torch.int32)
        idx[:, -3:] = -1                                # unreachable entries are masked
        idx = idx.contiguous()
    ns = 16
    o_part, ml = torch.zeros(n * heads * ns * hd, device=dev), torch.zeros(n * heads * ns * 2, device=dev)
    want, got = torch.zeros(n, heads * hd, device=dev), torch.zeros(n, heads * hd, device=dev)
    K.call("fb_d4_sparse_attn", q, heads * hd, ring, cap, W, comp, ccap, idx, ktop, ktop, None, 0, sink, freqs, rd, meta, 0, 0,
           float(hd ** -0.5), heads, hd, want, heads * hd, n, ns, o_part, ml, None, 0, 0, 0, None)
    nsp = max(1, min(ns, (W + ktop + 63) // 64))
    K.call("fb_d4_sparse_attn_tc", q, heads * hd, ring, cap, W, comp, ccap, idx, ktop, ktop, sink, freqs, rd, meta, 0, 0,
           float(hd ** -0.5), heads, got, heads * hd, n, nsp, o_part, ml, None, 0, 0, 0)
    torch.cuda.synchronize()
    err = (got - want).abs().max().item()
    assert err < 2e-2 * max(1.0, want.abs().max().item()), (err, want.abs().max().item())
