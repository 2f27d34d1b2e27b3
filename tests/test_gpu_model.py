"""GPU: the device engine against the fp32 reference engine run on the device-equivalent
weights -- per-sublayer residual parity, then token identity for chunked prefill, graph
replay and MTP speculative decoding (the reference's T5 tier and its "spec output equals
greedy output" invariant)."""
import pytest
import torch

from ferrite_b200.config import EngineConfig, GlmConfig
from ferrite_b200.models.glm_ref import GlmReference
from ferrite_b200.models.glm_weights import quantize_like_device, random_weights

pytestmark = pytest.mark.gpu


def _prompt(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _engine(cfg, w, mtp_n=3, graphs=True, prefill_rows=16, max_ctx=512):
    from ferrite_b200.engine.glm_engine import GlmEngine
    from ferrite_b200.models.glm import DictSource
    ecfg = EngineConfig(max_ctx=max_ctx, mtp_n=mtp_n, use_graphs=graphs, kv_dtype="f32")
    return GlmEngine(cfg, ecfg, DictSource(w, "cuda"), prefill_rows=prefill_rows)


@pytest.mark.parametrize("name", ["tiny", "golden4"])
def test_sublayer_parity(name):
    cfg = getattr(GlmConfig, name)()
    w = random_weights(cfg, 0, std=0.05)
    wq = quantize_like_device(cfg, w)
    ref = GlmReference(cfg, wq)
    ref.trace = []
    p = _prompt(cfg, 13)
    st = ref.new_seq()
    logits_ref, hf_ref = ref.forward(st, p)
    eng = _engine(cfg, w, mtp_n=1)
    got = []
    eng.model.debug_hook = lambda i, site, ws, n: got.append((i, site, ws["R"][:n].clone(), ws["y"][:n].clone()))
    m = eng.model
    m.reset_slot(0)
    eng.prefill_ids[:13].copy_(torch.tensor(p, dtype=torch.int32))
    m.main_forward(eng._rows(13), eng.prefill_ids, judges=eng.judges)
    torch.cuda.synchronize()
    report = []
    for (i, site, Rr, yr), (_, _, Rd, yd) in zip(ref.trace, got):
        ey = (yd.cpu() - yr).abs().max().item() / (yr.abs().max().item() + 1e-9)
        eR = (Rd.cpu() - Rr).abs().max().item() / (Rr.abs().max().item() + 1e-9)
        report.append(f"L{i}.{site}: y rel {ey:.2e} R rel {eR:.2e}")
    bad = [r for r in report if float(r.split("y rel ")[1].split()[0]) > 2e-3 or float(r.split("R rel ")[1]) > 2e-3]
    assert not bad, "\n".join(report)
    lg = m.ws["logits"][:13].cpu()
    rel = (lg - logits_ref).abs().max().item() / logits_ref.abs().max().item()
    assert rel < 2e-3, f"logits rel err {rel:.2e}\n" + "\n".join(report)
    assert m.main_len[0].item() == 13


@pytest.mark.parametrize("name,graphs", [("tiny", False), ("tiny", True), ("golden4", True)])
def test_greedy_tokens_match_reference(name, graphs):
    cfg = getattr(GlmConfig, name)()
    w = random_weights(cfg, 0, std=0.05)
    ref = GlmReference(cfg, quantize_like_device(cfg, w))
    p = _prompt(cfg, 37)
    want, _ = ref.generate(p, 14, chunk=16)
    eng = _engine(cfg, w, mtp_n=1, graphs=graphs)
    got, _ = eng.generate(p, 14, mtp=False)
    assert got == want


@pytest.mark.parametrize("name", ["tiny", "golden4"])
def test_mtp_equals_greedy_on_device(name):
    cfg = getattr(GlmConfig, name)()
    w = random_weights(cfg, 0, std=0.05)
    p = _prompt(cfg, 29)
    plain, _ = _engine(cfg, w, mtp_n=1).generate(p, 16, mtp=False)
    eng = _engine(cfg, w, mtp_n=3)
    spec, acc = eng.generate(p, 16, mtp=True)
    assert spec == plain, (spec, plain, acc)
    assert all(1 <= k <= 3 for k in acc)
    assert eng.launches_mtp > 0


def test_mtp_accepts_when_draft_is_right():
    """A model whose MTP layer is wired to reproduce the main model's next token would accept
    everything; with random weights we instead check the bookkeeping by forcing repetition: a
    zero-weight model emits token 0 forever, so every draft is accepted (k == 3)."""
    cfg = GlmConfig.tiny()
    w = {k: torch.zeros_like(v) if v.dim() > 1 else v for k, v in random_weights(cfg, 0).items()}
    eng = _engine(cfg, w, mtp_n=3)
    out, acc = eng.generate([5, 6, 7, 8], 12, mtp=True)
    assert out == [0] * 12
    assert acc and all(k == 3 for k in acc), acc


def test_batched_engine_speculative_steps_match_greedy():
    """Batched MTP: every live sequence is one group of the draft / verify / accept step; the tokens are the greedy
    engine's whatever the drafts were, across bucket changes, chunked prefill and prefix-cache restores."""
    from ferrite_b200.engine.gpu_engine import GpuEngine
    from ferrite_b200.models.glm import DictSource
    from ferrite_b200.serve.engine import RequestSpec
    cfg = GlmConfig.tiny()
    w = random_weights(cfg, 0, std=0.05)
    prompts = [_prompt(cfg, n, seed=10 + n) for n in (37, 5, 64, 18, 50, 2)] + [[7]]
    single = _engine(cfg, w, mtp_n=1)
    want = [single.generate(p if len(p) > 1 else p * 2, 11, mtp=False)[0] for p in prompts]
    ecfg = EngineConfig(max_ctx=512, mtp_n=3, kv_dtype="f32")
    eng = GpuEngine(cfg, ecfg, DictSource(w, "cuda"), max_rows=4, prefill_rows=16, prefill_budget=48)
    got = eng.run_all([RequestSpec(p, 11) for p in prompts])
    for (rid, toks), w_ in zip(sorted(got.items()), want):
        assert toks == w_, (rid, toks, w_)
    ticks = eng.stats()["engine"]["ticks"]
    again = eng.run_all([RequestSpec(prompts[2], 11), RequestSpec(prompts[0], 11)])
    (r2, t2), (r0, t0) = sorted(again.items())
    assert t2 == want[2] and t0 == want[0]
    assert eng.usage[r2].cached_tokens == 48 and eng.usage[r0].cached_tokens == 32
    assert ticks > 0 and eng.launches > 0


def test_batched_engine_matches_single_sequence_engine():
    """Continuous batching with chunked prefill, bucket graphs and the radix prefix cache gives
    every request the tokens the single-sequence engine gives it."""
    from ferrite_b200.engine.gpu_engine import GpuEngine
    from ferrite_b200.models.glm import DictSource
    from ferrite_b200.serve.engine import RequestSpec
    cfg = GlmConfig.tiny()
    w = random_weights(cfg, 0, std=0.05)
    prompts = [_prompt(cfg, n, seed=10 + n) for n in (37, 5, 64, 18, 50)]
    single = _engine(cfg, w, mtp_n=1)
    want = [single.generate(p, 9, mtp=False)[0] for p in prompts]
    ecfg = EngineConfig(max_ctx=512, mtp_n=1, kv_dtype="f32")
    eng = GpuEngine(cfg, ecfg, DictSource(w, "cuda"), max_rows=4, prefill_rows=16, prefill_budget=48)
    got = eng.run_all([RequestSpec(p, 9) for p in prompts])
    for (rid, toks), w_ in zip(sorted(got.items()), want):
        assert toks == w_, (rid, toks, w_)
    assert eng.stats()["radix"]["tree_blocks"] > 0 and eng.launches > 0
    # the same prompt again: served from the prefix cache (state restored from a snapshot)
    again = eng.run_all([RequestSpec(prompts[2], 9), RequestSpec(prompts[0], 9)])
    (r2, t2), (r0, t0) = sorted(again.items())
    assert t2 == want[2] and t0 == want[0]
    assert eng.usage[r2].cached_tokens == 48 and eng.usage[r0].cached_tokens == 32
    assert eng.stats()["radix"]["hits"] == 2
