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
            err = (a - b).abs().max().item()
            if err > 5e-2 * max(1.0, b.abs().max().item()):   # one flipped e4m3 rounding is 6 % of an element
                report.append(f"{name}: max err {err:.3e} (ref max {b.abs().max().item():.3e})")
    got = torch.cat(outs)
    err = (got - want).abs().max().item()
    assert not report and err < 5e-2 * max(1.0, want.abs().max().item()), (report[:12], err)
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.9
