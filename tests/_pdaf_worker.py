"""Worker run under torch.distributed.run by test_gpu_multi.py: PDAF hand-off of a prefilled
sequence from rank 0 (prefill) to rank 1 (decode) over NCCL p2p."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrite_b200.config import EngineConfig, GlmConfig  # noqa: E402
from ferrite_b200.engine.glm_engine import GlmEngine  # noqa: E402
from ferrite_b200.models.glm import DictSource  # noqa: E402
from ferrite_b200.models.glm_weights import random_weights  # noqa: E402
from ferrite_b200.parallel.pdaf import recv_sequence, send_sequence  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = GlmConfig.golden4()
    w = random_weights(cfg, 0, std=0.05)
    prompt = torch.randint(0, cfg.vocab_size, (45,), generator=torch.Generator().manual_seed(5)).tolist()
    for mtp_n in (1, 3):
        ecfg = EngineConfig(max_ctx=256, mtp_n=mtp_n, kv_dtype="f32")
        eng = GlmEngine(cfg, ecfg, DictSource(w, dev), device=dev, prefill_rows=16)
        if rank == 0:
            first = eng.prefill(prompt)
            plan = send_sequence(eng, dst=1)
            assert plan.n_pages == (45 + cfg.dsa.page_size - 1) // cfg.dsa.page_size
            dist.send(torch.tensor([first], device=dev), 1)
        elif rank == 1:
            recv_sequence(eng, src=0)
            t = torch.zeros(1, dtype=torch.int64, device=dev)
            dist.recv(t, 0)
            out = [int(t.item())]
            eng.build_graphs(mtp_n > 1)
            while len(out) < 14:
                out += eng.spec_step() if mtp_n > 1 else [eng.step_plain()]
            local_eng = GlmEngine(cfg, ecfg, DictSource(w, dev), device=dev, prefill_rows=16)
            want, _ = local_eng.generate(prompt, 14)
            assert out[:14] == want, (mtp_n, out, want)
            print(f"pdaf mtp_n={mtp_n}: decode rank continued {out[:14]}")
        dist.barrier()
    # DCP decode group of two: rank 0 prefills, hands rank 1 its share (latent pages p % 2 == 1, the whole
    # indexer caches, the recurrent state), poisons the latent pages it does not own, and both ranks decode
    # with the cross-rank LSE merge inside the attention epilogue.
    from ferrite_b200.parallel.symm import DcpAttentionMerge
    ds = cfg.dsa
    for mtp_n in (1, 3):
        ecfg = EngineConfig(max_ctx=256, mtp_n=mtp_n, kv_dtype="f32")
        eng = GlmEngine(cfg, ecfg, DictSource(w, dev), device=dev, prefill_rows=16)
        m = eng.model
        merge = DcpAttentionMerge(dev, rank, world, max_rows=16, heads=m.h_dsa, latent_dim=ds.kv_lora_rank)
        first = torch.zeros(1, dtype=torch.int64, device=dev)
        if rank == 0:
            first[0] = eng.prefill(prompt)
            send_sequence(eng, dst=1, n_dcp=2, d=1)
            n_pages = (eng.n_ctx + ds.page_size - 1) // ds.page_size
            m.lat_cache[:, [p for p in range(n_pages) if p % 2 == 1]] = float("nan")
        else:
            recv_sequence(eng, src=0, n_dcp=2, d=1)
        dist.broadcast(first, 0)
        m.dcp = (rank, 2, merge)
        out = [int(first.item())]
        eng.build_graphs(mtp_n > 1)
        while len(out) < 14:
            out += eng.spec_step() if mtp_n > 1 else [eng.step_plain()]
        merge.check()
        local_eng = GlmEngine(cfg, ecfg, DictSource(w, dev), device=dev, prefill_rows=16)
        want, _ = local_eng.generate(prompt, 14)
        same = sum(a == b for a, b in zip(out[:14], want))
        assert same >= 13, (mtp_n, rank, out, want)   # the merge sums partials in another order than one rank does
        t = torch.tensor(out[:14], device=dev)
        t0 = t.clone()
        dist.broadcast(t0, 0)
        assert torch.equal(t, t0), "DCP ranks emitted different tokens"
        if rank == 0:
            print(f"dcp2 mtp_n={mtp_n}: {out[:14]} ({same}/14 equal to one rank)")
        dist.barrier()
        merge.close()
    dist.destroy_process_group()
    if rank == 1:
        print("PDAF_WORKER_OK")


if __name__ == "__main__":
    main()
