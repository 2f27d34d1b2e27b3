"""Prefill / decode disaggregation: a layer-split (context-parallel) prefill group handing a long prompt off to a
tensor-parallel decode group on the other GPUs of the box.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_cp.py --prefill-ranks 4 --decode-ranks 4
  python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 bench_cp.py --prefill-ranks 4 --decode-ranks 0

The first P ranks are pipeline stages (each holds its layers with ALL their experts and runs no collective inside
prefill), the next D ranks a TP group that holds the model sharded.  The prompt streams through the stages in chunks
(NCCL p2p of the residual streams), every stage exports its layers' caches and recurrent states to the decode ranks
as soon as it is done, the last stage adds the first token and the draft inputs, and the decode group continues with
speculative steps.  Counterpart of the reference's ``PdafCluster`` (``crates/ferrite-exec/src/distributed.rs:85-257``)
and of its 65 536-token configuration.  Synthetic token ids, random-init weights of the production architecture.
Times are wall clock around device synchronisation, max over the ranks of a group.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--prefill-ranks", type=int, default=4)
    ap.add_argument("--decode-ranks", type=int, default=4)
    ap.add_argument("--prompt-tokens", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=1024, help="rows per pipeline chunk")
    ap.add_argument("--decode-steps", type=int, default=20)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers")
    ap.add_argument("--runs", type=int, default=3)
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist
    from ferrite_b200.config import EngineConfig, GlmConfig
    from ferrite_b200.models.glm import SyntheticSource
    from ferrite_b200.parallel.cp import CpStage, hand_off

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    P, D = args.prefill_ranks, args.decode_ranks
    assert P + D <= world and P >= 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    stage_ranks, decode_ranks = list(range(P)), list(range(P, P + D))
    dgroup = dist.new_group(decode_ranks) if D > 1 else None
    cfg = GlmConfig.production() if not args.layers else GlmConfig.scaled(args.layers)
    max_ctx = args.prompt_tokens + 256
    stage = eng = None
    t_load = time.time()
    if rank in stage_ranks:
        ecfg = EngineConfig(max_ctx=max_ctx, mtp_n=3)
        stage = CpStage(cfg, ecfg, SyntheticSource(cfg, dev, seed=0, exact_shards=True), rank, P, stage_ranks, dev,
                        prefill_rows=args.chunk)
    elif rank in decode_ranks:
        from ferrite_b200.engine.glm_engine import GlmEngine
        from ferrite_b200.parallel.collective import make_allreduce
        d = decode_ranks.index(rank)
        ar = make_allreduce(dev, d, D, max_elems=64 * cfg.hidden_size, kind="p2p", group=dgroup) if D > 1 else None
        ecfg = EngineConfig(tp=D, max_ctx=max_ctx, mtp_n=3)
        eng = GlmEngine(cfg, ecfg, SyntheticSource(cfg, dev, seed=0, exact_shards=True), d, D, dev, ar, prefill_rows=64)
    t_load = time.time() - t_load
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt_tokens,), generator=g).tolist()

    def sync_max(x: float) -> float:
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ttft, hand, stage_done = [], [], []
    first = torch.zeros(1, dtype=torch.int64, device=dev)
    for _ in range(args.runs):
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        t_stage = t_first = 0.0
        if stage is not None:
            tok = stage.prefill(prompt)               # returns after a device synchronise
            t_stage = time.perf_counter() - t0
            if tok is not None:
                first[0] = tok
                t_first = t_stage
        if D:
            hand_off(stage, eng, len(prompt), stage_ranks, decode_ranks, cfg, rank, mode="tp")
        t_hand = time.perf_counter() - t0
        ttft.append(sync_max(t_first))
        hand.append(sync_max(t_hand))
        stage_done.append(sync_max(t_stage if rank == 0 else 0.0))
    dist.broadcast(first, stage_ranks[-1])
    ms_step, toks = 0.0, []
    if eng is not None:
        eng.build_graphs(True)
        for _ in range(3):
            toks += eng.spec_step()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(args.decode_steps):
            toks += eng.spec_step()
        torch.cuda.synchronize()
        ms_step = (time.perf_counter() - t1) * 1e3 / args.decode_steps
    ms_step = sync_max(ms_step)
    if rank == 0:
        ttft_s, hand_s = sorted(ttft)[len(ttft) // 2], sorted(hand)[len(hand) // 2]
        s0 = sorted(stage_done)[len(stage_done) // 2]
        print(json.dumps({
            "metric": "cp_prefill_ttft_s", "value": round(ttft_s, 4), "unit": "s", "higher_is_better": False,
            "n_gpus": P + D, "prompt_tokens": args.prompt_tokens, "prefill_tok_s": round(args.prompt_tokens / ttft_s, 1),
            "first_stage_done_s": round(s0, 4),
            "handoff_complete_s": round(hand_s, 4) if D else None,
            "handoff_after_first_token_s": round(hand_s - ttft_s, 4) if D else None,
            "decode_ms_per_step": round(ms_step, 3) if D else None,
            "config": {"model": cfg.name, "layers": cfg.num_layers, "prefill_group": f"cp{P} (layer split)",
                       "decode_group": f"tp{D}" if D else "none", "chunk_rows": args.chunk, "runs": args.runs,
                       "weights": "random-init", "data": "synthetic", "load_s": round(t_load, 1),
                       "note": "the first stage finishes, and starts exporting, first_stage_done_s after the start; "
                               "exports of stages 0..P-2 overlap the later stages' prefill"}}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
