"""Batched output throughput of the continuous-batching engine (GLM-5.3-Flash, greedy, no MTP).

    python bench_batched.py --seqs 16 --prompt-len 64 --new-tokens 160 --window 100

Submits `--seqs` requests, lets the planner admit and prefill them, and then times a window of
decode ticks in which all sequences are live: CUDA events around the ticks (each tick = one graph
replay of the bucket plus the 4-byte-per-row token read-back the serving loop does anyway).
Reports whole-engine output tokens per second, the counterpart of the reference's "batched output
tok/s, 16 sequences, no MTP" row (971-985 tok/s at TP=4 on B300, docs/agent/perf-roadmap.md:3-5).
One JSON line on stdout.  Weights are random-init, prompts synthetic.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=64)
    ap.add_argument("--new-tokens", type=int, default=160)
    ap.add_argument("--window", type=int, default=100, help="timed decode ticks")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--layers", type=int, default=0, help="0 = the full 45-layer model")
    ap.add_argument("--experts-resident", type=int, default=0)
    ap.add_argument("--mtp", type=int, default=1, help="verify width of the batched speculative step (1 = greedy decode)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed ticks with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    args = ap.parse_args()

    from ferrite_b200.config import EngineConfig, GlmConfig
    from ferrite_b200.engine.gpu_engine import GpuEngine
    from ferrite_b200.models.glm import SyntheticSource
    from ferrite_b200.serve.engine import RequestSpec

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    allreduce = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from ferrite_b200.parallel.collective import make_allreduce
        allreduce = make_allreduce(dev, rank, world, max_elems=64 * 4096, kind="p2p")
    cfg = GlmConfig.production() if not args.layers else GlmConfig.scaled(args.layers)
    resident = args.experts_resident or (128 if world == 1 else cfg.n_routed_experts)
    ecfg = EngineConfig(tp=world, max_ctx=args.prompt_len + args.new_tokens + 64, mtp_n=args.mtp,
                        experts_resident=None if resident >= cfg.n_routed_experts else resident)
    t0 = time.time()
    eng = GpuEngine(cfg, ecfg, SyntheticSource(cfg, dev, seed=0), rank, world, dev, allreduce, max_rows=args.seqs,
                    prefill_rows=64)
    load_s = time.time() - t0
    g = torch.Generator().manual_seed(0)
    specs = [RequestSpec(torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist(), args.new_tokens, ())
             for _ in range(args.seqs)]
    for s in specs:
        eng.submit(s)
    produced = 0
    ticks = 0
    # admission + prefill + graph capture + warm-up ticks
    while True:
        evs = eng.tick()
        ticks += 1
        decoding = sum(1 for _, ev in evs if ev.kind == "tokens")
        if decoding == args.seqs:      # every sequence produced a token this tick: all are in the decode phase
            args.warmup -= 1
            if args.warmup <= 0:
                break
        assert ticks < 10000 and not eng.idle(), "the sequences finished before the timed window began"
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.profiler_range:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(args.window):
        for _, ev in eng.tick():
            if ev.kind == "tokens":
                produced += len(ev.ids)
    e1.record()
    torch.cuda.synchronize()
    if args.profiler_range:
        torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({
            "metric": "batched_output_tok_s", "value": round(produced / ms * 1e3, 2), "unit": "tok/s", "n_gpus": world,
            "ms_per_tick": round(ms / args.window, 4), "ticks": args.window, "tokens": produced, "impl": "ours",
            "dtype": "bf16", "data": "synthetic",
            "config": {"model": cfg.name, "sequences": args.seqs, "prompt_len": args.prompt_len,
                       "parallelism": f"tp{world}", "experts_resident_per_layer": resident,
                       "mtp": "off" if args.mtp <= 1 else f"batched, draft {args.mtp - 1} / verify {args.mtp}",
                       "accept_tokens_per_seq_step": round(produced / max(1, args.window * args.seqs), 3),
                       "kernel_launches_per_tick": eng.launches, "load_s": round(load_s, 1)},
            "vs_reference_published": round(produced / ms * 1e3 / 971.0, 3)}))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
