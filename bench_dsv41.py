"""DSV41 decode step time at production dimensions on a LAYER-REDUCED model (the full 40-layer model is
475 GiB and needs TP >= 4):

    python bench_dsv41.py --layers 4 --steps 50

Builds `--layers` backbone layers with the production widths (dim 5120, 64 heads x 512, 384 fp4 experts,
window 128, compressed KV + indexer; one layer of every attention flavour), random weights generated on
the device, prefills a short prompt and times graph-replayed decode steps with CUDA events.  The JSON
line gives ms per step, ms per layer and the 40-layer extrapolation, which is an ESTIMATE (labelled as
such), not a measurement of the full model.  Reference number for orientation: 6.15 ms/step at TP=8
on B300 (docs/agent/unified-engine-battle-plan.md:4).

    python bench_dsv41.py --layers 0 --emulate-tp 8 --steps 50

`--emulate-tp R` builds RANK 0's shard of an R-way tensor-parallel model on ONE GPU (its 1/R of the heads,
output groups, expert intermediate columns and vocabulary): at R = 8 the full-depth 40-layer shard is
~45 GB and fits, so `--layers 0` times the whole production model's per-rank kernel chain.  The collectives
run as one-rank instances of the same kernels (pushes and flags go to this GPU, nothing crosses NVLink), so
the number is the per-rank COMPUTE time of a TP=R step; the cross-GPU wait of the ~80 fused collectives
(7-8 us each on two GPUs) comes on top.  The engram tables (197 G parameters) are left out: the synthetic
source cannot build them.  The metric name says `emulated`.
"""
from __future__ import annotations

import argparse
import json
import time
import os
from dataclasses import replace

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--prompt-len", type=int, default=300)
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--max-rows", type=int, default=64,
                    help="rows per prefill chunk (>= 16: routed experts run as block-scaled tcgen05 grouped GEMMs)")
    ap.add_argument("--kernel-times", default=None, metavar="FILE",
                    help="after the timed loop: 5 more steps under torch.profiler on rank 0 (every rank steps), per-kernel "
                         "device times of one step written to FILE")
    ap.add_argument("--engram", action="store_true",
                    help="with --layers 0: keep the two engram layers and their hash tables (197 G e4m3 parameters, "
                         "row-sharded: 49 GB per rank at TP=4)")
    ap.add_argument("--seqs", type=int, default=1, help="N > 1: N sequences through the continuous-batching engine")
    ap.add_argument("--spec", action="store_true", help="DSpark draft/verify steps instead of plain decode")
    ap.add_argument("--pdl", action="store_true", help="launch with programmatic dependent launch")
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="build rank 0's shard of a TP=R model on one GPU with one-rank collectives (--layers 0: all 40 layers)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed steps with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    args = ap.parse_args()
    from ferrite_b200.engine.dsv41_engine import Dsv41Engine
    from ferrite_b200.models.dsv41_config import Dsv41Config
    from ferrite_b200.models.dsv41_synth import SyntheticDsv41Source

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
        allreduce = make_allreduce(dev, rank, world, max_elems=64 * 8192, kind="p2p")
    if args.pdl:
        from ferrite_b200 import _lib
        _lib.lib().lib.fb_set_pdl(1)
    model_rank, model_world = rank, world
    if args.emulate_tp > 1:
        assert world == 1, "--emulate-tp runs as one process"
        import torch.distributed as dist
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29571", rank=0, world_size=1, device_id=dev)
        from ferrite_b200.parallel.collective import make_allreduce
        allreduce = make_allreduce(dev, 0, 1, max_elems=64 * 8192, kind="p2p")   # one-rank instances of the collectives
        model_rank, model_world = 0, args.emulate_tp
    L = args.layers
    n_mtp = 3 if args.spec else 0
    if L == 0:
        base = Dsv41Config()
        L = base.n_layers
        cfg = replace(base, n_mtp_layers=n_mtp, compress_ratios=tuple(base.compress_ratios[:L]) + (0,) * n_mtp,
                      engram_layer_ids=base.engram_layer_ids if args.engram else (),
                      engram_num_embeddings=base.engram_num_embeddings if args.engram else (),
                      dspark_target_layer_ids=base.dspark_target_layer_ids if args.spec else (),
                      dspark_block_size=base.dspark_block_size if args.spec else 0,
                      n_routed_experts=args.experts).validate()
    else:
        assert L >= 4
        # one window-only layer, a ratio-2 source, a ratio-1 source (candidate source), an inheriting ratio-1 layer
        ratios = [0, 2, 1] + [1] * (L - 3)
        cfg = replace(Dsv41Config(), n_layers=L, n_mtp_layers=n_mtp, compress_ratios=tuple(ratios + [0] * n_mtp),
                      kv_source_layers=(1, 2), index_source_layers=(1, 2) + ((L - 1,) if L > 4 else ()),
                      candidate_source_layer=2, engram_layer_ids=(), engram_num_embeddings=(),
                      dspark_target_layer_ids=tuple(range(max(0, L - 3), L)) if args.spec else (),
                      dspark_block_size=5 if args.spec else 0, n_routed_experts=args.experts).validate()
    if args.seqs > 1:
        return bench_batched(args, cfg, dev, model_rank, model_world, rank, world, allreduce, L)
    eng = Dsv41Engine(cfg, SyntheticDsv41Source(cfg, dev), model_rank, model_world, dev, allreduce,
                      max_ctx=args.prompt_len + 1024, max_rows=args.max_rows)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist()
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    eng.prefill(prompt)
    p1.record()
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)   # chunked prefill of the prompt (eager launches, --max-rows rows per chunk)
    step = (lambda: eng.spec_step()) if args.spec else (lambda: eng.step_plain())
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    toks = 0
    if args.profiler_range:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(args.steps):
        r = step()
        toks += len(r) if isinstance(r, list) else 1
    e1.record()
    torch.cuda.synchronize()
    if args.profiler_range:
        torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    if args.kernel_times:
        kernel_times(args.kernel_times, step, rank, world, "decode steps")
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        full = L == Dsv41Config().n_layers
        name = "dsv41_decode_ms_per_step" + ("" if full else "_layer_reduced") + \
               (f"_rank0_of_tp{args.emulate_tp}_emulated" if args.emulate_tp > 1 else "")
        print(json.dumps({"metric": name, "value": round(ms, 4), "unit": "ms",
                          "higher_is_better": False, "n_gpus": world, "steps": args.steps, "layers": L,
                          "ms_per_layer": round(ms / L, 4),
                          "estimate_40_layers_ms": round(ms / L * 40, 3),
                          "estimate_note": "all 40 layers ran: measured" if full else "extrapolated, not measured",
                          "tokens_per_step": round(toks / args.steps, 3), "dtype": "bf16 dense / e2m1 experts",
                          "data": "synthetic", "config": {"dim": cfg.dim, "heads": cfg.n_heads, "experts": cfg.n_routed_experts,
                                                          "topk": cfg.n_activated_experts, "context": args.prompt_len,
                                                          "parallelism": f"tp{world}", "spec": bool(args.spec), "pdl": bool(args.pdl),
                                                          "emulated_tp": args.emulate_tp,
                                                          "engram": "2 layers, tables resident" if (args.engram and full) else "left out",
                                                          "prefill_rows_per_chunk": args.max_rows,
                                                          "prefill_ms": round(prefill_ms, 2),
                                                          "prefill_ms_per_token": round(prefill_ms / args.prompt_len, 4),
                                                          }}))
    if world > 1 or args.emulate_tp > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def kernel_times(path, step, rank, world, what):
    """5 more calls of `step` under torch.profiler on rank 0 (every rank steps): per-kernel device times to `path`."""
    from torch.profiler import ProfilerActivity, profile
    import torch.distributed as dist
    sync = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    sync()
    if rank == 0:
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            sync()                       # the profiler's start-up is over before the peers' bounded waits begin
            for _ in range(5):
                step()
            torch.cuda.synchronize()
        rows = {}
        for ev in prof.events():
            if ev.device_type is not None and "cuda" in str(ev.device_type).lower() and ev.name:
                r = rows.setdefault(ev.name, [0, 0.0])
                r[0] += 1
                r[1] += float(ev.time_range.elapsed_us())
        tot = sum(v[1] for v in rows.values())
        with open(path, "w") as f:
            f.write(f"# per-kernel device time, 5 {what}, rank 0; total {tot / 5:.1f} us of kernel time per step\n")
            f.write("# us_per_step  launches_per_step  avg_us  kernel\n")
            for name, (n, us) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
                f.write(f"{us / 5:10.1f} {n / 5:8.1f} {us / max(n, 1):8.2f}  {name[:110]}\n")
    else:
        sync()
        for _ in range(5):
            step()
        torch.cuda.synchronize()
    sync()


def bench_batched(args, cfg, dev, model_rank, model_world, rank, world, allreduce, L):
    """--seqs N: N sequences through the continuous-batching engine (engine/dsv41_batch.py): prompts of --prompt-len
    tokens are admitted and prefilled, then --steps decode ticks (one graph replay of N rows each, one token per
    sequence, token read-back included) are timed with CUDA events.  Greedy, no speculation."""
    from ferrite_b200.engine.dsv41_batch import Dsv41BatchEngine
    from ferrite_b200.models.dsv41_synth import SyntheticDsv41Source
    from ferrite_b200.serve.engine import RequestSpec
    N = args.seqs
    eng = Dsv41BatchEngine(cfg, SyntheticDsv41Source(cfg, dev), model_rank, model_world, dev, allreduce,
                           max_ctx=args.prompt_len + args.steps + 64, max_seqs=N, prefill_rows=args.max_rows,
                           prefill_budget=N * args.prompt_len)
    g = torch.Generator().manual_seed(0)
    budget = args.steps + max(args.warmup, 3) + 8
    for _ in range(N):
        eng.submit(RequestSpec(torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist(), budget))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while eng.n_decoding() < N:
        eng.tick()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(max(args.warmup, 3)):
        eng.tick()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    toks = 0
    e0.record()
    for _ in range(args.steps):
        toks += sum(len(ev.ids) for _, ev in eng.tick() if ev.kind == "tokens")
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if args.kernel_times:
        kernel_times(args.kernel_times, eng.tick, rank, world, "decode ticks")
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({"metric": "dsv41_batched_decode_tok_s" + (f"_rank0_of_tp{args.emulate_tp}_emulated" if args.emulate_tp > 1 else ""),
                          "value": round(toks / args.steps / ms * 1e3, 1), "unit": "tok/s", "higher_is_better": True,
                          "n_gpus": world, "steps": args.steps, "ms_per_tick": round(ms, 3), "seqs": N, "layers": L,
                          "tokens_per_tick": round(toks / args.steps, 2), "launches_per_tick": eng.launches,
                          "dtype": "bf16 dense / e2m1 experts", "data": "synthetic",
                          "config": {"dim": cfg.dim, "experts": cfg.n_routed_experts, "topk": cfg.n_activated_experts,
                                     "context": args.prompt_len, "parallelism": f"tp{world}", "emulated_tp": args.emulate_tp,
                                     "speculation": "none (greedy)", "prefill_all_s": round(prefill_s, 3),
                                     "routed_experts": "block-scaled tcgen05 grouped GEMM" if 0 < eng.model.mx_min_rows <= N else "per-pair mma kernels"}}))
    if world > 1 or args.emulate_tp > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
