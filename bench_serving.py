"""Serving workload through the engine driver: many concurrent requests with ragged prompts, continuous batching.

The shape of the reference's batched-serving configuration: N requests arrive together (default 64), prompt lengths
uniform in [--prompt-min, --prompt-max] (512-4096) with uniform-random token ids, --new-tokens output tokens each
(512), chunked prefill, continuous batching over --max-seqs rows.  Every request goes through the same seam the HTTP
server uses (`serve/engine.py::EngineDriver`: submit -> events on a sink), so admission, the tick loop, the per-tick
token read-back and the event hand-over are inside the measurement.  Reported: whole-engine output tokens per second
over the run (first submit to last finish, wall clock), p50 / p95 time to first token, p50 time per output token.

    python bench_serving.py --model mock --requests 64                      # CPU: the planner + driver without a model
    python bench_serving.py --model glm53 --requests 64 --max-seqs 32       # one GPU (128 of 288 experts resident)
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_serving.py --model glm53 --tp 8 \\
        --requests 64 --max-seqs 32
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 bench_serving.py --model dsv41 --tp 4 \\
        --requests 32 --max-seqs 32 --prompt-min 2048 --prompt-max 2048 --new-tokens 256

Weights are random-init, prompts synthetic.  Rank 0 prints one JSON line; the other ranks follow its commands.
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import statistics
import sys
import threading
import time


class _Sink:
    """Event sink of one request: records arrival times on the driver thread, wakes the collector at the end."""

    def __init__(self, done: "queue.Queue"):
        self.t_first = None
        self.t_last = None
        self.tokens = 0
        self.reason = None
        self.done = done
        self.rid = None

    def put(self, ev):
        now = time.perf_counter()
        if ev.kind == "tokens":
            if self.t_first is None:
                self.t_first = now
            self.t_last = now
            self.tokens += len(ev.ids)
        elif ev.kind == "finished":
            self.reason = ev.reason
            self.done.put(self)


def run_workload(driver, prompts, new_tokens: int, stop_ids=()):
    """Submit every prompt at once, wait for all to finish.  Returns (wall seconds, per-request sinks, submit times)."""
    from ferrite_b200.serve.engine import RequestSpec
    done: "queue.Queue" = queue.Queue()
    sinks = [_Sink(done) for _ in prompts]
    t_sub = [0.0] * len(prompts)

    def client(i):   # one client thread per request, as the HTTP server's handlers: the driver admits all that queued
        t_sub[i] = time.perf_counter()          # up between two ticks in one go
        sinks[i].rid, _ = driver.submit(RequestSpec(list(prompts[i]), new_tokens, tuple(stop_ids)), sinks[i])

    t0 = time.perf_counter()
    threads = [threading.Thread(target=client, args=(i,), daemon=True) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for _ in prompts:
        done.get(timeout=3600)
    for t in threads:
        t.join(timeout=60)
    return time.perf_counter() - t0, sinks, t_sub


def summarise(wall: float, sinks, t_sub, prompts) -> dict:
    ttft = [(s.t_first - t) * 1e3 for s, t in zip(sinks, t_sub) if s.t_first is not None]
    tpot = [(s.t_last - s.t_first) * 1e3 / (s.tokens - 1) for s in sinks if s.tokens > 1]
    toks = sum(s.tokens for s in sinks)
    q = lambda v, f: sorted(v)[min(len(v) - 1, int(f * len(v)))] if v else None
    reasons = {}
    for s in sinks:
        reasons[s.reason] = reasons.get(s.reason, 0) + 1
    return {"output_tok_s": round(toks / wall, 1), "wall_s": round(wall, 3), "output_tokens": toks,
            "prompt_tokens": sum(len(p) for p in prompts),
            "p50_ttft_ms": round(statistics.median(ttft), 1) if ttft else None, "p95_ttft_ms": round(q(ttft, 0.95), 1) if ttft else None,
            "p50_ms_per_output_token": round(statistics.median(tpot), 3) if tpot else None, "finish_reasons": reasons}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="glm53", help="mock | glm53 | glm-tiny | dsv41 | dsv41-tiny")
    ap.add_argument("--tp", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-seqs", type=int, default=32, help="rows of the continuous batch")
    ap.add_argument("--prompt-min", type=int, default=512)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--mtp", type=int, default=1)
    ap.add_argument("--experts-resident", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)

    import random
    from ferrite_b200.serve.__main__ import build_engine
    from ferrite_b200.serve.engine import EngineDriver
    resident = args.experts_resident or (128 if (args.tp == 1 and args.model == "glm53") else 0)
    eargs = argparse.Namespace(model=args.model, model_dir=None, backend="cuda", tp=args.tp, synthetic=True,
                               max_seqs=args.max_seqs, mtp=args.mtp, max_ctx=args.prompt_max + args.new_tokens + 64,
                               experts_resident=resident, prefill_rows=1024)
    eng, tok, rank, world = build_engine(eargs)
    if rank != 0:
        eng.follow()
        return 0
    rng = random.Random(args.seed)
    vocab = min(getattr(tok, "vocab_size", 256), 256) if args.model == "mock" else 4096
    prompts = [[rng.randrange(1, vocab) for _ in range(rng.randint(args.prompt_min, args.prompt_max))]
               for _ in range(args.requests)]
    driver = EngineDriver(eng, idle_sleep=0.001)
    try:
        wall, sinks, t_sub = run_workload(driver, prompts, args.new_tokens)
    finally:
        driver.shutdown()
        if hasattr(eng, "stop"):
            eng.stop()
    out = summarise(wall, sinks, t_sub, prompts)
    print(json.dumps({"metric": "serving_output_tok_s", "value": out.pop("output_tok_s"), "unit": "tok/s",
                      "higher_is_better": True, "n_gpus": world, **out,
                      "config": {"model": args.model, "requests": args.requests, "max_seqs": args.max_seqs,
                                 "prompt_tokens": f"uniform {args.prompt_min}-{args.prompt_max}",
                                 "new_tokens": args.new_tokens, "parallelism": f"tp{world}", "mtp": args.mtp,
                                 "experts_resident_per_layer": resident or "all", "weights": "random-init",
                                 "data": "synthetic", "path": "EngineDriver (the HTTP server's engine seam)"}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
