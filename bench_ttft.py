"""Time to first token through the HTTP server.

Protocol (the reference's ``scripts/campaign/bench_protocol.sh:1-16``): one request at a time, greedy, a prompt of
about 4096 tokens, streamed; TTFT is the wall time from sending the request to the first ``data:`` frame of the
response.  The server is the package's own (`serve/api.py` over `EngineDriver` over the single-sequence GLM engine
with MTP), started in this process on 127.0.0.1; the client is a plain HTTP client on a socket, so the number holds
JSON parsing, tokenisation, admission, chunked prefill, sampling, the event hand-over and SSE framing.

  python bench_ttft.py                       # 1 GPU, 128 of 288 experts resident (the model does not fit one GPU)
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench_ttft.py --tp 8

Prompts are byte-tokenised text (no tokenizer files here), so a prompt of N characters is N + 30 tokens; weights are
random-init at production shapes.  ``max_tokens`` is 1: with random weights the first token is rarely a printable
byte, so the first frame is the one that also ends the request.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--prompt-tokens", type=int, default=4096)
    ap.add_argument("--requests", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--port", type=int, default=18431)
    ap.add_argument("--max-ctx", type=int, default=8192)
    ap.add_argument("--experts-resident", type=int, default=0)
    ap.add_argument("--prefill-rows", type=int, default=1024)
    args = ap.parse_args(argv)

    from ferrite_b200.serve.__main__ import build_engine
    resident = args.experts_resident or (128 if args.tp == 1 else 0)
    eargs = argparse.Namespace(model="glm53", model_dir=None, backend="cuda", tp=args.tp, synthetic=True, max_seqs=1, mtp=3,
                               max_ctx=args.max_ctx, experts_resident=resident, prefill_rows=args.prefill_rows)
    eng, tok, rank, world = build_engine(eargs)
    if rank != 0:
        eng.follow()
        return 0

    import uvicorn
    from ferrite_b200.serve.api import create_app
    from ferrite_b200.serve.engine import EngineDriver
    driver = EngineDriver(eng)
    app = create_app(driver, tok, "glm-5.3-flash")
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=args.port, log_level="warning"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    while not server.started:
        time.sleep(0.05)

    import http.client
    overhead = len(tok.encode_chat([{"role": "user", "content": ""}]))
    chars = max(8, args.prompt_tokens - overhead)
    ttft, total, ntok = [], [], 0
    for i in range(args.warmup + args.requests):
        words = "".join(chr(97 + (7 * i + 3 * j) % 26) if j % 6 else " " for j in range(chars))
        body = json.dumps({"model": "glm-5.3-flash", "stream": True, "max_tokens": 1, "include_usage": True,
                           "messages": [{"role": "user", "content": words}]})
        conn = http.client.HTTPConnection("127.0.0.1", args.port, timeout=600)
        t0 = time.perf_counter()
        conn.request("POST", "/v1/chat/completions", body, {"Content-Type": "application/json"})
        resp = conn.getresponse()
        t_first = None
        while True:
            line = resp.readline()
            if not line:
                break
            if line.startswith(b"data:"):
                if t_first is None:
                    t_first = time.perf_counter()
                if b'"usage"' in line:
                    ntok = json.loads(line[5:])["usage"]["prompt_tokens"]
                if line.strip() == b"data: [DONE]":
                    break
        t_end = time.perf_counter()
        conn.close()
        if resp.status != 200 or t_first is None:
            print(json.dumps({"metric": "p50_ttft_ms", "error": f"request {i}: HTTP {resp.status}"}))
            return 1
        if i >= args.warmup:
            ttft.append((t_first - t0) * 1e3)
            total.append((t_end - t0) * 1e3)
    server.should_exit = True
    th.join(timeout=10)
    driver.shutdown()
    if hasattr(eng, "stop"):
        eng.stop()
    p50 = statistics.median(ttft)
    print(json.dumps({
        "metric": "p50_ttft_ms", "value": round(p50, 1), "unit": "ms", "higher_is_better": False, "n_gpus": world,
        "requests": args.requests, "warmup": args.warmup, "prompt_tokens": ntok,
        "min_ms": round(min(ttft), 1), "max_ms": round(max(ttft), 1),
        "prefill_tok_s": round(ntok / (p50 * 1e-3), 1),
        "config": {"model": "GLM-5.3-Flash (45 layers, 1 MTP layer)", "parallelism": f"tp{world}",
                   "experts_resident_per_layer": resident or 288, "path": "HTTP /v1/chat/completions, SSE, byte tokenizer",
                   "weights": "random-init", "batch": 1, "sampling": "greedy", "prefill_rows": args.prefill_rows}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
