"""Command line: one-shot generation or the HTTP server.

  python -m ferrite_b200.serve --model mock --serve --port 8000
  python -m ferrite_b200.serve --model glm53 --model-dir /ckpt --prompt "hi" --max-tokens 64
  python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m ferrite_b200.serve \
      --model glm53 --synthetic --tp 4 --serve --max-seqs 16

Flags follow the reference binary (``crates/ferrite-serve/src/main.rs:39-68``): ``--model``,
``--model-dir``, ``--backend cpu|cuda``, ``--tp``, ``--prompt``, ``--serve``, ``--port``,
``--max-seqs``, ``--model-name``, ``--max-tokens``; ``--mtp N`` selects the verify width of the
speculative step (single-sequence engine with ``--max-seqs 1``, batched engine otherwise; 1 = greedy).
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def build_engine(args):
    """Returns (ServeEngine, tokenizer, rank, world)."""
    from .engine import HostEngine, SingleFlight
    from .tokenizer import ChatTokenizer
    tok = ChatTokenizer.load(args.model_dir)
    if args.model == "mock":
        return HostEngine(vocab=tok.vocab_size, max_rows=args.max_seqs), tok, 0, 1
    import torch
    if args.model.startswith("dsv41"):
        return _build_dsv41(args, tok)
    from ..config import EngineConfig, GlmConfig
    cfgs = {"glm53": GlmConfig.production, "glm-tiny": GlmConfig.tiny, "glm-golden4": GlmConfig.golden4}
    if args.model not in cfgs:
        raise SystemExit(f"unknown --model {args.model} (mock, {', '.join(cfgs)})")
    cfg = GlmConfig.from_hf(os.path.join(args.model_dir, "config.json")) \
        if args.model_dir and os.path.exists(os.path.join(args.model_dir, "config.json")) else cfgs[args.model]()
    if args.backend == "cpu":
        from ..models.checkpoint import CheckpointSource
        from ..models.glm_ref import GlmReference
        from ..models.glm_weights import random_weights
        from ..models.glm_weights import weight_layout
        if args.model_dir and not args.synthetic:
            src = CheckpointSource(args.model_dir, cfg)
            w = {k: src.get(k) for k in weight_layout(cfg)}
        else:
            w = random_weights(cfg, 0)
        return SingleFlight(_RefStep(GlmReference(cfg, w))), tok, 0, 1
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.tp, f"--tp {args.tp} needs {args.tp} processes (torch.distributed.run), got {world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    allreduce = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.collective import make_allreduce, self_test
        allreduce = make_allreduce(dev, rank, world, max_elems=64 * cfg.hidden_size, kind="p2p")
        verdict = self_test(allreduce, dev, rank, world)   # a fused kernel that fails its check is detached
        if rank == 0:
            print(f"collective self-test: {verdict}", flush=True)
    from ..models.glm import SyntheticSource
    if args.model_dir and not args.synthetic:
        from ..models.checkpoint import CheckpointSource
        src = CheckpointSource(args.model_dir, cfg, dev)
    else:
        src = SyntheticSource(cfg, dev)
    mtp = args.mtp      # verify width: the single-sequence engine's step, or every sequence's group in the batched one
    ecfg = EngineConfig(tp=world, max_ctx=args.max_ctx, mtp_n=mtp, experts_resident=args.experts_resident or None)
    if args.max_seqs == 1:
        from ..engine.glm_engine import GlmEngine
        eng = SingleFlight(_GlmStep(GlmEngine(cfg, ecfg, src, rank, world, dev, allreduce,
                                              prefill_rows=getattr(args, "prefill_rows", 1024)), mtp > 1))
    else:
        from ..engine.gpu_engine import GpuEngine
        eng = GpuEngine(cfg, ecfg, src, rank, world, dev, allreduce, max_rows=args.max_seqs)
    if world > 1:
        from .tp_pool import ReplicatedEngine, make_control_group
        eng = ReplicatedEngine(eng, rank, world, make_control_group())
    return eng, tok, rank, world


def _build_dsv41(args, tok):
    """DSV41: ``--model dsv41-tiny`` (random weights) or ``--model dsv41 --model-dir DIR`` (checkpoint)."""
    import torch
    from ..engine.dsv41_engine import Dsv41Engine, Dsv41StepEngine
    from ..models.dsv41 import DictWeights
    from ..models.dsv41_config import Dsv41Config
    from .engine import SingleFlight
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.tp, f"--tp {args.tp} needs {args.tp} processes (torch.distributed.run), got {world}"
    cfg_path = os.path.join(args.model_dir, "config.json") if args.model_dir else None
    if cfg_path and os.path.exists(cfg_path):
        cfg = Dsv41Config.from_hf(cfg_path)
    else:
        cfg = Dsv41Config.tiny() if args.model == "dsv41-tiny" else Dsv41Config.flash()
    if args.model_dir and not args.synthetic:
        from ..models.dsv41_checkpoint import Dsv41CheckpointSource
        src = Dsv41CheckpointSource(args.model_dir, cfg)
    elif args.backend == "cpu" or args.model == "dsv41-tiny":
        from ..models.dsv41_weights import random_weights
        src = DictWeights(random_weights(cfg, 0))
    else:
        src = None   # production shapes: synthetic weights are generated on the device, shard by shard (below)
    if args.backend == "cpu":
        from ..models.dsv41_ref import Dsv41Reference
        from ..models.dsv41_weights import tensor_specs
        w = {k: src.get(k) for k in tensor_specs(cfg)}
        return SingleFlight(_Dsv41RefStep(Dsv41Reference(cfg, w), spec=args.mtp > 1)), tok, 0, 1
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # refuse a model that cannot fit before anything is allocated (475 GiB at production shapes: TP >= 4 on 180 GB parts)
    from ..models.dsv41_weights import estimate_device_bytes
    need, have = estimate_device_bytes(cfg, world), torch.cuda.get_device_properties(dev).total_memory
    if need > 0.92 * have:
        raise SystemExit(f"--model {args.model} at --tp {world} needs about {need / 2**30:.0f} GiB of weights per GPU, "
                         f"this GPU has {have / 2**30:.0f} GiB: use more ranks")
    if src is None:
        from ..models.dsv41_synth import SyntheticDsv41Source
        src = SyntheticDsv41Source(cfg, dev)
    allreduce = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from ..parallel.collective import make_allreduce, self_test
        allreduce = make_allreduce(dev, rank, world, max_elems=64 * max(cfg.dim, 4096), kind="p2p")
        verdict = self_test(allreduce, dev, rank, world)   # a fused kernel that fails its check is detached
        if rank == 0:
            print(f"collective self-test: {verdict}", flush=True)
    # prefill chunk: 256 rows measured 0.36 ms per prompt token against 0.69 ms with 64 rows (one-GPU shard of TP=4);
    # on several GPUs the 64-row chunk is the measured configuration
    chunk = min(256 if world == 1 else 64, getattr(args, "prefill_rows", 256))
    if args.max_seqs > 1:   # continuous batching, greedy: one row per live sequence in one forward per tick
        from ..engine.dsv41_batch import Dsv41BatchEngine
        serve_eng = Dsv41BatchEngine(cfg, src, rank, world, dev, allreduce, max_ctx=args.max_ctx, max_seqs=args.max_seqs,
                                     prefill_rows=chunk, prefill_budget=max(256, chunk))
    else:
        eng = Dsv41Engine(cfg, src, rank, world, dev, allreduce, max_ctx=args.max_ctx, max_rows=max(8, chunk))
        serve_eng = SingleFlight(Dsv41StepEngine(eng, spec=args.mtp > 1))
    if world > 1:
        from .tp_pool import ReplicatedEngine, make_control_group
        serve_eng = ReplicatedEngine(serve_eng, rank, world, make_control_group())
    return serve_eng, tok, rank, world


class _Dsv41RefStep:
    """StepEngine over the fp32 DSV41 golden model (CPU): plain greedy steps or DSpark speculation."""

    def __init__(self, ref, spec: bool):
        self.ref, self.spec = ref, spec and ref.cfg.dspark_block_size > 0

    def start(self, prompt):
        from ..ops.reference import argmax_first
        self.st = self.ref.new_seq()
        logits, mh = self.ref.forward(self.st, prompt)
        if self.spec:
            self.ref.dspark_seed(self.st, mh, 0)
        self.last = int(argmax_first(logits[-1:])[0])
        return self.last, 0

    def step(self):
        from ..ops.reference import argmax_first
        from ..spec import spec_accept
        ref, st = self.ref, self.st
        if not self.spec:
            logits, _ = ref.forward(st, [self.last])
            self.last = int(argmax_first(logits[-1:])[0])
            return [self.last]
        last_pos = st.pos - 1
        drafts, _, _ = ref.dspark_draft(st, self.last, last_pos)
        snap = st.clone()
        block = [self.last] + drafts
        logits, _ = ref.forward(st, block)
        judges = argmax_first(logits).tolist()
        m = spec_accept(drafts, judges, anchor_is_in_block=False)
        self.st = st = snap
        _, mh = ref.forward(st, block[:m + 1])
        ref.dspark_seed(st, mh, last_pos + 1)
        self.last = judges[m]
        return judges[:m + 1]


class _GlmStep:
    """StepEngine over the single-sequence GLM engine."""

    def __init__(self, eng, mtp: bool):
        self.eng, self.mtp = eng, mtp

    def start(self, prompt):
        first = self.eng.prefill(prompt if len(prompt) >= 2 else [prompt[0]] * 2)
        self.eng.build_graphs(self.mtp)
        return first, 0

    def step(self):
        return self.eng.spec_step() if self.mtp else [self.eng.step_plain()]

    def max_prompt(self):
        return self.eng.max_prompt()

    def room(self):
        return self.eng.room()


class _RefStep:
    """StepEngine over the fp32 CPU reference engine."""

    def __init__(self, ref):
        self.ref = ref

    def start(self, prompt):
        self.st = self.ref.new_seq()
        self.last = self.ref.prefill(self.st, prompt)
        return self.last, 0

    def step(self):
        self.last = self.ref.decode_greedy(self.st, self.last, 2)[-1]
        return [self.last]


def main(argv=None):
    ap = argparse.ArgumentParser(prog="ferrite_b200.serve")
    ap.add_argument("--model", default="mock")
    ap.add_argument("--model-dir", default=None)
    ap.add_argument("--backend", default="cuda", choices=["cpu", "cuda"])
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--serve", action="store_true")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-seqs", type=int, default=1)
    ap.add_argument("--model-name", default=None)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--max-ctx", type=int, default=8192)
    ap.add_argument("--mtp", type=int, default=3)
    ap.add_argument("--synthetic", action="store_true", help="random-init weights instead of a checkpoint")
    ap.add_argument("--experts-resident", type=int, default=0)
    ap.add_argument("--prefill-rows", type=int, default=1024,
                    help="rows per prefill chunk of the single-sequence engine (the tensor-core expert GEMM and the "
                         "chunked GatedDeltaNet scan take over from 64 rows)")
    ap.add_argument("--cpu-profile", default=None, metavar="FILE",
                    help="host CPU profile (cProfile) of the one-shot run, written as pstats to FILE with the 25 heaviest "
                         "functions on stderr: the counterpart of the reference's pprof switch (crates/ferrite-serve/src/main.rs)")
    args = ap.parse_args(argv)
    if args.cpu_profile and not args.serve:
        import cProfile
        import pstats
        prof = cProfile.Profile()
        args_file, args.cpu_profile = args.cpu_profile, None
        try:
            return prof.runcall(_run, args)
        finally:
            prof.dump_stats(args_file)
            pstats.Stats(prof, stream=sys.stderr).sort_stats("cumulative").print_stats(25)
    return _run(args)


def _run(args):
    eng, tok, rank, world = build_engine(args)
    if rank != 0:
        eng.follow()
        return 0
    name = args.model_name or args.model
    if args.serve:
        from .api import serve
        serve(eng, tok, args.host, args.port, name)
        return 0
    from .engine import RequestSpec
    prompt = tok.encode_chat([{"role": "user", "content": args.prompt or "Hello"}])
    rid = eng.submit(RequestSpec(prompt, args.max_tokens, tuple(tok.stop_ids())))
    t0, ids, t_first = time.time(), [], None
    while True:
        done = False
        for r, ev in eng.tick():
            if ev.kind == "tokens":
                t_first = t_first or time.time()
                ids += ev.ids
            elif ev.kind == "finished":
                done = True
        if done:
            break
    dt = time.time() - (t_first or t0)
    print(tok.decode(ids))
    print(f"[stats] prompt {len(prompt)} tok, ttft {((t_first or t0) - t0) * 1e3:.1f} ms, "
          f"{len(ids)} tok in {dt:.3f} s = {len(ids) / max(dt, 1e-9):.1f} tok/s", file=sys.stderr)
    if hasattr(eng, "stop"):
        eng.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
