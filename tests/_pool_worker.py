"""gloo worker for test_tp_pool.py: replicated HostEngine across ranks, plus failure injection."""
import os
import sys
from datetime import timedelta

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ferrite_b200.serve.engine import HostEngine, RequestSpec  # noqa: E402
from ferrite_b200.serve.tp_pool import RankFailure, ReplicatedEngine  # noqa: E402


class Flaky(HostEngine):
    """Raises on one rank at a chosen tick (a host-side fault; no GPU involved)."""

    def __init__(self, bad_rank, bad_tick, rank):
        super().__init__()
        self.bad = rank == bad_rank
        self.bad_tick, self.n = bad_tick, 0

    def tick(self):
        self.n += 1
        if self.bad and self.n == self.bad_tick:
            raise RuntimeError("injected fault")
        return super().tick()


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=timedelta(seconds=20))
    if mode == "ok":
        eng = ReplicatedEngine(HostEngine(), rank, world)
        if rank == 0:
            ids = [eng.submit(RequestSpec(list(range(40 + i, 70 + i)), 6)) for i in range(3)]
            toks = {i: [] for i in ids}
            while not eng.idle():
                for rid, ev in eng.tick():
                    if ev.kind == "tokens":
                        toks[rid] += ev.ids
            eng.stop()
            assert all(len(v) == 6 for v in toks.values()), toks
            print("POOL_OK", sorted(toks.items()))
        else:
            eng.follow()
        # every rank ended with the same planner state
        s = eng.stats()["engine"]
        out = [None] * world
        dist.all_gather_object(out, (s["ticks"], s["tokens_committed"]))
        assert len(set(out)) == 1, out
    elif mode == "dsv41batch":
        # the batched DSV41 engine (host stand-in model) under replicated control: rank 0 submits and cancels, every
        # rank plans the same ticks and commits the same tokens
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from test_dsv41_batch_sched import FakeModel, expected
        from ferrite_b200.engine.dsv41_batch import Dsv41BatchEngine
        inner = Dsv41BatchEngine(None, None, max_ctx=64, max_seqs=2, prefill_rows=4, prefill_budget=6,
                                 model=FakeModel(3, 64, 4))
        eng = ReplicatedEngine(inner, rank, world)
        if rank == 0:
            prompts = [[7, 8, 9], list(range(20, 31)), [5], [40, 41]]
            ids = [eng.submit(RequestSpec(p, 5)) for p in prompts]
            toks = {i: [] for i in ids}
            n = 0
            while not eng.idle():
                n += 1
                if n == 2:
                    eng.cancel(ids[3])
                for rid, ev in eng.tick():
                    if ev.kind == "tokens":
                        toks[rid] += ev.ids
            eng.stop()
            for i, p in zip(ids[:3], prompts):
                assert toks[i] == expected(p, 5), (i, toks[i])
            assert toks[ids[3]] == []
            print("POOL_OK", sorted(toks.items()))
        else:
            eng.follow()
        s = eng.stats()["engine"]
        out = [None] * world
        dist.all_gather_object(out, (s["ticks"], s["tokens_committed"], s["free_slots"]))
        assert len(set(out)) == 1 and out[0][2] == 2, out
    elif mode == "fault":
        eng = ReplicatedEngine(Flaky(bad_rank=1, bad_tick=3, rank=rank), rank, world)
        try:
            if rank == 0:
                eng.submit(RequestSpec(list(range(50)), 20))
                while not eng.idle():
                    eng.tick()
            else:
                eng.follow()
            raise SystemExit("fault was not reported")
        except RankFailure as f:
            assert f.errors[1] and "injected fault" in f.errors[1] and f.errors[0] is None
            print(f"FAULT_SEEN rank{rank}")
    elif mode == "absent":
        # rank 1 never joins the tick: the others time out instead of hanging
        if rank == 1:
            return
        eng = ReplicatedEngine(HostEngine(), rank, world)
        try:
            if rank == 0:
                eng.submit(RequestSpec(list(range(20)), 4))
                eng.tick()
            else:
                eng.follow()
            raise SystemExit("missing rank was not detected")
        except Exception as e:
            print(f"ABSENT_SEEN rank{rank} {type(e).__name__}")
            os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
