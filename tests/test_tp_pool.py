"""CPU, multi-process (gloo): replicated engine control, all-rank error reports, watchdog."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, world, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_pool_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=180)


def test_replicated_engine_keeps_ranks_in_step():
    r = _run("ok", 2, 29611)
    assert r.returncode == 0 and "POOL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_batched_dsv41_engine_under_replicated_control():
    r = _run("dsv41batch", 2, 29614)
    assert r.returncode == 0 and "POOL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_failing_rank_is_reported_by_every_rank():
    r = _run("fault", 3, 29612)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert all(f"FAULT_SEEN rank{i}" in r.stdout for i in range(3)), r.stdout


def test_rank_that_never_joins_times_out():
    r = _run("absent", 2, 29613)
    assert "ABSENT_SEEN rank0" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
