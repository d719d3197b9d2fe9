"""Multi-process plumbing on CPU (gloo, world size 2): sharded engine == single process,
tensor parallel == single process, and a rank that dies is reported instead of hanging."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

WORKER = str(Path(__file__).resolve().parent / "dist_worker.py")


def _run(nproc, dp_shard, tp, steps=4, fail_rank=-1, timeout=300, port=29631):
    env = dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1")
    if nproc == 1:
        cmd = [sys.executable, WORKER, str(dp_shard), str(tp), str(steps), str(fail_rank)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER, str(dp_shard), str(tp), str(steps),
               str(fail_rank)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


def _losses(proc):
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("LOSSES ")][-1]
    return json.loads(line[len("LOSSES "):])


@pytest.fixture(scope="module")
def single():
    return _losses(_run(1, 1, 1))


def test_fsdp_two_ranks_matches_single_process(single):
    two = _losses(_run(2, 2, 1, port=29632))
    assert len(two) == len(single)
    for a, b in zip(single, two):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, two)


def test_tensor_parallel_two_ranks_matches_single_process(single):
    two = _losses(_run(2, 1, 2, port=29633))
    for a, b in zip(single, two):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, two)


def test_rank_failure_is_detected_not_hung():
    # rank 1 raises between steps; the job must end with an error within the timeout
    proc = _run(2, 2, 1, fail_rank=1, timeout=240, port=29634)
    assert proc.returncode != 0
    assert "injected failure" in (proc.stderr + proc.stdout)
