"""Multi-process plumbing on CPU (gloo, world size 2): sharded engine == single process,
tensor parallel == single process, and a rank that dies is reported instead of hanging."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

WORKER = str(Path(__file__).resolve().parent / "dist_worker.py")


def _run(nproc, dp_shard, tp, steps=4, fail_rank=-1, timeout=300, port=29631, dp_replicate=1, clip=1.0, ckpt=""):
    env = dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1")
    tail = [str(dp_shard), str(tp), str(steps), str(fail_rank), str(dp_replicate), str(clip)] + ([ckpt] if ckpt else [])
    if nproc == 1:
        cmd = [sys.executable, WORKER] + tail
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), WORKER] + tail
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


def test_hybrid_sharding_two_by_two_matches_single_process(single):
    """dp_replicate 2 x dp_shard 2: shards inside a pair, averaged across the pairs (lingua/distributed.py:106-113)."""
    four = _losses(_run(4, 2, 1, port=29635, dp_replicate=2))
    for a, b in zip(single, four):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (single, four)


def test_tensor_parallel_gradient_norm_clips_like_single_process():
    """A clip threshold far below the gradient norm: every step's update depends on the global norm, which under
    tensor parallelism is the sum over the TP ranks' slices plus the replicated parameters counted once."""
    one = _losses(_run(1, 1, 1, clip=0.05))
    two = _losses(_run(2, 1, 2, port=29636, clip=0.05))
    for a, b in zip(one, two):
        assert abs(a - b) < 2e-4 * max(1.0, abs(a)), (one, two)


@pytest.mark.parametrize("nproc,dp_shard,tp", [(2, 1, 2), (2, 2, 1), (4, 2, 2)])
def test_checkpoint_round_trip_keeps_every_ranks_shard(tmp_path, nproc, dp_shard, tp):
    proc = _run(nproc, dp_shard, tp, steps=2, port=29637, ckpt=str(tmp_path / "ckpt"))
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    assert proc.stdout.count("CKPT_OK") == nproc


def test_tp_sharding_keeps_the_float8_mark():
    """Sharding a layer over the TP group replaces its parameter; the request for float8 products has to survive."""
    import torch.nn as nn

    from lingua_b200.float8 import convert_linears_to_fp8, wants_fp8
    from lingua_b200.parallel.tensor_parallel import _shard_param

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([nn.Linear(64, 128, bias=False), nn.Linear(64, 24, bias=False)])

    m = Blk()
    convert_linears_to_fp8(m, "rowwise", r"layers\.[0-9]+")
    assert wants_fp8(m.layers[0].weight) and not wants_fp8(m.layers[1].weight)  # 24 is not a multiple of 16
    _shard_param(m.layers[0], 0, 2, 1)
    assert m.layers[0].weight.shape == (64, 64) and wants_fp8(m.layers[0].weight)
    _shard_param(m.layers[0], 1, 4, 0)  # 16 columns left: still a float8 shape
    assert wants_fp8(m.layers[0].weight)
    _shard_param(m.layers[0], 1, 2, 0)  # 8 columns: the kernels do not take it, the layer falls back to bf16
    assert not wants_fp8(m.layers[0].weight)
