"""Worker for the multi-process CPU (gloo) tests; launched with torch.distributed.run.

Trains the small reference-path model for a few steps under a given (dp_shard, tp) layout on a
fixed global batch and prints the losses as JSON from rank 0."""
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist

from lingua_b200.api import Trainer
from lingua_b200.distributed import DistributedArgs
from lingua_b200.models.transformer import LMTransformerArgs
from lingua_b200.optim import OptimArgs


def roundtrip(tr, margs, dargs, ckpt_dir, rank):
    """Save the engine through torch.distributed.checkpoint, load it into a differently initialised engine of the
    same layout and compare every rank's weights and Adam moments with what was saved."""
    import torch.distributed.checkpoint as dcp

    from lingua_b200.checkpoint import engine_state_dict, load_engine_state_dict

    dcp.save(engine_state_dict(tr.engine, lr=1e-2), checkpoint_id=ckpt_dir)
    margs2 = LMTransformerArgs(**{**margs.__dict__, "seed": margs.seed + 1})
    other = Trainer(margs2, dargs, OptimArgs(lr=1e-2, warmup=1), total_steps=50, device=torch.device("cpu"))
    assert any(not torch.equal(a.master, b.master) for a, b in zip(tr.engine.groups, other.engine.groups))
    sd = engine_state_dict(other.engine)
    dcp.load(sd, checkpoint_id=ckpt_dir)
    load_engine_state_dict(other.engine, sd, load_optim=True)
    for a, b in zip(tr.engine.groups, other.engine.groups):
        n = a.shard_numel
        for key in ("master", "exp_avg", "exp_avg_sq"):
            x, y = getattr(a, key)[:n], getattr(b, key)[:n]
            assert torch.equal(x, y), f"rank {rank}: {a.name}.{key} differs after reload ({float((x - y).abs().max())})"
        assert torch.equal(a.full, b.full), f"rank {rank}: compute copy of {a.name} differs after reload"
    assert other.engine.step_count == tr.engine.step_count
    print(f"CKPT_OK rank {rank}", flush=True)


def main():
    dp_shard, tp, steps = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    fail_rank = int(sys.argv[4]) if len(sys.argv) > 4 else -1
    dp_replicate = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    clip = float(sys.argv[6]) if len(sys.argv) > 6 else 1.0
    ckpt_dir = sys.argv[7] if len(sys.argv) > 7 else ""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        dist.init_process_group("gloo")
    rank = dist.get_rank() if world > 1 else 0
    torch.manual_seed(0)
    margs = LMTransformerArgs(dim=64, n_layers=2, n_heads=4, vocab_size=128, max_seqlen=32, seed=3)
    dargs = DistributedArgs(dp_replicate=dp_replicate, dp_shard=dp_shard, tp_size=tp, fsdp_type="full_shard")
    tr = Trainer(margs, dargs, OptimArgs(lr=1e-2, warmup=1, clip=clip), total_steps=50, device=torch.device("cpu"))
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, 128, (steps, 4, 33), generator=g)  # global batch of 4 sequences per step
    dp_rank, dp = tr.mesh.local_rank("dp"), tr.mesh.size("dp")
    losses = []
    for s in range(steps):
        if rank == fail_rank and s == 1:
            raise RuntimeError("injected failure")
        part = tok[s].chunk(dp)[dp_rank]
        batch = torch.stack((part[:, :-1], part[:, 1:]), dim=-1)
        loss = tr.train_step_async(batch)
        if dp > 1:
            dist.all_reduce(loss, group=tr.mesh.group("dp"))
            loss = loss / dp
        losses.append(float(loss))
    if ckpt_dir:
        roundtrip(tr, margs, dargs, ckpt_dir, rank)
    if rank == 0:
        print("LOSSES " + json.dumps(losses), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
