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


def main():
    dp_shard, tp, steps = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    fail_rank = int(sys.argv[4]) if len(sys.argv) > 4 else -1
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        dist.init_process_group("gloo")
    rank = dist.get_rank() if world > 1 else 0
    torch.manual_seed(0)
    margs = LMTransformerArgs(dim=64, n_layers=2, n_heads=4, vocab_size=128, max_seqlen=32, seed=3)
    tr = Trainer(margs, DistributedArgs(dp_shard=dp_shard, tp_size=tp, fsdp_type="full_shard"),
                 OptimArgs(lr=1e-2, warmup=1, clip=1.0), total_steps=50, device=torch.device("cpu"))
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
    if rank == 0:
        print("LOSSES " + json.dumps(losses), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
