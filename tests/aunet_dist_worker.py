"""Worker for the multi-process CPU (gloo) test of the hierarchical byte model; launched with
torch.distributed.run. Trains a tiny two-level model under ``dp_shard`` ranks on a fixed global batch
(token and pooling level packed as the data pipeline ships them) and prints the losses from rank 0."""
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist

from lingua_b200.api import Trainer
from lingua_b200.data.pipeline import split_levels
from lingua_b200.distributed import DistributedArgs
from lingua_b200.models.aunet import HierarchicalArgs, HierarchicalTransformer, build_fsdp_grouping_plan
from lingua_b200.models.transformer import BaseTransformerArgs
from lingua_b200.optim import OptimArgs


def loss_fn(model, x, y):
    tok, lv = split_levels(x)
    tgt, tlv = split_levels(y)
    ce, mask_loss, _ = model(tok, lv, tgt, tlv)
    return ce + 0.1 * mask_loss


def main():
    dp_shard, steps = int(sys.argv[1]), int(sys.argv[2])
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        dist.init_process_group("gloo")
    rank = dist.get_rank() if world > 1 else 0
    margs = HierarchicalArgs(dimensions=[32, 64, 96], head_dims=[8, 16, 32], layers=[1, 1, 2], sliding_windows=[16, 16, 32],
                             max_seqlens=[48, 24, 10], vocab_size=258, lambda_level=0.1, seed=5,
                             block=BaseTransformerArgs(multiple_of=16, norm_eps=1e-5))
    tr = Trainer(margs, DistributedArgs(dp_shard=dp_shard, fsdp_type="full_shard"), OptimArgs(lr=1e-2, warmup=1, clip=1.0),
                 total_steps=50, device=torch.device("cpu"), model_cls=HierarchicalTransformer,
                 grouping_plan=build_fsdp_grouping_plan(margs), loss_fn=loss_fn)
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, 256, (steps, 4, 49), generator=g)
    lv = (torch.rand(steps, 4, 49, generator=g) < 0.35).long() + (torch.rand(steps, 4, 49, generator=g) < 0.12).long()
    packed = tok | (lv << 32)
    dp_rank, dp = tr.mesh.local_rank("dp"), tr.mesh.size("dp")
    losses = []
    for s in range(steps):
        part = packed[s].chunk(dp)[dp_rank]
        loss = tr.train_step_async(torch.stack((part[:, :-1], part[:, 1:]), dim=-1))
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
