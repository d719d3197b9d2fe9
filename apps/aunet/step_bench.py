"""Training-step throughput of the hierarchical byte model on one GPU, synthetic bytes and boundaries.

``python -m apps.aunet.step_bench --config apps/aunet/configs/2B_1level.yaml [--steps 6 --warmup 3] [--profile]``

Builds the model named by the config's ``model`` and ``data.{batch_size,seq_len}`` sections on the sharded
engine (one rank), runs forward + backward + AdamW per step, times the steps with CUDA events and prints one
JSON line. ``--profile`` adds one extra step under the PyTorch profiler and lists the device time per kernel
(shares only: times taken under a profiler are not throughput numbers)."""
from __future__ import annotations

import argparse
import json

import torch

from lingua_b200.config import dataclass_from_dict, load_yaml
from lingua_b200.models.aunet import HierarchicalArgs, HierarchicalTransformer, build_fsdp_grouping_plan
from lingua_b200.parallel.engine import EngineOptim, ShardedEngine


def build(cfg: dict, seq_len: int, device):
    margs = dataclass_from_dict(HierarchicalArgs, cfg["model"], strict=False)
    if margs.max_seqlens[0] < 0:
        margs.max_seqlens[0] = seq_len
    if margs.vocab_size < 0:
        margs.vocab_size = 258  # byte tokenizer: 256 values + <bos> + <eos>
    with torch.device("meta"):
        model = HierarchicalTransformer(margs)
    engine = ShardedEngine(model, build_fsdp_grouping_plan(margs), process_group=False, compute_dtype=torch.bfloat16,
                           optim=EngineOptim(), device=device)
    for mod in model.modules():
        for name, buf in list(mod._buffers.items()):
            if buf is not None and buf.device.type == "meta":
                mod._buffers[name] = torch.empty_like(buf, device=device)
    model._engine = engine
    engine.init_weights_fp32(model.init_weights)
    return margs, model, engine


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="apps/aunet/configs/2B_1level.yaml")
    ap.add_argument("--batch", type=int, default=0, help="0 = data.batch_size of the config")
    ap.add_argument("--seq", type=int, default=0, help="0 = data.seq_len of the config")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--boundary-rate", type=float, default=0.2, help="share of bytes that end a word")
    ap.add_argument("--profile", action="store_true")
    a = ap.parse_args(argv)
    cfg = load_yaml(a.config)
    B = a.batch or cfg["data"]["batch_size"]
    S = a.seq or cfg["data"]["seq_len"]
    dev = torch.device("cuda", 0)
    margs, model, engine = build(cfg, S, dev)
    n_levels = len(margs.dimensions) - 1
    gen = torch.Generator().manual_seed(0)
    host = []
    for _ in range(4):  # pinned host batches, token and level packed as the data pipeline ships them
        tok = torch.randint(0, 256, (B, S + 1), generator=gen)
        u = torch.rand(B, S + 1, generator=gen)
        lv = sum((u < a.boundary_rate * 0.3 ** l).long() for l in range(n_levels))
        lv[:, 0] = n_levels
        host.append((tok | (lv << 32)).pin_memory())

    def step(i):
        packed = host[i % len(host)].to(dev, non_blocking=True)
        tok, lv = packed & 0xFFFFFFFF, packed >> 32
        engine.zero_grad()
        loss, _, _ = model(tok[:, :-1], lv[:, :-1], tok[:, 1:].contiguous(), lv[:, 1:].contiguous())
        loss.backward()
        engine.step(1e-4)
        return loss

    for i in range(a.warmup):
        step(i)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for i in range(a.steps):
        loss = step(i)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / a.steps
    fpt = model.flops_per_token()
    print(json.dumps({"metric": "training bytes/s", "value": B * S / ms * 1e3, "ms_per_step": ms, "batch": B,
                      "seq_len": S, "params": engine.n_params, "model_flops_per_s": fpt * B * S / ms * 1e3,
                      "loss": float(loss), "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
                      "config": a.config, "data": "synthetic"}))
    if a.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            step(0)
            torch.cuda.synchronize()
        rows = [(e.key[:72], e.device_time_total / 1e3, e.count) for e in prof.key_averages()
                if e.device_time_total > 0 and e.device_type.name == "CUDA"]
        rows.sort(key=lambda r: -r[1])
        total = sum(r[1] for r in rows)
        print(f"device time of one step under the profiler: {total:.1f} ms")
        for name, t, c in rows[:30]:
            print(f"{t:9.2f} ms {100 * t / total:5.1f}% {c:5d}  {name}")


if __name__ == "__main__":
    main()
