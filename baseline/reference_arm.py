"""Runs the UNMODIFIED reference (facebookresearch/lingua, copied verbatim to baseline/_ref) for
bench.py's ``--impl reference`` arm: its own LMTransformer, parallelize_model (FSDP2 + SAC +
torch.compile), build_optimizer and the statements of its train-loop body
(apps/main/train.py:415-442) on synthetic token batches. Only import-time stand-ins for the
uninstallable xformers package are added (baseline/shims); none of this repository's models,
kernels or engine are on this path.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def available() -> str | None:
    if not (REF / "lingua" / "transformer.py").exists():
        return "baseline/_ref has no copy of the reference sources"
    return None


def build(model_kwargs: dict, n_gpus: int, lr: float, total_steps: int, compile_model: bool, sac: bool,
          tp: int = 1, float8: bool = False):
    """Returns (step_fn(tokens[B,S+1] on device) -> loss tensor, info dict)."""
    for p in (str(HERE / "shims"), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    from apps.main.transformer import (LMTransformer, LMTransformerArgs, build_fsdp_grouping_plan,
                                       get_no_recompute_ops, tp_parallelize)
    from lingua.distributed import DistributedArgs, get_device_mesh, parallelize_model
    from lingua.optim import OptimArgs, build_optimizer
    from torch.distributed._tensor import DTensor

    # the reference's own switches: tensor parallelism (which it runs without torch.compile) and its row-wise float8
    # recipe on the linear layers of the blocks (lingua/distributed.py:403-417)
    dist_args = DistributedArgs(dp_shard=n_gpus // tp, dp_replicate=1, tp_size=tp, fsdp_type="full_shard",
                                model_dtype="bf16", compile=compile_model and tp == 1,
                                selective_activation_checkpointing=sac,
                                float8_recipe="rowwise" if float8 else None)
    mesh = get_device_mesh(dist_args)
    margs = LMTransformerArgs(**model_kwargs)
    torch.manual_seed(777)
    with torch.device("meta"):
        model = LMTransformer(margs)
    model = parallelize_model(model, mesh, margs, dist_args, fsdp_grouping_plan=build_fsdp_grouping_plan(margs),
                              tp_parallelize=tp_parallelize, no_recompute_ops=get_no_recompute_ops())
    model = model.to_empty(device="cuda")
    with torch.random.fork_rng(devices=[torch.cuda.current_device()]):
        torch.manual_seed(margs.seed)
        model.init_weights()
    oargs = OptimArgs(lr=lr, warmup=2000, clip=1.0)
    optimizer, scheduler = build_optimizer(model, oargs, total_steps)

    def step_fn(tokens):
        input_ids, labels = tokens[:, :-1], tokens[:, 1:]
        loss = model(input_ids, labels)
        loss.backward()
        grad_norm = torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=oargs.clip, foreach=True)
        grad_norm = grad_norm.full_tensor() if isinstance(grad_norm, DTensor) else grad_norm
        optimizer.step()
        scheduler.step()
        optimizer.zero_grad()
        return loss.detach()

    return step_fn, {"compile": compile_model and tp == 1, "sac": sac}


RECURRENT = {
    "hawk_1b": ("apps.fastRNN.hawk.hawk", "LMHawk", "LMHawkArgs"),
    "mingru_1b": ("apps.fastRNN.minGRU.mingru", "LMMinGRU", "LMMinGRUArgs"),
    "minlstm_1b": ("apps.fastRNN.minLSTM.minlstm", "LMMinLSTM", "LMMinLSTMArgs"),
}


def build_recurrent(name: str, model_kwargs: dict, n_gpus: int, lr: float, total_steps: int, compile_model: bool,
                    sac: bool):
    """The reference's recurrent language models (apps/fastRNN) the way its own train script builds them
    (apps/fastRNN/train.py:258-300): model on the meta device, ``parallelize_model`` with the default grouping plan,
    ``init_weights``, ``build_optimizer``. Their third-party CUDA / Triton extensions (causal_conv1d, accelerated_scan)
    cannot be built offline; ``baseline/shims`` restates exactly those calls in PyTorch ops, so this arm measures the
    reference's model code on PyTorch-restated kernels."""
    import importlib

    for p in (str(HERE / "shims"), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    from lingua.distributed import DistributedArgs, get_device_mesh, parallelize_model
    from lingua.optim import OptimArgs, build_optimizer
    from torch.distributed._tensor import DTensor

    torch.set_grad_enabled(True)  # a failed traced attempt can leave gradient recording switched off
    mod_name, cls_name, args_name = RECURRENT[name]
    mod = importlib.import_module(mod_name)
    dist_args = DistributedArgs(dp_shard=n_gpus, dp_replicate=1, tp_size=1, fsdp_type="full_shard", model_dtype="bf16",
                                compile=compile_model, selective_activation_checkpointing=sac)
    mesh = get_device_mesh(dist_args)
    margs = getattr(mod, args_name)(**model_kwargs)
    torch.manual_seed(777)
    with torch.device("meta"):
        model = getattr(mod, cls_name)(margs)
    model = parallelize_model(model, mesh, margs, dist_args, fsdp_grouping_plan=None, tp_parallelize=None,
                              no_recompute_ops=model._get_no_recompute_ops())
    model = model.to_empty(device="cuda")
    with torch.random.fork_rng(devices=[torch.cuda.current_device()]):
        torch.manual_seed(margs.seed)
        model.init_weights()
    oargs = OptimArgs(lr=lr, warmup=2000, clip=1.0)
    optimizer, scheduler = build_optimizer(model, oargs, total_steps)

    def step_fn(tokens):
        input_ids, labels = tokens[:, :-1], tokens[:, 1:]
        loss = model(input_ids, labels)
        loss.backward()
        grad_norm = torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=oargs.clip, foreach=True)
        grad_norm = grad_norm.full_tensor() if isinstance(grad_norm, DTensor) else grad_norm
        optimizer.step()
        scheduler.step()
        optimizer.zero_grad()
        return loss.detach()

    return step_fn, {"compile": compile_model, "sac": sac,
                     "kernels": "causal_conv1d / accelerated_scan restated in PyTorch ops (baseline/shims)"}
