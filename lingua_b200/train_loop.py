"""The training loop shared by every app (apps.main, apps.mamba, apps.fastRNN, apps.mtp).

One function, ``run_training(args, spec)``, implements the sequence of apps/main/train.py:221-601:
tokenizer -> validate -> logger / signal handler / env / process group / mesh -> model on the meta
device -> parallelise (sharded engine) -> initialise or load weights -> optimiser state, scheduler,
data-loader state -> resume from the newest checkpoint -> loop {batch, forward + backward with
gradient accumulation, clip + AdamW + scheduler, metrics every ``logging.freq``, checkpoints,
evaluation, preemption}. The apps differ only in their ``ModelSpec`` (model class, args class,
grouping plan, loss unpacking), where the reference keeps four copies of the loop.
"""
from __future__ import annotations

import gc
import logging
import os
import sys
from contextlib import ExitStack
from copy import deepcopy
from dataclasses import asdict, dataclass, field
from pathlib import Path
from timeit import default_timer as timer
from typing import Any, Callable, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .checkpoint import CheckpointArgs, CheckpointManager, load_from_checkpoint
from .config import dataclass_from_dict, dump_config, flatten_dict
from .data.pipeline import DataArgs, build_dataloader_from_args, init_dataloader_state_from_args
from .distributed import (DistributedArgs, EnvironmentArgs, check_model_value_range, clean_env, dist_mean_dict,
                          get_device_mesh, get_is_master, get_world_size, init_signal_handler, parallelize_model,
                          requeue_slurm_job, setup_env, setup_torch_distributed)
from .logger import init_logger
from .metrics import GPUMemoryMonitor, LoggingArgs, MetricLogger, get_num_params, peak_flops
from .ops import _lib as kernel_lib
from .optim import LRScheduler, OptimArgs, build_engine_optim, build_lr_fn
from .profiling import ProfilerArgs, maybe_run_profiler, nvtx_range
from .tokenizer import build_tokenizer

logger = logging.getLogger()


@dataclass
class TrainArgs:
    name: str = "lingua"
    dump_dir: str = ""
    seed: int = 42
    # optimiser steps are taken every grad_acc_steps micro-batches
    grad_acc_steps: int = 1
    gc_collect_freq: int = 1000
    probe_freq: Optional[int] = None
    steps: int = 1000
    data: DataArgs = field(default_factory=DataArgs)
    optim: OptimArgs = field(default_factory=OptimArgs)
    model: Any = None
    distributed: DistributedArgs = field(default_factory=DistributedArgs)
    env: EnvironmentArgs = field(default_factory=EnvironmentArgs)
    checkpoint: CheckpointArgs = field(default_factory=CheckpointArgs)
    profiling: ProfilerArgs = field(default_factory=ProfilerArgs)
    logging: LoggingArgs = field(default_factory=LoggingArgs)
    # None runs evaluation in this process on the training GPUs; a number submits a separate job
    async_eval_gpus: Optional[int] = None
    eval: Optional[Any] = None


@dataclass
class ModelSpec:
    """What an app contributes to the loop."""
    model_cls: Callable
    build_plan: Optional[Callable] = None  # model_args -> [(module path, reshard_after_forward)]
    tp_parallelize: Optional[Callable] = None
    flops_per_token: Optional[Callable] = None  # (n_params, model_args, seq_len) -> float
    labels_from_batch: Callable = lambda batch: batch[:, :, 1]
    # (model, inputs, labels) -> loss or (loss, {name: tensor}) for extra logged losses
    loss_fn: Callable = lambda model, x, y: model(x, y)
    eval_module: str = "apps.main.eval"


@dataclass
class TrainState:
    step: int  # optimiser steps taken
    acc_step: int  # micro-batches accumulated since the last optimiser step
    scheduler: LRScheduler
    data_loader_state: Dict[str, Any]

    def state_dict(self) -> Dict[str, Any]:
        return {"step": self.step, "acc_step": self.acc_step, "data_loader_state": self.data_loader_state,
                "scheduler": self.scheduler.state_dict()}

    def load_state_dict(self, sd) -> None:
        self.step, self.acc_step = sd["step"], sd["acc_step"]
        self.data_loader_state = dict(sd["data_loader_state"])
        self.scheduler.load_state_dict(sd["scheduler"])


preemption_flag = dict(flag=False)


def set_preemption_flag(signum, frame):
    logger.warning("Signal handler called with signal " + str(signum))
    logger.warning("Preemption ! checkpointing asap and exiting.")
    preemption_flag["flag"] = True


def every_n_steps(train_state, freq, acc_step=None, acc_freq=None) -> bool:
    test = train_state.step % freq == 0
    if acc_step is not None:
        test = test and (train_state.acc_step == acc_step)
    elif acc_freq is not None:
        test = test and ((train_state.acc_step % acc_freq) == 0)
    return test


def validate_train_args(args: TrainArgs, output_size: int) -> None:
    if args.model.vocab_size < 0:
        logger.info(f"Setting model output size to {output_size}")
        args.model.vocab_size = output_size
    assert args.model.vocab_size == output_size, "Vocab size should be the same as output size"
    assert args.dump_dir, "Dump dir not set"
    if args.checkpoint.path is None:
        args.checkpoint.path = str(Path(args.dump_dir) / "checkpoints")
        logger.info(f"Setting checkpoint path to {args.checkpoint.path}")
    if args.data.root_dir is not None:
        for source in args.data.sources:
            data_path = os.path.join(args.data.root_dir, source)
            assert os.path.exists(data_path), f"{data_path} doesn't exist"
    d = args.distributed
    if d.dp_replicate * d.dp_shard * d.tp_size != get_world_size():
        assert get_world_size() % d.dp_shard == 0
        d.dp_replicate = get_world_size() // d.dp_shard
        assert d.dp_replicate % d.tp_size == 0
        d.dp_replicate = d.dp_replicate // d.tp_size
        logger.warning(f"Setting Data Parallel size to {d.dp_replicate * d.dp_shard}")
        assert d.dp_replicate * d.dp_shard * d.tp_size == get_world_size()
        if d.fsdp_type == "no_shard":
            assert d.dp_shard == 1 and d.dp_replicate == get_world_size()
    if hasattr(args.model, "max_seqlens"):  # hierarchical model: stage 0 runs at the data sequence length
        if args.model.max_seqlens[0] < 0:
            args.model.max_seqlens[0] = args.data.seq_len
    else:
        args.model.max_seqlen = args.data.seq_len
    if d.tp_size > 1:
        logger.warning("Tensor parallelism is less exercised than the data-parallel path")
    assert args.probe_freq != args.profiling.mem_steps, "Don't profile during probe step"
    assert args.probe_freq != args.profiling.profile_steps, "Don't profile during probe step"
    if args.logging.wandb is not None:
        args.logging.wandb.name = args.name
    if args.probe_freq is not None:
        assert d.tp_size == 1, "Probing not supported with tensor parallelism"
        assert d.selective_activation_checkpointing is False, "Probing not supported with selective activation checkpointing"


def run_training(args: TrainArgs, spec: ModelSpec) -> Dict[str, Any]:
    """Runs the job described by ``args``; returns the last logged metrics (handy in tests)."""
    last_metrics: Dict[str, Any] = {}
    with ExitStack() as stack:
        tokenizer = build_tokenizer(args.data.tokenizer.name, args.data.tokenizer.path)
        validate_train_args(args, tokenizer.n_words)
        if get_is_master():
            os.makedirs(args.dump_dir, exist_ok=True)
            dump_config(args, Path(args.dump_dir) / "config.yaml")
        init_logger(Path(args.dump_dir) / "train.log")
        init_signal_handler(set_preemption_flag)
        setup_env(args.env)
        setup_torch_distributed(args.distributed)
        mesh = get_device_mesh(args.distributed)
        logger.info(f"Starting job: {args.name}")
        dp_rank, dp_degree = mesh.local_rank("dp"), mesh.size("dp")
        logger.info(f"Running on dp rank : {dp_rank}")
        logger.info(f"Running on dp size : {dp_degree}")
        on_gpu = torch.cuda.is_available()
        device = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")

        torch.manual_seed(args.seed)
        logger.info("Building model")
        with torch.device("meta"):
            model = spec.model_cls(args.model)
        logger.info("Model is built !")
        model_param_count = get_num_params(model)
        plan = spec.build_plan(args.model) if spec.build_plan else None
        model, engine = parallelize_model(model, mesh, args.model, args.distributed, fsdp_grouping_plan=plan,
                                          tp_parallelize=spec.tp_parallelize, optim=build_engine_optim(args.optim),
                                          device=device, grad_acc_steps=args.grad_acc_steps)
        logger.info(f"Gradient / parameter collectives of the sharded engine: {engine.collective_path}")
        with torch.random.fork_rng(devices=[device] if on_gpu else []):
            torch.manual_seed(args.model.seed)
            engine.init_weights_fp32(model.init_weights)
        if args.checkpoint.init_ckpt_path:
            logger.info(f"Loading initial model from {args.checkpoint.init_ckpt_path}")
            load_from_checkpoint(args.checkpoint.init_ckpt_path, engine, model_key="model")
        check_model_value_range(model, range=10.0, std=1.0)
        logger.info(f"Model size: {model_param_count:,} total parameters")
        gpu_memory_monitor = GPUMemoryMonitor("cuda" if on_gpu else "cpu")
        logger.info(f"GPU capacity: {gpu_memory_monitor.device_name} ({gpu_memory_monitor.device_index}) "
                    f"with {gpu_memory_monitor.device_capacity_gib:.2f}GiB memory")

        scheduler = LRScheduler(args.optim.lr, build_lr_fn(args.optim, args.steps))
        data_loader_state = init_dataloader_state_from_args(args.data, dp_rank, dp_degree, args.model.vocab_size)
        train_state = TrainState(step=0, acc_step=0, scheduler=scheduler, data_loader_state=data_loader_state)
        checkpoint = CheckpointManager.instantiate_and_make_dir(args.checkpoint)
        checkpoint.load(engine, train_state, mesh)
        model.loss_grad_scale = 1.0 / args.grad_acc_steps

        probe = None
        if args.probe_freq is not None:
            from .probe import AutoProbeD

            if get_is_master():
                os.makedirs(Path(args.dump_dir) / "probe", exist_ok=True)
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.barrier()
            probe = AutoProbeD(model, Path(args.dump_dir) / "probe" / f"probe.{dp_rank}.jsonl"
                               if dp_rank % 128 == 0 else None)

        gc.disable()
        model.train()
        metric_logger = stack.enter_context(MetricLogger(Path(args.dump_dir) / "metrics.jsonl", args))
        data_loader = stack.enter_context(build_dataloader_from_args(args.data, state=train_state.data_loader_state))
        profiler = stack.enter_context(maybe_run_profiler(args.dump_dir, model, args.profiling))

        flops_per_token = spec.flops_per_token(model_param_count, args.model, args.data.seq_len) \
            if spec.flops_per_token else 0.0
        peak = peak_flops(args.distributed.model_dtype)
        nwords_since_last_log = 0
        time_last_log = timer()
        gc.collect()
        saved = False
        grad_norm = torch.zeros(())
        pinned = None
        while train_state.step < args.steps:
            train_state.acc_step = (train_state.acc_step + 1) % args.grad_acc_steps
            curr_lr = scheduler.get_lr()
            data_load_start = timer()
            batch, train_state.data_loader_state = next(data_loader)
            batch = torch.from_numpy(np.ascontiguousarray(batch)).long()
            if every_n_steps(train_state, args.gc_collect_freq, acc_step=0):
                logger.info("garbage collection")
                gc.collect()  # every rank collects on the same step so that nobody straggles
            if on_gpu:
                if pinned is None or pinned.shape != batch.shape:
                    pinned = torch.empty(batch.shape, dtype=batch.dtype).pin_memory()
                pinned.copy_(batch)
                batch = pinned.to(device, non_blocking=True)
            input_ids = batch[:, :, 0].contiguous()
            labels = spec.labels_from_batch(batch).contiguous()
            data_load_time = round(timer() - data_load_start, 4)
            nwords_since_last_log += input_ids.numel()
            bsz, seqlen = input_ids.shape
            start_timer = torch.cuda.Event(enable_timing=True) if on_gpu else None
            end_timer = torch.cuda.Event(enable_timing=True) if on_gpu else None
            t_start = timer()
            if on_gpu:
                start_timer.record()

            if probe is not None and every_n_steps(train_state, args.probe_freq, acc_step=1 % args.grad_acc_steps):
                # Half-batch forward + backward under the probe; its gradients are discarded.
                engine.zero_grad()
                with probe:
                    probe.metadata = {"it": train_state.step, "global_step": train_state.step, "loop": "lingua"}
                    saved_scale, model.loss_grad_scale = model.loss_grad_scale, None
                    engine.defer_reduce = True  # these gradients are thrown away: no reduction
                    out = spec.loss_fn(model, input_ids[: max(1, bsz // 2)], labels[: max(1, bsz // 2)])
                    (out[0] if isinstance(out, tuple) else out).backward()
                    model.loss_grad_scale = saved_scale
                engine.zero_grad()

            if train_state.acc_step == (1 % args.grad_acc_steps) or args.grad_acc_steps == 1:
                engine.zero_grad()
            engine.defer_reduce = train_state.acc_step != 0  # reduce only after the last micro-batch
            with nvtx_range("forward"):
                out = spec.loss_fn(model, input_ids, labels)
            loss, extra_losses = out if isinstance(out, tuple) else (out, {})
            with nvtx_range("backward"):
                (loss / args.grad_acc_steps if args.grad_acc_steps > 1 else loss).backward()
            loss = loss.detach() * 1.0

            if train_state.acc_step == 0:
                with nvtx_range("optimizer"):
                    grad_norm = engine.step(curr_lr)
                scheduler.step()
                train_state.step += 1
            if on_gpu:
                end_timer.record()
                torch.cuda.synchronize()
                # a kernel whose bounded wait ran out (a peer that never arrived at a barrier, a copy that never
                # landed) has left a code in the status word: stop here instead of training on partial data
                kernel_lib.check_status()
                curr_iter_time = round(start_timer.elapsed_time(end_timer) * 1e-3, 4)
            else:
                curr_iter_time = round(timer() - t_start, 4)
            if profiler is not None:
                profiler.step()

            if every_n_steps(train_state, args.logging.freq, acc_step=None if args.logging.acc_freq else 0,
                             acc_freq=args.logging.acc_freq):
                time_delta = timer() - time_last_log
                wps = nwords_since_last_log / (time_delta * args.distributed.tp_size)
                mem = gpu_memory_monitor.get_peak_stats()
                total_acc_steps = args.grad_acc_steps * train_state.step + train_state.acc_step
                total_tokens = dp_degree * total_acc_steps * args.data.batch_size * args.data.seq_len
                FLOPS = flops_per_token * wps
                metrics = flatten_dict({
                    "global_step": train_state.step, "acc_step": train_state.acc_step,
                    "speed": {"wps": wps, "FLOPS": FLOPS, "mfu": FLOPS / peak, "curr_iter_time": curr_iter_time,
                              "data_load_time": data_load_time},
                    "optim": {"grad_norm": float(grad_norm), "lr": curr_lr, "total_tokens": total_tokens},
                    "memory": mem._asdict(),
                }, sep="/")
                to_sync = {"loss/out": float(loss)}
                to_sync.update({(k if "/" in k else f"loss/{k}"): float(v) for k, v in extra_losses.items()})
                metrics.update(dist_mean_dict(to_sync))
                if get_is_master():
                    metric_logger.log(metrics)
                last_metrics = dict(metrics)
                gpu_memory_monitor.reset_peak_stats()
                nwords_since_last_log = 0
                time_last_log = timer()
                logger.info(f"step: {train_state.step}  acc: {train_state.acc_step}  loss: {round(float(loss), 4):>7}"
                            f"  grad: {float(grad_norm):.2e}  flops: {FLOPS:.2e}  wps: {wps:.2e}"
                            f"  iter: {curr_iter_time:>7}  data: {data_load_time:>5}  lr: {curr_lr:.2e}"
                            f"  mem: {mem.max_active_pct:.0f}%  pow: {mem.power_draw / 1000} W")

            saved = False
            if every_n_steps(train_state, args.checkpoint.dump.every, acc_step=0) or \
                    every_n_steps(train_state, args.checkpoint.eval.every, acc_step=0):
                saved = checkpoint.save(engine, train_state, args, mesh=mesh, lr=curr_lr)

            if args.eval is not None and (every_n_steps(train_state, args.checkpoint.eval.every, acc_step=0)
                                          or every_n_steps(train_state, args.steps, acc_step=0)):
                _run_eval(args, spec, train_state, checkpoint)

            if preemption_flag["flag"]:
                if not saved:
                    checkpoint.save(engine, train_state, args, mesh=mesh, lr=curr_lr)
                if "SLURM_JOB_ID" in os.environ:
                    requeue_slurm_job()
                sys.exit(0)

        if not saved:
            checkpoint.save(engine, train_state, args, mesh=mesh, lr=scheduler.get_lr())
        gc.collect()
    gc.enable()
    return last_metrics


def _run_eval(args: TrainArgs, spec: ModelSpec, train_state: TrainState, checkpoint: CheckpointManager) -> None:
    import importlib

    ev = importlib.import_module(spec.eval_module)
    eval_args = dataclass_from_dict(ev.EvalArgs, args.eval)
    eval_args.global_step = train_state.step
    eval_args.ckpt_dir = str(checkpoint.existing_saves[-1])
    eval_args.dump_dir = os.path.join(args.dump_dir, "evals", ev.EVAL_FOLDER_NAME.format(train_state.step))
    eval_args.metric_log_dir = args.dump_dir
    if args.async_eval_gpus is None:
        ev.launch_eval(eval_args)
    elif get_is_master():
        from .stool import StoolArgs, launch_job

        if args.logging.wandb is not None:
            eval_args.wandb = deepcopy(args.logging.wandb)
        assert args.async_eval_gpus > 0
        logger.info(f"Launching evals on {args.async_eval_gpus} gpus")
        with clean_env():
            launch_job(StoolArgs(asdict(eval_args), script=spec.eval_module, copy_code=False,
                                 nodes=max(1, args.async_eval_gpus // 8), qos="lowest"))


def main_from_cli(args_cls, spec_fn: Callable[[Any], ModelSpec], argv: Optional[List[str]] = None):
    """``python -m apps.<app>.train config=<yaml> a.b=c``: defaults <- yaml <- command line."""
    from .config import config_from_cli

    cfg = config_from_cli(args_cls, argv)
    return run_training(cfg, spec_fn(cfg))
