"""Process-group runtime: rank discovery, environment, device mesh, model parallelisation.

Covers lingua/distributed.py: DistributedArgs :57, EnvironmentArgs :82, get_device_mesh :97,
dist_max/mean/mean_dict :123-140, rank / address helpers :143-208, setup_env :211,
setup_torch_distributed :238, check_model_value_range :312, init_signal_handler :349,
requeue_slurm_job :357, clean_env :369, parallelize_model :394. Differences by design:
the backend is NCCL on GPUs and gloo on CPU (the reference has no CPU path), and
``parallelize_model`` builds this library's sharded-parameter engine instead of wrapping
modules in FSDP2.
"""
from __future__ import annotations

import atexit
import contextlib
import logging
import multiprocessing as mp
import os
import random
import shutil
import signal
import socket
import subprocess
import sys
import tempfile
from dataclasses import asdict, dataclass
from functools import lru_cache
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

logger = logging.getLogger()


@dataclass
class DistributedArgs:
    dp_shard: int = 1  # ranks that share one copy of the sharded state
    dp_replicate: int = 1  # replicas of that group (outer data-parallel dim)
    tp_size: int = 1
    fused_tp_forward: bool = True  # no-grad TP passes use the fused all-gather / reduce-scatter GEMMs
    # TP training keeps the residual stream sharded by rows inside a TP group and runs its all-gathers and
    # reduce-scatters inside the GEMM kernels (parallel/tp_train.py); off: all-reduce formulation
    tp_sequence_parallel: bool = True
    p2p_param_gather: bool = True  # parameter all-gather by NVLink copy engines instead of NCCL kernels
    selective_activation_checkpointing: bool = False
    compile: bool = False
    fsdp_type: str = "no_shard"
    model_dtype: str = "bf16"
    float8_recipe: Optional[str] = None
    float8_filter: str = r"layers\.[0-9]+\."
    matmul_allow_tf32: bool = False
    allow_bf16_reduced_precision_reduction = True
    detect_anomaly: bool = False
    compile_cache_size_limit: int = 8
    spawn_method: str = "forkserver"


@dataclass
class EnvironmentArgs:
    MKL_SERVICE_FORCE_INTEL: str = "GNU"
    OMP_NUM_THREADS: str = "1"
    MKL_NUM_THREADS: str = "1"
    # The reference sets this to "1" (PyTorch's own intra-node all-reduce). Off here: the engine has its own
    # peer-memory collectives, and with PyTorch 2.11 the option makes the NCCL process group fail to initialise
    # ("Could not resolve the process group registered under the name IntraNodeComm0").
    ENABLE_INTRA_NODE_COMM: str = "0"
    TORCH_NCCL_AVOID_RECORD_STREAMS: str = "1"
    NCCL_IB_TIMEOUT: str = "22"
    NCCL_DEBUG: str = "INFO"
    TORCH_NCCL_ASYNC_ERROR_HANDLING: str = "1"


# ----------------------------------------------------------------------------- rank discovery
@lru_cache()
def get_is_torch_run() -> bool:
    return os.environ.get("LOCAL_RANK") is not None


@lru_cache()
def get_is_slurm_job() -> bool:
    return "SLURM_JOB_ID" in os.environ and not get_is_torch_run()


@lru_cache()
def get_global_rank() -> int:
    if get_is_torch_run():
        return int(os.environ["RANK"])
    if get_is_slurm_job():
        return int(os.environ["SLURM_PROCID"])
    return 0


@lru_cache()
def get_local_rank() -> int:
    if get_is_torch_run():
        return int(os.environ["LOCAL_RANK"])
    if get_is_slurm_job():
        return int(os.environ["SLURM_LOCALID"])
    return 0


@lru_cache()
def get_world_size() -> int:
    if get_is_torch_run():
        return int(os.environ["WORLD_SIZE"])
    if get_is_slurm_job():
        return int(os.environ["SLURM_NTASKS"])
    return 1


@lru_cache()
def get_is_master() -> bool:
    return get_global_rank() == 0


@lru_cache()
def get_master_port(job_id: int) -> int:
    if get_is_torch_run():
        return int(os.environ["MASTER_PORT"])
    return random.Random(job_id).randint(20000, 60000)


@lru_cache()
def get_master_addr() -> str:
    if get_is_torch_run():
        return os.environ["MASTER_ADDR"]
    if get_is_slurm_job():
        hosts = subprocess.check_output(["scontrol", "show", "hostnames", os.environ["SLURM_JOB_NODELIST"]])
        return hosts.split()[0].decode("utf-8")
    return "127.0.0.1"


# ----------------------------------------------------------------------------- environment
def setup_env(env_args: EnvironmentArgs) -> None:
    env_vars = asdict(env_args)
    # a per-job scratch dir on SLURM keeps node-local /tmp from filling up
    if get_is_slurm_job():
        triton = tempfile.mkdtemp()
        tmp = f"/scratch/slurm_tmpdir/{os.environ['SLURM_JOB_ID']}"
        atexit.register(shutil.rmtree, triton, ignore_errors=True)
        env_vars["TRITON_CACHE_DIR"] = triton
        if os.path.isdir(tmp):
            env_vars["TMP_DIR"] = tmp
    for name, value in env_vars.items():
        if os.environ.get(name) != str(value):
            os.environ[name] = str(value)
            logger.warning(f"WARNING: Setting {name} to {value}")


def setup_torch_distributed(dist_args: DistributedArgs, device: Optional[str] = None) -> None:
    """Initialise the default process group from torchrun / SLURM / single-process context.
    NCCL on CUDA, gloo on CPU."""
    mp.set_start_method(dist_args.spawn_method, force=True)
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    local_rank = get_local_rank()
    os.environ["RANK"] = str(get_global_rank())
    os.environ["WORLD_SIZE"] = str(get_world_size())
    os.environ["MASTER_ADDR"] = get_master_addr()
    os.environ["MASTER_PORT"] = str(get_master_port(job_id=int(os.environ.get("SLURM_JOB_ID", -1))))
    if device == "cuda":
        if get_is_torch_run():
            logger.info(f"Run launched with torchrun, local rank: {local_rank}")
        elif get_is_slurm_job():
            logger.info(f"Run launched with slurm, local rank: {local_rank}")
        else:
            logger.info("Single GPU job")
        logger.info(f"ENV: {os.environ}")
        assert 0 <= local_rank < max(torch.cuda.device_count(), 8)
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
    if not dist.is_initialized():
        dist.init_process_group(init_method="env://", backend="nccl" if device == "cuda" else "gloo")
    torch.autograd.set_detect_anomaly(dist_args.detect_anomaly)


class Mesh:
    """3-D rank grid (dp_replicate, dp_shard, tp), tp fastest, with one process group per axis
    and one over dp_replicate x dp_shard."""

    def __init__(self, dp_replicate: int, dp_shard: int, tp: int):
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        assert dp_replicate * dp_shard * tp == world, (
            f"dp_replicate * dp_shard * tp_size ({dp_replicate} * {dp_shard} * {tp}) != world_size ({world})")
        self.shape = {"dp_replicate": dp_replicate, "dp_shard": dp_shard, "tp": tp}
        self.rank = rank
        self.coord = {"dp_replicate": rank // (dp_shard * tp), "dp_shard": (rank // tp) % dp_shard, "tp": rank % tp}
        self.groups: Dict[str, Optional[dist.ProcessGroup]] = {}
        if world == 1:
            self.groups = {k: None for k in ("dp_replicate", "dp_shard", "tp", "dp")}
            return
        grid = torch.arange(world).view(dp_replicate, dp_shard, tp)
        for name, dim in (("dp_replicate", 0), ("dp_shard", 1), ("tp", 2)):
            mine = None
            lines = grid.movedim(dim, -1).reshape(-1, grid.shape[dim])
            for ranks in lines.tolist():
                g = dist.new_group(ranks) if len(ranks) > 1 else None
                if rank in ranks:
                    mine = g
            self.groups[name] = mine
        mine = None
        for t in range(tp):
            ranks = grid[:, :, t].reshape(-1).tolist()
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                mine = g
        self.groups["dp"] = mine

    def size(self, name: str) -> int:
        if name == "dp":
            return self.shape["dp_replicate"] * self.shape["dp_shard"]
        return self.shape[name]

    def local_rank(self, name: str) -> int:
        if name == "dp":
            return self.coord["dp_replicate"] * self.shape["dp_shard"] + self.coord["dp_shard"]
        return self.coord[name]

    def group(self, name: str):
        return self.groups[name]


def get_device_mesh(dist_args: DistributedArgs) -> Mesh:
    return Mesh(dist_args.dp_replicate, dist_args.dp_shard, dist_args.tp_size)


# ----------------------------------------------------------------------------- small collectives
def _dev():
    return "cuda" if (torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl") else "cpu"


def dist_max(x: Union[int, float], group=None):
    t = torch.tensor(x, device=_dev())
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t


def dist_mean(x: Union[int, float], group=None):
    t = torch.tensor(float(x), device=_dev())
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        t /= dist.get_world_size(group)
    return t


def dist_mean_dict(x: Dict[str, float]) -> Dict[str, float]:
    keys = sorted(x)
    t = torch.tensor([float(x[k]) for k in keys], device=_dev())
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t /= dist.get_world_size()
    return {k: v for k, v in zip(keys, t.tolist())}


# ----------------------------------------------------------------------------- module helpers
def get_module(module, access_string):
    for name in access_string.split(sep="."):
        module = getattr(module, name)
    return module


def set_module(module, access_string, value):
    names = access_string.split(sep=".")
    setattr(get_module(module, ".".join(names[:-1])) if len(names) > 1 else module, names[-1], value)


def default_fsdp_grouping_plan(n_layers: int) -> List[Tuple[str, bool]]:
    return [(f"layers.{i}", i < n_layers - 1) for i in range(n_layers)]


@torch.no_grad()
def check_model_value_range(model: torch.nn.Module, range: float = 1e3, std: float = 1e3) -> None:
    """Warn about NaN / Inf / out-of-range / degenerate parameters right after initialisation."""
    for name, param in model.named_parameters():
        p = param.float()
        if p.numel() == 0:
            logger.warning(f"Model parameter {name} is empty, probably because of FSDP sharding")
            continue
        if torch.isnan(p).any() or torch.isinf(p).any():
            logger.warning(f"Model parameter {name} contains NaN or Inf")
        pmax, pmin = p.max().item(), p.min().item()
        if pmax > range or pmin < -range:
            logger.warning(f"Model parameter {name} has a suspiciously large range ({pmin}, {pmax}): please check initialization")
        pstd = p.std().item() if p.numel() > 1 else 0.0
        if pstd > std:
            logger.warning(f"Model parameter {name} has a suspiciously large standard deviation ({pstd}): please check initialization")
        if (p == 0).all():
            logger.warning(f"Model parameter {name} is all zeros: it might be because of a missing initialization")


def init_signal_handler(callable):
    """SIGUSR2 is what the batch scheduler sends shortly before preempting the job."""
    signal.signal(signal.SIGUSR2, callable)
    logger.warning("Signal handler installed.")


def requeue_slurm_job():
    prod_id = int(os.environ["SLURM_PROCID"])
    logger.warning("Host: %s - Global rank: %i" % (socket.gethostname(), prod_id))
    if prod_id == 0 and os.environ.get("LAUNCH_WITH", "") != "DORA":
        logger.warning("Requeuing job " + os.environ["SLURM_JOB_ID"])
        os.system("scontrol requeue " + os.environ["SLURM_JOB_ID"])
    else:
        logger.warning("Not the master process, no need to requeue.")
    sys.exit(0)


@contextlib.contextmanager
def clean_env():
    """Temporarily hide scheduler / launcher variables so that a child job starts from a clean slate."""
    distrib_names = ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE",
                     "TORCHELASTIC_RUN_ID", "DORA_FORCE_DISTRIB")
    cluster_env = {x: os.environ.pop(x) for x in list(os.environ)
                   if x.startswith(("SLURM_", "SLURMD_", "SRUN_", "SBATCH_", "SUBMITIT_", "WANDB_")) or x in distrib_names}
    try:
        yield
    finally:
        os.environ.update(cluster_env)


DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def parallelize_model(model, mesh: Mesh, model_args, distributed_args: DistributedArgs, fsdp_grouping_plan=None,
                      tp_parallelize=None, no_recompute_ops=None, optim=None, device=None, grad_acc_steps: int = 1):
    """Shard ``model`` over the mesh's data-parallel axis and return (model, engine).

    ``fsdp_type``: ``full_shard`` shards parameters, gradients and optimiser state over dp_shard;
    ``no_shard`` keeps whole copies (a dp_shard of 1). ``compile`` and
    ``selective_activation_checkpointing`` are accepted for config compatibility: the native ops
    are already fused and fix their own save / recompute set."""
    from .parallel.engine import ShardedEngine

    if distributed_args.float8_recipe is not None:
        from .float8 import convert_linears_to_fp8

        convert_linears_to_fp8(model, distributed_args.float8_recipe, distributed_args.float8_filter)
    if distributed_args.tp_size > 1:
        assert distributed_args.fsdp_type == "full_shard", "Only full shard is supported for TP parallelism"
        assert tp_parallelize is not None, "TP plan is required for TP parallelism"
        tp_parallelize(model, mesh, model_args, distributed_args)
    if fsdp_grouping_plan is None:
        fsdp_grouping_plan = default_fsdp_grouping_plan(len(model.layers))
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    dtype = DTYPES[distributed_args.model_dtype] if device.type == "cuda" else torch.float32
    assert distributed_args.fsdp_type in ("full_shard", "no_shard")
    # parameters, gradients and optimiser state are sharded over the dp_shard axis; the dp_replicate axis holds
    # copies whose reduced gradients are averaged (hybrid sharding, lingua/distributed.py:106-113,441-446). With
    # ``no_shard`` every data-parallel rank is a replica.
    if distributed_args.fsdp_type == "no_shard":
        shard_pg, rep_pg = False, (mesh.group("dp") if mesh.size("dp") > 1 else None)
    else:
        shard_pg = mesh.group("dp_shard") if mesh.size("dp_shard") > 1 else False
        rep_pg = mesh.group("dp_replicate") if mesh.size("dp_replicate") > 1 else None
    engine = ShardedEngine(model, fsdp_grouping_plan, process_group=shard_pg, replicate_group=rep_pg,
                           tp_group=mesh.group("tp") if mesh.size("tp") > 1 else None, compute_dtype=dtype,
                           optim=optim, device=device, p2p_gather=distributed_args.p2p_param_gather,
                           accumulate=grad_acc_steps > 1)
    for buf_owner in model.modules():
        for name, buf in list(buf_owner._buffers.items()):
            if buf is not None and buf.device.type == "meta":
                buf_owner._buffers[name] = torch.empty_like(buf, device=device)
            elif buf is not None and buf.device != device:
                buf_owner._buffers[name] = buf.to(device)
    model._engine = engine
    # selective activation checkpointing on = recompute the cheap activations in backward
    from .ops import fused

    fused.set_recompute(distributed_args.selective_activation_checkpointing)
    if distributed_args.tp_size > 1 and distributed_args.tp_sequence_parallel and device.type == "cuda" \
            and hasattr(model, "tok_embeddings") and dtype == torch.bfloat16:
        # training with a row-sharded residual stream and the TP collectives inside the GEMM kernels
        from .parallel.tp_train import enable_sp_training

        if enable_sp_training(model, mesh.group("tp"), device):
            engine.tp_partial = True  # replicated weights see one rank's rows only: their gradients are summed
    if distributed_args.tp_size > 1 and distributed_args.fused_tp_forward and device.type == "cuda" \
            and hasattr(model, "tok_embeddings"):
        # evaluation / scoring passes run with the TP collectives inside the GEMM kernels
        from .parallel.tp_fused import enable_fused_tp_forward

        enable_fused_tp_forward(model, mesh.group("tp"), device)
    return model, engine
