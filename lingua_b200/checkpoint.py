"""Sharded (torch.distributed.checkpoint) and consolidated checkpoints.

On-disk layout and retention rules are those of lingua/checkpoint.py (constants :37-47,
SaveEvery :51, CheckpointArgs :57, consolidate_checkpoints :69, load_from_checkpoint :90,
CheckpointManager :104): ``checkpoints/{step:010d}/`` holds the DCP files of
``{"model": {fqn: tensor}, "optim": {"state": {fqn: {step, exp_avg, exp_avg_sq}},
"param_groups": [...]}}``, ``params.json`` (the full training config) and one
``train_state_{dp_rank:05d}.json`` per data-parallel rank; ``consolidated/consolidated.pth`` is
the single-file form used by generation and evaluation.

The sharded engine keeps flat per-group slices that cut through parameters, so for the
checkpoint every parameter (fp32 master weights and both Adam moments) is re-presented as a
``DTensor`` sharded on dim 0 over the data-parallel group - the form FSDP2 checkpoints have -
which also lets a checkpoint be loaded on a different number of GPUs.
"""
from __future__ import annotations

import json
import logging
import os
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.api import CheckpointException  # derives from BaseException
from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

from .config import dataclass_to_dict
from .distributed import get_is_master

logger = logging.getLogger("CHECKPOINT")

FOLDER_NAME = "{:010d}"
RE_FOLDER = r"\d{10}"
RE_CKPT = r"__\d_\d\.distcp"
CONSOLIDATE_FOLDER = "consolidated"
CONSOLIDATE_NAME = "consolidated.pth"
CONFIG_NAME = "params.json"
TRAIN_STATE_NAME = "train_state_{:05d}.json"
RE_DIGITS = re.compile(r"\d+")


@dataclass
class SaveEvery:
    every: int = 1000
    keep: int = 0


@dataclass
class CheckpointArgs:
    dump: SaveEvery = field(default_factory=SaveEvery)
    eval: SaveEvery = field(default_factory=SaveEvery)
    path: Optional[str] = None
    init_ckpt_path: Optional[str] = None
    continue_training_from_init: bool = False


def _get_key_step(name: str) -> int:
    return int(re.findall(RE_DIGITS, name)[-1])


def _barrier() -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def consolidate_checkpoints(ckpt_dir: str) -> Path:
    """Merge a sharded checkpoint into ``<ckpt_dir>/consolidated/consolidated.pth`` (+ params.json)."""
    out = Path(ckpt_dir) / CONSOLIDATE_FOLDER
    if not (out / CONSOLIDATE_NAME).exists():
        out.mkdir(exist_ok=True)
        logger.info(f"Consolidating to: {out}")
        dcp_to_torch_save(ckpt_dir, str(out / CONSOLIDATE_NAME))
        (out / CONFIG_NAME).write_text((Path(ckpt_dir) / CONFIG_NAME).read_text())
        logger.info("Consolidated !")
    return out


# ----------------------------------------------------------------------------- engine <-> state dict
def _row_range(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    per = (n_rows + world - 1) // world
    return min(n_rows, rank * per), min(n_rows, (rank + 1) * per)


def _device_mesh(engine):
    from torch.distributed.device_mesh import DeviceMesh

    if getattr(engine, "_dcp_mesh", None) is None:
        engine._dcp_mesh = DeviceMesh.from_group(engine.pg if engine.pg not in (None, False) else dist.group.WORLD,
                                                 engine.device.type, mesh_dim_names=("dp_shard",))
    return engine._dcp_mesh


def _tp_info(engine, fqn: str):
    """(dim, degree, rank) of the tensor-parallel split of parameter ``fqn``, or None."""
    owner, _, attr = fqn.rpartition(".")
    try:
        mod = engine.model.get_submodule(owner)
    except AttributeError:
        return None
    info = getattr(mod, "tp_shard", None)
    return info if (info is not None and attr == "weight") else None


def _as_checkpoint_tensor(engine, fqn: str, p, full: torch.Tensor):
    """``full`` holds this process's whole fp32 tensor of one parameter (its tensor-parallel slice when TP is on).
    Returns what goes into the state dict under ``fqn``: always a description of the *unsplit* parameter, so that
    every TP rank writes the same values under the same key and a checkpoint loads on any layout. Tensor-parallel
    slices are first all-gathered over the TP group along their split dim; with more than one data-parallel rank
    the result is a DTensor sharded on dim 0 over the shard group (torch.chunk sizes, the form FSDP2 checkpoints of
    the reference have), else the plain tensor."""
    from torch.distributed.tensor import DTensor, Shard

    tp = _tp_info(engine, fqn) if engine.tp_pg is not None else None
    if tp is not None:
        dim, degree, _ = tp
        parts = [torch.empty_like(full) for _ in range(degree)]
        dist.all_gather(parts, full.contiguous(), group=engine.tp_pg)
        full = torch.cat(parts, dim=dim)
    W, R = engine.world, engine.rank
    if W == 1:
        return full
    r0, r1 = _row_range(full.shape[0], W, R)
    local = full[r0:r1].clone()
    return DTensor.from_local(local, _device_mesh(engine), [Shard(0)], run_check=False, shape=full.shape,
                              stride=_contig_stride(list(full.shape)))


def _contig_stride(shape):
    st, acc = [], 1
    for d in reversed(shape):
        st.append(acc)
        acc *= d
    return tuple(reversed(st))


def engine_state_dict(engine, lr: float = 0.0) -> Dict[str, Any]:
    """``{"model": ..., "optim": ...}`` with the reference's keys; tensors are plain (one rank) or
    dim-0 sharded DTensors holding this rank's rows."""
    from torch.distributed.tensor import DTensor, Shard

    W, R = engine.world, engine.rank
    model_sd: Dict[str, Any] = {}
    opt_state: Dict[str, Any] = {}
    names: List[str] = []
    step_t = torch.tensor(float(engine.step_count))
    for gi, g in enumerate(engine.groups):
        # every rank assembles the group's fp32 tensors in parameter order and keeps its dim-0 chunk of each
        # parameter: the engine's own shards are row slabs of uneven size, a DTensor wants torch.chunk sizes
        bufs = {key: engine.export_group_fp32(gi, which)
                for key, which in (("p", "master"), ("m", "exp_avg"), ("v", "exp_avg_sq"))}
        for fqn, p in g.params:
            o, n = g.offsets[fqn]
            names.append(fqn)
            out = {}
            for key in ("p", "m", "v"):
                full = bufs[key][o:o + n].view(p.shape)
                out[key] = _as_checkpoint_tensor(engine, fqn, p, full)
            model_sd[fqn] = out["p"]
            opt_state[fqn] = {"step": step_t.clone(), "exp_avg": out["m"], "exp_avg_sq": out["v"]}
        del bufs
    o = engine.optim
    group = {"lr": lr, "betas": (o.beta1, o.beta2), "eps": o.eps, "weight_decay": o.weight_decay, "amsgrad": False,
             "maximize": False, "foreach": None, "capturable": False, "differentiable": False, "fused": True,
             "initial_lr": lr, "params": names}
    return {"model": model_sd, "optim": {"state": opt_state, "param_groups": [group]}}


def load_engine_state_dict(engine, sd: Dict[str, Any], load_optim: bool = True) -> None:
    """Scatter a (loaded) state dict of the above form back into the engine's shards."""
    from torch.distributed.tensor import DTensor

    def local_of(fqn, t):
        t = (t.full_tensor() if isinstance(t, DTensor) else t).to(device=engine.device, dtype=torch.float32)
        tp = _tp_info(engine, fqn) if engine.tp_pg is not None else None
        if tp is not None:
            t = t.chunk(tp[1], dim=tp[0])[tp[2]]
        return t

    keys = [("master", lambda f: sd["model"][f])]
    if load_optim and "optim" in sd:
        keys += [("exp_avg", lambda f: sd["optim"]["state"][f]["exp_avg"]),
                 ("exp_avg_sq", lambda f: sd["optim"]["state"][f]["exp_avg_sq"])]
    for gi, g in enumerate(engine.groups):
        buf = torch.zeros(g.padded, dtype=torch.float32, device=engine.device)
        for which, get in keys:
            buf.zero_()
            for fqn, p in g.params:
                o, n = g.offsets[fqn]
                buf[o:o + n].copy_(local_of(fqn, get(fqn)).reshape(-1))
            engine.load_group_fp32(gi, buf, which)
        del buf
    if load_optim and "optim" in sd:
        steps = [float(v["step"]) for v in sd["optim"]["state"].values()]
        if steps:
            engine.step_count = int(max(steps))


def load_from_checkpoint(ckpt_dir: str, engine, model_key: str = "model", load_optim: bool = False) -> None:
    """Fill the engine (weights, optionally optimiser state) from a sharded checkpoint directory."""
    if not (Path(ckpt_dir) / ".metadata").exists():
        raise ValueError("Please convert the checkpoint to distcp format using "
                         "`torch.distributed.checkpoint.format_utils.torch_save_to_dcp` before loading it")
    sd = engine_state_dict(engine)
    # model_key "" means the directory stores the parameters at top level (a bare model checkpoint)
    to_load: Dict[str, Any] = {model_key: sd["model"]} if model_key else dict(sd["model"])
    if load_optim:
        to_load["optim"] = sd["optim"]
    dcp.load(to_load, checkpoint_id=ckpt_dir)
    load_engine_state_dict(engine, sd, load_optim=load_optim)


# ----------------------------------------------------------------------------- manager
class CheckpointManager:
    def __init__(self, args: CheckpointArgs):
        self.path = args.path
        self.dump_every = args.dump
        self.eval_every = args.eval
        self.init_ckpt_path = args.init_ckpt_path
        self.continue_training_from_init = args.continue_training_from_init
        assert os.path.exists(self.path), (
            f"Path {self.path} does not exist and needs to be created before using CheckpointManager "
            f"(use instantiate_and_make_dir)")
        self.existing_saves = self.get_existing_saves()

    def get_existing_saves(self) -> List[Path]:
        folders = [p for p in Path(self.path).iterdir() if p.is_dir() and re.match(RE_FOLDER, p.name)]
        folders.sort(key=lambda p: _get_key_step(p.name))
        return folders

    def clean_up(self) -> None:
        """Keep the last ``keep`` folders of each kind (all of them when keep <= 0); a folder that is
        neither a dump nor an eval step (e.g. a preemption save) is always kept."""
        logger.info("Cleaning up checkpoints...")
        dumps, evals, others = [], [], []
        for p in self.existing_saves:
            step = _get_key_step(p.name)
            is_dump = step % self.dump_every.every == 0
            is_eval = step % self.eval_every.every == 0
            if is_dump:
                dumps.append(p)
            if is_eval:
                evals.append(p)
            if not (is_dump or is_eval):
                others.append(p)
        if self.dump_every.keep > 0:
            dumps = dumps[-self.dump_every.keep:]
        if self.eval_every.keep > 0:
            evals = evals[-self.eval_every.keep:]
        keep = set(others + dumps + evals)
        remove = set(self.existing_saves) - keep
        logger.info(f"Removing folders: {remove}")
        if get_is_master():
            for folder in remove:
                for f in folder.iterdir():
                    if f.is_file():
                        f.unlink()
                    elif f.is_dir():
                        assert f.name in [CONSOLIDATE_FOLDER]
                        for ff in f.iterdir():
                            ff.unlink()
                        f.rmdir()
                folder.rmdir()
        _barrier()
        self.existing_saves = sorted(keep, key=lambda p: _get_key_step(p.name))

    def get_last_step_path(self, dp_rank: int = 0) -> Optional[Path]:
        for p in reversed(self.existing_saves):
            if (p / TRAIN_STATE_NAME.format(dp_rank)).is_file():
                return p
        return None

    def _create_folder(self, base_path: Path, folder_name: str) -> Path:
        folder = base_path / folder_name
        if get_is_master():
            folder.mkdir(parents=False, exist_ok=True)
        _barrier()
        return folder

    @staticmethod
    def _get_dp_tp_mesh(mesh=None) -> Tuple[int, int]:
        if mesh is None:
            return 0, 0
        return mesh.local_rank("dp"), mesh.local_rank("tp")

    @torch.no_grad()
    def save(self, engine, train_state, config, mesh=None, lr: float = 0.0) -> bool:
        path = Path(self.path)
        cur = self._create_folder(path, FOLDER_NAME.format(train_state.step))
        logger.info(f"Saving to: {cur}")
        _barrier()
        sd = engine_state_dict(engine, lr)
        dcp.save(sd, checkpoint_id=cur)
        del sd
        logger.info("State dict saved!")
        _barrier()
        if get_is_master():
            with open(cur / CONFIG_NAME, "w") as f:
                json.dump(dataclass_to_dict(config), f)
        dp_rank, tp_rank = self._get_dp_tp_mesh(mesh)
        if tp_rank == 0:
            name = TRAIN_STATE_NAME.format(dp_rank)
            logger.info(f"Saving train state to: {cur / name}")
            with open(cur / name, "w") as f:
                json.dump(train_state.state_dict(), f)
        self.existing_saves.append(cur)
        self.clean_up()
        _barrier()
        return True

    @torch.no_grad()
    def load(self, engine, train_state, mesh=None, path: Optional[Path] = None) -> None:
        """Resume from ``path`` or, by default, from the newest step folder that loads. A folder whose shards are
        damaged (a job killed in the middle of a save, a truncated ``.distcp`` file) is reported and skipped, and the
        next older one is tried, so a bad last save costs the steps since the previous one instead of the run."""
        dp_rank, _ = self._get_dp_tp_mesh(mesh)
        if path is not None:
            candidates = [Path(path)]
        else:
            candidates = [p for p in reversed(self.existing_saves) if (p / TRAIN_STATE_NAME.format(dp_rank)).is_file()]
        for i, cand in enumerate(candidates):
            try:
                with open(cand / TRAIN_STATE_NAME.format(dp_rank), "r") as f:
                    state = json.load(f)
                sd = engine_state_dict(engine)
                dcp.load(sd, checkpoint_id=cand)
            except (Exception, CheckpointException) as e:  # any reader error means the folder cannot be trusted
                if path is not None or i == len(candidates) - 1:
                    raise
                logger.error(f"Checkpoint {cand} cannot be loaded ({type(e).__name__}: {str(e)[:200]}); "
                             f"falling back to {candidates[i + 1]}")
                continue
            train_state.load_state_dict(state)
            logger.info(f"Train state reloaded; loading from: {cand}")
            load_engine_state_dict(engine, sd, load_optim=True)
            logger.info("Model and optim reloaded")
            return

    @classmethod
    def instantiate_and_make_dir(cls, args: CheckpointArgs):
        if get_is_master():
            os.makedirs(args.path, exist_ok=True)
        _barrier()
        return cls(args)
