"""Metric logging and device monitoring.

``MetricLogger`` appends one JSON object per call to ``metrics.jsonl`` (plus ``created_at``) and
mirrors it to wandb on rank 0 when configured; ``GPUMemoryMonitor`` reports the peak
active / reserved memory, allocator retries, OOM count and board power (lingua/metrics.py:
WandbArgs :22, LoggingArgs :48, MetricLogger :55, GPUMemoryMonitor :115,
upload_train_to_wandb :185, get_num_params :224). ``peak_flops`` adds what the reference leaves
to an offline trace analysis: the denominator for an in-loop ``speed/mfu``.
"""
from __future__ import annotations

import json
import logging
from collections import namedtuple
from dataclasses import asdict, dataclass
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Dict, List, Optional, Union

import torch
import torch.nn as nn

from .distributed import get_is_master

logger = logging.getLogger()


@dataclass
class WandbArgs:
    job_type: Optional[str] = None
    dir: Optional[str] = None
    project: Optional[str] = None
    entity: Optional[str] = None
    tags: Optional[List] = None
    group: Optional[str] = None
    name: Optional[str] = None
    notes: Optional[str] = None
    config_exclude_keys: Optional[List[str]] = None
    config_include_keys: Optional[List[str]] = None
    anonymous: Optional[str] = None
    mode: Optional[str] = None
    allow_val_change: Optional[bool] = None
    resume: Optional[Union[bool, str]] = None
    force: Optional[bool] = None
    tensorboard: Optional[bool] = None
    sync_tensorboard: Optional[bool] = None
    monitor_gym: Optional[bool] = None
    save_code: Optional[bool] = None
    id: Optional[str] = None
    fork_from: Optional[str] = None
    resume_from: Optional[str] = None


@dataclass
class LoggingArgs:
    freq: int = 10  # log every `freq` optimiser steps
    acc_freq: Optional[int] = None  # log every `acc_freq` gradient-accumulation steps
    wandb: Optional[WandbArgs] = None


def _wandb():
    try:
        import wandb

        return wandb
    except Exception:  # not installed / unusable offline
        return None


class MetricLogger:
    def __init__(self, outdir: Path, args: Optional[Any] = None):
        self.outdir, self.args, self.jsonl_writer = outdir, args, None
        self._wandb_on = False

    def open(self):
        if self.jsonl_writer is None:
            self.jsonl_writer = open(self.outdir, "a")
        wb = getattr(getattr(self.args, "logging", None), "wandb", None)
        if wb is not None and get_is_master():
            w = _wandb()
            if w is None:
                logger.warning("wandb logging requested but the wandb package is not usable; skipping")
            else:
                w.init(config=asdict(self.args), **{k: v for k, v in asdict(wb).items() if v is not None})
                self._wandb_on = True

    def log(self, metrics: Dict[str, Any]):
        if self._wandb_on:
            w = _wandb()
            if w is not None and w.run is not None:
                w.log(metrics, step=metrics["global_step"])
        metrics.update({"created_at": datetime.now(timezone.utc).isoformat()})
        print(json.dumps(metrics), file=self.jsonl_writer, flush=True)

    def close(self):
        if self.jsonl_writer is not None:
            self.jsonl_writer.close()
            self.jsonl_writer = None

    def __enter__(self):
        self.open()
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()

    def __del__(self):
        self.close()


GPUMemStats = namedtuple("GPUMemStats", ["max_active_gib", "max_active_pct", "max_reserved_gib", "max_reserved_pct",
                                         "num_alloc_retries", "num_ooms", "power_draw"])


class GPUMemoryMonitor:
    """Peak-memory and power statistics of the current CUDA device; all zeros without a GPU."""

    def __init__(self, device: str = "cuda:0"):
        self.cuda = torch.cuda.is_available() and str(device).startswith("cuda")
        if self.cuda:
            self.device = torch.device(device)
            self.device_name = torch.cuda.get_device_name(self.device)
            self.device_index = torch.cuda.current_device()
            self.device_capacity = torch.cuda.get_device_properties(self.device).total_memory
            torch.cuda.reset_peak_memory_stats()
            torch.cuda.empty_cache()
        else:
            self.device, self.device_name, self.device_index, self.device_capacity = torch.device("cpu"), "cpu", 0, 1
        self.device_capacity_gib = self._gib(self.device_capacity)

    @staticmethod
    def _gib(n: float) -> float:
        return n / (1024 ** 3)

    def get_peak_stats(self) -> GPUMemStats:
        if not self.cuda:
            return GPUMemStats(0.0, 0.0, 0.0, 0.0, 0, 0, 0.0)
        info = torch.cuda.memory_stats(self.device)
        active, reserved = info["active_bytes.all.peak"], info["reserved_bytes.all.peak"]
        retries, ooms = info["num_alloc_retries"], info["num_ooms"]
        try:
            power = torch.cuda.power_draw()
        except Exception:
            power = 0.0
        if retries > 0:
            logger.warning(f"{retries} CUDA memory allocation retries.")
        if ooms > 0:
            logger.warning(f"{ooms} CUDA OOM errors thrown.")
        cap = self.device_capacity
        return GPUMemStats(self._gib(active), 100 * active / cap, self._gib(reserved), 100 * reserved / cap, retries,
                           ooms, power)

    def reset_peak_stats(self):
        if self.cuda:
            torch.cuda.reset_peak_memory_stats()
            torch.cuda.reset_accumulated_memory_stats()

    def __str__(self):
        s = self.get_peak_stats()
        return (f"{self.device_name} ({self.device_index}): {self.device_capacity_gib} GiB capacity, "
                f"{s.max_reserved_gib} GiB peak, {s.max_reserved_pct}% peak")


def upload_train_to_wandb(ckpt_dir, project="lingua", entity=None, train=True, eval=True):
    """Replay metrics.jsonl / metrics.eval.jsonl of a finished run into wandb."""
    import yaml

    w = _wandb()
    if w is None:
        raise RuntimeError("wandb is not installed")
    cfg = yaml.safe_load(open(Path(ckpt_dir) / "config.yaml"))
    if train:
        w.init(config=cfg, name=cfg["name"], project=project, entity=entity)
        with open(Path(ckpt_dir) / "metrics.jsonl") as f:
            for line in f:
                m = json.loads(line)
                w.log(m, step=m["global_step"])
        w.finish()
    if eval:
        w.init(config=cfg, name=cfg["name"], project=project, entity=entity)
        with open(Path(ckpt_dir) / "metrics.eval.jsonl") as f:
            for line in f:
                m = json.loads(line)
                w.log({f"evals/{k.replace('/', '.')}": v for k, v in m.items() if "/" in k}, step=m["global_step"])
        w.finish()


def get_num_params(model: nn.Module) -> int:
    return sum(p.numel() for p in model.parameters())


def peak_flops(dtype: str = "bf16") -> float:
    """Dense tensor-core peak used as the MFU denominator: the measured sustained cuBLAS rate of
    this machine when a ``MEASURED_PEAKS.json`` sits at the repository root, else the nominal
    B200 figure."""
    root = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    nominal = {"bf16": 2.25e15, "fp16": 2.25e15, "fp8": 4.5e15, "fp32": 1.1e15}[dtype]
    try:
        peaks = json.loads(root.read_text())
        if dtype in ("bf16", "fp16") and peaks.get("bf16_tflops_sustained"):
            return float(peaks["bf16_tflops_sustained"]) * 1e12
    except Exception:
        pass
    return nominal
