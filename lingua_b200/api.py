"""Small public training API: build a sharded model from config dataclasses and step it.

    trainer = Trainer(model_args, dist_args, optim_args, total_steps)
    loss = trainer.train_step(batch)          # batch: [B, S, n_views] int64, host or device

``train_step`` does what one iteration of apps/main/train.py:347-442 does: host-to-device
copy of the batch, forward + backward (with gradient accumulation), gradient clipping, the
AdamW update and the scheduler step. It returns the loss as a Python float (one
device-to-host read); ``train_step_async`` returns the device tensor instead.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .distributed import DistributedArgs, Mesh, get_device_mesh, parallelize_model
from .models.transformer import LMTransformer, LMTransformerArgs, build_fsdp_grouping_plan
from .optim import LRScheduler, OptimArgs, build_engine_optim, build_lr_fn
from .profiling import nvtx_range


class Trainer:
    def __init__(self, model_args: LMTransformerArgs, dist_args: Optional[DistributedArgs] = None,
                 optim_args: Optional[OptimArgs] = None, total_steps: int = 1000, mesh: Optional[Mesh] = None,
                 grad_acc_steps: int = 1, device: Optional[torch.device] = None, model_cls=LMTransformer,
                 grouping_plan=None, loss_fn=None):
        # loss_fn(model, inputs, labels) -> scalar loss, for models whose forward is not (tokens, targets)
        self.loss_fn = loss_fn
        self.dist_args = dist_args or DistributedArgs()
        self.optim_args = optim_args or OptimArgs()
        self.mesh = mesh or get_device_mesh(self.dist_args)
        self.grad_acc_steps = grad_acc_steps
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = device
        with torch.device("meta"):
            model = model_cls(model_args)
        plan = grouping_plan if grouping_plan is not None else build_fsdp_grouping_plan(model_args)
        from .parallel.tensor_parallel import tp_parallelize as tp_plan
        self.model, self.engine = parallelize_model(model, self.mesh, model_args, self.dist_args,
                                                    fsdp_grouping_plan=plan, tp_parallelize=tp_plan,
                                                    optim=build_engine_optim(self.optim_args), device=device,
                                                    grad_acc_steps=grad_acc_steps)
        with torch.random.fork_rng(devices=[device] if device.type == "cuda" else []):
            torch.manual_seed(model_args.seed)
            self.engine.init_weights_fp32(self.model.init_weights)
        # the loss of every micro-batch receives the gradient 1 / grad_acc_steps (see train_step_async)
        self.model.loss_grad_scale = 1.0 / grad_acc_steps
        self.scheduler = LRScheduler(self.optim_args.lr, build_lr_fn(self.optim_args, total_steps))
        self.step = 0
        self.acc_step = 0
        self._staging = None

    def _to_device(self, batch) -> torch.Tensor:
        if isinstance(batch, np.ndarray):
            batch = torch.from_numpy(batch)
        if batch.device != self.device:
            if self.device.type == "cuda" and not batch.is_pinned():
                if self._staging is None or self._staging.shape != batch.shape:
                    self._staging = torch.empty(batch.shape, dtype=batch.dtype).pin_memory()
                self._staging.copy_(batch)
                batch = self._staging
            batch = batch.to(self.device, non_blocking=True)
        return batch

    def train_step_async(self, batch, doc_start=None, doc_end=None) -> torch.Tensor:
        batch = self._to_device(batch)
        inputs, labels = batch[:, :, 0].contiguous(), batch[:, :, 1].contiguous()
        if self.acc_step == 0:
            self.engine.zero_grad()
        kw = {}
        if doc_start is not None:
            kw["doc_start"] = doc_start
        if doc_end is not None:
            kw["doc_end"] = doc_end
        self.engine.defer_reduce = (self.acc_step + 1) % self.grad_acc_steps != 0
        with nvtx_range("forward"):
            loss = self.loss_fn(self.model, inputs, labels) if self.loss_fn else self.model(inputs, labels, **kw)
        with nvtx_range("backward"):
            (loss / self.grad_acc_steps if self.grad_acc_steps > 1 else loss).backward()
        self.acc_step = (self.acc_step + 1) % self.grad_acc_steps
        if self.acc_step == 0:
            with nvtx_range("optimizer"):
                self.last_grad_norm = self.engine.step(self.scheduler.get_lr())
            self.scheduler.step()
            self.step += 1
        return loss.detach()

    def train_step(self, batch, doc_start=None, doc_end=None) -> float:
        loss = float(self.train_step_async(batch, doc_start, doc_end).item())
        if self.device.type == "cuda":
            from .ops import _lib

            _lib.check_status()  # raises if a bounded wait of any kernel (peer barrier, copy) ran out during the step
        return loss
