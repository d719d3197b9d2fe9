"""Sharded-parameter engine: flat per-group buffers, ZeRO-style sharded AdamW, gradient clip.

This owns what FSDP2 ``fully_shard`` + ``torch.optim.AdamW(fused=True)`` + ``clip_grad_norm_``
do in the reference (lingua/distributed.py:419-463, lingua/optim.py:149-158,
apps/main/train.py:431-442), laid out for one NVSwitch domain:

* every group of the grouping plan (embeddings, each block, output head, leftovers) has one
  contiguous compute-dtype buffer holding all its parameters (so QKV and w1|w3 are adjacent and
  run as single GEMMs) and one contiguous fp32 gradient buffer that the wgrad GEMMs write into
  (``param.main_grad``);
* rank r owns the r-th 1/W slice of each buffer: fp32 master weights and both Adam moments
  exist only for that slice (the reference's "sharded fp32 parameters are the master weights");
* after a group's backward its gradient buffer is reduce-scattered in fp32 on a side stream;
  the optimiser step is one AdamW launch per group that also applies the clip factor computed
  on the device from the all-reduced squared norm (no host synchronisation) and writes the
  compute-dtype copy of the slice, which is then all-gathered for the next forward.

With ``reshard_after_forward=False`` semantics (the main app's plan) gathered parameters stay
resident for the whole step. The same code runs on CPU with gloo for plumbing tests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as F


@dataclass
class EngineOptim:
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    clip: float = 1.0


class ParamGroup:
    """One flat buffer worth of parameters."""

    def __init__(self, name: str, params: List[Tuple[str, nn.Parameter]], world: int, rank: int,
                 compute_dtype: torch.dtype, device: torch.device, alloc_full: Optional[Callable] = None,
                 alloc_grad: Optional[Callable] = None):
        self.name, self.params = name, params
        # peer-visible addresses of this rank's slice inside every rank's gradient buffer (own first), when the
        # gradient buffers live in symmetric memory: the reduce-scatter then pulls instead of staging
        self.peer_grad_ptrs: Optional[List[int]] = None
        self.peer_full: Optional[List[torch.Tensor]] = None  # every rank's ``full`` buffer, when peer-visible
        self.peer_stage: Optional[List[torch.Tensor]] = None  # every rank's reduce-scatter staging [world-1, shard]
        self.rs_stage: Optional[torch.Tensor] = None
        self.world, self.rank = world, rank
        align = 64 * world  # every shard starts on a 256-byte boundary in fp32
        self.offsets: Dict[str, Tuple[int, int]] = {}
        off = 0
        for fqn, p in params:
            n = p.numel()
            self.offsets[fqn] = (off, n)
            off += (n + 7) // 8 * 8  # keep every tensor 16-byte aligned in bf16 (TMA base rule)
        self.numel = off
        self.padded = (off + align - 1) // align * align
        self.shard_numel = self.padded // world
        self.full = (alloc_full(self.padded) if alloc_full is not None
                     else torch.zeros(self.padded, dtype=compute_dtype, device=device))
        self.grad = (alloc_grad(self.padded) if alloc_grad is not None
                     else torch.zeros(self.padded, dtype=torch.float32, device=device))
        s0 = rank * self.shard_numel
        self.shard_slice = slice(s0, s0 + self.shard_numel)
        self.master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = self.grad[self.shard_slice] if world == 1 else torch.zeros_like(self.master)
        self.params_ready: Optional[torch.cuda.Event] = None
        self.grads_ready: Optional[torch.cuda.Event] = None
        self.reduced = False
        for i, (fqn, p) in enumerate(params):
            o, n = self.offsets[fqn]
            view = self.full[o:o + n].view(p.shape)
            if p.device.type != "meta":
                view.copy_(p.data)
            # a fresh Parameter: meta / other-device / other-dtype tensors cannot be re-pointed in place
            new_p = nn.Parameter(view, requires_grad=p.requires_grad)
            new_p.main_grad = self.grad[o:o + n].view(p.shape)
            new_p.grad_written = False
            if getattr(p, "lb_fp8", False):  # float8 matmuls were requested for this weight
                new_p.lb_fp8 = True
            params[i] = (fqn, new_p)

    def sync_master_from_full(self) -> None:
        self.master.copy_(self.full[self.shard_slice])


class ShardedEngine:
    def __init__(self, model: nn.Module, plan: Sequence[Tuple[str, bool]], process_group=None,
                 compute_dtype: torch.dtype = torch.bfloat16, optim: Optional[EngineOptim] = None,
                 device: Optional[torch.device] = None, p2p_gather: bool = True, p2p_reduce: Optional[str] = None):
        self.model = model
        # gradient reduce-scatter over peer memory: "pull" (one kernel reads the peers' gradient buffers) or
        # "push" (copy engines fill staging slots, a kernel sums them); LB_P2P_REDUCE overrides the default
        import os

        self.p2p_reduce = p2p_reduce or os.environ.get("LB_P2P_REDUCE", "push")
        assert self.p2p_reduce in ("pull", "push")
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_initialized() and process_group is not False) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        self.optim = optim or EngineOptim()
        self.device = device or next(model.parameters()).device
        self.compute_dtype = compute_dtype
        self.is_cuda = self.device.type == "cuda"
        self.step_count = 0
        # True while micro-batches are still being accumulated: a group's backward must not start its
        # gradient reduction before the last micro-batch has added its share
        self.defer_reduce = False
        # side stream: gradient reduce-scatter / parameter all-gather, and each group's share of the
        # gradient norm, all of which overlap the backward pass of the groups that are still running
        self.comm_stream = torch.cuda.Stream(self.device, priority=-1) if self.is_cuda else None
        # Parameter all-gather over NVLink by the copy engines: the compute-dtype buffers live in peer-visible
        # (symmetric) memory, every rank pushes its freshly updated slice into the peers' buffers with plain
        # device-to-device copies and a small barrier kernel confirms arrival. No SM runs a communication
        # kernel while the next forward pass is computing. Falls back to NCCL when the group has no peer access.
        self._symm = None
        self._pad_ptrs: Optional[List[int]] = None
        self._barrier_epoch = 0
        if self.is_cuda and self.world > 1 and p2p_gather:
            try:
                import torch.distributed._symmetric_memory as sm

                pad = sm.empty(8, dtype=torch.int32, device=self.device)
                pad.zero_()
                hdl = sm.rendezvous(pad, group=self.pg if self.pg is not None else dist.group.WORLD)
                self._symm, self._pad = sm, pad
                from ..ops import _lib

                if self.p2p_reduce == "pull" and not hasattr(_lib.load(), "lb_reduce_peers"):
                    self.p2p_reduce = "push"  # a library built before the pull kernel existed
                self._pad_ptrs = [int(p) for p in hdl.buffer_ptrs]
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.pg)  # every pad is zero before the first barrier kernel runs
            except Exception as e:  # no peer access inside this group: NCCL all-gather
                import logging

                logging.getLogger(__name__).warning("peer-to-peer parameter gather disabled: %s", e)
                self._symm = None

        taken = set()
        self.groups: List[ParamGroup] = []
        self.group_of_module: Dict[str, int] = {}
        for path, _reshard in plan:
            mod = model.get_submodule(path)
            ps = [(f"{path}.{n}", p) for n, p in mod.named_parameters() if f"{path}.{n}" not in taken]
            taken.update(fqn for fqn, _ in ps)
            if ps:
                self._add_group(path, ps)
        rest = [(n, p) for n, p in model.named_parameters() if n not in taken]
        if rest:
            self._add_group("", rest)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.sumsq_parts = torch.zeros(len(self.groups), dtype=torch.float32, device=self.device)  # one per group
        self.n_params = sum(g.numel for g in self.groups)

    def _add_group(self, path: str, ps: List[Tuple[str, nn.Parameter]]) -> None:
        self.group_of_module[path] = len(self.groups)
        alloc = None
        if self._symm is not None:
            def alloc(n):
                t = self._symm.empty(n, dtype=self.compute_dtype, device=self.device)
                t.zero_()
                return t
        alloc_grad = None
        if self._symm is not None and self.p2p_reduce == "pull":
            def alloc_grad(n):
                t = self._symm.empty(n, dtype=torch.float32, device=self.device)
                t.zero_()
                return t
        g = ParamGroup(path, ps, self.world, self.rank, self.compute_dtype, self.device, alloc_full=alloc,
                       alloc_grad=alloc_grad)
        if self._symm is not None:
            try:
                hdl = self._symm.rendezvous(g.full, group=self.pg if self.pg is not None else dist.group.WORLD)
                g.peer_full = [hdl.get_buffer(r, (g.padded,), self.compute_dtype) for r in range(self.world)]
                if alloc_grad is not None:
                    hg = self._symm.rendezvous(g.grad, group=self.pg if self.pg is not None else dist.group.WORLD)
                    mine = self.rank * g.shard_numel * 4
                    ring = [(self.rank + k) % self.world for k in range(self.world)]  # own first, then the ring
                    g.peer_grad_ptrs = [int(hg.buffer_ptrs[r]) + mine for r in ring]
                if g.peer_grad_ptrs is None:
                    # staging of the gradient reduce-scatter: slot k-1 of rank r receives the slice from rank r - k
                    g.rs_stage = self._symm.empty((self.world - 1) * g.shard_numel, dtype=torch.float32,
                                                  device=self.device)
                    h2 = self._symm.rendezvous(g.rs_stage, group=self.pg if self.pg is not None else dist.group.WORLD)
                    g.peer_stage = [h2.get_buffer(r, (self.world - 1, g.shard_numel), torch.float32)
                                    for r in range(self.world)]
            except Exception as e:  # this group then uses the NCCL collectives
                import logging

                logging.getLogger(__name__).warning("no peer view of group %s: %s", path, e)
                g.peer_full = g.peer_stage = g.peer_grad_ptrs = None
        self.groups.append(g)
        for fqn, new_p in g.params:
            owner_path, _, attr = fqn.rpartition(".")
            self.model.get_submodule(owner_path)._parameters[attr] = new_p

    # ------------------------------------------------------------------ init / state
    def sync_master(self) -> None:
        """Call after (re-)initialising or loading the compute-dtype weights."""
        for g in self.groups:
            g.sync_master_from_full()

    def init_weights_fp32(self, init_fn: Callable[[], None]) -> None:
        """Initialise in fp32 so that master weights are not rounded through bf16: temporarily
        re-point the parameters at fp32 storage, run ``init_fn`` and split the result."""
        fp32_bufs = []
        for g in self.groups:
            buf = torch.zeros(g.padded, dtype=torch.float32, device=self.device)
            fp32_bufs.append(buf)
            for fqn, p in g.params:
                o, n = g.offsets[fqn]
                p.data = buf[o:o + n].view(p.shape)
        init_fn()
        for g, buf in zip(self.groups, fp32_bufs):
            g.master.copy_(buf[g.shard_slice])
            g.full.copy_(buf)
            for fqn, p in g.params:
                o, n = g.offsets[fqn]
                p.data = g.full[o:o + n].view(p.shape)
        del fp32_bufs

    # ------------------------------------------------------------------ per-step protocol
    def zero_grad(self) -> None:
        for g in self.groups:
            g.reduced = False
            for _, p in g.params:
                p.grad_written = False
                p.grad = None

    def wait_params(self, gi: int) -> None:
        """Block the compute stream until group gi's all-gathered weights have landed."""
        g = self.groups[gi]
        if g.params_ready is not None:
            torch.cuda.current_stream().wait_event(g.params_ready)
            g.params_ready = None

    def _flush_autograd_grads(self, g: ParamGroup) -> None:
        """Reference-path modules produce ``p.grad``; fold those into the flat fp32 buffer."""
        for _, p in g.params:
            if p.grad is not None:
                if p.grad_written:
                    p.main_grad.add_(p.grad.to(torch.float32))
                else:
                    p.main_grad.copy_(p.grad)
                    p.grad_written = True
                p.grad = None
            elif not p.grad_written:
                p.main_grad.zero_()
                p.grad_written = True

    def reduce_group(self, gi: int) -> None:
        """Reduce-scatter (mean) group gi's gradients; asynchronous on CUDA."""
        g = self.groups[gi]
        if g.reduced:
            return
        g.reduced = True
        self._flush_autograd_grads(g)
        part = self.sumsq_parts[gi:gi + 1]
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                part.zero_()
                if self.world > 1 and g.peer_grad_ptrs is not None:
                    # reduce-scatter by pulling: once every rank's gradients of this group are final (barrier),
                    # one kernel reads this rank's slice out of every rank's buffer over NVLink, sums, scales and
                    # accumulates the squared norm. Nobody writes these buffers again before the parameter
                    # all-gather barriers of this step, which every rank reaches only after its own pull.
                    self._peer_barrier()
                    self._reduce_peers(g, part)
                elif self.world > 1 and g.peer_stage is not None:
                    # reduce-scatter by the copy engines: every rank pushes the slice owned by rank r into the
                    # slot it has in r's staging buffer; after the barrier one kernel sums the slots with the
                    # local slice, scales by 1 / world and accumulates the squared norm
                    n = g.shard_numel
                    for k in range(1, self.world):
                        r = (self.rank + k) % self.world
                        g.peer_stage[r][k - 1].copy_(g.grad[r * n:(r + 1) * n], non_blocking=True)
                    self._peer_barrier()
                    self._reduce_slots(g, part)
                else:
                    if self.world > 1:
                        dist.reduce_scatter_tensor(g.grad_shard, g.grad, op=dist.ReduceOp.AVG, group=self.pg)
                    F.sumsq(g.grad_shard, part)
                g.grads_ready = torch.cuda.Event()
                g.grads_ready.record(self.comm_stream)
            return
        if self.world > 1:
            dist.all_reduce(g.grad, op=dist.ReduceOp.SUM, group=self.pg)
            g.grad_shard.copy_(g.grad[g.shard_slice]).div_(self.world)
        part.zero_()
        F.sumsq(g.grad_shard, part)

    def step(self, lr: float, grad_mul: float = 1.0) -> torch.Tensor:
        """Finish gradient reduction, clip by global norm, AdamW on the owned slices, re-gather.
        Returns the (pre-clip) gradient norm as a device tensor."""
        for gi in range(len(self.groups) - 1, -1, -1):
            self.reduce_group(gi)
        for g in self.groups:
            if g.grads_ready is not None:
                torch.cuda.current_stream().wait_event(g.grads_ready)
                g.grads_ready = None
        torch.sum(self.sumsq_parts, dim=0, keepdim=True, out=self.sumsq)
        if self.world > 1:
            dist.all_reduce(self.sumsq, op=dist.ReduceOp.SUM, group=self.pg)
        self.step_count += 1
        o = self.optim
        for g in self.groups:
            F.adamw_step(g.master, g.exp_avg, g.exp_avg_sq, g.grad_shard, g.full[g.shard_slice],
                         step=self.step_count, lr=lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps, wd=o.weight_decay,
                         sumsq_t=self.sumsq, max_norm=o.clip, grad_mul=grad_mul)
            if self.world > 1:
                self._gather_group(g)  # overlaps the AdamW launches of the groups that follow
        return self.sumsq.sqrt() * grad_mul

    def gather_params(self) -> None:
        """All-gather every group's compute-dtype slice into its full buffer (in group order, so
        the first layers of the next forward are ready first)."""
        if self.world == 1:
            return
        for g in self.groups:
            self._gather_group(g)

    def _gather_group(self, g: ParamGroup) -> None:
        """In-place all-gather of one group (every rank's slice already sits at its place in ``g.full``);
        on CUDA it runs on the side stream after everything queued so far on the compute stream."""
        if self.comm_stream is not None:
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(done)
            with torch.cuda.stream(self.comm_stream):
                if g.peer_full is not None:
                    mine = g.full[g.shard_slice]
                    for k in range(1, self.world):  # start with the next rank so that links are used evenly
                        r = (self.rank + k) % self.world
                        g.peer_full[r][g.shard_slice].copy_(mine, non_blocking=True)
                    self._peer_barrier()  # every rank's pushes, mine included, have landed
                else:
                    dist.all_gather_into_tensor(g.full, g.full[g.shard_slice], group=self.pg)
                g.params_ready = torch.cuda.Event()
                g.params_ready.record(self.comm_stream)
        else:
            dist.all_gather_into_tensor(g.full, g.full[g.shard_slice].clone(), group=self.pg)

    def _reduce_slots(self, g: ParamGroup, part: torch.Tensor) -> None:
        import ctypes as C

        from ..ops import _lib

        lib = _lib.load()
        if not getattr(lib, "_reduce_slots_declared", False):
            lib.lb_reduce_slots.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p, C.c_longlong,
                                            C.c_float, C.c_void_p, C.c_void_p]
            lib.lb_reduce_slots.restype = C.c_int
            lib._reduce_slots_declared = True
        own = g.grad[g.shard_slice]
        rc = lib.lb_reduce_slots(own.data_ptr(), g.rs_stage.data_ptr(), self.world - 1, g.shard_numel,
                                 g.grad_shard.data_ptr(), g.shard_numel, 1.0 / self.world, part.data_ptr(),
                                 _lib.stream_ptr())
        _lib.check(rc, "lb_reduce_slots")

    def _reduce_peers(self, g: ParamGroup, part: torch.Tensor) -> None:
        import ctypes as C

        from ..ops import _lib

        lib = _lib.load()
        if not getattr(lib, "_reduce_peers_declared", False):
            lib.lb_reduce_peers.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong, C.c_float, C.c_void_p,
                                            C.c_void_p]
            lib.lb_reduce_peers.restype = C.c_int
            lib._reduce_peers_declared = True
        srcs = (C.c_void_p * self.world)(*g.peer_grad_ptrs)
        rc = lib.lb_reduce_peers(srcs, self.world, g.grad_shard.data_ptr(), g.shard_numel, 1.0 / self.world,
                                 part.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "lb_reduce_peers")

    def _peer_barrier(self) -> None:
        from .tp_fused import peer_barrier

        self._barrier_epoch += 1
        # ranks of a training job drift (data loading, logging, checkpoints): generous but finite limit
        peer_barrier(self._pad_ptrs, self.rank, self._barrier_epoch, limit_s=120.0)

    def wait_all_params(self) -> None:
        for gi in range(len(self.groups)):
            self.wait_params(gi)

    # ------------------------------------------------------------------ hooks for the model
    def boundary(self, module_path: str, *tensors):
        """Identity on ``tensors`` placed at the input of a group's module: its forward waits for
        the group's gathered weights, its backward (which runs after every op of the module has
        been differentiated) starts the group's gradient reduce-scatter."""
        gi = self.group_of_module.get(module_path)
        if gi is None or (self.world == 1 and self.comm_stream is None):
            return tensors
        self.wait_params(gi)
        live = [t for t in tensors if t is not None]
        if not any(t.requires_grad for t in live):
            return tensors
        outs = list(_Boundary.apply(self, gi, *live))
        it = iter(outs)
        return tuple(next(it) if t is not None else None for t in tensors)

    # ------------------------------------------------------------------ introspection
    def full_tensor_fp32(self, gi: int) -> torch.Tensor:
        """All-gathered fp32 master weights of one group (checkpoint export)."""
        g = self.groups[gi]
        if self.world == 1:
            return g.master
        out = torch.empty(g.padded, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(out, g.master, group=self.pg)
        return out


class _Boundary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, engine, gi, *tensors):
        ctx.engine, ctx.gi = engine, gi
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        if not ctx.engine.defer_reduce:
            ctx.engine.reduce_group(ctx.gi)
        return (None, None, *grads)
