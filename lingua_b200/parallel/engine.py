"""Sharded-parameter engine: per-group buffers, row-sharded ownership, ZeRO-style AdamW, gradient clip.

This owns what FSDP2 ``fully_shard`` + ``torch.optim.AdamW(fused=True)`` + ``clip_grad_norm_``
do in the reference (lingua/distributed.py:419-463, lingua/optim.py:149-158,
apps/main/train.py:431-442), laid out for one NVSwitch domain:

* every group of the grouping plan (embeddings, each block, output head, leftovers) has one
  contiguous compute-dtype buffer holding all its parameters (so QKV and w1|w3 are adjacent and
  run as single GEMMs);
* ownership is by rows, like FSDP2's dim-0 sharding, in blocks of 128 rows: rank r owns a slab of
  every weight matrix (the *scatter* parameters) and the r-th 1/W slice of a small flat region
  that holds everything else (norm weights, biases, embeddings: the *plain* parameters). fp32
  master weights, both Adam moments and the fp32 gradient exist only for the owned part;
* the weight-gradient GEMM of a scatter parameter has no local output matrix at all: its epilogue
  stores every 128-row block straight into the owner's memory (``ops.gemm.gemm_scatter``: the own
  slab into the gradient shard, peer slabs over NVLink into this rank's slot of the owner's
  staging area), so the reduce-scatter's transfer rides underneath the backward GEMMs; after a
  barrier one kernel per group sums the slots, scales by 1 / W and accumulates the squared norm;
* plain parameters keep a local fp32 gradient that is pushed slice-wise by the copy engines;
* the optimiser step is one AdamW launch per owned segment that applies the clip factor computed
  on the device from the all-reduced squared norm (no host synchronisation) and writes the
  compute-dtype copy, which the copy engines then push into every peer's parameter buffer.

``replicate_group`` adds the outer axis of hybrid sharding (lingua/distributed.py:106-113,441-446):
gradients are reduce-scattered inside the shard group and the reduced shard is averaged over the
replicas. Without peer access (or on CPU with gloo) the same layout runs on all-reduce /
all-gather collectives and a full local gradient buffer.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as F

logger = logging.getLogger(__name__)

BLOCK_ROWS = 128  # ownership granularity of a weight matrix = rows stored by one CTA of the GEMM epilogue


@dataclass
class EngineOptim:
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    clip: float = 1.0


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def default_scatter_filter(fqn: str, p: torch.Tensor) -> bool:
    """Parameters whose gradient comes out of a weight-gradient GEMM: 2-D, TMA-compatible row pitch.
    Embedding tables are 2-D too but receive a scatter-add, so they stay with the plain parameters."""
    return p.dim() == 2 and p.shape[1] % 8 == 0 and p.shape[0] >= BLOCK_ROWS and "emb" not in fqn.lower()


def row_bounds(rows: int, world: int) -> List[int]:
    """Start row of every rank's slab (+ the end): blocks of 128 rows dealt out as evenly as possible."""
    nblk = (rows + BLOCK_ROWS - 1) // BLOCK_ROWS
    b = [min(rows, round(r * nblk / world) * BLOCK_ROWS) for r in range(world)]
    return b + [rows]


class ScatterTarget:
    """Attached to a scatter parameter as ``p.lb_scatter`` when its gradient has no local matrix, and as
    ``p.lb_gather`` when its remote rows are fetched by the first GEMM that multiplies with it."""

    def __init__(self, engine: "ShardedEngine", group: "ParamGroup", index: int):
        self.engine, self.group, self.index = engine, group, index


# Weights whose first use in a step is a forward GEMM of the native transformer block: their all-gather is fused
# into that GEMM (the kernel pulls the peers' row blocks while it computes), everything else is pushed by the
# copy engines right after the optimiser step.
DEFAULT_GATHER_IN_GEMM = ("attention.wq", "attention.wk", "attention.wv", "feed_forward.w1", "feed_forward.w3")


class ParamGroup:
    """One buffer worth of parameters and this rank's share of their optimiser state."""

    def __init__(self, name: str, params: List[Tuple[str, nn.Parameter]], world: int, rank: int,
                 compute_dtype: torch.dtype, device: torch.device, scatter_filter: Callable,
                 alloc_full: Optional[Callable] = None):
        self.name, self.world, self.rank = name, world, rank
        mats = [(f, p) for f, p in params if scatter_filter(f, p)]
        mat_ids = {id(p) for _, p in mats}
        plains = [(f, p) for f, p in params if id(p) not in mat_ids]
        self.params: List[Tuple[str, nn.Parameter]] = mats + plains
        self.n_mats = len(mats)
        self.offsets: Dict[str, Tuple[int, int]] = {}
        off = 0
        for fqn, p in mats:
            self.offsets[fqn] = (off, p.numel())
            off += _round_up(p.numel(), 8)  # every tensor starts 16-byte aligned in bf16 (TMA base rule)
        self.plain_off = _round_up(off, 64)
        off = self.plain_off
        for fqn, p in plains:
            self.offsets[fqn] = (off, p.numel())
            off += _round_up(p.numel(), 8)
        self.numel = off
        self.plain_padded = _round_up(off - self.plain_off, 64 * world)
        self.plain_shard = self.plain_padded // world
        self.padded = self.plain_off + self.plain_padded
        # per-rank row slabs of every matrix and the resulting shard layout: [slab of mat 0 | slab of mat 1 | ...
        # | plain slice], every piece starting on a multiple of 8 elements
        self.bounds: List[List[int]] = [row_bounds(p.shape[0], world) for _, p in mats]
        self.mat_shard_off: List[List[int]] = [[0] * len(mats) for _ in range(world)]  # [rank][mat]
        self.mat_numel: List[int] = []       # elements of the matrix part of every rank's shard
        self.shard_numels: List[int] = []
        self.segments: List[List[Tuple[int, int, int]]] = []  # [rank] -> (offset in full, n, offset in shard)
        for r in range(world):
            so, segs = 0, []
            for i, (fqn, p) in enumerate(mats):
                K = p.shape[1]
                n = (self.bounds[i][r + 1] - self.bounds[i][r]) * K
                self.mat_shard_off[r][i] = so
                if n:
                    segs.append((self.offsets[fqn][0] + self.bounds[i][r] * K, n, so))
                so += _round_up(n, 8)
            so = _round_up(so, 64)
            self.mat_numel.append(so)
            if self.plain_shard:
                segs.append((self.plain_off + r * self.plain_shard, self.plain_shard, so))
            self.segments.append(self._merge(segs))
            self.shard_numels.append(so + self.plain_shard)
        self.mat_cap = max(self.mat_numel)
        self.shard_cap = max(self.shard_numels)
        self.shard_numel = self.shard_numels[rank]
        self.my_segments = self.segments[rank]
        self.plain_shard_off = self.mat_numel[rank]

        self.full = (alloc_full(self.padded) if alloc_full is not None
                     else torch.zeros(self.padded, dtype=compute_dtype, device=device))
        self.master = torch.zeros(self.shard_cap, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = torch.zeros_like(self.master)
        self.grad_full: Optional[torch.Tensor] = None   # whole-group fp32 gradient (collective fallback only)
        self.plain_grad: Optional[torch.Tensor] = None  # fp32 gradient of the plain region (peer-memory mode)
        self.peer_full: Optional[List[torch.Tensor]] = None      # every rank's ``full`` buffer, when peer-visible
        self.plain_stage: Optional[torch.Tensor] = None           # [world-1, plain_shard] slots for plain slices
        self.peer_plain_stage: Optional[List[torch.Tensor]] = None
        self.full_ptrs: Optional[List[int]] = None   # peer-visible addresses of every rank's ``full``
        self.gather_idx: List[int] = []          # matrices whose all-gather happens inside their first forward GEMM
        self.gather_stale: set = set()           # ... and whose remote rows have not been fetched yet in this step
        self.push_segments: List[Tuple[int, int]] = []  # (offset in full, n) pushed to the peers after the step
        self.area: Optional[int] = None          # dedicated staging area of the matrix part (None: from the pool)
        self.area_active: Optional[int] = None   # staging area in use by the current backward pass
        self.area_use: int = -1
        self.params_ready: Optional[torch.cuda.Event] = None
        self.grads_ready: Optional[torch.cuda.Event] = None
        self.reduced = False
        self._tables: Dict[Tuple[int, ...], Tuple] = {}
        for i, (fqn, p) in enumerate(self.params):
            o, n = self.offsets[fqn]
            view = self.full[o:o + n].view(p.shape)
            if p.device.type != "meta":
                view.copy_(p.data)
            # a fresh Parameter: meta / other-device / other-dtype tensors cannot be re-pointed in place
            new_p = nn.Parameter(view, requires_grad=p.requires_grad)
            new_p.grad_written = False
            new_p.tp_sharded = bool(getattr(p, "tp_sharded", False))
            if getattr(p, "lb_fp8", False):  # float8 matmuls were requested for this weight
                new_p.lb_fp8 = True
            self.params[i] = (fqn, new_p)

    @staticmethod
    def _merge(segs: List[Tuple[int, int, int]]) -> List[Tuple[int, int, int]]:
        out: List[Tuple[int, int, int]] = []
        for fo, n, so in segs:
            if out and out[-1][0] + out[-1][1] == fo and out[-1][2] + out[-1][1] == so:
                out[-1] = (out[-1][0], out[-1][1] + n, out[-1][2])
            else:
                out.append((fo, n, so))
        return out

    # -- layout conversions (``flat`` is a [padded] tensor in parameter order)
    def shard_of(self, flat: torch.Tensor, rank: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        r = self.rank if rank is None else rank
        if out is None:
            out = torch.zeros(self.shard_cap, dtype=flat.dtype, device=flat.device)
        for fo, n, so in self.segments[r]:
            out[so:so + n].copy_(flat[fo:fo + n])
        return out

    def unshard_into(self, flat: torch.Tensor, shard: torch.Tensor, rank: int) -> None:
        for fo, n, so in self.segments[rank]:
            flat[fo:fo + n].copy_(shard[so:so + n])

    def classes(self) -> List[Tuple[int, int, int]]:
        """Owned pieces as (offset in shard, n, 0 if the parameter is tensor-parallel sharded else 1), per parameter."""
        out = []
        r = self.rank
        for i, (fqn, p) in enumerate(self.params[:self.n_mats]):
            n = (self.bounds[i][r + 1] - self.bounds[i][r]) * p.shape[1]
            if n:
                out.append((self.mat_shard_off[r][i], n, 0 if p.tp_sharded else 1))
        lo, hi = self.plain_off + r * self.plain_shard, self.plain_off + (r + 1) * self.plain_shard
        for fqn, p in self.params[self.n_mats:]:
            o, n = self.offsets[fqn]
            a, b = max(o, lo), min(o + n, hi)
            if b > a:
                out.append((self.plain_shard_off + a - lo, b - a, 0 if p.tp_sharded else 1))
        # neighbours of one class become one span (the alignment gaps between them hold zeros)
        merged: List[Tuple[int, int, int]] = []
        for so, n, cls in out:
            if merged and merged[-1][2] == cls:
                merged[-1] = (merged[-1][0], so + n - merged[-1][0], cls)
            else:
                merged.append((so, n, cls))
        return merged


class ShardedEngine:
    def __init__(self, model: nn.Module, plan: Sequence[Tuple[str, bool]], process_group=None,
                 compute_dtype: torch.dtype = torch.bfloat16, optim: Optional[EngineOptim] = None,
                 device: Optional[torch.device] = None, p2p_gather: bool = True, replicate_group=None,
                 tp_group=None, scatter_filter: Optional[Callable] = None, accumulate: bool = False,
                 n_pool_areas: int = 3, gather_in_gemm: Optional[Sequence[str]] = None):
        self.model = model
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_initialized() and process_group is not False) else 1
        self.rank = dist.get_rank(process_group) if self.world > 1 else 0
        # outer axis of hybrid sharding: replicas hold the same shard and average their reduced gradients
        self.rep_pg = replicate_group if replicate_group not in (None, False) else None
        self.rep_world = dist.get_world_size(self.rep_pg) if self.rep_pg is not None else 1
        self.tp_pg = tp_group if tp_group not in (None, False) else None
        # Sequence-parallel TP: every TP rank computes the gradients of the replicated weights (norms, embedding,
        # head) from its own rows only, so they are partial sums that still have to be added over the TP group.
        self.tp_partial = False
        self.optim = optim or EngineOptim()
        self.device = device or next(model.parameters()).device
        self.compute_dtype = compute_dtype
        self.is_cuda = self.device.type == "cuda"
        self.step_count = 0
        self.scatter_filter = scatter_filter or default_scatter_filter
        if os.environ.get("LB_SCATTER_IN_GEMM", "1") == "0":
            # every gradient is first written to a local fp32 buffer and its slices are pushed by the copy engines
            self.scatter_filter = lambda fqn, p: False
        # gradient accumulation over micro-batches keeps every group's staging slots alive for the whole step
        self.accumulate = accumulate
        self.n_pool_areas = max(2, n_pool_areas)
        self.reduce_blocks = int(os.environ.get("LB_REDUCE_TRICKLE_BLOCKS", "64"))
        # How the weight-gradient blocks of the ranks are combined at their owner: "slots" - every source rank stores
        # into a slot of its own and one kernel sums the slots in a fixed order (bitwise repeatable); "atomic" - every
        # rank's epilogue adds straight into the owner's gradient shard with TMA reductions (fp32 adds that are atomic
        # at the destination): no staging memory and no slot-sum traffic, but the order of the additions, and with it
        # the last bits of the result, varies from run to run.
        self.grad_mode = os.environ.get("LB_GRAD_REDUCE", "slots")
        assert self.grad_mode in ("slots", "atomic")
        # Which groups leave the all-gather of their first-use weights to the consuming GEMM: those the grouping plan
        # marks ``reshard_after_forward`` (their weights are fetched on demand), all with LB_GATHER_IN_GEMM=1, none
        # with =0. Groups whose weights stay gathered for the whole step (the main app's plan for its blocks) get
        # them pushed by the copy engines right after the optimiser step, which costs no SM time at all and measured
        # about 1 % faster per step at two ranks.
        mode = os.environ.get("LB_GATHER_IN_GEMM", "plan")
        if gather_in_gemm is None:
            gather_in_gemm = () if mode == "0" else DEFAULT_GATHER_IN_GEMM
        self.gather_in_gemm = tuple(gather_in_gemm)
        self.gather_all_groups = mode == "1"
        # True while micro-batches are still being accumulated: a group's backward must not start its
        # gradient reduction before the last micro-batch has added its share
        self.defer_reduce = False
        # side stream: gradient reduction / parameter all-gather, and each group's share of the
        # gradient norm, all of which overlap the backward pass of the groups that are still running
        self.comm_stream = torch.cuda.Stream(self.device, priority=-1) if self.is_cuda else None
        # Peer memory: the compute-dtype buffers and the gradient staging areas live in symmetric memory. Weight
        # gradients are stored into the owners' staging slots by the GEMM epilogue, everything else moves by
        # device-to-device copies (copy engines); a small barrier kernel orders the ranks. Falls back to NCCL /
        # gloo collectives when the group has no peer access.
        self._symm = None
        self._pad_ptrs: Optional[List[int]] = None
        self._barrier_epoch = 0
        self._barrier_events: Dict[int, "torch.cuda.Event"] = {}
        self._use_barrier: Dict[int, int] = {}  # pool use number -> epoch of the barrier in front of its reduction
        self._use_counter = 0
        self._areas: List[torch.Tensor] = []
        self._area_peers: List[List[torch.Tensor]] = []
        self._area_ptrs: List[List[int]] = []
        self._area_cap: List[int] = []
        self._n_pool = 0
        self.collective_path = "none" if self.world == 1 else ("gloo" if not self.is_cuda else "nccl")
        if self.is_cuda and self.world > 1 and p2p_gather:
            try:
                import torch.distributed._symmetric_memory as sm

                pad = sm.empty(8, dtype=torch.int32, device=self.device)
                pad.zero_()
                hdl = sm.rendezvous(pad, group=self._group())
                self._symm, self._pad = sm, pad
                self._pad_ptrs = [int(p) for p in hdl.buffer_ptrs]
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.pg)  # every pad is zero before the first barrier kernel runs
                self.collective_path = "p2p scatter"
            except Exception as e:  # no peer access inside this group: collectives of the process group
                logger.warning("peer-to-peer collectives disabled: %s", e)
                self._symm = None

        taken = set()
        self.groups: List[ParamGroup] = []
        self.group_of_module: Dict[str, int] = {}
        self._mark_tp_params(model)
        for path, reshard in plan:
            mod = model.get_submodule(path)
            ps = [(f"{path}.{n}", p) for n, p in mod.named_parameters() if f"{path}.{n}" not in taken]
            taken.update(fqn for fqn, _ in ps)
            if ps:
                self._add_group(path, ps, gather_on_demand=bool(reshard) or self.gather_all_groups)
        rest = [(n, p) for n, p in model.named_parameters() if n not in taken]
        if rest:
            self._add_group("", rest, gather_on_demand=self.gather_all_groups)
        if self._symm is not None and self.grad_mode == "slots":
            self._setup_areas()
        # squared gradient norm per group, split into [tensor-parallel sharded, replicated inside a TP group]
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.sumsq_parts = torch.zeros(len(self.groups), 2, dtype=torch.float32, device=self.device)
        self.n_params = sum(g.numel for g in self.groups)
        logger.info("sharded engine: %d groups, world %d (x%d replicas), collectives: %s", len(self.groups), self.world,
                    self.rep_world, self.collective_path)

    def _group(self):
        return self.pg if self.pg not in (None, False) else dist.group.WORLD

    @staticmethod
    def _mark_tp_params(model: nn.Module) -> None:
        for mod in model.modules():
            if getattr(mod, "tp_shard", None) is not None:
                for p in mod._parameters.values():
                    if p is not None and p.dim() >= 2:
                        p.tp_sharded = True

    @property
    def p2p(self) -> bool:
        return self._symm is not None

    def _symm_tensor(self, n: int, dtype: torch.dtype):
        t = self._symm.empty(n, dtype=dtype, device=self.device)
        t.zero_()
        hdl = self._symm.rendezvous(t, group=self._group())
        return t, hdl

    def _add_group(self, path: str, ps: List[Tuple[str, nn.Parameter]], gather_on_demand: bool = False) -> None:
        self.group_of_module[path] = len(self.groups)
        holder = {}
        alloc = None
        if self._symm is not None:
            def alloc(n):
                holder["t"], holder["h"] = self._symm_tensor(n, self.compute_dtype)
                return holder["t"]
        g = ParamGroup(path, ps, self.world, self.rank, self.compute_dtype, self.device, self.scatter_filter,
                       alloc_full=alloc)
        W = self.world
        if self._symm is not None:
            g.peer_full = [holder["h"].get_buffer(r, (g.padded,), self.compute_dtype) for r in range(W)]
            g.full_ptrs = [int(p) for p in holder["h"].buffer_ptrs]
            if self.grad_mode == "atomic" and g.mat_cap:
                g.grad_shard, hg = self._symm_tensor(g.shard_cap, torch.float32)
                g.grad_shard_ptrs = [int(p) for p in hg.buffer_ptrs]
                g.peer_grad_shard = [hg.get_buffer(r, (g.shard_cap,), torch.float32) for r in range(W)]
            if g.plain_shard:
                g.plain_grad = torch.zeros(g.plain_padded, dtype=torch.float32, device=self.device)
                g.plain_stage, h2 = self._symm_tensor((W - 1) * g.plain_shard, torch.float32)
                g.peer_plain_stage = [h2.get_buffer(r, (W - 1, g.plain_shard), torch.float32) for r in range(W)]
        elif W > 1:
            g.grad_full = torch.zeros(g.padded, dtype=torch.float32, device=self.device)
        for i, (fqn, p) in enumerate(g.params):
            o, n = g.offsets[fqn]
            if W == 1:
                p.main_grad = g.grad_shard[o:o + n].view(p.shape)  # one rank: the shard is the whole buffer
            elif g.grad_full is not None:
                p.main_grad = g.grad_full[o:o + n].view(p.shape)
            elif i >= g.n_mats:
                p.main_grad = g.plain_grad[o - g.plain_off:o - g.plain_off + n].view(p.shape)
            else:
                p.lb_scatter = ScatterTarget(self, g, i)
                stem = fqn[:-len(".weight")] if fqn.endswith(".weight") else fqn
                if (gather_on_demand and any(stem.endswith(pat) for pat in self.gather_in_gemm) and p.shape[0] % BLOCK_ROWS == 0
                        and p.shape[1] % 64 == 0 and self.compute_dtype == torch.bfloat16):
                    p.lb_gather = p.lb_scatter
                    g.gather_idx.append(i)
            owner_path, _, attr = fqn.rpartition(".")
            self.model.get_submodule(owner_path)._parameters[attr] = p
        # what the copy engines push after a step: this rank's pieces of everything that is not gathered in a GEMM
        r = self.rank
        for i, (fqn, p) in enumerate(g.params[:g.n_mats]):
            n = (g.bounds[i][r + 1] - g.bounds[i][r]) * p.shape[1]
            if n and i not in g.gather_idx:
                g.push_segments.append((g.offsets[fqn][0] + g.bounds[i][r] * p.shape[1], n))
        if g.plain_shard:
            g.push_segments.append((g.plain_off + r * g.plain_shard, g.plain_shard))
        g.push_segments = [(fo, n) for fo, n, _ in ParamGroup._merge([(fo, n, fo) for fo, n in g.push_segments])]
        self.groups.append(g)

    # -- parameter all-gather inside the first forward GEMM
    def gather_plan(self, targets: Sequence[ScatterTarget]):
        """(GatherPlan, peer addresses of the fused weight) for adjacent gather parameters, or None."""
        from ..ops.gemm import GatherPlan

        g = targets[0].group
        idx = [t.index for t in targets]
        if any(t.group is not g for t in targets) or idx != list(range(idx[0], idx[0] + len(idx))):
            return None
        mats = [g.params[i][1] for i in idx]
        K = mats[0].shape[1]
        if any(m.shape[1] != K or m.shape[0] % BLOCK_ROWS or m.numel() % 8 for m in mats) or g.full_ptrs is None:
            return None
        key = ("gather",) + tuple(idx)
        plan = g._tables.get(key)
        if plan is None:
            owners = []
            for i, m in zip(idx, mats):
                b = g.bounds[i]
                owners += [max(r for r in range(self.world) if b[r] <= blk * BLOCK_ROWS)
                           for blk in range(m.shape[0] // BLOCK_ROWS)]
            plan = GatherPlan(owners, self.rank, self.world, K, self.device)
            g._tables[key] = plan
        off = g.offsets[g.params[idx[0]][0]][0] * g.full.element_size()
        return plan, [ptr + off for ptr in g.full_ptrs]

    def gather_is_stale(self, targets: Sequence[ScatterTarget]) -> bool:
        return any(t.index in t.group.gather_stale for t in targets)

    def mark_gathered(self, targets: Sequence[ScatterTarget]) -> None:
        for t in targets:
            t.group.gather_stale.discard(t.index)

    def ensure_gathered(self, targets: Sequence[ScatterTarget]) -> None:
        """Fetch the remote rows of gather parameters that some consumer other than the fused GEMM needs (a float8
        quantiser, an evaluation path): plain peer -> local copies on the current stream."""
        for t in targets:
            g, i = t.group, t.index
            if i not in g.gather_stale:
                continue
            fqn, p = g.params[i]
            K = p.shape[1]
            for o in range(self.world):
                if o == self.rank:
                    continue
                r0, r1 = g.bounds[i][o], g.bounds[i][o + 1]
                if r1 > r0:
                    lo = g.offsets[fqn][0] + r0 * K
                    g.full[lo:lo + (r1 - r0) * K].copy_(g.peer_full[o][lo:lo + (r1 - r0) * K], non_blocking=True)
            g.gather_stale.discard(i)

    def _setup_areas(self) -> None:
        """Staging areas for the matrix gradients: [world-1 slots] x [largest matrix shard]. Groups of the most
        common size rotate through a small pool (a slot is free again once every owner has reduced it); the
        others, and every group when micro-batches are accumulated, get an area of their own."""
        sizes: Dict[int, int] = {}
        for g in self.groups:
            if g.mat_cap:
                sizes[g.mat_cap] = sizes.get(g.mat_cap, 0) + 1
        if not sizes:
            return
        pool_cap = max(sizes, key=lambda s: sizes[s] * s)
        use_pool = (not self.accumulate) and sizes[pool_cap] > self.n_pool_areas

        def new_area(cap: int) -> int:
            t, h = self._symm_tensor((self.world - 1) * cap, torch.float32)
            self._areas.append(t)
            self._area_peers.append([h.get_buffer(r, (self.world - 1, cap), torch.float32) for r in range(self.world)])
            self._area_ptrs.append([int(p) for p in h.buffer_ptrs])
            self._area_cap.append(cap)
            return len(self._areas) - 1

        if use_pool:
            for _ in range(self.n_pool_areas):
                new_area(pool_cap)
        for g in self.groups:
            if g.mat_cap and not (use_pool and g.mat_cap == pool_cap):
                g.area = new_area(g.mat_cap)
        self._n_pool = self.n_pool_areas if use_pool else 0

    # ------------------------------------------------------------------ init / state
    def sync_master(self) -> None:
        """Call after (re-)initialising or loading the compute-dtype weights."""
        for g in self.groups:
            g.shard_of(g.full.float(), out=g.master)

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
            g.shard_of(buf, out=g.master)
            g.full.copy_(buf)
            for fqn, p in g.params:
                o, n = g.offsets[fqn]
                p.data = g.full[o:o + n].view(p.shape)
        del fp32_bufs

    def load_group_fp32(self, gi: int, flat: torch.Tensor, which: str = "master") -> None:
        """Take this rank's share of a whole-group fp32 tensor in parameter order (``which``: master, exp_avg,
        exp_avg_sq); the master weights also refresh the compute-dtype buffer."""
        g = self.groups[gi]
        g.shard_of(flat, out=getattr(g, which))
        if which == "master":
            g.full.copy_(flat)
            from .. import float8

            float8.new_weight_epoch()

    def export_group_fp32(self, gi: int, which: str = "master") -> torch.Tensor:
        """The whole group's fp32 tensor in parameter order, assembled from every rank's shard."""
        g = self.groups[gi]
        shard = getattr(g, which)
        flat = torch.zeros(g.padded, dtype=torch.float32, device=self.device)
        if self.world == 1:
            g.unshard_into(flat, shard, 0)
            return flat
        gathered = torch.empty(self.world * g.shard_cap, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(gathered, shard.contiguous(), group=self.pg)
        for r in range(self.world):
            g.unshard_into(flat, gathered[r * g.shard_cap:(r + 1) * g.shard_cap], r)
        return flat

    def full_tensor_fp32(self, gi: int) -> torch.Tensor:
        return self.export_group_fp32(gi, "master")

    # ------------------------------------------------------------------ per-step protocol
    def zero_grad(self) -> None:
        for g in self.groups:
            g.reduced = False
            g.area_active = None  # a backward pass whose gradients were discarded may have left an area assigned
            for _, p in g.params:
                p.grad_written = False
                p.grad = None

    def wait_params(self, gi: int) -> None:
        """Block the compute stream until group gi's all-gathered weights have landed."""
        g = self.groups[gi]
        if g.params_ready is not None:
            torch.cuda.current_stream().wait_event(g.params_ready)
            g.params_ready = None

    # -- scatter targets (called by the weight-gradient emitters of ops/fused.py)
    def _acquire_area(self, g: ParamGroup) -> int:
        """Staging area the current backward pass of ``g`` writes into. A pool area is handed out in rotation;
        before this rank stores into it again the compute stream waits until every owner has reduced the
        area's previous contents, which is known once the barrier that followed that reduction has been passed."""
        if g.area_active is not None:
            return g.area_active
        if g.area is not None:
            g.area_active = g.area
            return g.area
        u = self._use_counter
        self._use_counter += 1
        prev = u - self._n_pool
        if prev >= 0:
            k = self._use_barrier.pop(prev, None)
            ev = self._barrier_events.get(k + 1) if k is not None else None
            if ev is None:
                # the reduction of the previous user has not been followed by a barrier yet (should not happen with
                # two or more pool areas): close the gap with one of its own
                with torch.cuda.stream(self.comm_stream):
                    self._peer_barrier()
                ev = self._barrier_events[self._barrier_epoch]
            torch.cuda.current_stream().wait_event(ev)
            for old in [e for e in self._barrier_events if e < (k or 0)]:
                del self._barrier_events[old]
        g.area_active, g.area_use = u % self._n_pool, u
        return g.area_active

    def scatter_plan(self, targets: Sequence[ScatterTarget]):
        """(block table, destination pointers, destination rows, row pitch, first tile) for the fused weight-gradient
        GEMM of adjacent scatter parameters, or None when they cannot share one GEMM."""
        g = targets[0].group
        idx = [t.index for t in targets]
        if any(t.group is not g for t in targets) or idx != list(range(idx[0], idx[0] + len(idx))):
            return None
        mats = [g.params[i][1] for i in idx]
        K = mats[0].shape[1]
        if any(m.shape[1] != K for m in mats) or any(m.shape[0] % BLOCK_ROWS for m in mats[:-1]):
            return None
        key = tuple(idx)
        cached = g._tables.get(key)
        if cached is None:
            W = self.world
            rows = [sum(g.bounds[i][o + 1] - g.bounds[i][o] for i in idx) for o in range(W)]
            table = []
            before = [0] * W
            for i, m in zip(idx, mats):
                b = g.bounds[i]
                for blk in range((m.shape[0] + BLOCK_ROWS - 1) // BLOCK_ROWS):
                    r0 = blk * BLOCK_ROWS
                    o = max(r for r in range(W) if b[r] <= r0)
                    table.append((o, before[o] + r0 - b[o]))
                for o in range(W):
                    before[o] += b[o + 1] - b[o]
            blocks = torch.tensor(table, dtype=torch.int32, device=self.device)
            # start the walk over row tiles with the next rank's rows: what has to travel goes first
            nxt = (self.rank + 1) % W
            first_blk = next((j for j, (o, _) in enumerate(table) if o == nxt), 0)
            cached = (blocks, rows, K, first_blk // 2)
            g._tables[key] = cached
        blocks, rows, K, m_rot = cached
        if self.grad_mode == "atomic":
            g.area_active = -1  # marks the group as having contributions in flight
            return blocks, [p + g.mat_shard_off[o][idx[0]] * 4 for o, p in enumerate(g.grad_shard_ptrs)], rows, K, m_rot
        a = self._acquire_area(g)
        cap = self._area_cap[a]
        ptrs = []
        for o in range(self.world):
            off = g.mat_shard_off[o][idx[0]]
            if o == self.rank:
                ptrs.append(g.grad_shard.data_ptr() + off * 4)
            else:
                slot = (o - self.rank) % self.world - 1  # slot k-1 of rank o receives from rank o - k
                ptrs.append(self._area_ptrs[a][o] + (slot * cap + off) * 4)
        return blocks, ptrs, rows, K, m_rot

    def _push_scatter_fallback(self, g: ParamGroup, i: int, grad: Optional[torch.Tensor], accumulate: bool) -> None:
        """A scatter parameter whose gradient did not come out of the fused GEMM (plain autograd, or no gradient at
        all): deliver its row slabs with device-to-device copies so that every slot holds defined data."""
        fqn, p = g.params[i]
        K = p.shape[1]
        gf = None if grad is None else grad.to(torch.float32).contiguous()
        if self.grad_mode == "atomic":
            g.area_active = -1
            if gf is not None:  # nothing to deliver for a parameter without a gradient: the shards start at zero
                from ..ops import _lib

                lib = _lib.load()
                import ctypes as C

                lib.lb_red_add.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]
                lib.lb_red_add.restype = C.c_int
                for o in range(self.world):
                    r0, r1 = g.bounds[i][o], g.bounds[i][o + 1]
                    if r1 > r0:
                        dst = g.grad_shard_ptrs[o] + g.mat_shard_off[o][i] * 4
                        _lib.check(lib.lb_red_add(dst, gf[r0:r1].data_ptr(), (r1 - r0) * K, _lib.stream_ptr()), "lb_red_add")
            return
        a = self._acquire_area(g)
        for o in range(self.world):
            r0, r1 = g.bounds[i][o], g.bounds[i][o + 1]
            n = (r1 - r0) * K
            if not n:
                continue
            off = g.mat_shard_off[o][i]
            if o == self.rank:
                dst = g.grad_shard[off:off + n]
            else:
                dst = self._area_peers[a][o][(o - self.rank) % self.world - 1, off:off + n]
            if gf is None:
                if not accumulate:
                    dst.zero_()
            elif accumulate:
                tmp = torch.empty(n, dtype=torch.float32, device=self.device)
                tmp.copy_(dst)          # copy engine: peer -> local
                tmp.add_(gf[r0:r1].reshape(-1))
                dst.copy_(tmp)
            else:
                dst.copy_(gf[r0:r1].reshape(-1))

    def _flush_autograd_grads(self, g: ParamGroup) -> None:
        """Reference-path modules produce ``p.grad``; fold those into the engine's fp32 buffers."""
        for i, (_, p) in enumerate(g.params):
            if hasattr(p, "main_grad"):
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
            elif p.grad is not None or not p.grad_written:
                self._push_scatter_fallback(g, i, p.grad, p.grad_written)
                p.grad_written = True
                p.grad = None

    def _sumsq_classes(self, g: ParamGroup, gi: int) -> None:
        for so, n, cls in g.classes():
            F.sumsq(g.grad_shard[so:so + n], self.sumsq_parts[gi, cls:cls + 1])

    def _uniform_class(self, g: ParamGroup, lo: int, hi: int) -> Optional[int]:
        cls = {(0 if p.tp_sharded else 1) for _, p in g.params[lo:hi]}
        return cls.pop() if len(cls) == 1 else None

    def reduce_group(self, gi: int) -> None:
        """Reduce-scatter (mean) group gi's gradients into ``grad_shard``; asynchronous on CUDA."""
        g = self.groups[gi]
        if g.reduced:
            return
        g.reduced = True
        parts = self.sumsq_parts[gi]
        W = self.world
        if self.comm_stream is not None:
            if self.p2p:
                self._flush_autograd_grads(g)  # may issue copies into peers' slots: before the barrier below
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                parts.zero_()
                fused_norm = self.rep_world == 1 and not self.tp_partial
                if self.p2p:
                    ps = g.plain_shard
                    for k in range(1, W):
                        if ps:
                            r = (self.rank + k) % W
                            g.peer_plain_stage[r][k - 1].copy_(g.plain_grad[r * ps:(r + 1) * ps], non_blocking=True)
                    self._peer_barrier()
                    # groups that are followed by more backward work have a layer's time for their slot sum: a small
                    # grid keeps it from competing with the GEMMs; the last ones are on the critical path
                    trickle = self.reduce_blocks if gi >= 2 else 0
                    if g.area_active is not None and self.grad_mode == "atomic":
                        # every rank's additions into this shard have landed (barrier): scale and take the norm
                        n = g.mat_numel[self.rank]
                        cls = self._uniform_class(g, 0, g.n_mats) if fused_norm else None
                        if n:
                            self._reduce_slots(g.grad_shard[:n], None, 0, g.grad_shard[:n],
                                               None if cls is None else parts[cls:cls + 1], trickle, n_slots=0)
                        fused_norm = fused_norm and cls is not None
                        g.area_active = None
                    elif g.area_active is not None:
                        if g.area is None:
                            self._use_barrier[g.area_use] = self._barrier_epoch
                        n = g.mat_numel[self.rank]
                        cls = self._uniform_class(g, 0, g.n_mats) if fused_norm else None
                        if n:
                            self._reduce_slots(g.grad_shard[:n], self._areas[g.area_active], self._area_cap[g.area_active],
                                               g.grad_shard[:n], None if cls is None else parts[cls:cls + 1], trickle)
                        fused_norm = fused_norm and cls is not None
                        g.area_active = None
                    if ps:
                        cls = self._uniform_class(g, g.n_mats, len(g.params)) if fused_norm else None
                        o = g.plain_shard_off
                        self._reduce_slots(g.plain_grad[self.rank * ps:(self.rank + 1) * ps], g.plain_stage, ps,
                                           g.grad_shard[o:o + ps], None if cls is None else parts[cls:cls + 1])
                        fused_norm = fused_norm and cls is not None
                else:
                    self._flush_autograd_grads(g)
                    self._reduce_by_collective(g)
                    fused_norm = False
                if self.rep_world > 1:
                    dist.all_reduce(g.grad_shard, op=dist.ReduceOp.SUM, group=self.rep_pg)
                    g.grad_shard.mul_(1.0 / self.rep_world)
                self._sum_tp_partials(g)
                if not fused_norm:
                    parts.zero_()
                    self._sumsq_classes(g, gi)
                g.grads_ready = torch.cuda.Event()
                g.grads_ready.record(self.comm_stream)
            return
        self._flush_autograd_grads(g)
        self._reduce_by_collective(g)
        if self.rep_world > 1:
            dist.all_reduce(g.grad_shard, op=dist.ReduceOp.SUM, group=self.rep_pg)
            g.grad_shard.mul_(1.0 / self.rep_world)
        self._sum_tp_partials(g)
        parts.zero_()
        self._sumsq_classes(g, gi)

    def _sum_tp_partials(self, g: ParamGroup) -> None:
        """Add up, over the TP group, this rank's shard of the gradients of weights that are replicated inside it
        (sequence-parallel training only; after the data-parallel reduction, so only shard-sized pieces travel)."""
        if not self.tp_partial or self.tp_pg is None:
            return
        for so, n, cls in g.classes():
            if cls == 1:
                dist.all_reduce(g.grad_shard[so:so + n], op=dist.ReduceOp.SUM, group=self.tp_pg)

    def _reduce_by_collective(self, g: ParamGroup) -> None:
        """Fallback without peer memory: all-reduce the whole-group gradient and keep the owned pieces."""
        if self.world == 1:
            return  # gradients were written into the shard directly
        dist.all_reduce(g.grad_full, op=dist.ReduceOp.SUM, group=self.pg)
        g.shard_of(g.grad_full, out=g.grad_shard)
        g.grad_shard.mul_(1.0 / self.world)

    def step(self, lr: float, grad_mul: float = 1.0) -> torch.Tensor:
        """Finish gradient reduction, clip by global norm, AdamW on the owned pieces, re-gather.
        Returns the (pre-clip) gradient norm as a device tensor."""
        for gi in range(len(self.groups) - 1, -1, -1):
            self.reduce_group(gi)
        for g in self.groups:
            if g.grads_ready is not None:
                torch.cuda.current_stream().wait_event(g.grads_ready)
                g.grads_ready = None
        tot = self.sumsq_parts.sum(dim=0)  # [sharded over the TP group, replicated inside it]
        if self.tp_pg is not None:
            sharded = tot[0:1].clone()
            dist.all_reduce(sharded, op=dist.ReduceOp.SUM, group=self.tp_pg)
            torch.add(sharded, tot[1:2], out=self.sumsq)
        else:
            torch.sum(tot, dim=0, keepdim=True, out=self.sumsq)
        if self.world > 1:
            dist.all_reduce(self.sumsq, op=dist.ReduceOp.SUM, group=self.pg)
        self.step_count += 1
        from .. import float8

        float8.new_weight_epoch()  # quantised copies of the weights are stale from here on
        o = self.optim
        for g in self.groups:
            for fo, n, so in g.my_segments:
                F.adamw_step(g.master[so:so + n], g.exp_avg[so:so + n], g.exp_avg_sq[so:so + n], g.grad_shard[so:so + n],
                             g.full[fo:fo + n], step=self.step_count, lr=lr, beta1=o.beta1, beta2=o.beta2, eps=o.eps,
                             wd=o.weight_decay, sumsq_t=self.sumsq, max_norm=o.clip, grad_mul=grad_mul)
            if self.world > 1:
                if self.grad_mode == "atomic" and self.p2p and g.mat_cap:
                    # the shard starts the next step at zero; the barrier of the gather below tells every peer so
                    g.grad_shard[:g.mat_numel[self.rank]].zero_()
                self._gather_group(g)  # overlaps the AdamW launches of the groups that follow
        return self.sumsq.sqrt() * grad_mul

    def gather_params(self) -> None:
        """All-gather every group's compute-dtype pieces into its full buffer (in group order, so
        the first layers of the next forward are ready first)."""
        if self.world == 1:
            return
        for g in self.groups:
            self._gather_group(g)

    def _gather_group(self, g: ParamGroup) -> None:
        """In-place all-gather of one group (every rank's pieces already sit at their place in ``g.full``);
        on CUDA it runs on the side stream after everything queued so far on the compute stream."""
        if self.comm_stream is not None:
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(done)
            with torch.cuda.stream(self.comm_stream):
                if g.peer_full is not None:
                    for k in range(1, self.world):  # start with the next rank so that links are used evenly
                        r = (self.rank + k) % self.world
                        for fo, n in g.push_segments:
                            g.peer_full[r][fo:fo + n].copy_(g.full[fo:fo + n], non_blocking=True)
                    # every rank's pushes, mine included, have landed, and every rank's own rows of the matrices
                    # that are gathered inside their first GEMM are final
                    self._peer_barrier()
                    g.gather_stale = set(g.gather_idx)
                else:
                    self._gather_by_collective(g)
                g.params_ready = torch.cuda.Event()
                g.params_ready.record(self.comm_stream)
        else:
            self._gather_by_collective(g)

    def _gather_by_collective(self, g: ParamGroup) -> None:
        mine = g.shard_of(g.full)
        gathered = torch.empty(self.world * g.shard_cap, dtype=g.full.dtype, device=self.device)
        dist.all_gather_into_tensor(gathered, mine, group=self.pg)
        for r in range(self.world):
            if r != self.rank:
                g.unshard_into(g.full, gathered[r * g.shard_cap:(r + 1) * g.shard_cap], r)

    def _reduce_slots(self, own: torch.Tensor, slots: Optional[torch.Tensor], slot_stride: int, out: torch.Tensor,
                      part: Optional[torch.Tensor], max_blocks: int = 0, n_slots: Optional[int] = None) -> None:
        import ctypes as C

        from ..ops import _lib

        lib = _lib.load()
        if not getattr(lib, "_reduce_slots_declared", False):
            lib.lb_reduce_slots_grid.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p,
                                                 C.c_longlong, C.c_float, C.c_void_p, C.c_int, C.c_void_p]
            lib.lb_reduce_slots_grid.restype = C.c_int
            lib._reduce_slots_declared = True
        rc = lib.lb_reduce_slots_grid(own.data_ptr(), None if slots is None else slots.data_ptr(),
                                      self.world - 1 if n_slots is None else n_slots, slot_stride, out.data_ptr(),
                                      own.numel(), 1.0 / self.world, None if part is None else part.data_ptr(),
                                      max_blocks, _lib.stream_ptr())
        _lib.check(rc, "lb_reduce_slots")

    def _peer_barrier(self) -> None:
        from .tp_fused import peer_barrier

        self._barrier_epoch += 1
        # ranks of a training job drift (data loading, logging, checkpoints): generous but finite limit
        peer_barrier(self._pad_ptrs, self.rank, self._barrier_epoch,
                     limit_s=float(os.environ.get("LB_BARRIER_LIMIT_S", "120")))
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self._barrier_events[self._barrier_epoch] = ev
        if len(self._barrier_events) > 4096:
            for old in sorted(self._barrier_events)[:2048]:
                del self._barrier_events[old]

    def wait_all_params(self) -> None:
        for gi in range(len(self.groups)):
            self.wait_params(gi)

    def finish_param_gather(self) -> None:
        """Make every rank's compute-dtype buffers complete now: wait for the pushes that are in flight and fetch the
        rows of the matrices whose all-gather is otherwise left to their first forward GEMM. For consumers that read
        the weights outside the model's forward pass."""
        self.wait_all_params()
        for g in self.groups:
            if g.gather_stale:
                self.ensure_gathered([g.params[i][1].lb_gather for i in sorted(g.gather_stale)])

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
