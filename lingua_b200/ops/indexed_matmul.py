"""Position-indexed ("multi-linear") projection: ``Y[t] = X[t] @ W[idx[t]]^T`` with a small bank of weights.

The hierarchical byte model upsamples a pooled vector back to the bytes it covers and gives each byte a
projection chosen by its distance to the pooled position (apps/aunet/index_matmul.py:12-91 of the reference,
which loops over the bank with a boolean ``torch.where`` -- a host synchronisation -- per weight in forward
and again in backward).

Here the rows are sorted by index once (``plan_groups``: one stable argsort and one bincount on the device).
On the GPU the sorted rows are laid out group by group, each group padded to the 256-row tile of the SM-pair
GEMM kernel, and forward, input gradient and weight gradients are one grouped launch each: the kernel picks
the weight of a row tile (or the row range of a weight's gradient) from a small device table, so the group
sizes never travel to the host. On the CPU, or for an fp32 model, the same plan drives a loop of plain
products over the contiguous row ranges (one device-to-host read of the sizes). A plan is built once per
step and shared by forward and backward and by every call that uses the same indices."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from . import gemm as _g


def _route(fn):
    """bf16 goes to the tcgen05 GEMM; an fp32 reference model on the GPU uses the plain fp32 product."""
    def run(a, b, **kw):
        if a.is_cuda and a.dtype != torch.bfloat16:
            at, bt = {"mm_nt": (a, b), "mm_nn": (a, b.transpose(-1, -2)),
                      "mm_tn": (a.transpose(-1, -2), b.transpose(-1, -2))}[fn.__name__]
            return _g.gemm_ref(at, bt, kw.get("out_dtype", a.dtype), kw.get("out"), kw.get("accumulate", False))
        return fn(a, b, **kw)
    return run


mm_nt, mm_nn, mm_tn = _route(_g.mm_nt), _route(_g.mm_nn), _route(_g.mm_tn)


@dataclass
class GroupPlan:
    """Row grouping of one index tensor. ``counts`` (host) drives the per-group loop; ``prow`` / ``pos`` /
    ``sel`` / ``k_range`` (device) drive the single-launch grouped kernels and never reach the host."""
    order: torch.Tensor  # [T] int64: rows in group order (stable)
    n: int
    counts_dev: torch.Tensor  # [n] int64 rows per group
    prow: Optional[torch.Tensor] = None  # [T] int64: row of the i-th sorted row in the padded group layout
    pos: Optional[torch.Tensor] = None  # [T] int64: padded row of original row t
    sel: Optional[torch.Tensor] = None  # [padded_rows / 256] int32: group of each 256-row tile
    k_range: Optional[torch.Tensor] = None  # [n, 2] int32: (first padded row, padded rows / 64) per group
    padded_rows: int = 0  # upper bound known without reading the group sizes
    _counts: Optional[List[int]] = None

    @property
    def counts(self) -> List[int]:
        """Rows per group on the host (one device-to-host read, cached)."""
        if self._counts is None:
            self._counts = [int(c) for c in self.counts_dev.tolist()]
        return self._counts

    @property
    def grouped(self) -> bool:
        return self.sel is not None

    @property
    def segments(self):
        o = 0
        for g, c in enumerate(self.counts):
            if c:
                yield g, o, c
            o += c


def _native_grouped(t: torch.Tensor) -> bool:
    from . import _lib
    return t.is_cuda and _lib.available()


def plan_groups(indices: torch.Tensor, n: int, grouped: Optional[bool] = None) -> GroupPlan:
    """Sort rows by index. With ``grouped`` (default: on a GPU with the native library) also lay the sorted rows
    out with every group padded to the grouped kernel's 256-row tile, all on the device."""
    flat = indices.reshape(-1)
    T = flat.numel()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n)
    plan = GroupPlan(order=order, n=n, counts_dev=counts)
    if grouped is None:
        grouped = _native_grouped(flat)
    if grouped:
        R = _g.GROUP_ROWS
        padded = (counts + (R - 1)) // R * R
        pend = torch.cumsum(padded, 0)
        poff = pend - padded
        start = torch.cumsum(counts, 0) - counts
        sidx = flat.index_select(0, order)
        plan.prow = poff.index_select(0, sidx) + (torch.arange(T, device=flat.device) - start.index_select(0, sidx))
        plan.pos = torch.empty_like(plan.prow)
        plan.pos.index_copy_(0, order, plan.prow)
        plan.padded_rows = (T + n * (R - 1) + R - 1) // R * R
        tiles = torch.arange(plan.padded_rows // R, device=flat.device) * R
        sel = torch.searchsorted(pend, tiles, right=True)
        plan.sel = torch.where(sel < n, sel, -1).to(torch.int32)  # -1: a tile past the last group, skipped
        plan.k_range = torch.stack((poff, padded // 64), dim=1).to(torch.int32).contiguous()
    return plan


def indexed_matmul_ref(x: torch.Tensor, w: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """fp32 oracle: gathers one weight per row."""
    x2 = x.reshape(-1, x.shape[-1]).float()
    y = torch.einsum("td,tod->to", x2, w.float()[indices.reshape(-1)])
    return y.view(*x.shape[:-1], w.shape[1])


def _use_grouped(x2d: torch.Tensor, w: torch.Tensor, plan: GroupPlan) -> bool:
    return (plan.grouped and x2d.is_cuda and x2d.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.is_contiguous() and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0)


class IndexedMatMulFn(torch.autograd.Function):
    """``rows`` (optional, [T] int64): output row t reads input row ``rows[t]`` -- the repeat-upsampling gather
    folded into the sort, so the repeated activations are never materialised in input order.

    On the GPU in bf16 each direction is ONE launch of the SM-pair GEMM in grouped mode (``gemm_grouped_rows``
    for forward and the input gradient, ``gemm_grouped_k`` for the weight gradients) over the padded group
    layout of the plan; otherwise a loop over the groups with plain products."""

    @staticmethod
    def forward(ctx, x2d, w, plan: GroupPlan, rows=None):
        src = plan.order if rows is None else rows.index_select(0, plan.order)
        ctx.plan, ctx.n_in, ctx.permutation = plan, x2d.shape[0], rows is None
        ctx.use_grouped = _use_grouped(x2d, w, plan)
        if ctx.use_grouped:
            xs = torch.zeros(plan.padded_rows, x2d.shape[1], dtype=x2d.dtype, device=x2d.device)
            xs.index_copy_(0, plan.prow, x2d.index_select(0, src))
            ys = _g.gemm_grouped_rows(xs, w, plan.sel)
            y = ys.index_select(0, plan.pos)
        else:
            xs = x2d.index_select(0, src)
            ys = torch.empty(xs.shape[0], w.shape[1], dtype=x2d.dtype, device=x2d.device)
            for g, o, c in plan.segments:
                mm_nt(xs[o:o + c], w[g], out=ys[o:o + c], out_dtype=x2d.dtype)
            y = torch.empty_like(ys)
            y.index_copy_(0, plan.order, ys)
        ctx.save_for_backward(xs, w, src)
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, w, src = ctx.saved_tensors
        plan: GroupPlan = ctx.plan
        main = getattr(w, "main_grad", None)  # fp32 gradient buffer of a training engine, if any
        acc = main is not None and getattr(w, "grad_written", False)
        if ctx.use_grouped:
            dys = torch.zeros(plan.padded_rows, dy.shape[1], dtype=dy.dtype, device=dy.device)
            dys.index_copy_(0, plan.pos, dy)
            dxs = _g.gemm_grouped_rows(dys, w, plan.sel, transpose_bank=True).index_select(0, plan.prow)
            if main is not None and main.is_contiguous():
                _g.gemm_grouped_k(dys, xs, plan.k_range, main, accumulate=acc)
                dw = None
            else:
                dw = _g.gemm_grouped_k(dys, xs, plan.k_range, torch.empty(w.shape, dtype=torch.float32, device=w.device))
                if main is not None:
                    main.add_(dw) if acc else main.copy_(dw)
                    dw = None
        else:
            dys = dy.index_select(0, plan.order)
            dxs = torch.empty_like(xs)
            dw = None if main is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            if main is not None and not acc:
                main.zero_()  # groups without rows keep a zero gradient
            for g, o, c in plan.segments:
                mm_nn(dys[o:o + c], w[g], out=dxs[o:o + c], out_dtype=dxs.dtype)
                mm_tn(dys[o:o + c], xs[o:o + c], out=(main if main is not None else dw)[g], accumulate=True,
                      out_dtype=torch.float32)
        if main is not None:
            w.grad_written = True
        if ctx.permutation:
            dx = torch.empty_like(dxs)
            dx.index_copy_(0, src, dxs)
        else:  # several output rows per input row: sum them (fp32, then back to the activation dtype)
            dx = torch.zeros(ctx.n_in, dxs.shape[1], dtype=torch.float32, device=dxs.device)
            dx.index_add_(0, src, dxs.float())
            dx = dx.to(dxs.dtype)
        return dx, (None if main is not None else dw.to(w.dtype)), None, None


def indexed_matmul(x: torch.Tensor, w: torch.Tensor, indices: torch.Tensor, plan: Optional[GroupPlan] = None,
                   rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [..., in], w [n, out, in], indices [...] in [0, n) -> [..., out]. With ``rows`` (same shape as
    ``indices``, values index the flattened rows of x) the result is ``x.flatten(0, -2)[rows] @ w[indices]^T``."""
    plan = plan or plan_groups(indices, w.shape[0])
    y = IndexedMatMulFn.apply(x.reshape(-1, x.shape[-1]), w, plan, None if rows is None else rows.reshape(-1))
    return y.view(*indices.shape, w.shape[1])


class IndexedMatMul(nn.Module):
    def __init__(self, num_linear: int, in_features: int, out_features: int):
        super().__init__()
        self.num_linear, self.in_features, self.out_features = num_linear, in_features, out_features
        self.weight = nn.Parameter(torch.empty(num_linear, out_features, in_features))

    def forward(self, x: torch.Tensor, indices: torch.Tensor, plan: Optional[GroupPlan] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return indexed_matmul(x, self.weight, indices, plan, rows)

    def extra_repr(self) -> str:
        return f"num_linear={self.num_linear}, in_features={self.in_features}, out_features={self.out_features}"

    def reset_parameters(self):
        std = self.in_features ** (-0.5)
        nn.init.trunc_normal_(self.weight, std=std, a=-3 * std, b=3 * std)
