"""Position-indexed ("multi-linear") projection: ``Y[t] = X[t] @ W[idx[t]]^T`` with a small bank of weights.

The hierarchical byte model upsamples a pooled vector back to the bytes it covers and gives each byte a
projection chosen by its distance to the pooled position (apps/aunet/index_matmul.py:12-91 of the reference,
which loops over the bank with a boolean ``torch.where`` -- a host synchronisation -- per weight in forward
and again in backward).

Here the rows are sorted by index once (``plan_groups``: one stable argsort and one bincount on the device,
one small device-to-host read of the group sizes per plan), after which forward, dgrad and wgrad are plain
tensor-core GEMMs over contiguous row ranges of the sorted activations. A plan is built once per step and
shared by forward and backward and by every call that uses the same indices."""
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
    order: torch.Tensor  # [T] int64: rows in group order (stable)
    counts: List[int]  # rows per group, on the host
    n: int

    @property
    def segments(self):
        o = 0
        for g, c in enumerate(self.counts):
            if c:
                yield g, o, c
            o += c


def plan_groups(indices: torch.Tensor, n: int) -> GroupPlan:
    flat = indices.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=n)
    return GroupPlan(order=order, counts=[int(c) for c in counts.tolist()], n=n)


def indexed_matmul_ref(x: torch.Tensor, w: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """fp32 oracle: gathers one weight per row."""
    x2 = x.reshape(-1, x.shape[-1]).float()
    y = torch.einsum("td,tod->to", x2, w.float()[indices.reshape(-1)])
    return y.view(*x.shape[:-1], w.shape[1])


class IndexedMatMulFn(torch.autograd.Function):
    """``rows`` (optional, [T] int64): output row t reads input row ``rows[t]`` -- the repeat-upsampling gather
    folded into the sort, so the repeated activations are never materialised in input order."""

    @staticmethod
    def forward(ctx, x2d, w, plan: GroupPlan, rows=None):
        src = plan.order if rows is None else rows.index_select(0, plan.order)
        xs = x2d.index_select(0, src)
        ys = torch.empty(xs.shape[0], w.shape[1], dtype=x2d.dtype, device=x2d.device)
        for g, o, c in plan.segments:
            mm_nt(xs[o:o + c], w[g], out=ys[o:o + c], out_dtype=x2d.dtype)
        y = torch.empty_like(ys)
        y.index_copy_(0, plan.order, ys)
        ctx.save_for_backward(xs, w, src)
        ctx.plan, ctx.n_in, ctx.permutation = plan, x2d.shape[0], rows is None
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, w, src = ctx.saved_tensors
        plan: GroupPlan = ctx.plan
        dys = dy.index_select(0, plan.order)
        dxs = torch.empty_like(xs)
        main = getattr(w, "main_grad", None)  # fp32 gradient buffer of a training engine, if any
        dw = None if main is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        acc = main is not None and getattr(w, "grad_written", False)
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
