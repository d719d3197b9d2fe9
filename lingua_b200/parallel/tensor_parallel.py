"""Tensor parallelism for the transformer blocks.

Same sharding plan as apps/main/transformer.py:165-221: wq / wk / wv / w1 / w3 are split by output
rows (column parallel, each rank owns ``n_heads / tp`` heads), wo / w2 by input columns (row
parallel); the number of heads seen by each block is divided by the TP degree. Parameters are
re-shaped on the meta device before the sharded engine allocates them, so every rank only ever
holds its slice. The partial sums of the row-parallel outputs are combined with an all-reduce in
forward, and the input gradient of the column-parallel projections with an all-reduce in
backward (the conjugate pair of Megatron-style TP). Embeddings, norms and the vocabulary head
stay replicated inside a TP group; their gradients are identical on every TP rank by construction.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn


class ReduceFwd(torch.autograd.Function):
    """All-reduce (sum) in forward, identity in backward: output of a row-parallel layer."""

    @staticmethod
    def forward(ctx, x, group):
        if group is not None:
            x = x.contiguous()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class ReduceBwd(torch.autograd.Function):
    """Identity in forward, all-reduce (sum) in backward: input of a column-parallel layer."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        if ctx.group is not None:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


def _shard_param(mod: nn.Module, dim: int, tp: int, rank: int) -> None:
    w = mod.weight
    assert w.shape[dim] % tp == 0, f"{tuple(w.shape)} not divisible by tp={tp} on dim {dim}"
    shape = list(w.shape)
    shape[dim] //= tp
    if w.device.type == "meta":
        new = torch.empty(shape, device="meta", dtype=w.dtype)
    else:
        new = w.data.chunk(tp, dim=dim)[rank].clone()
    mod.weight = nn.Parameter(new, requires_grad=w.requires_grad)
    if getattr(w, "lb_fp8", False) and shape[0] % 16 == 0 and shape[1] % 16 == 0:
        mod.weight.lb_fp8 = True  # float8 products were requested for this layer: the mark lives on the parameter
    mod.tp_shard = (dim, tp, rank)
    if dim == 0:
        mod.out_features = shape[0]
    else:
        mod.in_features = shape[1]


def tp_parallelize(model, mesh, model_args, distributed_args) -> None:
    """Shard every block of ``model`` over ``mesh``'s tp axis (in place)."""
    tp = mesh.size("tp")
    if tp == 1:
        return
    rank, group = mesh.local_rank("tp"), mesh.group("tp")
    for layer in model.layers:
        at, ff = layer.attention, layer.feed_forward
        assert at.n_heads % tp == 0 and at.n_kv_heads % tp == 0, "heads must divide by the TP degree"
        for lin in (at.wq, at.wk, at.wv):
            _shard_param(lin, 0, tp, rank)
        _shard_param(at.wo, 1, tp, rank)
        at.n_heads //= tp
        at.n_kv_heads //= tp
        _shard_param(ff.w1, 0, tp, rank)
        if ff.activation == "swiglu":
            _shard_param(ff.w3, 0, tp, rank)
        _shard_param(ff.w2, 1, tp, rank)
        # ff.hidden_dim keeps the full width: it sets the initialisation scale of w2
        layer.n_heads, layer.n_kv_heads = at.n_heads, at.n_kv_heads
        layer.tp_group = group
        at.tp_group = group
        ff.tp_group = group
    model.tp_group = group
    model.tp_size, model.tp_rank = tp, rank
