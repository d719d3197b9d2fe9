"""Tensor-parallel *training* with a sequence-sharded residual stream and the collectives inside the GEMM kernels.

The reference shards a block with DTensor plans (apps/main/transformer.py:165-221): ``SequenceParallel`` on the
three norms, ``ColwiseParallel`` on wq / wk / wv / w1 / w3, ``RowwiseParallel(output_layouts=Shard(1))`` on wo / w2,
and lets NCCL run an all-gather in front of every column-parallel matmul and a reduce-scatter behind every
row-parallel one - in forward and, mirrored, in backward. Here every rank of the TP group owns ``T / tp`` consecutive
rows of the residual stream and each half of a block (attention, feed-forward) is one autograd function built on the
two fused kernels of ``csrc/gemm_tp.cu``:

    forward    y = RMSNorm(h) (own rows)  ->  [all-gather -> GEMM] with the column-parallel weights
               ->  attention / gated activation on the local heads / features, all tokens
               ->  [GEMM -> reduce-scatter] with the row-parallel weight  ->  h + sum of the partials (own rows)
    backward   dh (own rows)  ->  [all-gather -> GEMM] with the row-parallel weight read as its transpose
               ->  attention / activation backward  ->  [GEMM -> reduce-scatter] with the column-parallel
               weights read as their transpose  ->  RMSNorm backward (own rows)
               the two weight gradients are ordinary wgrad GEMMs on the gathered operands, which the all-gather
               kernels leave behind in local memory.

Ranks meet at a bounded-wait barrier kernel twice per half-block and direction; no NCCL call is made on this path.
Weights of replicated modules (norms, embedding, vocabulary head) see only this rank's rows, so their gradients are
partial sums over the TP group: the sharded engine adds them up (``ShardedEngine.tp_partial``).
"""
from __future__ import annotations

import logging
from typing import Optional

import torch
import torch.distributed as dist

from ..float8 import fp8_dgrad_mm, fp8_forward_mm, wants_fp8
from ..ops import functional as F
from ..ops.attention import flash_bwd, flash_fwd
from ..ops.fused import _emit_vec_grad, _emit_wgrad, _weights
from .tp_fused import ROW_TILE, SymmetricPeers, ag_gemm, gemm_scatter, reduce_norm

logger = logging.getLogger(__name__)


class SPContext:
    """Peer-visible buffers of one TP group for a given (tokens, width): the normalised rows every rank publishes
    (``y``), the staging slots that receive the partial products (``stage``) and the local gather workspace."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device):
        self.peers = SymmetricPeers(group, device)
        self.group, self.device = group, device
        self.world, self.rank = self.peers.world, self.peers.rank
        self._shape = None

    def accepts(self, T: int) -> bool:
        return T % (ROW_TILE * self.world) == 0

    def setup(self, T: int, D: int) -> None:
        if self._shape == (T, D):
            return
        assert self._shape is None, "the sequence-parallel buffers are sized once (fixed tokens per step)"
        Tl = T // self.world
        self.T, self.Tl, self.D = T, Tl, D
        self.y = self.peers.alloc("sp_y", (Tl, D), torch.bfloat16)
        self.stage = self.peers.alloc("sp_stage", (self.world, Tl, D), torch.bfloat16)
        self.flags = torch.zeros(T // ROW_TILE + 1, dtype=torch.int32, device=self.device)
        self._shape = (T, D)

    def barrier(self) -> None:
        self.peers.barrier()

    def gathered(self, own_rows: torch.Tensor, w: torch.Tensor, transposed: bool = False):
        """(all rows @ w^T, all rows) -- with ``transposed``: all rows @ w. Publishes ``own_rows`` ([Tl, D]),
        multiplies every rank's rows with the weight (read in place in either orientation) and keeps the gathered
        rows for the weight gradient.

        bf16 weights: one kernel gathers and multiplies (``ag_gemm``). Weights marked for float8: the peers' rows are
        copied over NVLink into the local buffer first and the product is the row-wise scaled e4m3 one of
        ``lingua_b200.float8`` on local memory; every rank quantises what it holds, so operands that TP splits
        along the reduction dim get one scale per row and rank (the sub-row scaling of lingua/float8.py:14-21)."""
        self.y.copy_(own_rows)
        self.barrier()  # every rank's rows are in place (and nobody still reads the previous contents)
        full = torch.empty(self.T, self.D, dtype=torch.bfloat16, device=self.device)
        if not wants_fp8(w):
            out = ag_gemm(self.peers.ptrs("sp_y"), self.rank, self.Tl, w.t() if transposed else w, full, self.flags)
            full[self.rank * self.Tl:(self.rank + 1) * self.Tl].copy_(own_rows)  # the kernel reads the own slab in place
            return out, full
        for r in range(self.world):
            src = own_rows if r == self.rank else self.peers.peer("sp_y", r)
            full[r * self.Tl:(r + 1) * self.Tl].copy_(src, non_blocking=True)
        return (fp8_dgrad_mm(full, w) if transposed else fp8_forward_mm(full, w)), full

    def scattered_sum(self, x: torch.Tensor, w: torch.Tensor, resid: Optional[torch.Tensor],
                      transposed: bool = False) -> torch.Tensor:
        """Own rows of sum_ranks(x_r @ w_r^T) (+ resid) -- with ``transposed``: x_r @ w_r. bf16: the partial product
        of every rank is stored into the owners' slots by the GEMM epilogue; float8: the local e4m3 product is
        copied slab by slab into the owners' slots. Then the slots are summed."""
        if not wants_fp8(w):
            gemm_scatter(x, w.t() if transposed else w, self.peers.ptrs("sp_stage"), self.rank, self.Tl * self.D)
        else:
            part = fp8_dgrad_mm(x, w) if transposed else fp8_forward_mm(x, w)
            for k in range(self.world):
                r = (self.rank + k) % self.world  # own slab first, then the neighbours in ring order
                self.peers.peer("sp_stage", r)[self.rank].copy_(part[r * self.Tl:(r + 1) * self.Tl], non_blocking=True)
        self.barrier()  # every rank's partials have landed
        h, _ = reduce_norm(self.stage, resid, None, 0.0)
        return h


def _out_weight(w: torch.Tensor) -> torch.Tensor:
    """The row-parallel weight without its autograd history; ``detach`` drops the float8 mark, so it is put back."""
    d = w.detach()
    if wants_fp8(w):
        d.lb_fp8 = True
    return d


def _in_weight(ws_in) -> torch.Tensor:
    """The stacked column-parallel weight (wq|wk|wv or w1|w3) as one matrix, carrying the float8 mark of its parts."""
    w = _weights(ws_in)
    if wants_fp8(ws_in[0]) and not wants_fp8(w):
        w.lb_fp8 = True
    return w


class SPHalfBlockFn(torch.autograd.Function):
    """One half of a transformer block on a row-sharded residual stream: h -> h + Out(core(In(RMSNorm(h)))), where In
    is column-parallel (wq|wk|wv or w1|w3), Out row-parallel (wo or w2) and ``core`` is RoPE + attention or the gated
    activation. ``cfg`` is ("attn", B, S, H, Hkv, Dh, causal, window) or ("glu" | "act", mode)."""

    @staticmethod
    def forward(ctx, h, g, eps, sp: SPContext, cfg, cs, doc_start, doc_end, pos, w_out, *ws_in):
        y, _, rstd = F.rmsnorm_fwd(h, g.detach(), eps, None)
        pre, y_full = sp.gathered(y, _in_weight(ws_in))
        del y
        lse = o = None
        if cfg[0] == "attn":
            _, B, S, H, Hkv, Dh, causal, window = cfg
            F.rope_(pre, cs, H + Hkv, Dh, S, pos)
            t = pre.view(B, S, H + 2 * Hkv, Dh)
            o, lse = flash_fwd(t[:, :, :H], t[:, :, H:H + Hkv], t[:, :, H + Hkv:], causal, doc_start, window, Dh ** -0.5)
            core = o.view(B * S, H * Dh)
        elif cfg[0] == "glu":
            core = F.glu_fwd(pre, cfg[1])
        else:
            core = F.act_fwd(pre, cfg[1])
        h_out = sp.scattered_sum(core, _out_weight(w_out), h)
        ctx.save_for_backward(h, rstd, y_full, pre, o, lse, cs, doc_start, doc_end, pos)
        ctx.g, ctx.eps, ctx.sp, ctx.cfg, ctx.w_out, ctx.ws_in = g, eps, sp, cfg, w_out, ws_in
        return h_out

    @staticmethod
    def backward(ctx, dh_out):
        h, rstd, y_full, pre, o, lse, cs, doc_start, doc_end, pos = ctx.saved_tensors
        g, sp, cfg, w_out, ws_in = ctx.g, ctx.sp, ctx.cfg, ctx.w_out, ctx.ws_in
        dh_out = dh_out.contiguous()
        # d(core) = gather(dh_out) @ W_out  (W_out [D, K_local] read as the [K_local, D] operand it is the transpose of)
        dcore, dp_full = sp.gathered(dh_out, _out_weight(w_out), transposed=True)
        if cfg[0] == "attn":
            _, B, S, H, Hkv, Dh, causal, window = cfg
            core = o.view(B * S, H * Dh)
        elif cfg[0] == "glu":
            core = F.glu_fwd(pre, cfg[1])
        else:
            core = F.act_fwd(pre, cfg[1])
        (dw_out,) = _emit_wgrad([w_out], dp_full, core) if w_out.requires_grad else (None,)
        del dp_full
        if cfg[0] == "attn":
            t = pre.view(B, S, H + 2 * Hkv, Dh)
            dt = torch.empty_like(t)
            flash_bwd(dcore.view(B, S, H, Dh), t[:, :, :H], t[:, :, H:H + Hkv], t[:, :, H + Hkv:], o, lse,
                      dt[:, :, :H], dt[:, :, H:H + Hkv], dt[:, :, H + Hkv:], causal, doc_start, doc_end, window, Dh ** -0.5)
            dpre = dt.view(B * S, -1)
            F.rope_(dpre, cs, H + Hkv, Dh, S, pos, backward=True)
        elif cfg[0] == "glu":
            dpre = F.glu_bwd(pre, dcore, cfg[1])
        else:
            dpre = F.act_bwd(pre, dcore, cfg[1])
        del core, dcore
        dws_in = _emit_wgrad(ws_in, dpre, y_full) if ws_in[0].requires_grad else [None] * len(ws_in)
        # d(y) for the own rows = sum over ranks of dpre_r @ W_in_r
        dy = sp.scattered_sum(dpre, _in_weight(ws_in), None, transposed=True)
        holder = {}

        def run(dw_buf):
            holder["dx"], _ = F.rmsnorm_bwd(dy, h, g.detach(), rstd, dh_out, dw_buf)

        dg = _emit_vec_grad(g, run)
        return (holder["dx"], dg, None, None, None, None, None, None, None, dw_out, *dws_in)


class SumOverGroupFn(torch.autograd.Function):
    """All-reduce (sum) in forward, identity in backward: combines the ranks' shares of one loss."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, gx):
        return gx, None


def sp_block_forward(layer, sp: SPContext, h, cs, B, S, doc_start, doc_end, window, pos, causal):
    """Both halves of ``layer`` on the row-sharded residual stream ``h`` [T / tp, dim]."""
    at, ff = layer.attention, layer.feed_forward
    cfg = ("attn", B, S, at.n_heads, at.n_kv_heads, at.head_dim, causal, window)
    h = SPHalfBlockFn.apply(h, layer.attention_norm.weight, layer.attention_norm.eps, sp, cfg, cs, doc_start, doc_end,
                            pos, at.wo.weight, *at.qkv_weights())
    cfg = ("glu", F.ACT_SILU) if ff.activation == "swiglu" else ("act", F.ACT_RELU2)
    return SPHalfBlockFn.apply(h, layer.ffn_norm.weight, layer.ffn_norm.eps, sp, cfg, None, None, None, None,
                               ff.w2.weight, *ff.in_weights())


def enable_sp_training(model, group: dist.ProcessGroup, device: torch.device) -> bool:
    """Give a TP-sharded ``LMTransformer`` the sequence-parallel training path. False (the all-reduce formulation of
    ``tensor_parallel.py`` stays) when the group has no peer-visible memory, e.g. ranks on different nodes."""
    try:
        ctx = SPContext(group, device)
    except Exception as e:  # no NVLink peer access between the ranks of this group
        logger.warning("sequence-parallel tensor-parallel training disabled: %s", e)
        return False
    object.__setattr__(model, "tp_sp", ctx)
    return True
