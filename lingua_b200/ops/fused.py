"""Autograd functions of the native transformer path.

Each function is one "save point" of the layer: it keeps only what cannot be recomputed
cheaply (GEMM outputs, the attention output and its log-sum-exp) and recomputes the
memory-bound results (normalised activations, gated activation, logits) in backward.
This is the fixed, per-op form of the selective activation checkpointing policy of
lingua/distributed.py:43-53,298-308 (save matmul and attention outputs, recompute the rest).

Weight gradients: when a weight tensor carries a ``main_grad`` attribute (an fp32 view into
the sharded-parameter engine's gradient buffer) the wgrad GEMM writes or accumulates there
directly and autograd receives ``None``; otherwise a gradient of the weight's dtype is returned.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import functional as F
from .attention import flash_bwd, flash_fwd
from .gemm import gemm, gemm_gather, gemm_scatter, mm_nn, mm_nt, mm_tn


# Statistics probe (lingua_b200.probe.AutoProbeD): when set, the functions below report their
# operands to it. None on the normal path.
_OBSERVER = None


def set_observer(obs) -> None:
    global _OBSERVER
    _OBSERVER = obs


# True: keep only GEMM / attention outputs and recompute normalised and gated activations in
# backward (the selective-checkpointing policy). False: keep them too (more memory, ~1.5 % faster).
_RECOMPUTE = True


def set_recompute(flag: bool) -> None:
    global _RECOMPUTE
    _RECOMPUTE = bool(flag)


# ----------------------------------------------------------------------------- helpers
def fused_view(ws: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
    """[sum(N_i), K] view over row-blocks that are adjacent in memory, or None."""
    if len(ws) == 1:
        return ws[0]
    base = ws[0]
    K = base.shape[1]
    ptr = base.data_ptr()
    store = base.untyped_storage().data_ptr()
    for w in ws:
        if not w.is_contiguous() or w.shape[1] != K or w.data_ptr() != ptr or w.dtype != base.dtype:
            return None
        if w.untyped_storage().data_ptr() != store:  # neighbours by accident, not one buffer
            return None
        ptr += w.numel() * w.element_size()
    rows = sum(w.shape[0] for w in ws)
    return torch.as_strided(base, (rows, K), (K, 1), base.storage_offset())


def _stale_targets(ws: Sequence[torch.Tensor]):
    """Gather handles of weights whose remote rows have not been fetched since the last optimiser step (the sharded
    engine leaves the all-gather of some matrices to their first forward GEMM), or None."""
    t0 = getattr(ws[0], "lb_gather", None)
    if t0 is None or not t0.group.gather_stale:
        return None
    targets = [w.lb_gather for w in ws if hasattr(w, "lb_gather")]
    return targets if t0.engine.gather_is_stale(targets) else None


def _weights(ws: Sequence[torch.Tensor]) -> torch.Tensor:
    stale = _stale_targets(ws)
    if stale is not None:
        stale[0].engine.ensure_gathered(stale)
    v = fused_view([w.detach() for w in ws])
    return v if v is not None else torch.cat([w.detach() for w in ws], dim=0)


def _fwd_mm(x: torch.Tensor, ws: Sequence[torch.Tensor]) -> torch.Tensor:
    """x @ [W_0; W_1; ...]^T - in e4m3 with row-wise scales when the weights are marked for float8. The first
    product with a weight after an optimiser step may also be the one that gathers it from the other ranks."""
    stale = _stale_targets(ws)
    if (stale is not None and len(stale) == len(ws) and x.is_cuda and x.dim() == 2 and x.shape[0] >= 256
            and not getattr(ws[0], "lb_fp8", False)):
        engine = stale[0].engine
        plan = engine.gather_plan(stale)
        v = fused_view([w.detach() for w in ws])
        if plan is not None and v is not None and x.stride(1) == 1:
            out = gemm_gather(x, v, plan[0], plan[1])
            engine.mark_gathered(stale)
            return out
    w = _weights(ws)
    if getattr(ws[0], "lb_fp8", False) and x.is_cuda and x.shape[0] >= 16:
        from ..float8 import fp8_forward_mm

        return fp8_forward_mm(x, w)
    return mm_nt(x, w)


def _dgrad_mm(dy: torch.Tensor, ws: Sequence[torch.Tensor]) -> torch.Tensor:
    """dy @ [W_0; W_1; ...] - the float8 form scales dy by row and the stacked weight as one tensor."""
    w = _weights(ws)
    if getattr(ws[0], "lb_fp8", False) and dy.is_cuda and dy.shape[0] >= 16:
        from ..float8 import fp8_dgrad_mm

        return fp8_dgrad_mm(dy, w)
    return mm_nn(dy, w)


def _main_grads(ws: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
    if not all(hasattr(w, "main_grad") for w in ws):
        return None
    return fused_view([w.main_grad for w in ws])


def _emit_scatter(ws: Sequence[torch.Tensor], dy2d: torch.Tensor, x2d: torch.Tensor) -> bool:
    """Weight gradient of row-sharded parameters (``w.lb_scatter``, set by the sharded engine): no local matrix is
    written; the GEMM epilogue stores every 128-row block into its owner's buffer. One GEMM for the whole fused
    weight when the engine can describe it with one block table, else one per parameter."""
    targets = [w.lb_scatter for w in ws]
    engine = targets[0].engine
    written = [getattr(w, "grad_written", False) for w in ws]
    if not dy2d.is_cuda:
        return False
    if engine.grad_mode == "atomic":
        written = [True] * len(ws)  # every contribution is added into the owner's shard (which starts at zero)
    plan = engine.scatter_plan(targets) if (all(written) or not any(written)) else None
    if plan is not None:
        blocks, ptrs, rows, K, m_rot = plan
        gemm_scatter(dy2d.transpose(0, 1), x2d.transpose(0, 1), blocks, ptrs, rows, ldc=K, accumulate=written[0],
                     m_rot=m_rot)
        for w in ws:
            w.grad_written = True
        return True
    r0 = 0
    for w, t, wr in zip(ws, targets, written):
        n = w.shape[0]
        blocks, ptrs, rows, K, m_rot = engine.scatter_plan([t])
        gemm_scatter(dy2d[:, r0:r0 + n].transpose(0, 1), x2d.transpose(0, 1), blocks, ptrs, rows, ldc=K, accumulate=wr,
                     m_rot=m_rot)
        w.grad_written = True
        r0 += n
    return True


def _emit_wgrad(ws: Sequence[torch.Tensor], dy2d: torch.Tensor, x2d: torch.Tensor) -> List[Optional[torch.Tensor]]:
    """dW_i = dy[:, rows_i]^T x for the row-blocks ``ws`` of one fused weight."""
    if all(hasattr(w, "lb_scatter") for w in ws) and _emit_scatter(ws, dy2d, x2d):
        return [None] * len(ws)
    mg = _main_grads(ws)
    if mg is not None:
        written = [getattr(w, "grad_written", False) for w in ws]
        if all(written) or not any(written):
            mm_tn(dy2d, x2d, out=mg, accumulate=written[0])
            for w in ws:
                w.grad_written = True
            return [None] * len(ws)
    outs: List[Optional[torch.Tensor]] = []
    r0 = 0
    for w in ws:
        n = w.shape[0]
        dyi = dy2d[:, r0:r0 + n]
        r0 += n
        if hasattr(w, "main_grad"):
            mm_tn(dyi, x2d, out=w.main_grad, accumulate=getattr(w, "grad_written", False))
            w.grad_written = True
            outs.append(None)
        else:
            outs.append(mm_tn(dyi, x2d, out_dtype=torch.float32).to(w.dtype))
    return outs


def _emit_vec_grad(w: torch.Tensor, fn) -> Optional[torch.Tensor]:
    """Gradient of a 1-D weight through ``fn(dw_out)`` which accumulates into an fp32 buffer."""
    if hasattr(w, "main_grad"):
        if not getattr(w, "grad_written", False):
            w.main_grad.zero_()
            w.grad_written = True
        fn(w.main_grad)
        return None
    buf = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
    fn(buf)
    return buf.to(w.dtype)


# ----------------------------------------------------------------------------- linear
class LinearFn(torch.autograd.Function):
    """y = x [W_0; W_1; ...]^T for x [M, K] and row-blocks W_i [N_i, K]."""

    @staticmethod
    def forward(ctx, x, *ws):
        ctx.save_for_backward(x)
        ctx.ws = ws
        out = _fwd_mm(x, ws)
        if _OBSERVER is not None:
            _OBSERVER.linear_fwd(ws, x, out)
        return out

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        ws = ctx.ws
        dy = dy.contiguous()
        dx = _dgrad_mm(dy, ws) if ctx.needs_input_grad[0] else None
        dws = _emit_wgrad(ws, dy, x) if ws[0].requires_grad else [None] * len(ws)
        if _OBSERVER is not None:
            _OBSERVER.linear_bwd(ws, dy, dx, dws)
        return (dx, *dws)


class NormLinearFn(torch.autograd.Function):
    """h = x (+ res); out = rmsnorm(h) * g @ [W_0; W_1; ...]^T. Returns (out, h); h is None
    when no residual was given (the caller already holds x). ``tp_group``: the weights are
    column-parallel slices, so the input gradient is summed over that group in backward.

    Saves h and the per-row rstd; the normalised activation is recomputed in backward."""

    @staticmethod
    def forward(ctx, x, res, g, eps, tp_group, *ws):
        y, h, rstd = F.rmsnorm_fwd(x, g.detach(), eps, res)
        h = x if h is None else h
        out = _fwd_mm(y, ws)
        if _OBSERVER is not None:
            _OBSERVER.resid(g, h)
            _OBSERVER.linear_fwd(ws, y, out)
        if _RECOMPUTE:
            ctx.save_for_backward(h, rstd)
        else:
            ctx.save_for_backward(h, rstd, y)
        ctx.g, ctx.ws, ctx.eps, ctx.has_res, ctx.tp_group = g, ws, eps, res is not None, tp_group
        return out, (h if res is not None else None)

    @staticmethod
    def backward(ctx, dout, dh_out):
        h, rstd = ctx.saved_tensors[:2]
        g, ws = ctx.g, ctx.ws
        dout = dout.contiguous()
        if len(ctx.saved_tensors) == 3:
            y = ctx.saved_tensors[2]
        else:
            y, _, _ = F.rmsnorm_fwd(h, g.detach(), ctx.eps, None)
        dws = _emit_wgrad(ws, dout, y) if ws[0].requires_grad else [None] * len(ws)
        del y
        dy = _dgrad_mm(dout, ws)
        if _OBSERVER is not None:
            _OBSERVER.linear_bwd(ws, dout, dy, dws)
        if ctx.tp_group is not None:
            # column-parallel weights: every TP rank holds a partial sum of the input gradient
            torch.distributed.all_reduce(dy, group=ctx.tp_group)
        dres_in = dh_out.contiguous() if dh_out is not None else None
        holder = {}

        def run(dw_buf):
            holder["dx"], _ = F.rmsnorm_bwd(dy, h, g.detach(), rstd, dres_in, dw_buf)

        dg = _emit_vec_grad(g, run)
        dx = holder["dx"]
        return (dx, dx if ctx.has_res else None, dg, None, None, *dws)


def _pad_heads(t: torch.Tensor, Dh: int) -> torch.Tensor:
    """[..., heads, Dh] -> [..., heads, 128], zero-filled: the attention kernel takes heads of width 128.
    Scores are unchanged (the softmax scale is passed explicitly) and the padded output half is zero."""
    return t if Dh == 128 else torch.nn.functional.pad(t, (0, 128 - Dh))


class RopeAttnFn(torch.autograd.Function):
    """qkv [B*S, (H + 2 Hkv) * Dh] -> RoPE on q and k (in place) -> attention -> [B*S, H * Dh]. Dh <= 128."""

    @staticmethod
    def forward(ctx, qkv, cs, B, S, H, Hkv, Dh, causal, doc_start, doc_end, window, pos, anchor=None):
        F.rope_(qkv, cs, H + Hkv, Dh, S, pos)
        t = _pad_heads(qkv.view(B, S, H + 2 * Hkv, Dh), Dh)
        q, k, v = t[:, :, :H], t[:, :, H:H + Hkv], t[:, :, H + Hkv:]
        if _OBSERVER is not None and anchor is not None:
            _OBSERVER.attention(anchor, q[..., :Dh], k[..., :Dh], causal, doc_start)
        o, lse = flash_fwd(q, k, v, causal, doc_start, window, Dh ** -0.5)
        if Dh != 128:
            o = o[..., :Dh].contiguous()
        ctx.save_for_backward(qkv, o, lse, cs, doc_start, doc_end, pos)
        ctx.cfg = (B, S, H, Hkv, Dh, causal, window)
        return o.view(B * S, H * Dh)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cs, doc_start, doc_end, pos = ctx.saved_tensors
        B, S, H, Hkv, Dh, causal, window = ctx.cfg
        t = _pad_heads(qkv.view(B, S, H + 2 * Hkv, Dh), Dh)
        q, k, v = t[:, :, :H], t[:, :, H:H + Hkv], t[:, :, H + Hkv:]
        dt = torch.empty_like(t)
        flash_bwd(_pad_heads(do.contiguous().view(B, S, H, Dh), Dh), q, k, v, _pad_heads(o.view(B, S, H, Dh), Dh), lse,
                  dt[:, :, :H], dt[:, :, H:H + Hkv], dt[:, :, H + Hkv:], causal, doc_start, doc_end, window,
                  Dh ** -0.5)
        dqkv = dt.view(B * S, -1) if Dh == 128 else dt[..., :Dh].reshape(B * S, -1)
        F.rope_(dqkv, cs, H + Hkv, Dh, S, pos, backward=True)
        return (dqkv,) + (None,) * 12


class GluLinearFn(torch.autograd.Function):
    """out = (act(gu[:, :H]) * gu[:, H:]) @ W^T; saves only gu."""

    @staticmethod
    def forward(ctx, gu, w, mode):
        a = F.glu_fwd(gu, mode)
        if _RECOMPUTE:
            ctx.save_for_backward(gu)
        else:
            ctx.save_for_backward(gu, a)
        ctx.w, ctx.mode = w, mode
        out = _fwd_mm(a, (w,))
        if _OBSERVER is not None:
            _OBSERVER.linear_fwd([w], a, out)
        return out

    @staticmethod
    def backward(ctx, dy):
        gu = ctx.saved_tensors[0]
        w = ctx.w
        dy = dy.contiguous()
        a = ctx.saved_tensors[1] if len(ctx.saved_tensors) == 2 else F.glu_fwd(gu, ctx.mode)
        (dw,) = _emit_wgrad([w], dy, a) if w.requires_grad else (None,)
        del a
        da = _dgrad_mm(dy, (w,))
        if _OBSERVER is not None:
            _OBSERVER.linear_bwd([w], dy, da, [dw])
        return F.glu_bwd(gu, da, ctx.mode), dw, None


class ActLinearFn(torch.autograd.Function):
    """out = act(u) @ W^T for an ungated FFN (squared ReLU); saves only u."""

    @staticmethod
    def forward(ctx, u, w, mode):
        a = F.act_fwd(u, mode)
        ctx.save_for_backward(u)
        ctx.w, ctx.mode = w, mode
        out = _fwd_mm(a, (w,))
        if _OBSERVER is not None:
            _OBSERVER.linear_fwd([w], a, out)
        return out

    @staticmethod
    def backward(ctx, dy):
        (u,) = ctx.saved_tensors
        w = ctx.w
        dy = dy.contiguous()
        a = F.act_fwd(u, ctx.mode)
        (dw,) = _emit_wgrad([w], dy, a) if w.requires_grad else (None,)
        del a
        da = _dgrad_mm(dy, (w,))
        if _OBSERVER is not None:
            _OBSERVER.linear_bwd([w], dy, da, [dw])
        return F.act_bwd(u, da, ctx.mode), dw, None


class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, table):
        ctx.save_for_backward(tokens)
        ctx.table = table
        return F.embed_fwd(tokens, table.detach())

    @staticmethod
    def backward(ctx, dy):
        (tokens,) = ctx.saved_tensors
        table = ctx.table
        if not table.requires_grad:
            return None, None
        dy = dy.contiguous()
        if hasattr(table, "main_grad"):
            if not getattr(table, "grad_written", False):
                table.main_grad.zero_()
                table.grad_written = True
            F.embed_bwd(tokens, dy, table.main_grad)
            return None, None
        buf = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        F.embed_bwd(tokens, dy, buf)
        return None, buf.to(table.dtype)


# gradients of the logits are kept for a whole step (bf16) when they take no more than this
_DLOGITS_LIMIT_BYTES = 6 << 30


class LinearCrossEntropyFn(torch.autograd.Function):
    """mean_i CE(y_i W^T, target_i) over rows with target >= 0, without ever holding more than
    ``chunk`` rows of logits (the loss of lingua/transformer.py:51-56 applied to
    apps/main/transformer.py:115-117).

    ``grad_scale=None``: forward keeps the per-row log-sum-exp; backward recomputes each logits
    chunk, turns it into its gradient in one pass and feeds the two gradient GEMMs. Exact for any
    incoming gradient, at the price of one extra vocabulary GEMM.

    ``grad_scale=s`` (what the training engine uses): the caller promises that the gradient that
    will flow into the returned loss is the constant ``s`` (1 / grad_acc_steps). The gradient of
    every chunk is then produced in forward right after its loss, so the logits are computed once;
    backward only hands out the stored input gradient."""

    @staticmethod
    def forward(ctx, y, w, target, chunk, grad_scale=None, n_valid=None):
        # n_valid: number of rows the mean is taken over when ``y`` holds only a share of them (the rows of one
        # sequence-parallel rank); default: the valid rows of ``target``
        M = y.shape[0]
        wd = w.detach()
        tgt = target.reshape(-1)
        total = torch.zeros((), dtype=torch.float32, device=y.device)
        if n_valid is None:
            n_valid = (tgt >= 0).sum().clamp(min=1).float()
        fused_bwd = grad_scale is not None and (ctx.needs_input_grad[0] or w.requires_grad)
        ctx.fused_bwd, ctx.w, ctx.chunk, ctx.grad_scale = fused_bwd, w, chunk, grad_scale
        if not fused_bwd:
            lse = torch.empty(M, dtype=torch.float32, device=y.device)
            for r0 in range(0, M, chunk):
                r1 = min(M, r0 + chunk)
                logits = gemm(y[r0:r1], wd, out_dtype=torch.float32)
                loss_c, lse_c = F.ce_fwd(logits, tgt[r0:r1])
                lse[r0:r1] = lse_c
                total += loss_c.sum()
                del logits
            ctx.save_for_backward(y, tgt, lse, n_valid)
            return total / n_valid
        gscale = (float(grad_scale) / n_valid).reshape(1).contiguous()
        dy = torch.empty_like(y)
        has_mg = hasattr(w, "main_grad")
        dw_acc = None
        V = wd.shape[0]
        Vp = (V + 7) // 8 * 8
        if M > chunk and M * Vp * 2 <= _DLOGITS_LIMIT_BYTES:
            # The logits stay chunked (fp32), their gradients are kept for all rows in bf16, so that the
            # two gradient products are one GEMM each instead of one per chunk: the weight gradient then
            # is written once instead of being read and re-written per chunk.
            dl_all = torch.empty(M, Vp, dtype=torch.bfloat16, device=y.device)[:, :V]
            for r0 in range(0, M, chunk):
                r1 = min(M, r0 + chunk)
                logits = gemm(y[r0:r1], wd, out_dtype=torch.float32)
                loss_c, lse_c = F.ce_fwd(logits, tgt[r0:r1])
                total += loss_c.sum()
                F.ce_bwd(logits, tgt[r0:r1], lse_c, 1.0, gscale, out=dl_all[r0:r1])
                del logits
            mm_nn(dl_all, wd, out=dy)
            if w.requires_grad:
                if hasattr(w, "lb_scatter") and _emit_scatter([w], dl_all, y):
                    pass
                elif has_mg:
                    mm_tn(dl_all, y, out=w.main_grad, accumulate=getattr(w, "grad_written", False))
                    w.grad_written = True
                else:
                    dw_acc = mm_tn(dl_all, y, out_dtype=torch.float32)
            del dl_all
            ctx.save_for_backward(dy, dw_acc)
            return total / n_valid
        for r0 in range(0, M, chunk):
            r1 = min(M, r0 + chunk)
            logits = gemm(y[r0:r1], wd, out_dtype=torch.float32)
            loss_c, lse_c = F.ce_fwd(logits, tgt[r0:r1])
            total += loss_c.sum()
            dl = F.ce_bwd(logits, tgt[r0:r1], lse_c, 1.0, gscale)
            del logits
            mm_nn(dl, wd, out=dy[r0:r1])
            if w.requires_grad:
                if hasattr(w, "lb_scatter") and _emit_scatter([w], dl, y[r0:r1]):
                    pass
                elif has_mg:
                    mm_tn(dl, y[r0:r1], out=w.main_grad, accumulate=getattr(w, "grad_written", False))
                    w.grad_written = True
                else:
                    if dw_acc is None:
                        dw_acc = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
                    mm_tn(dl, y[r0:r1], out=dw_acc, accumulate=True)
            del dl
        ctx.save_for_backward(dy, dw_acc)
        return total / n_valid

    @staticmethod
    def backward(ctx, g):
        w, chunk = ctx.w, ctx.chunk
        if ctx.fused_bwd:
            dy, dw_acc = ctx.saved_tensors
            return dy, (None if dw_acc is None else dw_acc.to(w.dtype)), None, None, None, None
        y, tgt, lse, n_valid = ctx.saved_tensors
        wd = w.detach()
        M = y.shape[0]
        gscale = (g.float() / n_valid).reshape(1).contiguous()
        dy = torch.empty_like(y)
        has_mg = hasattr(w, "main_grad")
        dw_acc = None
        for r0 in range(0, M, chunk):
            r1 = min(M, r0 + chunk)
            logits = gemm(y[r0:r1], wd, out_dtype=torch.float32)
            dl = F.ce_bwd(logits, tgt[r0:r1], lse[r0:r1], 1.0, gscale)
            del logits
            mm_nn(dl, wd, out=dy[r0:r1])
            if w.requires_grad:
                if hasattr(w, "lb_scatter") and _emit_scatter([w], dl, y[r0:r1]):
                    pass
                elif has_mg:
                    mm_tn(dl, y[r0:r1], out=w.main_grad, accumulate=getattr(w, "grad_written", False))
                    w.grad_written = True
                else:
                    if dw_acc is None:
                        dw_acc = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
                    mm_tn(dl, y[r0:r1], out=dw_acc, accumulate=True)
            del dl
        dw = None if (has_mg or dw_acc is None) else dw_acc.to(w.dtype)
        return dy, dw, None, None, None, None
