"""Flash attention (``csrc/attention.cu``) with causal / block-causal / sliding-window masks.

Tensors are ``[B, S, H, Dh]`` views (any strides with a contiguous last dim), so q, k and v
can be slices of one fused QKV projection output. Documents packed into a sequence are
described by ``doc_start[b, s]`` (index of the first token of token s's document), the
per-token form of the ``lengths`` of lingua/transformer.py:146-217.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib


def doc_bounds_from_lengths(lengths: torch.Tensor, seq_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """lengths: 1-D document lengths of ONE packed sequence (sum == seq_len).
    Returns int32 (doc_start[s], doc_end[s])."""
    ends = torch.cumsum(lengths, 0)
    starts = ends - lengths
    doc_id = torch.repeat_interleave(torch.arange(lengths.numel(), device=lengths.device), lengths)
    assert doc_id.numel() == seq_len
    return starts[doc_id].int(), ends[doc_id].int()


def attention_ref(q, k, v, causal=True, doc_start=None, window=0, scale=None):
    """fp32 masked-softmax attention. Returns (o [B,S,H,Dh] in q.dtype, lse [B,H,S] fp32)."""
    B, S, H, Dh = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(Dh)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    qi = torch.arange(S, device=q.device).view(1, 1, S, 1)
    ki = torch.arange(S, device=q.device).view(1, 1, 1, S)
    mask = torch.ones(1, 1, S, S, dtype=torch.bool, device=q.device)
    if causal:
        mask = mask & (ki <= qi)
    if window and window > 0:
        mask = mask & (ki > qi - window)
    if doc_start is not None:
        mask = mask & (ki >= doc_start.view(B, 1, S, 1).long())
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype).contiguous(), lse


def _fill(args, q, k, v, causal, doc_start, doc_end, window, scale):
    B, S, H, Dh = q.shape
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    args.B, args.S, args.H, args.Hkv, args.D = B, S, H, k.shape[2], Dh
    args.causal, args.window = int(causal), int(window or 0)
    args.scale = float(scale if scale is not None else 1.0 / math.sqrt(Dh))
    args.q_sb, args.q_ss, args.q_sh = q.stride(0), q.stride(1), q.stride(2)
    args.k_sb, args.k_ss, args.k_sh = k.stride(0), k.stride(1), k.stride(2)
    args.v_sb, args.v_ss, args.v_sh = v.stride(0), v.stride(1), v.stride(2)
    if doc_start is not None:
        assert doc_start.dtype == torch.int32 and doc_start.is_contiguous() and doc_start.numel() == B * S
        args.doc_start = doc_start.data_ptr()
    if doc_end is not None:
        assert doc_end.dtype == torch.int32 and doc_end.is_contiguous() and doc_end.numel() == B * S
        args.doc_end = doc_end.data_ptr()
    args.status = _lib.status_word(q.device).data_ptr()


def flash_fwd(q, k, v, causal=True, doc_start=None, window=0, scale=None):
    """Returns (o [B,S,H,Dh] contiguous, lse [B,H,S] fp32)."""
    if not q.is_cuda:
        return attention_ref(q, k, v, causal, doc_start, window, scale)
    B, S, H, Dh = q.shape
    o = torch.empty(B, S, H, Dh, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    a = _lib.AttnArgs()
    _fill(a, q, k, v, causal, doc_start, None, window, scale)
    a.o, a.lse = o.data_ptr(), lse.data_ptr()
    _lib.check(_lib.load().lb_attn_fwd(C.byref(a), _lib.stream_ptr()), "lb_attn_fwd")
    return o, lse


def flash_bwd(dout, q, k, v, o, lse, dq, dk, dv, causal=True, doc_start=None, doc_end=None, window=0, scale=None):
    """Writes dq/dk/dv (views with the strides of q/k/v)."""
    if not q.is_cuda:
        with torch.enable_grad():
            qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            oo, _ = attention_ref(qq, kk, vv, causal, doc_start, window, scale)
            gq, gk, gv = torch.autograd.grad(oo, (qq, kk, vv), dout.float())
        dq.copy_(gq)
        dk.copy_(gk)
        dv.copy_(gv)
        return
    B, S, H, Dh = q.shape
    assert dout.is_contiguous() and o.is_contiguous()
    assert dq.stride() == q.stride() and dk.stride() == k.stride() and dv.stride() == v.stride()
    delta = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    dq_acc = torch.empty(B, S, H, Dh, dtype=torch.float32, device=q.device)
    a = _lib.AttnArgs()
    _fill(a, q, k, v, causal, doc_start, doc_end, window, scale)
    a.o, a.lse, a.dout = o.data_ptr(), lse.data_ptr(), dout.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.delta, a.dq_acc = delta.data_ptr(), dq_acc.data_ptr()
    _lib.check(_lib.load().lb_attn_bwd(C.byref(a), _lib.stream_ptr()), "lb_attn_bwd")


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, doc_start, doc_end, window, scale):
        # gradients are written with the operands' strides, so gapped views are packed first
        q, k, v = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v))
        o, lse = flash_fwd(q, k, v, causal, doc_start, window, scale)
        ctx.save_for_backward(q, k, v, o, lse, doc_start, doc_end)
        ctx.cfg = (causal, window, scale)
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse, doc_start, doc_end = ctx.saved_tensors
        causal, window, scale = ctx.cfg
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        flash_bwd(dout.contiguous(), q, k, v, o, lse, dq, dk, dv, causal, doc_start, doc_end, window, scale)
        return dq, dk, dv, None, None, None, None, None


def attention(q, k, v, causal=True, doc_start=None, doc_end=None, window=0, scale=None):
    """Differentiable attention on [B,S,H,Dh] tensors (GQA when k/v have fewer heads)."""
    return _FlashAttn.apply(q, k, v, causal, doc_start, doc_end, window, scale)
