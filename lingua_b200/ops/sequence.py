"""Causal depthwise conv1d and first-order linear recurrence on channel-last [B, S, C] tensors.

Native kernels: ``csrc/scan.cu``. References (CPU path and test oracles) restate the math of
``causal_conv1d_fn(x, w, seq_idx, activation="silu")`` and ``accelerated_scan.ref.scan`` as used
by apps/fastRNN/component/rnn_common.py:13-118 and apps/mamba/core_mamba.py:188-194. Documents
packed in a sequence are delimited by ``doc_start[b, s]`` (int32, index of the first token of the
token's document): neither the convolution window nor the recurrent state crosses a boundary.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as TF

from . import _lib


def _ptr(t):
    return None if t is None else t.data_ptr()


# ----------------------------------------------------------------------------- conv1d
def conv1d_ref(x, w, doc_start=None, act=True):
    """x: [B, S, C], w: [C, W]. Differentiable PyTorch version."""
    B, S, C = x.shape
    W = w.shape[1]
    xf = x.float()
    out = torch.zeros_like(xf)
    pos = torch.arange(S, device=x.device).view(1, S, 1)
    for j in range(W):
        shift = W - 1 - j
        xs = TF.pad(xf, (0, 0, shift, 0))[:, :S]
        if doc_start is not None:
            ok = (pos - shift) >= doc_start.view(B, S, 1)
        else:
            ok = (pos - shift) >= 0
        out = out + w[:, j].float().view(1, 1, C) * torch.where(ok, xs, torch.zeros_like(xs))
    return (TF.silu(out) if act else out).to(x.dtype)


class _Conv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, doc_start, act):
        B, S, C = x.shape
        W = w.shape[1]
        assert x.stride(2) == 1 and x.stride(0) == S * x.stride(1)
        y = torch.empty(B, S, C, dtype=x.dtype, device=x.device)
        wd = w.detach().contiguous()
        rc = _lib.load().lb_conv1d_fwd(x.data_ptr(), wd.data_ptr(), _ptr(doc_start), y.data_ptr(), B, S, C, W,
                                       x.stride(1), C, int(act), _lib.stream_ptr())
        _lib.check(rc, "lb_conv1d_fwd")
        ctx.save_for_backward(x, doc_start)
        ctx.w, ctx.act = w, act
        return y

    @staticmethod
    def backward(ctx, dy):
        x, doc_start = ctx.saved_tensors
        w = ctx.w
        B, S, C = x.shape
        W = w.shape[1]
        dy = dy.contiguous()
        dx = torch.empty(B, S, C, dtype=x.dtype, device=x.device)
        dw = torch.zeros(C, W, dtype=torch.float32, device=x.device)
        rc = _lib.load().lb_conv1d_bwd(x.data_ptr(), w.detach().contiguous().data_ptr(), _ptr(doc_start),
                                       dy.data_ptr(), dx.data_ptr(), dw.data_ptr(), B, S, C, W, x.stride(1), C, C,
                                       int(ctx.act), _lib.stream_ptr())
        _lib.check(rc, "lb_conv1d_bwd")
        if hasattr(w, "main_grad"):
            if getattr(w, "grad_written", False):
                w.main_grad.add_(dw)
            else:
                w.main_grad.copy_(dw)
                w.grad_written = True
            return dx, None, None, None
        return dx, dw.to(w.dtype), None, None


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, doc_start: Optional[torch.Tensor] = None, act: bool = True):
    """Depthwise causal convolution along S (+ SiLU). x: [B, S, C] (rows may be strided), w: [C, W]."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        ds = doc_start.reshape(-1).int().contiguous() if doc_start is not None else None
        return _Conv1d.apply(x, w, ds, act)
    return conv1d_ref(x, w, doc_start, act)


def conv1d_update_ref(x_t, conv_state, w, act=True):
    conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
    conv_state[:, :, -1] = x_t
    out = (conv_state.float() * w.float().unsqueeze(0)).sum(-1)
    return (TF.silu(out) if act else out).to(x_t.dtype)


def conv1d_update(x_t: torch.Tensor, conv_state: torch.Tensor, w: torch.Tensor, act: bool = True) -> torch.Tensor:
    """One decoding step. x_t: [N, C] (rows may be strided); conv_state: [N, C, W] holds the last W inputs
    (updated in place); returns [N, C]."""
    N, C = x_t.shape
    W = w.shape[1]
    if (x_t.is_cuda and x_t.dtype == torch.bfloat16 and conv_state.dtype == torch.bfloat16 and x_t.stride(1) == 1
            and conv_state.is_contiguous() and W in (2, 3, 4)):
        out = torch.empty(N, C, dtype=x_t.dtype, device=x_t.device)
        wd = w.detach().to(torch.bfloat16).contiguous()
        rc = _lib.load().lb_conv1d_update(x_t.data_ptr(), x_t.stride(0), conv_state.data_ptr(), wd.data_ptr(),
                                          out.data_ptr(), C, N, C, W, int(act), _lib.stream_ptr())
        _lib.check(rc, "lb_conv1d_update")
        return out
    return conv1d_update_ref(x_t, conv_state, w, act)


def conv_states_ref(x, lengths, width):
    ends = torch.cumsum(lengths, 0)
    starts = ends - lengths
    idx = ends.view(-1, 1) - width + torch.arange(width, device=x.device).view(1, -1)  # [n, width]
    valid = idx >= starts.view(-1, 1)
    g = x[idx.clamp(min=0)]  # [n, width, C]
    g = torch.where(valid.unsqueeze(-1), g, torch.zeros_like(g))
    return g.permute(0, 2, 1).contiguous()


def conv_states_from_packed(x: torch.Tensor, lengths: torch.Tensor, width: int) -> torch.Tensor:
    """Last ``width`` inputs of every document of a packed sequence x [T, C] -> [n_docs, C, width]
    (zero-padded on the left for documents shorter than the window)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1:
        ends = torch.cumsum(lengths.to(torch.int64), 0).contiguous()
        starts = (ends - lengths.to(torch.int64)).contiguous()
        n, C = lengths.numel(), x.shape[1]
        out = torch.empty(n, C, width, dtype=x.dtype, device=x.device)
        rc = _lib.load().lb_conv_states(x.data_ptr(), x.stride(0), starts.data_ptr(), ends.data_ptr(), out.data_ptr(),
                                        n, C, width, _lib.stream_ptr())
        _lib.check(rc, "lb_conv_states")
        return out
    return conv_states_ref(x, lengths, width)


def rnn_step(a: torch.Tensor, b: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """One step of h = a * h + b on the cached fp32 ``state`` [N, C] (updated in place); a, b: [N, C]."""
    if a.is_cuda and a.dtype == torch.bfloat16 and state.dtype == torch.float32 and state.is_contiguous():
        a, b = a.contiguous(), b.contiguous()
        out = torch.empty_like(a)
        rc = _lib.load().lb_rnn_step(a.data_ptr(), b.data_ptr(), state.data_ptr(), out.data_ptr(), a.numel(),
                                     _lib.stream_ptr())
        _lib.check(rc, "lb_rnn_step")
        return out
    h = a.float() * state + b.float()
    state.copy_(h)
    return h.to(a.dtype)


# ----------------------------------------------------------------------------- RG-LRU gates
_MAX_SQRT_GRADIENT = 1000.0


def rglru_gates_ref(gx, ga, x, sp, c: float = 8.0):
    """(a, b) of the RG-LRU recurrence from the gate pre-activations; differentiable PyTorch version."""
    gate_x = torch.sigmoid(gx.float())
    gate_a = torch.sigmoid(ga.float())
    log_a = -c * gate_a * sp.float().view(*([1] * (gx.dim() - 1)), -1)
    a = log_a.exp()
    mult = _SqrtBound.apply(1.0 - (2.0 * log_a).exp())
    return a.to(x.dtype), (mult * gate_x * x.float()).to(x.dtype)


class _SqrtBound(torch.autograd.Function):
    """sqrt whose gradient is clipped at 1000 (1 - a^2 can reach 0)."""

    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return torch.sqrt(x)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return g / torch.sqrt(torch.clip(4.0 * x, min=1 / (_MAX_SQRT_GRADIENT ** 2)))


class _RglruGates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gx, ga, x, sp):
        gx, ga, x = gx.contiguous(), ga.contiguous(), x.contiguous()
        sp = sp.float().contiguous()
        C = x.shape[-1]
        a, b = torch.empty_like(x), torch.empty_like(x)
        rc = _lib.load().lb_rglru_gates_fwd(gx.data_ptr(), ga.data_ptr(), x.data_ptr(), sp.data_ptr(), a.data_ptr(),
                                            b.data_ptr(), x.numel() // C, C, _lib.stream_ptr())
        _lib.check(rc, "lb_rglru_gates_fwd")
        ctx.save_for_backward(gx, ga, x, sp)
        return a, b

    @staticmethod
    def backward(ctx, da, db):
        gx, ga, x, sp = ctx.saved_tensors
        C = x.shape[-1]
        da, db = da.contiguous(), db.contiguous()
        dgx, dga, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        dsp = torch.zeros(C, dtype=torch.float32, device=x.device)
        rc = _lib.load().lb_rglru_gates_bwd(gx.data_ptr(), ga.data_ptr(), x.data_ptr(), sp.data_ptr(), da.data_ptr(),
                                            db.data_ptr(), dgx.data_ptr(), dga.data_ptr(), dx.data_ptr(),
                                            dsp.data_ptr(), x.numel() // C, C, _lib.stream_ptr())
        _lib.check(rc, "lb_rglru_gates_bwd")
        return dgx, dga, dx, dsp


def rglru_gates(gx: torch.Tensor, ga: torch.Tensor, x: torch.Tensor, sp: torch.Tensor):
    """a = exp(-8 sigmoid(ga) sp), b = sqrt(1 - a^2) sigmoid(gx) x for [..., C] gate pre-activations ``gx``, ``ga``,
    the input ``x`` and ``sp`` = softplus(lambda) per channel ([C], fp32). One kernel each way on the GPU."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RglruGates.apply(gx, ga, x, sp)
    return rglru_gates_ref(gx, ga, x, sp)


# ----------------------------------------------------------------------------- linear recurrence
def scan_ref(a, b, doc_start=None, h0=None):
    """h_t = a_t h_{t-1} + b_t along dim 1 of [B, S, C]; differentiable, fp32 math."""
    B, S, C = a.shape
    af, bf = a.float(), b.float()
    if doc_start is not None:
        first = doc_start.view(B, S) == torch.arange(S, device=a.device).view(1, S)
        af = torch.where(first.unsqueeze(-1), torch.zeros_like(af), af)
    h = h0.float() if h0 is not None else torch.zeros(B, C, device=a.device)
    out = []
    for s in range(S):
        h = af[:, s] * h + bf[:, s]
        out.append(h)
    return torch.stack(out, dim=1).to(a.dtype)


def _scratch(B, S, C, device):
    n_chunks = (S + 63) // 64
    return torch.empty(2 * B * n_chunks * C, dtype=torch.float32, device=device)


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, doc_start, h0):
        B, S, C = a.shape
        a, b = a.contiguous(), b.contiguous()
        h = torch.empty_like(a)
        rc = _lib.load().lb_scan_fwd(a.data_ptr(), b.data_ptr(), _ptr(doc_start), _ptr(h0), h.data_ptr(), None,
                                     _scratch(B, S, C, a.device).data_ptr(), B, S, C, _lib.stream_ptr())
        _lib.check(rc, "lb_scan_fwd")
        ctx.save_for_backward(a, h, doc_start, h0)
        return h

    @staticmethod
    def backward(ctx, dh):
        a, h, doc_start, h0 = ctx.saved_tensors
        B, S, C = a.shape
        dh = dh.contiguous()
        da, db = torch.empty_like(a), torch.empty_like(a)
        rc = _lib.load().lb_scan_bwd(a.data_ptr(), h.data_ptr(), dh.data_ptr(), _ptr(doc_start), _ptr(h0),
                                     da.data_ptr(), db.data_ptr(), _scratch(B, S, C, a.device).data_ptr(), B, S, C,
                                     _lib.stream_ptr())
        _lib.check(rc, "lb_scan_bwd")
        return da, db, None, None


def linear_scan(a: torch.Tensor, b: torch.Tensor, doc_start: Optional[torch.Tensor] = None,
                h0: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h_t = a_t * h_{t-1} + b_t for every channel; a, b: [B, S, C]; h0: optional fp32 [B, C]."""
    if a.is_cuda and a.dtype == torch.bfloat16:
        ds = doc_start.reshape(-1).int().contiguous() if doc_start is not None else None
        return _Scan.apply(a, b, ds, h0.float().contiguous() if h0 is not None else None)
    return scan_ref(a, b, doc_start, h0)


def last_states_from_packed(h: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
    """h: [T, C] states of a packed sequence -> state after the last token of every document."""
    return h[torch.cumsum(lengths, 0) - 1]
