"""Mamba-2 state-space duality (SSD): chunked scan, sequential reference and the decode update.

The recurrence per head (state h in R^{P x N}):

    h_t = exp(dt_t A) h_{t-1} + dt_t x_t B_t^T ,   y_t = h_t C_t + D x_t

``ssd_chunked`` evaluates it in chunks of ``chunk`` tokens: inside a chunk as masked matrix
products (C B^T with the decay kernel, then times x), between chunks through the P x N chunk
states - the algorithm behind ``mamba_chunk_scan_combined`` used by
apps/mamba/component/ssm_compilable.py:22-40 and apps/mamba/core_mamba.py:254-273. All four
matrix products run as batched GEMMs on this library's tcgen05 kernel (``BmmFn``) when the inputs
are CUDA bf16, and gradients flow through the same kernel; the decay / masking arithmetic is fp32
PyTorch. Documents packed in a sequence (``doc_start``) neither mix inside a chunk nor through
the carried state.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as TF

from .gemm import gemm


class BmmFn(torch.autograd.Function):
    """``a @ b^T`` for a [..., M, K], b [..., N, K] (up to two batch dims), bf16 on the native GEMM."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm(a, b)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy.contiguous()
        da = gemm(dy, b.transpose(-1, -2)) if ctx.needs_input_grad[0] else None  # [.., M, N] @ [.., N, K]
        db = gemm(dy.transpose(-1, -2), a.transpose(-1, -2)) if ctx.needs_input_grad[1] else None
        return da, db


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def bmm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched ``a @ b^T``; the native kernel needs contiguous rows whose length is a multiple of 8."""
    if _native(a) and _native(b) and a.shape[-1] % 8 == 0 and a.shape[-2] % 8 == 0 and b.shape[-2] % 8 == 0:
        lead = a.shape[:-2]
        a3 = a.reshape(-1, *a.shape[-2:]).contiguous()
        b3 = b.reshape(-1, *b.shape[-2:]).contiguous()
        return BmmFn.apply(a3, b3).view(*lead, a.shape[-2], b.shape[-2])
    return torch.matmul(a, b.transpose(-1, -2))


def ssd_ref(x, dt, A, B, C, D=None, doc_start=None, initial_states=None):
    """Token-by-token recurrence in fp64. x [b,s,h,p], dt [b,s,h], A [h], B/C [b,s,g,n]."""
    b, s, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    rep = h // g
    xd, dtd, Ad = x.double(), dt.double(), A.double()
    Bd = B.double().repeat_interleave(rep, dim=2)
    Cd = C.double().repeat_interleave(rep, dim=2)
    state = torch.zeros(b, h, p, n, dtype=torch.float64, device=x.device)
    if initial_states is not None:
        state = state + initial_states.double()
    ys = []
    for t in range(s):
        if doc_start is not None:
            new = (doc_start[:, t] == t).view(b, 1, 1, 1)
            state = torch.where(new, torch.zeros_like(state), state)
        decay = torch.exp(dtd[:, t] * Ad).view(b, h, 1, 1)
        state = decay * state + (dtd[:, t].view(b, h, 1, 1) * xd[:, t].unsqueeze(-1)) * Bd[:, t].unsqueeze(2)
        ys.append((state * Cd[:, t].unsqueeze(2)).sum(-1))
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + (D.double().view(1, 1, h, -1) * xd)
    return y.to(x.dtype), state


def ssd_chunked(x, dt, A, B, C, D=None, chunk: int = 256, doc_start: Optional[torch.Tensor] = None,
                initial_states: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (y [b,s,h,p], final state [b,h,p,n] fp32). ``dt`` is already positive (softplus applied)."""
    b, s, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    rep = h // g
    L = min(chunk, s)
    pad = (-s) % L
    if pad:
        # padded steps have dt = 0: they neither decay nor feed the state
        x = TF.pad(x, (0, 0, 0, 0, 0, pad))
        dt = TF.pad(dt, (0, 0, 0, pad))
        B = TF.pad(B, (0, 0, 0, 0, 0, pad))
        C = TF.pad(C, (0, 0, 0, 0, 0, pad))
        if doc_start is not None:
            # padding continues the last document, so the final state is that document's state
            doc_start = torch.cat([doc_start, doc_start[:, -1:].expand(-1, pad)], dim=1)
    sp = s + pad
    nc = sp // L
    cdt = x.dtype
    dtf = dt.float()
    dA = (dtf * A.float().view(1, 1, h)).view(b, nc, L, h).permute(0, 3, 1, 2)  # b h c l
    cs = torch.cumsum(dA, dim=-1)
    xdt = (x.float() * dtf.unsqueeze(-1)).to(cdt).view(b, nc, L, h, p)
    Bc = B.view(b, nc, L, g, n)
    Cc = C.view(b, nc, L, g, n)
    if doc_start is not None:
        doc = doc_start.view(b, nc, L)
        same = doc.unsqueeze(-1) == doc.unsqueeze(-2)  # b c l s
        same_as_last = doc == doc[:, :, -1:]  # b c l
        prev_last = torch.cat([torch.full_like(doc[:, :1, -1], -1), doc[:, :-1, -1]], dim=1)  # b c
        from_prev = doc == prev_last.unsqueeze(-1)  # token continues the document carried in
        cont = doc[:, :, -1] == prev_last  # whole chunk continues it
    # 1) inside a chunk: scores = C B^T (per group), kernel = exp(cs_l - cs_s) for l >= s
    scores = bmm_nt(Cc.permute(0, 1, 3, 2, 4).reshape(b * nc, g, L, n), Bc.permute(0, 1, 3, 2, 4).reshape(b * nc, g, L, n))
    scores = scores.view(b, nc, g, L, L).float()
    seg = cs.unsqueeze(-1) - cs.unsqueeze(-2)  # b h c l s
    tri = torch.tril(torch.ones(L, L, dtype=torch.bool, device=x.device))
    kern = torch.where(tri, torch.exp(seg.masked_fill(~tri, 0.0)), torch.zeros((), device=x.device))
    if doc_start is not None:
        kern = kern * same.unsqueeze(1)
    w = (scores.repeat_interleave(rep, dim=2).permute(0, 2, 1, 3, 4) * kern).to(cdt)  # b h c l s
    xh = xdt.permute(0, 3, 1, 4, 2)  # b h c p l  ([N=p, K=l] operand)
    y_diag = bmm_nt(w.reshape(b * h, nc, L, L), xh.reshape(b * h, nc, p, L))  # b*h c l p
    # 2) state contributed by each chunk: sum_l exp(cs_last - cs_l) B_l (dt x)_l^T
    decay_to_end = torch.exp(cs[..., -1:] - cs)  # b h c l
    if doc_start is not None:
        decay_to_end = decay_to_end * same_as_last.unsqueeze(1)
    xw = (xdt.float() * decay_to_end.permute(0, 2, 3, 1).unsqueeze(-1)).to(cdt)  # b c l h p
    Bh = Bc.repeat_interleave(rep, dim=3)  # b c l h n
    chunk_states = bmm_nt(xw.permute(0, 3, 1, 4, 2).reshape(b * h, nc, p, L),
                          Bh.permute(0, 3, 1, 4, 2).reshape(b * h, nc, n, L)).view(b, h, nc, p, n).float()
    # 3) carry the state over chunks (nc sequential steps on small tensors)
    chunk_decay = torch.exp(cs[..., -1])  # b h c
    if doc_start is not None:
        chunk_decay = chunk_decay * cont.unsqueeze(1)
    state = initial_states.float() if initial_states is not None else torch.zeros(b, h, p, n, device=x.device)
    carried = []
    for c in range(nc):
        carried.append(state)
        state = chunk_decay[:, :, c].view(b, h, 1, 1) * state + chunk_states[:, :, c]
    prev_states = torch.stack(carried, dim=2).to(cdt)  # b h c p n
    # 4) contribution of the carried state: (C_l . state) * exp(cs_l)
    Ch = Cc.repeat_interleave(rep, dim=3).permute(0, 3, 1, 2, 4)  # b h c l n
    y_off = bmm_nt(Ch.reshape(b * h, nc, L, n), prev_states.reshape(b * h, nc, p, n)).view(b, h, nc, L, p).float()
    out_decay = torch.exp(cs)
    if doc_start is not None:
        out_decay = out_decay * from_prev.unsqueeze(1)
    y = y_diag.view(b, h, nc, L, p).float() + y_off * out_decay.unsqueeze(-1)
    y = y.permute(0, 2, 3, 1, 4).reshape(b, sp, h, p)
    if D is not None:
        y = y + D.float().view(1, 1, h, -1) * x.float()
    return y[:, :s].to(cdt), state


def selective_state_update(state, x, dt, A, B, C, D=None):
    """One decode step. state [n, h, p, N] (updated in place, fp32); x [n,h,p]; dt [n,h]; B/C [n,g,N]."""
    nseq, h, p = x.shape
    rep = h // B.shape[1]
    Bh = B.float().repeat_interleave(rep, dim=1)
    Ch = C.float().repeat_interleave(rep, dim=1)
    dtf = dt.float()
    decay = torch.exp(dtf * A.float().view(1, h)).view(nseq, h, 1, 1)
    state.mul_(decay).add_((dtf.view(nseq, h, 1, 1) * x.float().unsqueeze(-1)) * Bh.unsqueeze(2))
    y = (state * Ch.unsqueeze(2)).sum(-1)
    if D is not None:
        y = y + D.float().view(1, h, -1) * x.float()
    return y.to(x.dtype)
