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


def _lib_ssd():
    import ctypes as C

    from . import _lib

    lib = _lib.load()
    if not getattr(lib, "_ssd_declared", False):
        lib.lb_ssd_decay_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_int, C.c_void_p]
        lib.lb_ssd_decay_fwd.restype = C.c_int
        lib.lb_ssd_decay_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        lib.lb_ssd_decay_bwd.restype = C.c_int
        lib._ssd_declared = True
    return lib


def decay_weights_ref(scores, cs, doc):
    """W[b,c,h,l,s] = scores[b,c,g(h),l,s] * exp(cs[b,h,c,l] - cs[b,h,c,s]) for s <= l in the same document."""
    b, nc, g, L, _ = scores.shape
    h = cs.shape[1]
    seg = cs.unsqueeze(-1) - cs.unsqueeze(-2)  # b h c l s
    tri = torch.tril(torch.ones(L, L, dtype=torch.bool, device=scores.device))
    kern = torch.where(tri, torch.exp(seg.masked_fill(~tri, 0.0)), torch.zeros((), device=scores.device))
    if doc is not None:
        kern = kern * (doc.unsqueeze(-1) == doc.unsqueeze(-2)).unsqueeze(1)
    return scores.float().repeat_interleave(h // g, dim=2) * kern.permute(0, 2, 1, 3, 4)


class SsdDecayFn(torch.autograd.Function):
    """(scores bf16 [b, nc, g, L, L], cs fp32 [b, h, nc, L], doc int32 [b, nc, L] | None) -> W bf16 [b, nc, h, L, L].

    One kernel each way (``csrc/ssd.cu``): nothing of size [b, h, nc, L, L] other than W and its gradient exists."""

    @staticmethod
    def forward(ctx, scores, cs, doc):
        from . import _lib

        b, nc, g, L, _ = scores.shape
        h = cs.shape[1]
        scores, cs = scores.contiguous(), cs.contiguous()
        doc = doc.contiguous() if doc is not None else None
        w = torch.empty(b, nc, h, L, L, dtype=torch.bfloat16, device=scores.device)
        _lib.check(_lib_ssd().lb_ssd_decay_fwd(scores.data_ptr(), cs.data_ptr(), None if doc is None else doc.data_ptr(),
                                               w.data_ptr(), b, h, g, nc, L, _lib.stream_ptr()), "lb_ssd_decay_fwd")
        ctx.save_for_backward(scores, cs, doc)
        return w

    @staticmethod
    def backward(ctx, dw):
        from . import _lib

        scores, cs, doc = ctx.saved_tensors
        b, nc, g, L, _ = scores.shape
        h = cs.shape[1]
        dw = dw.contiguous()
        dscores = torch.zeros(scores.shape, dtype=torch.float32, device=scores.device)
        dcs = torch.zeros_like(cs)
        _lib.check(_lib_ssd().lb_ssd_decay_bwd(dw.data_ptr(), scores.data_ptr(), cs.data_ptr(),
                                               None if doc is None else doc.data_ptr(), dscores.data_ptr(),
                                               dcs.data_ptr(), b, h, g, nc, L, _lib.stream_ptr()), "lb_ssd_decay_bwd")
        return dscores.to(scores.dtype), dcs, None


def decay_weights(scores, cs, doc):
    """bf16 W for the intra-chunk product; fused kernel on CUDA bf16, PyTorch otherwise."""
    L = scores.shape[-1]
    if _native(scores) and L % 8 == 0 and L <= 512:
        return SsdDecayFn.apply(scores, cs.float(), None if doc is None else doc.int())
    return decay_weights_ref(scores, cs, doc).to(scores.dtype)


def bmm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched ``a @ b^T``; the native kernel needs contiguous rows whose length is a multiple of 8."""
    if _native(a) and _native(b) and a.shape[-1] % 8 == 0 and a.shape[-2] % 8 == 0 and b.shape[-2] % 8 == 0:
        lead = a.shape[:-2]
        a3 = a.reshape(-1, *a.shape[-2:]).contiguous()
        b3 = b.reshape(-1, *b.shape[-2:]).contiguous()
        return BmmFn.apply(a3, b3).view(*lead, a.shape[-2], b.shape[-2])
    return torch.matmul(a, b.transpose(-1, -2))


def _tma_ok(t: torch.Tensor) -> bool:
    if not _native(t) or t.data_ptr() % 16:
        return False
    st = t.stride()
    if st[-1] == 1:
        lead = [st[-2]] + list(st[:-2])
    elif st[-2] == 1:
        lead = [st[-1]] + list(st[:-2])
    else:
        return False
    return all(v % 8 == 0 for v in lead)


def mm_views(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b^T`` for 4-D strided views a [b0, b1, M, K], b [b0, b1, N, K] without copying them when the
    tcgen05 GEMM can read them in place (unit stride along M/N or K, 16-byte aligned pitches)."""
    if _tma_ok(a) and _tma_ok(b) and a.shape[-2] % 8 == 0 and b.shape[-2] % 8 == 0 and a.shape[-1] % 8 == 0:
        return BmmFn.apply(a, b)
    if a.is_cuda and a.dtype == torch.bfloat16:
        return bmm_nt(a, b)
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
    hp = rep * p  # rows of one group's heads folded into one matrix dimension
    # 1) inside a chunk: scores = C B^T (per group), W = scores o decay kernel (lower triangle, same document)
    Cg = Cc.permute(0, 1, 3, 2, 4).reshape(b * nc, g, L, n)  # views: (b, nc) merge without a copy
    Bg = Bc.permute(0, 1, 3, 2, 4).reshape(b * nc, g, L, n)
    scores = mm_views(Cg, Bg)  # [b*nc, g, L, L]
    w = decay_weights(scores.view(b, nc, g, L, L), cs, doc if doc_start is not None else None)  # b c h l s
    xh = xdt.permute(0, 1, 3, 4, 2).reshape(b * nc, h, p, L)  # [N=p, K=l] operand, read in place
    y_diag = mm_views(w.reshape(b * nc, h, L, L), xh)  # [b*nc, h, L, p]
    # 2) state contributed by each chunk: sum_l exp(cs_last - cs_l) B_l (dt x)_l^T, all heads of a group at once
    decay_to_end = torch.exp(cs[..., -1:] - cs)  # b h c l
    if doc_start is not None:
        decay_to_end = decay_to_end * same_as_last.unsqueeze(1)
    xw = (xdt.float() * decay_to_end.permute(0, 2, 3, 1).unsqueeze(-1)).to(cdt)  # b c l h p
    xw_g = xw.view(b * nc, L, g, hp).permute(0, 2, 3, 1)  # [b*nc, g, M=hp, K=l]
    Bt = Bc.reshape(b * nc, L, g, n).permute(0, 2, 3, 1)  # [b*nc, g, N=n, K=l]
    chunk_states = mm_views(xw_g, Bt).view(b, nc, h, p, n).float()
    # 3) carry the state over chunks (nc sequential steps on small tensors)
    chunk_decay = torch.exp(cs[..., -1])  # b h c
    if doc_start is not None:
        chunk_decay = chunk_decay * cont.unsqueeze(1)
    state = initial_states.float() if initial_states is not None else torch.zeros(b, h, p, n, device=x.device)
    carried = []
    for c in range(nc):
        carried.append(state)
        state = chunk_decay[:, :, c].view(b, h, 1, 1) * state + chunk_states[:, c]
    prev_states = torch.stack(carried, dim=1).to(cdt)  # b c h p n
    # 4) contribution of the carried state: (C_l . state) * exp(cs_l)
    y_off = mm_views(Cg, prev_states.view(b * nc, g, hp, n))  # [b*nc, g, L, hp]
    out_decay = torch.exp(cs)
    if doc_start is not None:
        out_decay = out_decay * from_prev.unsqueeze(1)
    y = (y_diag.view(b, nc, h, L, p).permute(0, 1, 3, 2, 4).float()
         + y_off.view(b, nc, g, L, rep, p).permute(0, 1, 3, 2, 4, 5).reshape(b, nc, L, h, p).float()
         * out_decay.permute(0, 2, 3, 1).unsqueeze(-1))
    y = y.reshape(b, sp, h, p)
    if D is not None:
        y = y + D.float().view(1, 1, h, -1) * x.float()
    return y[:, :s].to(cdt), state


def selective_state_update(state, x, dt, A, B, C, D=None):
    """One decode step. state [n, h, p, N] (updated in place, fp32); x [n,h,p]; dt [n,h]; B/C [n,g,N]."""
    nseq, h, p = x.shape
    N = state.shape[-1]
    if (x.is_cuda and x.dtype == torch.bfloat16 and state.dtype == torch.float32 and state.is_contiguous()
            and N % 4 == 0 and x.stride(2) == 1 and x.stride(1) == p and B.stride(2) == 1 and B.stride(1) == N
            and C.stride(2) == 1 and C.stride(1) == N and B.dtype == torch.bfloat16 and C.dtype == torch.bfloat16
            and B.stride(0) % 4 == 0 and C.stride(0) % 4 == 0 and B.data_ptr() % 8 == 0 and C.data_ptr() % 8 == 0):
        from . import _lib

        y = torch.empty(nseq, h, p, dtype=x.dtype, device=x.device)
        dtf, Af = dt.float().contiguous(), A.float().contiguous()
        Df = D.float().contiguous() if D is not None else None
        rc = _lib.load().lb_ssm_state_update(state.data_ptr(), x.data_ptr(), x.stride(0), dtf.data_ptr(), Af.data_ptr(),
                                             B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0),
                                             None if Df is None else Df.data_ptr(), int(Df is not None and Df.dim() == 2),
                                             y.data_ptr(), nseq, h, p, N, B.shape[1], _lib.stream_ptr())
        _lib.check(rc, "lb_ssm_state_update")
        return y
    return selective_state_update_ref(state, x, dt, A, B, C, D)


def selective_state_update_ref(state, x, dt, A, B, C, D=None):
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
