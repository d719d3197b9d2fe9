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


# ----------------------------------------------------------------------------- fused glue of the chunked scan
def _lib_glue():
    import ctypes as C

    from . import _lib

    lib = _lib.load()
    if not getattr(lib, "_ssd_glue_declared", False):
        vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
        lib.lb_ssd_prep_fwd.argtypes = [vp, ll, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, vp]
        lib.lb_ssd_prep_bwd.argtypes = [vp, ll, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, vp]
        lib.lb_ssd_carry_fwd.argtypes = [vp, vp, vp, vp, vp, i, i, i, ll, vp]
        lib.lb_ssd_carry_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, ll, vp]
        lib.lb_ssd_combine_fwd.argtypes = [vp, vp, vp, vp, vp, ll, vp, i, vp, i, i, i, i, i, i, i, vp]
        lib.lb_ssd_combine_bwd.argtypes = [vp, vp, vp, vp, vp, ll, vp, i, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, vp]
        for name in ("prep_fwd", "prep_bwd", "carry_fwd", "carry_bwd", "combine_fwd", "combine_bwd"):
            getattr(lib, "lb_ssd_" + name).restype = C.c_int
        lib._ssd_glue_declared = True
    return lib


def _p(t):
    return None if t is None else t.data_ptr()


class SsdPrepFn(torch.autograd.Function):
    """(x [b,s,h,p] bf16 with any token pitch, dt [b,s,h] fp32, A [h] fp32, doc int32 [b,nc,L] | None) ->
    cs fp32 [b,h,nc,L], xdt = x dt and xw = xdt exp(cs_last - cs) (bf16, [b,s,h,p] contiguous). One kernel each way."""

    @staticmethod
    def forward(ctx, x, dt, A, doc, L):
        from . import _lib

        b, s, h, p = x.shape
        nc = s // L
        dt, A = dt.contiguous(), A.contiguous()
        cs = torch.empty(b, h, nc, L, dtype=torch.float32, device=x.device)
        xdt = torch.empty(b, s, h, p, dtype=torch.bfloat16, device=x.device)
        xw = torch.empty_like(xdt)
        _lib.check(_lib_glue().lb_ssd_prep_fwd(x.data_ptr(), x.stride(1), dt.data_ptr(), A.data_ptr(), _p(doc),
                                               cs.data_ptr(), xdt.data_ptr(), xw.data_ptr(), b, s, h, p, nc, L,
                                               _lib.stream_ptr()), "lb_ssd_prep_fwd")
        ctx.save_for_backward(x, dt, A, doc, cs)
        ctx.L = L
        return cs, xdt, xw

    @staticmethod
    def backward(ctx, d_cs, d_xdt, d_xw):
        from . import _lib

        x, dt, A, doc, cs = ctx.saved_tensors
        b, s, h, p = x.shape
        L = ctx.L
        d_cs = d_cs.contiguous() if d_cs is not None else None
        d_xdt = d_xdt.contiguous() if d_xdt is not None else None
        d_xw = d_xw.contiguous() if d_xw is not None else None
        dx = torch.empty(b, s, h, p, dtype=torch.bfloat16, device=x.device)
        ddt = torch.empty_like(dt)
        dA = torch.zeros_like(A)
        _lib.check(_lib_glue().lb_ssd_prep_bwd(x.data_ptr(), x.stride(1), dt.data_ptr(), A.data_ptr(), _p(doc),
                                               cs.data_ptr(), _p(d_cs), _p(d_xdt), _p(d_xw), dx.data_ptr(),
                                               ddt.data_ptr(), dA.data_ptr(), b, s, h, p, s // L, L,
                                               _lib.stream_ptr()), "lb_ssd_prep_bwd")
        return dx, ddt, dA, None, None


class SsdCarryFn(torch.autograd.Function):
    """State handed from chunk to chunk. T bf16 [b,nc,h,p,n] (state contributed by each chunk), a fp32 [b,h,nc]
    (decay over the chunk, zero where the chunk starts a new document), init fp32 [b,h,p,n] | None ->
    prev bf16 [b,nc,h,p,n] (state entering each chunk), final fp32 [b,h,p,n]."""

    @staticmethod
    def forward(ctx, T, a, init):
        from . import _lib

        b, nc, h, p, n = T.shape
        T, a = T.contiguous(), a.contiguous()
        init = init.float().contiguous() if init is not None else None
        prev = torch.empty_like(T)
        fin = torch.empty(b, h, p, n, dtype=torch.float32, device=T.device)
        _lib.check(_lib_glue().lb_ssd_carry_fwd(T.data_ptr(), a.data_ptr(), _p(init), prev.data_ptr(), fin.data_ptr(),
                                                b, h, nc, p * n, _lib.stream_ptr()), "lb_ssd_carry_fwd")
        ctx.save_for_backward(prev, a)
        ctx.has_init = init is not None
        return prev, fin

    @staticmethod
    def backward(ctx, d_prev, d_fin):
        from . import _lib

        prev, a = ctx.saved_tensors
        b, nc, h, p, n = prev.shape
        d_prev = d_prev.contiguous() if d_prev is not None else None
        d_fin = d_fin.float().contiguous() if d_fin is not None else None
        dT = torch.empty_like(prev)
        da = torch.zeros_like(a)
        d_init = torch.empty(b, h, p, n, dtype=torch.float32, device=prev.device) if ctx.has_init else None
        _lib.check(_lib_glue().lb_ssd_carry_bwd(prev.data_ptr(), a.data_ptr(), _p(d_prev), _p(d_fin), dT.data_ptr(),
                                                da.data_ptr(), _p(d_init), b, h, nc, p * n, _lib.stream_ptr()),
                   "lb_ssd_carry_bwd")
        return dT, da, d_init


class SsdCombineFn(torch.autograd.Function):
    """y = y_diag + y_off exp(cs) (for tokens that continue the carried document) + D x, as bf16 [b,s,h,p].
    y_diag bf16 [b,nc,h,L,p], y_off bf16 [b,nc,g,L,(h/g) p], cs fp32 [b,h,nc,L], x [b,s,h,p], D [h] | [h,p] | None."""

    @staticmethod
    def forward(ctx, y_diag, y_off, cs, doc, x, D):
        from . import _lib

        b, nc, h, L, p = y_diag.shape
        g = y_off.shape[2]
        y_diag, y_off = y_diag.contiguous(), y_off.contiguous()
        Df = D.float().contiguous() if D is not None else None
        y = torch.empty(b, nc * L, h, p, dtype=torch.bfloat16, device=x.device)
        _lib.check(_lib_glue().lb_ssd_combine_fwd(y_diag.data_ptr(), y_off.data_ptr(), cs.data_ptr(), _p(doc),
                                                  x.data_ptr(), x.stride(1), _p(Df), int(Df is not None and Df.dim() == 2),
                                                  y.data_ptr(), b, nc * L, h, g, p, nc, L, _lib.stream_ptr()),
                   "lb_ssd_combine_fwd")
        ctx.save_for_backward(y_off, cs, doc, x, Df)
        ctx.dims = (b, nc, h, L, p, g)
        ctx.d_dtype = D.dtype if D is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import _lib

        y_off, cs, doc, x, Df = ctx.saved_tensors
        b, nc, h, L, p, g = ctx.dims
        dy = dy.contiguous()
        d_ydiag = torch.empty(b, nc, h, L, p, dtype=torch.bfloat16, device=dy.device)
        d_yoff = torch.empty_like(y_off)
        dcs = torch.empty_like(cs)
        dx_d = torch.empty(b, nc * L, h, p, dtype=torch.bfloat16, device=dy.device) if Df is not None else None
        dD = torch.zeros_like(Df) if Df is not None else None
        _lib.check(_lib_glue().lb_ssd_combine_bwd(dy.data_ptr(), y_off.data_ptr(), cs.data_ptr(), _p(doc), x.data_ptr(),
                                                  x.stride(1), _p(Df), int(Df is not None and Df.dim() == 2),
                                                  d_ydiag.data_ptr(), d_yoff.data_ptr(), dcs.data_ptr(), _p(dx_d), _p(dD),
                                                  b, nc * L, h, g, p, nc, L, _lib.stream_ptr()), "lb_ssd_combine_bwd")
        return d_ydiag, d_yoff, dcs, None, dx_d, (dD.to(ctx.d_dtype) if dD is not None else None)


def _glue_ok(x, dt, B, C, L) -> bool:
    b, s, h, p = x.shape
    return (_native(x) and _native(B) and _native(C) and dt.dtype == torch.float32 and s % L == 0 and L <= 1024
            and p % 8 == 0 and p <= 256 and 32 % (p // 8) == 0 and (p * B.shape[3]) % 4 == 0
            and x.stride(3) == 1 and x.stride(2) == p and x.stride(0) == s * x.stride(1) and x.stride(1) % 8 == 0)


def _ssd_chunked_fused(x, dt, A, B, C, D, L, doc_start, initial_states):
    """The chunked scan as four batched tcgen05 GEMMs, the decay kernel and the three glue kernels of
    ``csrc/ssd_glue.cu``; every step has a hand-written backward, nothing else runs per token."""
    b, s, h, p = x.shape
    g, n = B.shape[2], B.shape[3]
    rep, nc, hp = h // g, s // L, (h // g) * p
    doc = doc_start.reshape(b, nc, L).int().contiguous() if doc_start is not None else None
    cs, xdt, xw = SsdPrepFn.apply(x, dt, A.float(), doc, L)
    Cg = C.view(b, nc, L, g, n).permute(0, 1, 3, 2, 4).reshape(b * nc, g, L, n)  # views: (b, nc) merge without a copy
    Bg = B.view(b, nc, L, g, n).permute(0, 1, 3, 2, 4).reshape(b * nc, g, L, n)
    scores = mm_views(Cg, Bg)  # [b*nc, g, L, L]
    w = decay_weights(scores.view(b, nc, g, L, L), cs, doc)  # [b, nc, h, L, L]
    xh = xdt.view(b, nc, L, h, p).permute(0, 1, 3, 4, 2).reshape(b * nc, h, p, L)
    y_diag = mm_views(w.reshape(b * nc, h, L, L), xh)  # [b*nc, h, L, p]
    xw_g = xw.view(b * nc, L, g, hp).permute(0, 2, 3, 1)  # [b*nc, g, M=hp, K=l]
    Bt = B.reshape(b * nc, L, g, n).permute(0, 2, 3, 1)  # [b*nc, g, N=n, K=l]
    T = mm_views(xw_g, Bt).reshape(b, nc, h, p, n)
    a = torch.exp(cs[..., -1])  # b h c: decay over a whole chunk
    if doc is not None:
        prev_last = torch.cat([torch.full_like(doc[:, :1, -1], -1), doc[:, :-1, -1]], dim=1)
        a = a * (doc[:, :, -1] == prev_last).unsqueeze(1)
    prev, final = SsdCarryFn.apply(T, a, initial_states)
    y_off = mm_views(Cg, prev.view(b * nc, g, hp, n))  # [b*nc, g, L, hp]
    y = SsdCombineFn.apply(y_diag.view(b, nc, h, L, p), y_off.view(b, nc, g, L, hp), cs, doc, x, D)
    return y, final


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
    if _glue_ok(x, dt, B, C, L) and L % 8 == 0 and L <= 512:
        y, state = _ssd_chunked_fused(x, dt, A, B.contiguous() if not B.is_contiguous() else B,
                                      C.contiguous() if not C.is_contiguous() else C, D, L, doc_start, initial_states)
        return y[:, :s], state
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
