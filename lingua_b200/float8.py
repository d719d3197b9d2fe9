"""Float8 (e4m3) matmuls for linear layers, row-wise scaled.

What is computed follows lingua/float8.py:83-141 (``Fp8LinearFn``):

* forward        ``out = q(x) q(W)^T`` with one scale per row of ``x`` and one per output feature of ``W``;
* input gradient ``dx = q(dy) q(W^T)^T`` with one scale per row of ``dy`` and a single scale for the whole
                 weight (the reference reduces its per-feature maxima to one value for this product);
* weight gradient stays in bf16.

A scale is ``max(|row|, 1e-12) / 448`` and the operand is divided by it before rounding to e4m3.
On a GPU the products run on this library's tcgen05 ``kind::f8f6f4`` kernel with both scale vectors applied
in its epilogue, and the quantisation runs in one pass per operand (``csrc/gemm_fp8.cu``); on CPU the same
arithmetic is spelled out in PyTorch, which is also the reference the kernels are tested against.

``convert_linears_to_fp8`` (lingua/float8.py:151-191) marks the weights of every matching linear layer;
the fused blocks of the model (``ops/fused.py``) consult that mark, and stand-alone ``Linear`` modules are
switched to ``Fp8Linear``.
"""
from __future__ import annotations

import ctypes as C
import os
import re
from typing import Optional, Tuple

import torch
import torch.nn as nn

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
EPS = 1e-12
_FMT = {"e4m3": (0, torch.float8_e4m3fn, E4M3_MAX), "e5m2": (1, torch.float8_e5m2, E5M2_MAX)}
# Format of the output gradient in the input-gradient product: e4m3 as lingua/float8.py:43-47 uses for every
# operand, or e5m2 (wider range, the usual choice for gradients). LB_FP8_GRAD_FORMAT / set_grad_format select it.
_GRAD_FORMAT = os.environ.get("LB_FP8_GRAD_FORMAT", "e4m3")


def set_grad_format(fmt: str) -> None:
    global _GRAD_FORMAT
    assert fmt in _FMT
    _GRAD_FORMAT = fmt


class GemmFp8Args(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p),
        ("row_scale", C.c_void_p), ("col_scale", C.c_void_p), ("status", C.c_void_p),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("out_dtype", C.c_int),
        ("lda", C.c_longlong), ("ldb", C.c_longlong), ("ldc", C.c_longlong),
        ("a_fmt", C.c_int), ("b_fmt", C.c_int),
    ]


def _L():
    from .ops import _lib

    lib = _lib.load()
    if not getattr(lib, "_fp8_declared", False):
        lib.lb_gemm_fp8.argtypes = [C.POINTER(GemmFp8Args), C.c_void_p]
        lib.lb_gemm_fp8.restype = C.c_int
        lib.lb_quant_rows.argtypes = [C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p, C.c_longlong,
                                      C.c_void_p, C.c_void_p]
        lib.lb_quant_rows.restype = C.c_int
        lib.lb_quant_rows_fmt.argtypes = [C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p, C.c_longlong,
                                          C.c_void_p, C.c_int, C.c_void_p]
        lib.lb_quant_rows_fmt.restype = C.c_int
        lib.lb_quant_transpose.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_longlong,
                                           C.c_void_p]
        lib.lb_quant_transpose.restype = C.c_int
        lib._fp8_declared = True
    return lib


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def supported(K: int, N: int) -> bool:
    """Shapes the float8 kernels take: K (reduction) and N (output) multiples of 16."""
    return K % 16 == 0 and N % 16 == 0


# ------------------------------------------------------------------ quantisation
def quant_rows_ref(x: torch.Tensor, fmt: str = "e4m3") -> Tuple[torch.Tensor, torch.Tensor]:
    """(float8 values, scale [rows]) - PyTorch statement of the row-wise quantisation."""
    _, dt, fmax = _FMT[fmt]
    amax = x.abs().amax(dim=-1).float()
    scale = amax.clamp(min=EPS) / fmax
    q = (x.float() * scale.reciprocal()[:, None]).clamp(-fmax, fmax).to(dt)
    return q, scale


def quant_rows(x: torch.Tensor, fmt: str = "e4m3") -> Tuple[torch.Tensor, torch.Tensor]:
    if not _native(x):
        return quant_rows_ref(x, fmt)
    from .ops import _lib

    code, dt, _ = _FMT[fmt]
    rows, K = x.shape
    assert x.stride(1) == 1
    q = torch.empty(rows, K, dtype=dt, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    _lib.check(_L().lb_quant_rows_fmt(x.data_ptr(), x.stride(0), rows, K, q.data_ptr(), K, scale.data_ptr(), code,
                                      _lib.stream_ptr()), "lb_quant_rows")
    return q, scale


def quant_transpose_ref(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    s = scale.float().clamp(min=EPS / E4M3_MAX)
    return (w.float().t() * s.reciprocal()).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).contiguous()


def quant_transpose(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """w [N, K] -> e4m3 [K, N], all elements divided by the one-element tensor ``scale``."""
    if not _native(w):
        return quant_transpose_ref(w, scale)
    from .ops import _lib

    N, K = w.shape
    w = w.contiguous()
    q = torch.empty(K, N, dtype=torch.float8_e4m3fn, device=w.device)
    _lib.check(_L().lb_quant_transpose(w.data_ptr(), N, K, scale.data_ptr(), q.data_ptr(), N, _lib.stream_ptr()),
               "lb_quant_transpose")
    return q


def scaled_mm_ref(a8, sa, b8, sb, out_dtype=torch.bfloat16):
    out = a8.float() @ b8.float().t()
    out = out * sa.float().reshape(-1, 1) * sb.float().reshape(1, -1)
    return out.to(out_dtype)


def scaled_mm(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor,
              out_dtype=torch.bfloat16) -> torch.Tensor:
    """(a8 @ b8^T) * sa[:, None] * sb[None, :]; a8 [M, K], b8 [N, K] e4m3; sa [M] or [1], sb [N] or [1]."""
    if not a8.is_cuda:
        return scaled_mm_ref(a8, sa, b8, sb, out_dtype)
    from .ops import _lib

    M, K = a8.shape
    N = b8.shape[0]
    if sa.numel() == 1:
        sa = sa.reshape(1).expand(M).contiguous()
    if sb.numel() == 1:
        sb = sb.reshape(1).expand(N).contiguous()
    out = torch.empty(M, N, dtype=out_dtype, device=a8.device)
    a = GemmFp8Args()
    a.A, a.B, a.C = a8.data_ptr(), b8.data_ptr(), out.data_ptr()
    a.row_scale, a.col_scale, a.status = sa.data_ptr(), sb.data_ptr(), _lib.status_word().data_ptr()
    a.M, a.N, a.K = M, N, K
    a.out_dtype = 0 if out_dtype == torch.bfloat16 else 1
    a.lda, a.ldb, a.ldc = a8.stride(0), b8.stride(0), out.stride(0)
    a.a_fmt = 1 if a8.dtype == torch.float8_e5m2 else 0
    a.b_fmt = 1 if b8.dtype == torch.float8_e5m2 else 0
    _lib.check(_L().lb_gemm_fp8(C.byref(a), _lib.stream_ptr()), "lb_gemm_fp8")
    return out


# ------------------------------------------------------------------ the three products of a linear layer
# Quantised weights of the current optimiser step: {(address, shape): (epoch, version, weight, e4m3 rows, row scales)}. The forward product of
# a step quantises a weight row-wise once; further products of the same step with the same weight (gradient
# accumulation) reuse the result, and the input-gradient product takes its single tensor scale as the maximum of
# the row scales instead of a separate pass over the weight. ``new_weight_epoch`` (called by the training engine
# after every optimiser step and after loading weights) invalidates everything.
_WEIGHT_EPOCH = 0
_WEIGHT_CACHE = {}


def new_weight_epoch() -> None:
    global _WEIGHT_EPOCH
    _WEIGHT_EPOCH += 1
    _WEIGHT_CACHE.clear()


def _cached_weight(w: torch.Tensor):
    """Cache entry of ``w`` if it is still valid: same optimiser-step epoch (the engine's AdamW writes through raw
    pointers) and same tensor version (in-place PyTorch updates). The entry keeps ``w`` alive, so its address cannot
    be handed to another tensor while the entry exists."""
    hit = _WEIGHT_CACHE.get((w.data_ptr(), tuple(w.shape)))
    if hit is not None and hit[0] == _WEIGHT_EPOCH and hit[1] == w._version:
        return hit
    return None


def _quant_weight_rows(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    hit = _cached_weight(w)
    if hit is not None:
        return hit[3], hit[4]
    w8, sw = quant_rows(w)
    if w.is_cuda:
        _WEIGHT_CACHE[(w.data_ptr(), tuple(w.shape))] = (_WEIGHT_EPOCH, w._version, w, w8, sw)
    return w8, sw


def fp8_forward_mm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T with row-wise scales on both operands."""
    x8, sx = quant_rows(x)
    w8, sw = _quant_weight_rows(w)
    return scaled_mm(x8, sx, w8, sw, x.dtype if x.dtype != torch.float32 else torch.float32)


def fp8_dgrad_mm(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """dy [M, N] @ w [N, K]: row-wise scales for dy, one scale for the weight."""
    dy8, sdy = quant_rows(dy, _GRAD_FORMAT)
    hit = _cached_weight(w)
    if hit is not None:
        sw = hit[4].max().reshape(1)  # max_r(amax_r / 448) = amax / 448: the row scales already hold the answer
    else:
        sw = (w.detach().abs().amax().float().clamp(min=EPS) / E4M3_MAX).reshape(1)
    wt8 = quant_transpose(w, sw)
    return scaled_mm(dy8, sdy, wt8, sw, dy.dtype if dy.dtype != torch.float32 else torch.float32)


class Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        out = fp8_forward_mm(x, w)
        if bias is not None:
            out = out + bias
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = fp8_dgrad_mm(dy, w) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            if _native(dy) and _native(x):
                from .ops.gemm import mm_tn

                dw = mm_tn(dy, x, out_dtype=torch.float32).to(w.dtype)
            else:
                dw = (dy.float().t() @ x.float()).to(w.dtype)
        db = dy.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db


class Fp8Linear(nn.Linear):
    """``nn.Linear`` whose forward and input-gradient products run in e4m3 (lingua/float8.py:144-148)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = Fp8LinearFn.apply(x.flatten(end_dim=-2), self.weight, self.bias)
        return out.unflatten(0, x.shape[:-1])


def convert_linears_to_fp8(root: nn.Module, recipe: str, filter: str) -> nn.Module:
    """Switch every linear layer whose qualified name matches ``filter`` to float8 products.

    Same selection rule as lingua/float8.py:151-191 (a regular expression searched in the module path);
    layers whose sizes the kernels do not take (not multiples of 16) stay in bf16."""
    if recipe not in ("rowwise",):
        raise RuntimeError(f"Unknown float8 recipe {recipe!r}")
    pat = re.compile(filter)
    for name, mod in list(root.named_modules()):
        w = getattr(mod, "weight", None)
        if not isinstance(w, nn.Parameter) or w.dim() != 2 or isinstance(mod, nn.Embedding):
            continue
        if not pat.search(name) or not hasattr(mod, "in_features"):
            continue
        if w.shape[0] % 16 != 0 or w.shape[1] % 16 != 0:
            continue
        w.lb_fp8 = True
        if type(mod) is nn.Linear:
            mod.__class__ = Fp8Linear
        else:
            mod.fp8 = True  # this library's Linear: its own forward checks the flag
    return root


def wants_fp8(w: torch.Tensor) -> bool:
    return bool(getattr(w, "lb_fp8", False))
