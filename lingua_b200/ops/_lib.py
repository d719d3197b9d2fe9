"""ctypes binding of ``liblingua_b200.so`` (the sm_100a kernels).

The library is loaded from ``lingua_b200/lib`` in this source tree. On a machine with a
GPU a missing library is an error (no silent PyTorch fallback); on a CPU-only machine
``available()`` is False and the callers use their PyTorch reference implementations.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

# LINGUA_B200_LIB: another build of the kernel library to load instead, e.g. the bounds-checked one
_LIB_PATH = Path(os.environ.get("LINGUA_B200_LIB") or Path(__file__).resolve().parent.parent / "lib" / "liblingua_b200.so")
_lib = None
_status = {}

LB_BF16, LB_F32, LB_E4M3, LB_E5M2 = 0, 1, 2, 3


class GemmArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("status", C.c_void_p),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("a_major", C.c_int), ("b_major", C.c_int),
        ("in_dtype", C.c_int), ("out_dtype", C.c_int),
        ("accumulate", C.c_int),
        ("nb0", C.c_int), ("nb1", C.c_int),
        ("force_bn", C.c_int),
        ("alpha", C.c_float),
        ("lda", C.c_longlong), ("ldb", C.c_longlong), ("ldc", C.c_longlong),
        ("a_bs0", C.c_longlong), ("a_bs1", C.c_longlong),
        ("b_bs0", C.c_longlong), ("b_bs1", C.c_longlong),
        ("c_bs0", C.c_longlong), ("c_bs1", C.c_longlong),
    ]


class ScatterArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("m_rot", C.c_int), ("blocks", C.c_void_p),
        ("dst", C.c_void_p * 8), ("dst_rows", C.c_longlong * 8),
    ]


class GatherArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("rank", C.c_int), ("n_remote", C.c_int),
        ("n_order", C.c_void_p), ("remote_blocks", C.c_void_p), ("flags_init", C.c_void_p), ("flags", C.c_void_p),
        ("b_peers", C.c_void_p * 8),
    ]


class GroupArgs(C.Structure):
    _fields_ = [("mode", C.c_int), ("n_groups", C.c_int), ("group_stride", C.c_longlong), ("sel", C.c_void_p)]


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("dout", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("delta", C.c_void_p), ("dq_acc", C.c_void_p),
        ("doc_start", C.c_void_p), ("doc_end", C.c_void_p), ("status", C.c_void_p),
        ("B", C.c_int), ("S", C.c_int), ("H", C.c_int), ("Hkv", C.c_int), ("D", C.c_int),
        ("causal", C.c_int), ("window", C.c_int), ("scale", C.c_float),
        ("q_sb", C.c_longlong), ("q_ss", C.c_longlong), ("q_sh", C.c_longlong),
        ("k_sb", C.c_longlong), ("k_ss", C.c_longlong), ("k_sh", C.c_longlong),
        ("v_sb", C.c_longlong), ("v_ss", C.c_longlong), ("v_sh", C.c_longlong),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    """True when the native kernels can run: a CUDA device is visible and the library loads."""
    if not torch.cuda.is_available():
        return False
    return load() is not None


def load():
    """dlopen the kernel library (building it first if the .so is missing and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        if os.environ.get("LINGUA_B200_NO_BUILD") == "1":
            raise RuntimeError(f"{_LIB_PATH} is missing; run `python -m lingua_b200.build`")
        from lingua_b200 import build as _build

        _build.build()
    lib = C.CDLL(str(_LIB_PATH))
    lib.lb_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
    lib.lb_gemm.restype = C.c_int
    if hasattr(lib, "lb_gemm_scatter"):
        lib.lb_gemm_scatter.argtypes = [C.POINTER(GemmArgs), C.POINTER(ScatterArgs), C.c_void_p]
        lib.lb_gemm_scatter.restype = C.c_int
    if hasattr(lib, "lb_gemm_grouped"):
        lib.lb_gemm_grouped.argtypes = [C.POINTER(GemmArgs), C.POINTER(GroupArgs), C.c_void_p]
        lib.lb_gemm_grouped.restype = C.c_int
    if hasattr(lib, "lb_gemm_gather"):
        lib.lb_gemm_gather.argtypes = [C.POINTER(GemmArgs), C.POINTER(GatherArgs), C.c_void_p]
        lib.lb_gemm_gather.restype = C.c_int
    lib.lb_launch_count.restype = C.c_longlong
    lib.lb_launch_count_add.argtypes = [C.c_longlong]
    _declare(lib)
    _lib = lib
    return lib


def _declare(lib) -> None:
    """Signatures of the remaining entry points; a symbol that is absent is left undeclared."""
    vp, i, ll, f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    fp, ip, llp = C.c_void_p, C.c_void_p, C.c_void_p  # device pointers are passed as integers
    sigs = {
        "lb_rmsnorm_fwd": [vp, vp, vp, vp, vp, fp, ll, i, f, vp],
        "lb_rmsnorm_bwd": [vp, vp, vp, fp, vp, vp, fp, ll, i, vp],
        "lb_rope": [vp, vp, ip, ll, i, i, i, i, i, vp],
        "lb_glu_fwd": [vp, vp, ll, i, i, vp],
        "lb_glu_bwd": [vp, vp, vp, ll, i, i, vp],
        "lb_act_fwd": [vp, vp, ll, i, vp],
        "lb_act_bwd": [vp, vp, vp, ll, i, vp],
        "lb_add": [vp, vp, vp, ll, vp],
        "lb_embed_fwd": [llp, vp, vp, ll, i, i, vp],
        "lb_embed_bwd": [llp, vp, fp, ll, i, i, vp],
        "lb_ce_fwd": [fp, llp, fp, fp, ll, i, ll, vp],
        "lb_ce_bwd": [fp, llp, fp, fp, f, vp, ll, i, ll, ll, vp],
        "lb_sumsq": [fp, ll, fp, vp],
        "lb_adamw": [fp, fp, fp, fp, vp, ll, fp, f, f, f, f, f, f, f, i, vp],
        "lb_cast_f32_bf16": [fp, vp, ll, vp],
        "lb_attn_fwd": [C.POINTER(AttnArgs), vp],
        "lb_attn_bwd": [C.POINTER(AttnArgs), vp],
        "lb_conv1d_fwd": [vp, vp, ip, vp, i, i, i, i, ll, ll, i, vp],
        "lb_conv1d_bwd": [vp, vp, ip, vp, vp, fp, i, i, i, i, ll, ll, ll, i, vp],
        "lb_scan_fwd": [vp, vp, ip, fp, vp, fp, fp, i, i, i, vp],
        "lb_scan_bwd": [vp, vp, vp, ip, fp, vp, vp, fp, i, i, i, vp],
        "lb_decode_attn": [vp, vp, vp, vp, vp, ip, ip, vp, i, i, i, i, ll, ll, f, vp],
        "lb_conv1d_update": [vp, ll, vp, vp, vp, ll, i, i, i, i, vp],
        "lb_conv_states": [vp, ll, llp, llp, vp, i, i, i, vp],
        "lb_ssm_state_update": [fp, vp, ll, fp, fp, vp, ll, vp, ll, fp, i, vp, i, i, i, i, i, vp],
        "lb_rnn_step": [vp, vp, fp, vp, ll, vp],
        "lb_rglru_gates_fwd": [vp, vp, vp, fp, vp, vp, ll, i, vp],
        "lb_rglru_gates_bwd": [vp, vp, vp, fp, vp, vp, vp, vp, vp, fp, ll, i, vp],
    }
    for name, args in sigs.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = C.c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device=None) -> torch.Tensor:
    """One uint32 status word per device, shared by every kernel that can time out."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    t = _status.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{dev}")
        _status[dev] = t
    return t


def check_status() -> None:
    """Synchronises and raises if any kernel recorded a timed-out wait since the last check."""
    for dev, t in _status.items():
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"lingua_b200 kernel reported status 0x{v & 0xFFFFFFFF:x} on cuda:{dev}")


def launch_count() -> int:
    return int(load().lb_launch_count())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
