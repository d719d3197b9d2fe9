"""The paths that protect a shared GPU and the repeatability of the reductions, exercised without faulting anything:
a bounded wait that is made to run out returns a status instead of hanging, and the deterministic kernels repeat
bit for bit."""
import ctypes as C

import pytest
import torch

from lingua_b200.ops import _lib
from lingua_b200.ops import attention as A

pytestmark = pytest.mark.gpu


def _barrier(pads, rank, epoch, limit_ns):
    lib = _lib.load()
    lib.lb_peer_barrier_limit.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_ulonglong, C.c_void_p]
    lib.lb_peer_barrier_limit.restype = C.c_int
    arr = (C.c_void_p * len(pads))(*[p.data_ptr() for p in pads])
    return lib.lb_peer_barrier_limit(arr, len(pads), rank, epoch, _lib.status_word().data_ptr(), limit_ns,
                                     _lib.stream_ptr())


def test_barrier_wait_runs_out_and_reports_status():
    """Two "ranks", but only rank 0 ever arrives (the second pad is a buffer nobody bumps): the kernel gives up after
    its limit, the host sees the time-out code, and the context is still usable afterwards."""
    pads = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    assert _barrier(pads, 0, 1, 2_000_000) == 0  # 2 ms limit
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 0x2"):  # ST_TIMEOUT_FLAG = 0x200 | site
        _lib.check_status()
    _lib.check_status()  # the word was cleared by the failed check
    assert int(pads[1][0]) == 1 and int(pads[0][0]) == 1  # rank 0 announced itself to both before waiting
    # the missing rank "arrives": the next barrier passes and nothing is reported
    pads[0][1] = 2
    assert _barrier(pads, 0, 2, 2_000_000_000) == 0
    torch.cuda.synchronize()
    _lib.check_status()
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0


def test_slot_reduction_repeats_bitwise():
    lib = _lib.load()
    lib.lb_reduce_slots.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p, C.c_longlong, C.c_float,
                                    C.c_void_p, C.c_void_p]
    lib.lb_reduce_slots.restype = C.c_int
    torch.manual_seed(0)
    n, slots_n = 1_000_003, 7
    own = torch.randn(n, device="cuda")
    slots = torch.randn(slots_n, n + 5, device="cuda")  # pitch 1_000_008: a multiple of 4 floats
    out = torch.empty(n, device="cuda")
    # a slot pitch that breaks the 16-byte alignment is refused before anything is launched
    assert lib.lb_reduce_slots(own.data_ptr(), slots.data_ptr(), slots_n, n + 2, out.data_ptr(), n, 0.125, None,
                               _lib.stream_ptr()) == 2
    outs = []
    for _ in range(2):
        out = torch.empty(n, device="cuda")
        assert lib.lb_reduce_slots(own.data_ptr(), slots.data_ptr(), slots_n, n + 5, out.data_ptr(), n, 0.125, None,
                                   _lib.stream_ptr()) == 0
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    ref = (own.double() + slots[:, :n].double().sum(0)) * 0.125
    assert torch.allclose(outs[0].double(), ref, rtol=1e-5, atol=1e-5)


def test_attention_backward_repeats():
    """dK and dV are accumulated in tensor memory by one CTA each and repeat bit for bit; dQ is summed over the key
    tiles with fp32 reductions in memory, whose order is not fixed: it repeats to fp32 rounding."""
    torch.manual_seed(0)
    B, S, H, Hkv = 1, 512, 4, 2
    qkv = torch.randn(B, S, H + 2 * Hkv, 128, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
    o, lse = A.flash_fwd(q, k, v)
    dout = torch.randn_like(o)
    res = []
    for _ in range(2):
        g = torch.zeros_like(qkv)
        A.flash_bwd(dout, q, k, v, o, lse, g[:, :, :H], g[:, :, H:H + Hkv], g[:, :, H + Hkv:])
        res.append(g)
    torch.cuda.synchronize()
    assert torch.equal(res[0][:, :, H:], res[1][:, :, H:])
    dq0, dq1 = res[0][:, :, :H].float(), res[1][:, :, :H].float()
    assert (dq0 - dq1).abs().max() <= 2 ** -7 * dq0.abs().max()  # at most one bf16 rounding step apart
