"""Kernel micro-benchmarks: ``python -m lingua_b200.ops.microbench <op> [--size ...] [--iters N]``.

Runs one native op on synthetic inputs, times it with CUDA events (after warm-up, inputs larger
than L2 or an L2 flush between iterations) and prints achieved TFLOP/s or GB/s next to the
measured peaks of ``MEASURED_PEAKS.json`` when that file is present. It is also the small,
self-terminating workload to put under ``ncu`` when profiling a single kernel.

ops: gemm, gemm_wgrad, gemm_gather, gemm_scatter, gemm_tp_ag, gemm_tp_rs, rglru_gates, ssm_update, ssd, attn_fwd, attn_bwd, rmsnorm, rmsnorm_bwd, glu, ce, adamw, rope, scan, conv1d, decode
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import _lib
from . import attention as A
from . import functional as F
from . import gemm as G
from . import sequence as Q


def _peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return json.loads(p.read_text())
    except Exception:
        return {}


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()  # 256 MB write evicts the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters


def _sustained(name, fn, flops, iters):
    """Back-to-back launches for a few seconds (no flush: the point is the power-capped steady state), CUDA
    events around the whole run, SM clock and board power sampled through NVML while the queue drains."""
    import time

    import pynvml

    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    clk, pw = [], []
    while not e1.query():
        clk.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
        pw.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000)
        time.sleep(0.05)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    med = lambda v: sorted(v[len(v) // 2:])[len(v[len(v) // 2:]) // 2] if v else 0  # second half: settled
    print(f"{name:42s} {ms:.4f} ms {flops / ms / 1e9:6.0f} TFLOP/s  SM {med(clk)} MHz  {med(pw):.0f} W  "
          f"ms x MHz {ms * med(clk):.0f}", flush=True)


def _gemm_sustained(a):
    """The three products of a linear layer (--m tokens, --n outputs, --k inputs) on this library's SM-pair
    kernel and on torch.matmul (cuBLAS), each run long enough to sit at the board's power cap."""
    dev, bf = "cuda", torch.bfloat16
    T, D, H = a.m, a.n, a.k
    it = a.iters if a.iters > 100 else 3000
    x, dy = torch.randn(T, H, device=dev, dtype=bf) * 0.5, torch.randn(T, D, device=dev, dtype=bf) * 0.5
    w = torch.randn(D, H, device=dev, dtype=bf) * 0.02
    wt = w.t().contiguous()
    dw32 = torch.empty(D, H, device=dev, dtype=torch.float32)
    dw16 = torch.empty(D, H, device=dev, dtype=bf)
    fl = 2.0 * T * D * H
    _sustained("ours forward x @ w^T (K-major, K-major)", lambda: G.gemm(x, w), fl, it)
    _sustained("ours input grad dy @ w (K, N-major)", lambda: G.gemm(dy, w.t()), fl, it)
    _sustained("ours input grad, transposed weight copy", lambda: G.gemm(dy, wt), fl, it)
    _sustained("ours weight grad dy^T @ x, fp32 out", lambda: G.gemm(dy.t(), x.t(), out_dtype=torch.float32, out=dw32), fl, it)
    _sustained("ours weight grad, bf16 out", lambda: G.gemm(dy.t(), x.t(), out=dw16), fl, it)
    import os
    for gm in (2, 4, 16, 32):  # tile walk: row tiles per group (default 8)
        os.environ["LB_GEMM_GROUP_M"] = str(gm)
        _sustained(f"ours forward, row tiles per group {gm}", lambda: G.gemm(x, w), fl, it)
        _sustained(f"ours input grad, row tiles per group {gm}", lambda: G.gemm(dy, w.t()), fl, it)
    os.environ.pop("LB_GEMM_GROUP_M")
    _sustained("cuBLAS forward", lambda: torch.matmul(x, w.t()), fl, it)
    _sustained("cuBLAS input grad", lambda: torch.matmul(dy, w), fl, it)
    _sustained("cuBLAS weight grad (bf16 out)", lambda: torch.matmul(dy.t(), x), fl, it)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("op")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--world", type=int, default=4, help="emulated group size of the fused-collective GEMMs")
    ap.add_argument("--bn", type=int, default=0, help="gemm tile selector: 0 auto, 128, 256, 512 (two-SM)")
    a = ap.parse_args(argv)
    dev, bf = "cuda", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flops = bytes_ = 0.0
    M, N, K = a.m, a.n, a.k
    if a.op == "gemm_sustained":
        return _gemm_sustained(a)
    if a.op == "gemm":
        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
        fn = lambda: G.gemm(x, w, force_bn=a.bn)
        flops = 2.0 * M * N * K
    elif a.op in ("gemm_fp8", "linear_fp8"):
        from .. import float8 as F8

        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
        x8, sx = F8.quant_rows(x)
        w8, sw = F8.quant_rows(w)
        # gemm_fp8: the scaled e4m3 product alone; linear_fp8: both quantisation passes included
        fn = (lambda: F8.scaled_mm(x8, sx, w8, sw)) if a.op == "gemm_fp8" else (lambda: F8.fp8_forward_mm(x, w))
        flops = 2.0 * M * N * K
    elif a.op in ("gemm_gather", "gemm_scatter"):
        # the fused-collective forms of the GEMM with every "peer" being a buffer of this GPU: what the fusion costs
        # the kernel itself (shorter TMA ring, gather warp, flag waits / owner-directed stores), NVLink aside
        W, rank = a.world, 0
        if a.op == "gemm_gather":
            x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
            nblk = N // 128
            owners = [min(W - 1, b * W // nblk) for b in range(nblk)]
            peers = [w] + [w.clone() for _ in range(W - 1)]
            plan = G.GatherPlan(owners, rank, W, K, dev)
            ptrs = [t.data_ptr() for t in peers]
            fn = lambda: G.gemm_gather(x, w, plan, ptrs)
        else:
            dy, x = torch.randn(K, M, device=dev, dtype=bf), torch.randn(K, N, device=dev, dtype=bf)
            nblk = (M + 127) // 128
            bounds = [round(r * nblk / W) * 128 for r in range(W)] + [M]
            table = []
            for b in range(nblk):
                o = max(r for r in range(W) if bounds[r] <= b * 128)
                table.append((o, b * 128 - bounds[o]))
            blocks = torch.tensor(table, dtype=torch.int32, device=dev)
            rows = [bounds[o + 1] - bounds[o] for o in range(W)]
            dst = [torch.empty(max(r, 1), N, device=dev) for r in rows]
            ptrs = [t.data_ptr() for t in dst]
            fn = lambda: G.gemm_scatter(dy.t(), x.t(), blocks, ptrs, rows, ldc=N, m_rot=bounds[1 % W] // 256)
        flops = 2.0 * M * N * K
    elif a.op in ("gemm_tp_ag", "gemm_tp_rs"):
        # tensor-parallel GEMMs with the collective inside (csrc/gemm_tp.cu), one emulated rank of --world, peers local:
        # ag = all-gather of the activation rows -> column-parallel GEMM, rs = row-parallel GEMM -> scatter to owners
        from ..parallel import tp_fused as TP

        W = a.world
        Tl = M // W
        if a.op == "gemm_tp_ag":
            slabs = [torch.randn(Tl, K, device=dev, dtype=bf) for _ in range(W)]
            w = torch.randn(N, K, device=dev, dtype=bf)
            gather = torch.empty(M, K, device=dev, dtype=bf)
            flags = torch.zeros(M // 128 + 1, dtype=torch.int32, device=dev)
            out = torch.empty(M, N, device=dev, dtype=bf)
            fn = lambda: TP.ag_gemm([t.data_ptr() for t in slabs], 0, Tl, w, gather, flags, out=out)
        else:
            x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
            stages = [torch.empty(W, Tl, N, device=dev, dtype=bf) for _ in range(W)]
            fn = lambda: TP.gemm_scatter(x, w, [t.data_ptr() for t in stages], 0, Tl * N)
        flops = 2.0 * M * N * K
    elif a.op == "rglru_gates":
        rows, C = a.batch * a.seq, 4096
        gx, ga, x = (torch.randn(rows, C, device=dev, dtype=bf) for _ in range(3))
        sp = torch.rand(C, device=dev) + 0.1
        fn = lambda: Q.rglru_gates(gx, ga, x, sp)
        bytes_ = 5.0 * rows * C * 2
    elif a.op == "ssm_update":
        from . import ssd as S

        n, h, pd, Ns, g = 32, 64, 64, 128, 1
        row = torch.randn(n, h * pd + 2 * g * Ns, device=dev, dtype=bf)
        x, Bm, Cm = row[:, :h * pd].view(n, h, pd), row[:, h * pd:h * pd + g * Ns].view(n, g, Ns), row[:, h * pd + g * Ns:].view(n, g, Ns)
        dt, A_log = torch.rand(n, h, device=dev) * 0.1, -torch.rand(h, device=dev)
        state = torch.randn(n, h, pd, Ns, device=dev)
        fn = lambda: S.selective_state_update(state, x, dt, A_log, Bm, Cm, None)
        bytes_ = 2.0 * state.numel() * 4
    elif a.op == "ssd":
        from . import ssd as S

        b, sq, h, pd, Ns = a.batch, a.seq, 64, 64, 128
        x = torch.randn(b, sq, h, pd, device=dev, dtype=bf)
        dt = torch.rand(b, sq, h, device=dev) * 0.1
        A_log = -torch.rand(h, device=dev)
        Bm, Cm = torch.randn(b, sq, 1, Ns, device=dev, dtype=bf), torch.randn(b, sq, 1, Ns, device=dev, dtype=bf)
        fn = lambda: S.ssd_chunked(x, dt, A_log, Bm, Cm, None, 256)
        flops = 2.0 * b * sq * h * (256 * Ns + 256 * pd + 2 * pd * Ns)  # the four chunk products
    elif a.op == "gemm_wgrad":
        dy, x = torch.randn(K, M, device=dev, dtype=bf), torch.randn(K, N, device=dev, dtype=bf)
        out = torch.zeros(M, N, device=dev)
        fn = lambda: G.mm_tn(dy, x, out=out, accumulate=True, force_bn=a.bn)
        flops = 2.0 * M * N * K
    elif a.op in ("attn_fwd", "attn_bwd"):
        B, S, H = a.batch, a.seq, a.heads
        qkv = torch.randn(B, S, 3 * H, 128, device=dev, dtype=bf)
        q, k, v = qkv[:, :, :H], qkv[:, :, H:2 * H], qkv[:, :, 2 * H:]
        o, lse = A.flash_fwd(q, k, v)
        do, dqkv = torch.randn_like(o), torch.empty_like(qkv)
        if a.op == "attn_fwd":
            fn = lambda: A.flash_fwd(q, k, v)
            flops = 4.0 * B * H * S * S * 128 / 2
        else:
            fn = lambda: A.flash_bwd(do, q, k, v, o, lse, dqkv[:, :, :H], dqkv[:, :, H:2 * H], dqkv[:, :, 2 * H:])
            flops = 10.0 * B * H * S * S * 128 / 2
    elif a.op in ("rmsnorm", "rmsnorm_bwd"):
        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.ones(K, device=dev, dtype=bf)
        y, _, rstd = F.rmsnorm_fwd(x, w, 1e-5)
        if a.op == "rmsnorm":
            fn = lambda: F.rmsnorm_fwd(x, w, 1e-5)
            bytes_ = 2.0 * M * K * 2
        else:
            dy, dw = torch.randn_like(x), torch.zeros(K, device=dev)
            fn = lambda: F.rmsnorm_bwd(dy, x, w, rstd, None, dw)
            bytes_ = 3.0 * M * K * 2
    elif a.op == "glu":
        gu = torch.randn(M, 2 * K, device=dev, dtype=bf)
        fn = lambda: F.glu_fwd(gu)
        bytes_ = 3.0 * M * K * 2
    elif a.op == "ce":
        logits = torch.randn(2048, 128256, device=dev)
        tgt = torch.randint(0, 128256, (2048,), device=dev)
        fn = lambda: F.ce_fwd(logits, tgt)
        bytes_ = 2.0 * logits.numel() * 4
    elif a.op == "adamw":
        n = 512 << 20
        p, m, v, g = (torch.zeros(n, device=dev) for _ in range(4))
        p16 = torch.zeros(n, device=dev, dtype=bf)
        fn = lambda: F.adamw_step(p, m, v, g, p16, step=1, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
        bytes_ = n * 30.0
    elif a.op == "rope":
        B, S, H = a.batch, a.seq, a.heads
        qkv = torch.randn(B * S, 3 * H * 128, device=dev, dtype=bf)
        cs = F.rope_table(128, S, 10000.0, dev)
        fn = lambda: F.rope_(qkv, cs, 2 * H, 128, S)
        bytes_ = 2.0 * B * S * 2 * H * 128 * 2
    elif a.op == "scan":
        B, S, C = 4, a.seq, 4096
        aa = torch.rand(B, S, C, device=dev).bfloat16()
        bb = torch.randn(B, S, C, device=dev, dtype=bf)
        fn = lambda: Q.linear_scan(aa, bb)
        bytes_ = 5.0 * B * S * C * 2
    elif a.op == "conv1d":
        B, S, C = 4, a.seq, 4352
        x, w = torch.randn(B, S, C, device=dev, dtype=bf), torch.randn(C, 4, device=dev, dtype=bf)
        fn = lambda: Q.causal_conv1d(x, w)
        bytes_ = 2.0 * B * S * C * 2
    elif a.op in ("indexed_matmul", "indexed_matmul_loop"):
        # the distance-indexed up-projection of the hierarchical byte model, forward + backward:
        # --m rows, --k inputs, --n outputs, 16 weights; "_loop" = one masked product per weight with a
        # torch.where per weight in forward and again in backward (the formulation this library replaces)
        from .indexed_matmul import indexed_matmul

        T, Din, Dout, nW = a.m, a.k, a.n, 16
        x = (torch.randn(T, Din, device=dev) * 0.5).to(bf).requires_grad_()
        w = (torch.randn(nW, Dout, Din, device=dev) * Din ** -0.5).to(bf).requires_grad_()
        idx = (torch.arange(T, device=dev) % 23 % nW).view(1, T)  # short distances are the common ones
        g = torch.randn(1, T, Dout, device=dev, dtype=bf)

        class Loop(torch.autograd.Function):
            @staticmethod
            def forward(ctx, X, W, I):
                ctx.save_for_backward(X, W, I)
                Y = X.new_empty(X.shape[0], X.shape[1], W.shape[1])
                for n_ in range(W.shape[0]):
                    bi, si = torch.where(I == n_)
                    if si.numel():
                        Y[bi, si] = torch.nn.functional.linear(X[bi, si], W[n_])
                return Y

            @staticmethod
            def backward(ctx, dY):
                X, W, I = ctx.saved_tensors
                dX, dW = torch.zeros_like(X), torch.zeros_like(W)
                for n_ in range(W.shape[0]):
                    bi, si = torch.where(I == n_)
                    if si.numel():
                        dX[bi, si] = dY[bi, si] @ W[n_]
                        dW[n_] = dY[bi, si].t() @ X[bi, si]
                return dX, dW, None

        def fn():
            x.grad = w.grad = None
            y = indexed_matmul(x.view(1, T, Din), w, idx) if a.op == "indexed_matmul" else Loop.apply(x.view(1, T, Din), w, idx)
            y.backward(g)
        flops = 3 * 2.0 * T * Din * Dout
    elif a.op == "decode":
        import math

        nseq, H, L = 32, a.heads, 768
        q = torch.randn(nseq, H, 128, device=dev, dtype=bf)
        kc, vc = torch.randn(nseq * L, H, 128, device=dev, dtype=bf), torch.randn(nseq * L, H, 128, device=dev, dtype=bf)
        start = (torch.arange(nseq, device=dev) * L).int()
        ln = torch.full((nseq,), L, device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        lib = _lib.load()
        fn = lambda: _lib.check(lib.lb_decode_attn(q.data_ptr(), None, None, kc.data_ptr(), vc.data_ptr(),
                                                   start.data_ptr(), ln.data_ptr(), out.data_ptr(), nseq, H, H, 128,
                                                   H * 128, H * 128, 1 / math.sqrt(128), _lib.stream_ptr()), "decode")
        bytes_ = 2.0 * nseq * L * H * 128 * 2
    else:
        raise SystemExit(f"unknown op {a.op}")
    ms = _time(fn, a.iters, flush)
    _lib.check_status()
    pk = _peaks()
    if flops:
        tf = flops / ms / 1e9
        frac = f", {tf / pk['bf16_tflops']:.2f} of measured cuBLAS burst peak" if pk.get("bf16_tflops") else ""
        print(f"{a.op}: {ms:.3f} ms, {tf:.0f} TFLOP/s{frac}")
    else:
        gbs = bytes_ / ms / 1e6
        frac = f", {gbs / pk['hbm_gbs']:.2f} of measured copy bandwidth" if pk.get("hbm_gbs") else ""
        print(f"{a.op}: {ms:.3f} ms, {gbs:.0f} GB/s{frac}")


if __name__ == "__main__":
    main()
