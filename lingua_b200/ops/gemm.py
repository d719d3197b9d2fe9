"""bf16 GEMM on the tcgen05 kernel (``csrc/gemm.cu``), with a PyTorch reference for CPU.

``gemm(a, b)`` computes ``a @ b.transpose(-1, -2)`` for ``a: [..., M, K]`` and
``b: [..., N, K]``. Either operand may be a transposed view: the kernel reads K-contiguous
and M/N-contiguous operands directly, so the dgrad and wgrad GEMMs of a linear layer
(lingua/transformer.py:357-359) need no transposed copies.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib


def _major_and_ld(t: torch.Tensor):
    """(major, leading stride) of the last two dims: 0 = last dim contiguous, 1 = second-to-last."""
    if t.stride(-1) == 1:
        return 0, t.stride(-2)
    if t.stride(-2) == 1:
        return 1, t.stride(-1)
    raise ValueError("operand needs a unit stride in one of its last two dims")


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """The kernel's TMA maps need row pitches that are multiples of 8 elements (16 bytes): an operand with a
    ragged pitch (a [rows, 258] gradient, say) is copied once into a padded buffer and viewed at its own size."""
    major, ld = _major_and_ld(t)
    if ld % 8 == 0 or (t.shape[-2] == 1 and major == 0) or (t.shape[-1] == 1 and major == 1):
        return t
    src = t if major == 0 else t.transpose(-1, -2)
    cols = src.shape[-1]
    buf = torch.empty(*src.shape[:-1], (cols + 7) // 8 * 8, dtype=t.dtype, device=t.device)[..., :cols]
    buf.copy_(src)
    return buf if major == 0 else buf.transpose(-1, -2)


def gemm_ref(a, b, out_dtype=torch.bfloat16, out=None, accumulate=False, alpha=1.0):
    r = torch.matmul(a.float(), b.float().transpose(-1, -2)) * alpha
    if out is not None:
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    return r.to(out_dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    out_dtype: torch.dtype = torch.bfloat16,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    force_bn: int = 0,
) -> torch.Tensor:
    """``out (+)= alpha * a @ b^T``; a: [*batch, M, K], b: [*batch, N, K], up to two batch dims."""
    if not a.is_cuda:
        return gemm_ref(a, b, out_dtype, out, accumulate, alpha)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 operands expected"
    assert a.dim() == b.dim() and 2 <= a.dim() <= 4
    M, K = a.shape[-2:]
    N, Kb = b.shape[-2:]
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    batch = list(a.shape[:-2])
    assert list(b.shape[:-2]) == batch
    if out is None:
        # rows are stored in 8-element vectors: pad the row pitch of a ragged N
        N8 = (N + 7) // 8 * 8
        out = torch.empty(*batch, M, N8, dtype=out_dtype, device=a.device)[..., :N]
    else:
        assert out.shape[-2:] == (M, N) and out.stride(-1) == 1
    if M == 0 or N == 0 or (K == 0 and accumulate):
        return out  # nothing to compute (an empty group of a grouped product, a step without active rows)
    if K == 0:
        return out.zero_()
    a, b = _aligned(a), _aligned(b)
    a_major, lda = _major_and_ld(a)
    b_major, ldb = _major_and_ld(b)
    # A unit-extent dim can report any stride; normalise so the TMA stride rule holds.
    if M == 1 and a_major == 0:
        lda = K
    if N == 1 and b_major == 0:
        ldb = K
    args = _lib.GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.status = _lib.status_word(a.device).data_ptr()
    args.M, args.N, args.K = M, N, K
    args.a_major, args.b_major = a_major, b_major
    args.in_dtype = _lib.LB_BF16
    args.out_dtype = _lib.LB_BF16 if out.dtype == torch.bfloat16 else _lib.LB_F32
    assert out.dtype in (torch.bfloat16, torch.float32)
    args.accumulate = int(accumulate)
    args.alpha = float(alpha)
    args.force_bn = force_bn
    args.lda, args.ldb, args.ldc = lda, ldb, out.stride(-2)
    # kernel batch index 0 is the fastest-varying (last) batch dim
    nb = batch[::-1] + [1] * (2 - len(batch))
    sa = list(a.stride()[:-2])[::-1] + [0] * (2 - len(batch))
    sb = list(b.stride()[:-2])[::-1] + [0] * (2 - len(batch))
    sc = list(out.stride()[:-2])[::-1] + [0] * (2 - len(batch))
    args.nb0, args.nb1 = nb
    args.a_bs0, args.a_bs1 = sa
    args.b_bs0, args.b_bs1 = sb
    args.c_bs0, args.c_bs1 = sc
    rc = _lib.load().lb_gemm(C.byref(args), _lib.stream_ptr())
    _lib.check(rc, f"lb_gemm(M={M},N={N},K={K},majors={a_major}{b_major})")
    return out


def gemm_scatter(a: torch.Tensor, b: torch.Tensor, blocks: torch.Tensor, dst_ptrs: Sequence[int],
                 dst_rows: Sequence[int], ldc: int, accumulate: bool = False, alpha: float = 1.0,
                 m_rot: int = 0) -> None:
    """``a @ b^T`` ([M, K] x [N, K]^T, bf16) in fp32, written by owner instead of into one matrix.

    ``blocks`` is an int32 device tensor [ceil(M / 128), 2] holding (owner, destination row) for every block of
    128 result rows; the rows of owner ``o`` land in the [dst_rows[o], N] fp32 matrix at address ``dst_ptrs[o]``
    (row pitch ``ldc`` elements), which may be peer memory. ``accumulate`` adds to the destination. The epilogue
    of the SM-pair GEMM kernel performs the stores, so the transfer overlaps the remaining tiles' main loops.
    """
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and blocks.dtype == torch.int32 and blocks.is_contiguous()
    assert blocks.numel() >= 2 * ((M + 127) // 128)
    a, b = _aligned(a), _aligned(b)
    a_major, lda = _major_and_ld(a)
    b_major, ldb = _major_and_ld(b)
    args = _lib.GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), 0
    args.status = _lib.status_word(a.device).data_ptr()
    args.M, args.N, args.K = M, N, K
    args.a_major, args.b_major = a_major, b_major
    args.in_dtype, args.out_dtype = _lib.LB_BF16, _lib.LB_F32
    args.accumulate = int(accumulate)
    args.alpha = float(alpha)
    args.force_bn = 0
    args.lda, args.ldb, args.ldc = lda, ldb, ldc
    args.nb0 = args.nb1 = 1
    sc = _lib.ScatterArgs()
    sc.world = len(dst_ptrs)
    sc.m_rot = int(m_rot)
    sc.blocks = blocks.data_ptr()
    for o, (ptr, rows) in enumerate(zip(dst_ptrs, dst_rows)):
        sc.dst[o] = ptr
        sc.dst_rows[o] = rows
    rc = _lib.load().lb_gemm_scatter(C.byref(args), C.byref(sc), _lib.stream_ptr())
    _lib.check(rc, f"lb_gemm_scatter(M={M},N={N},K={K})")


class GatherPlan:
    """Device-side tables of one weight matrix for ``gemm_gather``: which rank owns each 128-row block, the order in
    which the column tiles are computed (own rows first, then the next ranks') and the order in which remote blocks
    are pulled."""

    def __init__(self, owners: Sequence[int], rank: int, world: int, K: int, device):
        nblk = len(owners)
        dist_of = [(o - rank) % world for o in owners]  # 0 = own, then the ring
        n_tiles = (nblk + 1) // 2
        tile_key = [max(dist_of[2 * t:2 * t + 2]) for t in range(n_tiles)]
        order = sorted(range(n_tiles), key=lambda t: (tile_key[t], t))
        # pull blocks in the order the tile walk reaches them
        remote = [(b, owners[b]) for t in order for b in (2 * t, 2 * t + 1) if b < nblk and owners[b] != rank]
        ppb = K // 64
        self.rank, self.world, self.n_remote = rank, world, len(remote)
        self.n_order = torch.tensor(order, dtype=torch.int32, device=device)
        self.remote_blocks = torch.tensor(remote if remote else [(0, 0)], dtype=torch.int32, device=device)
        self.flags_init = torch.tensor([ppb if o == rank else 0 for o in owners] + [0], dtype=torch.int32, device=device)
        self.flags = torch.zeros(nblk + 1, dtype=torch.int32, device=device)


def gemm_gather(x: torch.Tensor, w: torch.Tensor, plan: GatherPlan, peer_ptrs: Sequence[int],
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w^T`` ([M, K] x [N, K]^T, bf16) where only this rank's 128-row blocks of ``w`` are current: the other
    blocks are pulled out of their owners' copies (``peer_ptrs[r]`` = address of the same matrix on rank r) into ``w``
    by the GEMM kernel itself while it computes the tiles that need only local rows. ``w`` is complete afterwards."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.is_contiguous() and x.stride(1) == 1 and N % 128 == 0 and K % 64 == 0
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    args = _lib.GemmArgs()
    args.A, args.B, args.C = x.data_ptr(), w.data_ptr(), out.data_ptr()
    args.status = _lib.status_word(x.device).data_ptr()
    args.M, args.N, args.K = M, N, K
    args.a_major = args.b_major = 0
    args.in_dtype = args.out_dtype = _lib.LB_BF16
    args.accumulate, args.alpha, args.force_bn = 0, 1.0, 0
    args.lda, args.ldb, args.ldc = x.stride(0), K, out.stride(0)
    args.nb0 = args.nb1 = 1
    ga = _lib.GatherArgs()
    ga.world, ga.rank, ga.n_remote = plan.world, plan.rank, plan.n_remote
    ga.n_order, ga.remote_blocks = plan.n_order.data_ptr(), plan.remote_blocks.data_ptr()
    ga.flags_init, ga.flags = plan.flags_init.data_ptr(), plan.flags.data_ptr()
    for r, ptr in enumerate(peer_ptrs):
        ga.b_peers[r] = ptr
    rc = _lib.load().lb_gemm_gather(C.byref(args), C.byref(ga), _lib.stream_ptr())
    _lib.check(rc, f"lb_gemm_gather(M={M},N={N},K={K})")
    return out


GROUP_ROWS = 256  # row granularity of a grouped product: the kernel's row tile (two SMs x 128 rows)


def _grouped_args(a_t, b_t, out, M, N, K, a_major, b_major, lda, ldb, out_f32, accumulate):
    args = _lib.GemmArgs()
    args.A, args.B, args.C = a_t.data_ptr(), b_t.data_ptr(), out.data_ptr()
    args.status = _lib.status_word(a_t.device).data_ptr()
    args.M, args.N, args.K = M, N, K
    args.a_major, args.b_major = a_major, b_major
    args.in_dtype = _lib.LB_BF16
    args.out_dtype = _lib.LB_F32 if out_f32 else _lib.LB_BF16
    args.accumulate, args.alpha, args.force_bn = int(accumulate), 1.0, 0
    args.lda, args.ldb, args.ldc = lda, ldb, out.stride(-2)
    args.nb0 = args.nb1 = 1
    return args


def gemm_grouped_rows(x: torch.Tensor, bank: torch.Tensor, sel: torch.Tensor, transpose_bank: bool = False,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One launch for ``out[m] = x[m] @ bank[sel[m // 256]]^T`` (or ``@ bank[...]`` with ``transpose_bank``).

    ``x`` [Mp, K] bf16 with rows laid out group by group, every group padded to a multiple of 256 rows;
    ``bank`` [G, N, K] (``transpose_bank``: [G, K, N]) bf16 contiguous; ``sel`` int32 [Mp / 256] on the device.
    ``sel`` = -1 marks a tile without rows, which is skipped (its output rows are not written). The grouping never
    reaches the host."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and bank.dtype == torch.bfloat16 and bank.is_contiguous()
    Mp, K = x.shape
    G = bank.shape[0]
    N = bank.shape[2] if transpose_bank else bank.shape[1]
    assert (bank.shape[1] if transpose_bank else bank.shape[2]) == K
    assert Mp % GROUP_ROWS == 0 and sel.dtype == torch.int32 and sel.numel() >= Mp // GROUP_ROWS and sel.is_contiguous()
    assert x.stride(1) == 1 and x.stride(0) % 8 == 0 and bank.shape[2] % 8 == 0
    if out is None:
        out = torch.empty(Mp, N, dtype=torch.bfloat16, device=x.device)
    args = _grouped_args(x, bank, out, Mp, N, K, 0, 1 if transpose_bank else 0, x.stride(0), bank.shape[2], False, False)
    gr = _lib.GroupArgs()
    gr.mode, gr.n_groups, gr.group_stride, gr.sel = 1, G, bank.stride(0), sel.data_ptr()
    rc = _lib.load().lb_gemm_grouped(C.byref(args), C.byref(gr), _lib.stream_ptr())
    _lib.check(rc, f"lb_gemm_grouped(rows, M={Mp},N={N},K={K},G={G})")
    return out


def gemm_grouped_k(dy: torch.Tensor, x: torch.Tensor, k_range: torch.Tensor, out: torch.Tensor,
                   accumulate: bool = False) -> torch.Tensor:
    """One launch for ``out[g] (+)= dy[r0:r1]^T @ x[r0:r1]`` with ``(r0, (r1 - r0) / 64) = k_range[g]``.

    ``dy`` [Mp, N] and ``x`` [Mp, K] bf16 row-major (rows are the contraction index), ``k_range`` int32 [G, 2]
    on the device, ``out`` [G, N, K] fp32 contiguous. A group with zero blocks gets zeros (nothing added when
    accumulating)."""
    assert dy.is_cuda and dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and out.dtype == torch.float32
    Mp, N = dy.shape
    K = x.shape[1]
    G = out.shape[0]
    assert x.shape[0] == Mp and out.shape[1:] == (N, K) and out.is_contiguous()
    assert dy.stride(1) == 1 and x.stride(1) == 1 and dy.stride(0) % 8 == 0 and x.stride(0) % 8 == 0
    assert k_range.dtype == torch.int32 and k_range.is_contiguous() and k_range.numel() >= 2 * G
    # operands of the kernel: A[k, m] = dy (m contiguous), B[k, n] = x (n contiguous); its "K" is the row count
    args = _grouped_args(dy, x, out, N, K, Mp, 1, 1, dy.stride(0), x.stride(0), True, accumulate)
    gr = _lib.GroupArgs()
    gr.mode, gr.n_groups, gr.group_stride, gr.sel = 2, G, out.stride(0), k_range.data_ptr()
    rc = _lib.load().lb_gemm_grouped(C.byref(args), C.byref(gr), _lib.stream_ptr())
    _lib.check(rc, f"lb_gemm_grouped(k, M={N},N={K},K={Mp},G={G})")
    return out


def mm_nt(x: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T -> [M,N] (linear forward)."""
    return gemm(x, w, **kw)


def mm_nn(dy: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """dy[M,N] @ w[N,K] -> [M,K] (linear dgrad)."""
    return gemm(dy, w.transpose(-1, -2), **kw)


def mm_tn(dy: torch.Tensor, x: torch.Tensor, **kw) -> torch.Tensor:
    """dy[M,N]^T @ x[M,K] -> [N,K] (linear wgrad)."""
    return gemm(dy.transpose(-1, -2), x.transpose(-1, -2), **kw)
