"""tcgen05 GEMM vs an fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

from lingua_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def _ref(a, b, alpha=1.0):
    return alpha * (a.float() @ b.float().transpose(-1, -2))


def _check(out, ref, k):
    tol = 2e-2 * max(1.0, (k / 256) ** 0.5)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g} (abs {err:.4g})"


# the last three leave 14, 34 and 0 tiles of 256 x 256 for the final wave of 74 SM pairs: split into half-width
# tiles, split, and not split
SHAPES = [(128, 256, 64), (256, 512, 512), (384, 128, 192), (200, 136, 72), (1024, 2048, 1024), (130, 72, 1032),
          (2048, 2816, 256), (4096, 4352, 128), (4096, 4736, 128)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_all_majors(M, N, K, a_t, b_t, out_dtype):
    torch.manual_seed(0)
    dev = "cuda"
    # transposed operands need their contiguous dim (M or N) to be a multiple of 8 for TMA
    if (a_t and M % 8) or (b_t and N % 8):
        pytest.skip("TMA stride alignment")
    a = torch.randn(K, M, device=dev, dtype=torch.bfloat16).t() if a_t else torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=dev, dtype=torch.bfloat16).t() if b_t else torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    out = G.gemm(a, b, out_dtype=out_dtype)
    torch.cuda.synchronize()
    _check(out, _ref(a, b), K)


def test_gemm_accumulate_and_alpha():
    torch.manual_seed(1)
    a = torch.randn(256, 320, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(384, 320, device="cuda", dtype=torch.bfloat16)
    c0 = torch.randn(256, 384, device="cuda", dtype=torch.float32)
    c = c0.clone()
    G.gemm(a, b, out=c, accumulate=True, alpha=0.5)
    _check(c, c0 + _ref(a, b, 0.5), 320)


def test_gemm_batched_strided():
    torch.manual_seed(2)
    B, S, H, D = 2, 256, 3, 128
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    s = G.gemm(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), out_dtype=torch.float32)
    ref = torch.einsum("bshd,bthd->bhst", q.float(), k.float())
    _check(s, ref, D)
    # P @ V with V as the MN-major operand: out[b,h,s,d] = sum_t p[b,h,s,t] v[b,t,h,d]
    p = torch.randn(B, H, S, S, device="cuda", dtype=torch.bfloat16)
    o = G.gemm(p, k.permute(0, 2, 3, 1), out_dtype=torch.bfloat16)
    ref = torch.einsum("bhst,bthd->bhsd", p.float(), k.float())
    _check(o, ref, S)


def test_linear_three_gemms():
    torch.manual_seed(3)
    M, K, N = 512, 256, 384
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    _check(G.mm_nt(x, w), x.float() @ w.float().t(), K)
    _check(G.mm_nn(dy, w), dy.float() @ w.float(), N)
    _check(G.mm_tn(dy, x, out_dtype=torch.float32), dy.float().t() @ x.float(), M)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 512), (300, 264, 200), (2048, 4096, 1024), (130, 72, 1032)])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_two_sm_variant(M, N, K, a_t, b_t, out_dtype):
    torch.manual_seed(0)
    dev = "cuda"
    if (a_t and M % 8) or (b_t and N % 8):
        pytest.skip("TMA stride alignment")
    a = torch.randn(K, M, device=dev, dtype=torch.bfloat16).t() if a_t else torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=dev, dtype=torch.bfloat16).t() if b_t else torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    out = G.gemm(a, b, out_dtype=out_dtype, force_bn=512)
    torch.cuda.synchronize()
    _check(out, _ref(a, b), K)


def test_gemm_two_sm_batched_accumulate():
    torch.manual_seed(5)
    a = torch.randn(3, 384, 320, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(3, 512, 320, device="cuda", dtype=torch.bfloat16)
    c0 = torch.randn(3, 384, 512, device="cuda", dtype=torch.float32)
    c = c0.clone()
    G.gemm(a, b, out=c, accumulate=True, alpha=2.0, force_bn=512)
    _check(c, c0 + _ref(a, b, 2.0), 320)


@pytest.mark.parametrize("W", [1, 2, 4, 8])
@pytest.mark.parametrize("M,N,K", [(1024, 512, 512), (1400, 264, 320), (4096, 1024, 256)])
def test_gemm_scatter_rows_to_owners(W, M, N, K):
    """The scatter epilogue delivers every 128-row block to its owner's matrix (all "owners" are buffers of this
    GPU here: the kernel never waits on a peer, so one device can stand in for the group). Uneven splits, a
    rotated tile walk, overwrite and accumulate."""
    torch.manual_seed(W)
    dy = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)  # [tokens, out]: the wgrad's MN-major A operand
    x = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)   # [tokens, in]
    ref = dy.float().t() @ x.float()
    nblk = (M + 127) // 128
    bounds = [round(r * nblk / W) * 128 for r in range(W + 1)]
    bounds[-1] = M
    dst = [torch.full((max(bounds[o + 1] - bounds[o], 1) + 3, N), 7.0, device="cuda") for o in range(W)]
    table = []
    for blk in range(nblk):
        o = max(i for i in range(W) if bounds[i] <= blk * 128)
        table.append((o, blk * 128 - bounds[o]))
    blocks = torch.tensor(table, dtype=torch.int32, device="cuda")
    rows = [bounds[o + 1] - bounds[o] for o in range(W)]
    ptrs = [d.data_ptr() for d in dst]
    G.gemm_scatter(dy.t(), x.t(), blocks, ptrs, rows, ldc=N, m_rot=(bounds[1 % W] // 256) % max(1, (M + 255) // 256))
    torch.cuda.synchronize()
    for o in range(W):
        if rows[o]:
            _check(dst[o][:rows[o]], ref[bounds[o]:bounds[o + 1]], K)
        assert (dst[o][rows[o]:] == 7.0).all(), "rows beyond an owner's share were touched"
    G.gemm_scatter(dy.t(), x.t(), blocks, ptrs, rows, ldc=N, accumulate=True, alpha=0.5)
    torch.cuda.synchronize()
    for o in range(W):
        if rows[o]:
            _check(dst[o][:rows[o]], 1.5 * ref[bounds[o]:bounds[o + 1]], K)


@pytest.mark.parametrize("W,rank", [(1, 0), (2, 1), (4, 2), (8, 7)])
@pytest.mark.parametrize("M,N,K", [(512, 1024, 512), (2048, 1408, 256), (8192, 4096, 1024)])
def test_gemm_gather_pulls_remote_weight_blocks(W, rank, M, N, K):
    """Only this rank's blocks of the weight are valid locally; the kernel fetches the rest from the "peers" (buffers
    of this GPU here) while it multiplies, and leaves the local copy complete."""
    torch.manual_seed(W + rank)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w_true = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    nblk = N // 128
    bounds = [round(r * nblk / W) for r in range(W + 1)]
    owners = [max(r for r in range(W) if bounds[r] <= b) for b in range(nblk)]
    w_local = torch.full_like(w_true, float("nan"))
    for b, o in enumerate(owners):
        if o == rank:
            w_local[b * 128:(b + 1) * 128] = w_true[b * 128:(b + 1) * 128]
    # every peer's copy is valid only in the blocks that peer owns
    peers = []
    for r in range(W):
        if r == rank:
            peers.append(w_local)
            continue
        c = torch.full_like(w_true, float("nan"))
        for b, o in enumerate(owners):
            if o == r:
                c[b * 128:(b + 1) * 128] = w_true[b * 128:(b + 1) * 128]
        peers.append(c)
    plan = G.GatherPlan(owners, rank, W, K, "cuda")
    out = G.gemm_gather(x, w_local, plan, [p.data_ptr() for p in peers])
    torch.cuda.synchronize()
    assert torch.equal(w_local, w_true), "the local copy of the weight is not complete after the call"
    _check(out, _ref(x, w_true), K)
    # a second call on the same plan (flags are re-initialised by the launch) gives the same result
    out2 = G.gemm_gather(x, w_local, plan, [p.data_ptr() for p in peers])
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


def _group_layout(counts, dev):
    """Padded layout the grouped kernels expect: every group starts on a 256-row boundary."""
    R = G.GROUP_ROWS
    padded = [(c + R - 1) // R * R for c in counts]
    offs = [sum(padded[:g]) for g in range(len(counts))]
    Mp = sum(padded) + R  # one spare tile past the last group, as the device-side plan leaves
    sel = torch.full((Mp // R,), -1, dtype=torch.int32)  # -1: no rows in this tile
    for g, (o, p) in enumerate(zip(offs, padded)):
        sel[o // R:(o + p) // R] = g
    k_range = torch.tensor([[o, p // 64] for o, p in zip(offs, padded)], dtype=torch.int32)
    return offs, Mp, sel.to(dev), k_range.to(dev)


@pytest.mark.parametrize("transpose_bank", [False, True])
def test_grouped_rows_picks_the_matrix_of_each_row_tile(transpose_bank):
    torch.manual_seed(3)
    dev = "cuda"
    counts = [300, 0, 17, 1024, 255, 256]
    K, N = 192, 136
    offs, Mp, sel, _ = _group_layout(counts, dev)
    x = torch.zeros(Mp, K, device=dev, dtype=torch.bfloat16)
    bank = (torch.randn(len(counts), *((K, N) if transpose_bank else (N, K)), device=dev) * 0.1).bfloat16()
    for o, c in zip(offs, counts):
        x[o:o + c] = (torch.randn(c, K, device=dev) * 0.5).bfloat16()
    y = torch.full((Mp, N), 7.0, device=dev, dtype=torch.bfloat16)
    G.gemm_grouped_rows(x, bank, sel, transpose_bank=transpose_bank, out=y)
    for g, (o, c) in enumerate(zip(offs, counts)):
        w = bank[g].float().t() if transpose_bank else bank[g].float()
        if c:
            _check(y[o:o + c], x[o:o + c].float() @ w.t(), K)
    assert y[offs[-1] + counts[-1]:Mp - G.GROUP_ROWS].abs().max() == 0 if counts[-1] % G.GROUP_ROWS else True
    assert y[offs[2] + counts[2]:offs[3]].abs().max() == 0  # padding rows of a group are zero rows
    assert (y[Mp - G.GROUP_ROWS:] == 7.0).all()  # the tile past the last group is skipped
    from lingua_b200.ops import _lib
    _lib.check_status()


@pytest.mark.parametrize("accumulate", [False, True])
def test_grouped_contraction_over_row_ranges(accumulate):
    torch.manual_seed(4)
    dev = "cuda"
    counts = [300, 0, 17, 1024, 255, 256]
    N, K = 136, 192
    offs, Mp, _, k_range = _group_layout(counts, dev)
    dy = torch.zeros(Mp, N, device=dev, dtype=torch.bfloat16)
    x = torch.zeros(Mp, K, device=dev, dtype=torch.bfloat16)
    for o, c in zip(offs, counts):
        dy[o:o + c] = (torch.randn(c, N, device=dev) * 0.5).bfloat16()
        x[o:o + c] = (torch.randn(c, K, device=dev) * 0.5).bfloat16()
    base = torch.randn(len(counts), N, K, device=dev)
    out = base.clone() if accumulate else torch.full_like(base, float("nan"))  # stale values must not survive
    G.gemm_grouped_k(dy, x, k_range, out, accumulate=accumulate)
    for g, (o, c) in enumerate(zip(offs, counts)):
        want = dy[o:o + c].float().t() @ x[o:o + c].float() + (base[g] if accumulate else 0)
        if c:
            _check(out[g], want, max(c, 256))
        else:
            assert torch.equal(out[g], base[g] if accumulate else torch.zeros_like(base[g]))
    from lingua_b200.ops import _lib
    _lib.check_status()
