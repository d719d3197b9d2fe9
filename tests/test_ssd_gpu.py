"""The chunked Mamba-2 scan on its native path (four batched tcgen05 GEMMs, decay kernel, three glue kernels, all
with hand-written backward) against the token-by-token recurrence in fp64."""
import pytest
import torch

from lingua_b200.ops import ssd as S

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.double() - b.double()).abs().max().item() / (b.double().abs().max().item() + 1e-9)


@pytest.mark.parametrize("g,d_kind,docs,init", [(1, "head", False, False), (2, "head_dim", True, False),
                                                (1, "none", True, True), (4, "head", False, True)])
def test_fused_chunked_scan_matches_sequential_reference(g, d_kind, docs, init):
    torch.manual_seed(0)
    b, s, h, p, n, L = 2, 384, 8, 64, 128, 128
    dev = "cuda"
    wide = torch.randn(b, s, h * p + 2 * g * n + 16, device=dev) * 0.5  # x, B, C as slices of one projection output
    xb = wide.bfloat16()
    x = xb[..., :h * p].reshape(b, s, h, p).requires_grad_()
    Bm = xb[..., h * p:h * p + g * n].reshape(b, s, g, n).requires_grad_()
    Cm = xb[..., h * p + g * n:h * p + 2 * g * n].reshape(b, s, g, n).requires_grad_()
    dt = (torch.rand(b, s, h, device=dev) * 0.2 + 0.01).requires_grad_()
    A = (-torch.rand(h, device=dev) * 2 - 0.1).requires_grad_()
    D = {"none": None, "head": torch.randn(h, device=dev), "head_dim": torch.randn(h, p, device=dev)}[d_kind]
    if D is not None:
        D.requires_grad_()
    ds = None
    if docs:
        ds = torch.zeros(b, s, dtype=torch.int32, device=dev)
        ds[0, 100:] = 100
        ds[0, 290:] = 290
        ds[1, 128:] = 128  # a boundary exactly at a chunk edge
    h0 = (torch.randn(b, h, p, n, device=dev) * 0.3).requires_grad_() if init else None
    assert S._glue_ok(x, dt, Bm, Cm, L)
    y, st = S.ssd_chunked(x, dt, A, Bm, Cm, D, L, ds, h0)
    # (with document masks the first token starts a document, so the initial state is dropped by both formulations)
    yr, str_ = S.ssd_ref(x, dt, A, Bm, Cm, D, ds, h0)
    assert _rel(y, yr) < 3e-2, _rel(y, yr)
    assert _rel(st, str_) < 3e-2
    gy = torch.randn_like(y)
    leaves = [t for t in (x, dt, A, Bm, Cm, D, h0 if not docs else None) if t is not None]
    got = torch.autograd.grad(y, leaves, gy, allow_unused=True)
    want = torch.autograd.grad(yr, leaves, gy.to(yr.dtype), allow_unused=True)
    names = [nm for nm, t in zip(("x", "dt", "A", "B", "C", "D", "h0"), (x, dt, A, Bm, Cm, D, h0 if not docs else None))
             if t is not None]
    for nm, a_, b_ in zip(names, got, want):
        assert a_ is not None and b_ is not None, nm
        assert _rel(a_, b_) < 6e-2, (nm, _rel(a_, b_))
