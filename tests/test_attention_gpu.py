"""tcgen05 flash attention fwd/bwd vs fp32 masked-softmax attention."""
import pytest
import torch

from lingua_b200.ops import attention as A

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item() + 1e-6
    assert err / ref < tol, f"rel {err / ref:.4g} abs {err:.4g}"


def make(B, S, H, Hkv, fused=True, seed=0):
    torch.manual_seed(seed)
    Dh = 128
    if fused:
        qkv = torch.randn(B, S, H + 2 * Hkv, Dh, device=DEV, dtype=torch.bfloat16)
        return qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:]
    return tuple(torch.randn(B, S, h, Dh, device=DEV, dtype=torch.bfloat16) for h in (H, Hkv, Hkv))


def docs(B, S, seed=0):
    g = torch.Generator().manual_seed(seed)
    starts, ends = [], []
    for _ in range(B):
        lens = []
        left = S
        while left > 0:
            n = min(left, int(torch.randint(1, max(2, S // 3), (1,), generator=g)))
            lens.append(n)
            left -= n
        s, e = A.doc_bounds_from_lengths(torch.tensor(lens), S)
        starts.append(s)
        ends.append(e)
    return torch.stack(starts).to(DEV).contiguous(), torch.stack(ends).to(DEV).contiguous()


CASES = [
    dict(B=1, S=128, H=1, Hkv=1), dict(B=2, S=384, H=4, Hkv=4), dict(B=1, S=1024, H=2, Hkv=1),
    dict(B=1, S=200, H=2, Hkv=2), dict(B=2, S=640, H=4, Hkv=2),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mask", ["causal", "doc", "window", "full"])
def test_flash_fwd_bwd(case, mask):
    B, S, H, Hkv = case["B"], case["S"], case["H"], case["Hkv"]
    q, k, v = make(B, S, H, Hkv, fused=True)
    causal, ds, de, window = True, None, None, 0
    if mask == "doc":
        ds, de = docs(B, S)
    elif mask == "window":
        window = 96
    elif mask == "full":
        causal = False
    o, lse = A.flash_fwd(q, k, v, causal, ds, window)
    orf, lser = A.attention_ref(q, k, v, causal, ds, window)
    close(o, orf, 2e-2)
    close(lse, lser, 1e-3)
    dout = torch.randn_like(o)
    dqkv = torch.zeros(B, S, H + 2 * Hkv, 128, device=DEV, dtype=torch.bfloat16)
    dq, dk, dv = dqkv[:, :, :H], dqkv[:, :, H:H + Hkv], dqkv[:, :, H + Hkv:]
    A.flash_bwd(dout, q, k, v, o, lse, dq, dk, dv, causal, ds, de, window)
    qq, kk, vv = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    oo, _ = A.attention_ref(qq, kk, vv, causal, ds, window)
    gq, gk, gv = torch.autograd.grad(oo, (qq, kk, vv), dout.float())
    close(dv, gv, 3e-2)
    close(dk, gk, 3e-2)
    close(dq, gq, 3e-2)


def test_autograd_wrapper():
    q, k, v = make(1, 256, 2, 2, fused=False)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    o = A.attention(q, k, v)
    o.float().square().mean().backward()
    assert q.grad is not None and torch.isfinite(q.grad.float()).all()
