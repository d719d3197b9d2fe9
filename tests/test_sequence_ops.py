"""conv1d / linear-scan: references vs a brute-force loop on CPU, and the CUDA kernels vs the references."""
import pytest
import torch

from lingua_b200.ops import sequence as Q


def _docs(B, S, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = torch.zeros(B, S, dtype=torch.int32)
    for b in range(B):
        s = 0
        while s < S:
            n = int(torch.randint(1, max(2, S // 2), (1,), generator=g))
            out[b, s:s + n] = s
            s += n
    return out


def test_references_match_bruteforce_cpu():
    torch.manual_seed(0)
    B, S, C, W = 2, 37, 5, 4
    x, w = torch.randn(B, S, C), torch.randn(C, W)
    ds = _docs(B, S)
    y = Q.conv1d_ref(x, w, ds, act=False)
    for b in range(B):
        for s in range(S):
            for c in range(C):
                acc = 0.0
                for j in range(W):
                    t = s - (W - 1) + j
                    if t >= int(ds[b, s]):
                        acc += float(w[c, j] * x[b, t, c])
                assert abs(acc - float(y[b, s, c])) < 1e-5
    a, bb = torch.rand(B, S, C), torch.randn(B, S, C)
    h = Q.scan_ref(a, bb, ds)
    for b in range(B):
        st = torch.zeros(C)
        for s in range(S):
            if int(ds[b, s]) == s:
                st = torch.zeros(C)
            st = a[b, s] * st + bb[b, s]
            assert torch.allclose(st, h[b, s], atol=1e-5)


def test_conv_state_helpers_cpu():
    x = torch.arange(10.0).view(10, 1)
    st = Q.conv_states_from_packed(x, torch.tensor([3, 7]), 4)
    assert st.shape == (2, 1, 4)
    assert st[0, 0].tolist() == [0.0, 0.0, 1.0, 2.0] and st[1, 0].tolist() == [6.0, 7.0, 8.0, 9.0]
    w = torch.randn(1, 4)
    full = Q.conv1d_ref(x.view(1, 10, 1), w, None, act=True)
    state = Q.conv_states_from_packed(x[:9], torch.tensor([9]), 4)
    step = Q.conv1d_update(x[9:10], state, w)
    assert torch.allclose(step[0], full[0, 9], atol=1e-5)


def _close(a, b, tol=3e-2):
    a, b = a.float().cpu(), b.float().cpu()
    assert (a - b).abs().max().item() < tol * (b.abs().max().item() + 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("with_docs", [False, True])
@pytest.mark.parametrize("C", [264, 100])  # 8-channel vector kernels / scalar kernels
def test_conv1d_kernels(W, with_docs, C):
    torch.manual_seed(0)
    B, S = 2, 300
    buf = torch.randn(B, S, C + 40, device="cuda", dtype=torch.bfloat16)
    x = buf[:, :, 8:8 + C]  # strided rows, as a slice of a wider projection
    w = torch.randn(C, W, device="cuda", dtype=torch.bfloat16)
    ds = _docs(B, S).cuda() if with_docs else None
    xg = x.detach().clone().requires_grad_(True)
    wg = w.detach().clone().requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    y = Q.causal_conv1d(xg, wg, ds)
    yr = Q.conv1d_ref(xr, wr, ds)
    _close(y, yr)
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    _close(xg.grad, xr.grad)
    _close(wg.grad, wr.grad)


@pytest.mark.gpu
@pytest.mark.parametrize("S", [64, 200, 1024])
@pytest.mark.parametrize("with_docs", [False, True])
@pytest.mark.parametrize("C", [136, 75])  # two channels per thread / one
def test_scan_kernels(S, with_docs, C):
    torch.manual_seed(1)
    B = 2
    a = torch.rand(B, S, C, device="cuda").mul(0.3).add(0.69).bfloat16()
    b = torch.randn(B, S, C, device="cuda", dtype=torch.bfloat16)
    ds = _docs(B, S, seed=3).cuda() if with_docs else None
    ag, bg = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ar, br = a.float().requires_grad_(True), b.float().requires_grad_(True)
    h = Q.linear_scan(ag, bg, ds)
    hr = Q.scan_ref(ar, br, ds)
    _close(h, hr)
    dh = torch.randn_like(h)
    h.backward(dh)
    hr.backward(dh.float())
    _close(bg.grad, br.grad, 4e-2)
    _close(ag.grad, ar.grad, 4e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("L,g,with_docs", [(256, 1, False), (64, 2, True), (128, 4, True)])
def test_ssd_decay_kernels(L, g, with_docs):
    """Fused W = (C B^T) o decay-kernel and its backward vs the PyTorch statement."""
    from lingua_b200.ops import ssd as SSD

    torch.manual_seed(5)
    b, nc, h = 2, 3, 4
    scores = (torch.randn(b, nc, g, L, L, device="cuda") * 0.5).bfloat16()
    cs = -torch.rand(b, h, nc, L, device="cuda").cumsum(-1) * 0.05
    doc = None
    if with_docs:
        starts = torch.zeros(b, nc * L, dtype=torch.int32, device="cuda")
        starts[:, L // 3:] = L // 3
        starts[:, L + 5:] = L + 5
        doc = starts.view(b, nc, L)
    s1 = scores.clone().requires_grad_(True)
    c1 = cs.clone().requires_grad_(True)
    s2 = scores.float().requires_grad_(True)
    c2 = cs.clone().requires_grad_(True)
    w = SSD.decay_weights(s1, c1, doc)
    wr = SSD.decay_weights_ref(s2, c2, doc)
    assert w.dtype == torch.bfloat16 and w.shape == (b, nc, h, L, L)
    _close(w, wr, 1e-2)
    dw = torch.randn_like(wr)
    w.backward(dw.bfloat16())
    wr.backward(dw.bfloat16().float())
    _close(s1.grad, s2.grad, 2e-2)
    _close(c1.grad, c2.grad, 2e-2)
