"""Decoding-step kernels of the recurrent models and the fused RG-LRU gates vs plain PyTorch fp32 references."""
import pytest
import torch

from lingua_b200.ops import sequence as Q
from lingua_b200.ops import ssd as S

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item() + 1e-6
    assert err / ref < tol, f"rel {err / ref:.4g}"


@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("act", [True, False])
def test_conv1d_update_matches_reference_over_several_steps(W, act):
    torch.manual_seed(W)
    N, C = 5, 264
    w = torch.randn(C, W, device="cuda", dtype=torch.bfloat16)
    state = torch.randn(N, C, W, device="cuda", dtype=torch.bfloat16)
    ref_state = state.clone()
    wide = torch.randn(4, N, C + 40, device="cuda", dtype=torch.bfloat16)  # strided rows, like a slice of a projection
    for t in range(4):
        x = wide[t, :, 8:8 + C]
        out = Q.conv1d_update(x, state, w, act)
        ref = Q.conv1d_update_ref(x, ref_state, w, act)
        _close(out, ref)
        assert torch.equal(state, ref_state)


def test_conv_states_of_packed_documents():
    torch.manual_seed(0)
    lengths = torch.tensor([5, 1, 9, 2, 3], device="cuda")
    x = torch.randn(int(lengths.sum()), 96 + 16, device="cuda", dtype=torch.bfloat16)[:, 8:104]
    for W in (2, 4):
        assert torch.equal(Q.conv_states_from_packed(x, lengths, W), Q.conv_states_ref(x, lengths, W))


@pytest.mark.parametrize("d_kind", ["none", "head", "head_dim"])
def test_selective_state_update_matches_reference(d_kind):
    torch.manual_seed(1)
    n, h, p, N, g = 3, 8, 64, 128, 2
    row = torch.randn(n, h * p + 2 * g * N, device="cuda", dtype=torch.bfloat16)  # [x | B | C] as the model lays them out
    x = row[:, :h * p].view(n, h, p)
    B = row[:, h * p:h * p + g * N].view(n, g, N)
    C = row[:, h * p + g * N:].view(n, g, N)
    dt = torch.rand(n, h, device="cuda") * 0.1 + 0.01
    A = -torch.rand(h, device="cuda") * 4
    D = {"none": None, "head": torch.randn(h, device="cuda"), "head_dim": torch.randn(h, p, device="cuda")}[d_kind]
    state = torch.randn(n, h, p, N, device="cuda")
    ref_state = state.clone()
    for _ in range(3):
        y = S.selective_state_update(state, x, dt, A, B, C, D)
        y_ref = S.selective_state_update_ref(ref_state, x, dt, A, B, C, D)
        _close(y, y_ref)
        _close(state, ref_state, 1e-5)


def test_rnn_step_updates_the_cached_state():
    torch.manual_seed(2)
    a = torch.rand(7, 320, device="cuda").bfloat16()
    b = torch.randn(7, 320, device="cuda").bfloat16()
    state = torch.randn(7, 320, device="cuda")
    want = a.float() * state + b.float()
    out = Q.rnn_step(a, b, state)
    assert torch.allclose(state, want, rtol=1e-6, atol=1e-6)
    _close(out, want, 1e-2)


def test_rglru_gates_forward_and_backward():
    torch.manual_seed(3)
    Bsz, Sq, C = 2, 96, 256
    mk = lambda s=1.0: (torch.randn(Bsz, Sq, C, device="cuda") * s).bfloat16().requires_grad_()
    gx, ga, x = mk(), mk(2.0), mk()
    lam = torch.randn(C, device="cuda", requires_grad=True)
    sp = torch.nn.functional.softplus(lam)
    a, b = Q.rglru_gates(gx, ga, x, sp)
    gx2, ga2, x2 = (t.detach().clone().requires_grad_() for t in (gx, ga, x))
    lam2 = lam.detach().clone().requires_grad_()
    a_ref, b_ref = Q.rglru_gates_ref(gx2.float(), ga2.float(), x2.float(), torch.nn.functional.softplus(lam2))
    _close(a, a_ref, 1e-2)
    _close(b, b_ref, 1e-2)
    da, db = torch.randn_like(a), torch.randn_like(b)
    torch.autograd.backward([a, b], [da, db])
    torch.autograd.backward([a_ref, b_ref], [da.float(), db.float()])
    _close(gx.grad, gx2.grad, 3e-2)
    _close(ga.grad, ga2.grad, 3e-2)
    _close(x.grad, x2.grad, 3e-2)
    _close(lam.grad, lam2.grad, 3e-2)
