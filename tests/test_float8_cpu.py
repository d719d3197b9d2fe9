"""Float8 linear layers: the PyTorch statement of the arithmetic (runs on CPU)."""
import torch
import torch.nn as nn

from lingua_b200 import float8 as F8
from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs


def test_row_quantisation_round_trip():
    torch.manual_seed(0)
    x = torch.randn(32, 64) * torch.logspace(-3, 3, 32)[:, None]
    q, s = F8.quant_rows_ref(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (32,)
    back = q.float() * s[:, None]
    # e4m3 keeps 3 mantissa bits: relative error of a normal value <= 2^-4, and the row maximum maps to 448
    assert ((back - x).abs() <= x.abs() * 2 ** -4 + s[:, None] * 2 ** -7).all()
    assert torch.allclose(q.float().abs().amax(-1), torch.full((32,), 448.0))
    zq, zs = F8.quant_rows_ref(torch.zeros(2, 16))
    assert torch.isfinite(zs).all() and (zq.float() == 0).all()


def test_linear_fn_matches_fp32_within_fp8_error():
    torch.manual_seed(1)
    x = torch.randn(48, 64, requires_grad=True)
    w = torch.randn(32, 64, requires_grad=True)
    b = torch.randn(32, requires_grad=True)
    out = F8.Fp8LinearFn.apply(x, w, b)
    ref = x @ w.t() + b
    assert (out - ref).abs().max() < 0.08 * ref.abs().max()
    dy = torch.randn_like(ref)
    dx, dw, db = torch.autograd.grad(out, (x, w, b), dy)
    rx, rw, rb = torch.autograd.grad(ref, (x, w, b), dy)
    assert (dx - rx).abs().max() < 0.1 * rx.abs().max()
    assert torch.allclose(dw, rw, atol=1e-4) and torch.allclose(db, rb, atol=1e-5)  # weight gradient is not float8


def test_convert_marks_filtered_linears_only():
    args = LMTransformerArgs(dim=64, n_layers=2, n_heads=2, vocab_size=128, max_seqlen=32)
    m = LMTransformer(args)
    m.init_weights()
    F8.convert_linears_to_fp8(m, "rowwise", r"layers\.[0-9]+\.")
    marked = {n for n, p in m.named_parameters() if getattr(p, "lb_fp8", False)}
    assert marked and all(n.startswith("layers.") and "norm" not in n for n in marked)
    assert "output.weight" not in marked and "tok_embeddings.weight" not in marked
    seq = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 10))
    F8.convert_linears_to_fp8(seq, "rowwise", r".*")
    assert isinstance(seq[0], F8.Fp8Linear) and not isinstance(seq[2], F8.Fp8Linear)  # 10 is not a multiple of 16
    try:
        F8.convert_linears_to_fp8(seq, "tensorwise", ".*")
        assert False
    except RuntimeError:
        pass


def test_fp8_model_trains_on_cpu():
    torch.manual_seed(2)
    args = LMTransformerArgs(dim=64, n_layers=2, n_heads=2, vocab_size=64, max_seqlen=32)
    m = LMTransformer(args)
    m.init_weights()
    ref_loss = None
    tok = torch.randint(0, 64, (4, 33))
    with torch.no_grad():
        ref_loss = m(tok[:, :-1], tok[:, 1:]).item()
    F8.convert_linears_to_fp8(m, "rowwise", r"layers\.[0-9]+\.")
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(15):
        loss = m(tok[:, :-1], tok[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert abs(losses[0] - ref_loss) < 0.05 * ref_loss
    assert losses[-1] < losses[0] - 0.3


def test_row_parallel_split_equals_sub_row_scaling():
    """Under tensor parallelism a row-parallel product splits the reduction dim over the ranks and every rank
    quantises its own slice with its own per-row scales. That is the sub-row scaling the reference switches to
    for operands sharded along the reduction dim (lingua/float8.py:14-21, 86-88): one scale per row and K-chunk."""
    from lingua_b200 import float8 as F8

    torch.manual_seed(0)
    M, N, K, tp = 24, 40, 128, 2
    x = torch.randn(M, K) * torch.logspace(-2, 1, K)  # very different magnitudes in the two halves of K
    w = torch.randn(N, K) * 0.05
    ours = sum(F8.fp8_forward_mm(xc.contiguous(), wc.contiguous()) for xc, wc in zip(x.chunk(tp, 1), w.chunk(tp, 1)))

    def sub_row(t):  # the reference's formula, restated: amax over (rows, tp chunks)
        amax = t.abs().unflatten(-1, (tp, -1)).amax(dim=-1)
        scale = amax.float().clamp(min=1e-12) / torch.finfo(torch.float8_e4m3fn).max
        q = (t.unflatten(-1, (tp, -1)) / scale[..., None]).to(torch.float8_e4m3fn)
        return q, scale

    x8, sx = sub_row(x)
    w8, sw = sub_row(w)
    want = sum((x8[:, c].float() @ w8[:, c].float().t()) * sx[:, c, None] * sw[None, :, c] for c in range(tp))
    assert torch.allclose(ours, want, rtol=1e-5, atol=1e-6)
    one_scale = F8.fp8_forward_mm(x, w)  # a single scale per row loses the small half of K
    exact = x @ w.t()
    assert (ours - exact).abs().max() < (one_scale - exact).abs().max()
