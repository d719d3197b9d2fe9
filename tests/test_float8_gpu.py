"""Float8 kernels (quantisation, scaled tcgen05 GEMM) against their PyTorch statements, and a float8 model."""
import copy

import pytest
import torch

from lingua_b200 import float8 as F8
from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs, build_fsdp_grouping_plan
from lingua_b200.ops import _lib
from lingua_b200.parallel.engine import EngineOptim, ShardedEngine

pytestmark = pytest.mark.gpu
bf = torch.bfloat16


@pytest.mark.parametrize("rows,K", [(64, 128), (300, 4096), (17, 11008), (8, 16384), (5, 22016)])
def test_quant_rows_matches_reference(rows, K):
    torch.manual_seed(0)
    x = (torch.randn(rows, K, device="cuda") * torch.logspace(-2, 2, rows, device="cuda")[:, None]).to(bf)
    q, s = F8.quant_rows(x)
    qr, sr = F8.quant_rows_ref(x)
    assert torch.allclose(s, sr, rtol=1e-6, atol=0)
    # the kernel multiplies by an approximate reciprocal: a value that sits on a rounding boundary may land on the
    # neighbouring code, never further
    a, b = q.float(), qr.float()
    assert ((a - b).abs() <= b.abs() * 0.126 + 2 ** -9).all()
    assert (a != b).float().mean().item() < 1e-3


def test_quant_transpose_matches_reference():
    torch.manual_seed(1)
    w = torch.randn(272, 200, device="cuda").to(bf)
    s = (w.abs().amax().float() / 448).reshape(1)
    q = F8.quant_transpose(w, s)
    qr = F8.quant_transpose_ref(w, s)
    assert q.shape == (200, 272)
    a, b = q.float(), qr.float()
    assert ((a - b).abs() <= b.abs() * 0.126 + 2 ** -9).all() and (a != b).float().mean().item() < 1e-3


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (1000, 528, 1024), (4096, 4096, 4096), (16, 48, 80)])
def test_scaled_mm_matches_fp32(M, N, K):
    torch.manual_seed(2)
    a8, sa = F8.quant_rows(torch.randn(M, K, device="cuda").to(bf))
    b8, sb = F8.quant_rows(torch.randn(N, K, device="cuda").to(bf))
    out = F8.scaled_mm(a8, sa, b8, sb)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = F8.scaled_mm_ref(a8, sa, b8, sb, torch.float32)
    assert (out.float() - ref).abs().max().item() < 1e-2 * ref.abs().max().item()
    out32 = F8.scaled_mm(a8, sa[:1] * 0 + 0.5, b8, sb[:1] * 0 + 2.0, torch.float32)  # one scale per operand
    ref32 = a8.float() @ b8.float().t()
    assert (out32 - ref32).abs().max().item() < 1e-4 * ref32.abs().max().item()


def test_fp8_products_close_to_bf16():
    torch.manual_seed(3)
    x = torch.randn(512, 1024, device="cuda").to(bf)
    w = (torch.randn(768, 1024, device="cuda") * 0.03).to(bf)
    dy = torch.randn(512, 768, device="cuda").to(bf)
    y = F8.fp8_forward_mm(x, w)
    ref = x.float() @ w.float().t()
    assert (y.float() - ref).abs().max().item() < 0.06 * ref.abs().max().item()
    dx = F8.fp8_dgrad_mm(dy, w)
    rdx = dy.float() @ w.float()
    assert (dx.float() - rdx).abs().max().item() < 0.08 * rdx.abs().max().item()


def test_fp8_model_matches_bf16_and_trains():
    args = LMTransformerArgs(dim=512, n_layers=2, n_heads=4, vocab_size=1024, max_seqlen=256)
    torch.manual_seed(4)
    base = LMTransformer(args)
    base.init_weights()
    models = []
    for fp8 in (False, True):
        m = copy.deepcopy(base).cuda()
        if fp8:
            F8.convert_linears_to_fp8(m, "rowwise", r"layers\.[0-9]+\.")
        eng = ShardedEngine(m, build_fsdp_grouping_plan(args), process_group=False, compute_dtype=bf,
                            optim=EngineOptim(), device=torch.device("cuda"))
        eng.sync_master()
        models.append((m, eng))
    (m16, _), (m8, e8) = models
    assert any(getattr(p, "lb_fp8", False) for p in m8.parameters()), "marks must survive the engine's re-homing"
    tok = torch.randint(0, 1024, (4, 257), device="cuda")
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    with torch.no_grad():
        l16, l8 = m16(x, y).item(), m8(x, y).item()
    assert abs(l16 - l8) < 0.02 * l16
    losses = []
    for step in range(12):
        e8.zero_grad()
        loss = m8(x, y)
        loss.backward()
        e8.step(lr=2e-3)
        losses.append(loss.item())
    _lib.check_status()
    assert losses[-1] < losses[0] - 0.5, losses


@pytest.mark.parametrize("M,N,K", [(2048, 4096, 1024), (8192, 2560, 512), (2304, 2304, 4096)])
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_scaled_mm_on_sm_pairs_and_e5m2(M, N, K, fmt):
    """Problems large enough for the SM-pair kernel (256 x 256 tiles, scales applied in its TMA-store epilogue);
    the activation operand in either float8 format."""
    torch.manual_seed(4)
    a8, sa = F8.quant_rows(torch.randn(M, K, device="cuda").to(bf), fmt)
    assert a8.dtype == (torch.float8_e5m2 if fmt == "e5m2" else torch.float8_e4m3fn)
    b8, sb = F8.quant_rows(torch.randn(N, K, device="cuda").to(bf))
    for dt in (bf, torch.float32):
        out = F8.scaled_mm(a8, sa, b8, sb, dt)
        torch.cuda.synchronize()
        _lib.check_status()
        ref = F8.scaled_mm_ref(a8, sa, b8, sb, torch.float32)
        assert (out.float() - ref).abs().max().item() < 1e-2 * ref.abs().max().item()
