"""Memory-bound kernels vs their fp32 PyTorch references."""
import pytest
import torch

from lingua_b200.ops import functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item() + 1e-6
    assert err / ref < tol, f"rel {err / ref:.4g}"


@pytest.mark.parametrize("M,D", [(64, 256), (300, 4096), (17, 2048), (33, 8192), (21, 1000), (9, 5120), (3, 3072)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(M, D, with_res):
    torch.manual_seed(0)
    x = torch.randn(M, D, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, D, device=DEV, dtype=torch.bfloat16) if with_res else None
    w = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    y, h, rstd = F.rmsnorm_fwd(x, w, 1e-5, res)
    yr, hr, rr = F.rmsnorm_fwd_ref(x, w, 1e-5, res)
    close(y, yr)
    close(rstd, rr, 1e-3)
    if with_res:
        close(h, hr)
    hh = h if with_res else x
    dy = torch.randn(M, D, device=DEV, dtype=torch.bfloat16)
    dres = torch.randn(M, D, device=DEV, dtype=torch.bfloat16)
    dx, dw = F.rmsnorm_bwd(dy, hh, w, rstd, dres)
    dxr, dwr = F.rmsnorm_bwd_ref(dy, hh, w, rr.view(M), dres)
    close(dx, dxr)
    close(dw, dwr)


def test_rope_roundtrip_and_ref():
    torch.manual_seed(0)
    B, S, H, Dh = 2, 96, 13, 128  # eleven rotated heads: one group of eight and three single ones
    qkv = torch.randn(B * S, H * Dh, device=DEV, dtype=torch.bfloat16)
    R = 11
    cs = F.rope_table(Dh, S, 10000.0, DEV)
    ref = F.rope_ref(qkv[:, : R * Dh].reshape(B, S, R, Dh), cs)
    orig = qkv.clone()
    F.rope_(qkv, cs, R, Dh, S)
    close(qkv[:, : R * Dh].reshape(B, S, R, Dh), ref)
    assert torch.equal(qkv[:, R * Dh:], orig[:, R * Dh:])
    F.rope_(qkv, cs, R, Dh, S, backward=True)
    close(qkv, orig, 3e-2)
    pos = torch.randint(0, S, (B * S,), device=DEV, dtype=torch.int32)
    q2 = orig.clone()
    F.rope_(q2, cs, R, Dh, S, pos=pos)
    ref2 = F.rope_ref(orig[:, : R * Dh].reshape(B, S, R, Dh), cs, pos)
    close(q2[:, : R * Dh].reshape(B, S, R, Dh), ref2)


@pytest.mark.parametrize("mode", [F.ACT_SILU, F.ACT_RELU2])
def test_glu_and_act(mode):
    torch.manual_seed(0)
    M, H = 130, 512
    gu = torch.randn(M, 2 * H, device=DEV, dtype=torch.bfloat16)
    out = F.glu_fwd(gu, mode)
    close(out, F.glu_fwd(gu.cpu(), mode))
    d = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    close(F.glu_bwd(gu, d, mode), F.glu_bwd(gu.cpu(), d.cpu(), mode))
    x = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    close(F.act_fwd(x, mode), F.act_fwd(x.cpu(), mode))
    close(F.act_bwd(x, d, mode), F.act_bwd(x.cpu(), d.cpu(), mode))
    close(F.add(x, d), x.float() + d.float())


def test_embedding():
    torch.manual_seed(0)
    V, D = 1000, 256
    table = torch.randn(V, D, device=DEV, dtype=torch.bfloat16)
    tok = torch.randint(0, V, (4, 33), device=DEV)
    out = F.embed_fwd(tok, table)
    assert torch.equal(out, table[tok])
    dy = torch.randn(4, 33, D, device=DEV, dtype=torch.bfloat16)
    dt = torch.zeros(V, D, device=DEV)
    F.embed_bwd(tok, dy, dt)
    ref = torch.zeros(V, D, device=DEV).index_add_(0, tok.reshape(-1), dy.reshape(-1, D).float())
    close(dt, ref, 1e-3)


def test_cross_entropy():
    torch.manual_seed(0)
    rows, V = 64, 32008
    logits = torch.randn(rows, V, device=DEV) * 3
    tgt = torch.randint(0, V, (rows,), device=DEV)
    tgt[5] = -100
    loss, lse = F.ce_fwd(logits, tgt)
    lr, lser = F.ce_fwd(logits.cpu(), tgt.cpu())
    close(loss, lr, 1e-4)
    close(lse, lser, 1e-4)
    g = torch.tensor([0.5], device=DEV)
    d = F.ce_bwd(logits, tgt, lse, 1.0 / rows, g)
    dr = F.ce_bwd(logits.cpu(), tgt.cpu(), lser, 1.0 / rows, g.cpu())
    close(d, dr, 2e-2)
    assert d[5].abs().max().item() == 0


def test_adamw_and_sumsq_match_torch():
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 0.1
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        ref_p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        ss = torch.zeros(1, device=DEV)
        F.sumsq(g, ss)
        close(ss.sqrt(), g.norm().reshape(1), 1e-4)
        F.adamw_step(p, m, v, g, p16, step=step, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1,
                     sumsq_t=ss, max_norm=1.0)
        close(p, ref_p.data, 1e-4)
    close(p16, p, 1e-2)
