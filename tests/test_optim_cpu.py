"""LR schedules (closed forms) and the sharded AdamW against torch.optim.AdamW."""
import math

import torch

from lingua_b200.optim import LRScheduler, OptimArgs, build_lr_fn, lr_cosine, lr_inv_sqrt, lr_linear, lr_wsd
from lingua_b200.ops import functional as F


def test_schedules():
    assert lr_linear(5, 10, 100, 0.1) == 0.5
    assert abs(lr_linear(55, 10, 100, 0.1) - (0.5 * 0.1 + 0.5)) < 1e-12
    assert lr_linear(1000, 10, 100, 0.1) == 0.1
    assert abs(lr_inv_sqrt(400, 100, 0.5, 0.01) - 0.5) < 1e-12
    assert abs(lr_cosine(10, 10, 110, 1.0, 1.0, 0.1) - 1.0) < 1e-12
    assert 0.1 <= lr_cosine(109, 10, 110, 1.0, 1.0, 0.1) < 0.101
    assert lr_cosine(500, 10, 110, 1.0, 1.0, 0.1) == 0.1
    assert abs(lr_cosine(60, 10, 110, 1.0, 1.0, 0.0) - 0.5) < 1e-12
    assert lr_wsd(50, 10, 100, 0.1, 1.0, 0.1) == 1.0
    assert abs(lr_wsd(100, 10, 100, 0.1, 1.0, 0.1) - 0.1) < 1e-12
    assert abs(lr_wsd(95, 10, 100, 0.1, 1.0, 0.1) - 1 / (0.5 * 10 + 0.5)) < 1e-12


def test_scheduler_matches_lambdalr_and_state_roundtrip():
    args = OptimArgs(lr=1e-2, warmup=3, scheduler="cosine", lr_min_ratio=0.1)
    fn = build_lr_fn(args, 20)
    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.AdamW([p], lr=args.lr)
    ref = torch.optim.lr_scheduler.LambdaLR(opt, fn)
    mine = LRScheduler(args.lr, fn)
    for _ in range(20):
        assert abs(opt.param_groups[0]["lr"] - mine.get_lr()) < 1e-15
        opt.step()
        ref.step()
        mine.step()
    sd = mine.state_dict()
    assert set(ref.state_dict()) >= {"last_epoch", "base_lrs"} and sd["last_epoch"] == ref.state_dict()["last_epoch"]
    other = LRScheduler(args.lr, fn)
    other.load_state_dict(sd)
    assert other.get_lr() == mine.get_lr()


def test_flat_adamw_matches_torch_cpu():
    torch.manual_seed(0)
    n = 1001
    p = torch.randn(n)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(n), torch.zeros(n)
    p16 = torch.zeros(n)
    for step in range(1, 5):
        g = torch.randn(n)
        ref_p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        ss = torch.zeros(1)
        F.sumsq(g, ss)
        F.adamw_step(p, m, v, g, p16, step=step, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, sumsq_t=ss,
                     max_norm=1.0)
        assert torch.allclose(p, ref_p.data, atol=1e-6)
    assert torch.equal(p16, p)
