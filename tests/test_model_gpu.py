"""Native (fused sm_100a) LMTransformer vs the fp32 PyTorch reference path on the same weights."""
import copy

import pytest
import torch

from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs, build_fsdp_grouping_plan
from lingua_b200.parallel.engine import EngineOptim, ShardedEngine

pytestmark = pytest.mark.gpu


def _build(args, seed=0):
    torch.manual_seed(seed)
    ref = LMTransformer(args)
    ref.init_weights()
    nat = copy.deepcopy(ref).cuda()
    eng = ShardedEngine(nat, build_fsdp_grouping_plan(args), process_group=False, compute_dtype=torch.bfloat16,
                        optim=EngineOptim(), device=torch.device("cuda"))
    eng.sync_master()
    return ref.cuda().float(), nat, eng


@pytest.mark.parametrize("act,vocab,kvh", [("swiglu", 1024, 4), ("relu2", 1000, 2), ("swiglu", 259, 1)])
def test_loss_and_grads_match_reference(act, vocab, kvh):
    args = LMTransformerArgs(dim=512, n_layers=2, n_heads=4, n_kv_heads=kvh, vocab_size=vocab, max_seqlen=256,
                             ffn_activation=act, loss_chunk=192)
    ref, nat, eng = _build(args)
    # the reference runs on the bf16-rounded weights so that only arithmetic differs
    for (n, pr), (_, pn) in zip(ref.named_parameters(), nat.named_parameters()):
        pr.data.copy_(pn.data.float())
    tok = torch.randint(0, vocab, (2, 257), device="cuda")
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    y[0, 5] = -100
    ds = torch.zeros(2, 256, dtype=torch.int32, device="cuda")
    ds[:, 100:] = 100
    de = torch.full((2, 256), 100, dtype=torch.int32, device="cuda")
    de[:, 100:] = 256
    eng.zero_grad()
    loss_n = nat(x, y, doc_start=ds, doc_end=de)
    loss_n.backward()
    loss_r = ref(x, y.clone().masked_fill(y < 0, -100), doc_start=ds)
    loss_r.backward()
    assert abs(loss_n.item() - loss_r.item()) < 2e-2 * abs(loss_r.item())
    for (n, pr), (_, pn) in zip(ref.named_parameters(), nat.named_parameters()):
        g_ref, g_nat = pr.grad.float(), pn.main_grad.float()
        denom = g_ref.abs().max().item() + 1e-8
        err = (g_ref - g_nat).abs().max().item() / denom
        assert err < 6e-2, f"{n}: rel grad err {err:.3g}"
    # logits path
    logits = nat(x)
    lr = ref(x)
    assert (logits.float() - lr).abs().max().item() < 5e-2 * lr.abs().max().item()


def test_native_training_reduces_loss():
    args = LMTransformerArgs(dim=256, n_layers=2, n_heads=2, vocab_size=512, max_seqlen=128)
    _, nat, eng = _build(args, seed=1)
    tok = torch.randint(0, 512, (4, 129), device="cuda")
    losses = []
    for step in range(8):
        eng.zero_grad()
        loss = nat(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
        loss.backward()
        eng.step(1e-3)
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.5, losses


def test_fused_loss_backward_equals_recompute_mode():
    args = LMTransformerArgs(dim=256, n_layers=1, n_heads=2, vocab_size=1000, max_seqlen=128, loss_chunk=100)
    _, nat, eng = _build(args, seed=2)
    tok = torch.randint(0, 1000, (2, 129), device="cuda")
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    grads = []
    for scale in (None, 0.5):
        eng.zero_grad()
        nat.loss_grad_scale = scale
        loss = nat(x, y)
        (loss * 0.5).backward()
        grads.append({n: p.main_grad.clone() for n, p in nat.named_parameters()})
    for n in grads[0]:
        a, b = grads[0][n], grads[1][n]
        assert (a - b).abs().max().item() <= 2e-2 * (a.abs().max().item() + 1e-8), n
