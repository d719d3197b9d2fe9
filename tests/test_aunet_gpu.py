"""Hierarchical byte model on a B200: the indexed projection and the padded-head attention against fp32
oracles, and the sharded-engine training path against the same model in fp32 on the CPU."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_indexed_matmul_bf16_vs_fp32_oracle():
    from lingua_b200.ops.indexed_matmul import indexed_matmul, indexed_matmul_ref

    torch.manual_seed(0)
    dev = "cuda"
    x = (torch.randn(4, 1024, 256, device=dev) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(16, 128, 256, device=dev) * 0.06).bfloat16().requires_grad_()
    idx = torch.randint(0, 16, (4, 1024), device=dev)
    idx[idx == 7] = 3  # one bank entry without rows
    y = indexed_matmul(x, w, idx)
    yr = indexed_matmul_ref(x, w, idx)
    assert (y.float() - yr).abs().max() < 0.03 * yr.abs().max()
    g = torch.randn_like(y)
    gx, gw = torch.autograd.grad(y, (x, w), g)
    rx, rw = torch.autograd.grad(yr, (x, w), g.float())
    assert (gx.float() - rx.float()).abs().max() < 0.03 * rx.abs().max()
    assert (gw.float() - rw.float()).abs().max() < 0.03 * rw.abs().max() and gw[7].abs().max() == 0


def test_indexed_matmul_grouped_launch_matches_the_group_loop():
    """The single-launch grouped path against the loop of plain products, with repeated source rows and an
    engine-style fp32 gradient buffer that is accumulated into over two backward passes."""
    from lingua_b200.ops.indexed_matmul import indexed_matmul, plan_groups

    torch.manual_seed(5)
    dev = "cuda"
    x = (torch.randn(700, 256, device=dev) * 0.5).bfloat16().requires_grad_()
    idx = torch.randint(0, 16, (2, 1500), device=dev)
    idx[idx == 2] = 9
    rows = torch.randint(0, 700, (2, 1500), device=dev)
    outs = []
    for grouped in (True, False):
        w = (torch.randn(16, 128, 256, generator=torch.Generator().manual_seed(6)) * 0.06).bfloat16().to(dev).requires_grad_()
        w.main_grad = torch.full((16, 128, 256), float("nan"), device=dev)
        plan = plan_groups(idx, 16, grouped=grouped)
        assert plan.grouped == grouped and (not grouped or plan._counts is None)
        gx = 0
        for rep in range(2):
            y = indexed_matmul(x, w, idx, plan, rows)
            g = torch.randn(y.shape, generator=torch.Generator().manual_seed(7 + rep)).to(dev).bfloat16()
            gx = gx + torch.autograd.grad(y, x, g)[0].float()
        assert plan._counts is None or not grouped  # the grouped path never reads the sizes
        outs.append((y.float(), gx, w.main_grad.clone()))
    (y1, gx1, gw1), (y0, gx0, gw0) = outs
    assert (y1 - y0).abs().max() < 0.02 * y0.abs().max()
    assert (gx1 - gx0).abs().max() < 0.02 * gx0.abs().max()
    assert torch.isfinite(gw1).all() and (gw1 - gw0).abs().max() < 0.01 * gw0.abs().max() and gw1[2].abs().max() == 0


def test_gemm_operands_with_ragged_pitch():
    """A byte-vocabulary head has 258 outputs: its gradient has a row pitch that TMA cannot address."""
    from lingua_b200.ops.gemm import mm_nn, mm_tn

    torch.manual_seed(2)
    dy = (torch.randn(1000, 258, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(258, 512, device="cuda") * 0.1).bfloat16()
    x = (torch.randn(1000, 512, device="cuda") * 0.5).bfloat16()
    dx = mm_nn(dy, w)
    assert (dx.float() - dy.float() @ w.float()).abs().max() < 0.05
    dw = mm_tn(dy, x, out_dtype=torch.float32)
    want = dy.float().t() @ x.float()
    assert dw.shape == (258, 512) and (dw - want).abs().max() < 0.02 * want.abs().max()


@pytest.mark.parametrize("head_dim,window", [(64, 0), (64, 96), (32, 40)])
def test_narrow_heads_through_the_128_wide_kernel(head_dim, window):
    from lingua_b200.models.transformer import _attention_flash_padded, _attention_torch

    torch.manual_seed(1)
    q, k, v = ((torch.randn(2, 384, 4, head_dim, device="cuda")).bfloat16().requires_grad_() for _ in range(3))
    o = _attention_flash_padded(q, k, v, True, window)
    ref = _attention_torch(q.float(), k.float(), v.float(), True, None, window)
    assert o.shape == ref.shape and (o.float() - ref).abs().max() < 0.03
    g = torch.randn_like(o)
    got = torch.autograd.grad(o, (q, k, v), g)
    want = torch.autograd.grad(ref, (q, k, v), g.float())
    for a, b in zip(got, want):
        assert (a.float() - b.float()).abs().max() < 0.05 * max(1.0, b.abs().max().item())


def test_generator_decoding_matches_full_forward_bf16():
    """Prefill + byte-by-byte decoding against the one-pass forward: the trunk (heads of 128) runs the native
    prefill and decode-attention kernels, the byte stage (heads of 64) the generic cached path."""
    from lingua_b200.data.regex_cutting import RegexArgs, RegexPool
    from lingua_b200.generation_aunet import (PackedHierarchicalCausalTransformerGenerator as Generator,
                                              PackedHierarchicalCausalTransformerGeneratorArgs as GenArgs)
    from lingua_b200.models.aunet import HierarchicalArgs, HierarchicalTransformer
    from lingua_b200.models.transformer import BaseTransformerArgs
    from lingua_b200.tokenizer import build_tokenizer

    args = HierarchicalArgs(dimensions=[128, 256], head_dims=[64, 128], layers=[1, 2], sliding_windows=[32, 128],
                            max_seqlens=[128, 128], vocab_size=258, block=BaseTransformerArgs(multiple_of=64, norm_eps=1e-5))
    torch.manual_seed(0)
    model = HierarchicalTransformer(args)
    model.init_weights()
    model = model.cuda().bfloat16().eval()
    for mod in model.modules():
        if hasattr(mod, "reset_parameters") and type(mod).__name__ == "RotaryEmbedding":
            mod.reset_parameters()
    n, L, P = 3, 80, [30, 41, 36]
    tok = torch.randint(0, 256, (n, L), device="cuda")
    lv = (torch.rand(n, L, device="cuda") < 0.35).long()
    lv[:, 0] = 1
    gen = Generator(GenArgs(max_gen_len=40, max_tokens=600), model, build_tokenizer("bytes"),
                    RegexPool(RegexArgs({"word1": "1@1"})))
    ptok, plv = torch.zeros(n, max(P), dtype=torch.long, device="cuda"), torch.zeros(n, max(P), dtype=torch.long, device="cuda")
    for i in range(n):
        ptok[i, :P[i]], plv[i, :P[i]] = tok[i, :P[i]], lv[i, :P[i]]
    with torch.no_grad():
        full = model(tok, lv).float()
        pre = gen.prefill(ptok, plv, torch.tensor(P, device="cuda")).float()
        for i in range(n):
            assert (pre[i, :P[i]] - full[i, :P[i]]).abs().max() < 0.08
        for s in range(30):
            cur = torch.stack([tok[i, P[i] + s] for i in range(n)])
            cur_lv = torch.stack([lv[i, P[i] + s] for i in range(n)])
            logits = gen.generate_next_token(cur, cur_lv).float()
            for i in range(n):
                assert (logits[i] - full[i, P[i] + s]).abs().max() < 0.08, (s, i)
    gen.release_cache()


def test_engine_training_step_matches_fp32():
    import copy

    from lingua_b200.models.aunet import HierarchicalArgs, HierarchicalTransformer, build_fsdp_grouping_plan
    from lingua_b200.models.transformer import BaseTransformerArgs
    from lingua_b200.parallel.engine import EngineOptim, ShardedEngine

    args = HierarchicalArgs(dimensions=[128, 256], head_dims=[64, 128], layers=[1, 2], sliding_windows=[64, 128],
                            max_seqlens=[256, 96], vocab_size=258, lambda_level=0.1,
                            block=BaseTransformerArgs(multiple_of=64, norm_eps=1e-5))
    torch.manual_seed(0)
    ref = HierarchicalTransformer(args)
    ref.init_weights()
    model = copy.deepcopy(ref).cuda()
    model._engine = engine = ShardedEngine(model, build_fsdp_grouping_plan(args), process_group=False,
                                           compute_dtype=torch.bfloat16, optim=EngineOptim(),
                                           device=torch.device("cuda"))
    engine.sync_master()
    ref = ref.cuda().float()
    for (_, pr), (_, pn) in zip(ref.named_parameters(), model.named_parameters()):
        pr.data.copy_(pn.data.float())  # same bf16-rounded weights: only the arithmetic differs
    tok, tgt = torch.randint(0, 258, (2, 256), device="cuda"), torch.randint(0, 258, (2, 256), device="cuda")
    lv = (torch.rand(2, 256, device="cuda") < 0.3).long()
    l_ref, m_ref, nb_ref = ref(tok, lv, tgt, lv.roll(-1, 1))
    (l_ref + 0.1 * m_ref).backward()
    engine.zero_grad()
    l, m, nb = model(tok, lv, tgt, lv.roll(-1, 1))
    (l + 0.1 * m).backward()
    assert abs(float(l) - float(l_ref)) < 0.03 and abs(float(m) - float(m_ref)) < 0.03
    assert [int(a) for a in nb] == [int(b) for b in nb_ref]
    gn = float(engine.step(1e-3))
    gn_ref = math.sqrt(sum(float(p.grad.float().pow(2).sum()) for p in ref.parameters()))
    assert abs(gn - gn_ref) < 0.05 * gn_ref
