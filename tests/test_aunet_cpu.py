"""Hierarchical byte model on CPU: regex pooling levels, the packed data pipeline, the pooling plan against a
direct restatement, the indexed projection against an fp32 gather oracle, every pooling type end to end."""
import json
import os

import numpy as np
import pytest
import torch

from lingua_b200.data.pipeline import (DataArgs, build_dataloader, build_dataloader_from_args,
                                       init_dataloader_state_from_args, split_levels)
from lingua_b200.data.regex_cutting import RegexArgs, RegexPool, map_codepoint_to_byte, shrink_to_valid_bytes
from lingua_b200.models.aunet import (HierarchicalArgs, HierarchicalTransformer, build_fsdp_grouping_plan,
                                      make_level_plan, pool_indices)
from lingua_b200.models.transformer import BaseTransformerArgs
from lingua_b200.ops.indexed_matmul import indexed_matmul, indexed_matmul_ref, plan_groups
from lingua_b200.tokenizer import TokenizerArgs

TEXT = "Hello wörld, this is 1234 a test.\nNew line here "


def test_regex_levels_single_and_two_rules():
    one = RegexPool(RegexArgs({"word1": "1@1"}))
    lv = one.text_levels(TEXT)
    assert len(lv) == len(TEXT.encode())
    # last byte of "Hello ", of "wörld" + the comma that opens a punctuation run, digits in groups of three, ...
    assert [i for i, v in enumerate(lv) if v][:8] == [5, 12, 13, 18, 21, 22, 25, 26]
    two = RegexPool(RegexArgs({"word1": "1@1", "word": "2@1"}))
    lv2 = two.text_levels(TEXT)
    assert set(lv2) == {0, 1, 2}
    assert all((a > 0) == (b > 0) for a, b in zip(lv, lv2))  # the second rule only deepens boundaries here
    assert lv2[5] == 1 and lv2[12] == 2  # every second word end is a level-2 boundary
    with pytest.raises(ValueError):
        RegexPool(RegexArgs({"sentence": "1"}))


def test_byte_windows_specials_and_truncated_characters():
    pool = RegexPool(RegexArgs({"word1": "1@1"}))
    b = list(TEXT.encode())
    full = pool.text_levels(TEXT)
    assert pool.get_levels_mask([256] + b + [257]) == [0] + full + [0]
    cut = b[8:]  # starts inside the two-byte character: its continuation byte gets level 0
    kept, start, end = shrink_to_valid_bytes(cut)
    assert start == 1 and end is None and kept == cut[1:]
    assert len(pool.get_levels_mask(cut)) == len(cut)
    assert pool.get_levels_mask(b[:8])[-1] == 0 and shrink_to_valid_bytes(b[:8])[2] == -1
    assert map_codepoint_to_byte("aé€😀").tolist() == [0, 2, 5, 9]
    first = pool.get_levels_mask_prefill([b[:10], b[:4]], size=64, force_first=True)
    assert len(first) == 14 and first[0] == 1 and first[10] == max(pool.get_levels_mask(b[:4]))
    nxt = pool.get_levels_mask_gen([b[10], b[4]])
    assert nxt == [pool.get_levels_mask(b[:11])[-1], pool.get_levels_mask(b[:5])[-1]]


def test_pipeline_packs_levels_with_tokens(tmp_path):
    src = tmp_path / "src"
    src.mkdir()
    with open(src / "a.chunk.00.jsonl", "w") as f:
        for i in range(40):
            f.write(json.dumps({"text": f"Doc {i}: the quick brown fox, jumps over {i * 37} lazy dogs.\nNext wörld!"}) + "\n")
    args = DataArgs(root_dir=str(tmp_path), sources={"src": 1.0}, batch_size=2, seq_len=64, load_async=False,
                    prefetch_size=4, tokenizer=TokenizerArgs(name="bytes"), regex=RegexArgs({"word1": "1@1"}))
    state = init_dataloader_state_from_args(args, 0, 1)
    with build_dataloader_from_args(args, state) as it:
        batch, st = next(it)
        batch2, _ = next(it)
    tok, lv = split_levels(batch)
    assert batch.shape == (2, 64, 2) and tok.max() <= 257 and set(np.unique(lv)) <= {0, 1}
    assert (tok[:, 1:, 0] == tok[:, :-1, 1]).all() and (lv[:, 1:, 0] == lv[:, :-1, 1]).all()
    assert (lv[tok == 256] == 1).all()  # every document opens at the deepest level
    with build_dataloader_from_args(args, st) as it:  # the state carries the strategy: resuming reproduces
        again, _ = next(it)
    assert (again == batch2).all()


def test_synthetic_levels():
    args = DataArgs(sources={"synthetic": 1.0}, batch_size=4, seq_len=512,
                    regex=RegexArgs({"word1": "1@1", "word": "2@1"}))
    with build_dataloader(init_dataloader_state_from_args(args, 0, 1, 258)) as it:
        batch, _ = next(it)
    tok, lv = split_levels(batch)
    assert tok.max() < 258 and (lv[:, 0, 0] == 2).all()
    assert 0.1 < (lv[:, :, 0] >= 1).mean() < 0.3 and 0.02 < (lv[:, :, 0] >= 2).mean() < 0.12


def _tiny_args(kind="simple_indexed_matmul", lam=0.1):
    return HierarchicalArgs(dimensions=[32, 64, 128], head_dims=[8, 16, 32], layers=[1, 1, 2],
                            sliding_windows=[8, 16, 32], max_seqlens=[48, 20, 8], vocab_size=258, pooling_type=kind,
                            lambda_level=lam, block=BaseTransformerArgs(multiple_of=16, norm_eps=1e-5))


def _pool_mask_oracle(level_mask, caps, n_levels):
    """Row by row, in plain Python: which positions of each stage continue, in that stage's coordinates."""
    B, S = level_mask.shape
    out = [torch.zeros(B, S, dtype=torch.bool) for _ in range(n_levels)]
    for b in range(B):
        lv = level_mask[b].tolist()
        lv[0] = n_levels
        alive = list(range(S))  # byte positions that exist at the current stage
        for i in range(n_levels):
            chosen, taken = [], 0
            for p in range(S):  # the cap counts over all bytes, as the reference does
                if lv[p] > i and taken < caps[i + 1]:
                    taken += 1
                    chosen.append(p)
            for j, p in enumerate(alive):
                out[i][b, j] = p in chosen
            alive = [p for p in alive if p in chosen]
    return out


def test_pool_mask_and_level_plan_match_restatement():
    torch.manual_seed(1)
    model = HierarchicalTransformer(_tiny_args())
    lv = (torch.rand(4, 48) < 0.45).long() + (torch.rand(4, 48) < 0.2).long()
    keep = lv.clone()
    masks, idcs, nb = model.get_pool_mask(lv, [48, 20, 8], return_idcs=True, force_first=True)
    assert (lv == keep).all(), "the caller's level mask is left alone"
    want = _pool_mask_oracle(lv, [48, 20, 8], 2)
    for m, w, n, ids in zip(masks, want, nb, idcs):
        assert (m == w).all() and int(n) == int(w.sum()) and ids.numel() == int(n)
    assert int(masks[0].sum(1).max()) == 20  # the cap binds with this density
    plan = make_level_plan(masks[0], 48, 20, repeat=True, indexed=True)
    for b in range(4):
        true_pos = masks[0][b].nonzero().flatten().tolist()
        assert plan.idx[b, :len(true_pos)].tolist() == true_pos and plan.idx.shape == (4, 20)
        for p in range(48):
            last = max(t for t in true_pos if t <= p)
            assert int(plan.idx[b, plan.repeat_idx[b, p]]) == last and int(plan.position[b, p]) == (p - last) % 16
    assert sum(plan.groups.counts) == 4 * 48
    assert pool_indices(torch.tensor([[False, True, False, True]]), 3).tolist() == [[1, 3, 0]]


def test_indexed_matmul_matches_gather_oracle():
    torch.manual_seed(0)
    x = torch.randn(2, 37, 24, requires_grad=True)
    w = torch.randn(6, 16, 24, requires_grad=True)
    idx = torch.randint(0, 5, (2, 37))  # bank entry 5 is never used: its gradient must be zero
    y, yr = indexed_matmul(x, w, idx), indexed_matmul_ref(x, w, idx)
    assert torch.allclose(y, yr, atol=1e-5)
    g = torch.randn_like(y)
    gx, gw = torch.autograd.grad(y, (x, w), g)
    rx, rw = torch.autograd.grad(yr, (x, w), g)
    assert torch.allclose(gx, rx, atol=1e-5) and torch.allclose(gw, rw, atol=1e-4) and gw[5].abs().max() == 0
    # rows: every output row names the input row it reads (the repeat-upsampling gather folded in)
    small = torch.randn(2, 9, 24, requires_grad=True)
    rows = torch.randint(0, 18, (2, 37))
    y2 = indexed_matmul(small, w, idx, rows=rows)
    ref2 = indexed_matmul_ref(small.reshape(-1, 24)[rows.flatten()].view(2, 37, 24), w, idx)
    assert y2.shape == (2, 37, 16) and torch.allclose(y2, ref2, atol=1e-5)
    for a, b in zip(torch.autograd.grad(y2, (small, w), g), torch.autograd.grad(ref2, (small, w), g)):
        assert torch.allclose(a, b, atol=1e-4)
    plan = plan_groups(idx, 6)
    assert plan.counts == torch.bincount(idx.flatten(), minlength=6).tolist()
    assert (idx.flatten()[plan.order].diff() >= 0).all()


def test_grouped_plan_layout_is_consistent():
    """The device-side layout of the single-launch grouped products, computed here on CPU tensors: every row gets
    its own slot inside its group's 256-row tiles, tiles name their group, contraction ranges cover the tiles."""
    torch.manual_seed(1)
    n, R = 7, 256
    idx = torch.randint(0, n, (3, 1000))
    idx[idx == 4] = 1  # a group without rows
    plan = plan_groups(idx, n, grouped=True)
    flat = idx.flatten()
    T = flat.numel()
    assert plan.grouped and plan._counts is None and plan.padded_rows % R == 0
    assert plan.padded_rows >= int(((plan.counts_dev + R - 1) // R * R).sum())
    assert plan.prow.unique().numel() == T and int(plan.prow.max()) < plan.padded_rows  # one slot per row
    assert torch.equal(plan.pos[plan.order], plan.prow)
    tile_group = plan.sel[plan.pos // R].long()
    assert torch.equal(tile_group, flat)  # the tile a row lands in belongs to the row's group
    k0, kb = plan.k_range[:, 0].long(), plan.k_range[:, 1].long()
    assert kb[4] == 0 and (k0 % R == 0).all()
    for g in range(n):
        rows = plan.pos[flat == g]
        if rows.numel():
            assert int(rows.min()) == int(k0[g]) and int(rows.max()) < int(k0[g] + 64 * kb[g])
    used = int((k0 + 64 * kb).max())
    assert (plan.sel[used // R:] == -1).all() and (plan.sel[:used // R] >= 0).all()  # tiles past the end are skipped


@pytest.mark.parametrize("kind", ["simple_indexed_matmul", "simple", "simple_repeat",
                                  "simple_non_param_indexed_matmul", "simple_non_param"])
def test_model_every_pooling_type(kind):
    torch.manual_seed(0)
    args = _tiny_args(kind)
    model = HierarchicalTransformer(args)
    model.init_weights()
    tok, tgt = torch.randint(0, 258, (3, 48)), torch.randint(0, 258, (3, 48))
    lv = (torch.rand(3, 48) < 0.3).long() + (torch.rand(3, 48) < 0.1).long()
    loss, mask_loss, nb = model(tok, lv, tgt, lv.roll(-1, 1))
    assert abs(float(loss) - np.log(258)) < 1.0 and mask_loss is not None and len(nb) == 2
    (loss + args.lambda_level * mask_loss).backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    logits = model(tok, lv)
    assert logits.shape == (3, 48, 258)
    # causality through pooling and un-pooling: a change at byte 30 leaves every earlier output alone
    tok2, lv2 = tok.clone(), lv.clone()
    tok2[:, 30], lv2[:, 30] = (tok[:, 30] + 1) % 258, 2 - lv[:, 30].clamp(max=2)
    with torch.no_grad():
        assert torch.allclose(model(tok2, lv2)[:, :30], logits[:, :30], atol=1e-5)


def test_estimators_and_plan():
    args = _tiny_args()
    model = HierarchicalTransformer(args)
    blocks = sum(p.numel() for n, p in model.named_parameters() if ".layers." in n and "norm" not in n)
    assert args.estimated_non_embed_param_count == blocks
    assert args.estimated_param_count == blocks + 2 * 32 * 258
    assert args.flops_per_token(48) > args.non_embed_flops_per_token(48) > 0
    assert args.max_batch_size(1e9, 48) > 0 and args.tokens_per_second(48, 1e12) > 0
    assert model.flops_per_token() > 0
    names = [n for n, _ in build_fsdp_grouping_plan(args)]
    assert names == ["encoders.0.layers.0", "decoders.0.layers.0", "encoders.1.layers.0", "decoders.1.layers.0",
                     "trunk.layers.0", "trunk.layers.1"]
    for n in names:
        model.get_submodule(n)


def test_train_app_end_to_end(tmp_path):
    from apps.aunet.train import TrainArgs, train
    from lingua_b200.config import dataclass_from_dict

    cfg = dict(dump_dir=str(tmp_path / "run"), name="aunet", steps=4, seed=1,
               optim=dict(lr=1e-3, warmup=2), distributed=dict(model_dtype="fp32"),
               model=dict(dimensions=[32, 64], head_dims=[8, 16], layers=[1, 2], sliding_windows=[16, 32],
                          max_seqlens=[-1, 24], block=dict(multiple_of=16), lambda_level=0.1),
               data=dict(sources={"synthetic": 1.0}, batch_size=2, seq_len=64, load_async=False,
                         tokenizer=dict(name="bytes"), regex=dict(strategy={"word1": "1@1"})),
               checkpoint=dict(dump=dict(every=2, keep=1)), logging=dict(freq=1))
    import multiprocessing as mp

    method = mp.get_start_method(allow_none=True)
    try:
        metrics = train(dataclass_from_dict(TrainArgs, cfg))
    finally:  # the job sets the worker start method for its data loader: leave the process as it was
        mp.set_start_method(method, force=True)
    assert {"loss/out", "ce/out", "mask_loss/out", "nb_toks/enc_0"} <= set(metrics)
    assert 0 < metrics["nb_toks/enc_0"] <= 2 * 24 and metrics["loss/out"] > metrics["ce/out"]
    assert os.path.isdir(tmp_path / "run" / "checkpoints" / "0000000004")


def test_sharded_two_ranks_match_single_process():
    """gloo, world size 2: the engine shards every block of every stage plus the root group (embeddings,
    transitions, heads); the losses of three optimiser steps equal the single-process run."""
    import subprocess
    import sys
    from pathlib import Path

    worker = str(Path(__file__).resolve().parent / "aunet_dist_worker.py")
    env = dict(os.environ, OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1")

    def losses(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
        assert proc.returncode == 0, proc.stderr[-2000:]
        line = [l for l in proc.stdout.splitlines() if l.startswith("LOSSES ")][-1]
        return json.loads(line[len("LOSSES "):])

    one = losses([sys.executable, worker, "1", "3"])
    two = losses([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                  "127.0.0.1", "--master-port", "29641", worker, "2", "3"])
    assert len(one) == 3 and all(abs(a - b) < 2e-4 * max(1.0, abs(a)) for a, b in zip(one, two)), (one, two)
