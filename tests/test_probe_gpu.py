"""The statistics probe on the native (fused-kernel) path: same keys as on the PyTorch path and matching values.
Mirrors the self-checks of lingua/probe.py:554-630 (keys present for every linear layer, statistics equal to
directly computed ones)."""
import json

import pytest
import torch

import copy

from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs, build_fsdp_grouping_plan
from lingua_b200.parallel.engine import EngineOptim, ShardedEngine
from lingua_b200.probe import AutoProbeD

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


def test_probe_native_path_matches_reference_path(tmp_path):
    args = LMTransformerArgs(dim=256, n_layers=2, n_heads=2, vocab_size=512, max_seqlen=128)
    ref, nat, eng = _build(args, seed=2)
    for (_, pr), (_, pn) in zip(ref.named_parameters(), nat.named_parameters()):
        pr.data.copy_(pn.data.float())
    tok = torch.randint(0, 512, (2, 129), device="cuda")
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    out = {}
    for name, model in (("native", nat), ("reference", ref)):
        path = tmp_path / f"{name}.jsonl"
        if name == "native":
            eng.zero_grad()
        with AutoProbeD(model, str(path)) as probe:
            probe.metadata = {"it": 0}
            model(x, y).backward()
        out[name] = json.loads(path.read_text().splitlines()[-1])
    nd, rd = out["native"]["data"], out["reference"]["data"]
    assert out["native"]["version"] == 2 and len(out["native"]["quantiles"]) == 19
    for layer in range(2):
        for lin in ("attention.wq", "attention.wk", "attention.wv", "attention.wo", "feed_forward.w1",
                    "feed_forward.w3", "feed_forward.w2"):
            for what in ("in", "w", "out", "in.g", "out.g", "w.g"):
                key = f"layers.{layer}.{lin}::{what}"
                assert key in nd, key
        assert f"layers.{layer}.attention_norm::resid" in nd and f"layers.{layer}.ffn_norm::resid" in nd
        assert f"layers.{layer}.attention::attn_logits" in nd and f"layers.{layer}.attention::attn_entropy" in nd
    # values: weights are identical; activations and gradients differ by bf16 arithmetic only
    w = dict(nat.named_parameters())["layers.0.attention.wq.weight"]
    assert abs(nd["layers.0.attention.wq::w"]["abs.mean"] - w.float().abs().mean().item()) < 1e-6
    assert tuple(nd["layers.0.attention.wq::w"]["shape"]) == tuple(w.shape)
    for key in ("layers.0.attention.wq::in", "layers.1.feed_forward.w2::out", "layers.0.attention_norm::resid",
                "layers.1.attention.wo::out.g", "layers.0.attention.wo::in.g"):
        # (the input gradient of projections that run as one stacked GEMM - wq|wk|wv, w1|w3 - is reported as
        # their sum on the native path, so those keys are compared by presence only)
        if key in rd:
            a, b = nd[key]["abs.mean"], rd[key]["abs.mean"]
            assert abs(a - b) <= 0.05 * abs(b) + 1e-7, (key, a, b)
            assert abs(nd[key]["std"] - rd[key]["std"]) <= 0.05 * abs(rd[key]["std"]) + 1e-7, key
