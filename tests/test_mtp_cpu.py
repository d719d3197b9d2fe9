"""Multi-token prediction: per-head losses, head 0 in eval, training through the shared loop."""
import json
from pathlib import Path

import torch

from apps.mtp.train import TrainArgs, train
from lingua_b200.config import dataclass_from_dict, load_yaml
from lingua_b200.models.mtp import LMMTPArgs, LMTransformer
from lingua_b200.models.transformer import cross_entropy

ROOT = Path(__file__).resolve().parent.parent


def test_heads_and_eval_mode():
    torch.manual_seed(0)
    m = LMTransformer(LMMTPArgs(dim=64, n_layers=2, n_heads=2, vocab_size=100, n_future_head=3, max_seqlen=16))
    m.init_weights()
    tok = torch.randint(0, 100, (2, 16))
    tgt = torch.randint(0, 100, (2, 16, 3))
    losses = m.train()(tok, tgt)
    assert len(losses) == 3
    logits0 = m.eval()(tok)
    assert torch.allclose(m(tok, tgt[..., 0]), cross_entropy(logits0, tgt[..., 0]))
    assert torch.allclose(losses[0], cross_entropy(logits0, tgt[..., 0]), atol=1e-6)


def test_mtp_app_trains_on_cpu(tmp_path, monkeypatch):
    from lingua_b200 import tokenizer

    monkeypatch.setattr(tokenizer.MockTokenizer, "n_words", 512)
    cfg = {"name": "mtp", "dump_dir": str(tmp_path / "d"), "steps": 4,
           "optim": {"lr": 1e-3, "warmup": 1}, "model": {"dim": 64, "n_layers": 2, "n_heads": 2, "n_future_head": 2},
           "data": {"root_dir": None, "sources": {"synthetic": 1.0}, "batch_size": 2, "seq_len": 32, "n_views": 3,
                    "load_async": False, "tokenizer": {"name": "mock"}},
           "checkpoint": {"dump": {"every": 100}, "eval": {"every": 100}}, "logging": {"freq": 1}}
    train(dataclass_from_dict(TrainArgs, cfg))
    rows = [json.loads(l) for l in open(tmp_path / "d" / "metrics.jsonl")]
    assert len(rows) == 4 and {"loss/out", "loss/head_0", "loss/head_1"} <= set(rows[0])
    assert abs(rows[0]["loss/out"] - rows[0]["loss/head_0"] - rows[0]["loss/head_1"]) < 1e-4
    dataclass_from_dict(TrainArgs, load_yaml(str(ROOT / "apps" / "mtp" / "configs" / "debug.yaml")))
