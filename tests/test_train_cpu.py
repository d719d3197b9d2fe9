"""End-to-end CPU runs of the training app: the fp32 debug configuration (dim 256, 4 layers, 4 heads,
vocab 32000, 2 x 512 tokens, 10 AdamW steps), checkpoint layout, exact resume, consolidation,
generation from the consolidated checkpoint, probe output."""
import json
from pathlib import Path

import pytest
import torch

from apps.main.train import TrainArgs, train
from lingua_b200.config import dataclass_from_dict


def _cfg(dump_dir, steps=10, **over):
    cfg = {
        "name": "cpu_debug", "dump_dir": str(dump_dir), "steps": steps, "seed": 42,
        "optim": {"lr": 3e-4, "weight_decay": 0.1, "warmup": 2, "scheduler": "cosine"},
        "model": {"dim": 256, "n_layers": 4, "n_heads": 4, "norm_eps": 1e-5, "rope_theta": 10000.0,
                  "ffn_dim_multiplier": 1.0, "multiple_of": 768 // 3, "vocab_size": 32000, "init_base_std": 0.02},
        "data": {"root_dir": None, "sources": {"synthetic": 1.0}, "batch_size": 2, "seq_len": 512,
                 "load_async": False, "tokenizer": {"name": "mock"}},
        "distributed": {"fsdp_type": "full_shard", "model_dtype": "bf16"},
        "checkpoint": {"dump": {"every": 5, "keep": 0}, "eval": {"every": 1000, "keep": 0}},
        "logging": {"freq": 1},
    }
    for k, v in over.items():
        cfg[k] = v
    return cfg


class _MockVocab:
    pass


@pytest.fixture(autouse=True)
def _mock_tokenizer_vocab(monkeypatch):
    # the mock tokenizer reports 256 words; the debug config uses a 32000-word synthetic vocabulary
    from lingua_b200 import tokenizer

    monkeypatch.setattr(tokenizer.MockTokenizer, "n_words", 32000)


def _losses(dump_dir):
    return [json.loads(l)["loss/out"] for l in open(Path(dump_dir) / "metrics.jsonl")]


def test_debug_config_trains_and_is_repeatable(tmp_path):
    a = train(dataclass_from_dict(TrainArgs, _cfg(tmp_path / "a")))
    la = _losses(tmp_path / "a")
    assert len(la) == 10 and la[-1] < la[0], la
    assert abs(la[0] - 10.37) < 0.7  # about ln(32000) at initialisation
    train(dataclass_from_dict(TrainArgs, _cfg(tmp_path / "b")))
    assert _losses(tmp_path / "b") == la  # bitwise repeatable on CPU
    assert a["global_step"] == 10


def test_checkpoint_layout_resume_consolidate_generate(tmp_path):
    import shutil

    d = tmp_path / "run"
    train(dataclass_from_dict(TrainArgs, _cfg(d, steps=10)))
    full = _losses(d)
    ck = d / "checkpoints" / "0000000005"
    names = {p.name for p in ck.iterdir()}
    assert {".metadata", "params.json", "train_state_00000.json"} <= names
    assert any(n.endswith(".distcp") for n in names)
    ts = json.loads((ck / "train_state_00000.json").read_text())
    assert ts["step"] == 5 and set(ts) == {"step", "acc_step", "data_loader_state", "scheduler"}
    # a job that died after step 5: only that checkpoint is left; rerunning the same command resumes
    r = tmp_path / "resumed"
    shutil.copytree(d, r)
    shutil.rmtree(r / "checkpoints" / "0000000010")
    (r / "metrics.jsonl").unlink()
    cfg = _cfg(r, steps=10)
    train(dataclass_from_dict(TrainArgs, cfg))
    assert _losses(r) == full[5:]
    # consolidated checkpoint has the reference's key names
    from lingua_b200.checkpoint import consolidate_checkpoints
    from lingua_b200.generation import (PackedCausalTransformerGenerator, PackedCausalTransformerGeneratorArgs,
                                        load_consolidated_model_and_tokenizer)

    cons = consolidate_checkpoints(str(d / "checkpoints" / "0000000010"))
    sd = torch.load(cons / "consolidated.pth", weights_only=True)
    assert {"tok_embeddings.weight", "layers.0.attention.wq.weight", "layers.3.feed_forward.w2.weight",
            "layers.0.attention_norm.weight", "norm.weight", "output.weight"} <= set(sd["model"])
    assert "layers.0.attention.wq.weight" in sd["optim"]["state"]
    assert {"exp_avg", "exp_avg_sq", "step"} <= set(sd["optim"]["state"]["norm.weight"])
    model, tok, _ = load_consolidated_model_and_tokenizer(str(cons))
    from lingua_b200.tokenizer import ByteTokenizer

    gen = PackedCausalTransformerGenerator(
        PackedCausalTransformerGeneratorArgs(max_gen_len=4, max_tokens=64, dtype="fp32", device="cpu"), model,
        ByteTokenizer())
    texts, lls, greedy = gen.generate(["hello", "ab"])
    assert len(texts) == 2 and len(lls[0]) == 5 and len(lls[1]) == 2  # bos + chars, minus one
    # decode through the cache == recomputing the whole sequence
    ids = ByteTokenizer().encode("hello", add_bos=True)
    logits_full = model(torch.tensor([ids]))
    gen2 = PackedCausalTransformerGenerator(
        PackedCausalTransformerGeneratorArgs(max_gen_len=2, max_tokens=32, dtype="fp32", device="cpu"), model,
        ByteTokenizer())
    out = gen2.prefill(torch.tensor([ids[:-1]]), torch.tensor([len(ids) - 1]))
    nxt = gen2.generate_next_token(torch.tensor([[ids[-1]]]))
    gen2.release_cache()
    assert torch.allclose(out[0], logits_full[0, :-1], atol=1e-4)
    assert torch.allclose(nxt[0, 0], logits_full[0, -1], atol=1e-4)


def test_grad_accumulation_and_probe(tmp_path):
    cfg = _cfg(tmp_path / "p", steps=3, grad_acc_steps=2, probe_freq=1)
    train(dataclass_from_dict(TrainArgs, cfg))
    lines = [json.loads(l) for l in open(tmp_path / "p" / "probe" / "probe.0.jsonl")]
    assert lines and lines[0]["version"] == 2
    keys = set(lines[0]["data"])
    assert "layers.0.attention.wq::in" in keys and "layers.0.attention.wq::out.g" in keys
    assert "layers.0.attention_norm::resid" in keys
    assert any(k.endswith("::w.g") for k in keys)


def test_preemption_signal_saves_and_resume_continues_bitwise(tmp_path, monkeypatch):
    """SIGUSR2 (what the scheduler sends before it preempts a job, lingua/stool.py:57) in the middle of a run: the
    loop finishes the step, writes a checkpoint and exits; the same command then resumes, and the losses of the two
    halves are exactly those of an uninterrupted run (apps/main/train.py:203-209,582-592)."""
    import os
    import signal

    from lingua_b200 import train_loop

    train(dataclass_from_dict(TrainArgs, _cfg(tmp_path / "whole", steps=8)))
    whole = _losses(tmp_path / "whole")

    real_log = train_loop.MetricLogger.log
    seen = {"n": 0}

    def log_and_signal(self, metrics):
        real_log(self, metrics)
        seen["n"] += 1
        if seen["n"] == 3:
            os.kill(os.getpid(), signal.SIGUSR2)

    monkeypatch.setattr(train_loop.MetricLogger, "log", log_and_signal)
    monkeypatch.delenv("SLURM_JOB_ID", raising=False)
    train_loop.preemption_flag["flag"] = False
    d = tmp_path / "cut"
    with pytest.raises(SystemExit) as ex:
        train(dataclass_from_dict(TrainArgs, _cfg(d, steps=8)))
    assert ex.value.code == 0
    first = _losses(d)
    assert first == whole[:3]
    assert (d / "checkpoints" / "0000000003" / "train_state_00000.json").is_file()  # not a regular dump step
    monkeypatch.setattr(train_loop.MetricLogger, "log", real_log)
    train_loop.preemption_flag["flag"] = False
    (d / "metrics.jsonl").unlink()
    train(dataclass_from_dict(TrainArgs, _cfg(d, steps=8)))
    assert _losses(d) == whole[3:]


def test_damaged_last_checkpoint_falls_back_to_the_previous_one(tmp_path):
    d = tmp_path / "run"
    train(dataclass_from_dict(TrainArgs, _cfg(d, steps=10)))
    full = _losses(d)
    shard = next((d / "checkpoints" / "0000000010").glob("*.distcp"))
    data = shard.read_bytes()
    shard.write_bytes(data[: len(data) // 3])  # a save that was cut short
    (d / "metrics.jsonl").unlink()
    train(dataclass_from_dict(TrainArgs, _cfg(d, steps=10)))
    assert _losses(d) == full[5:]  # resumed from step 5, not from the damaged step 10
    # an explicitly requested folder that is damaged is an error, not a silent fallback
    from lingua_b200.checkpoint import CheckpointArgs, CheckpointManager

    mgr = CheckpointManager(CheckpointArgs(path=str(d / "checkpoints")))
    shard2 = next((d / "checkpoints" / "0000000005").glob("*.distcp"))
    shard2.write_bytes(shard2.read_bytes()[:100])
    with pytest.raises(BaseException):
        mgr.load(_FakeEngineNeverUsed(), None, path=d / "checkpoints" / "0000000005")


class _FakeEngineNeverUsed:
    """Loading must fail while reading the folder, before anything is written into an engine."""

    world = 1
    rank = 0
    groups = []
    step_count = 0
    tp_pg = None

    class optim:  # noqa: N801
        beta1 = beta2 = eps = weight_decay = 0.0
