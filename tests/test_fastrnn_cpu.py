"""minGRU / minLSTM / Hawk: gate math vs an explicit per-token loop, document isolation,
training, and prefill + sequential decoding through the state cache."""
import glob
from pathlib import Path

import pytest
import torch

from lingua_b200.config import dataclass_from_dict, load_yaml
from lingua_b200.generation_recurrent import PackedRNNGenerator, PackedRNNGeneratorArgs
from lingua_b200.models import fastrnn as R
from lingua_b200.tokenizer import ByteTokenizer

ROOT = Path(__file__).resolve().parent.parent


def _model(kind, **kw):
    cls, args_cls = R.MODEL_TYPES[kind]
    args = args_cls(dim=64, n_layers=2, n_heads=2, multiple_of=16, conv_size=4, vocab_size=258, **kw)
    torch.manual_seed(0)
    m = cls(args)
    m.init_weights()
    return m


def test_mingru_matches_explicit_recurrence():
    m = _model("minGRU")
    g = m.layers[0].gru
    x = torch.randn(1, 9, 64)
    out = g(x)
    z_pre = R.causal_conv1d(g.wz(x), g.conv_weight, None, act=True)
    z = torch.sigmoid(z_pre)[0]
    ht = g.wh_tilde(x)[0]
    h = torch.zeros(g.hidden_dim)
    rows = []
    for t in range(9):
        h = (1 - z[t]) * h + z[t] * ht[t]
        rows.append(h)
    ref = g.wo(torch.stack(rows) * torch.nn.functional.silu(g.w(x)[0]))
    assert torch.allclose(out[0], ref, atol=1e-5)


@pytest.mark.parametrize("kind", ["minGRU", "minLSTM", "hawk"])
def test_documents_do_not_leak_and_training_works(kind):
    m = _model(kind)
    tok = torch.randint(0, 258, (1, 24))
    ds = torch.zeros(1, 24, dtype=torch.int32)
    ds[:, 10:] = 10
    packed = m(tok, doc_start=ds)
    alone = m(tok[:, 10:])
    assert torch.allclose(packed[:, 10:], alone, atol=1e-4)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        loss = m(tok[:, :-1], tok[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("kind", ["minGRU", "minLSTM", "hawk"])
def test_cached_generation_matches_full_forward(kind):
    m = _model(kind).eval()
    tok = ByteTokenizer()
    gen = PackedRNNGenerator(PackedRNNGeneratorArgs(max_gen_len=3, max_tokens=128, dtype="fp32", device="cpu"), m, tok)
    prompts = ["hello there", "xy"]
    ids = [tok.encode(p, add_bos=True) for p in prompts]
    with torch.no_grad():
        full = [m(torch.tensor([i])) for i in ids]
        packed = torch.cat([torch.tensor(i[:-1]) for i in ids])
        lengths = torch.tensor([len(i) - 1 for i in ids])
        pre = gen.prefill(packed.unsqueeze(0), lengths)[0]
        nxt = gen.generate_next_token(torch.tensor([[i[-1] for i in ids]]))[0]
        gen.release_cache()
    off = 0
    for k, i in enumerate(ids):
        n = len(i) - 1
        assert torch.allclose(pre[off:off + n], full[k][0, :n], atol=1e-4)
        assert torch.allclose(nxt[k], full[k][0, n], atol=1e-4)
        off += n
    texts, lls, _ = gen.generate(prompts)
    assert len(texts) == 2 and len(lls[0]) == len(ids[0]) - 1


def test_hawk_block_diagonal_gates_and_shipped_configs():
    m = _model("hawk", gate_structure="block_diagonal")
    assert m.layers[0].rlgru_block.rglru.input_gate.weight.shape[0] == 2
    m(torch.randint(0, 258, (1, 8)), torch.randint(0, 258, (1, 8))).backward()
    from apps.fastRNN.train import TrainArgs, model_spec

    for path in sorted(glob.glob(str(ROOT / "apps" / "fastRNN" / "*" / "configs" / "*.yaml"))):
        cfg = dataclass_from_dict(TrainArgs, load_yaml(path))
        model_spec(cfg)
        assert cfg.model.dim > 0
