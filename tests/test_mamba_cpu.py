"""Mamba-2: chunked SSD vs the token-by-token recurrence (incl. documents, ragged length, gradients),
the decode update, model training and cached generation."""
import glob
from pathlib import Path

import pytest
import torch

from lingua_b200.config import dataclass_from_dict, load_yaml
from lingua_b200.generation_recurrent import PackedRNNGenerator, PackedRNNGeneratorArgs
from lingua_b200.models.mamba import LMMamba, LMMambaArgs
from lingua_b200.ops import ssd
from lingua_b200.tokenizer import ByteTokenizer

ROOT = Path(__file__).resolve().parent.parent


def _inputs(b=2, s=50, h=4, p=8, g=2, n=16, seed=0):
    torch.manual_seed(seed)
    x = torch.randn(b, s, h, p)
    dt = torch.rand(b, s, h) * 0.5 + 0.01
    A = -torch.rand(h) * 2 - 0.1
    B, C = torch.randn(b, s, g, n) * 0.3, torch.randn(b, s, g, n) * 0.3
    D = torch.randn(h)
    return x, dt, A, B, C, D


@pytest.mark.parametrize("chunk", [8, 16, 64])
@pytest.mark.parametrize("docs", [False, True])
def test_chunked_ssd_matches_recurrence(chunk, docs):
    x, dt, A, B, C, D = _inputs()
    ds = None
    if docs:
        ds = torch.zeros(2, 50, dtype=torch.int32)
        ds[0, 13:] = 13
        ds[0, 40:] = 40
        ds[1, 7:] = 7
    y, st = ssd.ssd_chunked(x, dt, A, B, C, D, chunk, ds)
    yr, str_ = ssd.ssd_ref(x, dt, A, B, C, D, ds)
    assert torch.allclose(y, yr, atol=2e-4), (y - yr).abs().max()
    assert torch.allclose(st, str_.float(), atol=2e-4)


def test_ssd_gradients_and_decode_step():
    x, dt, A, B, C, D = _inputs(b=1, s=20, seed=1)
    leaves = [t.clone().requires_grad_(True) for t in (x, dt, A, B, C, D)]
    y, _ = ssd.ssd_chunked(*leaves, chunk=8)
    g = torch.randn_like(y)
    grads = torch.autograd.grad(y, leaves, g)
    leaves_r = [t.clone().double().requires_grad_(True) for t in (x, dt, A, B, C, D)]
    yr, _ = ssd.ssd_ref(*leaves_r)
    grads_r = torch.autograd.grad(yr, leaves_r, g.double())
    for a, b in zip(grads, grads_r):
        assert torch.allclose(a, b.float(), atol=2e-3, rtol=1e-3)
    # one decode step continues the scan
    y_full, st_full = ssd.ssd_ref(x, dt, A, B, C, D)
    _, st = ssd.ssd_chunked(x[:, :-1], dt[:, :-1], A, B[:, :-1], C[:, :-1], D, 8)
    y_last = ssd.selective_state_update(st, x[:, -1], dt[:, -1], A, B[:, -1], C[:, -1], D)
    assert torch.allclose(y_last, y_full[:, -1], atol=2e-4) and torch.allclose(st, st_full.float(), atol=2e-4)


def _model():
    torch.manual_seed(0)
    args = LMMambaArgs(dim=64, n_layers=2, n_heads=4, state_dim=16, n_groups=1, conv_size=4, multiple_of=16,
                       ssm_chunk_size=8, vocab_size=258)
    m = LMMamba(args)
    m.init_weights()
    return m


def test_mamba_trains_and_isolates_documents():
    m = _model()
    tok = torch.randint(0, 258, (1, 24))
    ds = torch.zeros(1, 24, dtype=torch.int32)
    ds[:, 9:] = 9
    assert torch.allclose(m(tok, doc_start=ds)[:, 9:], m(tok[:, 9:]), atol=1e-4)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        loss = m(tok[:, :-1], tok[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]


def test_mamba_cached_generation_matches_full_forward():
    m = _model().eval()
    tok = ByteTokenizer()
    gen = PackedRNNGenerator(PackedRNNGeneratorArgs(max_gen_len=3, max_tokens=128, dtype="fp32", device="cpu"), m, tok)
    ids = [tok.encode(p, add_bos=True) for p in ("hello there", "xyz")]
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


def test_shipped_mamba_configs_load():
    from apps.mamba.train import TrainArgs
    from lingua_b200.evaluation import EvalArgs

    for path in sorted(glob.glob(str(ROOT / "apps" / "mamba" / "configs" / "*.yaml"))):
        cls = EvalArgs if path.endswith("eval.yaml") else TrainArgs
        dataclass_from_dict(cls, load_yaml(path))
