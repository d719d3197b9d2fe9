"""Native (bf16 CUDA) minGRU / minLSTM / Hawk / Mamba-2 vs their fp32 PyTorch reference path."""
import copy

import pytest
import torch

from lingua_b200.models import fastrnn as R
from lingua_b200.models.mamba import LMMamba, LMMambaArgs

pytestmark = pytest.mark.gpu


def _compare(ref, tok, tgt, ds, tol=4e-2):
    nat = copy.deepcopy(ref).cuda().bfloat16()
    for pr, pn in zip(ref.parameters(), nat.parameters()):
        pr.data.copy_(pn.data.float().cpu())
    loss_r = ref(tok, tgt, doc_start=ds)
    loss_r.backward()
    loss_n = nat(tok.cuda(), tgt.cuda(), doc_start=ds.cuda())
    loss_n.backward()
    assert abs(loss_n.item() - loss_r.item()) < tol * abs(loss_r.item()), (loss_n.item(), loss_r.item())
    bad = []
    for (n, pr), (_, pn) in zip(ref.named_parameters(), nat.named_parameters()):
        g_r, g_n = pr.grad.float(), pn.grad.float().cpu()
        err = (g_r - g_n).abs().max().item() / (g_r.abs().max().item() + 1e-8)
        if err > 0.1:
            bad.append((n, err))
    assert not bad, bad


@pytest.mark.parametrize("kind", ["minGRU", "minLSTM", "hawk"])
def test_fastrnn_native_matches_reference(kind):
    cls, args_cls = R.MODEL_TYPES[kind]
    torch.manual_seed(0)
    ref = cls(args_cls(dim=256, n_layers=2, n_heads=4, multiple_of=64, conv_size=4, vocab_size=512))
    ref.init_weights()
    tok = torch.randint(0, 512, (2, 160))
    tgt = torch.randint(0, 512, (2, 160))
    ds = torch.zeros(2, 160, dtype=torch.int32)
    ds[:, 70:] = 70
    _compare(ref, tok, tgt, ds)


def test_mamba_native_matches_reference():
    torch.manual_seed(0)
    ref = LMMamba(LMMambaArgs(dim=256, n_layers=2, n_heads=8, state_dim=64, conv_size=4, multiple_of=64,
                              ssm_chunk_size=64, vocab_size=512))
    ref.init_weights()
    tok = torch.randint(0, 512, (2, 192))
    tgt = torch.randint(0, 512, (2, 192))
    ds = torch.zeros(2, 192, dtype=torch.int32)
    ds[:, 100:] = 100
    _compare(ref, tok, tgt, ds)
