"""Fused tensor-parallel kernels on one GPU: the ranks of a group are emulated one after the other
(``LocalPeers``), so every data path of the kernels runs, only the NVLink hop is a local copy."""
import copy

import pytest
import torch

from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs
from lingua_b200.ops import _lib
from lingua_b200.parallel import tp_fused as T
from lingua_b200.parallel.tensor_parallel import tp_parallelize

pytestmark = pytest.mark.gpu
bf = torch.bfloat16


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


@pytest.mark.parametrize("world,rows,K,N", [(1, 256, 256, 512), (2, 128, 512, 768), (4, 256, 1024, 264), (8, 128, 64, 256)])
def test_all_gather_gemm(world, rows, K, N):
    torch.manual_seed(0)
    slabs = [torch.randn(rows, K, device="cuda", dtype=bf) for _ in range(world)]
    w = torch.randn(N, K, device="cuda", dtype=bf)
    ref = torch.cat(slabs).float() @ w.float().t()
    for rank in range(world):
        gather = torch.zeros(world * rows, K, device="cuda", dtype=bf)
        flags = torch.zeros(world * rows // 128 + 1, device="cuda", dtype=torch.int32)
        out = T.ag_gemm([s.data_ptr() for s in slabs], rank, rows, w, gather, flags)
        torch.cuda.synchronize()
        _lib.check_status()
        assert _rel(out, ref) < 1e-2, f"rank {rank}"
        if world > 1:
            # every remote slab arrived whole, and nothing wrote into the slot of the own rows
            for r in range(world):
                got = gather[r * rows:(r + 1) * rows]
                assert torch.equal(got, slabs[r]) if r != rank else not got.any()


@pytest.mark.parametrize("world,rows,K,N", [(1, 256, 256, 512), (2, 128, 512, 320), (4, 128, 256, 1024)])
def test_gemm_scatter_then_reduce_norm(world, rows, K, N):
    torch.manual_seed(1)
    M = world * rows
    xs = [torch.randn(M, K, device="cuda", dtype=bf) for _ in range(world)]
    ws = [torch.randn(N, K, device="cuda", dtype=bf) * 0.1 for _ in range(world)]
    resid = [torch.randn(rows, N, device="cuda", dtype=bf) for _ in range(world)]
    g = torch.rand(N, device="cuda", dtype=bf) + 0.5
    stages = [torch.zeros(world, rows, N, device="cuda", dtype=bf) for _ in range(world)]
    for rank in range(world):
        T.gemm_scatter(xs[rank], ws[rank], [s.data_ptr() for s in stages], rank, rows * N)
    torch.cuda.synchronize()
    _lib.check_status()
    partial = [x.float() @ w.float().t() for x, w in zip(xs, ws)]
    for o in range(world):
        for r in range(world):
            assert _rel(stages[o][r], partial[r][o * rows:(o + 1) * rows]) < 1e-2, f"slot {r} of owner {o}"
        h, y = T.reduce_norm(stages[o], resid[o], g, 1e-5)
        h_ref, y_ref, _ = T.reduce_norm_ref(stages[o], resid[o], g, 1e-5)
        assert _rel(h, h_ref) < 1e-2 and _rel(y, y_ref) < 2e-2
        h2, none = T.reduce_norm(stages[o], None, None, 1e-5)
        assert none is None and _rel(h2, stages[o].float().sum(0)) < 1e-2


class _Mesh:
    def __init__(self, tp, rank):
        self.tp, self.rank = tp, rank

    def size(self, name):
        return self.tp

    def local_rank(self, name):
        return self.rank

    def group(self, name):
        return None


@pytest.mark.parametrize("world,act,kvh", [(2, "swiglu", 4), (4, "swiglu", 4), (2, "relu2", 2)])
def test_fused_tp_forward_matches_single_gpu_model(world, act, kvh):
    args = LMTransformerArgs(dim=512, n_layers=2, n_heads=4, n_kv_heads=kvh, vocab_size=1024, max_seqlen=256,
                             ffn_activation=act)
    torch.manual_seed(2)
    full = LMTransformer(args)
    full.init_weights()
    full = full.cuda()
    for p in full.parameters():
        p.data = p.data.to(bf)
    tok = torch.randint(0, 1024, (4, 257), device="cuda")
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    y[1, 7] = -100
    with torch.no_grad():
        loss_ref = full(x, y)
        logits_ref = full(x).float().view(-1, 1024)
    peers = T.LocalPeers(world, "cuda")
    runners = []
    for rank in range(world):
        shard = copy.deepcopy(full)
        tp_parallelize(shard, _Mesh(world, rank), args, None)
        runners.append(T.FusedTPForward(shard, peers.view(rank)))
    outs = T.run_local_group(runners, x, y)
    torch.cuda.synchronize()
    _lib.check_status()
    logits = torch.cat([o["logits"] for o in outs])
    assert _rel(logits, logits_ref) < 3e-2
    loss = sum(o["loss_sum"] for o in outs) / sum(o["count"] for o in outs)
    assert abs(loss.item() - loss_ref.item()) < 1e-2 * abs(loss_ref.item())
