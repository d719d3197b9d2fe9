"""One rank of the multi-GPU check of the fused tensor-parallel kernels (started by torchrun from
test_tp_fused_multigpu.py, or by hand with ``--bench`` to time them against NCCL + plain GEMM).

Every comparison is against NCCL collectives around this library's ordinary GEMM on the same data.
"""
import argparse
import copy
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs  # noqa: E402
from lingua_b200.ops import _lib  # noqa: E402
from lingua_b200.ops.gemm import gemm  # noqa: E402
from lingua_b200.parallel import tp_fused as T  # noqa: E402
from lingua_b200.parallel.tensor_parallel import tp_parallelize  # noqa: E402

bf = torch.bfloat16


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


class Mesh:
    def __init__(self, group):
        self.g = group

    def size(self, name):
        return dist.get_world_size(self.g)

    def local_rank(self, name):
        return dist.get_rank(self.g)

    def group(self, name):
        return self.g


def timed(fn, iters, flush):
    """Device time per call in ms, max over ranks."""
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor(sorted(ts)[len(ts) // 2], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def check_ops(P, W, R):
    rows, K, N = 256, 1024, 768
    torch.manual_seed(10 + R)
    slab = P.alloc("t_a", (rows, K), bf)
    slab.copy_(torch.randn(rows, K, device="cuda", dtype=bf))
    torch.manual_seed(5)
    w = torch.randn(N, K, device="cuda", dtype=bf)
    gather = torch.zeros(W * rows, K, device="cuda", dtype=bf)
    flags = torch.zeros(W * rows // 128 + 1, device="cuda", dtype=torch.int32)
    P.barrier()
    out = T.ag_gemm(P.ptrs("t_a"), R, rows, w, gather, flags)
    full = torch.empty(W * rows, K, device="cuda", dtype=bf)
    dist.all_gather_into_tensor(full, slab)
    ref = gemm(full, w)
    P.barrier()
    torch.cuda.synchronize()
    _lib.check_status()
    assert rel(out, ref) < 1e-3, f"ag_gemm rank {R}: {rel(out, ref)}"

    M = W * rows
    torch.manual_seed(20 + R)
    x = torch.randn(M, K, device="cuda", dtype=bf)
    wr = torch.randn(N, K, device="cuda", dtype=bf) * 0.05
    resid = torch.randn(rows, N, device="cuda", dtype=bf)
    g = torch.rand(N, device="cuda", dtype=bf) + 0.5
    stage = P.alloc("t_stage", (W, rows, N), bf)
    P.barrier()
    T.gemm_scatter(x, wr, P.ptrs("t_stage"), R, rows * N)
    P.barrier()
    h, y = T.reduce_norm(stage, resid, g, 1e-5)
    part = gemm(x, wr, out_dtype=torch.float32)
    mine = torch.empty(rows, N, device="cuda")
    dist.reduce_scatter_tensor(mine, part)
    h_ref = (mine + resid.float()).to(bf)
    P.barrier()
    torch.cuda.synchronize()
    _lib.check_status()
    assert rel(h, h_ref) < 2e-2, f"gemm_scatter rank {R}: {rel(h, h_ref)}"


def check_model(P, W, R):
    args = LMTransformerArgs(dim=1024, n_layers=2, n_heads=8, n_kv_heads=8, vocab_size=2048, max_seqlen=512)
    torch.manual_seed(3)
    full = LMTransformer(args)
    full.init_weights()
    full = full.cuda()
    for p in full.parameters():
        p.data = p.data.to(bf)
    shard = copy.deepcopy(full)
    tp_parallelize(shard, Mesh(dist.group.WORLD), args, None)
    tok = torch.randint(0, 2048, (2, 513), device="cuda")
    dist.broadcast(tok, 0)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    with torch.no_grad():
        loss_nccl = shard(x, y)  # all-reduce formulation
        loss_one = full(x, y)
    fused = T.FusedTPForward(shard, P)
    loss_fused = fused.loss(x, y)
    torch.cuda.synchronize()
    _lib.check_status()
    for name, ref in (("nccl tp", loss_nccl), ("single gpu", loss_one)):
        assert abs(loss_fused.item() - ref.item()) < 1e-2 * abs(ref.item()), (name, loss_fused.item(), ref.item())


def bench(P, W, R, out_path):
    """Llama-7B block shapes, 8192 tokens per step: fused kernels vs NCCL collective + plain GEMM."""
    T_tok, D, Fh = 8192, 4096, 11008
    Tl = T_tok // W
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    res = {"world": W, "tokens": T_tok}
    y = P.alloc("b_y", (Tl, D), bf)
    y.normal_()
    gather = torch.empty(T_tok, D, device="cuda", dtype=bf)
    flags = torch.zeros(T_tok // 128 + 1, device="cuda", dtype=torch.int32)
    full = torch.empty(T_tok, D, device="cuda", dtype=bf)
    for name, N in (("qkv", 3 * D // W), ("w13", 2 * (Fh // W // 8 * 8))):
        w = torch.randn(N, D, device="cuda", dtype=bf) * 0.02
        out = torch.empty(T_tok, N, device="cuda", dtype=bf)

        def fused():
            P.barrier()
            T.ag_gemm(P.ptrs("b_y"), R, Tl, w, gather, flags, out=out)

        def unfused():
            dist.all_gather_into_tensor(full, y)
            gemm(full, w, out=out)

        def math_only():
            gemm(full, w, out=out)

        res[f"ag_gemm_{name}"] = {"fused_ms": timed(fused, 10, flush), "nccl_ms": timed(unfused, 10, flush),
                                  "gemm_only_ms": timed(math_only, 10, flush), "N": N, "K": D,
                                  "nvlink_bytes_in": (W - 1) * Tl * D * 2}
    stage = P.alloc("b_stage", (W, Tl, D), bf)
    resid = torch.randn(Tl, D, device="cuda", dtype=bf)
    g = torch.ones(D, device="cuda", dtype=bf)
    h, yo = torch.empty(Tl, D, device="cuda", dtype=bf), torch.empty(Tl, D, device="cuda", dtype=bf)
    for name, K in (("wo", D // W), ("w2", Fh // W // 64 * 64)):
        x = torch.randn(T_tok, K, device="cuda", dtype=bf)
        w = torch.randn(D, K, device="cuda", dtype=bf) * 0.02
        part = torch.empty(T_tok, D, device="cuda", dtype=bf)
        mine = torch.empty(Tl, D, device="cuda", dtype=bf)

        def fused():
            T.gemm_scatter(x, w, P.ptrs("b_stage"), R, Tl * D)
            P.barrier()
            T.reduce_norm(stage, resid, g, 1e-5, h_out=h, y_out=yo)
            P.barrier()

        def unfused():
            gemm(x, w, out=part)
            dist.reduce_scatter_tensor(mine, part)
            T.reduce_norm(mine.unsqueeze(0), resid, g, 1e-5, h_out=h, y_out=yo)

        def math_only():
            gemm(x, w, out=part)

        res[f"gemm_rs_{name}"] = {"fused_ms": timed(fused, 10, flush), "nccl_ms": timed(unfused, 10, flush),
                                  "gemm_only_ms": timed(math_only, 10, flush), "N": D, "K": K,
                                  "nvlink_bytes_out": (W - 1) * Tl * D * 2}
    _lib.check_status()
    if R == 0:
        print(json.dumps(res))
        if out_path:
            Path(out_path).parent.mkdir(parents=True, exist_ok=True)
            Path(out_path).write_text(json.dumps(res, indent=1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    W = dist.get_world_size()
    P = T.SymmetricPeers(dist.group.WORLD, torch.device("cuda", torch.cuda.current_device()))
    check_ops(P, W, rank)
    check_model(P, W, rank)
    if a.bench:
        bench(P, W, rank, a.out)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("TP_FUSED_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
