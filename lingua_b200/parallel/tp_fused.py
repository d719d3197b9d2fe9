"""Tensor parallelism with the collectives fused into the GEMM kernels (forward path).

The reference shards a block with DTensor plans (apps/main/transformer.py:165-221) and lets NCCL
run an all-gather / reduce-scatter (or all-reduce) around every sharded matmul. Here the residual
stream is sharded by rows (sequence parallel) and the two collectives live inside the tcgen05 GEMM
kernels of ``csrc/gemm_tp.cu``:

* ``ag_gemm``       reads every rank's normalised activations straight out of peer memory while
                    the tiles of the local rows are being multiplied (all-gather -> GEMM);
* ``gemm_scatter``  stores each output tile into the owner rank's staging buffer from the GEMM
                    epilogue (GEMM -> reduce-scatter), and ``reduce_norm`` sums the staged partials
                    together with the residual add and the RMSNorm that follow.

Ranks are ordered with ``peer_barrier`` (a bounded-wait kernel, no NCCL call on this path).
Peer-visible memory comes from ``torch.distributed._symmetric_memory``; only its allocator and
address exchange are used. ``LocalPeers`` emulates a group inside one process (every "rank" runs
on the same GPU, one after the other), which is how the kernels are tested on a single GPU.

``FusedTPForward`` runs a TP-sharded ``LMTransformer`` this way without autograd: evaluation,
scoring and prefill. Training keeps the all-reduce formulation of ``tensor_parallel.py``.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Generator, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import attention as A
from ..ops import functional as F
from ..ops.fused import _weights

ROW_TILE = 128
MAX_PEERS = 8


class TpGemmArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("world", C.c_int), ("rank", C.c_int),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("alpha", C.c_float),
        ("B", C.c_void_p), ("ldb", C.c_longlong),
        ("status", C.c_void_p),
        ("a_peers", C.c_void_p * MAX_PEERS),
        ("gather", C.c_void_p), ("flags", C.c_void_p), ("C", C.c_void_p), ("ldc", C.c_longlong),
        ("A", C.c_void_p), ("lda", C.c_longlong),
        ("c_peers", C.c_void_p * MAX_PEERS),
        ("slot_stride", C.c_longlong),
        ("b_major", C.c_int),
    ]


def _lib_tp():
    lib = _lib.load()
    if not getattr(lib, "_tp_declared", False):
        lib.lb_gemm_tp.argtypes = [C.POINTER(TpGemmArgs), C.c_void_p]
        lib.lb_gemm_tp.restype = C.c_int
        lib.lb_peer_barrier.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p]
        lib.lb_peer_barrier.restype = C.c_int
        lib.lb_peer_barrier_limit.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_uint32, C.c_void_p,
                                              C.c_ulonglong, C.c_void_p]
        lib.lb_peer_barrier_limit.restype = C.c_int
        lib.lb_reduce_norm.argtypes = [C.c_void_p, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p, C.c_float,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]
        lib.lb_reduce_norm.restype = C.c_int
        lib._tp_declared = True
    return lib


# ------------------------------------------------------------------ raw ops
def _b_layout(w: torch.Tensor):
    """(b_major, ldb) of a [N, K] weight operand: K contiguous, or - the transposed view of a [K, N] matrix -
    N contiguous, which the kernels read in place."""
    if w.stride(1) == 1:
        return 0, w.stride(0)
    assert w.stride(0) == 1, "weight operand needs a unit stride in one dim"
    return 1, w.stride(1)


def ag_gemm(a_ptrs: Sequence[int], rank: int, rows_per_rank: int, w: torch.Tensor,
            gather: Optional[torch.Tensor], flags: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
            alpha: float = 1.0) -> torch.Tensor:
    """``concat_r(A_r) @ w.T`` where ``A_r`` ([rows_per_rank, K] bf16, contiguous) lives at ``a_ptrs[r]``."""
    world = len(a_ptrs)
    N, K = w.shape
    M = rows_per_rank * world
    assert w.dtype == torch.bfloat16
    b_major, ldb = _b_layout(w)
    assert rows_per_rank % ROW_TILE == 0, "rows per rank must be a multiple of 128"
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=w.device)
    a = TpGemmArgs()
    a.mode, a.world, a.rank, a.M, a.N, a.K, a.alpha = 1, world, rank, M, N, K, alpha
    a.B, a.ldb, a.b_major, a.status = w.data_ptr(), ldb, b_major, _lib.status_word().data_ptr()
    for r in range(world):
        a.a_peers[r] = a_ptrs[r]
    if world > 1:
        assert gather is not None and gather.numel() >= M * K and gather.dtype == torch.bfloat16
        assert flags is not None and flags.numel() >= M // ROW_TILE + 1 and flags.dtype == torch.int32
        a.gather, a.flags = gather.data_ptr(), flags.data_ptr()
    a.C, a.ldc = out.data_ptr(), out.stride(0)
    _lib.check(_lib_tp().lb_gemm_tp(C.byref(a), _lib.stream_ptr()), "lb_gemm_tp(all-gather)")
    return out


def gemm_scatter(x: torch.Tensor, w: torch.Tensor, c_ptrs: Sequence[int], rank: int, slot_stride: int,
                 ldc: Optional[int] = None, alpha: float = 1.0) -> None:
    """Partial product ``x @ w.T`` ([M, N]); rows of owner ``o`` land in slot ``rank`` of ``c_ptrs[o]``."""
    world = len(c_ptrs)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1
    assert M % (ROW_TILE * world) == 0, "rows per rank must be a multiple of 128"
    b_major, ldb = _b_layout(w)
    a = TpGemmArgs()
    a.mode, a.world, a.rank, a.M, a.N, a.K, a.alpha = 2, world, rank, M, N, K, alpha
    a.B, a.ldb, a.b_major, a.status = w.data_ptr(), ldb, b_major, _lib.status_word().data_ptr()
    a.A, a.lda = x.data_ptr(), x.stride(0)
    for r in range(world):
        a.c_peers[r] = c_ptrs[r]
    a.slot_stride, a.ldc = slot_stride, (N if ldc is None else ldc)
    _lib.check(_lib_tp().lb_gemm_tp(C.byref(a), _lib.stream_ptr()), "lb_gemm_tp(scatter)")


def reduce_norm_ref(slots, resid, w, eps):
    h = slots.float().sum(0)
    if resid is not None:
        h = h + resid.float()
    h = h.to(slots.dtype)
    if w is None:
        return h, None, None
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    return h, (hf * rstd * w.float()).to(slots.dtype), rstd.squeeze(-1)


def reduce_norm(slots: torch.Tensor, resid: Optional[torch.Tensor], w: Optional[torch.Tensor], eps: float,
                h_out: Optional[torch.Tensor] = None, y_out: Optional[torch.Tensor] = None):
    """slots [n, rows, D] -> (h, y): h = resid + slots.sum(0) (bf16), y = rmsnorm(h) * w (None without w)."""
    if not slots.is_cuda:
        h, y, _ = reduce_norm_ref(slots, resid, w, eps)
        return h, y
    n, rows, D = slots.shape
    assert slots.dtype == torch.bfloat16 and slots.stride(2) == 1 and slots.stride(1) == D
    if h_out is None:
        h_out = torch.empty(rows, D, dtype=slots.dtype, device=slots.device)
    if w is not None and y_out is None:
        y_out = torch.empty(rows, D, dtype=slots.dtype, device=slots.device)
    rc = _lib_tp().lb_reduce_norm(slots.data_ptr(), n, slots.stride(0), None if resid is None else resid.data_ptr(),
                                  None if w is None else w.data_ptr(), eps, h_out.data_ptr(),
                                  None if w is None else y_out.data_ptr(), None, rows, D, _lib.stream_ptr())
    _lib.check(rc, "lb_reduce_norm")
    return h_out, (y_out if w is not None else None)


def peer_barrier(pad_ptrs: Sequence[int], rank: int, epoch: int, limit_s: float = 2.0) -> None:
    """All ranks meet; ``limit_s`` bounds the wait (on expiry the status word is set and the kernel returns)."""
    arr = (C.c_void_p * len(pad_ptrs))(*pad_ptrs)
    rc = _lib_tp().lb_peer_barrier_limit(arr, len(pad_ptrs), rank, epoch & 0xFFFFFFFF, _lib.status_word().data_ptr(),
                                         int(limit_s * 1e9), _lib.stream_ptr())
    _lib.check(rc, "lb_peer_barrier")


# ------------------------------------------------------------------ peer-visible memory
class SymmetricPeers:
    """Buffers of a process group that every member GPU can address (NVLink peer memory)."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device):
        import torch.distributed._symmetric_memory as sm

        self._sm = sm
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= MAX_PEERS
        self._bufs: Dict[str, torch.Tensor] = {}
        self._ptrs: Dict[str, List[int]] = {}
        self._peer_views: Dict[str, List[torch.Tensor]] = {}
        self._epoch = 0
        self.alloc("__pad", (MAX_PEERS,), torch.int32).zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def alloc(self, name: str, shape, dtype) -> torch.Tensor:
        if name not in self._bufs:
            t = self._sm.empty(*shape, dtype=dtype, device=self.device)
            hdl = self._sm.rendezvous(t, group=self.group)
            self._bufs[name] = t
            self._ptrs[name] = [int(p) for p in hdl.buffer_ptrs]
            self._peer_views[name] = [hdl.get_buffer(r, tuple(shape), dtype) for r in range(self.world)]
        t = self._bufs[name]
        assert tuple(t.shape) == tuple(shape) and t.dtype == dtype, f"buffer {name} re-allocated with another shape"
        return t

    def ptrs(self, name: str) -> List[int]:
        return self._ptrs[name]

    def local(self, name: str) -> torch.Tensor:
        return self._bufs[name]

    def peer(self, name: str, rank: int) -> torch.Tensor:
        """Rank ``rank``'s buffer as a tensor of this device (peer mapping): for copies, never as a kernel operand
        of a library product."""
        return self._peer_views[name][rank]

    def barrier(self) -> None:
        self._epoch += 1
        peer_barrier(self._ptrs["__pad"], self.rank, self._epoch)


class LocalPeers:
    """``world`` emulated ranks in one process on one GPU. Kernels of different "ranks" never wait on each
    other here: the caller runs them phase by phase on one stream, which orders them."""

    def __init__(self, world: int, device):
        self.world = world
        self.device = torch.device(device)
        self._bufs: Dict[str, List[torch.Tensor]] = {}

    def view(self, rank: int) -> "_LocalRank":
        return _LocalRank(self, rank)


class _LocalRank:
    def __init__(self, parent: LocalPeers, rank: int):
        self.parent, self.rank, self.world, self.device = parent, rank, parent.world, parent.device

    def alloc(self, name, shape, dtype):
        if name not in self.parent._bufs:
            self.parent._bufs[name] = [torch.zeros(*shape, dtype=dtype, device=self.device) for _ in range(self.world)]
        return self.parent._bufs[name][self.rank]

    def ptrs(self, name):
        return [t.data_ptr() for t in self.parent._bufs[name]]

    def local(self, name):
        return self.parent._bufs[name][self.rank]

    def barrier(self):  # stream order stands in for the barrier
        pass


# ------------------------------------------------------------------ fused forward of a TP-sharded model
class FusedTPForward:
    """Forward pass (no autograd) of a tensor-parallel ``LMTransformer`` with fused collectives.

    ``model`` holds this rank's shards (``tp_parallelize`` already applied; norms, embedding and head
    replicated). Tokens [B, S] are the same on every rank; every rank owns ``B*S / world`` consecutive rows
    of the residual stream. ``loss(tokens, targets)`` returns the mean cross-entropy over all rows.
    """

    def __init__(self, model, peers):
        self.model = model
        self.peers = peers
        self.world, self.rank = peers.world, peers.rank
        self._w: Dict[int, torch.Tensor] = {}

    def _cat(self, key, ws):
        # weights of one fused projection as a single [N, K] matrix (a view when they are adjacent)
        if key not in self._w:
            v = _weights(ws)
            if v.data_ptr() != ws[0].data_ptr():
                return v  # a copy: it would go stale after the next optimiser step, so it is not kept
            self._w[key] = v
        return self._w[key]

    def steps(self, tokens: torch.Tensor, targets: Optional[torch.Tensor], out: dict) -> Generator[None, None, None]:
        """The forward pass as a generator that yields wherever all ranks have to meet."""
        m, P, W, R = self.model, self.peers, self.world, self.rank
        B, S = tokens.shape
        T = B * S
        assert T % (ROW_TILE * W) == 0, f"tokens per step ({T}) must be a multiple of {ROW_TILE * W}"
        Tl = T // W
        D = m.dim
        rows = slice(R * Tl, (R + 1) * Tl)
        dev = tokens.device
        l0 = m.layers[0]
        at0, ff0 = l0.attention, l0.feed_forward
        n_qkv = (at0.n_heads + 2 * at0.n_kv_heads) * at0.head_dim
        n_ff = sum(w.shape[0] for w in ff0.in_weights())
        y_a = P.alloc("y_attn", (Tl, D), torch.bfloat16)
        y_f = P.alloc("y_ffn", (Tl, D), torch.bfloat16)
        stage_a = P.alloc("stage_attn", (W, Tl, D), torch.bfloat16)
        stage_f = P.alloc("stage_ffn", (W, Tl, D), torch.bfloat16)
        gather = torch.empty(T, D, dtype=torch.bfloat16, device=dev) if W > 1 else None
        flags = torch.zeros(T // ROW_TILE + 1, dtype=torch.int32, device=dev) if W > 1 else None
        qkv = torch.empty(T, n_qkv, dtype=torch.bfloat16, device=dev)
        u = torch.empty(T, n_ff, dtype=torch.bfloat16, device=dev)
        cs = m.rope_embeddings.freqs_cis[:S]
        window = m.sliding_window or 0

        x = F.embed_fwd(tokens.reshape(-1)[rows], m.tok_embeddings.weight)
        h, _ = reduce_norm(x.unsqueeze(0), None, l0.attention_norm.weight, l0.attention_norm.eps, y_out=y_a)
        for li, layer in enumerate(m.layers):
            at, ff = layer.attention, layer.feed_forward
            yield  # y_attn written everywhere
            ag_gemm(P.ptrs("y_attn"), R, Tl, self._cat((li, "qkv"), at.qkv_weights()), gather, flags, out=qkv)
            F.rope_(qkv, cs, at.n_heads + at.n_kv_heads, at.head_dim, S)
            t = qkv.view(B, S, at.n_heads + 2 * at.n_kv_heads, at.head_dim)
            o, _ = A.flash_fwd(t[:, :, :at.n_heads], t[:, :, at.n_heads:at.n_heads + at.n_kv_heads],
                               t[:, :, at.n_heads + at.n_kv_heads:], causal=True, window=window)
            gemm_scatter(o.view(T, -1), at.wo.weight, P.ptrs("stage_attn"), R, Tl * D)
            yield  # every rank's partials have landed in stage_attn
            h, _ = reduce_norm(stage_a, h, layer.ffn_norm.weight, layer.ffn_norm.eps, h_out=h, y_out=y_f)
            yield  # y_ffn written everywhere
            ag_gemm(P.ptrs("y_ffn"), R, Tl, self._cat((li, "ffn"), ff.in_weights()), gather, flags, out=u)
            a = F.glu_fwd(u, F.ACT_SILU) if ff.activation == "swiglu" else F.act_fwd(u, F.ACT_RELU2)
            gemm_scatter(a, ff.w2.weight, P.ptrs("stage_ffn"), R, Tl * D)
            yield  # partials in stage_ffn
            nxt = m.layers[li + 1].attention_norm if li + 1 < len(m.layers) else m.norm
            h, _ = reduce_norm(stage_f, h, nxt.weight, nxt.eps, h_out=h, y_out=y_a)
        # y_attn now holds norm(h) of the final norm for the local rows
        from ..ops.gemm import gemm

        logits = gemm(y_a, m.output.weight, out_dtype=torch.float32)
        out["logits"] = logits
        if targets is not None:
            loss_rows, _ = F.ce_fwd(logits, targets.reshape(-1)[rows].contiguous())
            out["loss_sum"] = loss_rows.sum()
            out["count"] = (targets.reshape(-1)[rows] >= 0).sum()
        yield  # nobody reuses a shared buffer before everyone is done with it

    @torch.no_grad()
    def forward(self, tokens, targets=None) -> dict:
        out: dict = {}
        for _ in self.steps(tokens, targets, out):
            self.peers.barrier()
        return out

    def accepts(self, B: int, S: int) -> bool:
        """Row tiles of 128 tokens must not straddle ranks."""
        return (B * S) % (ROW_TILE * self.world) == 0

    @torch.no_grad()
    def __call__(self, tokens, targets=None) -> torch.Tensor:
        """Same contract as ``LMTransformer.forward``: mean loss with targets, else logits [B, S, vocab]."""
        if targets is not None:
            return self.loss(tokens, targets)
        local = self.forward(tokens)["logits"]
        if self.world == 1 or not isinstance(self.peers, SymmetricPeers):
            return local.view(*tokens.shape, -1)
        full = torch.empty(local.shape[0] * self.world, local.shape[1], dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(full, local.contiguous(), group=self.peers.group)
        return full.view(*tokens.shape, -1)

    @torch.no_grad()
    def loss(self, tokens, targets) -> torch.Tensor:
        out = self.forward(tokens, targets)
        tot = torch.stack([out["loss_sum"].float(), out["count"].float()])
        if isinstance(self.peers, SymmetricPeers) and self.world > 1:
            dist.all_reduce(tot, group=self.peers.group)
        return tot[0] / tot[1].clamp(min=1)


@torch.no_grad()
def run_local_group(runners: Sequence[FusedTPForward], tokens, targets=None) -> List[dict]:
    """Drive emulated ranks (``LocalPeers``) in lock-step: each runs up to its next meeting point in turn."""
    outs = [dict() for _ in runners]
    gens = [r.steps(tokens, targets, o) for r, o in zip(runners, outs)]
    alive = True
    while alive:
        for g in gens:
            try:
                next(g)
            except StopIteration:
                alive = False
    return outs


def enable_fused_tp_forward(model, group: dist.ProcessGroup, device: torch.device) -> bool:
    """Route no-grad forward passes of a TP-sharded model through ``FusedTPForward``.

    Returns False (and leaves the NCCL all-reduce path in place) when peer-visible memory cannot be
    set up for ``group``, e.g. ranks on different nodes."""
    import logging

    try:
        peers = SymmetricPeers(group, device)
    except Exception as e:  # no NVLink peer access between the ranks of this group
        logging.getLogger(__name__).warning("fused tensor-parallel forward disabled: %s", e)
        return False
    object.__setattr__(model, "tp_fused", FusedTPForward(model, peers))
    return True
