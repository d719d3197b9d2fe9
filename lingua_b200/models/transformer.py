"""Llama-style decoder: core blocks and the language-model wrapper.

Parameter names, shapes, initialisation and the config dataclasses follow
lingua/transformer.py (BaseTransformerArgs :30, Attention :306, FeedForward :431,
TransformerBlock :496, BaseTransformer :553) and apps/main/transformer.py (LMTransformerArgs
:64, LMTransformer :74, FLOP estimator :46-56), so checkpoints and YAML configs are
interchangeable. Every module has two execution paths over the same parameters:

* native: bf16 CUDA parameters -> the fused sm_100a ops of ``lingua_b200.ops.fused`` on a
  flattened [tokens, dim] activation layout (QKV and w1|w3 run as one GEMM each when their
  weights are adjacent in the flat parameter buffer, which the sharded engine guarantees);
* reference: plain PyTorch in the parameters' dtype (CPU, fp32 oracles, gloo plumbing tests).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..ops import fused
from ..ops.attention import attention_ref
from ..parallel.tensor_parallel import ReduceBwd, ReduceFwd


class InitStdFactor(Enum):
    DISABLED = "disabled"  # std / 1
    GLOBAL_DEPTH = "global_depth"  # std / sqrt(2 * (n_layers + 1))
    CURRENT_DEPTH = "current_depth"  # std / sqrt(2 * (depth + 1))
    DIM_RATIO = "dim_ratio"  # std / (dim / 4096)


@dataclass
class BaseTransformerArgs:
    dim: int = 512
    n_layers: int = 8
    head_dim: Optional[int] = None
    n_heads: Optional[int] = None
    n_kv_heads: Optional[int] = None
    ffn_dim_multiplier: Optional[float] = None
    multiple_of: int = 256
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    init_base_std: Optional[float] = None
    init_std_factor: str = "disabled"
    max_seqlen: int = 1024
    # Extension: "swiglu" (silu(w1 x) * w3 x) or "relu2" (relu(w1 x)^2, no w3).
    ffn_activation: str = "swiglu"


@dataclass
class LMTransformerArgs(BaseTransformerArgs):
    seed: int = 42
    vocab_size: int = -1
    weight_tying: bool = False
    sliding_window: Optional[int] = None
    # Extension: rows of logits held at once by the fused linear + cross-entropy.
    loss_chunk: int = 2048


def cross_entropy(pred: torch.Tensor, target: torch.Tensor, **kw) -> torch.Tensor:
    return TF.nll_loss(TF.log_softmax(pred.flatten(end_dim=-2).float(), -1), target.flatten(end_dim=-1), **kw)


def _is_native(w: torch.Tensor) -> bool:
    return w.is_cuda and w.dtype == torch.bfloat16


def _trunc(w: torch.Tensor, std: float, bound_std: Optional[float] = None) -> None:
    b = 3 * (bound_std if bound_std is not None else std)
    nn.init.trunc_normal_(w, mean=0.0, std=std, a=-b, b=b)


def _init_linear(mod: nn.Module, std: float, bound_std: Optional[float] = None) -> None:
    """Truncated-normal init of ``mod.weight``. A tensor-parallel slice (``mod.tp_shard = (dim, tp,
    rank)``) takes its part of a full-size draw, so that the assembled weight does not depend on
    the TP degree and replicas of the random stream stay in step on every rank."""
    shard = getattr(mod, "tp_shard", None)
    w = mod.weight
    if shard is None:
        _trunc(w, std, bound_std)
        return
    dim, tp, rank = shard
    shape = list(w.shape)
    shape[dim] *= tp
    full = torch.empty(shape, dtype=w.dtype, device=w.device)
    _trunc(full, std, bound_std)
    with torch.no_grad():
        w.copy_(full.chunk(tp, dim=dim)[rank])


class Linear(nn.Module):
    """Bias-free linear layer; ``weight`` is [out_features, in_features]."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _is_native(self.weight):
            y = fused.LinearFn.apply(x.reshape(-1, self.in_features), self.weight)
            return y.view(*x.shape[:-1], self.out_features)
        if getattr(self.weight, "lb_fp8", False):
            from ..float8 import Fp8LinearFn

            y = Fp8LinearFn.apply(x.reshape(-1, self.in_features), self.weight, None)
            return y.view(*x.shape[:-1], self.out_features)
        return TF.linear(x, self.weight)


class TiedLinear(nn.Module):
    def __init__(self, tied_module: nn.Module):
        super().__init__()
        self.tied_module = tied_module

    @property
    def weight(self):
        return self.tied_module.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return TF.linear(x, self.tied_module.weight)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _is_native(self.weight) and x.dtype == torch.bfloat16:
            y = _AddNormFn.apply(x.reshape(-1, x.shape[-1]).contiguous(), None, self.weight, self.eps)
            return y.view(x.shape)
        xf = x.float()
        out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (out * self.weight.float()).type_as(x)

    def reset_parameters(self):
        nn.init.ones_(self.weight)


class RotaryEmbedding(nn.Module):
    """Holds the (cos, sin) table as a non-persistent buffer ``freqs_cis`` [max_seqlen, head_dim/2, 2]."""

    def __init__(self, theta: float, head_dim: int, max_seqlen: int = 1024):
        super().__init__()
        self.theta, self.head_dim, self.max_seqlen = theta, head_dim, max_seqlen
        self.register_buffer("freqs_cis", F.rope_table(head_dim, max_seqlen, theta), persistent=False)

    def reset_parameters(self):
        # always fp32, whatever dtype the module was cast to
        self.freqs_cis = F.rope_table(self.head_dim, self.max_seqlen, self.theta, self.freqs_cis.device)

    def forward(self) -> torch.Tensor:
        return self.freqs_cis


class Attention(nn.Module):
    def __init__(self, dim: int, head_dim: int, n_heads: int, n_kv_heads: int, rope_theta: float):
        super().__init__()
        self.dim, self.head_dim, self.rope_theta = dim, head_dim, rope_theta
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.heads_per_group = n_heads // n_kv_heads
        self.wq = Linear(dim, n_heads * head_dim)
        self.wk = Linear(dim, n_kv_heads * head_dim)
        self.wv = Linear(dim, n_kv_heads * head_dim)
        self.wo = Linear(n_heads * head_dim, dim)
        self.kv_cache = None  # set by the generator

    def qkv_weights(self) -> Tuple[torch.Tensor, ...]:
        return (self.wq.weight, self.wk.weight, self.wv.weight)

    def forward_ref(self, x, cs, tok_idx=None, doc_start=None, window=0, causal=True):
        """x: [B, S, dim] already normalised."""
        B, S, _ = x.shape
        tpg = getattr(self, "tp_group", None)
        if tpg is not None:
            x = ReduceBwd.apply(x, tpg)
        q = self.wq(x).view(B, S, self.n_heads, self.head_dim)
        k = self.wk(x).view(B, S, self.n_kv_heads, self.head_dim)
        v = self.wv(x).view(B, S, self.n_kv_heads, self.head_dim)
        pos = tok_idx
        q = F.rope_ref(q, cs, pos)
        k = F.rope_ref(k, cs, pos)
        if self.kv_cache is not None:
            out = self.wo(self.kv_cache.attend(q, k, v, tok_idx).reshape(B, S, -1))
            return ReduceFwd.apply(out, tpg) if tpg is not None else out
        if q.is_cuda and q.dtype == torch.bfloat16 and doc_start is None and self.head_dim <= 128:
            o = _attention_flash_padded(q, k, v, causal, window)
        else:
            o = _attention_torch(q, k, v, causal, doc_start, window)
        out = self.wo(o.reshape(B, S, self.n_heads * self.head_dim))
        return ReduceFwd.apply(out, tpg) if tpg is not None else out

    def reset_parameters(self, init_std=None, factor=1.0):
        std = init_std or (self.dim ** (-0.5))
        for w in (self.wq, self.wk, self.wv):
            _init_linear(w, std)
        _init_linear(self.wo, std / factor, std)


def _attention_flash_padded(q, k, v, causal, window, doc_start=None):
    """The flash-attention kernel takes heads of width 128: narrower heads are zero-padded (the scores
    do not change, the padded half of the output is zero and is dropped)."""
    from ..ops.attention import attention

    Dh = q.shape[-1]
    if Dh < 128:
        q, k, v = (TF.pad(t, (0, 128 - Dh)) for t in (q, k, v))
    if doc_start is not None:
        doc_start = doc_start.reshape(q.shape[0], q.shape[1]).int().contiguous()
    o = attention(q.contiguous(), k.contiguous(), v.contiguous(), causal=causal, doc_start=doc_start,
                  window=window or 0, scale=1.0 / math.sqrt(Dh))
    return o[..., :Dh]


def _attention_torch(q, k, v, causal, doc_start, window):
    """Differentiable masked attention in PyTorch on [B,S,H,Dh] (reference path)."""
    B, S, H, Dh = q.shape
    Hkv = k.shape[2]
    qf = q.permute(0, 2, 1, 3)
    kf = k.permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    qi = torch.arange(S, device=q.device).view(1, 1, S, 1)
    ki = torch.arange(S, device=q.device).view(1, 1, 1, S)
    mask = torch.ones(1, 1, S, S, dtype=torch.bool, device=q.device)
    if causal:
        mask = mask & (ki <= qi)
    if window and window > 0:
        mask = mask & (ki > qi - window)
    if doc_start is not None:
        mask = mask & (ki >= doc_start.view(B, 1, S, 1).long())
    s = torch.matmul(qf.float(), kf.float().transpose(-1, -2)) / math.sqrt(Dh)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf.float()).to(q.dtype).permute(0, 2, 1, 3)


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, multiple_of: int, ffn_dim_multiplier: Optional[float],
                 mp_size: int = 1, activation: str = "swiglu"):
        super().__init__()
        hidden_dim = int(2 * hidden_dim / 3)
        if ffn_dim_multiplier is not None:
            hidden_dim = int(ffn_dim_multiplier * hidden_dim)
        hidden_dim = multiple_of * ((hidden_dim + multiple_of - 1) // multiple_of)
        assert hidden_dim % mp_size == 0
        assert activation in ("swiglu", "relu2")
        self.dim, self.hidden_dim, self.activation = dim, hidden_dim, activation
        self.w1 = Linear(dim, hidden_dim)
        if activation == "swiglu":
            self.w3 = Linear(dim, hidden_dim)
        self.w2 = Linear(hidden_dim, dim)

    def in_weights(self) -> Tuple[torch.Tensor, ...]:
        return (self.w1.weight, self.w3.weight) if self.activation == "swiglu" else (self.w1.weight,)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _is_native(self.w1.weight):
            x2 = x.reshape(-1, self.dim)
            if getattr(self, "tp_group", None) is not None:
                x2 = ReduceBwd.apply(x2, self.tp_group)
            if self.activation == "swiglu":
                gu = fused.LinearFn.apply(x2, *self.in_weights())
                out = fused.GluLinearFn.apply(gu, self.w2.weight, F.ACT_SILU)
            else:
                u = fused.LinearFn.apply(x2, self.w1.weight)
                out = fused.ActLinearFn.apply(u, self.w2.weight, F.ACT_RELU2)
            tpg = getattr(self, "tp_group", None)
            if tpg is not None:
                out = ReduceFwd.apply(out, tpg)
            return out.view(*x.shape[:-1], self.dim)
        tpg = getattr(self, "tp_group", None)
        if tpg is not None:
            x = ReduceBwd.apply(x, tpg)
        if self.activation == "swiglu":
            out = self.w2(TF.silu(self.w1(x)) * self.w3(x))
        else:
            out = self.w2(torch.relu(self.w1(x)).pow(2))
        return ReduceFwd.apply(out, tpg) if tpg is not None else out

    def reset_parameters(self, init_std=None, factor=1.0):
        in_std = init_std or (self.dim ** (-0.5))
        out_std = (init_std or (self.hidden_dim ** (-0.5))) / factor
        _init_linear(self.w1, in_std)
        if self.activation == "swiglu":
            _init_linear(self.w3, in_std)
        _init_linear(self.w2, out_std)


class TransformerBlock(nn.Module):
    def __init__(self, args: BaseTransformerArgs):
        super().__init__()
        assert (args.head_dim is not None) or (args.n_heads is not None), "Should specify at least head_dim or n_heads"
        self.head_dim = args.head_dim or args.dim // args.n_heads
        self.n_heads = args.n_heads or args.dim // args.head_dim
        self.n_kv_heads = args.n_kv_heads or self.n_heads
        assert self.n_heads % self.n_kv_heads == 0
        assert args.dim % self.n_heads == 0
        self.dim = args.dim
        self.attention = Attention(args.dim, self.head_dim, self.n_heads, self.n_kv_heads, args.rope_theta)
        self.feed_forward = FeedForward(args.dim, 4 * args.dim, args.multiple_of, args.ffn_dim_multiplier,
                                        activation=args.ffn_activation)
        self.attention_norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, eps=args.norm_eps)

    # ---- reference path: x [B, S, dim]
    def forward(self, x, cs, tok_idx=None, doc_start=None, window=0, causal=True):
        h = x + self.attention.forward_ref(self.attention_norm(x), cs, tok_idx, doc_start, window, causal)
        return h + self.feed_forward(self.ffn_norm(h))

    # ---- native path: x, pending are [B*S, dim]; the residual stream is x + pending
    def forward_native(self, x, pending, cs, B, S, doc_start=None, doc_end=None, window=0, pos=None, causal=True):
        at, ff = self.attention, self.feed_forward
        tpg = getattr(self, "tp_group", None)
        qkv, h = fused.NormLinearFn.apply(x, pending, self.attention_norm.weight, self.attention_norm.eps, tpg,
                                          *at.qkv_weights())
        x = x if h is None else h
        if at.kv_cache is not None:  # generation: rotate, then attend through the KV cache
            F.rope_(qkv, cs, at.n_heads + at.n_kv_heads, at.head_dim, S, pos)
            t = qkv.view(B * S, at.n_heads + 2 * at.n_kv_heads, at.head_dim)
            o = at.kv_cache.native_attention(t[:, :at.n_heads], t[:, at.n_heads:at.n_heads + at.n_kv_heads],
                                             t[:, at.n_heads + at.n_kv_heads:])
        else:
            o = fused.RopeAttnFn.apply(qkv, cs, B, S, at.n_heads, at.n_kv_heads, at.head_dim, causal, doc_start,
                                       doc_end, window, pos, at.wo.weight)
        ao = fused.LinearFn.apply(o, at.wo.weight)
        if tpg is not None:
            ao = ReduceFwd.apply(ao, tpg)
        u, x2 = fused.NormLinearFn.apply(x, ao, self.ffn_norm.weight, self.ffn_norm.eps, tpg, *ff.in_weights())
        if ff.activation == "swiglu":
            out = fused.GluLinearFn.apply(u, ff.w2.weight, F.ACT_SILU)
        else:
            out = fused.ActLinearFn.apply(u, ff.w2.weight, F.ACT_RELU2)
        if tpg is not None:
            out = ReduceFwd.apply(out, tpg)
        return x2, out

    def init_weights(self, init_std=None, factor=1.0):
        self.attention.reset_parameters(init_std, factor)
        self.attention_norm.reset_parameters()
        self.feed_forward.reset_parameters(init_std, factor)
        self.ffn_norm.reset_parameters()


class BaseTransformer(nn.Module):
    def __init__(self, args: BaseTransformerArgs):
        super().__init__()
        self.dim = args.dim
        self.init_base_std = args.init_base_std
        self.init_std_factor = InitStdFactor(args.init_std_factor)
        self.max_seqlen = args.max_seqlen
        self.rope_embeddings = RotaryEmbedding(args.rope_theta, args.head_dim or args.dim // args.n_heads,
                                               args.max_seqlen)
        self.layers = nn.ModuleList(TransformerBlock(args) for _ in range(args.n_layers))

    def reset_parameters(self):
        self.rope_embeddings.reset_parameters()

    def init_weights(self):
        self.reset_parameters()
        for depth, layer in enumerate(self.layers):
            factor = {
                InitStdFactor.CURRENT_DEPTH: (2 * (depth + 1)) ** 0.5,
                InitStdFactor.GLOBAL_DEPTH: (2 * (len(self.layers) + 1)) ** 0.5,
                InitStdFactor.DIM_RATIO: self.dim / 4096,
                InitStdFactor.DISABLED: 1.0,
            }[self.init_std_factor]
            layer.init_weights(self.init_base_std, factor)


class LMTransformer(BaseTransformer):
    """Token embedding -> blocks -> final norm -> vocabulary head (-> cross-entropy if targets given)."""

    def __init__(self, args: LMTransformerArgs):
        super().__init__(args)
        assert args.vocab_size > 0
        self.weight_tying = args.weight_tying
        self.sliding_window = args.sliding_window
        self.loss_chunk = args.loss_chunk
        self.vocab_size = args.vocab_size
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.output = TiedLinear(self.tok_embeddings) if args.weight_tying else Linear(args.dim, args.vocab_size)

    def forward(self, token_values: torch.Tensor, target: Optional[torch.Tensor] = None,
                tok_idx: Optional[torch.Tensor] = None, doc_start: Optional[torch.Tensor] = None,
                doc_end: Optional[torch.Tensor] = None, causal: bool = True):
        """Returns the mean cross-entropy if ``target`` is given, else logits [B, S, vocab].

        ``doc_start`` / ``doc_end`` ([B, S] int32): block-causal attention over packed documents.
        ``tok_idx``: explicit RoPE positions (generation)."""
        B, S = token_values.shape
        window = self.sliding_window or 0
        cs = self.rope_embeddings()
        if _is_native(self.tok_embeddings.weight):
            tpf = getattr(self, "tp_fused", None)
            if (tpf is not None and not torch.is_grad_enabled() and causal and tok_idx is None
                    and doc_start is None and tpf.accepts(B, S) and self.layers[0].attention.kv_cache is None):
                # tensor-parallel scoring / evaluation: collectives fused into the GEMM kernels
                return tpf(token_values, target)
            sp = getattr(self, "tp_sp", None)
            if (sp is not None and causal and tok_idx is None and sp.accepts(B * S)
                    and self.layers[0].attention.kv_cache is None and self.layers[0].attention.head_dim == 128):
                # tensor parallel with a row-sharded residual stream, collectives inside the GEMM kernels
                return self._forward_sp(sp, token_values, target, doc_start, doc_end, window, causal, cs, B, S)
            return self._forward_native(token_values, target, tok_idx, doc_start, doc_end, window, causal, cs, B, S)
        h = self.tok_embeddings(token_values)
        for layer in self.layers:
            h = layer(h, cs, tok_idx, doc_start, window, causal)
        logits = self.output(self.norm(h))
        if target is not None:
            return cross_entropy(logits, target)
        return logits

    def _forward_native(self, tokens, target, tok_idx, doc_start, doc_end, window, causal, cs, B, S):
        pos = tok_idx.reshape(-1).int().contiguous() if tok_idx is not None else None
        if doc_start is not None:
            doc_start = doc_start.reshape(-1).int().contiguous()
        if doc_end is not None:
            doc_end = doc_end.reshape(-1).int().contiguous()
        eng = getattr(self, "_engine", None)
        if eng is not None:
            eng.boundary("tok_embeddings")
        x = fused.EmbeddingFn.apply(tokens.reshape(-1), self.tok_embeddings.weight)
        pending = None
        for i, layer in enumerate(self.layers):
            if eng is not None:
                x, pending = eng.boundary(f"layers.{i}", x, pending)
            x, pending = layer.forward_native(x, pending, cs, B, S, doc_start, doc_end, window, pos, causal)
        if eng is not None:
            x, pending = eng.boundary("output", x, pending)
            eng.boundary("")
        w_out = self.output.weight
        if target is not None:
            y, _ = _final_norm(x, pending, self.norm)
            # set by the training engine: the constant gradient that will reach the loss
            gs = getattr(self, "loss_grad_scale", None) if torch.is_grad_enabled() else None
            return fused.LinearCrossEntropyFn.apply(y, w_out, target.reshape(-1), self.loss_chunk, gs)
        y, _ = _final_norm(x, pending, self.norm)
        return fused.LinearFn.apply(y, w_out).view(B, S, -1)

    def _forward_sp(self, sp, tokens, target, doc_start, doc_end, window, causal, cs, B, S):
        """Sequence-parallel tensor-parallel pass (``parallel/tp_train.py``): every TP rank carries ``B*S / tp``
        consecutive rows of the residual stream; every rank of the group is given the same tokens."""
        from ..parallel.tp_train import SumOverGroupFn, sp_block_forward

        T = B * S
        sp.setup(T, self.dim)
        rows = slice(sp.rank * sp.Tl, (sp.rank + 1) * sp.Tl)
        if doc_start is not None:
            doc_start = doc_start.reshape(-1).int().contiguous()
        if doc_end is not None:
            doc_end = doc_end.reshape(-1).int().contiguous()
        eng = getattr(self, "_engine", None)
        if eng is not None:
            eng.boundary("tok_embeddings")
        x = fused.EmbeddingFn.apply(tokens.reshape(-1)[rows].contiguous(), self.tok_embeddings.weight)
        for i, layer in enumerate(self.layers):
            if eng is not None:
                (x,) = eng.boundary(f"layers.{i}", x)
            x = sp_block_forward(layer, sp, x, cs, B, S, doc_start, doc_end, window, None, causal)
        if eng is not None:
            (x,) = eng.boundary("output", x)
            eng.boundary("")
        y, _ = _final_norm(x, None, self.norm)
        w_out = self.output.weight
        if target is not None:
            tgt = target.reshape(-1)
            n_valid = (tgt >= 0).sum().clamp(min=1).float()  # over all rows: every rank sees the same targets
            gs = getattr(self, "loss_grad_scale", None) if torch.is_grad_enabled() else None
            part = fused.LinearCrossEntropyFn.apply(y, w_out, tgt[rows].contiguous(), self.loss_chunk, gs, n_valid)
            return SumOverGroupFn.apply(part, sp.group)
        local = fused.LinearFn.apply(y, w_out)
        full = torch.empty(T, local.shape[1], dtype=local.dtype, device=local.device)
        torch.distributed.all_gather_into_tensor(full, local.contiguous(), group=sp.group)
        return full.view(B, S, -1)

    def reset_parameters(self, init_std=None):
        super().reset_parameters()
        std = init_std or (self.dim ** (-0.5))
        self.norm.reset_parameters()
        _trunc(self.tok_embeddings.weight, std)
        if not self.weight_tying:
            _trunc(self.output.weight, std)

    def init_weights(self):
        self.reset_parameters()
        super().init_weights()


class _AddNormFn(torch.autograd.Function):
    """y = rmsnorm(x + res) * g (final norm of the native path)."""

    @staticmethod
    def forward(ctx, x, res, g, eps):
        y, h, rstd = F.rmsnorm_fwd(x, g.detach(), eps, res)
        ctx.save_for_backward(x if h is None else h, rstd)
        ctx.g, ctx.has_res = g, res is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        h, rstd = ctx.saved_tensors
        g = ctx.g
        holder = {}

        def run(buf):
            holder["dx"], _ = F.rmsnorm_bwd(dy.contiguous(), h, g.detach(), rstd, None, buf)

        dg = fused._emit_vec_grad(g, run)
        dx = holder["dx"]
        return dx, (dx if ctx.has_res else None), dg, None


def _final_norm(x, pending, norm: RMSNorm):
    return _AddNormFn.apply(x, pending, norm.weight, norm.eps), None


# ----------------------------------------------------------------------------- FLOPs and plans
def attention_flops_per_token(n_layers, seq_len, dim, causal):
    # 3.5 = 1 forward + 2 backward + 0.5 recomputed forward of the score matrix
    return 3.5 * (4 * n_layers * seq_len * dim // (2 if causal else 1))


def get_num_flop_per_token(num_non_embed_params: int, n_layers: int, dim: int, seq_len: int) -> int:
    return 6 * num_non_embed_params + attention_flops_per_token(n_layers, seq_len, dim, True)


def build_fsdp_grouping_plan(model_args: LMTransformerArgs):
    """(module path, reshard_after_forward) per sharding group: embeddings, every block, output head."""
    plan = [("tok_embeddings", False)]
    plan += [(f"layers.{i}", False) for i in range(model_args.n_layers)]
    plan.append(("output", True))
    return plan


def get_no_recompute_ops():
    """The native path fixes what is saved (GEMM and attention outputs) inside its autograd functions."""
    return None
