"""Linear-recurrence language models: minGRU, minLSTM and Hawk (RG-LRU).

Parameter names, shapes, initialisation and gate math follow apps/fastRNN/minGRU/core_gru.py
(GRU :40), apps/fastRNN/minLSTM/core_lstm.py (LSTM :34) and apps/fastRNN/hawk/core_hawk.py (RGLRU
:59, RGLRUBlock :166, HawkBlock :240) and their LM wrappers, so configs and checkpoints are
interchangeable. Everything runs channel-last on [B, S, C]: the projections are GEMMs on
[tokens, C], the causal conv1d and the recurrence h_t = a_t h_{t-1} + b_t are this library's
kernels (``lingua_b200.ops.sequence``) with document resets from ``doc_start``, so there is no
transpose to a [B, C, S] layout and no power-of-two padding of the sequence.

Generation: a ``StateCache`` per recurrent block holds the conv window and the recurrent state
of every sequence; ``impl="sequential"`` advances them by one token.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import fused
from ..ops.sequence import (causal_conv1d, conv1d_update, conv_states_from_packed, last_states_from_packed,
                            rglru_gates, rnn_step,
                            linear_scan)
from .transformer import (FeedForward, InitStdFactor, Linear, RMSNorm, TiedLinear, _is_native, _trunc,
                          cross_entropy)


def _hidden(hidden_dim: int, multiple_of: int, mult: Optional[float], two_thirds: bool = True) -> int:
    if two_thirds:
        hidden_dim = int(2 * hidden_dim / 3)
    if mult is not None:
        hidden_dim = int(mult * hidden_dim)
    return multiple_of * ((hidden_dim + multiple_of - 1) // multiple_of)


def doc_start_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """[1, total] int32 document-start index per token of a packed sequence."""
    lengths = cu_seqlens[1:] - cu_seqlens[:-1]
    return torch.repeat_interleave(cu_seqlens[:-1], lengths).int().view(1, total)


class StateCache(nn.Module):
    """Per-block generation state: last ``conv_size`` inputs and the recurrent state of each sequence."""

    def __init__(self, bsz, hidden, conv_size, conv_dim, dtype, device):
        super().__init__()
        conv_shape = (0,) if conv_size is None else (bsz, conv_dim, conv_size)
        self.register_buffer("conv_cache", torch.zeros(conv_shape, dtype=dtype, device=device), persistent=False)
        self.register_buffer("state_cache", torch.zeros(bsz, hidden, dtype=torch.float32, device=device),
                             persistent=False)
        self.lengths = None  # set by the generator before a packed prefill

    def reset(self):
        self.conv_cache.zero_()
        self.state_cache.zero_()


class _Recurrent(nn.Module):
    """Shared plumbing: optional conv on some gate pre-activation and the cached / uncached scan."""

    conv_size: Optional[int]
    cache: Optional[StateCache] = None

    def make_cache(self, n_seqs: int, dtype, device) -> StateCache:
        width = getattr(self, "hidden_dim", None) or self.dim  # channels of the recurrent state
        return StateCache(n_seqs, width, self.conv_size, getattr(self, "conv_dim", 0), dtype, device)

    def _conv(self, u, doc_start, impl):
        """u: [B, S, C] pre-activation -> conv + SiLU (identity when the block has no conv)."""
        if self.conv_size is None:
            return u
        cache = self.cache
        if impl == "sequential":
            return conv1d_update(u[0], cache.conv_cache, self.conv_weight).unsqueeze(0)
        if cache is not None:
            cache.conv_cache.copy_(conv_states_from_packed(u[0], cache.lengths, self.conv_size))
        return causal_conv1d(u, self.conv_weight, doc_start, act=True)

    def _scan(self, a, b, doc_start, impl):
        cache = self.cache
        if impl == "sequential":
            return rnn_step(a[0], b[0], cache.state_cache).unsqueeze(0)
        h = linear_scan(a, b, doc_start)
        if cache is not None:
            cache.state_cache.copy_(last_states_from_packed(h[0], cache.lengths).float())
        return h

    def _init_conv(self, init_std):
        if self.conv_size is not None:
            std = init_std or (self.conv_size ** (-0.5))
            _trunc(self.conv_weight, std)


# ----------------------------------------------------------------------------- minGRU
@dataclass
class BaseMinGRUArgs:
    dim: int = 512
    n_layers: int = 8
    n_heads: int = 1
    multiple_of: int = 256
    ffn_dim_multiplier: Optional[float] = None
    conv_size: Optional[int] = None
    norm_eps: float = 1e-5
    init_base_std: Optional[float] = None
    init_std_factor: str = "disabled"


class GRU(_Recurrent):
    """z = sigmoid(conv(wz x)); h_t = (1 - z_t) h_{t-1} + z_t (wh_tilde x)_t; out = wo(h * silu(w x))."""

    def __init__(self, dim, hidden_dim, n_heads, multiple_of, ffn_dim_multiplier, conv_size=None):
        super().__init__()
        hidden_dim = _hidden(hidden_dim, multiple_of, ffn_dim_multiplier)
        assert hidden_dim % n_heads == 0, f"Hidden dim must be divisible by n_heads: {hidden_dim} % {n_heads} != 0"
        self.dim, self.hidden_dim, self.n_heads, self.head_dim = dim, hidden_dim, n_heads, hidden_dim // n_heads
        self.conv_size = conv_size
        if conv_size is not None:
            assert hidden_dim % 8 == 0 and conv_size in (2, 3, 4)
            self.conv_dim = hidden_dim
            self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, conv_size))
        self.w = Linear(dim, hidden_dim)
        self.wz = Linear(dim, hidden_dim)
        self.wh_tilde = Linear(dim, hidden_dim)
        self.wo = Linear(hidden_dim, dim)

    def forward(self, x, doc_start=None, impl="parallel"):
        w0 = self.w(x)
        z = torch.sigmoid(self._conv(self.wz(x), doc_start, impl).float())
        h_tilde = self.wh_tilde(x).float()
        h = self._scan((1 - z).to(x.dtype), (z * h_tilde).to(x.dtype), doc_start, impl)
        return self.wo(h * TF.silu(w0))

    def reset_parameters(self, init_std, factor):
        in_std = init_std or (self.dim ** (-0.5))
        out_std = (init_std or (self.hidden_dim ** (-0.5))) / factor
        for m in (self.w, self.wz, self.wh_tilde):
            _trunc(m.weight, in_std)
        _trunc(self.wo.weight, out_std, in_std)
        self._init_conv(init_std)


# ----------------------------------------------------------------------------- minLSTM
@dataclass
class BaseMinLSTMArgs(BaseMinGRUArgs):
    pass


class LSTM(_Recurrent):
    """f, i = sigmoid(conv(wfi x)) per head; h_t = f/(f+i+eps) h_{t-1} + i/(f+i+eps) (wh_tilde x)_t."""

    def __init__(self, dim, hidden_dim, n_heads, multiple_of, ffn_dim_multiplier, conv_size=None):
        super().__init__()
        hidden_dim = _hidden(hidden_dim, multiple_of, ffn_dim_multiplier)
        assert hidden_dim % n_heads == 0
        self.dim, self.hidden_dim, self.n_heads, self.head_dim = dim, hidden_dim, n_heads, hidden_dim // n_heads
        self.conv_size = conv_size
        if conv_size is not None:
            assert hidden_dim % 8 == 0 and conv_size in (2, 3, 4)
            self.conv_dim = 2 * hidden_dim
            self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, conv_size))
        self.w = Linear(dim, hidden_dim)
        self.wfi = Linear(dim, 2 * hidden_dim)
        self.wh_tilde = Linear(dim, hidden_dim)
        self.wo = Linear(hidden_dim, dim)

    def forward(self, x, doc_start=None, impl="parallel"):
        B, S, _ = x.shape
        w0 = self.w(x)
        fi = self._conv(self.wfi(x), doc_start, impl).float()
        # channels are laid out per head as [f (head_dim) | i (head_dim)]
        fi = fi.view(B, S, self.n_heads, 2, self.head_dim)
        f = torch.sigmoid(fi[:, :, :, 0]).reshape(B, S, self.hidden_dim)
        i = torch.sigmoid(fi[:, :, :, 1]).reshape(B, S, self.hidden_dim)
        denom = 1 / (f + i + 1e-4)
        h_tilde = self.wh_tilde(x).float()
        h = self._scan((f * denom).to(x.dtype), (h_tilde * i * denom).to(x.dtype), doc_start, impl)
        return self.wo(h * TF.silu(w0))

    def reset_parameters(self, init_std, factor):
        in_std = init_std or (self.dim ** (-0.5))
        out_std = (init_std or (self.hidden_dim ** (-0.5))) / factor
        for m in (self.w, self.wfi, self.wh_tilde):
            _trunc(m.weight, in_std)
        _trunc(self.wo.weight, out_std, in_std)
        self._init_conv(init_std)


class _ResidualBlock(nn.Module):
    def __init__(self, inner_name: str, norm_name: str, inner: nn.Module, dim: int, eps: float):
        super().__init__()
        self._inner_name, self._norm_name = inner_name, norm_name
        setattr(self, norm_name, RMSNorm(dim, eps=eps))
        setattr(self, inner_name, inner)

    def forward(self, x, doc_start=None, impl="parallel"):
        inner, norm = getattr(self, self._inner_name), getattr(self, self._norm_name)
        return x + inner(norm(x), doc_start=doc_start, impl=impl)

    def init_weights(self, init_std, factor):
        getattr(self, self._inner_name).reset_parameters(init_std, factor)
        getattr(self, self._norm_name).reset_parameters()


class GRUBlock(_ResidualBlock):
    def __init__(self, args: BaseMinGRUArgs):
        super().__init__("gru", "gru_norm", GRU(args.dim, 3 * args.dim, args.n_heads, args.multiple_of,
                                                args.ffn_dim_multiplier, args.conv_size), args.dim, args.norm_eps)


class LSTMBlock(_ResidualBlock):
    def __init__(self, args: BaseMinLSTMArgs):
        super().__init__("lstm", "lstm_norm", LSTM(args.dim, 3 * args.dim, args.n_heads, args.multiple_of,
                                                   args.ffn_dim_multiplier, args.conv_size), args.dim, args.norm_eps)


# ----------------------------------------------------------------------------- Hawk
@dataclass
class BaseHawkArgs:
    dim: int = 512
    n_layers: int = 8
    n_heads: int = 1
    multiple_of: int = 256
    ffn_dim_multiplier: Optional[float] = None
    lru_dim_multiplier: Optional[float] = None
    conv_size: Optional[int] = None
    norm_eps: float = 1e-5
    init_base_std: Optional[float] = None
    init_std_factor: str = "disabled"
    # Extension: "dense" gates (full Linear, as the reference) or "block_diagonal" (one block per head).
    gate_structure: str = "dense"


class BlockDiagonalLinear(nn.Module):
    """``n_blocks`` independent [w, w] maps applied to consecutive channel groups."""

    def __init__(self, dim: int, n_blocks: int):
        super().__init__()
        self.dim, self.n_blocks = dim, n_blocks
        self.weight = nn.Parameter(torch.empty(n_blocks, dim // n_blocks, dim // n_blocks))

    def forward(self, x):
        shp = x.shape
        xb = x.reshape(-1, self.n_blocks, self.dim // self.n_blocks)
        return torch.einsum("tbi,boi->tbo", xb, self.weight.to(x.dtype)).reshape(shp)


class RGLRU(_Recurrent):
    """Real-gated linear recurrent unit: log a_t = -8 * sigmoid(a_gate x) * softplus(a);
    h_t = a_t h_{t-1} + sqrt(1 - a_t^2) * sigmoid(input_gate x) * x_t (x after conv + SiLU)."""

    def __init__(self, dim, n_heads, head_dim, conv_size=None, gate_structure="dense"):
        super().__init__()
        assert head_dim * n_heads == dim
        self.dim, self.head_dim, self.n_heads, self.c = dim, head_dim, n_heads, 8.0
        self.conv_size = conv_size
        if conv_size is not None:
            assert dim % 8 == 0 and conv_size in (2, 3, 4)
            self.conv_dim = dim
            self.conv_weight = nn.Parameter(torch.empty(dim, conv_size))
        self.a = nn.Parameter(torch.empty(head_dim))
        if gate_structure == "block_diagonal":
            self.input_gate, self.a_gate = BlockDiagonalLinear(dim, n_heads), BlockDiagonalLinear(dim, n_heads)
        else:
            self.input_gate, self.a_gate = Linear(dim, dim), Linear(dim, dim)

    def forward(self, x, doc_start=None, impl="parallel"):
        B, S, _ = x.shape
        x = self._conv(x, doc_start, impl)
        # both gates, the decay and the input scaling in one kernel each way (ops.sequence.rglru_gates)
        sp = TF.softplus(self.a.float()).repeat(self.n_heads)
        a, b = rglru_gates(self.input_gate(x), self.a_gate(x), x, sp)
        return self._scan(a, b, doc_start, impl)

    def reset_parameters(self, init_std, factor):
        in_std = (init_std or (self.dim ** (-0.5))) / factor
        for m in (self.input_gate, self.a_gate):
            _trunc(m.weight, in_std)
        min_rad, max_rad = 0.9, 0.999
        with torch.no_grad():
            self.a.uniform_(min_rad ** 2 + 1e-8, max_rad ** 2 + 1e-8)
            self.a.log_().mul_(0.5)
        self._init_conv(init_std)


class RGLRUBlock(nn.Module):
    def __init__(self, dim, hidden_dim, n_heads, multiple_of, lru_dim_multiplier, conv_size=None,
                 gate_structure="dense"):
        super().__init__()
        hidden_dim = _hidden(hidden_dim, multiple_of, lru_dim_multiplier, two_thirds=False)
        assert hidden_dim % n_heads == 0, f"Hidden dim must be divisible by n_heads: {hidden_dim} % {n_heads} != 0"
        self.dim, self.hidden_dim = dim, hidden_dim
        self.wy = Linear(dim, hidden_dim)
        self.wx = Linear(dim, hidden_dim)
        self.rglru = RGLRU(hidden_dim, n_heads, hidden_dim // n_heads, conv_size, gate_structure)
        self.wo = Linear(hidden_dim, dim)

    def forward(self, x, doc_start=None, impl="parallel"):
        h = self.rglru(self.wx(x), doc_start=doc_start, impl=impl)
        h = h * TF.silu(self.wy(x))
        return x + self.wo(h)  # the block adds its (normalised) input, as the reference does

    def init_weights(self, init_std, factor):
        self.rglru.reset_parameters(init_std, factor)
        in_std = (init_std or (self.dim ** (-0.5))) / factor
        out_std = (init_std or (self.hidden_dim ** (-0.5))) / factor
        for m in (self.wy, self.wx):
            _trunc(m.weight, in_std)
        _trunc(self.wo.weight, out_std)


class HawkBlock(nn.Module):
    def __init__(self, args: BaseHawkArgs):
        super().__init__()
        self.rlgru_block = RGLRUBlock(args.dim, int(4 / 3 * args.dim), args.n_heads, args.multiple_of,
                                      args.lru_dim_multiplier, args.conv_size, args.gate_structure)
        self.feed_forward = FeedForward(args.dim, 4 * args.dim, args.multiple_of, args.ffn_dim_multiplier)
        self.rlgru_norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, eps=args.norm_eps)

    def forward(self, x, doc_start=None, impl="parallel"):
        x = x + self.rlgru_block(self.rlgru_norm(x), doc_start=doc_start, impl=impl)
        return x + self.feed_forward(self.ffn_norm(x))

    def init_weights(self, init_std, factor):
        self.rlgru_block.init_weights(init_std, factor)
        self.rlgru_norm.reset_parameters()
        self.feed_forward.reset_parameters()
        self.ffn_norm.reset_parameters()


# ----------------------------------------------------------------------------- LM wrappers
@dataclass
class LMMinGRUArgs(BaseMinGRUArgs):
    seed: int = 42
    vocab_size: int = -1
    weight_tying: bool = False
    loss_reduction: str = "mean"
    loss_chunk: int = 2048


@dataclass
class LMMinLSTMArgs(BaseMinLSTMArgs):
    seed: int = 42
    vocab_size: int = -1
    weight_tying: bool = False
    loss_reduction: str = "mean"
    loss_chunk: int = 2048


@dataclass
class LMHawkArgs(BaseHawkArgs):
    seed: int = 42
    vocab_size: int = -1
    weight_tying: bool = False
    loss_reduction: str = "mean"
    loss_chunk: int = 2048


class _LMRecurrent(nn.Module):
    block_cls = None

    def __init__(self, args):
        super().__init__()
        self.dim = args.dim
        self.init_base_std = args.init_base_std
        self.init_std_factor = InitStdFactor(args.init_std_factor)
        self.layers = nn.ModuleList(self.block_cls(args) for _ in range(args.n_layers))
        self.weight_tying, self.loss_reduction, self.seed = args.weight_tying, args.loss_reduction, args.seed
        self.loss_chunk = args.loss_chunk
        assert args.vocab_size > 0
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.output = TiedLinear(self.tok_embeddings) if args.weight_tying else Linear(args.dim, args.vocab_size)

    def forward(self, token_values, target=None, tok_idx=None, cu_seqlens=None, impl="parallel", doc_start=None):
        """``doc_start`` ([B, S] int32) or ``cu_seqlens`` (packed, B = 1) delimit documents."""
        B, S = token_values.shape
        if doc_start is None and cu_seqlens is not None and impl == "parallel":
            doc_start = doc_start_from_cu_seqlens(cu_seqlens, S)
        native = _is_native(self.tok_embeddings.weight)
        eng = getattr(self, "_engine", None) if native else None
        if native:
            if eng is not None:
                eng.boundary("tok_embeddings")
            h = fused.EmbeddingFn.apply(token_values.reshape(-1), self.tok_embeddings.weight).view(B, S, self.dim)
        else:
            h = self.tok_embeddings(token_values)
        for i, layer in enumerate(self.layers):
            if eng is not None:
                (h,) = eng.boundary(f"layers.{i}", h)
            h = layer(h, doc_start=doc_start, impl=impl)
        if eng is not None:
            (h,) = eng.boundary("output", h)
            eng.boundary("")
        y = self.norm(h)
        if target is None:
            return self.output(y)
        if native and self.loss_reduction == "mean":
            gs = getattr(self, "loss_grad_scale", None) if torch.is_grad_enabled() else None
            return fused.LinearCrossEntropyFn.apply(y.reshape(-1, self.dim), self.output.weight, target.reshape(-1),
                                                    self.loss_chunk, gs)
        return cross_entropy(self.output(y).flatten(0, 1), target.flatten(0, 1), reduction=self.loss_reduction)

    def reset_parameters(self, init_std=None):
        std = init_std or (self.dim ** (-0.5))
        self.norm.reset_parameters()
        _trunc(self.tok_embeddings.weight, std)
        if not self.weight_tying:
            _trunc(self.output.weight, std)

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


class LMMinGRU(_LMRecurrent):
    block_cls = GRUBlock


class LMMinLSTM(_LMRecurrent):
    block_cls = LSTMBlock


class LMHawk(_LMRecurrent):
    block_cls = HawkBlock


MODEL_TYPES = {"minGRU": (LMMinGRU, LMMinGRUArgs), "minLSTM": (LMMinLSTM, LMMinLSTMArgs),
               "hawk": (LMHawk, LMHawkArgs)}


def recurrent_modules(model: nn.Module):
    return [m for m in model.modules() if isinstance(m, _Recurrent)]


def build_fsdp_grouping_plan(model_args):
    plan = [("tok_embeddings", False)]
    plan += [(f"layers.{i}", False) for i in range(model_args.n_layers)]
    plan.append(("output", True))
    return plan
