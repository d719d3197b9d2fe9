"""Mamba-2 language model.

Parameter names, shapes, initialisation and config follow apps/mamba/core_mamba.py (InitArgs :25,
BaseMambaArgs :36, SSM :72, MambaBlock :366, BaseMamba :403) and apps/mamba/mamba.py (LMMambaArgs
:14, StateCache :37, LMMamba :64). Block: ``in_proj -> [z | xBC | dt] -> causal conv1d + SiLU on
xBC -> split x, B, C -> chunked SSD (softplus(dt + bias), A = -exp(A_log), D skip) ->
RMSNorm(y * silu(z)) -> out_proj``. The conv and the SSD run channel-last with document resets
(``doc_start``); generation keeps a conv window and an SSM state per sequence.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import fused
from ..ops.sequence import causal_conv1d, conv1d_update, conv_states_from_packed
from ..ops.ssd import selective_state_update, ssd_chunked
from .fastrnn import doc_start_from_cu_seqlens
from .transformer import InitStdFactor, Linear, RMSNorm, TiedLinear, _is_native, _trunc, cross_entropy


@dataclass
class InitArgs:
    dt_max: float = 0.1
    dt_min: float = 0.001
    dt_init_floor: float = 1e-4
    A_init_min: float = 1
    A_init_max: float = 16


@dataclass
class BaseMambaArgs:
    dim: int = 512
    n_layers: int = 8
    n_heads: int = 8
    state_dim: int = 128
    n_groups: int = 1
    conv_size: Optional[int] = None
    dt_bias: bool = False
    D_has_head_dim: bool = False
    learnable_init_states: bool = False
    ssm_chunk_size: int = 256
    vocab_size: int = -1
    ffn_dim_multiplier: Optional[float] = None
    multiple_of: int = 256
    norm_eps: float = 1e-5
    init_use_depth: bool = False
    init_base_std: Optional[float] = None
    init_std_factor: str = "disabled"
    init_args: InitArgs = field(default_factory=InitArgs)
    seed: int = 42


@dataclass
class LMMambaArgs(BaseMambaArgs):
    seed: int = 42
    vocab_size: int = -1
    weight_tying: bool = False
    loss_reduction: str = "mean"
    loss_chunk: int = 2048


class StateCache(nn.Module):
    def __init__(self, bsz, n_heads, head_dim, state_dim, conv_size, conv_dim, dtype, device):
        super().__init__()
        conv_shape = (0,) if conv_size is None else (bsz, conv_dim, conv_size)
        self.register_buffer("conv_cache", torch.zeros(conv_shape, dtype=dtype, device=device), persistent=False)
        self.register_buffer("state_cache", torch.zeros(bsz, n_heads, head_dim, state_dim, dtype=torch.float32,
                                                        device=device), persistent=False)
        self.lengths = None

    def reset(self):
        self.conv_cache.zero_()
        self.state_cache.zero_()


class SSM(nn.Module):
    def __init__(self, dim, hidden_dim, multiple_of, ffn_dim_multiplier, state_dim, n_heads, n_groups, conv_size,
                 dt_bias, D_has_head_dim, learnable_init_states, dt_limit: Tuple[float, float] = (0.0, float("inf")),
                 chunk_size=256):
        super().__init__()
        self.dim = dim
        hidden_dim = int(2 * hidden_dim / 3)
        if ffn_dim_multiplier is not None:
            hidden_dim = int(ffn_dim_multiplier * hidden_dim)
        self.hidden_dim = multiple_of * ((hidden_dim + multiple_of - 1) // multiple_of)
        assert self.hidden_dim % n_heads == 0, f"Hidden dim must be divisible by n_heads: {self.hidden_dim} % {n_heads} != 0"
        self.state_dim, self.head_dim = state_dim, self.hidden_dim // n_heads
        self.n_heads, self.n_groups, self.dt_limit, self.chunk_size = n_heads, n_groups, dt_limit, chunk_size
        self.in_proj = Linear(dim, 2 * self.hidden_dim + 2 * n_groups * state_dim + n_heads)
        self.conv_size, self.conv_dim = conv_size, None
        if conv_size is not None:
            self.conv_dim = self.hidden_dim + 2 * n_groups * state_dim
            assert self.conv_dim % 8 == 0 and conv_size in (2, 3, 4)
            self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, conv_size))
        self.learnable_init_states = learnable_init_states
        if learnable_init_states:
            self.init_states = nn.Parameter(torch.zeros(n_heads, self.head_dim, state_dim))
        self.dt_bias = nn.Parameter(torch.empty(n_heads)) if dt_bias else None
        self.A_log = nn.Parameter(torch.empty(n_heads))
        if D_has_head_dim is None:
            self.D = None
        else:
            self.D = nn.Parameter(torch.ones(n_heads, self.head_dim) if D_has_head_dim else torch.ones(n_heads))
        self.out_proj = Linear(self.hidden_dim, dim)
        self.ssm_norm = RMSNorm(self.hidden_dim, eps=1e-5)

    def make_cache(self, n_seqs, dtype, device) -> StateCache:
        return StateCache(n_seqs, self.n_heads, self.head_dim, self.state_dim, self.conv_size, self.conv_dim, dtype,
                          device)

    def forward(self, x, doc_start=None, ssm_impl="ssm"):
        bsz, S, _ = x.shape
        cache = getattr(self, "cache", None)
        gn = self.n_groups * self.state_dim
        zxbcdt = self.in_proj(x)
        z = zxbcdt[..., : self.hidden_dim]
        xBC = zxbcdt[..., self.hidden_dim: 2 * self.hidden_dim + 2 * gn]
        dt = zxbcdt[..., 2 * self.hidden_dim + 2 * gn:]
        if self.conv_size is not None:
            if ssm_impl == "ssm":
                if cache is not None:
                    cache.conv_cache.copy_(conv_states_from_packed(xBC[0], cache.lengths, self.conv_size))
                xBC = causal_conv1d(xBC, self.conv_weight, doc_start, act=True)
            elif ssm_impl == "ssm_update":
                xBC = conv1d_update(xBC[0], cache.conv_cache, self.conv_weight).unsqueeze(0)
            else:
                raise NotImplementedError(f"SSM implementation {ssm_impl} not supported")
        xs = xBC[..., : self.hidden_dim].reshape(bsz, S, self.n_heads, self.head_dim)
        B = xBC[..., self.hidden_dim: self.hidden_dim + gn].reshape(bsz, S, self.n_groups, self.state_dim)
        C = xBC[..., self.hidden_dim + gn:].reshape(bsz, S, self.n_groups, self.state_dim)
        A = -torch.exp(self.A_log.float())
        dtp = dt.float() + (self.dt_bias.float() if self.dt_bias is not None else 0.0)
        dtp = TF.softplus(dtp)
        if self.dt_limit != (0.0, float("inf")):
            dtp = dtp.clamp(self.dt_limit[0], self.dt_limit[1])
        if ssm_impl == "ssm":
            init = self.init_states.expand(bsz, -1, -1, -1) if self.learnable_init_states else None
            if cache is not None and doc_start is not None:
                # packed prefill: documents are scanned separately so that each final state is kept
                y, states = _ssd_per_document(xs, dtp, A, B, C, self.D, self.chunk_size, cache.lengths, init)
                cache.state_cache.copy_(states)
            elif torch.is_grad_enabled() and xs.requires_grad and not (xs.is_cuda and xs.dtype == torch.bfloat16):
                # PyTorch formulation (CPU, fp32): the decay / mask tensors of the chunked scan ([b, h, chunks, L, L]
                # fp32) are rebuilt in backward instead of being kept for every layer. The native path keeps only
                # bf16 operands of its GEMMs and needs no recomputation.
                from torch.utils.checkpoint import checkpoint

                y, _ = checkpoint(ssd_chunked, xs, dtp, A, B, C, self.D, self.chunk_size, doc_start, init,
                                  use_reentrant=False)
            else:
                y, _ = ssd_chunked(xs, dtp, A, B, C, self.D, self.chunk_size, doc_start, init)
        else:
            y = selective_state_update(cache.state_cache, xs[0], dtp[0], A, B[0], C[0], self.D).unsqueeze(0)
        y = y.reshape(bsz, S, self.hidden_dim)
        y = self.ssm_norm(y * TF.silu(z))
        return self.out_proj(y)

    def reset_parameters(self, init_std, factor, init_args: InitArgs):
        in_std = init_std or (self.dim ** (-0.5))
        out_std = (init_std or (self.hidden_dim ** (-0.5))) / factor
        _trunc(self.in_proj.weight, in_std)
        _trunc(self.out_proj.weight, out_std)
        with torch.no_grad():
            if self.dt_bias is not None:
                self.dt_bias.uniform_(init_args.dt_min, init_args.dt_max)
                self.dt_bias.clamp_(min=init_args.dt_init_floor)
                self.dt_bias.copy_(self.dt_bias + torch.log(-torch.expm1(-self.dt_bias)))  # inverse softplus
            if self.conv_size is not None:
                _trunc(self.conv_weight, init_std or (self.conv_size ** (-0.5)))
            if self.learnable_init_states:
                self.init_states.zero_()
            self.A_log.uniform_(init_args.A_init_min, init_args.A_init_max)
            self.A_log.log_()
            if self.D is not None:
                self.D.fill_(1.0)
        self.ssm_norm.reset_parameters()


def _ssd_per_document(xs, dt, A, B, C, D, chunk, lengths, init):
    """Packed sequence [1, T, ...]: run the SSD on every document and collect the final states."""
    ys, states, off = [], [], 0
    for n in lengths.tolist():
        sl = slice(off, off + n)
        y, st = ssd_chunked(xs[:, sl], dt[:, sl], A, B[:, sl], C[:, sl], D, chunk, None, init)
        ys.append(y)
        states.append(st[0])
        off += n
    return torch.cat(ys, dim=1), torch.stack(states)


class MambaBlock(nn.Module):
    def __init__(self, args: BaseMambaArgs):
        super().__init__()
        self.ssm_norm = RMSNorm(args.dim, args.norm_eps)
        self.ssm = SSM(args.dim, 3 * args.dim, args.multiple_of, args.ffn_dim_multiplier, args.state_dim,
                       args.n_heads, args.n_groups, args.conv_size, args.dt_bias, args.D_has_head_dim,
                       args.learnable_init_states, chunk_size=args.ssm_chunk_size)

    def forward(self, x, doc_start=None, ssm_impl="ssm"):
        return x + self.ssm(self.ssm_norm(x), doc_start=doc_start, ssm_impl=ssm_impl)

    def init_weights(self, init_std=None, factor=1.0, init_args: InitArgs = InitArgs()):
        self.ssm_norm.reset_parameters()
        self.ssm.reset_parameters(init_std, factor, init_args)


class LMMamba(nn.Module):
    def __init__(self, args: LMMambaArgs):
        super().__init__()
        self.model_dim = self.dim = args.dim
        self.init_base_std, self.init_args = args.init_base_std, args.init_args
        self.init_std_factor = InitStdFactor(args.init_std_factor)
        self.layers = nn.ModuleList(MambaBlock(args) for _ in range(args.n_layers))
        self.weight_tying, self.loss_reduction, self.loss_chunk = args.weight_tying, args.loss_reduction, args.loss_chunk
        assert args.vocab_size > 0
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.output = TiedLinear(self.tok_embeddings) if args.weight_tying else Linear(args.dim, args.vocab_size)

    def forward(self, token_values, target=None, tok_idx=None, cu_seqlens=None, ssm_impl="ssm", doc_start=None,
                impl=None):
        if impl is not None:  # the generator's vocabulary: parallel | sequential
            ssm_impl = "ssm" if impl == "parallel" else "ssm_update"
        B, S = token_values.shape
        if doc_start is None and cu_seqlens is not None and ssm_impl == "ssm":
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
            h = layer(h, doc_start=doc_start, ssm_impl=ssm_impl)
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
            layer.init_weights(self.init_base_std, factor, self.init_args)


def get_num_flop_per_token(num_non_embed_params: int, n_layers: int, dim: int, seq_len: int) -> int:
    # the reference keeps the transformer's attention term for this model too (apps/mamba/mamba.py:24-34)
    return 6 * num_non_embed_params + 3.5 * (4 * n_layers * seq_len * dim // 2)


def build_fsdp_grouping_plan(model_args):
    plan = [("tok_embeddings", False)]
    plan += [(f"layers.{i}", False) for i in range(model_args.n_layers)]
    plan.append(("output", True))
    return plan
