"""Hierarchical byte-level U-Net language model ("AUNet").

Stage 0 runs on bytes. Each transition keeps only the positions that the data pipeline marked as
boundaries of the next level (words, word groups, ...), projects them to the next stage's width and
hands them to the next stage; the innermost stage is the trunk. On the way back every pooled vector is
repeated over the positions it covers and projected by a weight chosen by the distance to the boundary
(``IndexedMatMul``), added to the skip connection and refined by the stage's decoder.
Behaviour follows apps/aunet/hierarchical.py of the reference (args :33-50, estimators :95-190, stage :204-236,
transition :275-434, model :436-646, sharding plan :651-662).

What is different here: the pooling plan (gather indices, repeat indices, distances, group order of the
indexed projection) is computed once per forward for all levels from the level mask, before the first
stage runs, so that the only host synchronisation of a step (reading sixteen group sizes per level) happens
while the device is still busy with the previous step; stages whose head width is 128 run through the fused
native blocks, narrower heads are zero-padded to 128 for the flash-attention kernel."""
from __future__ import annotations

import math
from copy import deepcopy
from dataclasses import asdict, dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..metrics import get_num_params
from ..ops import functional as F
from ..ops.indexed_matmul import GroupPlan, IndexedMatMul, plan_groups
from .transformer import (BaseTransformer, BaseTransformerArgs, Linear, RMSNorm, _is_native, _trunc, cross_entropy,
                          get_num_flop_per_token)

MAX_POS = 16  # size of the weight bank of the indexed up-projection (distances are taken modulo this)


@dataclass
class CausalTransformerArgs(BaseTransformerArgs):
    sliding_window: Optional[int] = None


def _ffn_hidden(dim: int, mult: Optional[float], multiple_of: int) -> int:
    h = int(2 * (4 * dim) / 3)
    h = int(h * (mult if mult is not None else 1.0))
    return multiple_of * math.ceil(h / multiple_of)


def _stage_layers(layers: List[int]) -> List[int]:
    """Every stage but the trunk has an encoder and a decoder of ``layers[k]`` blocks each."""
    return [2 * l if k < len(layers) - 1 else l for k, l in enumerate(layers)]


def _block_params(dim: int, kv_ratio: float, ffn: int) -> float:
    return 2 * dim * dim + 2 * dim * dim * kv_ratio + 3 * dim * ffn


@dataclass
class HierarchicalArgs:
    dimensions: Optional[List[int]] = None
    head_dims: Optional[List[int]] = None
    layers: Optional[List[int]] = None
    sliding_windows: Optional[List[int]] = None
    max_seqlens: Optional[List[int]] = None
    residuals: Optional[List[bool]] = None
    block: BaseTransformerArgs = field(default_factory=BaseTransformerArgs)
    pooling_type: str = "simple_indexed_matmul"
    seed: int = 42
    vocab_size: int = -1
    lambda_level: float = 0.0
    norm_eps: float = 1e-5

    # ---- estimates that need no model instance (planning of batch size and throughput)
    def _kv_ratios(self) -> List[float]:
        out = []
        for d, hd in zip(self.dimensions, self.head_dims):
            heads = d / hd
            out.append((self.block.n_kv_heads or heads) / heads)
        return out

    def _linear_params(self, ratios: Optional[List[float]] = None) -> float:
        ratios = ratios or [1.0] * len(self.dimensions)
        total = 0.0
        for d, n, kv, r in zip(self.dimensions, _stage_layers(self.layers), self._kv_ratios(), ratios):
            total += n * r * _block_params(d, kv, _ffn_hidden(d, self.block.ffn_dim_multiplier, self.block.multiple_of))
        return total

    @property
    def estimated_non_embed_param_count(self) -> int:
        return int(self._linear_params())

    @property
    def estimated_param_count(self) -> int:
        return int(self._linear_params() + 2 * self.dimensions[0] * self.vocab_size)

    def _flops(self, seq_len: int, with_vocab: bool) -> float:
        seqlens = [seq_len] + list(self.max_seqlens[1:])
        ratios = [s / seq_len for s in seqlens]
        lin = self._linear_params(ratios) + (self.dimensions[0] * self.vocab_size if with_vocab else 0)
        windows = self.sliding_windows or seqlens
        attn = 0.0
        for d, s, w, n, r in zip(self.dimensions, seqlens, windows, _stage_layers(self.layers), ratios):
            w = min(s, w or s)
            attn += r * 6 * d * s * n * (w * (2 * s - w)) / (s * s)  # banded-causal share of the s x s scores
        return attn + 6 * lin

    def non_embed_flops_per_token(self, seq_len: int) -> float:
        return self._flops(seq_len, with_vocab=False)

    def flops_per_token(self, seq_len: int) -> float:
        return self._flops(seq_len, with_vocab=True)

    def tokens_per_second(self, seq_len: int, flops_per_second: float) -> float:
        return flops_per_second / self.flops_per_token(seq_len)

    def mem_usage(self, batch_size: int, seq_len: int) -> Tuple[float, float]:
        """(activation bytes with a 20 % margin, bytes of the vocabulary-sized tensors), bf16."""
        seqlens = [seq_len] + list(self.max_seqlens[1:])
        act = 0.0
        for d, n, s in zip(self.dimensions, _stage_layers(self.layers), seqlens):
            ffn = _ffn_hidden(d, self.block.ffn_dim_multiplier, self.block.multiple_of)
            act += 2 * (8 * d + 3 * ffn) * batch_size * s * n
        vocab = sum(2 * 2 * self.vocab_size * batch_size * s for s in seqlens)
        return act * 1.2, vocab

    def max_batch_size(self, max_mem_budget: float = 180e9, seq_len: int = 1024) -> int:
        act, vocab = self.mem_usage(1, seq_len)
        return math.floor(max_mem_budget / (act + vocab))


class CausalTransformer(BaseTransformer):
    """One stage: a stack of blocks with sliding-window causal attention over [B, S, dim] activations."""

    def __init__(self, args: CausalTransformerArgs):
        super().__init__(args)
        self.n_layers, self.sliding_window = args.n_layers, args.sliding_window
        self.head_dim = args.head_dim or args.dim // args.n_heads
        self.num_params = get_num_params(self)

    def forward(self, h: torch.Tensor, tok_idx: Optional[torch.Tensor] = None, engine=None, prefix: str = ""):
        B, S, D = h.shape
        cs = self.rope_embeddings()
        window = self.sliding_window or 0
        first = self.layers[0].attention
        if _is_native(first.wq.weight) and h.dtype == torch.bfloat16 and self.head_dim <= 128 \
                and self.head_dim % 8 == 0 and (first.kv_cache is None or self.head_dim == 128):
            x, pending = h.reshape(B * S, D), None
            pos = tok_idx.reshape(-1).int().contiguous() if tok_idx is not None else None
            for i, layer in enumerate(self.layers):
                if engine is not None:
                    x, pending = engine.boundary(f"{prefix}.layers.{i}", x, pending)
                x, pending = layer.forward_native(x, pending, cs, B, S, None, None, window, pos, True)
            return (x if pending is None else x + pending).view(B, S, D)
        for i, layer in enumerate(self.layers):
            if engine is not None:
                (h,) = engine.boundary(f"{prefix}.layers.{i}", h)
            h = layer(h, cs, tok_idx, None, window, True)
        return h

    def flops_per_token(self) -> float:
        span = min(self.max_seqlen, self.sliding_window or self.max_seqlen)
        return get_num_flop_per_token(self.num_params, self.n_layers, self.dim, span)


@dataclass
class LevelPlan:
    """Everything one transition needs, in the coordinates of its input stage."""
    mask: torch.Tensor  # [B, S_in] bool: positions that continue to the next stage
    idx: torch.Tensor  # [B, S_out]: kept positions in order, then filler positions up to S_out
    repeat_idx: Optional[torch.Tensor] = None  # [B, S_in]: which pooled position covers each input position
    position: Optional[torch.Tensor] = None  # [B, S_in]: distance to that pooled position, modulo MAX_POS
    groups: Optional[GroupPlan] = None  # row order of the indexed projection


def pool_indices(mask: torch.Tensor, numel: int) -> torch.Tensor:
    """First ``numel`` columns of the stable order that lists the True positions before the False ones
    (apps/aunet/hierarchical.py:259-273): exactly ``numel`` positions per row whatever the mask holds."""
    return (~mask).int().argsort(dim=1, stable=True)[:, :numel]


def make_level_plan(mask: torch.Tensor, s_in: int, s_out: int, repeat: bool, indexed: bool) -> LevelPlan:
    mask = mask[:, :s_in]
    idx = pool_indices(mask, s_out)
    plan = LevelPlan(mask=mask, idx=idx)
    if repeat:
        rep = mask.long().cumsum(1)
        rep = (rep - rep[:, :1]).clamp_(max=s_out - 1)
        here = torch.arange(s_in, device=mask.device).unsqueeze(0)
        plan.repeat_idx = rep
        plan.position = (here - idx.gather(1, rep)) % MAX_POS
        if indexed:
            plan.groups = plan_groups(plan.position, MAX_POS)
    return plan


def _gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return x.gather(1, idx.unsqueeze(-1).expand(-1, -1, x.shape[-1]))


class SimpleTransition(nn.Module):
    """Pooling (``down``) and un-pooling (``up``) between two stages.

    ``pooling_type`` flags: ``non_param`` replaces the two linear maps by feature interleaving / averaging,
    ``repeat`` upsamples by repeating the pooled vector (with a learned distance embedding) instead of
    scattering it back to the boundary positions only, ``indexed_matmul`` (implies repeat) adds the
    distance-indexed projection."""

    def __init__(self, seqlen_in: int, seqlen_out: int, dim_in: int, dim_out: int, eps_norm: float,
                 non_parametric: bool = False, indexed_matmul: bool = False, repeat: bool = False):
        super().__init__()
        self.seqlen_in, self.seqlen_out, self.dim_in, self.dim_out = seqlen_in, seqlen_out, dim_in, dim_out
        self.non_parametric, self.indexed_matmul = non_parametric, indexed_matmul
        self.repeat = repeat or indexed_matmul
        self.max_pos = MAX_POS
        if not non_parametric:
            self.down_norm = RMSNorm(dim_in, eps=eps_norm)
            self.trans_down = Linear(dim_in, dim_out)
            self.up_norm = RMSNorm(dim_out, eps=eps_norm)
            self.trans_up = Linear(dim_out, dim_in)
        else:
            assert dim_out % dim_in == 0, f"dim_out {dim_out} must be a multiple of dim_in {dim_in}"
            self.features_ratio = r = dim_out // dim_in
            self.register_buffer("features_weight", (torch.arange(1, r + 1) / r).repeat(dim_in), persistent=True)
            self.register_buffer("expand_idx", torch.arange(dim_in).repeat_interleave(r), persistent=True)
        if indexed_matmul:
            self.indexed_linear = IndexedMatMul(self.max_pos, dim_out, dim_in)
            if non_parametric:
                self.indexed_norm = RMSNorm(dim_out, eps=eps_norm)
        elif self.repeat:
            self.pos_encoding = nn.Embedding(self.max_pos, dim_out)

    # ---- the two feature maps
    def _down_map(self, x):
        if not self.non_parametric:
            return self.trans_down(self.down_norm(x))
        if self.dim_in == self.dim_out:
            return x
        w = self.features_weight.to(x.dtype)
        wide = x[..., self.expand_idx]  # every feature repeated r times, blended with its left neighbour
        return wide * w + wide.roll(self.features_ratio, -1) * (1 - w)

    def _up_map(self, x):
        if not self.non_parametric:
            return self.trans_up(x)
        if self.dim_in == self.dim_out:
            return x
        return x.unflatten(-1, (self.dim_in, self.features_ratio)).mean(-1)

    def down(self, x: torch.Tensor, plan: LevelPlan) -> torch.Tensor:
        if plan.idx.numel() == 0:  # generation: nothing crosses this boundary in this step
            return x.new_zeros(x.shape[0], 0, self.dim_out)
        return self._down_map(_gather_rows(x, plan.idx))

    def up(self, x: torch.Tensor, res: torch.Tensor, plan: LevelPlan) -> torch.Tensor:
        if hasattr(self, "up_norm"):
            x = self.up_norm(x)
        if self.repeat:
            rep = plan.repeat_idx
            if self.indexed_matmul:
                # the position-independent map commutes with the repeat: apply it to the pooled rows, then
                # repeat its narrow output; the indexed map reads the pooled rows through the repeat index
                xi = self.indexed_norm(x) if hasattr(self, "indexed_norm") else x
                rows = rep + torch.arange(x.shape[0], device=x.device).unsqueeze(1) * x.shape[1]
                return _gather_rows(self._up_map(x), rep) + self.indexed_linear(xi, plan.position, plan.groups, rows)
            return self._up_map(_gather_rows(x, rep) + self.pos_encoding(plan.position).to(x.dtype))
        keep = plan.mask.gather(1, plan.idx).to(x.dtype).unsqueeze(-1)  # filler positions contribute nothing
        out = torch.zeros_like(res)
        return out.scatter(1, plan.idx.unsqueeze(-1).expand(-1, -1, self.dim_in), keep * self._up_map(x))

    def reset_parameters(self):
        for name, std in (("trans_down", self.dim_in ** -0.5), ("trans_up", self.dim_out ** -0.5)):
            if hasattr(self, name):
                _trunc(getattr(self, name).weight, std)
        for name in ("down_norm", "up_norm", "indexed_norm", "indexed_linear", "pos_encoding"):
            if hasattr(self, name):
                getattr(self, name).reset_parameters()
        if self.non_parametric:
            r = self.features_ratio
            self.features_weight.copy_((torch.arange(1, r + 1) / r).repeat(self.dim_in))
            self.expand_idx.copy_(torch.arange(self.dim_in).repeat_interleave(r))


class HierarchicalTransformer(nn.Module):
    """encoders[0] -> pool -> encoders[1] -> ... -> trunk -> ... -> unpool -> decoders[0] -> vocabulary head."""

    def __init__(self, args: HierarchicalArgs):
        super().__init__()
        n = len(args.dimensions)
        assert len(args.head_dims) == n and len(args.layers) == n and len(args.max_seqlens) == n
        assert args.pooling_type.startswith("simple"), f"Pooling type {args.pooling_type} not supported"
        self.seed, self.dim, self.vocab_size = args.seed, args.dimensions[0], args.vocab_size
        self.lambda_level, self.pooling_type = args.lambda_level, args.pooling_type
        self.tok_embeddings = nn.Embedding(args.vocab_size, self.dim)
        self.vocab_norm = RMSNorm(self.dim, eps=args.norm_eps)
        self.vocab = Linear(self.dim, args.vocab_size)
        if self.lambda_level > 0:  # auxiliary head: predicts the pooling level of the next byte
            self.level_mask_norm = RMSNorm(2 * self.dim, eps=args.norm_eps)
            self.level_mask = Linear(2 * self.dim, n)
        self.adding_residuals = list(args.residuals or [True] * (n - 1))
        windows = args.sliding_windows or [None] * n
        kind = args.pooling_type.lower()
        flags = dict(non_parametric="non_param" in kind, repeat="repeat" in kind, indexed_matmul="indexed_matmul" in kind)

        def stage(k: int) -> CausalTransformer:
            a = CausalTransformerArgs(**asdict(deepcopy(args.block)))
            a.dim, a.head_dim, a.n_heads, a.n_layers = args.dimensions[k], args.head_dims[k], None, args.layers[k]
            a.sliding_window, a.max_seqlen = windows[k], args.max_seqlens[k]
            return CausalTransformer(a)

        self.encoders, self.decoders, self.transitions = nn.ModuleList(), nn.ModuleList(), nn.ModuleList()
        for k in range(n - 1):
            self.encoders.append(stage(k))
            self.transitions.append(SimpleTransition(args.max_seqlens[k], args.max_seqlens[k + 1], args.dimensions[k],
                                                     args.dimensions[k + 1], args.block.norm_eps, **flags))
            self.decoders.append(stage(k))
        self.trunk = stage(n - 1)
        self.num_params = [get_num_params(e) for e in self.encoders] + [get_num_params(self.trunk)]

    # ---- pooling plan
    @torch.no_grad()
    def get_pool_mask(self, level_mask: torch.Tensor, max_seqlen: Optional[List[int]] = None, return_idcs: bool = True,
                      force_first: bool = False):
        """Per level: the mask of positions that go one stage deeper, written in the coordinates of the
        stage they leave (its positions packed to the front of the row), their column indices, and how many
        there are. ``max_seqlen[i + 1]`` caps the positions that level i may pass on
        (apps/aunet/hierarchical.py:582-608). The input is not modified."""
        n = len(self.encoders)
        if force_first:
            level_mask = level_mask.clone()
            level_mask[:, 0] = n
        cols = torch.arange(level_mask.shape[1], device=level_mask.device).unsqueeze(0)
        remaining = torch.ones_like(level_mask, dtype=torch.bool)
        masks, idcs, nb_toks = [], [], []
        for i in range(n):
            m = level_mask > i
            if max_seqlen is not None:
                m = m & (m.long().cumsum(1) <= max_seqlen[i + 1])
            order = (~remaining).int().argsort(dim=1, stable=True)  # this stage's positions first, in order
            compact = m.gather(1, order) & (cols < remaining.sum(1, keepdim=True))
            masks.append(compact)
            nb_toks.append(compact.sum())
            if return_idcs:
                idcs.append(compact.nonzero(as_tuple=True)[1])
            remaining = m & remaining
        return masks, idcs, nb_toks

    def plan_levels(self, level_mask: torch.Tensor, seq_len: int):
        caps = [seq_len]  # a stage is never longer than the one above it
        for stage in (*self.encoders[1:], self.trunk):
            caps.append(min(stage.max_seqlen, caps[-1]))
        masks, _, nb_toks = self.get_pool_mask(level_mask, caps, return_idcs=False, force_first=True)
        plans = [make_level_plan(m, caps[i], caps[i + 1], t.repeat, t.indexed_matmul)
                 for i, (m, t) in enumerate(zip(masks, self.transitions))]
        return plans, nb_toks

    def features(self, token_values: torch.Tensor, level_mask: torch.Tensor):
        """Final byte-level hidden states [B, S, dim] and the number of positions that reached each stage."""
        eng = getattr(self, "_engine", None)
        plans, nb_toks = self.plan_levels(level_mask, token_values.shape[1])
        if eng is not None:
            eng.boundary("")  # embeddings, transitions and heads live in the root group
        x = self.tok_embeddings(token_values)
        skips = []
        for k, (enc, trans, plan) in enumerate(zip(self.encoders, self.transitions, plans)):
            x = enc(x, engine=eng, prefix=f"encoders.{k}")
            skips.append(x)
            x = trans.down(x, plan)
        x = self.trunk(x, engine=eng, prefix="trunk")
        for k in reversed(range(len(self.decoders))):
            x = self.transitions[k].up(x, skips[k], plans[k])
            if self.adding_residuals[k]:
                x = skips[k] + x
            x = self.decoders[k](x, engine=eng, prefix=f"decoders.{k}")
        return x, nb_toks

    def forward(self, token_values: torch.Tensor, level_mask: torch.Tensor, target: Optional[torch.Tensor] = None,
                target_level_mask: Optional[torch.Tensor] = None):
        """With targets: (next-byte loss, level-prediction loss or None, positions per stage); without: logits."""
        x, nb_toks = self.features(token_values, level_mask)
        logits = self.vocab(self.vocab_norm(x))
        if target is None:
            return logits
        loss = cross_entropy(logits, target)
        mask_loss = None
        mask_logits = self._level_mask_logits(x, target)
        if mask_logits is not None and target_level_mask is not None:
            mask_loss = cross_entropy(mask_logits, target_level_mask.clamp(max=mask_logits.shape[-1] - 1))
        return loss, mask_loss, nb_toks

    def _level_mask_logits(self, features: torch.Tensor, target: torch.Tensor) -> Optional[torch.Tensor]:
        if self.lambda_level <= 0:
            return None
        both = torch.cat([features, self.tok_embeddings(target).to(features.dtype)], dim=-1)
        return self.level_mask(self.level_mask_norm(both))

    def flops_per_token(self) -> float:
        s0 = self.encoders[0].max_seqlen if len(self.encoders) else self.trunk.max_seqlen
        total = self.trunk.max_seqlen / s0 * self.trunk.flops_per_token()
        for enc, dec in zip(self.encoders, self.decoders):
            total += enc.max_seqlen / s0 * (enc.flops_per_token() + dec.flops_per_token())
        return total

    def reset_parameters(self, init_std=None):
        std = init_std or (self.dim ** (-0.5))
        _trunc(self.tok_embeddings.weight, std)
        _trunc(self.vocab.weight, std)
        self.vocab_norm.reset_parameters()
        if self.lambda_level > 0:
            self.level_mask_norm.reset_parameters()
            _trunc(self.level_mask.weight, (2 * self.dim) ** (-0.5))
        for t in self.transitions:
            t.reset_parameters()

    def init_weights(self):
        self.reset_parameters()
        for stage in (*self.encoders, *self.decoders, self.trunk):
            stage.init_weights()


def get_no_recompute_ops():
    return None


def build_fsdp_grouping_plan(model_args: HierarchicalArgs):
    """One shard group per block, encoder and decoder blocks of a level interleaved, then the trunk."""
    plan = []
    for k, n in enumerate(model_args.layers[:-1]):
        for i in range(n):
            plan.append((f"encoders.{k}.layers.{i}", False))
            plan.append((f"decoders.{k}.layers.{i}", False))
    plan.extend((f"trunk.layers.{i}", False) for i in range(model_args.layers[-1]))
    return plan
