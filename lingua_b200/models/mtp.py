"""Multi-token prediction: a shared Llama trunk with ``n_future_head`` independent vocabulary heads,
head i predicting token t + 1 + i (apps/mtp/transformer.py: LMMTPArgs :54, LMTransformer :67).

Training returns the list of per-head cross-entropies (their sum is optimised, each is logged).
The reference wraps every head in activation checkpointing so that only one [tokens, vocab]
logits tensor is alive at a time; the native path gets the same bound from the fused
linear + cross-entropy, which never holds more than ``loss_chunk`` rows of logits. Evaluation and
generation use head 0 only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from ..ops import fused
from .transformer import (BaseTransformer, BaseTransformerArgs, Linear, RMSNorm, _final_norm, _is_native, _trunc,
                          cross_entropy)


@dataclass
class LMMTPArgs(BaseTransformerArgs):
    seed: int = 42
    n_future_head: int = 1
    vocab_size: int = -1
    attn_impl: str = "sdpa"  # accepted for config compatibility
    mask: str = "causal"
    sliding_window: Optional[int] = None
    loss_chunk: int = 2048


class LMTransformer(BaseTransformer):
    def __init__(self, args: LMMTPArgs):
        super().__init__(args)
        self.sliding_window, self.mask, self.attn_impl = args.sliding_window, args.mask, args.attn_impl
        self.n_future_head, self.loss_chunk = args.n_future_head, args.loss_chunk
        assert self.n_future_head >= 1 and args.vocab_size > 0
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.norm = RMSNorm(args.dim, eps=args.norm_eps)
        self.heads = nn.ModuleList(Linear(args.dim, args.vocab_size) for _ in range(self.n_future_head))

    def _trunk(self, tokens, tok_idx, doc_start, doc_end):
        """Normalised trunk output, [B*S, dim] on the native path and [B, S, dim] otherwise."""
        B, S = tokens.shape
        window = self.sliding_window or 0
        cs = self.rope_embeddings()
        if _is_native(self.tok_embeddings.weight):
            eng = getattr(self, "_engine", None)
            pos = tok_idx.reshape(-1).int().contiguous() if tok_idx is not None else None
            ds = doc_start.reshape(-1).int().contiguous() if doc_start is not None else None
            de = doc_end.reshape(-1).int().contiguous() if doc_end is not None else None
            if eng is not None:
                eng.boundary("tok_embeddings")
            x = fused.EmbeddingFn.apply(tokens.reshape(-1), self.tok_embeddings.weight)
            pending = None
            for i, layer in enumerate(self.layers):
                if eng is not None:
                    x, pending = eng.boundary(f"layers.{i}", x, pending)
                x, pending = layer.forward_native(x, pending, cs, B, S, ds, de, window, pos, True)
            if eng is not None:
                eng.boundary("")
            return _final_norm(x, pending, self.norm)[0]
        h = self.tok_embeddings(tokens)
        for layer in self.layers:
            h = layer(h, cs, tok_idx, doc_start, window, True)
        return self.norm(h)

    def forward(self, token_values, target=None, tok_idx=None, doc_start=None, doc_end=None):
        """``target``: [B, S, n_future_head] in training (one column per head), [B, S] in eval mode."""
        B, S = token_values.shape
        y = self._trunk(token_values, tok_idx, doc_start, doc_end)
        native = _is_native(self.tok_embeddings.weight)
        if target is None:
            out = self.heads[0](y)
            return out.view(B, S, -1) if native else out
        heads = self.heads if self.training else self.heads[:1]
        losses: List[torch.Tensor] = []
        for i, head in enumerate(heads):
            tgt = target[..., i] if target.dim() == 3 else target
            if native:
                gs = getattr(self, "loss_grad_scale", None) if torch.is_grad_enabled() else None
                losses.append(fused.LinearCrossEntropyFn.apply(y, head.weight, tgt.reshape(-1), self.loss_chunk, gs))
            else:
                losses.append(cross_entropy(head(y), tgt))
        return losses if self.training else losses[0]

    def reset_parameters(self, init_std=None):
        super().reset_parameters()
        std = init_std or (self.dim ** (-0.5))
        self.norm.reset_parameters()
        _trunc(self.tok_embeddings.weight, std)
        for head in self.heads:
            _trunc(head.weight, std)

    def init_weights(self):
        self.reset_parameters()
        super().init_weights()


def build_fsdp_grouping_plan(model_args: LMMTPArgs):
    return [("tok_embeddings", False)] + [(f"layers.{i}", False) for i in range(model_args.n_layers)]
