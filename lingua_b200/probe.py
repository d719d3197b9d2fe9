"""Activation / weight / gradient statistics ("probe") for debugging training dynamics.

``with AutoProbeD(model, "probe.jsonl") as probe: loss = model(x, y); loss.backward()`` appends one
JSON line ``{"data": {"<module>::<what>": stats}, "meta": probe.metadata, "version": 2,
"quantiles": QUANTILES}`` with, for every linear layer, ``in / w / out`` and their gradients
``in.g / w.g / out.g``, for every RMSNorm the residual stream ``resid``, and for every attention
``attn_logits`` and ``attn_entropy`` computed on a subset of at most 128 queries - the schema of
lingua/probe.py (QUANTILES :75, _get_stats :87, AutoProbeD :281, JSONL dump :322-335), which
apps/plots/probe_animation.py consumes.

The reference intercepts aten ops with a TorchDispatchMode; the native path here never calls
aten matmuls, so the fused autograd functions report to an observer instead
(``lingua_b200.ops.fused.set_observer``), and the PyTorch reference path is covered by module
hooks. Statistics use ordinary PyTorch reductions: this is a cold path (every ``probe_freq`` steps).
"""
from __future__ import annotations

import json
import math
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, Optional, Sequence

import torch
import torch.nn as nn

from .ops import fused

QUANTILES = [
    0.0000001, 0.000001, 0.00001, 0.0001, 0.001, 0.01, 0.05, 0.1, 0.3, 0.5, 0.7, 0.9, 0.95,
    0.99, 0.999, 0.9999, 0.99999, 0.999999, 0.9999999,
]
MAX_ATTN_QUERIES = 128


def _get_stats(x_: torch.Tensor, remove_inf: bool = False) -> Dict[str, Any]:
    if x_.dtype not in (torch.float, torch.double, torch.float16, torch.bfloat16):
        return {}
    x = x_.detach().flatten()
    if remove_inf:
        x = x[x.abs() < float("inf")]
    if x.dtype is not torch.double:
        x = x.float()
    mean, std = x.mean(), x.std()
    q = torch.tensor(QUANTILES, device=x.device, dtype=x.dtype)
    z = (x - mean) / std
    return {
        "shape": tuple(x_.shape), "mean": mean, "std": std,
        "skew": (z ** 3).double().mean(), "kurtosis": (z ** 4).double().mean(),
        "abs.mean": x.abs().mean(), "max": x.max(), "min": x.min(),
        "quantiles": torch.quantile(x[: 2 ** 24], q),  # torch.quantile accepts at most 2^24 elements
    }


def _to_python(v):
    if isinstance(v, torch.Tensor):
        return v.tolist() if v.numel() > 1 else v.item()
    if isinstance(v, dict):
        return {k: _to_python(x) for k, x in v.items()}
    if isinstance(v, tuple):
        return list(v)
    return v


def attention_stats(q: torch.Tensor, k: torch.Tensor, causal: bool = True,
                    doc_start: Optional[torch.Tensor] = None) -> Dict[str, Dict[str, Any]]:
    """Logit and entropy statistics of softmax(q k^T / sqrt(d)) for evenly spaced queries.
    q: [B, S, H, Dh], k: [B, S, Hkv, Dh]."""
    B, S, H, Dh = q.shape
    Hkv = k.shape[2]
    n = min(S, MAX_ATTN_QUERIES)
    qi = torch.linspace(0, S - 1, n, device=q.device).long()
    qs = q[:, qi].float().permute(0, 2, 1, 3)  # B H n Dh
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    logits = torch.matmul(qs, kf.transpose(-1, -2)) / math.sqrt(Dh)  # B H n S
    kv = torch.arange(S, device=q.device).view(1, 1, 1, S)
    mask = torch.ones(1, 1, n, S, dtype=torch.bool, device=q.device)
    if causal:
        mask = mask & (kv <= qi.view(1, 1, n, 1))
    if doc_start is not None:
        mask = mask & (kv >= doc_start.view(B, S)[:, qi].view(B, 1, n, 1).long())
    logits = logits.masked_fill(~mask, float("-inf"))
    p = torch.softmax(logits, dim=-1)
    ent = -(p * torch.where(p > 0, p.log(), torch.zeros_like(p))).sum(-1)
    return {"attn_logits": _get_stats(logits, remove_inf=True), "attn_entropy": _get_stats(ent)}


class AutoProbeD:
    def __init__(self, module: nn.Module, write_file: Optional[str] = None) -> None:
        self.module = module
        self.write_file = Path(write_file) if write_file is not None else None
        self.store: Dict[str, Dict[str, Any]] = {}
        self.count_per_path: Dict[str, int] = defaultdict(int)
        self.metadata: Any = None
        self.enabled = False
        self._handles = []
        self._name_of: Dict[int, str] = {}

    # ------------------------------------------------------------------ observer API (native path)
    def _path(self, t: torch.Tensor) -> str:
        name = self._name_of.get(id(t), "unknown")
        return name[: -len(".weight")] if name.endswith(".weight") else name

    def _put(self, path: str, what: str, stats: Dict[str, Any]) -> None:
        key = f"{path}::{what}"
        c = self.count_per_path[key]
        self.count_per_path[key] += 1
        self.store[key if c == 0 else f"{key}.{c}"] = stats

    def linear_fwd(self, ws: Sequence[torch.Tensor], x: torch.Tensor, out: torch.Tensor) -> None:
        r0 = 0
        for w in ws:
            p = self._path(w)
            self._put(p, "in", _get_stats(x))
            self._put(p, "w", _get_stats(w))
            self._put(p, "out", _get_stats(out[..., r0:r0 + w.shape[0]]))
            r0 += w.shape[0]

    def linear_bwd(self, ws, dy, dx, dws) -> None:
        r0 = 0
        for w, dw in zip(ws, dws):
            p = self._path(w)
            self._put(p, "out.g", _get_stats(dy[..., r0:r0 + w.shape[0]]))
            if dx is not None:
                self._put(p, "in.g", _get_stats(dx))
            g = dw if dw is not None else getattr(w, "main_grad", None)
            if g is not None:
                self._put(p, "w.g", _get_stats(g))
            r0 += w.shape[0]

    def resid(self, norm_w: torch.Tensor, h: torch.Tensor) -> None:
        self._put(self._path(norm_w), "resid", _get_stats(h))

    def attention(self, anchor_w: torch.Tensor, q, k, causal, doc_start) -> None:
        path = self._path(anchor_w).rsplit(".", 1)[0]
        for what, st in attention_stats(q, k, causal, doc_start).items():
            self._put(path, what, st)

    # ------------------------------------------------------------------ module hooks (reference path)
    def _install_hooks(self) -> None:
        from .models.transformer import Linear, RMSNorm

        for name, mod in self.module.named_modules():
            if isinstance(mod, (Linear, nn.Linear)) and not (mod.weight.is_cuda and mod.weight.dtype == torch.bfloat16):
                def fwd(m, args, out, name=name):
                    self._put(name, "in", _get_stats(args[0]))
                    self._put(name, "w", _get_stats(m.weight))
                    self._put(name, "out", _get_stats(out))

                def bwd(m, gin, gout, name=name):
                    if gout[0] is not None:
                        self._put(name, "out.g", _get_stats(gout[0]))
                    if gin[0] is not None:
                        self._put(name, "in.g", _get_stats(gin[0]))

                self._handles.append(mod.register_forward_hook(fwd))
                self._handles.append(mod.register_full_backward_hook(bwd))
            elif isinstance(mod, RMSNorm) and not (mod.weight.is_cuda and mod.weight.dtype == torch.bfloat16):
                self._handles.append(mod.register_forward_hook(
                    lambda m, args, out, name=name: self._put(name, "resid", _get_stats(args[0]))))

    def _collect_reference_weight_grads(self) -> None:
        for name, p in self.module.named_parameters():
            if p.grad is not None and p.dim() == 2 and not p.is_cuda:
                self._put(name[: -len(".weight")] if name.endswith(".weight") else name, "w.g", _get_stats(p.grad))

    # ------------------------------------------------------------------ context manager
    def __enter__(self):
        assert not self.enabled, "Entered probe twice"
        self._name_of = {id(p): n for n, p in self.module.named_parameters()}
        self._install_hooks()
        fused.set_observer(self)
        self.enabled = True
        return self

    def __exit__(self, *args) -> None:
        assert self.enabled, "Exiting probe without entering it"
        fused.set_observer(None)
        self._collect_reference_weight_grads()
        for h in self._handles:
            h.remove()
        self._handles.clear()
        self._flush_and_clear()
        self.enabled = False

    def _flush_and_clear(self) -> None:
        if self.write_file is not None:
            self.write_file.parent.mkdir(parents=True, exist_ok=True)
            with self.write_file.open("a") as fd:
                json.dump({"data": _to_python(self.store), "meta": self.metadata, "version": 2,
                           "quantiles": QUANTILES}, fd)
                fd.write("\n")
        self.store.clear()
        self.count_per_path.clear()
