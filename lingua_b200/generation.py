"""Packed-prompt generation with a fixed-size KV cache.

Behaviour of apps/main/generate.py (sample_top_p :30, sample_top_k :40, sample_tokens :49,
pack_prompts :66, batch_prompts :79, KVCache :104, PackedCausalTransformerGenerator :140):
prompts are concatenated into one packed sequence, each document gets ``len + max_gen_len``
consecutive cache slots, prefill attends block-causally inside each document, and decoding
advances every document by one token per step. ``generate`` returns the decoded texts, the
per-token log-likelihood of every prompt and whether each prompt token was the greedy choice.

B200-first differences: prefill runs the flash-attention kernel with per-token document bounds
(no block-mask construction), and a decode step runs one kernel per layer that appends the new
K/V to the cache and attends to the document's own cache span (no dense (n_seqs x cache) mask).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from .checkpoint import CONSOLIDATE_NAME
from .config import dataclass_from_dict, load_yaml
from .models.transformer import Attention, LMTransformer, LMTransformerArgs
from .ops import _lib
from .ops.attention import flash_fwd
from .tokenizer import Tokenizer, build_tokenizer


def sample_top_p(probs: torch.Tensor, p: float) -> torch.Tensor:
    """Nucleus sampling: keep the smallest set of tokens whose mass exceeds p."""
    sorted_p, idx = torch.sort(probs, dim=-1, descending=True)
    cum = torch.cumsum(sorted_p, dim=-1)
    sorted_p[cum - sorted_p > p] = 0.0
    choice = torch.multinomial(sorted_p, num_samples=1)
    return torch.gather(idx, -1, choice)


def sample_top_k(probs: torch.Tensor, k: int) -> torch.Tensor:
    top, _ = torch.topk(probs, k)
    probs[probs < top[:, [-1]]] = 0.0
    probs.div_(probs.sum(dim=-1, keepdim=True))
    return torch.multinomial(probs, num_samples=1)


def sample_tokens(logits, temperature=0.0, top_p=None, top_k=None):
    shape = logits.shape
    logits = logits.flatten(end_dim=-2)
    if temperature > 0.0:
        probs = torch.softmax(logits.float() / temperature, dim=-1)
        if top_p is not None:
            nxt = sample_top_p(probs, top_p)
        elif top_k is not None:
            nxt = sample_top_k(probs, top_k)
        else:
            nxt = torch.multinomial(probs, num_samples=1)
    else:
        nxt = torch.argmax(logits, dim=-1)
    return nxt.view(shape[:-1])


def pack_prompts(prompts: List[List[int]]):
    lengths = torch.tensor([len(p) for p in prompts], dtype=torch.long)
    return torch.cat([torch.tensor(p, dtype=torch.long) for p in prompts]), lengths


def batch_prompts(prompts, max_elements, lengths=None):
    """Greedy grouping of prompts so that each group's total (padded) length fits the cache."""
    batches, cur, count = [], [], 0
    for i, p in enumerate(prompts):
        size = len(p) if lengths is None else lengths[i]
        if count + size <= max_elements:
            cur.append(p)
            count += size
        else:
            if cur:
                batches.append(cur)
            cur, count = [p], size
    if cur:
        batches.append(cur)
    return batches


def lengths_to_start_ids(lengths: torch.Tensor) -> torch.Tensor:
    return torch.cumsum(lengths, 0) - lengths


def lengths_to_local_ids(lengths: torch.Tensor):
    """(document id, position inside the document) of every token of a packed sequence."""
    n = lengths.numel()
    doc_id = torch.repeat_interleave(torch.arange(n, device=lengths.device), lengths)
    tok_id = torch.arange(int(lengths.sum()), device=lengths.device) - lengths_to_start_ids(lengths)[doc_id]
    return doc_id, tok_id


class CachePlan:
    """What the current forward pass does with the caches; shared by all layers."""

    def __init__(self):
        self.mode = "prefill"
        self.slots = None  # prefill: cache slot of every packed token
        self.doc_start = None  # prefill: [1, T] int32, in packed-token coordinates
        self.start = None  # decode: first cache slot of every sequence (int32)
        self.len = None  # decode: visible keys per sequence, current token included (int32)
        self.window = 0  # prefill: sliding-window width (0 = none); decode callers shrink start / len instead


class KVCache(nn.Module):
    def __init__(self, max_tokens, n_kv_heads, head_dim, dtype, device, plan: CachePlan):
        super().__init__()
        self.register_buffer("k_cache", torch.zeros(max_tokens, n_kv_heads, head_dim, dtype=dtype, device=device))
        self.register_buffer("v_cache", torch.zeros(max_tokens, n_kv_heads, head_dim, dtype=dtype, device=device))
        self.plan = plan

    # ---- native path: q/k/v are [T, heads, Dh] bf16 views of the rotated QKV projection
    def native_attention(self, q, k, v):
        pl = self.plan
        T, H, Dh = q.shape
        if pl.mode == "prefill":
            self.k_cache.index_copy_(0, pl.slots, k)
            self.v_cache.index_copy_(0, pl.slots, v)
            o, _ = flash_fwd(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), True, pl.doc_start, pl.window)
            return o.view(T, H * Dh)
        out = torch.empty(T, H, Dh, dtype=q.dtype, device=q.device)
        rc = _lib.load().lb_decode_attn(q.data_ptr(), k.data_ptr(), v.data_ptr(), self.k_cache.data_ptr(),
                                        self.v_cache.data_ptr(), pl.start.data_ptr(), pl.len.data_ptr(),
                                        out.data_ptr(), T, H, k.shape[1], Dh, q.stride(0), k.stride(0),
                                        1.0 / math.sqrt(Dh), _lib.stream_ptr())
        _lib.check(rc, "lb_decode_attn")
        return out.view(T, H * Dh)

    # ---- reference path: q/k/v are [1, T, heads, Dh]
    def attend(self, q, k, v, tok_idx=None):
        from .models.transformer import _attention_flash_padded, _attention_torch

        pl = self.plan
        if pl.mode == "prefill":
            self.k_cache.index_copy_(0, pl.slots, k[0].to(self.k_cache.dtype))
            self.v_cache.index_copy_(0, pl.slots, v[0].to(self.v_cache.dtype))
            if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] <= 128:
                return _attention_flash_padded(q, k, v, True, pl.window, pl.doc_start)
            return _attention_torch(q, k, v, True, pl.doc_start, pl.window)
        n = q.shape[1]
        slot = (pl.start + pl.len - 1).long()
        self.k_cache.index_copy_(0, slot, k[0].to(self.k_cache.dtype))
        self.v_cache.index_copy_(0, slot, v[0].to(self.v_cache.dtype))
        H, Hkv = q.shape[2], k.shape[2]
        pos = torch.arange(self.k_cache.shape[0], device=q.device).view(1, -1)
        mask = (pos >= pl.start.view(-1, 1)) & (pos < (pl.start + pl.len).view(-1, 1))  # [n, slots]
        kc = self.k_cache.float().repeat_interleave(H // Hkv, dim=1)  # [slots, H, Dh]
        vc = self.v_cache.float().repeat_interleave(H // Hkv, dim=1)
        s = torch.einsum("nhd,shd->nhs", q[0].float(), kc) / math.sqrt(q.shape[-1])
        s = s.masked_fill(~mask.view(n, 1, -1), float("-inf"))
        o = torch.einsum("nhs,shd->nhd", torch.softmax(s, dim=-1), vc)
        return o.to(q.dtype).unsqueeze(0)


@dataclass
class PackedCausalTransformerGeneratorArgs:
    temperature: float = 0.0
    top_p: Optional[float] = None
    top_k: Optional[float] = None
    max_gen_len: int = 512  # tokens generated per prompt
    max_tokens: int = 1024  # cache slots = upper bound on sum(prompt + generated) per batch
    max_prompt_len: Optional[int] = None
    until: List[str] = field(default_factory=list)
    compile_prefilling: bool = False  # accepted for config compatibility
    reduce_generation_overhead: bool = False  # replay the decode step as a CUDA graph (launch-bound otherwise)
    show_progress: bool = False
    dtype: Optional[str] = "bf16"
    device: Optional[str] = "cuda"


class PackedCausalTransformerGenerator:
    def __init__(self, cfg: PackedCausalTransformerGeneratorArgs, model: nn.Module, tokenizer: Tokenizer):
        self.model, self.tokenizer = model, tokenizer
        self.temperature, self.top_p, self.top_k = cfg.temperature, cfg.top_p, cfg.top_k
        self.max_gen_len, self.max_tokens, self.max_prompt_len = cfg.max_gen_len, cfg.max_tokens, cfg.max_prompt_len
        self.until = cfg.until
        self.max_until_size = max(len(e) for e in self.until) if self.until else 1
        self.device = cfg.device if (cfg.device != "cuda" or torch.cuda.is_available()) else "cpu"
        self.show_progress = cfg.show_progress
        self.dtype = dict(fp32=torch.float32, bf16=torch.bfloat16)[cfg.dtype]
        self.plan = CachePlan()
        self.padded_doc_start = None
        self.current_tok_id = None
        # decode step as a CUDA graph (the reference gets the same effect from torch.compile's
        # "reduce-overhead" mode, apps/main/generate.py:175-180)
        self.use_graph = bool(cfg.reduce_generation_overhead)
        self._graph = None
        self._eager_steps = 0

    # ---- cache management (overridden by the state-space / recurrent generators)
    def clear_cache(self):
        for module in self.model.modules():
            if isinstance(module, Attention):
                if getattr(module, "kv_cache", None) is None:
                    p = next(module.parameters())
                    module.kv_cache = KVCache(self.max_tokens, module.n_kv_heads, module.head_dim, p.dtype,
                                              p.device, self.plan)
                module.kv_cache.plan = self.plan

    def release_cache(self):
        for module in self.model.modules():
            if isinstance(module, Attention):
                module.kv_cache = None

    def setup_prefilling(self, lengths: torch.Tensor):
        padded = lengths + self.max_gen_len
        max_tokens = self.max_tokens or int(padded.sum())
        assert int(padded.sum()) <= max_tokens, "batch does not fit the cache"
        self.padded_doc_start = lengths_to_start_ids(padded)
        doc_id, tok_id = lengths_to_local_ids(lengths)
        self.clear_cache()
        pl = self.plan
        pl.mode = "prefill"
        pl.slots = self.padded_doc_start[doc_id] + tok_id
        pl.doc_start = lengths_to_start_ids(lengths)[doc_id].int().view(1, -1).contiguous()
        self.prefill_tok_id = tok_id

    def setup_generation(self, lengths: torch.Tensor):
        pl = self.plan
        pl.mode = "decode"
        pl.start = self.padded_doc_start.int().contiguous()
        self.current_tok_id = lengths.clone()
        pl.len = (self.current_tok_id + 1).int().contiguous()
        self._graph, self._eager_steps = None, 0  # new cache plan tensors: a captured step is stale

    def prefill(self, tokens: torch.Tensor, lengths: torch.Tensor):
        self.setup_prefilling(lengths)
        out = self.model(tokens, tok_idx=self.prefill_tok_id.view(1, -1))
        self.setup_generation(lengths)
        return out

    def generate_next_token(self, current_token: torch.Tensor):
        if self.use_graph and current_token.is_cuda:
            return self._graphed_next_token(current_token)
        self.plan.len = (self.current_tok_id + 1).int().contiguous()
        out = self.model(current_token, tok_idx=self.current_tok_id.view(1, -1))
        self.current_tok_id += 1
        return out

    def _graphed_next_token(self, current_token: torch.Tensor):
        """Two eager steps (lazy initialisation of kernels and allocator), then the step is captured once with
        static input / position / length tensors and replayed; the returned logits live in the graph's pool."""
        if self._graph is None:
            if self._eager_steps < 2:
                self._eager_steps += 1
                self.plan.len = (self.current_tok_id + 1).int().contiguous()
                out = self.model(current_token, tok_idx=self.current_tok_id.view(1, -1))
                self.current_tok_id += 1
                return out
            self._g_token = current_token.clone()
            self.plan.len = (self.current_tok_id + 1).int().contiguous()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                self.plan.len.copy_((self.current_tok_id + 1).int())
                out = self.model(self._g_token, tok_idx=self.current_tok_id.view(1, -1))
                self.current_tok_id += 1
            self._graph, self._g_out = graph, out
        self._g_token.copy_(current_token)
        self._graph.replay()
        return self._g_out

    @torch.inference_mode()
    def generate(self, prompts: List[str]):
        prompts = [self.tokenizer.encode(p, add_bos=True, add_eos=False) for p in prompts]
        max_seqlen = getattr(self.model, "max_seqlen", self.max_tokens)
        max_prompt_len = self.max_prompt_len or min(max_seqlen - self.max_gen_len, self.max_tokens - self.max_gen_len)
        prompts = [p[-max_prompt_len:] for p in prompts]
        padded_lengths = [len(p) + self.max_gen_len for p in prompts]
        generation, loglikelihood, greedy = [], [], []
        batches = batch_prompts(prompts, self.max_tokens, lengths=padded_lengths)
        if self.show_progress:
            from tqdm import tqdm

            batches = tqdm(batches)
        for batch in batches:
            n_seqs = len(batch)
            generated = [[] for _ in range(n_seqs)]
            is_done = [False] * n_seqs
            packed, lengths = pack_prompts(batch)
            packed, lengths = packed.to(self.device), lengths.to(self.device)
            prompt_logits = self.prefill(packed.unsqueeze(0), lengths)
            all_tokens = sample_tokens(prompt_logits, self.temperature, self.top_p, self.top_k)
            start_token = all_tokens[:, lengths.cumsum(0) - 1]
            for i, tok in enumerate(start_token.squeeze(0).tolist()):
                generated[i].append(tok)
            current = start_token
            for _ in range(1, self.max_gen_len):
                logits = self.generate_next_token(current)
                nxt = sample_tokens(logits.clone(), self.temperature, self.top_p, self.top_k)
                for i, tok in enumerate(nxt.squeeze(0).tolist()):
                    if not is_done[i]:
                        generated[i].append(tok)
                        is_done[i] = tok == self.tokenizer.eos_id
                        if self.until and not is_done[i]:
                            tail = self.tokenizer.decode(generated[i][-self.max_until_size:])
                            is_done[i] = any(e in tail for e in self.until)
                if all(is_done):
                    break
                current = nxt
            generation.extend(self.tokenizer.decode(g) for g in generated)
            for p, logit in zip(batch, prompt_logits.squeeze(0).split(lengths.tolist())):
                x = logit[:-1].float()
                y = torch.tensor(p[1:], device=x.device)
                loglikelihood.append(-TF.cross_entropy(x, y, reduction="none").cpu())
                greedy.append((x.argmax(dim=-1) == y).cpu())
        self.release_cache()
        return generation, loglikelihood, greedy


def load_consolidated_model_and_tokenizer(consolidated_path, model_cls=LMTransformer,
                                          model_args_cls=LMTransformerArgs):
    """Rebuild model + tokenizer from ``consolidated.pth`` + ``params.json`` (apps/main/generate.py:403-423)."""
    ckpt = Path(consolidated_path)
    config = load_yaml(str(ckpt / "params.json"))  # JSON is a subset of YAML
    dtype = dict(fp32=torch.float32, fp16=torch.float16, bf16=torch.bfloat16)[config["distributed"]["model_dtype"]]
    margs = dataclass_from_dict(model_args_cls, config["model"], strict=False)
    tok = config["data"]["tokenizer"]
    tokenizer = build_tokenizer(tok["name"], tok.get("path"))
    model = model_cls(margs)
    sd = torch.load(ckpt / CONSOLIDATE_NAME, weights_only=True)
    model.load_state_dict(sd["model"])
    if torch.cuda.is_available():
        model = model.cuda().to(dtype)
    model = model.eval()
    if hasattr(model, "rope_embeddings"):
        model.rope_embeddings.reset_parameters()  # non-persistent buffer: not in the checkpoint
    return model, tokenizer, config


def main(argv=None):
    from .config import from_cli

    cfg = from_cli(argv)
    gen_cfg = dataclass_from_dict(PackedCausalTransformerGeneratorArgs, cfg, strict=False)
    print(cfg)
    model, tokenizer, _ = load_consolidated_model_and_tokenizer(cfg["ckpt"])
    generator = PackedCausalTransformerGenerator(gen_cfg, model, tokenizer)
    prompts = []
    while True:
        prompt = input("Enter a prompt (or press enter to finish): ")
        if not prompt:
            break
        prompts.append(prompt)
    t0 = time.time()
    generation, _, _ = generator.generate(prompts)
    dt = time.time() - t0
    total = sum(len(tokenizer.encode(g, False, False)) for g in generation)
    for i, g in enumerate(generation):
        print(f"\nPrompt {i + 1}: {prompts[i]}")
        print(f"Generated Text: {g}")
    print(f"\nTokens per second: {total / dt:.2f}")
