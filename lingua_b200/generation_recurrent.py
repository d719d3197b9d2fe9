"""Generation for the recurrent (minGRU / minLSTM / Hawk) and Mamba-2 models.

Same packing as the transformer generator, but the per-layer state is O(1) per sequence: a
``StateCache`` (conv window + recurrent state) for every recurrent block, filled by one packed
prefill pass with document resets and then advanced token by token (apps/fastRNN/generate.py
:61-174, apps/mamba/generate.py:62-108).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from pathlib import Path

import torch

from .config import dataclass_from_dict, load_yaml
from .evaluation import EvalArgs, launch_eval as _launch_eval
from .generation import (PackedCausalTransformerGenerator, PackedCausalTransformerGeneratorArgs,
                         lengths_to_local_ids, lengths_to_start_ids, load_consolidated_model_and_tokenizer)


@dataclass
class PackedRNNGeneratorArgs(PackedCausalTransformerGeneratorArgs):
    pass


def _stateful_modules(model):
    from .models.fastrnn import recurrent_modules

    mods = list(recurrent_modules(model))
    try:
        from .models.mamba import SSM

        mods += [m for m in model.modules() if isinstance(m, SSM)]
    except ImportError:
        pass
    return mods


class PackedRNNGenerator(PackedCausalTransformerGenerator):
    def clear_cache(self, n_seqs: int, lengths: torch.Tensor):
        p = next(self.model.parameters())
        for m in _stateful_modules(self.model):
            cache = getattr(m, "cache", None)
            if cache is None or cache.state_cache.shape[0] != n_seqs:
                # plain attribute (not a registered sub-module): generation state stays out of state_dict
                object.__setattr__(m, "cache", m.make_cache(n_seqs, p.dtype, p.device))
            m.cache.reset()
            m.cache.lengths = lengths

    def release_cache(self):
        for m in _stateful_modules(self.model):
            object.__setattr__(m, "cache", None)

    def prefill(self, tokens: torch.Tensor, lengths: torch.Tensor):
        self.clear_cache(lengths.numel(), lengths)
        doc_start = lengths_to_start_ids(lengths)[lengths_to_local_ids(lengths)[0]].int().view(1, -1)
        out = self.model(tokens, doc_start=doc_start, impl="parallel")
        self.current_tok_id = lengths.clone()
        return out

    def generate_next_token(self, current_token: torch.Tensor):
        out = self.model(current_token, impl="sequential")
        self.current_tok_id += 1
        return out


def load_recurrent_model(consolidated_path):
    """Pick the model class from ``model_type`` (fastRNN apps) or the mamba marker in params.json."""
    cfg = load_yaml(str(Path(consolidated_path) / "params.json"))
    if "model_type" in cfg:
        from .models.fastrnn import MODEL_TYPES

        cls, args_cls = MODEL_TYPES[cfg["model_type"]]
    else:
        from .models.mamba import LMMamba as cls, LMMambaArgs as args_cls
    return load_consolidated_model_and_tokenizer(consolidated_path, model_cls=cls, model_args_cls=args_cls)


def launch_eval(cfg: EvalArgs):
    ck = Path(cfg.ckpt_dir)
    params = ck / "params.json" if (ck / "params.json").exists() else None
    tcfg = load_yaml(str(params)) if params else {}
    if "model_type" in tcfg:
        from .models.fastrnn import MODEL_TYPES

        cls, args_cls = MODEL_TYPES[tcfg["model_type"]]
    else:
        from .models.mamba import LMMamba as cls, LMMambaArgs as args_cls
    return _launch_eval(cfg, generator_cls=PackedRNNGenerator, model_cls=cls, model_args_cls=args_cls)


def main(argv=None):
    from .config import from_cli

    cfg = from_cli(argv)
    gen_cfg = dataclass_from_dict(PackedRNNGeneratorArgs, cfg, strict=False)
    model, tokenizer, _ = load_recurrent_model(cfg["ckpt"])
    generator = PackedRNNGenerator(gen_cfg, model, tokenizer)
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
