"""Evaluation: lm-evaluation-harness adapter and validation-set negative log-likelihood.

Follows apps/main/eval.py (LMHarnessArgs :39, ValidationArgs :64, EvalArgs :71, MockAccelerator
:96, EvalHarnessLM :107, eval_on_val :166, launch_eval :219): a checkpoint directory is
consolidated on rank 0 if needed, the model is rebuilt from ``params.json``, the harness tasks
run through the packed generator, ``*.val.jsonl`` files of the training sources are scored, and
rank 0 writes ``results.json`` / ``validation.json`` and appends to ``metrics.eval.jsonl`` /
``metrics.validation.jsonl``. The harness part needs the ``lm_eval`` package; when it is not
installed, tasks are skipped with a warning and only the validation scores are produced.
"""
from __future__ import annotations

import json
import logging
import os
from collections import defaultdict
from dataclasses import asdict, dataclass, field
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, List, Optional, Union

import torch
import torch.distributed as dist

from .checkpoint import CONSOLIDATE_FOLDER, consolidate_checkpoints
from .config import dump_config
from .data.pipeline import init_choice_state, setup_sources
from .distributed import (DistributedArgs, dist_mean_dict, get_global_rank, get_world_size,
                          setup_torch_distributed)
from .generation import (PackedCausalTransformerGenerator, PackedCausalTransformerGeneratorArgs,
                         load_consolidated_model_and_tokenizer)

EVAL_FOLDER_NAME = "{:010d}"
logger = logging.getLogger()


@dataclass
class LMHarnessArgs:
    tasks: Optional[List[Any]] = None
    num_fewshot: Optional[int] = None
    device: Optional[str] = None
    use_cache: Optional[str] = None
    cache_requests: bool = False
    rewrite_requests_cache: bool = False
    delete_requests_cache: bool = False
    limit: Optional[Union[int, float]] = None
    bootstrap_iters: int = 100000
    check_integrity: bool = False
    write_out: bool = False
    log_samples: bool = True
    system_instruction: Optional[str] = None
    apply_chat_template: Union[bool, str] = False
    fewshot_as_multiturn: bool = False
    gen_kwargs: Optional[str] = None
    verbosity: str = "INFO"
    predict_only: bool = False
    random_seed: int = 0
    numpy_random_seed: int = 1234
    torch_random_seed: int = 1234
    fewshot_random_seed: int = 1234


@dataclass
class ValidationArgs:
    max_steps: Optional[int] = None  # documents per rank; None = the whole validation file
    use_val_from_train_src: bool = True
    root_dir: str = ""
    sources: List[str] = field(default_factory=list)


@dataclass
class EvalArgs:
    name: str = "evals"
    dump_dir: Optional[str] = None
    metric_log_dir: Optional[str] = None
    ckpt_dir: str = ""
    generator: PackedCausalTransformerGeneratorArgs = field(default_factory=PackedCausalTransformerGeneratorArgs)
    harness: Optional[LMHarnessArgs] = field(default_factory=LMHarnessArgs)
    validation: Optional[ValidationArgs] = field(default_factory=ValidationArgs)
    wandb: Optional[Any] = None
    global_step: Optional[int] = None


class MockAccelerator:
    """The two calls lm_eval makes on an ``accelerator`` to combine per-rank results."""

    def gather(self, tensor):
        out = [torch.zeros_like(tensor) for _ in range(get_world_size())]
        dist.all_gather(out, tensor)
        return torch.stack(out)

    def wait_for_everyone(self):
        dist.barrier()


def build_harness_lm(generator):
    """lm_eval ``LM`` subclass driving ``generator``; raises ImportError without lm_eval."""
    from lm_eval.api.model import LM

    class EvalHarnessLM(LM):
        def __init__(self, gen):
            super().__init__()
            self.generator = gen
            self.accelerator = MockAccelerator()
            self._rank, self._world_size = get_global_rank(), get_world_size()
            self.device = gen.device

        def generate_until(self, requests):
            prompts, gen_args = zip(*[r.args for r in requests])
            assert all(g == gen_args[0] for g in gen_args), "Doesn't support different gen args for now"
            ga = gen_args[0]
            self.generator.temperature = ga.get("temperature", 0.0)
            self.generator.top_p = ga.get("top_p", None)
            self.generator.top_k = ga.get("top_k", None)
            until = ga.get("until", [])
            self.generator.until = until
            generations, _, _ = self.generator.generate(list(prompts))
            out = []
            for g in generations:
                for e in until:
                    g = g.replace(e, "")
                out.append(g)
            return out

        def loglikelihood(self, requests):
            prompts, continuations = zip(*[r.args for r in requests])
            inputs = [p + c for p, c in zip(prompts, continuations)]
            saved = self.generator.max_gen_len
            self.generator.max_gen_len = 1
            _, lls, greedy = self.generator.generate(inputs)
            self.generator.max_gen_len = saved
            results = []
            for p, ll, gr in zip(prompts, lls, greedy):
                p_len = len(self.generator.tokenizer.encode(p, add_bos=False, add_eos=False))
                results.append((ll[p_len:].sum().item(), gr[p_len:].all().item()))
            return results

        def loglikelihood_rolling(self, requests):
            prompts = [r.args[0] for r in requests]
            saved = self.generator.max_gen_len
            self.generator.max_gen_len = 1
            _, lls, _ = self.generator.generate(prompts)
            self.generator.max_gen_len = saved
            return [(ll.sum().item(),) for ll in lls]

    return EvalHarnessLM(generator)


def eval_on_val(generator, val_args: ValidationArgs, train_cfg: dict):
    """Mean NLL (total, per token, per character) of the ``*.val.jsonl`` documents of every source."""
    srcs = {os.path.join(val_args.root_dir, s): 1.0 for s in val_args.sources}
    if val_args.use_val_from_train_src and train_cfg["data"].get("root_dir"):
        for s in train_cfg["data"]["sources"]:
            srcs[os.path.join(train_cfg["data"]["root_dir"], s)] = 1.0
    srcs = {p: w for p, w in srcs.items() if list(Path(p).glob("*.val.jsonl"))}
    if not srcs:
        return {}
    multi = init_choice_state("", srcs, 0, get_global_rank(), get_world_size(), "*.val.jsonl")
    iters = setup_sources(multi)
    saved = generator.max_gen_len
    generator.max_gen_len = 1
    all_metrics = {}
    for src, it in iters.items():
        texts = []
        logger.info(f"Running validation on {src}...")
        for step, (content, state) in enumerate(it):
            if state["current_iter"] > 0 or (val_args.max_steps is not None and step >= val_args.max_steps):
                break
            texts.append(content["text"] if "text" in content else content["content"])
        _, lls, _ = generator.generate(texts)
        m = defaultdict(list)
        for i, ll in enumerate(lls):
            tot = -ll.sum().item()
            m["nll"].append(tot)
            m["nll_per_token"].append(tot / max(len(ll), 1))
            m["nll_per_char"].append(tot / max(len(texts[i]), 1))
            m["avg_seqlen"].append(len(ll))
        m = {k: sum(v) / len(v) for k, v in m.items()}
        m.update(dist_mean_dict(m))
        name = os.path.basename(src)
        if name in all_metrics:
            logger.warning(f"Duplicate source name {name}, path {src} in validation sources, renaming to {name}_1")
            name = f"{name}_1"
        all_metrics[name] = m
    generator.max_gen_len = saved
    return all_metrics


def launch_eval(cfg: EvalArgs, generator_cls=PackedCausalTransformerGenerator, model_cls=None, model_args_cls=None,
                loader=None):
    """``loader(consolidated_dir) -> (model, tokenizer, train config)`` replaces the default checkpoint loader."""
    if not dist.is_initialized():
        setup_torch_distributed(DistributedArgs())
    ck = Path(cfg.ckpt_dir)
    if ck.exists() and (ck / "params.json").exists() and next(ck.glob("*.pth"), None) is not None:
        consolidated = ck
    else:
        consolidated = ck / CONSOLIDATE_FOLDER
        if not consolidated.exists() and get_global_rank() == 0:
            consolidated = consolidate_checkpoints(cfg.ckpt_dir)
    Path(cfg.dump_dir).mkdir(parents=True, exist_ok=True)
    dump_config(cfg, Path(cfg.dump_dir) / "config.yaml", log_config=False)
    if dist.get_world_size() > 1:
        dist.barrier()
    logger.info("Loading model")
    kw = {}
    if model_cls is not None:
        kw = dict(model_cls=model_cls, model_args_cls=model_args_cls)
    if loader is not None:
        model, tokenizer, train_cfg = loader(str(consolidated))
    else:
        model, tokenizer, train_cfg = load_consolidated_model_and_tokenizer(str(consolidated), **kw)
    model.eval()
    generator = generator_cls(cfg.generator, model, tokenizer)
    results = {"results": {}}
    if cfg.harness is not None and cfg.harness.tasks:
        try:
            from lm_eval import simple_evaluate

            results = simple_evaluate(build_harness_lm(generator), **asdict(cfg.harness))
        except ImportError:
            logger.warning("lm_eval is not installed: skipping harness tasks %s", cfg.harness.tasks)
    val_results = eval_on_val(generator, cfg.validation, train_cfg) if cfg.validation else None
    if get_global_rank() == 0:
        (Path(cfg.dump_dir) / "results.json").write_text(json.dumps(results, default=str))
        logger.info(f"All evaluation results: {results['results']}")
        if val_results is not None:
            (Path(cfg.dump_dir) / "validation.json").write_text(json.dumps(val_results))
            logger.info(f"All validation results: {val_results}")
    if cfg.metric_log_dir and get_global_rank() == 0:
        stamp = {"created_at": datetime.now(timezone.utc).isoformat()}
        if cfg.global_step is not None:
            stamp["global_step"] = cfg.global_step
        with open(Path(cfg.metric_log_dir) / "metrics.eval.jsonl", "a") as f:
            print(json.dumps({**stamp, **results["results"]}, default=str), file=f, flush=True)
        if val_results is not None:
            with open(Path(cfg.metric_log_dir) / "metrics.validation.jsonl", "a") as f:
                print(json.dumps({**stamp, **val_results}), file=f, flush=True)
    del generator
    return results, val_results


def main(args_cls=EvalArgs, launch=launch_eval, argv=None):
    from .config import config_from_cli

    launch(config_from_cli(args_cls, argv))
