"""Learning-rate schedules and the optimiser front-end.

Schedules are the multiplicative factors of lingua/optim.py (lr_linear :34, lr_inv_sqrt :45,
lr_cosine :53, lr_wsd :73, build_lr_fn :111). ``LRScheduler`` mirrors ``LambdaLR``: the factor
for optimiser step k (0-based) is ``lr_fn(k)``, and its ``state_dict`` has the keys a
``LambdaLR.state_dict()`` has, so ``train_state_*.json`` files stay interchangeable.
The optimiser itself is the sharded AdamW of ``lingua_b200.parallel.engine``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from functools import partial
from typing import Callable, Dict


@dataclass
class OptimArgs:
    lr: float = 3e-4
    weight_decay: float = 0.1
    epsilon: float = 1e-8
    beta1: float = 0.9
    beta2: float = 0.95
    clip: float = 1.0
    scheduler: str = "cosine"
    warmup: int = 2000
    lr_min_ratio: float = 0.1
    cycle_length: float = 1.0
    cosine_theta: float = 1.0
    annealing_step: int = 1000
    decay_fraction: float = 0.1
    exp_factor: float = 0.5


def lr_linear(step: int, warmup: int, n_steps: int, min_ratio: float) -> float:
    if step < warmup:
        return step / warmup
    if step <= n_steps:
        s = (step - warmup) / (n_steps - warmup)
        return s * min_ratio + (1 - s)
    return min_ratio


def lr_inv_sqrt(step: int, warmup: int, exp_factor: float, min_ratio: float) -> float:
    if step < warmup:
        return step / warmup
    return max((warmup ** exp_factor) / (step ** exp_factor), min_ratio)


def lr_cosine(step: int, warmup: int, n_steps: int, cycle_length: float, theta: float, min_ratio: float) -> float:
    sign = ((step // (n_steps * cycle_length)) % 2) * -2 + 1
    if step < warmup:
        return step / warmup
    if step <= n_steps:
        s = (step - warmup) / (n_steps - warmup)
        return min_ratio + 0.5 * (1 - min_ratio) * (sign * math.cos(math.pi * s ** theta / cycle_length) + 1)
    return min_ratio


def lr_wsd(step: int, warmup: int, n_steps: int, decay_fraction: float, cycle_length: float, min_ratio: float) -> float:
    """Warmup - stable - decay, repeated every ``cycle_length * n_steps`` steps; the decay branch is
    the inverse-linear interpolation 1 / (t / min_ratio + (1 - t))."""
    cycle = int(n_steps * cycle_length)
    cycle_num = step // cycle + 1
    cur_end = cycle * cycle_num
    decay_len = int(cur_end * decay_fraction)
    if step == n_steps:
        cur_end = n_steps
    if step < warmup:
        return step / warmup
    if step <= cur_end - decay_len:
        return 1.0
    if step <= cur_end:
        t = (step - (cur_end - decay_len)) / decay_len
        return 1 / (t * (1 / min_ratio) + (1 - t))
    return min_ratio


def build_lr_fn(args: OptimArgs, n_steps: int) -> Callable[[int], float]:
    if args.scheduler == "constant":
        return lambda step: 1.0
    if args.scheduler == "linear":
        return partial(lr_linear, warmup=args.warmup, n_steps=n_steps, min_ratio=args.lr_min_ratio)
    if args.scheduler == "inv_sqrt":
        return partial(lr_inv_sqrt, warmup=args.warmup, exp_factor=args.exp_factor, min_ratio=args.lr_min_ratio)
    if args.scheduler == "cosine":
        return partial(lr_cosine, warmup=args.warmup, n_steps=n_steps, cycle_length=args.cycle_length,
                       theta=args.cosine_theta, min_ratio=args.lr_min_ratio)
    if args.scheduler == "wsd":
        assert args.decay_fraction < args.cycle_length
        return partial(lr_wsd, warmup=args.warmup, n_steps=n_steps, decay_fraction=args.decay_fraction,
                       cycle_length=args.cycle_length, min_ratio=args.lr_min_ratio)
    raise NotImplementedError(f"Unknown scheduler: {args.scheduler}")


class LRScheduler:
    """``get_lr()`` is the rate for the next optimiser step; ``step()`` advances by one."""

    def __init__(self, base_lr: float, lr_fn: Callable[[int], float]):
        self.base_lr, self.lr_fn = base_lr, lr_fn
        self.last_epoch = 0

    def get_lr(self) -> float:
        return self.base_lr * self.lr_fn(self.last_epoch)

    def get_last_lr(self):
        return [self.get_lr()]

    def step(self) -> None:
        self.last_epoch += 1

    def state_dict(self) -> Dict:
        return {"base_lrs": [self.base_lr], "last_epoch": self.last_epoch, "_step_count": self.last_epoch + 1,
                "_get_lr_called_within_step": False, "_last_lr": [self.get_lr()], "lr_lambdas": [None]}

    def load_state_dict(self, sd: Dict) -> None:
        self.last_epoch = int(sd["last_epoch"])


def build_engine_optim(args: OptimArgs):
    from .parallel.engine import EngineOptim

    return EngineOptim(beta1=args.beta1, beta2=args.beta2, eps=args.epsilon, weight_decay=args.weight_decay,
                       clip=args.clip)
