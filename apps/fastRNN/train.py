"""``python -m apps.fastRNN.train config=apps/fastRNN/hawk/configs/debug.yaml``

Pre-training of the linear-recurrence models. ``model_type`` (minGRU | minLSTM | hawk) selects the
architecture and ``model`` holds its arguments as a mapping (apps/fastRNN/train.py:100-102,264-271).
The reference logs FLOPS = 0 for these models; here 6 x non-embedding parameters is reported."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Dict

from lingua_b200.config import dataclass_from_dict
from lingua_b200.models.fastrnn import MODEL_TYPES, LMMinGRUArgs, build_fsdp_grouping_plan
from lingua_b200.train_loop import ModelSpec, TrainArgs as _BaseTrainArgs, main_from_cli, run_training


@dataclass
class TrainArgs(_BaseTrainArgs):
    model_type: str = "minGRU"
    model: Dict[str, Any] = field(default_factory=lambda: asdict(LMMinGRUArgs()))


def model_spec(args: TrainArgs) -> ModelSpec:
    if args.model_type not in MODEL_TYPES:
        raise ValueError(f"Model type {args.model_type} not recognized")
    model_cls, args_cls = MODEL_TYPES[args.model_type]
    if isinstance(args.model, dict):
        args.model = dataclass_from_dict(args_cls, args.model)
    return ModelSpec(model_cls=model_cls, build_plan=build_fsdp_grouping_plan,
                     flops_per_token=lambda n, m, s: 6.0 * (n - m.vocab_size * m.dim),
                     eval_module="apps.fastRNN.eval")


def train(args: TrainArgs):
    return run_training(args, model_spec(args))


def main():
    main_from_cli(TrainArgs, model_spec)


if __name__ == "__main__":
    main()
