"""``python -m apps.main.train config=apps/main/configs/debug.yaml [key=value ...]``

Pre-training entry point of the Llama-style transformer app (the CLI and ``TrainArgs`` schema of
apps/main/train.py:76-104,605-657; the loop itself lives in ``lingua_b200.train_loop``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from lingua_b200.models.transformer import (LMTransformer, LMTransformerArgs, build_fsdp_grouping_plan,
                                            get_num_flop_per_token)
from lingua_b200.parallel.tensor_parallel import tp_parallelize
from lingua_b200.train_loop import ModelSpec, TrainArgs as _BaseTrainArgs, main_from_cli, run_training


@dataclass
class TrainArgs(_BaseTrainArgs):
    model: LMTransformerArgs = field(default_factory=LMTransformerArgs)


def model_spec(args: TrainArgs) -> ModelSpec:
    def flops(n_params, m, seq_len):
        return get_num_flop_per_token(n_params - m.vocab_size * m.dim, m.n_layers, m.dim, seq_len)

    return ModelSpec(model_cls=LMTransformer, build_plan=build_fsdp_grouping_plan, tp_parallelize=tp_parallelize,
                     flops_per_token=flops, eval_module="apps.main.eval")


def train(args: TrainArgs):
    return run_training(args, model_spec(args))


def main():
    main_from_cli(TrainArgs, model_spec)


if __name__ == "__main__":
    main()
