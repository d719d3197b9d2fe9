"""``python -m apps.mamba.train config=apps/mamba/configs/debug.yaml``: Mamba-2 pre-training
(apps/mamba/train.py; no tensor parallelism for this model, as in the reference)."""
from __future__ import annotations

from dataclasses import dataclass, field

from lingua_b200.models.mamba import LMMamba, LMMambaArgs, build_fsdp_grouping_plan, get_num_flop_per_token
from lingua_b200.train_loop import ModelSpec, TrainArgs as _BaseTrainArgs, main_from_cli, run_training


@dataclass
class TrainArgs(_BaseTrainArgs):
    model: LMMambaArgs = field(default_factory=LMMambaArgs)


def model_spec(args: TrainArgs) -> ModelSpec:
    def flops(n_params, m, seq_len):
        return get_num_flop_per_token(n_params - m.vocab_size * m.dim, m.n_layers, m.dim, seq_len)

    return ModelSpec(model_cls=LMMamba, build_plan=build_fsdp_grouping_plan, flops_per_token=flops,
                     eval_module="apps.mamba.eval")


def train(args: TrainArgs):
    return run_training(args, model_spec(args))


def main():
    main_from_cli(TrainArgs, model_spec)


if __name__ == "__main__":
    main()
