"""``python -m apps.mtp.train config=apps/mtp/configs/debug.yaml``: multi-token-prediction pre-training.

The loader must produce one more view than there are heads (``data.n_views == model.n_future_head + 1``);
labels are views 1.. (apps/mtp/train.py:199,367), the optimised loss is the sum over heads and every
head's loss is logged as ``loss/head_i`` (:414-421,507-508)."""
from __future__ import annotations

from dataclasses import dataclass, field

from lingua_b200.models.mtp import LMMTPArgs, LMTransformer, build_fsdp_grouping_plan
from lingua_b200.models.transformer import get_num_flop_per_token
from lingua_b200.train_loop import ModelSpec, TrainArgs as _BaseTrainArgs, main_from_cli, run_training


@dataclass
class TrainArgs(_BaseTrainArgs):
    model: LMMTPArgs = field(default_factory=LMMTPArgs)


def _loss(model, x, y):
    losses = model(x, y)
    total = losses[0]
    for l in losses[1:]:
        total = total + l
    return total, {f"head_{i}": l.detach() for i, l in enumerate(losses)}


def model_spec(args: TrainArgs) -> ModelSpec:
    assert args.model.n_future_head == args.data.n_views - 1, "need one data view per head plus the input view"

    def flops(n_params, m, seq_len):
        return get_num_flop_per_token(n_params - m.vocab_size * m.dim, m.n_layers, m.dim, seq_len)

    return ModelSpec(model_cls=LMTransformer, build_plan=build_fsdp_grouping_plan, flops_per_token=flops,
                     labels_from_batch=lambda batch: batch[:, :, 1:], loss_fn=_loss, eval_module="apps.mtp.eval")


def train(args: TrainArgs):
    return run_training(args, model_spec(args))


def main():
    main_from_cli(TrainArgs, model_spec)


if __name__ == "__main__":
    main()
