"""``python -m apps.aunet.train config=apps/aunet/configs/debug.yaml``: pre-training of the hierarchical byte model.

The data pipeline marks every byte with its pooling level (``data.regex.strategy``, one rule per level) and
ships token and level packed in one integer, so that the loop, the prefetcher and the host-to-device copy are
the ones every other app uses; the two are separated on the device. The optimised loss is the next-byte
cross-entropy plus ``model.lambda_level`` times the level-prediction loss; ``ce/out``, ``mask_loss/out`` and
the number of positions that reached each stage (``nb_toks/enc_i``) are logged (apps/aunet/train.py:359-436,
521-529 of the reference)."""
from __future__ import annotations

from dataclasses import dataclass, field

from lingua_b200.data.pipeline import split_levels
from lingua_b200.models.aunet import HierarchicalArgs, HierarchicalTransformer, build_fsdp_grouping_plan
from lingua_b200.train_loop import ModelSpec, TrainArgs as _BaseTrainArgs, main_from_cli, run_training


@dataclass
class TrainArgs(_BaseTrainArgs):
    model: HierarchicalArgs = field(default_factory=HierarchicalArgs)


def model_spec(args: TrainArgs) -> ModelSpec:
    lam = args.model.lambda_level
    assert args.data.regex is not None and args.data.regex.strategy, "data.regex.strategy defines the pooling levels"
    assert len(args.data.regex.strategy) == len(args.model.dimensions) - 1, "one pooling rule per transition"

    def loss(model, x, y):
        tokens, levels = split_levels(x)
        target, target_levels = split_levels(y)
        ce, mask_loss, nb_toks = model(tokens, levels, target, target_levels)
        extra = {"ce/out": ce.detach()}
        extra.update({f"nb_toks/enc_{i}": n.float() for i, n in enumerate(nb_toks)})
        if mask_loss is None:
            return ce, extra
        extra["mask_loss/out"] = mask_loss.detach()
        return ce + lam * mask_loss, extra

    def flops(n_params, m, seq_len):
        return m.flops_per_token(seq_len)

    return ModelSpec(model_cls=HierarchicalTransformer, build_plan=build_fsdp_grouping_plan, flops_per_token=flops,
                     loss_fn=loss, eval_module="apps.aunet.eval")


def train(args: TrainArgs):
    return run_training(args, model_spec(args))


def main():
    main_from_cli(TrainArgs, model_spec)


if __name__ == "__main__":
    main()
