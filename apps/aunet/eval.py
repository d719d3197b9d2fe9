"""``python -m apps.aunet.eval config=apps/aunet/configs/eval.yaml ckpt_dir=... dump_dir=...`` (apps/aunet/eval.py)."""
from dataclasses import dataclass, field

from lingua_b200.evaluation import EVAL_FOLDER_NAME, EvalArgs as _EvalArgs, main as _main  # noqa: F401
from lingua_b200.generation_aunet import PackedHierarchicalCausalTransformerGeneratorArgs, launch_eval  # noqa: F401


@dataclass
class EvalArgs(_EvalArgs):
    generator: PackedHierarchicalCausalTransformerGeneratorArgs = field(
        default_factory=PackedHierarchicalCausalTransformerGeneratorArgs)


def main():
    _main(EvalArgs, launch_eval)


if __name__ == "__main__":
    main()
