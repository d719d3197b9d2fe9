"""``python -m apps.mamba.eval config=apps/mamba/configs/eval.yaml ckpt_dir=... dump_dir=...`` (apps/mamba/eval.py)."""
from lingua_b200.evaluation import EVAL_FOLDER_NAME, EvalArgs, main as _main  # noqa: F401
from lingua_b200.generation_recurrent import launch_eval  # noqa: F401


def main():
    _main(EvalArgs, launch_eval)


if __name__ == "__main__":
    main()
