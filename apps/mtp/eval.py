"""``python -m apps.mtp.eval config=... ckpt_dir=... dump_dir=...``: evaluation with head 0 (apps/mtp/eval.py)."""
from lingua_b200.evaluation import EVAL_FOLDER_NAME, EvalArgs, launch_eval as _launch, main as _main  # noqa: F401
from lingua_b200.models.mtp import LMMTPArgs, LMTransformer


def launch_eval(cfg: EvalArgs):
    return _launch(cfg, model_cls=LMTransformer, model_args_cls=LMMTPArgs)


def main():
    _main(EvalArgs, launch_eval)


if __name__ == "__main__":
    main()
