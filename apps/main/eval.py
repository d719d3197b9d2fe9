"""``python -m apps.main.eval config=apps/main/configs/eval.yaml ckpt_dir=... dump_dir=...``

Evaluation entry point of the transformer app (apps/main/eval.py:287-338); see
``lingua_b200.evaluation``."""
from lingua_b200.evaluation import (EVAL_FOLDER_NAME, EvalArgs, LMHarnessArgs, ValidationArgs,  # noqa: F401
                                    eval_on_val, launch_eval, main)

if __name__ == "__main__":
    main()
