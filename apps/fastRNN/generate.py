"""``python -m apps.fastRNN.generate ckpt=<consolidated dir> ...``: generation with the recurrent models
(apps/fastRNN/generate.py); see ``lingua_b200.generation_recurrent``."""
from lingua_b200.generation_recurrent import PackedRNNGenerator, PackedRNNGeneratorArgs, main  # noqa: F401

if __name__ == "__main__":
    main()
