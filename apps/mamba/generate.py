"""``python -m apps.mamba.generate ckpt=<consolidated dir> ...`` (apps/mamba/generate.py)."""
from lingua_b200.generation_recurrent import PackedRNNGenerator as PackedCausalMambaGenerator  # noqa: F401
from lingua_b200.generation_recurrent import PackedRNNGeneratorArgs as PackedCausalMambaGeneratorArgs  # noqa: F401
from lingua_b200.generation_recurrent import main

if __name__ == "__main__":
    main()
