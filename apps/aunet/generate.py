"""``python -m apps.aunet.generate ckpt=<consolidated dir> ...`` (apps/aunet/generate.py)."""
from lingua_b200.generation_aunet import (PackedHierarchicalCausalTransformerGenerator,  # noqa: F401
                                          PackedHierarchicalCausalTransformerGeneratorArgs,  # noqa: F401
                                          load_consolidated_model_and_tokenizer, main)  # noqa: F401

if __name__ == "__main__":
    main()
