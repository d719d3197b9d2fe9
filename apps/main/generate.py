"""``python -m apps.main.generate ckpt=<consolidated dir> [temperature=.. top_p=.. max_gen_len=..]``

Interactive generation from a consolidated checkpoint (apps/main/generate.py:426-464); the
generator itself lives in ``lingua_b200.generation``."""
from lingua_b200.generation import (KVCache, PackedCausalTransformerGenerator,  # noqa: F401
                                    PackedCausalTransformerGeneratorArgs, batch_prompts,
                                    load_consolidated_model_and_tokenizer, main, pack_prompts, sample_tokens,
                                    sample_top_k, sample_top_p)

if __name__ == "__main__":
    main()
