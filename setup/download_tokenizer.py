"""Fetch a tokenizer file for ``lingua_b200.tokenizer`` (needs network access).

    python setup/download_tokenizer.py llama3 <SAVE_PATH> [--api_key <HF_TOKEN>]

Same choices as setup/download_tokenizer.py:9-51 of the reference: ``llama2`` / ``llama3`` / ``gemma`` come
from the Hugging Face hub (a token with access to the gated repository is required), ``tiktoken`` encodings
(``cl100k_base`` ...) are fetched by the tiktoken package itself and only need to be named in the config.
"""
from __future__ import annotations

import argparse
from pathlib import Path

TOKENIZER = {
    "llama2": ("meta-llama/Llama-2-7b", "tokenizer.model"),
    "llama3": ("meta-llama/Meta-Llama-3-8B", "original/tokenizer.model"),
    "gemma": ("google/gemma-2-9b", "tokenizer.model"),
}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("tokenizer_name")
    ap.add_argument("tokenizer_dir", nargs="?", default=None)
    ap.add_argument("--api_key", default=None)
    a = ap.parse_args(argv)
    if a.tokenizer_name in TOKENIZER:
        from huggingface_hub import hf_hub_download

        repo, fname = TOKENIZER[a.tokenizer_name]
        dest = Path(a.tokenizer_dir or "tokenizers") / a.tokenizer_name
        path = hf_hub_download(repo_id=repo, filename=fname, local_dir=str(dest), token=a.api_key)
        print(path)
    else:
        import tiktoken

        tiktoken.get_encoding(a.tokenizer_name)  # downloads and caches the encoding
        print(f"tiktoken encoding {a.tokenizer_name} cached; use tokenizer.name=tiktoken, path={a.tokenizer_name}")


if __name__ == "__main__":
    main()
