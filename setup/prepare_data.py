"""Turn a dataset into the shuffled, chunked JSONL layout the data loader reads.

    python setup/prepare_data.py <dataset> <memory_gb> [--data_dir data] [--source DIR] [--seed 42] [--nchunks 32]

Output (same layout as setup/download_prepare_hf_data.py:112-140 of the reference):
``<data_dir>/<dataset>_shuffled/<dataset>.chunk.NN.jsonl`` (``nchunks`` round-robin shards of the globally
shuffled lines) and ``<dataset>.val.jsonl`` (the first ``k_validation`` lines of every shard, removed from it).

Source of the lines, in this order: ``--source DIR`` with ``*.jsonl`` / ``*.parquet`` files; else the Hugging
Face hub through ``huggingface_hub.snapshot_download`` for the datasets the reference knows (needs network).
Parquet is read with pyarrow. Shuffling is done by the in-tree external-memory shuffler ``setup/lineshuf.cpp``
(built on first use with g++), so datasets larger than RAM work.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
HF_REPOS = {
    "fineweb_edu": "HuggingFaceFW/fineweb-edu",
    "fineweb_edu_10bt": "HuggingFaceFW/fineweb-edu",
    "dclm_baseline_1.0": "mlfoundations/dclm-baseline-1.0",
    "dclm_baseline_1.0_10prct": "mlfoundations/dclm-baseline-1.0",
}
HF_PATTERNS = {"fineweb_edu_10bt": "sample/10BT/*", "dclm_baseline_1.0_10prct": "global-shard_01_of_10/*"}


def build_lineshuf() -> Path:
    exe = HERE / "lineshuf"
    src = HERE / "lineshuf.cpp"
    if not exe.exists() or exe.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["g++", "-O2", "-std=c++17", "-o", str(exe), str(src)], check=True)
    return exe


def download(dataset: str, dest: Path) -> Path:
    if dataset not in HF_REPOS:
        raise SystemExit(f"unknown dataset {dataset!r}: pass --source DIR or one of {sorted(HF_REPOS)}")
    from huggingface_hub import snapshot_download

    snapshot_download(HF_REPOS[dataset], repo_type="dataset", local_dir=str(dest),
                      allow_patterns=HF_PATTERNS.get(dataset), resume_download=True)
    return dest


def iter_lines(src: Path):
    """JSON lines of every ``*.jsonl`` / ``*.jsonl.zst``-free / ``*.parquet`` file below ``src``."""
    for f in sorted(src.rglob("*")):
        if f.suffix == ".jsonl":
            with open(f, "rb") as fh:
                for line in fh:
                    if line.strip():
                        yield line if line.endswith(b"\n") else line + b"\n"
        elif f.suffix == ".parquet":
            import pyarrow.parquet as pq

            pf = pq.ParquetFile(f)
            for batch in pf.iter_batches(batch_size=4096):
                for row in batch.to_pylist():
                    yield (json.dumps(row, ensure_ascii=False) + "\n").encode()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("dataset")
    ap.add_argument("memory", type=float, help="GB of RAM the shuffler may use")
    ap.add_argument("--data_dir", default="data")
    ap.add_argument("--source", default=None, help="local directory with .jsonl / .parquet files")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--nchunks", type=int, default=32)
    ap.add_argument("--k_validation", type=int, default=10000)
    a = ap.parse_args(argv)

    src = Path(a.source) if a.source else download(a.dataset, Path(a.data_dir) / a.dataset)
    out_dir = Path(a.data_dir) / f"{a.dataset}_shuffled"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = build_lineshuf()
    env = dict(os.environ, MEMORY=str(a.memory), SEED=str(a.seed))
    env.setdefault("TMPDIR", str(out_dir))
    shuf = subprocess.Popen([str(exe)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, env=env)

    def feed():
        for line in iter_lines(src):
            shuf.stdin.write(line)
        shuf.stdin.close()

    import threading

    t = threading.Thread(target=feed, daemon=True)
    t.start()
    chunks = [open(out_dir / f"{a.dataset}.chunk.{i:02d}.jsonl", "wb") for i in range(a.nchunks)]
    val = open(out_dir / f"{a.dataset}.val.jsonl", "wb")
    taken = [0] * a.nchunks
    n = 0
    for line in shuf.stdout:  # round-robin split; the head of every shard becomes validation data
        i = n % a.nchunks
        if taken[i] < a.k_validation:
            val.write(line)
            taken[i] += 1
        else:
            chunks[i].write(line)
        n += 1
    t.join()
    for f in chunks + [val]:
        f.close()
    if shuf.wait() != 0:
        raise SystemExit("lineshuf failed")
    print(f"{n} lines -> {out_dir} ({a.nchunks} chunks, {sum(taken)} validation lines)")


if __name__ == "__main__":
    main()
