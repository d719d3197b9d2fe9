"""setup/: the external-memory line shuffler and the dataset preparation built on it."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "setup"))
import prepare_data  # noqa: E402


def test_lineshuf_is_a_permutation_with_and_without_spilling(tmp_path):
    exe = prepare_data.build_lineshuf()
    lines = [f"line {i} " + "x" * (i % 50) for i in range(20000)]
    data = ("\n".join(lines)).encode()  # last line has no terminator
    for mem in ("1", "0.0002"):  # all in memory / ~200 KB chunks on disk
        env = dict(os.environ, MEMORY=mem, SEED="7", TMPDIR=str(tmp_path))
        out = subprocess.run([str(exe)], input=data, capture_output=True, env=env, check=True).stdout.decode()
        got = out.splitlines()
        assert sorted(got) == sorted(lines) and got != lines
        again = subprocess.run([str(exe)], input=data, capture_output=True, env=env, check=True).stdout.decode()
        assert again == out  # same seed, same order
    assert not list(tmp_path.glob("lineshuf.*"))  # temporary files are removed


def test_prepare_data_layout_feeds_the_loader(tmp_path):
    src = tmp_path / "raw"
    src.mkdir()
    with open(src / "a.jsonl", "w") as f:
        for i in range(300):
            f.write(json.dumps({"text": f"document {i}"}) + "\n")
    prepare_data.main(["toy", "0.5", "--data_dir", str(tmp_path / "data"), "--source", str(src), "--nchunks", "4",
                       "--k_validation", "5", "--seed", "1"])
    out = tmp_path / "data" / "toy_shuffled"
    chunks = sorted(out.glob("toy.chunk.*.jsonl"))
    assert [c.name for c in chunks] == [f"toy.chunk.{i:02d}.jsonl" for i in range(4)]
    n_val = sum(1 for _ in open(out / "toy.val.jsonl"))
    n_train = sum(sum(1 for _ in open(c)) for c in chunks)
    assert n_val == 20 and n_train == 280
    from lingua_b200.data.pipeline import DataArgs, build_dataloader_from_args, init_dataloader_state_from_args
    from lingua_b200.tokenizer import TokenizerArgs

    args = DataArgs(root_dir=str(tmp_path / "data"), sources={"toy_shuffled": 1.0}, batch_size=2, seq_len=16,
                    n_views=2, load_async=False, tokenizer=TokenizerArgs(name="bytes"))
    state = init_dataloader_state_from_args(args, rank=0, world_size=1)
    with build_dataloader_from_args(args, state=state) as it:
        batch, _ = next(it)
    assert batch.shape == (2, 16, 2)
