"""Data pipeline: determinism, exact resume at every step, rank sharding, async loader, tokenizers."""
import json
import os
import signal
import time

import numpy as np
import pytest

from lingua_b200.data import pipeline as P
from lingua_b200.tokenizer import ByteTokenizer, build_tokenizer


@pytest.fixture()
def corpus(tmp_path):
    rng = np.random.default_rng(0)
    for src, n_chunks in (("a", 2), ("b", 1)):
        d = tmp_path / src
        d.mkdir()
        for c in range(n_chunks):
            with open(d / f"{src}.chunk.{c:02d}.jsonl", "w") as f:
                for i in range(40):
                    n = int(rng.integers(5, 200))
                    f.write(json.dumps({"text": f"{src}{c}-{i} " + "x" * n}) + "\n")
    return tmp_path


def _args(root, **kw):
    base = dict(root_dir=str(root), sources={"a": 2.0, "b": 1.0}, batch_size=2, seq_len=32, n_views=2, seed=7,
                load_async=False, prefetch_size=4)
    base.update(kw)
    return P.DataArgs(**base)


def _take(args, state, n):
    out, states = [], []
    with P.build_dataloader_from_args(args, state=state) as it:
        for _ in range(n):
            b, s = next(it)
            out.append(b.copy())
            states.append(json.loads(json.dumps(s)))  # states must survive a JSON round trip
    return out, states


def test_batches_shape_views_and_determinism(corpus):
    args = _args(corpus)
    st = P.init_dataloader_state_from_args(args, 0, 2)
    a, _ = _take(args, st, 6)
    b, _ = _take(args, st, 6)
    assert a[0].shape == (2, 32, 2)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    assert np.array_equal(a[0][:, 1:, 0], a[0][:, :-1, 1])  # view 1 is view 0 shifted by one token


def test_resume_from_every_step_reproduces_stream(corpus):
    args = _args(corpus)
    st = P.init_dataloader_state_from_args(args, 1, 2)
    full, states = _take(args, st, 12)
    for k in (0, 3, 4, 7, 10):
        rest, _ = _take(args, states[k], 12 - k - 1)
        for i, r in enumerate(rest):
            assert np.array_equal(r, full[k + 1 + i]), f"resume after step {k}, batch {i}"


def test_ranks_read_disjoint_lines(corpus):
    seen = []
    for rank in range(2):
        js = P.distribute_data_to_rank(str(corpus / "b"), rank, 2, P.TRAIN_DATA_FILE_PATTERN)
        lines = [c["text"] for c, _ in P.read_jsonl(js["file_path"], 0, js["block_size"], js["offset"], 0)]
        seen.append(set(lines))
    assert len(seen[0]) == 20 and len(seen[1]) == 20 and not (seen[0] & seen[1])


def test_async_loader_matches_sync_and_detects_dead_worker(corpus):
    args = _args(corpus)
    st = P.init_dataloader_state_from_args(args, 0, 1)
    sync, _ = _take(args, st, 5)
    args_async = _args(corpus, load_async=True)
    with P.build_dataloader_from_args(args_async, state=st) as it:
        for i in range(5):
            b, _ = next(it)
            assert np.array_equal(b, sync[i])
    # a producer that dies is reported as an error instead of a hang
    with P.async_iterator(2, lambda: P.build_dataloader(st)) as it:
        next(it)
        gen_frame = it.gi_frame.f_locals
        producer = gen_frame["producer"]
        os.kill(producer.pid, signal.SIGKILL)
        with pytest.raises(RuntimeError):
            for _ in range(50):
                next(it)


def test_synthetic_source_resumes(tmp_path):
    args = P.DataArgs(root_dir=None, sources={"synthetic": 1.0}, batch_size=3, seq_len=16, load_async=False)
    st = P.init_dataloader_state_from_args(args, 0, 1, vocab_size=1000)
    full, states = _take(args, st, 4)
    assert full[0].shape == (3, 16, 2) and full[0].max() < 1000
    rest, _ = _take(args, states[1], 2)
    assert np.array_equal(rest[0], full[2]) and np.array_equal(rest[1], full[3])


def test_byte_tokenizer():
    t = build_tokenizer("bytes")
    assert isinstance(t, ByteTokenizer) and t.n_words == 258
    ids = t.encode("héllo", add_bos=True, add_eos=True)
    assert ids[0] == 256 and ids[-1] == 257 and t.decode(ids) == "héllo"
    chars, offs = t.get_token_offsets("hello")
    assert "".join(chars) == "hello" and offs == [0, 1, 2, 3, 4]
