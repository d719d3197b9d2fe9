"""Deterministic, resumable text-to-batches pipeline.

Stages, each a generator that yields ``(item, state)`` where ``state`` is a plain (JSON
serialisable) dict from which the stage can be rebuilt at exactly that position:

    JSONL lines -> weighted choice over sources -> tokens -> packed (seq_len, n_views)
    windows -> block-shuffled batches (batch, seq_len, n_views)

The nested state dictionaries use the same keys as lingua/data.py (JSONLState :64,
MultiChoiceState :83, TokenizerState :99, PackTokensState :107, PrefetchState :123), so a
``train_state_*.json`` written by either implementation restores the other's stream, and
the per-rank seeding follows init_choice_state :511 / init_state :539. A synthetic
uniform-random source (``SyntheticArgs``) shares the batch contract for benchmarking.
"""
from __future__ import annotations

import contextlib
import copy
import json
import logging
import os
from dataclasses import dataclass, field
from functools import partial
from multiprocessing import Event, Process, Queue
from pathlib import Path
from queue import Empty, Full
from typing import Any, Dict, Iterator, Optional

import numpy as np

from ..tokenizer import TokenizerArgs, build_tokenizer
from .regex_cutting import RegexArgs

logger = logging.getLogger()

TRAIN_DATA_FILE_PATTERN = "*.chunk.*.jsonl"


# ----------------------------------------------------------------------------- JSONL
def read_jsonl(file_path: str, position: int, block_size: int, offset: int, current_iter: int):
    """Yield every ``block_size``-th line (those with index % block_size == offset) from byte
    ``position`` on; the state carries the byte position after the yielded line."""
    if not 0 <= offset < block_size:
        raise RuntimeError("JSONL iterator offset value is invalid")
    # A non-zero position is always the byte after a yielded line, i.e. line index offset + 1.
    line_no = offset + 1 if position > 0 else 0
    with open(file_path, "r") as f:
        f.seek(position)
        while True:
            line = f.readline()
            if not line:
                return
            if line_no % block_size == offset:
                st = dict(file_path=file_path, position=f.tell(), block_size=block_size, offset=offset,
                          current_iter=current_iter)
                yield json.loads(line), st
            line_no += 1


def loop_on_jsonl(file_path: str, position: int, block_size: int, offset: int, current_iter: int):
    """Infinite version of read_jsonl; each wrap-around increments ``current_iter``."""
    while True:
        n = 0
        for item in read_jsonl(file_path, position, block_size, offset, current_iter):
            n += 1
            yield item
        if n == 0 and position == 0:
            raise RuntimeError(f"{file_path} yields no line for offset {offset} / block {block_size}")
        current_iter += 1
        position = 0


# ----------------------------------------------------------------------------- sources
def choose_source(source_to_iterator, source_to_state, root_dir, sources, rng_state):
    """Pick the next document from one of the sources with probability ~ its weight."""
    names = list(sources.keys())
    w = np.array(list(sources.values()), dtype=float)
    w = w / w.sum()
    rng = np.random.default_rng()
    rng.bit_generator.state = rng_state
    while True:
        name = names[rng.choice(len(names), p=w)]
        seq, st = next(source_to_iterator[name])
        source_to_state = {**source_to_state, name: st}
        yield seq, dict(root_dir=root_dir, sources=sources, source_to_state=source_to_state,
                        rng_state=rng.bit_generator.state)


LEVEL_SHIFT = 32  # a token and its pooling level travel through the pipeline as ``token | level << 32``


def split_levels(batch):
    """Undo the packing done by ``tokenize(..., regex=...)``: (token ids, pooling levels)."""
    return batch & ((1 << LEVEL_SHIFT) - 1), batch >> LEVEL_SHIFT


def tokenize(iterator, add_bos: bool, add_eos: bool, tokenizer_type: str, tokenizer_path: Optional[str] = None,
             regex: Optional[dict] = None):
    """Documents -> token lists. With ``regex`` (a pooling strategy, apps/aunet/data/data.py:231-253 of the
    reference) the byte tokenizer is required and every token carries its pooling level in its upper bits;
    the first token of a document (its <bos>) gets the deepest level found in that document."""
    tok = build_tokenizer(tokenizer_type, tokenizer_path)
    pool = None
    if regex:
        from .regex_cutting import RegexArgs, RegexPool

        pool = RegexPool(RegexArgs(strategy=dict(regex.get("strategy", regex))))
    for content, st in iterator:
        if "text" in content:
            text = content["text"]
        elif "content" in content:
            text = content["content"]
        else:
            raise AssertionError("JSON line must contain either text or content key")
        tokens = tok.encode(text, add_bos=add_bos, add_eos=add_eos)
        if pool is not None:
            body = pool.text_levels(text)
            levels = np.zeros(len(tokens), dtype=np.int64)
            assert len(body) + int(add_bos) + int(add_eos) == len(tokens), "regex pooling needs the byte tokenizer"
            levels[int(add_bos):int(add_bos) + len(body)] = body
            levels[0] = max(body) if body and max(body) > 0 else pool.n_levels
            tokens = (np.asarray(tokens, dtype=np.int64) | (levels << LEVEL_SHIFT)).tolist()
        yield tokens, dict(it_state=st, add_bos=add_bos, add_eos=add_eos, name=tokenizer_type, path=tokenizer_path,
                           **({"regex": regex} if regex else {}))


# ----------------------------------------------------------------------------- packing
def _resume_point(rewound_token: int, pieces: list) -> dict:
    """State from which re-reading reproduces the tokens that are still in the buffer.

    ``pieces`` lists, oldest first, what was appended to the buffer; the last n_views-1
    tokens must be re-read after a restart, so walk back over pieces until the rewound
    index is inside one of them."""
    k = -1
    while rewound_token < 0:
        k -= 1
        rewound_token += pieces[k]["seq_len"]
    st = copy.deepcopy(pieces[k])
    st["start_token"] = rewound_token
    del pieces[:k]
    st.pop("seq_len", None)
    return st


def pack_tokens(iterator, empty_buffer_state: dict):
    """Concatenate documents and cut windows of ``output_seq_len + n_views - 1`` tokens that
    advance by ``output_seq_len``; each is returned as a (output_seq_len, n_views) array whose
    column v is the window shifted by v tokens."""
    out_len = empty_buffer_state["output_seq_len"]
    n_views = empty_buffer_state["n_views"]
    start = empty_buffer_state["start_token"]
    prev_state = empty_buffer_state["it_state"]
    cap = out_len + n_views - 1
    buf: list = []
    pieces: list = []
    for tokens, st in iterator:
        done = False
        while not done:
            assert start < len(tokens), f"Start token index {start} bigger than sequence {len(tokens)}"
            take = min(cap - len(buf), len(tokens) - start)
            buf.extend(tokens[start:start + take])
            start += take
            pieces.append(dict(start_token=start, seq_len=take, it_state=prev_state, output_seq_len=out_len,
                               n_views=n_views))
            assert len(buf) <= cap, "Buffer overflow"
            if len(buf) == cap:
                arr = np.array(buf)
                assert arr.ndim == 1, "Iterator should return 1D sequences"
                win = np.lib.stride_tricks.sliding_window_view(arr, n_views, axis=0)
                resume = _resume_point(start - (n_views - 1), pieces)
                buf = buf[out_len:]
                yield win, resume
            if start == len(tokens):
                start = 0
                done = True
                prev_state = st


# ----------------------------------------------------------------------------- batching
def batch_and_shuffle_prefetched_sequences(data_loader, batch_size: int, prefetch_size: int, seq_len: int,
                                           n_views: int, state: dict):
    """Keep ``prefetch_size * batch_size`` windows in a buffer that is reshuffled once per pass,
    hand out consecutive groups of ``batch_size`` and refill each group right after use.
    The state records the upstream position and rng at the start of the pass plus the index
    of the next group, which is enough to rebuild the buffer bit for bit."""
    n = prefetch_size * batch_size
    pool = -np.ones((n, seq_len, n_views), dtype=int)
    rng = np.random.default_rng()
    rng.bit_generator.state = state["rng_state"]
    idx = state["seq_idx"]
    assert 0 <= idx < prefetch_size, "Prefetch state seq_idx should be in 0 <= seq_idx < prefetch_size."
    pass_rng_state = state["rng_state"]
    pass_it_state = state["it_state"]
    upstream_state = None
    for i in range(n):
        pool[i], upstream_state = next(data_loader)
    rng.shuffle(pool, axis=0)
    for i in range(idx * batch_size):  # replay the refills of the groups already consumed
        pool[i], _ = next(data_loader)
    while True:
        if idx == prefetch_size - 1:
            pass_it_state = upstream_state
            pass_rng_state = rng.bit_generator.state
        out_state = dict(it_state=pass_it_state, seq_idx=(idx + 1) % prefetch_size, rng_state=pass_rng_state,
                         batch_size=batch_size, prefetch_size=prefetch_size)
        yield pool[idx * batch_size:(idx + 1) * batch_size].copy(), out_state
        last = None
        for i in range(batch_size):
            pool[idx * batch_size + i], last = next(data_loader)
        if idx == prefetch_size - 1:
            upstream_state = last
            rng.shuffle(pool, axis=0)
        idx = (idx + 1) % prefetch_size


# ----------------------------------------------------------------------------- sharding
def find_and_sanitize_chunks(dataset_path: str, world_size: int, file_pattern: str = TRAIN_DATA_FILE_PATTERN):
    chunks = sorted(str(p) for p in Path(dataset_path).glob(file_pattern))
    assert len(chunks) > 0, f"No valid chunks in {dataset_path}"
    if len(chunks) > world_size:
        chunks = chunks[:world_size]
    else:
        assert world_size % len(chunks) == 0, "World size should be a multiple of number of chunks"
    return chunks


def distribute_data_to_rank(dataset_path: str, rank: int, world_size: int, file_pattern: str):
    """Each chunk file is shared by world_size / n_chunks ranks that interleave its lines."""
    chunks = find_and_sanitize_chunks(dataset_path, world_size, file_pattern)
    per = world_size // len(chunks)
    params = [dict(file_path=c, position=0, block_size=per, offset=i, current_iter=0)
              for c in chunks for i in range(per)]
    return params[rank]


def init_choice_state(root_dir, sources, seed, rank, world_size, file_pattern):
    src = {s: distribute_data_to_rank(os.path.join(root_dir, s), rank, world_size, file_pattern) for s in sources}
    rng_state = np.random.default_rng((seed, rank, world_size)).bit_generator.state
    return dict(root_dir=root_dir, sources=sources, source_to_state=src, rng_state=rng_state)


def init_state(root_dir, sources, batch_size, prefetch_size, seq_len, n_views, seed, rank, world_size, add_bos,
               add_eos, tokenizer_name, tokenizer_path=None, file_pattern=TRAIN_DATA_FILE_PATTERN, regex=None):
    multi = init_choice_state(root_dir, sources, seed, rank, world_size, file_pattern)
    tok = dict(it_state=multi, add_bos=add_bos, add_eos=add_eos, name=tokenizer_name, path=tokenizer_path)
    if regex:
        tok["regex"] = regex
    pack = dict(start_token=0, it_state=tok, output_seq_len=seq_len, n_views=n_views, seq_len=0)
    rng_state = np.random.default_rng((seed + 1, rank, world_size)).bit_generator.state
    return dict(it_state=pack, seq_idx=0, rng_state=rng_state, batch_size=batch_size, prefetch_size=prefetch_size)


def setup_sources(multi_state):
    out = {}
    for s in multi_state["sources"]:
        js = multi_state["source_to_state"][s]
        out[s] = loop_on_jsonl(js["file_path"], js["position"], js["block_size"], js["offset"], js["current_iter"])
    return out


@contextlib.contextmanager
def build_dataloader(state: dict):
    """Context manager yielding the batch iterator rebuilt from ``state``."""
    if state.get("synthetic") is not None:
        it = synthetic_batches(state)
        try:
            yield it
        finally:
            it.close()
        return
    pack_state = state["it_state"]
    tok_state = pack_state["it_state"]
    multi = tok_state["it_state"]
    srcs = setup_sources(multi)
    it = choose_source(srcs, multi["source_to_state"], multi["root_dir"], multi["sources"], multi["rng_state"])
    it = tokenize(it, tok_state["add_bos"], tok_state["add_eos"], tok_state["name"], tok_state["path"],
                  tok_state.get("regex"))
    it = pack_tokens(it, pack_state)
    it = batch_and_shuffle_prefetched_sequences(it, state["batch_size"], state["prefetch_size"],
                                                pack_state["output_seq_len"], pack_state["n_views"], state)
    try:
        yield it
    finally:
        it.close()
        for s in srcs.values():
            s.close()


# ----------------------------------------------------------------------------- synthetic
def synthetic_batches(state: dict):
    """Uniform-random token ids in [0, vocab): batches of (batch, seq_len, n_views) windows of one
    random stream per rank, resumable from the batch counter alone."""
    cfg = state["synthetic"]
    bs, sl, nv, vocab = state["batch_size"], cfg["seq_len"], cfg["n_views"], cfg["vocab_size"]
    step = state["seq_idx"]
    while True:
        rng = np.random.default_rng((cfg["seed"], cfg["rank"], cfg["world_size"], step))
        stream = rng.integers(0, vocab, size=(bs, sl + nv - 1), dtype=np.int64)
        probs = cfg.get("level_probs")
        if probs:  # pooling levels: level >= l with probability probs[l-1]; every row starts at the deepest level
            u = rng.random(size=stream.shape)
            levels = sum((u < p).astype(np.int64) for p in probs)
            levels[:, 0] = len(probs)
            stream = stream | (levels << LEVEL_SHIFT)
        batch = np.lib.stride_tricks.sliding_window_view(stream, nv, axis=1).copy()
        step += 1
        yield batch, {**state, "seq_idx": step}


def init_synthetic_state(batch_size, seq_len, n_views, vocab_size, seed, rank, world_size, level_probs=None):
    cfg = dict(seq_len=seq_len, n_views=n_views, vocab_size=vocab_size, seed=seed, rank=rank, world_size=world_size)
    if level_probs:
        cfg["level_probs"] = sorted((float(p) for p in level_probs), reverse=True)
    return dict(it_state=None, seq_idx=0, rng_state=None, batch_size=batch_size, prefetch_size=1, synthetic=cfg)


# ----------------------------------------------------------------------------- async
def feed_buffer(queue: Queue, stop_event, iterator_builder):
    """Producer process body: push batches until asked to stop; never blocks for more than 0.1 s."""
    with iterator_builder() as iterator:
        for item in iterator:
            while not stop_event.is_set():
                try:
                    queue.put(item, timeout=0.1)
                    break
                except Full:
                    pass
            if stop_event.is_set():
                break


def consume_buffer(producer: Process, queue: Queue):
    """Consumer side: raises as soon as the producer process is gone."""
    while producer.exitcode is None:
        try:
            yield queue.get(timeout=0.1)
        except Empty:
            pass
    raise RuntimeError("Data loader quit unexpectedly, real error has been raised previously")


@contextlib.contextmanager
def async_iterator(buffer_size: int, iterator_builder):
    queue = Queue(maxsize=buffer_size)
    stop_event = Event()
    producer = Process(target=feed_buffer, args=(queue, stop_event, iterator_builder), daemon=True)
    logger.info("Async dataloader started")
    producer.start()
    consumer = consume_buffer(producer, queue)
    try:
        yield consumer
    finally:
        stop_event.set()
        consumer.close()
        producer.join(timeout=0.2)
        if producer.exitcode is None:
            logger.info(f"Killing async data process {producer.pid} ...")
            producer.kill()
        else:
            logger.info(f"Async data process {producer.pid} exited with code {producer.exitcode}")
        logger.info("Async dataloader cleaned up")


# ----------------------------------------------------------------------------- args
@dataclass
class DataArgs:
    root_dir: Optional[str] = None
    sources: Dict[str, float] = field(default_factory=dict)
    batch_size: int = 2
    seq_len: int = 2048
    n_views: int = 2
    seed: int = 42
    add_bos: bool = True
    add_eos: bool = True
    load_async: bool = True
    prefetch_size: int = 64
    tokenizer: TokenizerArgs = field(default_factory=TokenizerArgs)
    # hierarchical byte models: pooling strategy, one rule per level (apps/aunet/data/data.py:746 of the reference)
    regex: Optional[RegexArgs] = None


def init_dataloader_state_from_args(args: DataArgs, rank: int, world_size: int, vocab_size: Optional[int] = None):
    """``sources: {synthetic: 1.0}`` with no root_dir selects the uniform-random token source."""
    if args.root_dir is None and list(args.sources.keys()) == ["synthetic"]:
        assert vocab_size is not None and vocab_size > 0
        probs = None
        if args.regex is not None and args.regex.strategy:  # word-like boundary rates, thinning with depth
            probs = [0.2 * 0.3 ** l for l in range(len(args.regex.strategy))]
        return init_synthetic_state(args.batch_size, args.seq_len, args.n_views, vocab_size, args.seed, rank,
                                    world_size, level_probs=probs)
    regex = {"strategy": dict(args.regex.strategy)} if args.regex is not None and args.regex.strategy else None
    return init_state(root_dir=args.root_dir, sources=args.sources, seq_len=args.seq_len,
                      batch_size=args.batch_size, prefetch_size=args.prefetch_size, n_views=args.n_views,
                      seed=args.seed, rank=rank, world_size=world_size, tokenizer_name=args.tokenizer.name,
                      tokenizer_path=args.tokenizer.path, add_bos=args.add_bos, add_eos=args.add_eos, regex=regex)


def build_dataloader_from_args(args: DataArgs, state: Optional[dict] = None):
    builder = partial(build_dataloader, state)
    if args.load_async:
        return async_iterator(args.prefetch_size, builder)
    return builder()
