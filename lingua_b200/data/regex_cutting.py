"""Pooling boundaries of the hierarchical byte model, found with regular expressions.

Every byte of a document gets a level: 0 = stays at byte resolution only, ``l`` >= 1 = this byte is also a
position of stages 1..l. A strategy is one named rule per pooling level (first key = level 1):

* ``word*: "gs@a-b"``  -- boundaries at the last byte of every group of ``gs`` whitespace-terminated words
  plus the first byte of digit groups, punctuation runs and line ends; for the key ``word`` itself only the
  groups whose running number is a multiple of one of ``a, b, ...`` are kept,
* ``pretok*``          -- the first byte of every pre-tokenisation piece (word, number, punctuation, space run),
* ``punct*``           -- the first byte of digit triplets, punctuation runs and line ends.

Behaviour follows apps/aunet/data/regex_cutting.py:76-218 of the reference; the merge of several levels is
done with one dictionary pass instead of the reference's back-to-front deque walk (same mask)."""
from __future__ import annotations

import logging
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

try:  # the third-party engine: \p{..} classes and possessive quantifiers
    import regex as re
except ImportError:  # pragma: no cover
    re = None

logger = logging.getLogger(__name__)

_START_PRETOK = r"( ?\p{L}{1,16})|\p{N}{1,3}| ?([^\s\p{L}\p{N}]){1,3}+[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+"
_START_WORD = r"\p{N}{1,3}|(?:[^\s\p{L}\p{N}]{1,3}[\r\n]*)|\s*[\r\n]"
_END_WORD = r"(\S+?\s){%d}"
_START_PUNCT = r"\d{1,3}(?=(\d{3})+(?!\d))|\d{1,3}(?=\D|$)|([^\s\p{L}\p{N}]){1,3}+[\r\n]*|\s*[\r\n]"


@dataclass
class RegexArgs:
    strategy: Dict[str, str] = field(default_factory=dict)


def utf8_lead_length(first_byte: int) -> int:
    """Length announced by a UTF-8 lead byte; 0 for a continuation or invalid byte."""
    if first_byte < 0x80 or first_byte > 0xFF:  # ASCII, or a special token of the byte vocabulary
        return 1
    if first_byte >> 5 == 0b110:
        return 2
    if first_byte >> 4 == 0b1110:
        return 3
    if first_byte >> 3 == 0b11110:
        return 4
    return 0


def map_codepoint_to_byte(text: str) -> np.ndarray:
    """Index of the LAST byte of each character in the UTF-8 encoding of ``text``."""
    if not text:
        return np.zeros(0, dtype=np.int32)
    cp = np.frombuffer(text.encode("utf-32-le", errors="surrogatepass"), dtype=np.uint32)
    nbytes = 1 + (cp > 0x7F) + (cp > 0x7FF) + (cp > 0xFFFF)
    return (np.cumsum(nbytes) - 1).astype(np.int32)


def shrink_to_valid_bytes(tokens: Sequence[int]) -> Tuple[List[int], Optional[int], Optional[int]]:
    """Drop a truncated character at either end of a byte window. Returns (kept, start, end) with
    ``kept == tokens[start:end]``; ``start`` / ``end`` are None when nothing was cut on that side."""
    def is_cont(b):
        return 128 <= b < 192

    head = list(tokens[:5])
    n = 0
    while n < len(head) and is_cont(head[n]):
        n += 1
    start = n if n > 0 else None  # leading continuation bytes belong to a character that began earlier
    tail = list(tokens[:-5:-1])
    m = 0
    while m < len(tail) and is_cont(tail[m]):
        m += 1
    end = None
    if m < len(tail) and utf8_lead_length(tail[m]) != m + 1:
        end = -(m + 1)  # the last character is incomplete: cut it with its lead byte
    return list(tokens[start:end]), start, end


class RegexPool:
    """Compiled strategy: text -> (boundary offsets, their levels) and byte windows -> level masks."""

    def __init__(self, args: RegexArgs):
        assert re is not None, "the 'regex' package is required for regex pooling"
        self.strategy = dict(args.strategy)
        self.rules: List[Tuple[Optional["re.Pattern"], Optional["re.Pattern"], List[int]]] = []
        for name, spec in self.strategy.items():
            logger.info(f"Pooling level {len(self.rules) + 1}: {name} = {spec}")
            if name.startswith("word"):
                group, _, mods = str(spec).partition("@")
                keep = [int(m) for m in mods.split("-")] if name == "word" and mods else [1]
                self.rules.append((re.compile(_START_WORD), re.compile(_END_WORD % int(group)), keep))
            elif name.startswith("pretok"):
                self.rules.append((re.compile(_START_PRETOK), None, [1]))
            elif name.startswith("punct"):
                self.rules.append((re.compile(_START_PUNCT), None, [1]))
            else:
                raise ValueError(f"Unknown strategy: {name}")
        self.prefill_byte: Optional[List[deque]] = None

    @property
    def n_levels(self) -> int:
        return len(self.rules)

    def str_offset(self, text: str) -> Tuple[List[int], List[int]]:
        """Character offsets of the boundaries (ascending) and the 0-based rule index of each; where
        several rules mark the same character the deepest one wins."""
        best: Dict[int, int] = {}
        for lvl, (start_pat, end_pat, keep) in enumerate(self.rules):
            if start_pat is not None:
                for m in start_pat.finditer(text):
                    best[m.start()] = lvl
            if end_pat is not None:
                for n, m in enumerate(end_pat.finditer(text)):
                    if any(n % k == 0 for k in keep):
                        best[m.end() - 1] = lvl
        offsets = sorted(best)
        return offsets, [best[o] for o in offsets]

    def text_levels(self, text: str) -> List[int]:
        """Level of every UTF-8 byte of ``text`` (a boundary character marks its last byte)."""
        last_byte = map_codepoint_to_byte(text)
        if len(last_byte) == 0:
            return []
        levels = np.zeros(int(last_byte[-1]) + 1, dtype=np.int64)
        offsets, lv = self.str_offset(text)
        if offsets:
            levels[last_byte[np.asarray(offsets)]] = np.asarray(lv) + 1
        return levels.tolist()

    def get_levels_mask(self, tokens: Sequence[int]) -> List[int]:
        """Levels of a window of byte-vocabulary ids: special ids (> 255) split the window into text
        segments and get level 0, as do the bytes of a character cut by the window's ends."""
        kept, start, end = shrink_to_valid_bytes(tokens)
        out = [0] * len(kept)
        i = 0
        while i < len(kept):
            if kept[i] > 255:
                i += 1
                continue
            j = i
            while j < len(kept) and kept[j] <= 255:
                j += 1
            raw = bytes(kept[i:j])
            try:
                text = raw.decode("utf-8")
                out[i:j] = self.text_levels(text)
            except UnicodeDecodeError as e:
                logger.warning("Byte segment is not valid UTF-8, decoding with replacement characters: %s", e)
                lv = self.text_levels(raw.decode("utf-8", errors="replace"))
                out[i:j] = (lv + [0] * (j - i))[: j - i]
            i = j
        if start:
            out = [0] * start + out
        if end:
            out = out + [0] * (-end)
        return out

    # ---- generation: a bounded history per sequence, relabelled after every new byte
    def get_levels_mask_prefill(self, prompts: List[List[int]], size: Optional[int] = None,
                                force_first: bool = False) -> List[int]:
        """Levels of every prompt, concatenated; also starts the per-sequence history of ``size`` bytes."""
        self.prefill_byte, flat = [], []
        for p in prompts:
            self.prefill_byte.append(deque(p, maxlen=size))
            lv = self.get_levels_mask(p)
            if force_first and lv:
                lv[0] = max(lv)
            flat.extend(lv)
        return flat

    def get_levels_mask_gen(self, new_bytes: Sequence[int]) -> List[int]:
        """Level of the byte just generated for each sequence, given its history."""
        assert self.prefill_byte is not None, "call get_levels_mask_prefill first"
        assert len(new_bytes) == len(self.prefill_byte), "one new byte per prefilled sequence"
        out = []
        for hist, b in zip(self.prefill_byte, new_bytes):
            hist.append(int(b))
            out.append(self.get_levels_mask(list(hist))[-1])
        return out
