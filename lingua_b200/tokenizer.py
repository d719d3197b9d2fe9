"""Tokenizers: ``bytes`` (no files needed), ``mock`` (identity), ``sp`` (SentencePiece) and
``tiktoken`` (byte-pair ranks file plus 256 special tokens placed after the ranks).

Same ids and special-token conventions as lingua/tokenizer.py (ByteTokenizer :48: bytes are
ids 0-255, bos 256, eos 257; TikTokenTokenizer :130: specials at ``len(ranks) + k``, text
encoded in chunks of 400k characters).
"""
from __future__ import annotations

import abc
import logging
import os
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Tuple

logger = logging.getLogger(__name__)


@dataclass
class TokenizerArgs:
    name: str = "bytes"
    path: Optional[str] = None


class Tokenizer(abc.ABC):
    n_words: int
    bos_id: int
    eos_id: int

    @abc.abstractmethod
    def encode(self, text, add_bos: bool = False, add_eos: bool = False) -> List[int]: ...

    @abc.abstractmethod
    def decode(self, tokens: List[int]) -> str: ...

    @abc.abstractmethod
    def get_token_offsets(self, text: str, tokens: Optional[List[int]] = None) -> Tuple[List[str], List[int]]:
        """Sub-strings and start offsets of every token of ``text`` (used by evaluation)."""


class MockTokenizer(Tokenizer):
    """Inputs are already token lists; encode is the identity."""

    n_words = 256
    bos_id = 0
    eos_id = 1

    def encode(self, tokens, add_bos=False, add_eos=False):
        return tokens

    def decode(self, tokens):
        return " ".join(str(t) for t in tokens)

    def get_token_offsets(self, text, tokens=None):
        raise NotImplementedError


class ByteTokenizer(Tokenizer):
    def __init__(self) -> None:
        self.bos_id, self.eos_id, self.n_words = 256, 257, 258

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        ids = list(text.encode())
        if add_bos:
            ids.insert(0, self.bos_id)
        if add_eos:
            ids.append(self.eos_id)
        return ids

    def decode(self, tokens: List[int]) -> str:
        return bytes(t for t in tokens if t < 256).decode("utf-8", errors="backslashreplace")

    def get_token_offsets(self, text, tokens=None):
        tokens = self.encode(text) if tokens is None else tokens
        chars, offsets, pos = [], [], 0
        for t in tokens:
            if t >= 256:
                continue
            ch = bytes([t]).decode("utf-8", errors="ignore")
            if ch:
                chars.append(ch)
                offsets.append(pos)
            pos += len(ch.encode("utf-8"))
        return chars, offsets


class SentencePieceTokenizer(Tokenizer):
    def __init__(self, model_path: str) -> None:
        from sentencepiece import SentencePieceProcessor

        assert os.path.isfile(model_path), model_path
        self.sp_model = SentencePieceProcessor(model_file=model_path)
        self.n_words = self.sp_model.vocab_size()
        self.bos_id, self.eos_id, self.pad_id = self.sp_model.bos_id(), self.sp_model.eos_id(), self.sp_model.pad_id()
        logger.info(f"#words: {self.n_words} - BOS ID: {self.bos_id} - EOS ID: {self.eos_id}")

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        assert isinstance(text, str)
        return [self.bos_id] * add_bos + self.sp_model.encode(text) + [self.eos_id] * add_eos

    def decode(self, tokens: List[int]) -> str:
        return self.sp_model.decode(tokens)

    def get_token_offsets(self, text, tokens=None):
        pieces = self.sp_model.encode_as_immutable_proto(text).pieces
        return [p.surface for p in pieces], [p.begin for p in pieces]


TIKTOKEN_PATTERN = (
    r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
)
TIKTOKEN_NAMED_SPECIALS = {
    "<|begin_of_text|>": 0, "<|end_of_text|>": 1, "<|fim_prefix|>": 2, "<|fim_middle|>": 3,
    "<|fim_end_fill|>": 253, "<|fim_pad|>": 254, "<|fim_suffix|>": 255,
}
TIKTOKEN_MAX_ENCODE_CHARS = 400_000


class TikTokenTokenizer(Tokenizer):
    def __init__(self, model_path: str) -> None:
        import tiktoken
        from tiktoken.load import load_tiktoken_bpe

        ranks = load_tiktoken_bpe(model_path)
        specials = dict(TIKTOKEN_NAMED_SPECIALS)
        used = set(specials.values())
        for i in range(256):
            if i not in used:
                specials[f"<|reserved_special_token_{i}|>"] = i
        specials = {k: v + len(ranks) for k, v in specials.items()}
        self.tkt_model = tiktoken.core.Encoding(name=Path(model_path).stem, pat_str=TIKTOKEN_PATTERN,
                                                mergeable_ranks=ranks, special_tokens=specials)
        self.bos_id = self.tkt_model.encode_single_token("<|begin_of_text|>")
        self.eos_id = self.tkt_model.encode_single_token("<|end_of_text|>")
        self.n_words = self.tkt_model.n_vocab
        logger.info(f"#words: {self.n_words} - BOS ID: {self.bos_id} - EOS ID: {self.eos_id}")

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        assert isinstance(text, str)
        parts = [text[i:i + TIKTOKEN_MAX_ENCODE_CHARS] for i in range(0, len(text), TIKTOKEN_MAX_ENCODE_CHARS)]
        ids: List[int] = [self.bos_id] if add_bos else []
        for chunk in self.tkt_model.encode_ordinary_batch(parts):
            ids.extend(chunk)
        if add_eos:
            ids.append(self.eos_id)
        return ids

    def decode(self, tokens: List[int]) -> str:
        return self.tkt_model.decode(tokens)

    def get_token_offsets(self, text, tokens=None):
        if tokens is None:
            tokens = self.tkt_model.encode(text, allowed_special="all")
        offsets, n_chars = [], 0
        for tb in self.tkt_model.decode_tokens_bytes(tokens):
            # a token that starts inside a multi-byte character belongs to the previous character
            offsets.append(max(0, n_chars - (0x80 <= tb[0] < 0xC0)))
            n_chars += sum(1 for c in tb if not 0x80 <= c < 0xC0)
        return [text[s:e] for s, e in zip(offsets, offsets[1:] + [None])], offsets


def build_tokenizer(name: str, path: Optional[str] = None) -> Tokenizer:
    if name == "bytes":
        return ByteTokenizer()
    if name == "mock":
        return MockTokenizer()
    if name == "sp":
        return SentencePieceTokenizer(path)
    if name == "tiktoken":
        return TikTokenTokenizer(path)
    raise NotImplementedError(f"{name} tokenizer type is not implemented")
