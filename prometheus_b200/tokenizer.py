"""Byte-fallback BPE tokenizer: the Python face of the C++ implementation.

Id layout: 4 specials (bos, eos, pad, unk), 256 byte tokens, 10 ARC colour tokens, merges
from id 270. ``Tokenizer.train`` / ``encode`` / ``decode`` / ``encode_grid`` / ``freeze`` /
``save`` / ``load`` / ``to_contract`` keep the names and artifacts (``vocab.jsonl``,
``tokenizer.json``) of the reference's ``tokenizer/__init__.py`` (:282-517); the work is done by
``native.tokenizer`` so the loader, the data pipeline and this module share one vocabulary
implementation. ``encode_batch`` returns padded id tensors for the trainer.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Sequence

import torch

from .native import NativeError
from .native import tokenizer as _n

SCHEMA_ID = "prometheus.tokenizer"
VOCAB_SCHEMA_ID = "prometheus.vocab"
SCHEMA_VERSION = 1
ALGORITHM = "byte_fallback_bpe"
PRODUCTION_VOCAB_SIZE = _n.PRODUCTION_VOCAB_SIZE
ARC_N_COLORS = _n.ARC_N_COLORS
FIRST_BYTE, FIRST_ARC, FIRST_MERGE = 4, 260, 270


class TokenizerError(ValueError):
    """Training, encoding or an artifact on disk is invalid."""


@dataclass(frozen=True)
class TrainConfig:
    tokenizer_id: str
    vocab_size: int
    byte_fallback: bool = True


def _wrap(fn, *args):
    try:
        return fn(*args)
    except NativeError as e:
        raise TokenizerError(str(e)) from None


def _ids(values, what: str) -> list:
    out = [int(v) for v in values]
    if any(v < 0 for v in out):
        raise TokenizerError(f"negative {what} {min(out)}")
    return out


class Tokenizer:
    def __init__(self, impl) -> None:
        self._t = impl

    @classmethod
    def train(cls, docs: Iterable[str], config: TrainConfig) -> "Tokenizer":
        return cls(_wrap(_n.Tokenizer.train, list(docs), config.tokenizer_id, int(config.vocab_size),
                         bool(config.byte_fallback)))

    @classmethod
    def load(cls, directory) -> "Tokenizer":
        return cls(_wrap(_n.Tokenizer.load, str(directory)))

    def save(self, directory) -> dict:
        """Writes ``vocab.jsonl`` and ``tokenizer.json``; returns the ``prometheus.vocab`` pointer."""
        return json.loads(_wrap(self._t.save, str(Path(directory))))

    def freeze(self, frozen_at: str) -> None:
        _wrap(self._t.freeze, frozen_at)

    def encode(self, text: str) -> list:
        return _wrap(self._t.encode, text)

    def decode(self, ids: Sequence[int]) -> str:
        return _wrap(self._t.decode, _ids(ids, "token id"))

    def encode_bytes(self, data: bytes) -> list:
        return _wrap(self._t.encode_bytes, data)

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        return bytes(_wrap(self._t.decode_bytes, _ids(ids, "token id")))

    def encode_grid(self, cells: Sequence[int]) -> list:
        """One token per cell (``FIRST_ARC + colour``) for the row-major flattening of a grid."""
        return _wrap(self._t.encode_grid, _ids(cells, "grid color"))

    def tokens_per_word(self, text: str) -> float:
        return _wrap(self._t.tokens_per_word, text)

    def to_contract(self) -> dict:
        return json.loads(_wrap(self._t.to_contract))

    def encode_batch(self, texts: Sequence[str], *, max_len: int | None = None, add_bos: bool = False,
                     add_eos: bool = False) -> tuple:
        """(ids, mask): int64 ``(B, L)`` padded with the pad id, and the 0/1 float mask of real tokens."""
        sp = self.special_tokens
        rows = []
        for t in texts:
            ids = ([sp["bos"]] if add_bos else []) + self.encode(t) + ([sp["eos"]] if add_eos else [])
            rows.append(ids[:max_len] if max_len else ids)
        width = max((len(r) for r in rows), default=0)
        ids = torch.full((len(rows), width), sp["pad"], dtype=torch.int64)
        mask = torch.zeros((len(rows), width))
        for i, r in enumerate(rows):
            ids[i, :len(r)] = torch.tensor(r, dtype=torch.int64)
            mask[i, :len(r)] = 1.0
        return ids, mask

    @property
    def special_tokens(self) -> dict:
        sp = self._t.special_tokens
        return dict(sp) if isinstance(sp, dict) else {k: getattr(sp, k) for k in ("bos", "eos", "pad", "unk")}

    vocab_size = property(lambda self: self._t.vocab_size)
    tokenizer_id = property(lambda self: self._t.tokenizer_id)
    vocab_hash = property(lambda self: self._t.vocab_hash() if callable(self._t.vocab_hash) else self._t.vocab_hash)
    corpus_hash = property(lambda self: self._t.corpus_hash)
    frozen = property(lambda self: self._t.frozen)
    frozen_at = property(lambda self: self._t.frozen_at)
    merges = property(lambda self: list(self._t.merges))


def baseline_byte_tokens_per_word(text: str) -> float:
    return _n.baseline_byte_tokens_per_word(text)
