"""Byte-fallback BPE restated in plain Python, with other algorithms than the C++ module.

``native.tokenizer`` recounts every adjacent pair for every merge and encodes by searching the
whole sequence for its lowest-ranked pair each round. This twin reaches the same results another
way, so that the two check each other (``tests/test_tokenizer_twin.py``):

* training keeps the pair counts between merges and only updates the pairs a merge touches
  (linked positions per document), picking the best pair by (count, smallest (left, right));
* encoding walks the merges in rank order, restricted to the ranks whose two parts occur in the
  sequence, and applies each one left to right. A merge can only create pairs whose rank is
  higher than its own (they contain the token it has just made), so this visits pairs in the
  order "lowest rank first, leftmost first" that defines the encoding;
* the vocabulary file is built line by line from the id layout and hashed with ``hashlib``.

Id layout (reference ``tokenizer/__init__.py:22-40``, ``tokenizer/src/lib.rs:28-33``): 0..3 bos,
eos, pad, unk; 4..259 the bytes; 260..269 the ten ARC colours; merges from 270.
"""
from __future__ import annotations

import hashlib
import json
from collections import Counter
from typing import Iterable, Sequence

FIRST_BYTE, FIRST_ARC, FIRST_MERGE, ARC_N_COLORS = 4, 260, 270, 10
SPECIALS = {"bos": 0, "eos": 1, "pad": 2, "unk": 3}
ALGORITHM = "byte_fallback_bpe"


class TokenizerTwinError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def _dumps(obj) -> str:
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=False)


class _Doc:
    """One training document as a doubly linked list of token slots, so that a merge rewrites
    two neighbours in place and only their two outer pairs change count."""

    __slots__ = ("tok", "prev", "next")

    def __init__(self, ids: list[int]):
        n = len(ids)
        self.tok = ids
        self.prev = list(range(-1, n - 1))
        self.next = list(range(1, n)) + [-1] if n else []


class TokenizerTwin:
    def __init__(self, tokenizer_id: str, vocab_size: int, merges: Sequence[tuple[int, int]],
                 corpus_hash: str | None = None):
        self.tokenizer_id, self.vocab_size = tokenizer_id, int(vocab_size)
        self.merges = [tuple(m) for m in merges]
        self.corpus_hash = corpus_hash
        self._rank = {m: r for r, m in enumerate(self.merges)}

    # ------------------------------------------------------------------ training
    @classmethod
    def train(cls, docs: Iterable[str | bytes], tokenizer_id: str, vocab_size: int) -> "TokenizerTwin":
        if not tokenizer_id:
            raise TokenizerTwinError("Message", "tokenizer_id must be non-empty")
        if vocab_size < FIRST_MERGE + 1:
            raise TokenizerTwinError("VocabTooSmall", f"vocab size {vocab_size} is too small for specials, bytes, and ARC colors")
        raw = [d.encode("utf-8") if isinstance(d, str) else bytes(d) for d in docs]
        corpus_hash = hashlib.sha256(b"\n".join(raw)).hexdigest()
        seqs = [_Doc([FIRST_BYTE + b for b in r]) for r in raw]
        counts: Counter = Counter()
        where: dict[tuple[int, int], set] = {}            # pair -> {(doc index, left slot)}
        for di, doc in enumerate(seqs):
            for i in range(len(doc.tok) - 1):
                pair = (doc.tok[i], doc.tok[i + 1])
                counts[pair] += 1
                where.setdefault(pair, set()).add((di, i))
        merges: list[tuple[int, int]] = []
        for new_id in range(FIRST_MERGE, vocab_size):
            live = [(n, p) for p, n in counts.items() if n > 0]
            if not live:
                break
            top = max(n for n, _p in live)
            best = min(p for n, p in live if n == top)
            merges.append(best)
            # occurrences left to right inside each document; overlapping ones ("aaa") are
            # consumed greedily from the left, like the rewrite pass of the reference trainer
            for di, i in sorted(where.pop(best, ())):
                doc = seqs[di]
                j = doc.next[i] if doc.tok[i] == best[0] else -1
                if j < 0 or doc.tok[i] != best[0] or doc.tok[j] != best[1]:
                    continue                                  # a neighbour was merged away already
                left, right = doc.prev[i], doc.next[j]

                def drop(a, b):
                    pair = (doc.tok[a], doc.tok[b])
                    counts[pair] -= 1
                    where.get(pair, set()).discard((di, a))

                def add(a, b):
                    pair = (doc.tok[a], doc.tok[b])
                    counts[pair] += 1
                    where.setdefault(pair, set()).add((di, a))

                if left >= 0:
                    drop(left, i)
                if right >= 0:
                    drop(j, right)
                counts[best] -= 1
                doc.tok[i], doc.tok[j] = new_id, -1           # slot j leaves the list
                doc.next[i] = right
                if right >= 0:
                    doc.prev[right] = i
                if left >= 0:
                    add(left, i)
                if right >= 0:
                    add(i, right)
            counts.pop(best, None)
        return cls(tokenizer_id, vocab_size, merges, corpus_hash)

    # ------------------------------------------------------------------ encode / decode
    def encode_bytes(self, data: bytes) -> list[int]:
        ids = [FIRST_BYTE + b for b in data]
        if len(ids) < 2 or not self.merges:
            return ids
        rank = self._rank
        while True:
            present = {rank[p] for p in zip(ids, ids[1:]) if p in rank}
            if not present:
                return ids
            r = min(present)                                  # ranks only grow from here on
            a, b = self.merges[r]
            out, i, n = [], 0, len(ids)
            while i < n:
                if i + 1 < n and ids[i] == a and ids[i + 1] == b:
                    out.append(FIRST_MERGE + r)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            ids = out

    def encode(self, text: str) -> list[int]:
        return self.encode_bytes(text.encode("utf-8"))

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        out = bytearray()
        stack = list(reversed([int(i) for i in ids]))
        while stack:
            t = stack.pop()
            if FIRST_BYTE <= t < FIRST_BYTE + 256:
                out.append(t - FIRST_BYTE)
            elif t >= FIRST_MERGE and t - FIRST_MERGE < len(self.merges):
                a, b = self.merges[t - FIRST_MERGE]
                stack += [b, a]
            else:
                raise TokenizerTwinError("UnknownId", f"unknown token id {t}")
        return bytes(out)

    def decode(self, ids: Sequence[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    @staticmethod
    def encode_grid(cells: Sequence[int]) -> list[int]:
        for c in cells:
            if not 0 <= int(c) < ARC_N_COLORS:
                raise TokenizerTwinError("BadColor", f"grid color {c} out of range")
        return [FIRST_ARC + int(c) for c in cells]

    # ------------------------------------------------------------------ artifacts
    def vocab_jsonl(self) -> str:
        rows = [{"id": i, "kind": "special", "name": n} for n, i in SPECIALS.items()]
        rows += [{"byte": b, "id": FIRST_BYTE + b, "kind": "byte"} for b in range(256)]
        rows += [{"color": c, "id": FIRST_ARC + c, "kind": "arc"} for c in range(ARC_N_COLORS)]
        rows += [{"id": FIRST_MERGE + r, "kind": "merge", "left": a, "right": b} for r, (a, b) in enumerate(self.merges)]
        rows.append({"algorithm": ALGORITHM, "byte_fallback": True, "kind": "header",
                     "tokenizer_id": self.tokenizer_id, "vocab_size": self.vocab_size})
        return "".join(_dumps(r) + "\n" for r in rows)

    def vocab_hash(self) -> str:
        return hashlib.sha256(self.vocab_jsonl().encode("utf-8")).hexdigest()

    def to_contract(self) -> dict:
        out = {"schema_id": "prometheus.tokenizer", "schema_version": 1, "tokenizer_id": self.tokenizer_id,
               "algorithm": ALGORITHM, "vocab_size": self.vocab_size, "byte_fallback": True,
               "special_tokens": dict(SPECIALS),
               "arc_grid_token_range": {"start": FIRST_ARC, "end": FIRST_ARC + ARC_N_COLORS},
               "vocab_hash": self.vocab_hash(), "frozen": False}
        if self.corpus_hash:
            out["corpus_hash"] = self.corpus_hash
        return out
