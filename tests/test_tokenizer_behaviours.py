"""Behaviour list of the byte-fallback BPE tokenizer (``prometheus_b200.tokenizer`` over the C++
``native.tokenizer``; reference tests/test_tokenizer.py, tokenizer/__init__.py:282-517): the id
layout, deterministic training, exact byte round trips (valid and invalid UTF-8), decode
errors, grid tokens, the tokens-per-word measure, freezing, the contract record and the
artifacts on disk."""
import hashlib
import json

import pytest
import torch

from prometheus_b200 import contracts, tokenizer as T
from prometheus_b200.tokenizer_twin import TokenizerTwin

DOCS = ["the cat sat on the mat", "the dog sat on the log", "a cat and a dog sat together on the mat", "héllo wörld ☃"]


def trained(vocab=300, docs=DOCS, tid="tok-test"):
    return T.Tokenizer.train(docs, T.TrainConfig(tid, vocab))


def test_layout_constants():
    assert (T.FIRST_BYTE, T.FIRST_ARC, T.FIRST_MERGE, T.ARC_N_COLORS) == (4, 260, 270, 10)
    assert T.ALGORITHM == "byte_fallback_bpe" and T.SCHEMA_ID == "prometheus.tokenizer" and T.PRODUCTION_VOCAB_SIZE >= 100_000
    t = trained()
    assert t.special_tokens == {"bos": 0, "eos": 1, "pad": 2, "unk": 3} and t.vocab_size == 300 and t.tokenizer_id == "tok-test"
    assert len(t.merges) <= 30 and all(a < 270 + i and b < 270 + i for i, (a, b) in enumerate(t.merges))    # a merge joins older tokens only


@pytest.mark.parametrize("kw", [dict(vocab_size=269), dict(vocab_size=270), dict(vocab_size=0), dict(byte_fallback=False), dict(tokenizer_id="")])
def test_training_argument_errors(kw):
    base = dict(tokenizer_id="t", vocab_size=300, byte_fallback=True)
    base.update(kw)
    with pytest.raises(T.TokenizerError):
        T.Tokenizer.train(DOCS, T.TrainConfig(**base))


def test_training_is_deterministic_and_agrees_with_the_other_implementation():
    a, b = trained(), trained()
    assert a.merges == b.merges and a.vocab_hash == b.vocab_hash and a.corpus_hash == b.corpus_hash
    twin = TokenizerTwin.train(DOCS, "tok-test", 300)
    assert [tuple(m) for m in a.merges] == twin.merges and a.vocab_hash == twin.vocab_hash()
    assert trained(docs=DOCS[::-1]).corpus_hash != a.corpus_hash                         # the corpus hash sees document order
    assert trained(vocab=280).merges == a.merges[:10]                                    # a smaller vocabulary is a prefix
    counts = {}
    for d in DOCS:
        ids = [4 + c for c in d.encode()]
        for p in zip(ids, ids[1:]):
            counts[p] = counts.get(p, 0) + 1
    top = max(counts.values())
    assert tuple(a.merges[0]) == min(p for p, n in counts.items() if n == top)           # most frequent pair, ties to the smallest


@pytest.mark.parametrize("text", ["", "a", "the cat", "unseen ☃ text 🙂", "tabs\tand\nnewlines\r\n", "日本語のテキスト", "the the the the", " leading and trailing "])
def test_text_round_trips_exactly(text):
    t = trained()
    ids = t.encode(text)
    assert t.decode(ids) == text and all(isinstance(i, int) and 4 <= i < 300 for i in ids)
    assert len(ids) <= len(text.encode())                                                # merges only ever shorten
    assert ids == TokenizerTwin.train(DOCS, "tok-test", 300).encode(text)


def test_arbitrary_bytes_round_trip():
    t = trained()
    for blob in (b"\xff\xfe\x00bad", bytes(range(256)), b"\xc3\x28", b"the cat\x80sat"):
        ids = t.encode_bytes(blob)
        assert t.decode_bytes(ids) == blob
    assert t.encode_bytes(b"the cat") == t.encode("the cat")
    assert len(t.encode("the cat sat on the mat")) < len("the cat sat on the mat")


def test_decode_errors():
    t = trained()
    for bad in ([0], [1], [2], [3], [299 + 1], [10 ** 6], [-1], [260], [269]):          # specials, out of range, colour tokens
        with pytest.raises(T.TokenizerError):
            t.decode(bad)
    unused = 270 + len(t.merges)
    if unused < 300:
        with pytest.raises(T.TokenizerError):
            t.decode([unused])                                                           # a merge slot that training never filled


def test_grid_tokens():
    t = trained()
    assert t.encode_grid(range(10)) == list(range(260, 270)) and t.encode_grid([]) == []
    assert t.encode_grid([0, 9, 3, 3]) == [260, 269, 263, 263]
    for bad in ([10], [-1], [0, 11]):
        with pytest.raises(T.TokenizerError):
            t.encode_grid(bad)
    assert set(t.encode_grid(range(10))).isdisjoint(t.encode("0123456789 the cat"))      # text never lands in the colour range


def test_tokens_per_word():
    t = trained()
    text = "the cat sat on the mat"
    assert t.tokens_per_word(text) == pytest.approx(len(t.encode(text)) / 6)
    assert t.tokens_per_word(text) < T.baseline_byte_tokens_per_word(text) == pytest.approx(len(text.encode()) / 6)
    assert t.tokens_per_word("") == 0.0 and t.tokens_per_word("   ") == 0.0
    assert t.tokens_per_word("zebra") == pytest.approx(len(t.encode("zebra")))


def test_freeze_and_contract():
    t = trained()
    before = t.vocab_hash
    rec = t.to_contract()
    contracts.validate(rec)
    assert rec["frozen"] is False and rec["vocab_hash"] == before and rec["algorithm"] == "byte_fallback_bpe" and rec["byte_fallback"] is True
    assert rec["special_tokens"] == {"bos": 0, "eos": 1, "pad": 2, "unk": 3} and rec["arc_grid_token_range"] == {"start": 260, "end": 270}
    t.freeze("2026-01-02T03:04:05Z")
    assert t.frozen and t.frozen_at == "2026-01-02T03:04:05Z" and t.vocab_hash == before and t.decode(t.encode("the cat")) == "the cat"
    t.freeze("2026-01-02T03:04:05Z")                                                     # same stamp again: fine
    with pytest.raises(T.TokenizerError):
        t.freeze("2027-01-01T00:00:00Z")
    frozen = t.to_contract()
    contracts.validate(frozen)
    assert frozen["frozen"] is True and frozen["frozen_at"] == "2026-01-02T03:04:05Z"


def test_artifacts_on_disk(tmp_path):
    t = trained()
    pointer = t.save(tmp_path / "tok")
    contracts.validate(pointer)
    assert pointer["schema_id"] == "prometheus.vocab" and pointer["artifact"]["content_hash"] == t.vocab_hash
    assert pointer["artifact"]["path"] == "vocab.jsonl" and pointer["vocab_size"] == 300 and pointer["special_token_ids"] == t.special_tokens
    vocab = (tmp_path / "tok" / "vocab.jsonl").read_bytes()
    assert pointer["artifact"]["bytes"] == len(vocab)
    assert hashlib.sha256(vocab).hexdigest() == t.vocab_hash
    rows = [json.loads(line) for line in vocab.decode().splitlines()]
    assert [r["kind"] for r in rows[:4]] == ["special"] * 4 and rows[4] == {"byte": 0, "id": 4, "kind": "byte"} and rows[-1]["kind"] == "header"
    assert sum(r["kind"] == "merge" for r in rows) == len(t.merges) and sum(r["kind"] == "arc" for r in rows) == 10
    back = T.Tokenizer.load(tmp_path / "tok")
    assert back.merges == t.merges and back.vocab_hash == t.vocab_hash and back.encode("the cat sat") == t.encode("the cat sat")
    assert json.loads((tmp_path / "tok" / "tokenizer.json").read_text())["tokenizer_id"] == "tok-test"
    with pytest.raises(T.TokenizerError):
        T.Tokenizer.load(tmp_path / "missing")
    (tmp_path / "tok" / "vocab.jsonl").write_bytes(vocab + b"{}\n")
    with pytest.raises(T.TokenizerError):
        T.Tokenizer.load(tmp_path / "tok")                                               # the file no longer matches its hash


def test_padded_batches():
    t = trained()
    ids, mask = t.encode_batch(["the cat", "a", ""], add_bos=True, add_eos=True)
    assert ids.dtype == torch.int64 and ids.shape == mask.shape and ids.shape[0] == 3
    assert ids[0, 0] == 0 and ids[1].tolist()[:3] == [0, 4 + ord("a"), 1] and ids[2].tolist()[:2] == [0, 1]
    assert mask.sum(1).tolist() == [len(t.encode("the cat")) + 2, 3.0, 2.0] and bool((ids[mask == 0] == 2).all())
    clipped, m2 = t.encode_batch(["the cat sat on the mat"], max_len=3)
    assert clipped.shape == (1, 3) and m2.sum() == 3
