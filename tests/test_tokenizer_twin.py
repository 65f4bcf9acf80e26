"""The plain-Python BPE (incremental pair counts, rank-ordered encoder) against the C++ tokenizer
(full recount, lowest-rank-pair search): same merges, same encodings, same vocabulary file hash."""
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.tokenizer_twin import FIRST_ARC, TokenizerTwin, TokenizerTwinError

N = native.tokenizer


def _docs(rng, alphabet, n_docs, max_len):
    return ["".join(rng.choice(alphabet) for _ in range(rng.randrange(0, max_len))) for _ in range(n_docs)]


@pytest.mark.parametrize("alphabet,vocab", [("ab", 290), ("abc ", 330), ("aab\n é", 300), ("the quick brown fox ", 400)])
def test_training_gives_the_same_merges_on_repetitive_corpora(alphabet, vocab):
    rng = random.Random(len(alphabet) * 1000 + vocab)
    for trial in range(6):
        docs = _docs(rng, alphabet, rng.randrange(1, 6), 60) + ["aaaa", "aaa", ""]
        mine = TokenizerTwin.train(docs, "t", vocab)
        theirs = N.Tokenizer.train(docs, "t", vocab, True)
        assert mine.merges == [tuple(m) for m in theirs.merges], (trial, docs)
        assert mine.corpus_hash == theirs.corpus_hash
        vh = theirs.vocab_hash() if callable(theirs.vocab_hash) else theirs.vocab_hash
        assert mine.vocab_hash() == vh


def test_encoding_decoding_and_artifacts_agree():
    rng = random.Random(7)
    corpus = ["the cat sat on the mat. the cat ate.", "naïve café — 北京 the mat", "aaaaaaa bbbb abababab"] * 3
    mine = TokenizerTwin.train(corpus, "tok-x", 420)
    theirs = N.Tokenizer.train(corpus, "tok-x", 420, True)
    assert len(mine.merges) > 50
    for _ in range(300):
        text = "".join(rng.choice("the cat mï北ab \n") for _ in range(rng.randrange(0, 40)))
        ids = mine.encode(text)
        assert ids == list(theirs.encode(text)), repr(text)
        assert mine.decode(ids) == text == theirs.decode(ids)
    blob = bytes(rng.randrange(256) for _ in range(200))
    assert mine.encode_bytes(blob) == list(theirs.encode_bytes(blob)) and mine.decode_bytes(mine.encode_bytes(blob)) == blob
    assert mine.encode_grid([0, 9, 3]) == [FIRST_ARC, FIRST_ARC + 9, FIRST_ARC + 3] == list(theirs.encode_grid([0, 9, 3]))
    import json
    want = json.loads(theirs.to_contract())
    got = mine.to_contract()
    assert got == {k: want[k] for k in got} and set(want) - set(got) <= {"frozen_at"}
    for bad, kind in ((lambda: mine.decode_bytes([3]), "UnknownId"), (lambda: mine.decode_bytes([10 ** 6]), "UnknownId"),
                      (lambda: mine.encode_grid([10]), "BadColor"), (lambda: TokenizerTwin.train(["a"], "t", 270), "VocabTooSmall"),
                      (lambda: TokenizerTwin.train(["a"], "", 300), "Message")):
        with pytest.raises(TokenizerTwinError) as e:
            bad()
        assert e.value.kind == kind


def test_training_stops_when_no_pair_is_left():
    mine = TokenizerTwin.train(["ab"], "t", 400)
    theirs = N.Tokenizer.train(["ab"], "t", 400, True)
    assert mine.merges == [tuple(m) for m in theirs.merges] == [(4 + ord("a"), 4 + ord("b"))]
    assert mine.encode("abab") == [270, 270]
