"""Behaviour list of the decontamination index (C++ ``native.decontam``; reference
data/decontam/tests/{ngrams,index,method_hash,ngram_match,scan_text,scan_shard,planted,
fail_closed,report,embedding}.rs): eight-word grams, fail-closed scans on an empty index,
insertion-order independence of the method hash, unique unions of hits over a shard."""
import hashlib
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

DC = native.decontam

Q1 = "What is the capital city of the ancient kingdom of Lydia in Anatolia"
Q2 = "Compute the integral of x squared from zero to one exactly please"
Q3 = "Name the river that flows through the old town of Regensburg in Bavaria"


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def index(*items):
    ix = DC.Index()
    for suite, iid, text in items or (("mmlu", "q1", Q1), ("aime", "p7", Q2)):
        ix.add(DC.EvalItem(suite, iid, text))
    return ix


def hits(found):
    return sorted((h.suite, h.item_id, h.method) for h in found)


# ------------------------------------------------------------------------------ n-grams
def test_grams_are_eight_lowercased_words_overlapping():
    assert DC.NGRAM_N == 8
    words = [f"w{i}" for i in range(11)]
    grams = DC.ngrams(" ".join(words))
    assert grams == [" ".join(words[i:i + 8]) for i in range(4)] and all(len(g.split(" ")) == 8 for g in grams)
    assert DC.ngrams("A  b\tC\nd E f G h") == ["a b c d e f g h"] == DC.ngrams("a b c d e f g h")
    assert DC.ngrams("") == [] and DC.ngrams("one two three four five six seven") == []
    assert DC.ngrams("Hello, world! it's a fine-day (really) now ok?") == ["hello, world! it's a fine-day (really) now ok?"]
    rng = random.Random(0)
    for _ in range(50):
        n = rng.randint(0, 20)
        text = "  ".join(rng.choice(["Alpha", "beta,", "GAMMA", "d", "e.e"]) for _ in range(n))
        got = DC.ngrams(text)
        assert len(got) == max(0, n - 7) and got == DC.ngrams(text.upper()) == DC.ngrams(text)


# ------------------------------------------------------------------------------ index
def test_items_are_keyed_by_suite_and_id():
    ix = DC.Index()
    assert len(ix) == 0
    ix.add(DC.EvalItem("mmlu", "q1", Q1))
    ix.add(DC.EvalItem("aime", "q1", Q2))                              # same id, other suite
    ix.add(DC.EvalItem("mmlu", "q2", Q3))                              # same suite, other id
    assert len(ix) == 3
    e = err(lambda: ix.add(DC.EvalItem("mmlu", "q1", "different text")))
    assert e.kind == "Config" and "mmlu" in str(e) and "q1" in str(e) and len(ix) == 3


def test_an_empty_index_fails_closed_everywhere():
    ix = DC.Index()
    for call in (ix.method_hash, lambda: ix.ngram_match(Q1), lambda: ix.scan_text(Q1), lambda: ix.scan_shard([Q1]),
                 lambda: ix.scan_shard([]), lambda: ix.planted_caught([], [Q1]), lambda: ix.embedding_match(Q1)):
        assert err(call).kind == "MissingIndex"                        # never "clean"


# ------------------------------------------------------------------------------ method hash
def test_method_hash_depends_on_contents_not_on_insertion_order():
    items = [("mmlu", "q1", Q1), ("aime", "p7", Q2), ("mmlu", "q0", Q3)]
    want = hashlib.sha256()
    want.update(b"prometheus-decontam/v1\nngram_n=8\nembed_model=\n")
    for s, i, t in sorted(items):
        want.update(s.encode() + b"\0" + i.encode() + b"\0" + t.encode() + b"\n")
    seen = set()
    for order in (items, items[::-1], items[1:] + items[:1]):
        h = index(*order).method_hash()
        seen.add(h)
        assert h == want.hexdigest() and h == h.lower() and len(h) == 64
    assert len(seen) == 1
    changed_text = index(("mmlu", "q1", Q1 + " now"), *items[1:]).method_hash()
    fewer = index(*items[:2]).method_hash()
    renamed = index(("mmlu", "q9", Q1), *items[1:]).method_hash()
    assert len({want.hexdigest(), changed_text, fewer, renamed}) == 4


# ------------------------------------------------------------------------------ matching
def test_one_shared_gram_is_a_hit_and_seven_words_are_not():
    ix = index()
    eight = " ".join(Q1.split()[2:10])
    seven = " ".join(Q1.split()[2:9])
    assert hits(ix.ngram_match(eight)) == [("mmlu", "q1", "ngram")]
    assert hits(ix.ngram_match("intro words first then " + eight + " and a long tail after it")) == [("mmlu", "q1", "ngram")]
    assert ix.ngram_match(seven) == [] and ix.ngram_match(seven + " something else entirely here") == []
    assert hits(ix.ngram_match("  ".join(w.upper() for w in eight.split()))) == [("mmlu", "q1", "ngram")]
    assert ix.ngram_match("") == [] and ix.ngram_match("nothing shared with the evaluation items at all here") == []
    short = index(("s", "i", "only seven words in this item here"))
    assert short.ngram_match("only seven words in this item here") == []     # an item below eight words cannot match
    assert hits(ix.ngram_match(Q1 + " ... " + Q2)) == [("aime", "p7", "ngram"), ("mmlu", "q1", "ngram")]


def test_scan_text_reports_status_every_suite_and_the_method_hash():
    ix = index(("mmlu", "q1", Q1), ("aime", "p7", Q2), ("gpqa", "g1", Q3))
    clean = ix.scan_text("a document about growing tomatoes in a cold northern climate zone all year")
    assert (clean.status, clean.hits, clean.against, clean.method_hash) == ("clean", [], ["aime", "gpqa", "mmlu"], ix.method_hash())
    flagged = ix.scan_text("someone asked: " + Q2.lower())
    assert flagged.status == "flagged" and hits(flagged.hits) == [("aime", "p7", "ngram")]
    assert flagged.against == ["aime", "gpqa", "mmlu"]                  # all suites checked, not only the one that hit
    assert ix.scan_text("").status == "clean"


def test_scan_shard_unions_hits_uniquely():
    ix = index()
    assert ix.scan_shard([]).status == "clean" and ix.scan_shard(["", "nothing to see here"]).status == "clean"
    rep = ix.scan_shard(["clean text", Q1, "more clean text", Q1.upper(), Q2 + " " + Q1])
    assert rep.status == "flagged" and hits(rep.hits) == [("aime", "p7", "ngram"), ("mmlu", "q1", "ngram")]
    assert rep.method_hash == ix.method_hash() and rep.against == ["aime", "mmlu"]


def test_planted_items_must_all_be_caught():
    ix = index()
    p1, p2 = DC.EvalItem("mmlu", "q1", Q1), DC.EvalItem("aime", "p7", Q2)
    ix.planted_caught([p1, p2], ["x", Q1, Q2])
    ix.planted_caught([], ["x"])
    assert err(lambda: ix.planted_caught([p1, p2], [Q1])).kind == "PlantedMiss"          # every planted item
    e = err(lambda: ix.planted_caught([p2], [Q1]))                                        # another item's hit does not count
    assert e.kind == "PlantedMiss" and "p7" in str(e)


def test_embedding_match_without_an_embedder_is_an_error_not_clean():
    ix = index()
    e = err(lambda: ix.embedding_match("anything"))
    assert e.kind == "Config" and "embedder" in str(e)
    assert ix.scan_text("anything at all that is not an evaluation item in the index").status == "clean"   # the scan needs none
