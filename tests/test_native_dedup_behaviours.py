"""Behaviour list of the dedup passes (C++ ``native.dedup``; reference data/dedup/tests/
{normalize,paragraphs,shingles,exact_hash,minhash,lsh,dedup_exact,dedup_near,dedup_corpus,
errors}.rs), with a plain-Python model of the three passes that is compared against the C++ on
generated corpora in every input order."""
import hashlib
import random
import struct
import unicodedata

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

DD = native.dedup
ZERO_WIDTH = "​‌‍⁠﻿᠎"


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


# ------------------------------------------------------------------------------ the model
def m_normalize(text):
    text = "".join(ch for ch in text if ch not in ZERO_WIDTH).lower()
    return " ".join(text.split())


def m_paragraphs(text):
    text = text.replace("\r\n", "\n")
    out, cur = [], []
    for line in text.split("\n"):
        if m_normalize(line) == "":
            if cur:
                out.append(m_normalize(" ".join(cur)))
                cur = []
        else:
            cur.append(line)
    if cur:
        out.append(m_normalize(" ".join(cur)))
    return [p for p in out if p]


def m_hash(text):
    return hashlib.sha256(m_normalize(text).encode()).hexdigest()


def m_shingles(text, n):
    w = m_normalize(text).split()
    return [" ".join(w[i:i + n]) for i in range(len(w) - n + 1)] if n and len(w) >= n else []


def m_signature(text, hashes=128, n=5):
    sh = set(m_shingles(text, n))
    if not sh:
        return None
    return [min(struct.unpack("<Q", hashlib.sha256(struct.pack("<Q", i) + s.encode()).digest()[:8])[0] for s in sh)
            for i in range(hashes)]


def m_bands(sig, bands=32, rows=4):
    return [hashlib.sha256(b"".join(struct.pack("<Q", v) for v in sig[rows * b:rows * b + rows])).digest()[:8] for b in range(bands)]


def keeper(doc):
    return (doc[2], doc[0])                                  # lowest content hash, then lowest id


def m_exact_document(docs):
    groups = {}
    for d in docs:
        groups.setdefault(m_hash(d[1]), []).append(d)
    kept, dropped = [], []
    for members in groups.values():
        members.sort(key=keeper)
        kept.append(members[0])
        dropped += members[1:]
    return kept, dropped


def m_exact_paragraph(docs):
    seen, kept, dropped = set(), [], []
    for d in sorted(docs, key=keeper):
        hs = {hashlib.sha256(p.encode()).hexdigest() for p in m_paragraphs(d[1])}
        if hs & seen:
            dropped.append(d)
        else:
            kept.append(d)
            seen |= hs
    return kept, dropped


def m_near(docs):
    keys = {d[0]: (m_bands(sig) if (sig := m_signature(d[1])) else None) for d in docs}
    # connected components of "shares a band key", by repeated merging of id sets
    comps = [{d[0]} for d in docs]
    by_id = {d[0]: d for d in docs}
    for b in range(32):
        buckets = {}
        for d in docs:
            if keys[d[0]]:
                buckets.setdefault(keys[d[0]][b], set()).add(d[0])
        for ids in buckets.values():
            touching = [c for c in comps if c & ids]
            if len(touching) > 1:
                merged = set().union(*touching)
                comps = [c for c in comps if not (c & ids)] + [merged]
    kept, dropped, clusters = [], [], []
    for c in comps:
        members = sorted((by_id[i] for i in c), key=keeper)
        kept.append(members[0])
        dropped += members[1:]
        if len(members) > 1:
            clusters.append((members[0][0], sorted(m[0] for m in members[1:])))
    return kept, dropped, clusters


def m_corpus(docs):
    k1, d1 = m_exact_document(docs)
    k2, d2 = m_exact_paragraph(k1)
    k3, d3, clusters = m_near(k2) if k2 else ([], [], [])
    ids = lambda ds: sorted(d[0] for d in ds)
    return ids(k3), ids(d1 + d2), ids(d3), sorted(clusters)


def native_docs(docs):
    return [DD.Document(*d) for d in docs]


def report(r):
    return sorted(r.kept), sorted(r.dropped_exact), sorted(r.dropped_near), sorted((c.kept, sorted(c.dropped)) for c in r.clusters)


# ------------------------------------------------------------------------------ text primitives
WORDS = "alpha bravo charlie delta echo foxtrot golf hotel india juliet kilo lima mike november oscar papa quebec romeo".split()


def test_normalize_rules_and_idempotence():
    rng = random.Random(3)
    pieces = WORDS + ["  ", "\t", "\n", "\r\n", "​", "﻿", "⁠", "É", "Ünï", "ß", "  ‍ "]
    for _ in range(300):
        s = "".join(rng.choice(pieces) + rng.choice(["", " ", ""]) for _ in range(rng.randint(0, 12)))
        s = "".join(ch.upper() if rng.random() < 0.3 else ch for ch in s)
        if unicodedata.normalize("NFC", s.lower()) != s.lower() or "ß".upper() in s:
            continue                                                          # keep to one-to-one case mappings
        got = DD.normalize(s)
        assert got == m_normalize(s) and DD.normalize(got) == got
        assert got == got.strip() and "  " not in got and not any(z in got for z in ZERO_WIDTH)
    assert DD.normalize("") == DD.normalize(" \t\r\n ") == DD.normalize("​﻿") == ""
    assert DD.normalize("a​b") == "ab" and DD.normalize("a ​ b") == "a b"   # stripping leaves no space behind


def test_exact_hash_is_sha256_of_the_normalised_text():
    assert DD.exact_hash("Hello World") == hashlib.sha256(b"hello world").hexdigest()
    assert DD.exact_hash("hello​WORLD") == hashlib.sha256(b"helloworld").hexdigest() != DD.exact_hash("hello world")
    assert DD.exact_hash("  hello   WORLD ") == DD.exact_hash("hello world") == DD.exact_hash("HELLO\nWORLD")
    assert DD.exact_hash("hello world") != DD.exact_hash("hello worlds")
    assert DD.exact_hash("") == hashlib.sha256(b"").hexdigest()


def test_paragraph_splitting():
    cases = ["one\n\ntwo", "one\n\n\n\n  \n\t\ntwo", "line a\nline b\n\nsecond", "\n\n  \nfirst\n\n", "", "a\r\n\r\nb",
             "MiXed​ Case\n\nNEXT", " \n \n ", "only one paragraph\nwith two lines"]
    for text in cases:
        assert DD.paragraphs(text) == m_paragraphs(text), text
    assert DD.paragraphs("line a\nline b\n\nsecond") == ["line a line b", "second"]
    assert DD.paragraphs("") == [] and DD.paragraphs("​\n\n​") == []       # empties after the strip are dropped


def test_shingles():
    assert DD.shingles("a b c d e", 3) == ["a b c", "b c d", "c d e"]
    assert DD.shingles("a b c", 1) == ["a", "b", "c"] and DD.shingles("a b c", 3) == ["a b c"]
    assert DD.shingles("a b", 3) == [] and DD.shingles("a b c", 0) == [] and DD.shingles("", 2) == []
    assert DD.shingles("  A   b\tC ", 2) == DD.shingles("a b c", 2)
    for text in (" ".join(WORDS), "x"):
        for n in (1, 2, 5, 30):
            assert DD.shingles(text, n) == m_shingles(text, n)


def test_minhash_signatures():
    a = " ".join(WORDS)
    close = " ".join(WORDS[:-1] + ["zulu"])
    far = " ".join(reversed(WORDS))
    sa, sc, sf = (DD.minhash_signature(t) for t in (a, close, far))
    assert sa == m_signature(a) and len(sa) == 128 and DD.minhash_signature("  " + a.upper()) == sa
    agree = lambda x, y: sum(p == q for p, q in zip(x, y))
    assert agree(sa, sc) > agree(sa, sf)                                    # more shared shingles, more equal minima
    small = DD.DedupConfig(shingle_size=2, num_hashes=8, bands=4, rows=2)
    assert len(DD.minhash_signature(a, small)) == 8 and DD.minhash_signature(a, small) == m_signature(a, 8, 2)
    assert DD.minhash_signature("too short") == DD.minhash_signature("") == [2 ** 64 - 1] * 128


def test_band_keys_and_their_configuration_errors():
    sig = DD.minhash_signature(" ".join(WORDS))
    keys = DD.lsh_band_keys(sig)
    assert len(keys) == 32 and [struct.pack("<Q", k) for k in keys] == m_bands(sig)
    assert DD.lsh_band_keys(list(sig)) == keys
    small = DD.DedupConfig(shingle_size=2, num_hashes=8, bands=4, rows=2)
    assert len(DD.lsh_band_keys(sig[:8], small)) == 4
    bad = [(DD.DedupConfig(5, 128, 16, 4), sig), (DD.DedupConfig(5, 128, 32, 4), sig[:64]), (DD.DedupConfig(5, 64, 32, 4), sig),
           (DD.DedupConfig(5, 0, 0, 4), []), (DD.DedupConfig(5, 0, 4, 0), []), (DD.DedupConfig(0, 128, 32, 4), sig),
           (DD.DedupConfig(5, 128, 2 ** 32, 2 ** 32), sig)]
    for cfg, s in bad:
        assert err(lambda: DD.lsh_band_keys(s, cfg)).kind == "Config"


# ------------------------------------------------------------------------------ passes
def test_document_grain_keeps_the_lowest_content_hash_then_the_lowest_id():
    docs = [("later", "Same Text", "b"), ("winner", "same  text", "a"), ("also", "SAME TEXT", "c"), ("unique", "other", "d"),
            ("z", "tie text", "h"), ("m", "Tie  Text", "h")]
    for order in (docs, docs[::-1], docs[2:] + docs[:2]):
        r = DD.dedup_exact(native_docs(order))
        assert (sorted(r.kept), sorted(r.dropped_exact)) == (["m", "unique", "winner"], ["also", "later", "z"])
        assert not r.dropped_near and not r.clusters
    # the given content hash is used as is, never recomputed from the text
    r = DD.dedup_exact(native_docs([("a", "same", "zzz"), ("b", "same", "000")]))
    assert r.kept == ["b"] and r.dropped_exact == ["a"]


def test_paragraph_grain_drops_a_whole_document_for_one_shared_paragraph():
    docs = [("long", "shared paragraph here\n\nplus plenty of own material", "2"), ("short", "Shared  PARAGRAPH here", "1"),
            ("other", "nothing in common", "3"), ("same-doc-level", "shared paragraph\nhere", "4")]
    r = DD.dedup_exact(native_docs(docs), "paragraph")
    assert sorted(r.kept) == ["other", "short"] and sorted(r.dropped_exact) == ["long", "same-doc-level"]   # the lower hash wins, even if shorter
    twins = DD.dedup_exact(native_docs([("a", "p one\n\np two", "9"), ("b", "p one\n\np two", "8")]), "paragraph")
    assert twins.kept == ["b"] and twins.dropped_exact == ["a"]
    assert err(lambda: DD.dedup_exact(native_docs(docs), "sentence")).kind == "Config"


def test_near_duplicates_cluster_through_shared_band_keys():
    base = " ".join(WORDS)
    docs = [("src", base, "1"), ("near-1", base.replace("romeo", "zulu"), "2"), ("near-2", base.replace("alpha", "zulu"), "0"),
            ("far", " ".join(reversed(WORDS)), "3"), ("tiny-a", "hi", "4"), ("tiny-b", "hi", "5")]
    r = DD.dedup_near(native_docs(docs))
    assert sorted(r.kept) == ["far", "near-2", "tiny-a", "tiny-b"]          # texts too short to shingle never join anything
    assert [(c.kept, sorted(c.dropped)) for c in r.clusters] == [("near-2", ["near-1", "src"])] and not r.dropped_exact
    assert report(DD.dedup_near(native_docs(docs[::-1]))) == report(r)
    for cfg in (DD.DedupConfig(5, 128, 16, 4), DD.DedupConfig(0, 128, 32, 4), DD.DedupConfig(5, 0, 0, 0)):
        assert err(lambda: DD.dedup_near(native_docs(docs), cfg)).kind == "Config"
        assert err(lambda: DD.dedup_corpus(native_docs(docs), cfg)).kind == "Config"
    assert sorted(DD.dedup_exact(native_docs(docs)).kept) == ["far", "near-1", "near-2", "src", "tiny-a"]   # exact pass has no config to reject


def test_empty_corpora_are_errors_and_a_single_document_is_kept():
    for fn in (DD.dedup_exact, lambda d: DD.dedup_exact(d, "paragraph"), DD.dedup_near, DD.dedup_corpus):
        err(lambda: fn([]))
    r = DD.dedup_corpus(native_docs([("only", "just one document", "1")]))
    assert report(r) == (["only"], [], [], [])


def _generated_corpus(rng, n):
    docs = []
    for i in range(n):
        roll = rng.random()
        if docs and roll < 0.15:                                            # exact copy, differently spaced and cased
            src = rng.choice(docs)[1]
            text = "  ".join(w.upper() if rng.random() < 0.5 else w for w in src.replace("\n\n", " \n\n ").split(" "))
        elif docs and roll < 0.3:                                           # shares one paragraph
            text = rng.choice(rng.choice(docs)[1].split("\n\n")) + "\n\n" + " ".join(rng.choices(WORDS, k=12))
        elif docs and roll < 0.45:                                          # one word changed
            w = rng.choice(docs)[1].split(" ")
            w[rng.randrange(len(w))] = "zulu"
            text = " ".join(w)
        elif roll < 0.5:
            text = rng.choice(["hi", "", "ok then"])
        else:
            text = "\n\n".join(" ".join(rng.choices(WORDS, k=rng.randint(6, 30))) for _ in range(rng.randint(1, 3)))
        docs.append((f"d{i:03d}", text, f"{rng.randrange(10 ** 6):06d}"))
    return docs


@pytest.mark.parametrize("seed", range(8))
def test_three_passes_match_the_model_in_every_order(seed):
    rng = random.Random(seed)
    docs = _generated_corpus(rng, 30)
    want = m_corpus(docs)
    kept, dropped_exact, dropped_near, _clusters = want
    assert sorted(kept + dropped_exact + dropped_near) == sorted(d[0] for d in docs)     # a partition of the input
    for _ in range(3):
        rng.shuffle(docs)
        assert report(DD.dedup_corpus(native_docs(docs))) == want
    k, d = m_exact_document(docs)
    assert report(DD.dedup_exact(native_docs(docs)))[:2] == (sorted(x[0] for x in k), sorted(x[0] for x in d))
    k, d = m_exact_paragraph(docs)
    assert report(DD.dedup_exact(native_docs(docs), "paragraph"))[:2] == (sorted(x[0] for x in k), sorted(x[0] for x in d))
    k, d, c = m_near(docs)
    assert report(DD.dedup_near(native_docs(docs))) == (sorted(x[0] for x in k), [], sorted(x[0] for x in d), sorted(c))
