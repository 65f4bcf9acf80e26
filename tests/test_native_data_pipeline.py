"""Extraction, dedup, decontamination, classifier orchestration and the batch generation
engine (C++), against the contracts of the reference's data/* crates and serve::LocalEngine."""
import hashlib
import json
import struct
import zlib

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

EX, DD, DC, CL, SV = native.extract, native.dedup, native.decontam, native.classifiers, native.serve


def _kind(e):
    return e.value.kind


def _in_order(text, phrases):
    at = 0
    for p in phrases:
        at = text.index(p, at) + len(p)


# ------------------------------------------------------------------------------- extract
HTML = b"""<!DOCTYPE html><html><head><meta charset="utf-8"><style>body { color: red; }</style>
<script type="text/javascript">alert("nope");</script></head><body>
<!-- secret-comment-should-not-appear --><h1>Title One</h1>
<p>Hello <b>world</b> &amp; friends.</p><p>Math stays as $x^2$.</p><noscript>hidden</noscript></body></html>"""

TEX = rb"""\documentclass{article}
\begin{document}
The energy equation is $E=mc^2$. % a comment that goes away
Display:
$$
\int_0^1 x^2 \, dx
$$
\begin{equation}
\alpha + \beta
\end{equation}
100\% kept. Plain text remains.
\end{document}
"""


def _pdf(stream: bytes, flate: bool) -> bytes:
    body = zlib.compress(stream) if flate else stream
    filt = b"/Filter /FlateDecode " if flate else b""
    return (b"%PDF-1.4\n1 0 obj\n<< /Type /Catalog >>\nendobj\n4 0 obj\n<< " + filt + b"/Length "
            + str(len(body)).encode() + b" >>\nstream\n" + body + b"\nendstream\nendobj\ntrailer\n<< >>\n%%EOF\n")


def test_extract_html_latex_pdf():
    d = EX.extract(HTML, "html")
    _in_order(d.text, ["Title One", "Hello world & friends.", "Math stays as $x^2$."])
    for gone in ("alert", "color: red", "secret-comment", "hidden"):
        assert gone not in d.text
    assert d.format == "html" and d.bytes_in == len(HTML) and d.source is None
    assert d.content_hash == hashlib.sha256(d.text.encode()).hexdigest()
    assert d.text.index("Title One") < d.text.index("\n", d.text.index("Title One"))   # block break after h1

    t = EX.extract(TEX, "latex")
    _in_order(t.text, ["The energy equation is $E=mc^2$.", r"\int_0^1 x^2", r"\begin{equation}", r"\alpha + \beta",
                       r"\end{equation}", r"100\% kept. Plain text remains."])
    assert "a comment" not in t.text and EX.preserves_latex_math(t.text)
    assert not EX.preserves_latex_math(r"costs \$5 and \$6") and not EX.preserves_latex_math("plain")
    assert EX.preserves_latex_math(r"\begin{align*}x\end{align*}") and EX.preserves_latex_math("$$ x $$")

    content = b"BT /F1 12 Tf 72 720 Td (Hello \\(PDF\\)) Tj 0 -14 Td [(sec) -20 (ond)] TJ ET"
    for flate in (False, True):
        p = EX.extract(_pdf(content, flate), "pdf")
        _in_order(p.text, ["Hello (PDF)", "second"])
        assert p.format == "pdf"


def test_extract_errors_and_format_detection():
    with pytest.raises(NativeError) as e:
        EX.extract(b"", "html")
    assert _kind(e) == "Empty"
    with pytest.raises(NativeError) as e:
        EX.extract(b"\xff\xfe\x00bad", "html")
    assert _kind(e) == "Unparseable"
    with pytest.raises(NativeError) as e:
        EX.extract(b"not a pdf", "pdf")
    assert _kind(e) == "Unparseable"
    with pytest.raises(NativeError) as e:
        EX.extract_from(b"x", path="notes.txt", media_type="text/plain")
    assert _kind(e) == "Unsupported"
    assert EX.format_from_path("a/b/Page.HTML") == "html" and EX.format_from_path("x.tex") == "latex"
    assert EX.format_from_path("x.pdf") == "pdf" and EX.format_from_path("x.md") is None
    assert EX.format_from_media_type("application/pdf") == "pdf" and EX.format_from_media_type("text/x-tex") == "latex"
    assert EX.format_from_media_type("image/png") is None
    d = EX.extract_from(HTML, path="crawl/page.htm")
    assert d.source == "crawl/page.htm" and d.format == "html"
    assert EX.extract_from(TEX, media_type="application/x-latex").format == "latex"
    doc = EX.ExtractedDocument("abc", "html", "s", 3)
    assert doc.content_hash == hashlib.sha256(b"abc").hexdigest()


# --------------------------------------------------------------------------------- dedup
NORMALIZE = [("Hello World", "hello world"), ("  Hello   WORLD  ", "hello world"), ("Hello\t\nWorld", "hello world"),
             ("", ""), ("   \t\n  ", ""), ("Hello\u200bWorld", "helloworld"), ("Hello \u200b World", "hello world"),
             ("HELLO\ufeffWORLD", "helloworld"), ("a\u200cb\u200dc\u2060d", "abcd"),
             ("na\u00efve CAF\u00c9", "na\u00efve caf\u00e9"), ("A\r\n\r\nB", "a b"), ("one\u180etwo", "onetwo")]

CORPUS = [
    ("keep-unique", "unique document about quantum foam and zebra orchids only", "10"),
    ("keep-cats", "the quick brown fox jumps over the lazy dog and then runs home quickly today\n\n"
                  "second paragraph about cats sitting on mats quietly", "01"),
    ("drop-exact-doc", "The  Quick   BROWN fox jumps over the lazy dog and then runs home quickly today\n\n"
                       "second paragraph about cats sitting on mats quietly", "02"),
    ("drop-exact-para", "second paragraph about cats sitting on mats quietly\n\n"
                        "this other paragraph is brand new material about volcanoes", "03"),
    ("keep-near-src", "alpha bravo charlie delta echo foxtrot golf hotel india juliet kilo lima mike november oscar "
                      "papa quebec romeo sierra tango", "04"),
    ("drop-near", "alpha bravo charlie delta echo foxtrot golf hotel india juliet kilo lima mike november oscar "
                  "papa quebec romeo sierra ultra", "05"),
    ("keep-short", "hi", "06"),
]


def _py_minhash(text, num_hashes=128, n=5):
    words = DD.normalize(text).split()
    sh = {" ".join(words[i:i + n]) for i in range(len(words) - n + 1)} if len(words) >= n else set()
    if not sh:
        return [2 ** 64 - 1] * num_hashes
    return [min(struct.unpack("<Q", hashlib.sha256(struct.pack("<Q", i) + s.encode()).digest()[:8])[0] for s in sh)
            for i in range(num_hashes)]


def test_dedup_normalize_paragraphs_shingles_minhash():
    for src, want in NORMALIZE:
        assert DD.normalize(src) == want
    assert DD.exact_hash("Hello   WORLD") == hashlib.sha256(b"hello world").hexdigest()
    assert DD.paragraphs("A  b\nc\n\n\n  \nSecond One\r\n\r\nthird") == ["a b c", "second one", "third"]
    assert DD.paragraphs(" \n ") == []
    assert DD.shingles("a b c d e f", 5) == ["a b c d e", "b c d e f"]
    assert DD.shingles("a b c", 5) == [] and DD.shingles("a b", 0) == []
    text = CORPUS[4][1]
    sig = DD.minhash_signature(text)
    assert sig == _py_minhash(text) and len(sig) == 128
    assert DD.minhash_signature("hi") == [2 ** 64 - 1] * 128
    keys = DD.lsh_band_keys(sig)
    want = [struct.unpack("<Q", hashlib.sha256(b"".join(struct.pack("<Q", v) for v in sig[4 * b:4 * b + 4])).digest()[:8])[0]
            for b in range(32)]
    assert keys == want
    for cfg, bad_sig in ((DD.DedupConfig(5, 128, 16, 4), sig), (DD.DedupConfig(), sig[:10]), (DD.DedupConfig(5, 0, 0, 0), [])):
        with pytest.raises(NativeError) as e:
            DD.lsh_band_keys(bad_sig, cfg)
        assert _kind(e) == "Config"


def test_dedup_corpus_golden_and_grains():
    docs = [DD.Document(i, t, h) for i, t, h in CORPUS]
    r = DD.dedup_corpus(docs)
    assert r.kept == ["keep-cats", "keep-near-src", "keep-short", "keep-unique"]
    assert r.dropped_exact == ["drop-exact-doc", "drop-exact-para"] and r.dropped_near == ["drop-near"]
    assert [(c.kept, c.dropped) for c in r.clusters] == [("keep-near-src", ["drop-near"])]
    assert sorted(r.kept + r.dropped_exact + r.dropped_near) == sorted(i for i, _, _ in CORPUS)

    ex = DD.dedup_exact([DD.Document("later", "Same Text", "b"), DD.Document("winner", "same  text", "a"),
                         DD.Document("also", "same text", "c"), DD.Document("unique", "other", "d")])
    assert ex.kept == ["unique", "winner"] and ex.dropped_exact == ["also", "later"] and not ex.clusters
    tie = DD.dedup_exact([DD.Document("z", "t", "h"), DD.Document("a", "t", "h")])
    assert tie.kept == ["a"] and tie.dropped_exact == ["z"]
    para = DD.dedup_exact([DD.Document("keep-src", "shared para here\n\nown text one", "1"),
                           DD.Document("drop-me", "fresh words\n\nShared  PARA here", "2"),
                           DD.Document("unrelated", "nothing in common", "3")], "paragraph")
    assert para.kept == ["keep-src", "unrelated"] and para.dropped_exact == ["drop-me"]
    # default content hash is the sha256 of the raw text
    assert DD.Document("x", "abc").content_hash == hashlib.sha256(b"abc").hexdigest()
    near = DD.dedup_near([DD.Document(i, t, h) for i, t, h in CORPUS[4:]])
    assert near.kept == ["keep-near-src", "keep-short"] and near.dropped_near == ["drop-near"]
    for fn in (DD.dedup_corpus, DD.dedup_near, DD.dedup_exact):
        with pytest.raises(NativeError):
            fn([])
    with pytest.raises(NativeError) as e:
        DD.dedup_exact(docs, "sentence")
    assert _kind(e) == "Config"


# ------------------------------------------------------------------------------ decontam
def test_decontam_index_scan_and_method_hash():
    ix = DC.Index()
    for call in (ix.method_hash, lambda: ix.ngram_match("x"), lambda: ix.scan_shard(["x"])):
        with pytest.raises(NativeError) as e:
            call()
        assert _kind(e) == "MissingIndex"
    q1 = "What is the capital city of the ancient kingdom of Lydia in Anatolia"
    q2 = "Compute the integral of x squared from zero to one exactly please"
    ix.add(DC.EvalItem("mmlu", "q1", q1))
    ix.add(DC.EvalItem("aime", "p7", q2))
    with pytest.raises(NativeError) as e:
        ix.add(DC.EvalItem("mmlu", "q1", "other"))
    assert _kind(e) == "Config" and len(ix) == 2
    assert DC.NGRAM_N == 8 and len(DC.ngrams(q1)) == 13 - 8 + 1 and DC.ngrams("too short") == []
    assert DC.ngrams("A B C D E F G H")[0] == "a b c d e f g h"

    items = sorted([("mmlu", "q1", q1), ("aime", "p7", q2)])
    h = hashlib.sha256()
    h.update(b"prometheus-decontam/v1\nngram_n=8\nembed_model=\n")
    for s, i, t in items:
        h.update(s.encode() + b"\0" + i.encode() + b"\0" + t.encode() + b"\n")
    assert ix.method_hash() == h.hexdigest()

    clean = ix.scan_text("an unrelated document about growing tomatoes in a cold northern climate zone")
    assert clean.status == "clean" and clean.hits == [] and clean.against == ["aime", "mmlu"]
    leaked = "blog post: WHAT IS THE CAPITAL city of the ancient kingdom of lydia, someone asked"
    hits = ix.ngram_match(leaked)
    assert [(x.suite, x.item_id, x.method) for x in hits] == [("mmlu", "q1", "ngram")]
    rep = ix.scan_shard(["nothing here at all", leaked, leaked])
    assert rep.status == "flagged" and len(rep.hits) == 1 and rep.method_hash == ix.method_hash()
    ix.planted_caught([DC.EvalItem("mmlu", "q1", q1)], ["x", leaked])
    with pytest.raises(NativeError) as e:
        ix.planted_caught([DC.EvalItem("aime", "p7", q2)], [leaked])
    assert _kind(e) == "PlantedMiss"
    with pytest.raises(NativeError) as e:
        ix.embedding_match("anything")
    assert _kind(e) == "Config" and "no embedder" in str(e.value)


# --------------------------------------------------------------------------- classifiers
def _fnv64(b):
    h = 0xcbf29ce484222325
    for c in b:
        h = ((h ^ c) * 0x100000001b3) % 2 ** 64
    return h


def _mix64(x):
    m = 2 ** 64
    x = (x + 0x9E3779B97F4A7C15) % m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) % m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) % m
    return x ^ (x >> 31)


def test_classifier_orchestrator_journal_and_gate(tmp_path):
    q, s = CL.local_scores(7, "some text")
    h = _fnv64(b"some text")
    assert q == pytest.approx((_mix64(7 ^ _mix64(h + 0x51)) >> 40) / 2 ** 24)
    assert s == pytest.approx((_mix64(7 ^ _mix64(h + 0x53)) >> 40) / 2 ** 24)
    cq, cs = CL.scores_from_completion("abc")
    assert cq == pytest.approx((_fnv64(b"abc") >> 40) / 2 ** 24) and cs == pytest.approx((_mix64(_fnv64(b"abc")) >> 40) / 2 ** 24)

    with pytest.raises(NativeError) as e:
        CL.Orchestrator.create(str(tmp_path / "z"), CL.ClassifierConfig(shard_size=0))
    assert _kind(e) == "BadShardSize"
    d = str(tmp_path / "clf")
    o = CL.Orchestrator.create(d, CL.ClassifierConfig(shard_size=2))
    with pytest.raises(NativeError) as e:
        o.run_local(1, 0)
    assert _kind(e) == "Empty"
    docs = [EX.ExtractedDocument(f"document number {i}", "html", f"p{i}.html", 10 + i) for i in range(5)]
    for doc in docs:
        o.ingest(doc)
    with pytest.raises(NativeError) as e:
        o.ingest(docs[0])
    assert _kind(e) == "WrongState"
    assert [len(x) for x in o.shards()] == [2, 2, 1] and len(o) == 5

    calls = []

    def scorer(texts, now):
        calls.append((len(texts), now))
        return [CL.local_scores(3, t) for t in texts]

    preds = o.run(scorer, 99)
    assert calls == [(2, 99), (2, 99), (1, 99)] and [p.content_hash for p in preds] == [x.content_hash for x in docs]
    same = o.run_local(3, 0)
    assert [(p.quality, p.safety) for p in same] == [(p.quality, p.safety) for p in preds]
    with pytest.raises(NativeError) as e:
        o.run(lambda texts, now: [], 0)
    assert _kind(e) == "WrongState"

    labels = [CL.HumanLabel(p.content_hash, p.quality >= 0.5, p.safety >= 0.5) for p in preds]
    assert o.agreement(labels) == 1.0
    o.gate(labels)
    wrong = [CL.HumanLabel(preds[0].content_hash, preds[0].quality < 0.5, preds[0].safety >= 0.5)] + labels[1:]
    assert o.agreement(wrong) == pytest.approx(0.8)
    with pytest.raises(NativeError) as e:
        o.gate(wrong)
    assert _kind(e) == "GateFailed"
    with pytest.raises(NativeError) as e:
        o.agreement([CL.HumanLabel("nope", True, True)])
    assert _kind(e) == "MissingLabel"
    with pytest.raises(NativeError) as e:
        o.agreement([])
    assert _kind(e) == "Empty"

    events = [json.loads(x) for x in (tmp_path / "clf" / "events.jsonl").read_text().splitlines()]
    assert [x["event"] for x in events] == ["clf.ingest"] * 5 + ["clf.score"] * 2
    assert events[0]["doc"]["source"] == "p0.html" and events[0]["doc"]["bytes_in"] == 10
    back = CL.Orchestrator.open(d, CL.ClassifierConfig(shard_size=2))
    assert len(back) == 5 and [(p.content_hash, p.quality) for p in back.predictions] == [(p.content_hash, p.quality) for p in preds]
    assert back.agreement(labels) == 1.0
    with pytest.raises(NativeError):
        CL.Orchestrator.create(d)


# --------------------------------------------------------------------------------- serve
def test_local_engine_generate_and_body():
    for bad in (0, 3, 8):
        with pytest.raises(NativeError) as e:
            SV.LocalEngine(gpus=bad)
        assert _kind(e) == "BadGpuCount"
    eng = SV.LocalEngine("m", 2, 2, 30001)
    assert (eng.model, eng.gpus, eng.max_batch, eng.port) == ("m", 2, 2, 30001) and eng.is_up()
    out = eng.generate(["a", "b"], 3, 0.0)
    assert [c[0] for c in out] == [0, 1] and all(c[2] == "stop" for c in out)
    assert all(len(c[1].split()) == 3 and all(len(t) == 8 for t in c[1].split()) for c in out)
    assert out[0][1] != out[1][1] and eng.generate(["a"], 3, 0.0)[0][1] == out[0][1]
    assert eng.generate(["a"], 3, 0.5)[0][1] != out[0][1] and eng.generate(["a"], 0)[0][1] == ""
    for prompts, kind in (([], "EmptyBatch"), (["a", "b", "c"], "BatchTooLarge")):
        with pytest.raises(NativeError) as e:
            eng.generate(prompts, 1)
        assert _kind(e) == kind
    eng.mark_down()
    with pytest.raises(NativeError) as e:
        eng.generate(["a"], 1)
    assert _kind(e) == "EngineDown"
    eng.mark_up()
    body = json.loads(eng.openai_body(out))
    assert body["model"] == "m" and [c["index"] for c in body["choices"]] == [0, 1]
    assert body["choices"][0]["message"] == {"role": "assistant", "content": out[0][1]}
    assert body["choices"][1]["finish_reason"] == "stop"


def test_router_failover_and_deployer():
    eng = SV.LocalEngine("m", 1, 4, 30000)
    r = SV.Router(["hosted-a", "hosted-b"], eng, native.providers.AimdConfig(min_window=1, max_window=8))
    assert r.providers == ["hosted-a", "hosted-b", "sglang"] and r.last_resort() == "sglang" and r.window == 8
    assert SV.Router(["x", "sglang"], eng).providers == ["x", "sglang"]
    with pytest.raises(NativeError) as e:
        r.generate(["p"], 2)
    assert _kind(e) == "Hosted" and r.current() == "hosted-a"
    r.mark_down("hosted-a")
    assert r.window == 4 and r.current() == "hosted-b"
    r.mark_down("hosted-a")                      # already down: the window is not cut twice
    assert r.window == 4
    r.mark_down("hosted-b")
    assert r.window == 2 and r.current() == "sglang"
    out = r.generate(["p", "q"], 2)
    assert out == eng.generate(["p", "q"], 2)
    r.mark_down("sglang")                        # the last resort does not count as a hosted outage
    assert r.window == 2
    with pytest.raises(NativeError) as e:
        r.generate(["p"], 2)
    assert _kind(e) == "EngineDown"
    r.mark_up("sglang"); r.mark_up("hosted-a")
    assert r.current() == "hosted-a" and r.down == ["hosted-b"]
    with pytest.raises(NativeError) as e:
        r.mark_down("nobody")
    assert _kind(e) == "NotFound"
    r.engine.mark_down()
    r.mark_down("hosted-a")
    with pytest.raises(NativeError) as e:
        r.generate(["p"], 1)
    assert _kind(e) == "EngineDown"

    class FakeSlurm:
        def __init__(self):
            self.calls = []

        def submit(self, run_id, suffix, script, walltime, gpus):
            self.calls.append(("submit", run_id, suffix, script, walltime, gpus))
            return "4242"

        def cancel(self, job):
            self.calls.append(("cancel", job))

    fake = FakeSlurm()
    dep = SV.Deployer(fake, "serve/sglang.sbatch")
    d = dep.submit(SV.LocalEngine("big", 4, 8, 31000), "run-1", "serve", "02:00:00")
    assert (d.job, d.endpoint, d.model, d.gpus) == ("4242", "http://127.0.0.1:31000", "big", 4)
    dep.teardown(d)
    assert fake.calls == [("submit", "run-1", "serve", "serve/sglang.sbatch", "02:00:00", 4), ("cancel", "4242")]
    assert dep.script == "serve/sglang.sbatch" and dep.client is fake
