"""Behaviour list of the classifier orchestrator (C++ ``native.classifiers``; reference
data/classifiers/tests/{create_open,ingest,shards,score,agreement,gate,replay,properties}.rs):
the journal directory, duplicate rejection by content hash, shard boundaries, scorer calls,
the keep rule on two thresholds, agreement with human labels, the gate and replay on open.
The last test runs random mixed operations against a dictionary model."""
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

CL, EX = native.classifiers, native.extract


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def doc(i, text=None):
    return EX.ExtractedDocument(text if text is not None else f"document number {i}", "html", f"p{i}.html", 10 + i)


def new(tmp_path, name="clf", **cfg):
    return CL.Orchestrator.create(str(tmp_path / name), CL.ClassifierConfig(**cfg))


# ------------------------------------------------------------------------------ create / open
def test_defaults():
    assert CL.DEFAULT_SHARD_SIZE == 32
    CL.ClassifierConfig()                                              # thresholds 0.5 / 0.5, unanimous gate


def test_create_makes_the_directory_and_refuses_an_existing_one(tmp_path):
    o = new(tmp_path)
    assert (tmp_path / "clf").is_dir() and len(o) == 0 and o.shards() == [] and o.predictions == []
    err(lambda: new(tmp_path))                                         # twice
    (tmp_path / "afile").write_text("x")
    err(lambda: CL.Orchestrator.create(str(tmp_path / "afile")))
    assert err(lambda: new(tmp_path, "zero", shard_size=0)).kind == "BadShardSize"
    assert not (tmp_path / "zero").exists()
    assert err(lambda: CL.Orchestrator.open(str(tmp_path / "missing"))).kind == "Other"
    assert err(lambda: CL.Orchestrator.open(str(tmp_path / "afile"))).kind == "Other"
    back = CL.Orchestrator.open(str(tmp_path / "clf"))
    assert len(back) == 0 and back.shards() == []


# ------------------------------------------------------------------------------ ingest / shards
def test_ingest_keeps_order_and_rejects_a_repeated_content_hash(tmp_path):
    o = new(tmp_path, shard_size=2)
    docs = [doc(i) for i in range(3)]
    for d in docs:
        o.ingest(d)
    assert err(lambda: o.ingest(docs[1])).kind == "WrongState" and len(o) == 3
    assert [d.text for shard in o.shards() for d in shard] == [d.text for d in docs]
    o.ingest(doc(9, ""))                                               # empty text is a document like any other
    assert len(o) == 4 and o.shards()[1][1].text == ""
    o.run_local(1, 0)
    o.ingest(doc(10))                                                  # ingest after a run appends
    assert len(o) == 5 and [len(s) for s in o.shards()] == [2, 2, 1]


@pytest.mark.parametrize("n, size, want", [(0, 4, []), (8, 4, [4, 4]), (9, 4, [4, 4, 1]), (3, 1, [1, 1, 1]), (3, 50, [3]), (33, 32, [32, 1])])
def test_shard_boundaries(tmp_path, n, size, want):
    o = new(tmp_path, shard_size=size)
    for i in range(n):
        o.ingest(doc(i))
    assert [len(s) for s in o.shards()] == want
    assert [d.source for s in o.shards() for d in s] == [f"p{i}.html" for i in range(n)]


# ------------------------------------------------------------------------------ scoring
def test_local_scorer_is_a_pure_function_of_seed_and_text():
    a = CL.local_scores(7, "some text")
    assert a == CL.local_scores(7, "some text") and all(0.0 <= v < 1.0 for v in a)
    assert a != CL.local_scores(8, "some text") and a != CL.local_scores(7, "some text!")
    assert a[0] != a[1]
    qs, ss = zip(*(CL.local_scores(1, f"t{i}") for i in range(400)))
    assert 0.4 < sum(qs) / 400 < 0.6 and 0.4 < sum(ss) / 400 < 0.6
    both = sum((q >= 0.5) == (s >= 0.5) for q, s in zip(qs, ss))
    assert 120 < both < 280                                            # the two axes are not copies of each other


def test_run_calls_the_scorer_once_per_shard_and_aligns_predictions(tmp_path):
    o = new(tmp_path, shard_size=2)
    assert err(lambda: o.run(lambda t, n: [], 0)).kind == "Empty"
    docs = [doc(i) for i in range(5)]
    for d in docs:
        o.ingest(d)
    assert o.predictions == []                                         # nothing before a run
    calls = []

    def scorer(texts, now):
        calls.append((list(texts), now))
        return [(len(t) / 100.0, 0.25) for t in texts]

    preds = o.run(scorer, 1234)
    assert [c[1] for c in calls] == [1234] * 3 and [len(c[0]) for c in calls] == [2, 2, 1]
    assert [t for c in calls for t in c[0]] == [d.text for d in docs]
    assert [p.content_hash for p in preds] == [d.content_hash for d in docs]
    assert [(p.content_hash, p.quality, p.safety) for p in o.predictions] == [(p.content_hash, p.quality, p.safety) for p in preds]
    assert preds[0].quality == pytest.approx(len(docs[0].text) / 100.0) and preds[0].safety == 0.25
    again = o.run(lambda texts, now: [(0.9, 0.9)] * len(texts), 0)    # a second run re-scores everything
    assert [p.quality for p in again] == pytest.approx([0.9] * 5) and [p.quality for p in o.predictions] == pytest.approx([0.9] * 5)


def test_scorer_failures(tmp_path):
    o = new(tmp_path, shard_size=2)
    for i in range(3):
        o.ingest(doc(i))
    assert err(lambda: o.run(lambda texts, now: [(0.5, 0.5)], 0)).kind == "WrongState"      # wrong length
    assert o.predictions == []

    def boom(texts, now):
        raise RuntimeError("scorer exploded")

    with pytest.raises(Exception, match="exploded"):
        o.run(boom, 0)


# ------------------------------------------------------------------------------ agreement / gate
def P(preds):
    return [(p.content_hash, p.quality, p.safety) for p in preds]


def test_keep_needs_both_thresholds_and_equality_keeps(tmp_path):
    o = new(tmp_path, shard_size=8, quality_threshold=0.6, safety_threshold=0.3)
    table = {"a": (0.6, 0.3), "b": (0.59, 0.9), "c": (0.9, 0.29), "d": (0.1, 0.1)}
    for i, name in enumerate(table):
        o.ingest(doc(i, name))
    preds = o.run(lambda texts, now: [table[t] for t in texts], 0)
    h = {t: p.content_hash for t, p in zip(table, preds)}
    # humans: a keep/keep, b quality-only, c safety-only, d neither; model axes: a T/T, b F/T, c T/F, d F/F
    labels = [CL.HumanLabel(h["a"], True, True), CL.HumanLabel(h["b"], False, True), CL.HumanLabel(h["c"], True, False),
              CL.HumanLabel(h["d"], False, False)]
    assert o.agreement(labels) == 1.0
    one_axis_off = [CL.HumanLabel(h["a"], True, False)] + labels[1:]
    assert o.agreement(one_axis_off) == pytest.approx(0.75)            # both axes must match to count
    assert CL.agreement(preds, labels, 0.6, 0.3) == 1.0 and CL.agreement(preds, labels, 0.5, 0.5) < 1.0


def test_agreement_errors_and_ignored_predictions(tmp_path):
    o = new(tmp_path, shard_size=8)
    for i in range(4):
        o.ingest(doc(i))
    preds = o.run_local(5, 0)
    truth = [CL.HumanLabel(p.content_hash, p.quality >= 0.5, p.safety >= 0.5) for p in preds]
    assert err(lambda: o.agreement([])).kind == "Empty"
    assert o.agreement(truth[:2]) == 1.0                                # unlabeled predictions are ignored
    flipped = [CL.HumanLabel(p.content_hash, p.quality < 0.5, p.safety < 0.5) for p in preds]
    assert o.agreement(flipped) == 0.0 and o.agreement(truth[:2] + flipped[2:]) == 0.5
    e = err(lambda: o.agreement(truth[:1] + [CL.HumanLabel("ghost-1", True, True), CL.HumanLabel("ghost-2", True, True)]))
    assert e.kind == "MissingLabel" and "ghost-1" in str(e)             # the first missing one, in label order
    fresh = new(tmp_path, "fresh")
    fresh.ingest(doc(0))
    assert err(lambda: fresh.agreement(truth[:1])).kind == "MissingLabel"     # no predictions yet


def test_gate(tmp_path):
    o = new(tmp_path, shard_size=8, min_agreement=0.75)
    for i in range(4):
        o.ingest(doc(i))
    preds = o.run_local(5, 0)
    truth = [CL.HumanLabel(p.content_hash, p.quality >= 0.5, p.safety >= 0.5) for p in preds]
    wrong = lambda k: [CL.HumanLabel(p.content_hash, p.quality < 0.5, p.safety >= 0.5) for p in preds[:k]] + truth[k:]
    o.gate(truth)
    o.gate(wrong(1))                                                     # 0.75: equality passes
    e = err(lambda: o.gate(wrong(2)))
    assert e.kind == "GateFailed" and "0.5" in str(e) and "0.75" in str(e)
    assert err(lambda: o.gate([])).kind == "Empty"
    assert err(lambda: o.gate([CL.HumanLabel("ghost", True, True)])).kind == "MissingLabel"
    strict = new(tmp_path, "strict", shard_size=8)                       # default: unanimous
    for i in range(4):
        strict.ingest(doc(i))
    strict.run_local(5, 0)
    assert err(lambda: strict.gate(wrong(1))).kind == "GateFailed"
    lax = new(tmp_path, "lax", shard_size=8, min_agreement=0.0)
    for i in range(4):
        lax.ingest(doc(i))
    lax.run_local(5, 0)
    lax.gate(wrong(4))


# ------------------------------------------------------------------------------ replay
def test_open_replays_documents_and_scores(tmp_path):
    o = new(tmp_path, shard_size=2)
    for i in range(3):
        o.ingest(doc(i))
    before_run = CL.Orchestrator.open(str(tmp_path / "clf"), CL.ClassifierConfig(shard_size=2))
    assert len(before_run) == 3 and before_run.predictions == [] and [len(s) for s in before_run.shards()] == [2, 1]
    preds = o.run_local(3, 0)
    truth = [CL.HumanLabel(p.content_hash, p.quality >= 0.5, p.safety >= 0.5) for p in preds]
    back = CL.Orchestrator.open(str(tmp_path / "clf"), CL.ClassifierConfig(shard_size=3))
    assert P(back.predictions) == P(preds) and back.agreement(truth) == 1.0
    back.gate(truth)
    assert [len(s) for s in back.shards()] == [3]                        # the configuration passed to open is the one in force
    assert err(lambda: back.ingest(doc(0))).kind == "WrongState"         # duplicates are still known after a replay
    back.ingest(doc(7))
    assert len(CL.Orchestrator.open(str(tmp_path / "clf"))) == 4


# ------------------------------------------------------------------------------ model check
@pytest.mark.parametrize("seed", range(6))
def test_random_operations_match_a_dictionary_model(tmp_path, seed):
    rng = random.Random(seed)
    size = rng.randint(1, 5)
    o = new(tmp_path, shard_size=size)
    texts, hashes, scores = [], [], {}
    for _step in range(60):
        op = rng.choice(["ingest", "ingest", "ingest", "run", "agree", "reopen"])
        if op == "ingest":
            i = rng.randint(0, 25)
            d = doc(i)
            if d.text in texts:
                assert err(lambda: o.ingest(d)).kind == "WrongState"
            else:
                o.ingest(d)
                texts.append(d.text)
                hashes.append(d.content_hash)
        elif op == "run":
            s = rng.randint(0, 9)
            if not texts:
                assert err(lambda: o.run_local(s, 0)).kind == "Empty"
            else:
                got = o.run_local(s, 0)
                scores = {h: CL.local_scores(s, t) for h, t in zip(hashes, texts)}
                assert [(p.content_hash, (p.quality, p.safety)) for p in got] == list(scores.items())
        elif op == "agree" and scores:
            picks = rng.sample(sorted(scores), k=rng.randint(1, len(scores)))
            labels, right = [], 0
            for h in picks:
                q, s = rng.random() < 0.5, rng.random() < 0.5
                labels.append(CL.HumanLabel(h, q, s))
                right += (scores[h][0] >= 0.5) == q and (scores[h][1] >= 0.5) == s
            assert o.agreement(labels) == pytest.approx(right / len(picks))
        elif op == "reopen":
            o = CL.Orchestrator.open(str(tmp_path / "clf"), CL.ClassifierConfig(shard_size=size))
        assert len(o) == len(texts)
        assert [len(s) for s in o.shards()] == [min(size, len(texts) - k) for k in range(0, len(texts), size)]
