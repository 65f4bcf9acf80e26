"""Behaviour list of the experiment ledger (C++ ``native.ledger``; reference
harness/ledger/tests/{append,query,roundtrip,search,supersedes}.rs and
harness/kernel/tests/ledger.rs): append-only rows keyed by experiment id, superseding
without rewriting, every field surviving a round trip, a query language that is not SQL
(metacharacters in values are data), negatives, similarity search, durability. Queries are
compared with a Python filter on random rows."""
import json
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

LG = native.ledger


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    return e.value


def rec(eid, hyp, role="researcher", rung=None, **kw):
    r = {"experiment_id": eid, "hypothesis": hyp, "prediction": "loss goes down", "config_hash": "c" * 8, "results": None, "delta_rci": None,
         "replication": None, "gpu_hours": None, "author_role": role, "rung": rung, "created_at": "2026-01-01T00:00:00Z", "closed_at": None,
         "supersedes": None}
    r.update(kw)
    return r


def ids(rows):
    return [json.loads(r)["experiment_id"] for r in rows]


@pytest.fixture
def ledger(tmp_path):
    return LG.Ledger(str(tmp_path / "ledger.jsonl")), tmp_path


def test_empty_ledger(ledger):
    l, _ = ledger
    assert len(l) == 0 and l.query("all") == [] and l.query("") == [] and l.list_negatives() == [] and l.search_similar("anything", 3) == []
    assert err(l.get, "e1").kind == "NotFound"


def test_round_trip_of_every_field(ledger):
    l, tmp = ledger
    full = rec("e-full", "ünï hypothesis ☃", "engineer", 2, results={"passed": True, "loss": 1.25}, delta_rci=-0.5, gpu_hours=1.5,
               replication={"status": "replicated", "n": 2, "notes": "ok"}, closed_at="2026-01-02T00:00:00Z")
    bare = rec("e-bare", "nothing optional set")
    assert l.append(json.dumps(full)) == "e-full" and l.append(json.dumps(bare)) == "e-bare"
    assert json.loads(l.get("e-full")) == full and json.loads(l.get("e-bare")) == bare
    again = LG.Ledger(str(tmp / "ledger.jsonl"))                                               # a second open sees the same rows in the same order
    assert len(again) == 2 and [json.loads(r) for r in again.query("all")] == [full, bare]
    for bad in ("not json", "[]", json.dumps({"experiment_id": "x"}), json.dumps({k: v for k, v in bare.items() if k != "prediction"})):
        err(l.append, bad)
    assert len(l) == 2


def test_rows_are_never_rewritten(ledger):
    l, _ = ledger
    l.append(json.dumps(rec("e1", "first claim")))
    assert err(l.append, json.dumps(rec("e1", "second claim"))).kind == "Duplicate"
    assert err(l.append, json.dumps(rec("e1", "second claim", supersedes="e1"))).kind == "Duplicate"    # superseding is a new id, not a rewrite
    assert err(l.append, json.dumps(rec("e2", "fix", supersedes="e0"))).kind == "NotFound"
    l.append(json.dumps(rec("e2", "corrected claim", supersedes="e1")))
    assert json.loads(l.get("e1"))["hypothesis"] == "first claim" and json.loads(l.get("e2"))["supersedes"] == "e1" and len(l) == 2


def test_values_with_metacharacters_are_data(ledger):
    l, _ = ledger
    odd = "it's \"quoted\" 100% _under_ back\\slash ; -- /* x */"
    l.append(json.dumps(rec("e'1;--", odd, role="engineer")))
    l.append(json.dumps(rec("e2", "plain")))
    assert json.loads(l.get("e'1;--"))["hypothesis"] == odd and len(l) == 2
    assert ids(l.query('hypothesis~"%"')) == ["e'1;--"] and ids(l.query('hypothesis~"_under_"')) == ["e'1;--"]   # not wildcards
    assert ids(l.query("author_role=engineer")) == ["e'1;--"] and ids(l.query("all")) == ["e'1;--", "e2"]
    for sql in ("SELECT * FROM records", "author_role=engineer; DROP TABLE records", "delete from records"):
        assert err(l.query, sql).kind == "Message" and len(l) == 2
    for bad in ("colour=red", 'hypothesis~"open', "rung=x", "a= AND ", "author_role"):
        err(l.query, bad)


def test_negatives_and_similarity(ledger):
    l, _ = ledger
    l.append(json.dumps(rec("pos", "muon learning rate transfers across width", results={"passed": True})))
    l.append(json.dumps(rec("neg1", "fp8 training matches bf16 loss curves", results={"passed": False})))
    l.append(json.dumps(rec("neg2", "delta rule gates help long context recall", replication={"status": "failed", "n": 3, "notes": None})))
    l.append(json.dumps(rec("open", "unrelated statement about tokenizers")))
    assert ids(l.list_negatives()) == ["neg1", "neg2"]
    hits = l.search_similar("does fp8 training match bf16", 2)
    assert hits[0][0] == "neg1" and hits[0][1] > hits[1][1] >= 0 and len(hits) == 2             # a prior negative surfaces first
    assert l.search_similar("fp8", 0) == [] and len(l.search_similar("fp8", 10)) <= 4
    assert [h[0] for h in l.search_similar("long context recall with the delta rule", 1)] == ["neg2"]


@pytest.mark.parametrize("seed", range(4))
def test_random_rows_and_queries_agree_with_a_python_filter(tmp_path, seed):
    rng = random.Random(seed)
    l = LG.Ledger(str(tmp_path / "l.jsonl"))
    roles, words = ["researcher", "engineer", "reviewer"], ["muon", "fp8", "delta", "rope", "moe"]
    rows = []
    for i in range(40):
        tag = rng.choice(["", "CHECK:", "PREREG:"])
        topic = rng.choice(words)
        r = rec(f"e{i}", f"{tag}{topic} {' '.join(rng.sample(words, 2))}", rng.choice(roles), rng.choice([None, 0, 1, 2, 3]))
        rows.append(r)
        l.append(json.dumps(r))
    kind = lambda r: "check" if r["hypothesis"].startswith("CHECK:") else "prereg" if r["hypothesis"].startswith("PREREG:") else None
    for _ in range(60):
        preds, keep = [], list(rows)
        if rng.random() < 0.5:
            role = rng.choice(roles)
            preds.append(f"author_role={role}")
            keep = [r for r in keep if r["author_role"] == role]
        if rng.random() < 0.5:
            rung = rng.choice([None, 0, 1, 2, 3])
            preds.append("rung=none" if rung is None else f"rung={rung}")
            keep = [r for r in keep if r["rung"] == rung]
        if rng.random() < 0.4:
            w = rng.choice(words)
            preds.append(f'hypothesis~"{w}"')
            keep = [r for r in keep if w in r["hypothesis"]]
        if rng.random() < 0.3:
            kd = rng.choice(["check", "prereg"])
            preds.append(f"kind={kd}")
            keep = [r for r in keep if kind(r) == kd]
        if rng.random() < 0.2:
            eid = f"e{rng.randrange(45)}"
            preds.append(f"experiment_id={eid}")
            keep = [r for r in keep if r["experiment_id"] == eid]
        rng.shuffle(preds)
        assert ids(l.query(" AND ".join(preds) if preds else "all")) == [r["experiment_id"] for r in keep], preds   # in append order
