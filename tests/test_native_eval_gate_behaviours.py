"""Behaviour list of the held-out evaluation gate (C++ ``native.eval_gate``; reference
harness/eval-gate/tests/{determinism,errors,leak,fault,iface,now,properties,request,rotate}.rs):
which suites it serves, a scores-only answer that never carries task text (a canary string
is planted in prompts and must never come back), byte-exact scoring compared with a Python
model, the suite hash against a published value, fail-closed reads of a damaged tree, and
the rotation rules on injected time."""
import hashlib
import json
import random
import time

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

E = native.eval_gate
CANARY = "CANARY-7f3a-held-out-task-text"
GOLDEN_A = "b1f97a1b6089e43fd1eadfd1961819ce90696d9c677817cc08ff754083fc11b9"


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    assert CANARY not in str(e.value)                                                          # no error ever quotes a task
    return e.value


def item(i, answer="yes", weight=100, prompt=None):
    return {"id": str(i), "prompt": prompt or f"{CANARY} question {i}", "answer": answer, "weight_milli": weight}


def suite_hash(items):
    lines = sorted((json.dumps(i, sort_keys=True, separators=(",", ":"), ensure_ascii=False) for i in items), key=lambda s: json.loads(s)["id"])
    return hashlib.sha256("".join(x + "\n" for x in lines).encode()).hexdigest()


def pend(root, suite, items, written, compute=7):
    d = root / suite / "pending"
    d.mkdir(parents=True, exist_ok=True)
    (d / "items.jsonl").write_text("".join(json.dumps(i, ensure_ascii=False) + "\n" for i in items), encoding="utf-8")
    (d / "meta.json").write_text(json.dumps({"written_ms": written, "compute_ms": compute}))


def subject(root, kind, name, answers):
    d = root / "subjects" / kind
    d.mkdir(parents=True, exist_ok=True)
    (d / f"{name}.json").write_text(json.dumps(answers, ensure_ascii=False), encoding="utf-8")


@pytest.fixture
def gate(tmp_path):
    root = tmp_path / "suites"
    root.mkdir()
    return E.EvalGate(str(root), "hv-1"), root


def installed(gate, items, suite="re_bench", compute=7):
    g, root = gate
    pend(root, suite, items, 5, compute)
    return g.rotate(suite, 0, 0)


# ------------------------------------------------------------------------------ surface / open
def test_surface(tmp_path):
    assert E.HELD_OUT_SUITES == ["re_bench", "mle_bench", "paperbench", "speedrun", "metr_time_horizon"] and E.ROTATION_MS == 90 * 24 * 3600 * 1000
    assert all(E.is_held_out_suite(s) for s in E.HELD_OUT_SUITES)
    assert not any(E.is_held_out_suite(s) for s in ("gpqa", "aime", "", "RE_BENCH", "re-bench", "nope"))
    assert sorted(n for n in dir(E.EvalGate) if not n.startswith("_")) == ["request", "rotate", "suite_hash"]      # nothing that returns items
    assert sorted(n for n in dir(E.Scores) if not n.startswith("_")) == \
        ["compute_ms", "harness_version", "n_items", "rci_milli", "subject", "subject_kind", "suite", "suite_hash"]
    err(E.EvalGate, str(tmp_path / "missing"), "hv")
    (tmp_path / "file").write_text("x")
    err(E.EvalGate, str(tmp_path / "file"), "hv")
    err(E.EvalGate, str(tmp_path), "")
    E.EvalGate(str(tmp_path), "hv")                                                            # an empty directory is fine


def test_suite_names_are_checked_before_anything_else(gate):
    g, root = gate
    for call in (lambda s: g.suite_hash(s), lambda s: g.rotate(s, 0, 1), lambda s: g.request("genome", "r", s)):
        assert err(call, "gpqa").kind == "NotHeldOut" and err(call, "nope").kind == "UnknownSuite" and err(call, "Re_Bench").kind == "UnknownSuite"
    assert err(g.suite_hash, "re_bench").kind == "Message"                                     # known, but nothing installed yet
    e = err(g.request, "genome", "r", "nope")
    assert not any(word in str(e) for word in ("prompt", "answer", "items"))


# ------------------------------------------------------------------------------ hashing
def test_suite_hash_value_and_independence_of_file_order(gate):
    g, root = gate
    assert installed(gate, [{"id": "a", "prompt": "p", "answer": "s", "weight_milli": 1}]) == GOLDEN_A
    items = [item(3), item(1, "ünï ☃"), item(2, "")]
    pend(root, "speedrun", items, 5)
    h = g.rotate("speedrun", 0, 0)
    assert h == suite_hash(items) == suite_hash(list(reversed(items))) == g.suite_hash("speedrun")
    assert len(h) == 64 and set(h) <= set("0123456789abcdef")
    other = E.EvalGate(str(root), "another-version")
    assert other.suite_hash("speedrun") == h and other.suite_hash("re_bench") == GOLDEN_A      # stable across opens and harness versions


# ------------------------------------------------------------------------------ requests
def model_rci(items, answers):
    return sum(i["weight_milli"] for i in items if answers.get(i["id"]) == i["answer"])


def test_scores_only_and_byte_exact(gate):
    g, root = gate
    items = [item(1, "yes", 500), item(2, "Paris", 300), item(3, "ünï", 200)]
    h = installed(gate, items, compute=42)
    subject(root, "genome", "perfect", {"1": "yes", "2": "Paris", "3": "ünï", "99": "ignored"})
    subject(root, "genome", "sloppy", {"1": "yes ", "2": "paris", "3": "uni"})
    subject(root, "checkpoint", "perfect", {"1": "yes", "2": "Paris", "3": "ünï"})
    subject(root, "genome", "none", {})
    s = g.request("genome", "perfect", "re_bench")
    assert (s.suite, s.subject_kind, s.subject, s.rci_milli, s.n_items, s.compute_ms, s.harness_version, s.suite_hash) == \
        ("re_bench", "genome", "perfect", 1000, 3, 42, "hv-1", h)
    assert g.request("genome", "sloppy", "re_bench").rci_milli == 0                           # trailing space, case and accents all count
    assert g.request("checkpoint", "perfect", "re_bench").rci_milli == 1000 and g.request("genome", "none", "re_bench").rci_milli == 0
    again = g.request("genome", "perfect", "re_bench")
    assert (again.rci_milli, again.suite_hash) == (s.rci_milli, s.suite_hash) and g.suite_hash("re_bench") == h   # asking changes nothing
    assert CANARY not in repr(s) and CANARY not in "".join(str(getattr(s, n)) for n in dir(s) if not n.startswith("_"))
    assert E.EvalGate(str(root), "hv-2").request("genome", "perfect", "re_bench").harness_version == "hv-2"


def test_missing_and_malformed_subjects(gate):
    g, root = gate
    installed(gate, [item(1)])
    subject(root, "genome", "ok", {"1": "yes"})
    for kind, name in (("genome", "ghost"), ("checkpoint", "ok"), ("genome", "../genome/ok"), ("genome", ""), ("genome", "a/b"), ("genome", "..")):
        assert err(g.request, kind, name, "re_bench").kind == "SubjectNotFound"
    err(g.request, "GenomeRev", "ok", "re_bench")
    (root / "subjects" / "genome" / "array.json").write_text("[1, 2]")
    (root / "subjects" / "genome" / "torn.json").write_text('{"1": "ye')
    (root / "subjects" / "genome" / "number.json").write_text('{"1": 5}')
    for name in ("array", "torn", "number"):
        assert err(g.request, "genome", name, "re_bench").kind == "Message"


@pytest.mark.parametrize("seed", range(5))
def test_random_suites_and_answers_agree_with_the_model(tmp_path, seed):
    rng = random.Random(seed)
    root = tmp_path / "s"
    root.mkdir()
    g = E.EvalGate(str(root), "hv")
    words = ["yes", "no", "Yes", "yes ", "", "ünï", "42", "4 2"]
    for suite in E.HELD_OUT_SUITES:
        items = [item(f"{suite}-{i}", rng.choice(words), rng.randint(0, 400)) for i in range(rng.randint(1, 8))]
        rng.shuffle(items)
        pend(root, suite, items, 5, compute=rng.randint(0, 10 ** 6))
        assert g.rotate(suite, 0, 0) == suite_hash(items)
        for s in range(4):
            answers = {i["id"]: rng.choice([i["answer"], rng.choice(words)]) for i in items if rng.random() < 0.8}
            subject(root, "genome", f"r{s}", answers)
            got = g.request("genome", f"r{s}", suite)
            assert (got.rci_milli, got.n_items) == (model_rci(items, answers), len(items))
            assert 0 <= got.rci_milli <= sum(i["weight_milli"] for i in items)


# ------------------------------------------------------------------------------ damaged trees
def test_a_damaged_suite_fails_closed_and_leaves_its_siblings_alone(gate):
    g, root = gate
    h = installed(gate, [item(1), item(2)])
    installed(gate, [item(9)], suite="speedrun")
    subject(root, "genome", "r", {"1": "yes", "9": "yes"})
    cur, gen = root / "re_bench" / "current.json", root / "re_bench" / "generations" / h / "items.jsonl"
    good_cur, good_items = cur.read_text(), gen.read_text()

    def broken():
        fresh = E.EvalGate(str(root), "hv-1")
        assert err(fresh.request, "genome", "r", "re_bench").kind == "Message" and err(fresh.suite_hash, "re_bench").kind == "Message"
        assert fresh.request("genome", "r", "speedrun").rci_milli == 100                      # the sibling still answers

    for text in (good_cur[:-9], "[]", json.dumps(dict(json.loads(good_cur), suite_hash="0" * 64))):
        cur.write_text(text)
        broken()
    cur.write_text(good_cur)
    lines = good_items.splitlines()
    for text in (good_items[:-12], lines[0] + "\n" + lines[0] + "\n", lines[0] + "\n", json.dumps(dict(json.loads(lines[0]), hint="x")) + "\n" + lines[1] + "\n", ""):
        gen.write_text(text)
        broken()
    gen.unlink()
    broken()
    gen.write_text(good_items)
    assert E.EvalGate(str(root), "hv-1").request("genome", "r", "re_bench").rci_milli == 100


# ------------------------------------------------------------------------------ rotation
def test_rotation_rules(gate):
    g, root = gate
    R = E.ROTATION_MS
    assert err(g.rotate, "re_bench", 0, 0).kind == "RotationRefused"                           # nothing pending
    first = [item(1)]
    pend(root, "re_bench", first, 5, compute=100)
    assert err(g.rotate, "re_bench", 5, 10).kind == "RotationRefused" and err(g.rotate, "re_bench", 6, 10).kind == "RotationRefused"   # written after the cutoff, strictly
    assert err(g.rotate, "re_bench", 3, 2).kind == "RotationRefused"                           # a cutoff in the future
    h1 = g.rotate("re_bench", 0, 0)                                                            # a first install may happen at time zero
    assert h1 == suite_hash(first) and not (root / "re_bench" / "pending").exists()            # pending is consumed
    assert err(g.rotate, "re_bench", 0, R).kind == "RotationRefused"
    second = [item(1), item(2, "no")]
    pend(root, "re_bench", second, R, compute=200)
    assert err(g.rotate, "re_bench", 10, R - 1).kind == "RotationRefused" and g.suite_hash("re_bench") == h1     # ninety days, not a millisecond less
    for bad in ([], [item(1), item(1)], [dict(item(1), extra=1)], [{"id": "1", "prompt": "p"}]):
        pend(root, "re_bench", bad, R)
        assert err(g.rotate, "re_bench", 10, R).kind == "RotationRefused" and g.suite_hash("re_bench") == h1
    pend(root, "re_bench", second, R, compute=200)
    t0 = time.monotonic()
    h2 = g.rotate("re_bench", 10, R)
    assert time.monotonic() - t0 < 2 and h2 == suite_hash(second) != h1 and CANARY not in h2
    assert (root / "re_bench" / "generations" / h1 / "items.jsonl").exists()                   # the old generation stays on disk
    hist = [json.loads(x) for x in (root / "re_bench" / "history.jsonl").read_text().splitlines()]
    assert [x["suite_hash"] for x in hist] == [h1]
    subject(root, "genome", "r", {"1": "yes", "2": "no"})
    s = E.EvalGate(str(root), "hv-1").request("genome", "r", "re_bench")                      # a reopened gate serves the new generation
    assert (s.suite_hash, s.rci_milli, s.n_items, s.compute_ms) == (h2, 200, 2, 200)
