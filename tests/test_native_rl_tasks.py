"""Task factories, solve-rate filter and horizon curriculum (C++), against the contracts of
the reference's rl/tasks crate."""
import hashlib
import json
import struct

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

T = native.tasks


def _sha(b):
    return hashlib.sha256(b if isinstance(b, bytes) else b.encode()).hexdigest()


def _kind(e):
    return e.value.kind


def _rows(*bodies):
    return json.dumps([{"id": f"s{i}", "source": "unit-test", "body": b} for i, b in enumerate(bodies)])


def test_math_code_swe_factories_mint_spec_and_payload():
    assert T.FACTORY_KINDS == ["code", "swe", "math", "research", "long_horizon", "arc", "forecast", "open_ended"]
    f = T.Factory("math", "mf", _rows("what is 2+2", "what is 3+3"))
    assert (f.id, f.domain, f.kind, len(f)) == ("mf", "math", "math", 2)
    t = json.loads(f.mint(0, "2026-01-01T00:00:00Z"))
    spec = t["spec"]
    expected = _sha("math-expected:what is 2+2")
    assert spec == {"schema_id": "prometheus.task_spec", "schema_version": 1, "task_id": "mf:s0", "domain": "math",
                    "split": "train", "statement_hash": _sha("what is 2+2"), "hidden_tests_hash": _sha(expected),
                    "verifier_id": "symbolic-math", "horizon_s": 30, "max_tool_calls": 10,
                    "provenance": {"source": "unit-test"}, "created_at": "2026-01-01T00:00:00Z"}
    assert t["math"] == {"expected": expected} and t["code"] is None and t["verifier_kind"] == "symbolic_math"
    assert t["statement"] == "what is 2+2"
    T.schema_ok(json.dumps(spec))
    with pytest.raises(NativeError) as e:
        T.schema_ok(json.dumps({**spec, "schema_version": 2}))
    assert _kind(e) == "Schema"
    # round-robin over the catalog
    assert [json.loads(f.mint(0, "t"))["spec"]["task_id"] for _ in range(3)] == ["mf:s1", "mf:s0", "mf:s1"]

    c = json.loads(T.Factory("code", "cf", _rows("print hello")).mint(0, "t"))
    hidden = _sha(b"/grader/hidden.py\0# hidden\nprint(open('/workspace/out.txt').read())\n")
    assert c["spec"]["hidden_tests_hash"] == hidden and c["spec"]["env_image"] == "img:cf:s0"
    assert c["spec"]["domain"] == "code" and c["spec"]["horizon_s"] == 30 and c["spec"]["max_tool_calls"] == 10
    assert c["code"]["expected_stdout"] == _sha("code-stdout:print hello") and c["code"]["run"]["timeout_s"] == 5
    assert c["code"]["mutants"] == [{"id": "wrong-stdout", "files": {"/workspace/out.txt": "WRONG\n"}}]
    assert c["code"]["image"]["hidden_tests_hash"] == hidden and c["code"]["image"]["agent_files"] == {}

    s = json.loads(T.Factory("swe", "sf", _rows("repo@abc")).mint(0, "t"))
    assert s["spec"]["horizon_s"] == 60 and s["spec"]["max_tool_calls"] == 20 and s["code"]["run"]["timeout_s"] == 10
    assert s["code"]["image"]["agent_files"] == {"/workspace/repo": "repo@abc"}
    assert s["code"]["expected_stdout"] == _sha("swe-stdout:repo@abc") and s["code"]["mutants"][0]["id"] == "wrong-patch"

    for rows, kind in (("[]", "EmptyCatalog"), (_rows(""), "EmptyStatement")):
        with pytest.raises(NativeError) as e:
            T.Factory("math", "x", rows).mint(0, "t")
        assert _kind(e) == kind
    with pytest.raises(NativeError):
        T.Factory("poetry", "x", "[]")
    prov = json.dumps([{"id": "a", "source": "s", "body": "b", "license": "MIT", "author": "me"}])
    assert json.loads(T.Factory("math", "x", prov).mint(0, "t"))["spec"]["provenance"] == {
        "source": "s", "license": "MIT", "author": "me"}


def test_wave2_factories_and_scoring():
    grid = [[1, 2], [3, 4]]
    arc = T.Factory("arc", "af", json.dumps([{"id": "g", "source": "s", "body": "solve", "expected": grid}]))
    a = arc.mint(0, "t")
    aj = json.loads(a)
    assert aj["spec"]["hidden_tests_hash"] == _sha("[[1,2],[3,4]]") and aj["spec"]["domain"] == "arc"
    assert aj["verifier_kind"] == "grid_match"
    assert T.score_attempt(a, "[[1,2],[3,4]]") and T.score_attempt(a, " [[[9]], [[1,2],[3,4]]] ")
    assert not T.score_attempt(a, "[[1,2],[3,5]]") and not T.score_attempt(a, "[[[1]],[[2]],[[1,2],[3,4]]]")  # pass@2
    assert not T.score_attempt(a, "garbage") and not T.score_attempt(a, "[[1,2],[3]]") and not T.score_attempt(a, "[[10]]")

    fc = T.Factory("forecast", "ff", json.dumps([{"id": "m", "source": "s", "body": "will it rain",
                                                  "market": {"outcome": True, "market_p": 0.25}}]))
    m = fc.mint(0, "t")
    assert json.loads(m)["spec"]["hidden_tests_hash"] == _sha("true:0.25")
    assert T.score_attempt(m, "0.5") and not T.score_attempt(m, "0.25") and not T.score_attempt(m, "0.1")
    assert not T.score_attempt(m, "1.5") and not T.score_attempt(m, "nan") and not T.score_attempt(m, "abc")

    rs = T.Factory("research", "rf", json.dumps([{"id": "r", "source": "s", "body": "speedrun", "kind": "speedrun",
                                                  "target": 3.28, "budget_gpu_minutes": 5}]))
    r = rs.mint(0, "t")
    rj = json.loads(r)
    assert rj["spec"]["hidden_tests_hash"] == _sha(struct.pack("<d", 3.28)) and rj["spec"]["horizon_s"] == 600
    assert rj["research"] == {"kind": "speedrun", "target": 3.28, "budget_gpu_minutes": 5, "rubric": None}
    assert rj["spec"]["domain"] == "science"
    assert T.score_attempt(r, " 3.28 ") and not T.score_attempt(r, "3.29") and not T.score_attempt(r, "x")

    rubric = {"criteria": [{"id": "clarity", "prompt": "is it clear", "weight": 1.0},
                           {"id": "rigor", "prompt": "is it rigorous", "weight": 3.0}]}
    oe = T.Factory("open_ended", "of", json.dumps([{"id": "o", "source": "s", "body": "write", "rubric": rubric}]))
    o = oe.mint(0, "t")
    assert json.loads(o)["spec"]["hidden_tests_hash"] == _sha(b"clarity\0is it clear\0rigor\0is it rigorous\0")
    assert T.score_attempt(o, json.dumps({"clarity": 0.0, "rigor": 0.8}))          # 0.6
    assert not T.score_attempt(o, json.dumps({"clarity": 1.0, "rigor": 0.2}))      # 0.4
    assert not T.score_attempt(o, json.dumps({"clarity": 1.0})) and not T.score_attempt(o, json.dumps({"clarity": 2, "rigor": 1}))

    cps = [{"id": "c1", "statement": "step 1", "math": {"expected": "4"}, "code": None, "grid": None},
           {"id": "c2", "statement": "step 2", "math": None, "code": None, "grid": {"expected": grid}}]
    lh = T.Factory("long_horizon", "lf", json.dumps([{"id": "l", "source": "s", "body": "long", "checkpoints": cps,
                                                      "final_math": {"expected": "done"}}]))
    l = lh.mint(0, "t")
    lj = json.loads(l)
    want = ("math:4\0grid:" + _sha("[[1,2],[3,4]]") + "\0final:math:done").encode()
    assert lj["spec"]["hidden_tests_hash"] == _sha(want)
    assert lj["spec"]["horizon_s"] == 3600 and lj["spec"]["max_tool_calls"] == 2000 and lj["spec"]["domain"] == "agent"
    good = json.dumps({"checkpoints": ["4", "[[1,2],[3,4]]"], "final": "done"})
    assert T.score_attempt(l, good)
    assert not T.score_attempt(l, json.dumps({"checkpoints": ["4"], "final": "done"}))
    assert not T.score_attempt(l, json.dumps({"checkpoints": ["5", "[[1,2],[3,4]]"], "final": "done"}))
    assert not T.score_attempt(l, json.dumps({"checkpoints": ["4", "[[1,2],[3,4]]"], "final": "nope"}))
    assert not T.score_attempt(l, "not json")
    with pytest.raises(NativeError) as e:
        T.score_attempt(json.dumps({"statement": "s"}), "x")
    assert _kind(e) == "Unverifiable"


def test_solve_rate_filter_and_horizon():
    f = T.Factory("math", "mf", _rows("q1"))
    task = f.mint(0, "t")
    expected = json.loads(task)["math"]["expected"]
    solver = T.ScriptedSolver()
    with pytest.raises(NativeError) as e:
        T.SolveRateFilter.probe(solver, task, 3)
    assert _kind(e) == "Unverifiable"
    solver.insert("q1", expected)
    always = T.SolveRateFilter.probe(solver, task, 4)
    assert (always.passed, always.n, always.rate(), always.in_open_interval()) == (4, 4, 1.0, False)
    with pytest.raises(NativeError) as e:
        T.SolveRateFilter.keep(always)
    assert _kind(e) == "Trivial"
    solver.insert("q1", "wrong")
    never = T.SolveRateFilter.probe(solver, task, 4)
    with pytest.raises(NativeError) as e:
        T.SolveRateFilter.keep(never)
    assert _kind(e) == "Impossible"
    calls = []

    def flaky(statement, now):
        calls.append((statement, now))
        return expected if len(calls) % 2 else "wrong"

    some = T.SolveRateFilter.probe(flaky, task, 4, 77)
    assert (some.passed, some.n) == (2, 4) and some.in_open_interval() and calls[0] == ("q1", 77)
    kept = T.SolveRateFilter.keep(some)
    assert kept.rate() == 0.5
    for call in (lambda: T.SolveRateFilter.probe(flaky, task, 0), lambda: T.SolveRateFilter.keep(T.SolveRate(0, 0))):
        with pytest.raises(NativeError) as e:
            call()
        assert _kind(e) == "BadN"
    assert T.SolveRate(0, 0).rate() == 0.0

    h = T.Horizon()
    assert h.tool_calls == T.START_TOOL_CALLS == 10
    h.raise_if(0.5)
    assert h.tool_calls == 10
    h.raise_if(0.51)
    h.raise_if(0.9)
    assert h.tool_calls == 40
    for _ in range(40):
        h.raise_if(1.0)
    assert h.tool_calls == 2 ** 32 - 1
