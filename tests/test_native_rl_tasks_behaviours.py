"""Remaining behaviour rules of the task factories, the solve-rate filter and the horizon
curriculum (C++ ``native.tasks``; reference rl/tasks/tests/{factories,filter,horizon,types,
wave2_factories,wave2_filter}.rs): cursor and id stability, what a public statement may
contain, byte-exact code scoring, the open-interval gate and the doubling curriculum."""
import hashlib
import json
import math

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

T = native.tasks


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def rows(*bodies, **extra):
    return json.dumps([{"id": f"s{i}", "source": f"src-{i}", "body": b, **extra} for i, b in enumerate(bodies)])


def sha(x):
    return hashlib.sha256(x if isinstance(x, bytes) else x.encode()).hexdigest()


# ------------------------------------------------------------------------------ factories
@pytest.mark.parametrize("kind", ["math", "code", "swe"])
def test_task_ids_are_factory_id_colon_source_id_and_round_robin_wraps(kind):
    f = T.Factory(kind, "fac", rows("a", "b", "c"))
    ids = [json.loads(f.mint(i, "t"))["spec"]["task_id"] for i in range(7)]
    assert ids == ["fac:s0", "fac:s1", "fac:s2", "fac:s0", "fac:s1", "fac:s2", "fac:s0"]
    one = T.Factory(kind, "fac", rows("only"))
    assert json.loads(one.mint(0, "t"))["spec"]["task_id"] == json.loads(one.mint(1, "u"))["spec"]["task_id"] == "fac:s0"


def test_created_at_is_the_callers_string_and_now_is_not_encoded():
    f, g = T.Factory("math", "m", rows("q")), T.Factory("math", "m", rows("q"))
    a, b = json.loads(f.mint(1, "yesterday-ish")), json.loads(g.mint(999999, "yesterday-ish"))
    assert a == b and a["spec"]["created_at"] == "yesterday-ish"


def test_an_empty_statement_does_not_advance_the_cursor():
    f = T.Factory("math", "m", json.dumps([{"id": "bad", "source": "s", "body": ""}, {"id": "ok", "source": "s", "body": "q"}]))
    for _ in range(3):
        assert err(lambda: f.mint(0, "t")).kind == "EmptyStatement"      # still pointing at the same row
    g = T.Factory("math", "m", json.dumps([{"id": "ok", "source": "s", "body": "q"}, {"id": "bad", "source": "s", "body": ""}]))
    assert json.loads(g.mint(0, "t"))["spec"]["task_id"] == "m:ok"
    assert err(lambda: g.mint(0, "t")).kind == "EmptyStatement"


def test_hashes_are_lowercase_hex_and_the_expected_answer_is_not_in_the_statement():
    t = json.loads(T.Factory("math", "m", rows("what is 2+2")).mint(0, "t"))
    for h in (t["spec"]["statement_hash"], t["spec"]["hidden_tests_hash"]):
        assert len(h) == 64 and h == h.lower() and all(c in "0123456789abcdef" for c in h)
    assert t["spec"]["statement_hash"] == sha("what is 2+2") and t["math"]["expected"] not in t["statement"]
    assert sha("") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    code = json.loads(T.Factory("code", "c", rows("print hello")).mint(0, "t"))
    assert code["code"]["expected_stdout"] not in code["statement"] and "hidden" not in code["statement"]


def test_swe_is_strictly_longer_than_code_and_provenance_follows_the_row():
    src = rows("same body")
    code, swe = (json.loads(T.Factory(k, "f", src).mint(0, "t"))["spec"] for k in ("code", "swe"))
    assert swe["horizon_s"] > code["horizon_s"] and swe["max_tool_calls"] > code["max_tool_calls"]
    f = T.Factory("math", "m", rows("a", "b"))
    assert [json.loads(f.mint(0, "t"))["spec"]["provenance"]["source"] for _ in range(3)] == ["src-0", "src-1", "src-0"]
    assert "license" not in json.loads(f.mint(0, "t"))["spec"]["provenance"]          # absent, not null


def test_second_wave_domains_verifiers_and_horizons_are_pinned():
    grid = [[0, 1], [1, 0]]
    specs = {
        "arc": dict(expected=grid),
        "forecast": dict(market={"outcome": False, "market_p": 0.5}),
        "research": dict(kind="paper_repro", target=1.5, budget_gpu_minutes=3),
        "open_ended": dict(rubric={"criteria": [{"id": "c", "prompt": "p", "weight": 1.0}]}),
        "long_horizon": dict(checkpoints=[], final_math={"expected": "x"}),
    }
    got = {}
    for kind, extra in specs.items():
        f = T.Factory(kind, "w2", rows("body", **extra))
        got[kind] = json.loads(f.mint(0, "when"))
        assert got[kind]["spec"]["task_id"] == "w2:s0" and got[kind]["spec"]["created_at"] == "when"
        assert got[kind]["spec"]["statement_hash"] == sha("body")
    assert {k: v["spec"]["domain"] for k, v in got.items()} == {
        "arc": "arc", "forecast": "other", "research": "science", "open_ended": "other", "long_horizon": "agent"}
    assert got["arc"]["verifier_kind"] == "grid_match" and json.dumps(grid, separators=(",", ":")) not in got["arc"]["statement"]
    assert got["long_horizon"]["spec"]["horizon_s"] == 3600 and got["long_horizon"]["spec"]["max_tool_calls"] == 2000
    for kind in ("speedrun", "paper_repro", "kaggle"):
        r = json.loads(T.Factory("research", "r", rows("b", kind=kind, target=2.0, budget_gpu_minutes=1)).mint(0, "t"))
        assert r["research"]["kind"] == kind


def test_empty_catalogs_of_every_kind():
    for kind in T.FACTORY_KINDS:
        assert err(lambda: T.Factory(kind, "f", "[]").mint(0, "t")).kind == "EmptyCatalog"


# ------------------------------------------------------------------------------ scoring
def test_forecast_scoring_beats_the_market_strictly():
    def task(outcome, p):
        return T.Factory("forecast", "f", rows("q", market={"outcome": outcome, "market_p": p})).mint(0, "t")
    yes, no = task(True, 0.6), task(False, 0.6)
    assert T.score_attempt(yes, "0.7") and not T.score_attempt(yes, "0.6") and not T.score_attempt(yes, "0.5")
    assert T.score_attempt(no, "0.0") and T.score_attempt(no, "0.59") and not T.score_attempt(no, "0.6") and not T.score_attempt(no, "0.9")


def test_grid_scoring_is_pass_at_two():
    grid = [[1, 2], [3, 4]]
    t = T.Factory("arc", "a", rows("solve", expected=grid)).mint(0, "t")
    g = json.dumps(grid)
    assert T.score_attempt(t, g) and T.score_attempt(t, f"[{g}]") and T.score_attempt(t, f"[[[0]],{g}]") and T.score_attempt(t, f"[{g},[[0]]]")
    assert not T.score_attempt(t, f"[[[0]],[[1]],{g}]")                     # three candidates is one too many
    assert not T.score_attempt(t, "[[1,2],[3,9]]") and not T.score_attempt(t, "") and not T.score_attempt(t, "{}")


def test_open_ended_needs_a_weighted_score_above_one_half():
    rubric = {"criteria": [{"id": "a", "prompt": "p", "weight": 1.0}, {"id": "b", "prompt": "q", "weight": 1.0}]}
    t = T.Factory("open_ended", "o", rows("write", rubric=rubric)).mint(0, "t")
    assert T.score_attempt(t, json.dumps({"a": 1.0, "b": 0.5})) and not T.score_attempt(t, json.dumps({"a": 0.5, "b": 0.5}))
    assert not T.score_attempt(t, json.dumps({"a": 0.0, "b": 0.9}))


def test_long_horizon_with_no_checkpoints_is_its_final_check_only():
    t = T.Factory("long_horizon", "l", rows("long", checkpoints=[], final_math={"expected": "done"})).mint(0, "t")
    assert T.score_attempt(t, json.dumps({"checkpoints": [], "final": "done"}))
    assert not T.score_attempt(t, json.dumps({"checkpoints": [], "final": "almost"}))
    assert not T.score_attempt(t, json.dumps({"checkpoints": ["extra"], "final": "done"}))


# ------------------------------------------------------------------------------ solve-rate filter
def _math_task(body="q1"):
    task = T.Factory("math", "mf", rows(body)).mint(0, "t")
    return task, json.loads(task)["math"]["expected"]


def test_probe_validates_before_it_calls_the_solver():
    task, _ = _math_task()
    calls = []
    assert err(lambda: T.SolveRateFilter.probe(lambda s, now: calls.append(s) or "x", task, 0)).kind == "BadN"
    assert calls == []
    assert err(lambda: T.SolveRateFilter.probe(lambda s, now: "x", json.dumps({"statement": "s", "math": None, "code": None}), 2)).kind == "Unverifiable"


def test_probe_counts_and_sees_only_the_public_statement():
    task, expected = _math_task("what is it")
    seen = []

    def solver(statement, now):
        seen.append(statement)
        return expected if len(seen) <= 3 else "nope"

    rate = T.SolveRateFilter.probe(solver, task, 5)
    assert (rate.passed, rate.n) == (3, 5) and seen == ["what is it"] * 5 and expected not in seen[0]
    assert T.SolveRateFilter.probe(lambda s, n: expected, task, 3).rate() == 1.0
    assert T.SolveRateFilter.probe(lambda s, n: "", task, 3).rate() == 0.0


def test_code_attempts_are_compared_byte_for_byte():
    task = T.Factory("code", "cf", rows("print hello")).mint(0, "t")
    want = json.loads(task)["code"]["expected_stdout"]
    for reply, ok in ((want, True), (want + "\n", False), (want[:-1], False), (" " + want, False), (want.upper(), False)):
        assert T.SolveRateFilter.probe(lambda s, n: reply, task, 1).passed == (1 if ok else 0)


def test_math_wins_when_a_task_carries_both_payloads_and_solver_errors_propagate():
    task, expected = _math_task()
    both = json.loads(task)
    both["code"] = json.loads(T.Factory("code", "cf", rows("p")).mint(0, "t"))["code"]
    assert T.SolveRateFilter.probe(lambda s, n: expected, json.dumps(both), 2).passed == 2

    def broken(statement, now):
        raise RuntimeError("solver fell over")

    with pytest.raises(Exception, match="fell over"):
        T.SolveRateFilter.probe(broken, task, 2)
    solver = T.ScriptedSolver()
    assert err(lambda: solver.attempt("never inserted", 0)).kind == "Unverifiable"
    solver.insert("q", "a")
    assert solver.attempt("q", 0) == "a"


@pytest.mark.parametrize("passed, n, verdict", [(0, 4, "Impossible"), (4, 4, "Trivial"), (9, 4, "Trivial"), (0, 0, "BadN"),
                                                (1, 4, None), (2, 4, None), (3, 4, None), (1, 1000, None), (999, 1000, None)])
def test_keep_is_an_open_interval_gate(passed, n, verdict):
    rate = T.SolveRate(passed, n)
    if verdict is None:
        assert T.SolveRateFilter.keep(rate).passed == passed and rate.in_open_interval()
    else:
        assert err(lambda: T.SolveRateFilter.keep(rate)).kind == verdict and not rate.in_open_interval()


# ------------------------------------------------------------------------------ horizon
def test_horizon_doubles_only_strictly_above_the_threshold():
    h = T.Horizon()
    assert h.tool_calls == T.START_TOOL_CALLS == 10 and T.RAISE_THRESHOLD == 0.5
    for rate in (0.0, 0.25, 0.5, math.nan, -1.0):
        h.raise_if(rate)
        assert h.tool_calls == 10
    seen = []
    for rate in (0.500001, 0.75, math.inf):
        h.raise_if(rate)
        seen.append(h.tool_calls)
    assert seen == [20, 40, 80]


def test_horizon_follows_the_rule_on_a_grid_of_rates():
    h, want = T.Horizon(), 10
    for i in range(24):
        rate = (i * 7 % 11) / 10.0
        h.raise_if(rate)
        if rate > 0.5:
            want = min(want * 2, 2 ** 32 - 1)
        assert h.tool_calls == want
