"""Behaviour list of the learned-reward layer (``prometheus_b200.rewards`` over the C++
``native.rewards``): rubric panels, pair filters, trajectory views, the tampering detector and
the reward-API records (reference rl/rewards/tests/{rubric,pairs,trajectory,tampering,refuse,
serde_f1,types}.rs)."""
import hashlib
import itertools
import math

import pytest

from prometheus_b200 import contracts, rewards as R
from prometheus_b200.native import NativeError


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def request(**kw):
    base = dict(request_id="rew-1", task_id="task-1", rollout_id="roll-1", trajectory_hash="ab" * 32, verifier_id="panel",
                env_snapshot_id="snap-1")
    base.update(kw)
    return R.reward_request(**base)


def panel(graders=("g0", "g1"), criteria=(("clarity", "is it clear?", 1.0), ("rigor", "is it rigorous?", 3.0)),
          replies=None, output="the answer"):
    rubric = R.Rubric("rub")
    for c in criteria:
        rubric.add(*c)
    judge = R.ScriptedJudge()
    for (g, c), reply in (replies or {}).items():
        prompt = next(p for cid, p, _w in criteria if cid == c)
        judge.insert(R.grader_prompt(g, c, prompt, output), reply)
    return R.RubricPanel("panel", rubric, list(graders), judge)


FULL = {("g0", "clarity"): "1.0", ("g0", "rigor"): "0.5", ("g1", "clarity"): "0.5", ("g1", "rigor"): " 0.5 "}


# ------------------------------------------------------------------------------ rubric panel
def test_prompt_layout_is_pinned():
    assert R.grader_prompt("g1", "clarity", "is it clear?", "the answer") == "grader:g1\ncriterion:clarity\nis it clear?\n\nthe answer"


def test_scores_per_grader_in_rubric_order():
    got = panel(replies=FULL).score("the answer")
    assert [s.grader_id for s in got] == ["g0", "g1"]
    assert got[0].scores == [("clarity", 1.0), ("rigor", 0.5)] and got[1].scores == [("clarity", 0.5), ("rigor", 0.5)]
    assert got[0].weighted == pytest.approx((1.0 * 1 + 0.5 * 3) / 4) and got[1].weighted == pytest.approx(0.5)
    assert R.Rubric("r").total_weight() == 0.0 and panel().rubric.total_weight() == 4.0


def test_empty_rubric_and_empty_panel():
    assert err(lambda: panel(criteria=(), replies={}).score("x")).kind == "EmptyRubric"
    assert err(lambda: panel(graders=()).score("x")).kind == "EmptyPanel"
    assert err(lambda: panel(graders=(), criteria=()).score("x")).kind in ("EmptyRubric", "EmptyPanel")
    assert err(lambda: R.RubricPanel.combine([])).kind == "EmptyPanel"


@pytest.mark.parametrize("weight", [0.0, -1.0, math.nan, math.inf])
def test_bad_weights_are_found_when_scoring_not_when_building(weight):
    p = panel(graders=("g0",), criteria=(("c", "p", weight),), replies={("g0", "c"): "0.5"}, output="x")
    assert err(lambda: p.score("x")).kind == "BadWeight"


@pytest.mark.parametrize("reply, kind", [("1.5", "BadScore"), ("-0.1", "BadScore"), ("nan", "BadScore"), ("inf", "BadScore"),
                                         ("seven", "Unverifiable"), ("   ", "Unverifiable"), ("", "Unverifiable"),
                                         ("0.5 points", "Unverifiable")])
def test_replies_outside_the_unit_interval_or_not_numbers(reply, kind):
    p = panel(graders=("g0",), criteria=(("c", "p", 1.0),), replies={("g0", "c"): reply}, output="x")
    assert err(lambda: p.score("x")).kind == kind


def test_missing_scripted_reply_is_unverifiable_and_endpoints_are_scores():
    assert err(lambda: panel(replies={}).score("the answer")).kind == "Unverifiable"
    p = panel(graders=("g0",), criteria=(("a", "p", 1.0), ("b", "q", 1.0)), replies={("g0", "a"): "0", ("g0", "b"): " 1 "}, output="x")
    assert p.score("x")[0].scores == [("a", 0.0), ("b", 1.0)]


def test_combine_is_mean_times_one_minus_spread_and_never_drops():
    S = lambda *ws: [R.RubricScore(f"g{i}", [], w) for i, w in enumerate(ws)]
    assert R.RubricPanel.combine(S(0.7)) == pytest.approx(0.7)                     # one grader: spread 0
    assert R.RubricPanel.combine(S(0.7, 0.7, 0.7)) == pytest.approx(0.7)
    assert R.RubricPanel.combine(S(0.2, 0.5, 0.9)) == pytest.approx((1.6 / 3) * (1 - 0.7))
    got = R.RubricPanel.combine(S(1.0, 0.7))                                        # spread above the named threshold
    assert 0.3 >= R.DISAGREE_EPS == 0.25 and got == pytest.approx(0.85 * 0.7) and got != 0.0
    assert R.RubricPanel.combine(S(0.625, 0.5)) == pytest.approx(0.5625 * 0.875)
    with_criteria = [R.RubricScore("g", [("c", 0.0)], 0.9)]                          # criterion values are not consulted
    assert R.RubricPanel.combine(with_criteria) == pytest.approx(0.9)


def test_verify_builds_a_contract_response():
    p = panel(replies=FULL)
    resp = p.verify(request(), "the answer", "2026-01-02T03:04:05Z")
    value = 0.5625 * 0.875
    assert resp["score"] == pytest.approx(value) and resp["passed"] is False        # 0.49: not above one half
    assert resp["scored_at"] == "2026-01-02T03:04:05Z" and resp["request_id"] == "rew-1" and resp["scorer_id"] == "panel"
    assert resp["evidence"] == {"kind": "rubric", "hash": hashlib.sha256(b"the answer").hexdigest()} and resp["flags"] == []
    contracts.validate_named("prometheus.reward_response", resp)
    contracts.validate_named("prometheus.reward_request", request())
    half = panel(graders=("g0",), criteria=(("c", "p", 1.0),), replies={("g0", "c"): "0.5"}, output="x")
    assert half.verify(request(), "x", "2026-01-02T03:04:05Z")["passed"] is False   # strictly greater
    more = panel(graders=("g0",), criteria=(("c", "p", 1.0),), replies={("g0", "c"): "0.51"}, output="x")
    assert more.verify(request(), "x", "2026-01-02T03:04:05Z")["passed"] is True
    for bad in (dict(schema_id="prometheus.reward_response"), dict(schema_version=2)):
        req = dict(request(), **bad)
        assert err(lambda: p.verify(req, "the answer", "t")).kind == "Schema"


# ------------------------------------------------------------------------------ trajectory views
def test_hack_kinds_for_every_flag_combination():
    for wrote, special, visible, hidden in itertools.product([False, True], repeat=4):
        v = R.TrajectoryView(wrote_test_file=wrote, special_cased=special, visible_passed=visible, hidden_passed=hidden)
        want = [k for k, on in zip(R.HACK_KINDS, (wrote, special, visible and not hidden)) if on]
        assert list(v.kinds()) == want and v.is_confirmed_hack() == bool(want)       # fixed order of kinds
    paths_only = R.TrajectoryView(test_write_paths=["tests/test_x.py"])
    assert not paths_only.is_confirmed_hack() and list(paths_only.kinds()) == []     # paths alone prove nothing
    assert not R.TrajectoryView(hidden_passed=True).is_confirmed_hack()              # hidden pass, visible fail


# ------------------------------------------------------------------------------ pair filters
CLEAN = R.TrajectoryView(visible_passed=True, hidden_passed=True)
HACK = R.TrajectoryView(visible_passed=True, hidden_passed=False)
PAIR = R.ContrastivePair("in", "be honest", "cheat", "good", "bad")


def test_tamper_pair_filter():
    f = R.TamperPairFilter()
    f.keep(PAIR, CLEAN, HACK)
    for pos, neg in ((CLEAN, CLEAN), (HACK, HACK), (HACK, CLEAN), (CLEAN, R.TrajectoryView(hidden_passed=True))):
        assert err(lambda: f.keep(PAIR, pos, neg)).kind == "UnconfirmedPair"
    f.keep(R.ContrastivePair("", "", "", "", ""), CLEAN, R.TrajectoryView(special_cased=True))   # text is ignored
    held = R.HeldOutHacks()
    held.insert("planted-1", HACK)
    e = err(lambda: f.keep(PAIR, CLEAN, HACK, held_out=held, trajectory_ids=["fresh", "planted-1"]))
    assert e.kind == "HeldOutLeak" and "held-out" in str(e)
    f.keep(PAIR, CLEAN, HACK, held_out=held, trajectory_ids=["fresh-a", "fresh-b"])


def test_rescore_filter_needs_a_strictly_higher_positive():
    f = R.RescoreFilter()
    vals = [-2.0, -0.5, 0.0, 0.25, 0.5, 1.0, 3.0]
    for p, n in itertools.product(vals, vals):
        if p > n:
            f.keep(p, n)
        else:
            assert err(lambda: f.keep(p, n)).kind == "UnconfirmedPair"
    for p, n in ((math.nan, 0.0), (1.0, math.nan), (math.nan, math.nan)):
        assert err(lambda: f.keep(p, n)).kind == "UnconfirmedPair"


# ------------------------------------------------------------------------------ detector
def test_detector_responses():
    d = R.TamperingDetector("detector-v1")
    bad = d.verify(request(), R.TrajectoryView(wrote_test_file=True), "2026-01-02T03:04:05Z")
    assert (bad["score"], bad["passed"], bad["flags"]) == (0.0, False, ["tampering"])
    good = d.verify(request(), CLEAN, "2026-01-02T03:04:05Z")
    assert (good["score"], good["passed"], good["flags"]) == (1.0, True, []) and good["scorer_id"] == "detector-v1"
    for resp in (bad, good):
        contracts.validate_named("prometheus.reward_response", resp)
        assert resp["scored_at"] == "2026-01-02T03:04:05Z"
    assert err(lambda: d.verify(dict(request(), schema_version=9), CLEAN, "t")).kind == "Schema"
    assert d.kinds(HACK) == ["visible_pass_hidden_fail"] and d.is_hack(HACK) and not d.is_hack(CLEAN)


def test_held_out_set_measures_recall_only():
    d, held = R.TamperingDetector("d"), R.HeldOutHacks()
    assert held.eval(d).recall() == 0.0 and held.eval(d) == R.DetectReport(0, 0)
    held.insert("a", R.TrajectoryView(wrote_test_file=True))
    held.insert("b", R.TrajectoryView(special_cased=True))
    held.insert("c", HACK)
    assert held.eval(d) == R.DetectReport(3, 3) and held.eval(d).recall() == 1.0
    held.insert("clean", CLEAN)
    held.insert("hidden-only", R.TrajectoryView(hidden_passed=True))
    assert held.eval(d) == R.DetectReport(5, 3) and held.eval(d).recall() == pytest.approx(0.6)
    held.insert("a", R.TrajectoryView(wrote_test_file=True))                        # same id: replaced, not counted twice
    assert len(held) == 5 and held.contains("a") and not held.contains("zz") and held.get("zz") is None
    assert held.get("c").kinds() == ["visible_pass_hidden_fail"]


# ------------------------------------------------------------------------------ exact verifiers
@pytest.mark.parametrize("verifier", ["sympy-exact", "sandboxed_tests", ""])
def test_a_learned_grader_is_refused_where_an_exact_verifier_scores(verifier):
    e = err(lambda: R.refuse_exact(verifier))
    assert e.kind == "ExactVerifier" and verifier in str(e)


def test_module_reads_no_clock():
    import inspect
    src = inspect.getsource(R)
    assert "time.time" not in src and "datetime.now" not in src and "import time" not in src
