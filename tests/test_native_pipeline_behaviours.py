"""Behaviour list of the oracle -> implementers -> review -> merge pipeline (C++
``native.pipeline``; reference harness/pipeline/tests/{create_open,payload,planted,review,
stages,replay,properties}.rs): task ids and payloads, the planted-bad marker, the review
rule and the merge gate, every stage transition and every refusal, replay from the queue's
log. A Python model of the state machine is driven with the same random operations."""
import json
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

P, L = native.pipeline, native.leases
MARK = b"PLANTED_BAD_PATCH"


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def cand(i, angle="a", patch=b"good"):
    return P.Candidate(str(i), angle, patch)


def to_implement(p, now=0):
    p.start_oracle(now)
    p.record_oracle(False, now)
    return p.start_implementers(now)


# ------------------------------------------------------------------------------ create / open
def test_create_and_open(tmp_path):
    assert (P.DEFAULT_N_IMPLEMENTERS, P.DEFAULT_MAX_ROUNDS, P.PLANTED_BAD_MARKER) == (3, 3, MARK)
    d = str(tmp_path / "p")
    p = P.Pipeline.create(d, "kernels")
    assert (p.stage, p.round, p.stub_failed, p.module, p.candidates) == ("Interface", 0, False, "kernels", [])
    assert p.queue().dir == d + "/queue" and p.queue().log_len() == 0                       # the pipeline owns a queue of its own
    err(lambda: P.Pipeline.create(d, "kernels"))
    err(lambda: P.Pipeline.open(str(tmp_path / "missing"), "kernels"))
    again = P.Pipeline.open(d, "kernels")
    assert (again.stage, again.round, again.stub_failed) == ("Interface", 0, False)
    five = P.Pipeline.create(str(tmp_path / "five"), "m", 5, 1)
    assert len(to_implement(five)) == 5


# ------------------------------------------------------------------------------ payloads
def test_work_payload_task_ids_and_merging():
    tid, body = P.work_payload("m", "oracle", "{}")
    assert tid == "oracle/m/0" and json.loads(body) == {"module": "m", "role": "oracle"}
    tid, body = P.work_payload("m", "r", json.dumps({"module": "other", "role": "x", "round": 4, "keep": [1]}))
    assert tid == "r/m/4" and json.loads(body) == {"module": "m", "role": "r", "round": 4, "keep": [1]}        # the arguments win
    assert P.work_payload("m", "r", json.dumps({"round": 1, "op": "submit", "candidate": "2"}))[0] == "r/m/1/submit/2"
    assert P.work_payload("m", "r", json.dumps({"candidate": "2"}))[0] == "r/m/0/2" and P.work_payload("m", "r", json.dumps({"op": "x"}))[0] == "r/m/0/x"
    assert P.work_payload("m", "r", json.dumps({"op": 3, "candidate": None}))[0] == "r/m/0"                    # only strings extend the id
    for extra in (None, [1, 2], 3, "text", True):
        tid, body = P.work_payload("m", "r", json.dumps(extra))
        assert tid == "r/m/0" and json.loads(body) == {"extra": extra, "module": "m", "role": "r"}             # a non-object is nested
    for bad_round in (-1, 2.5, "7", None, [1]):
        assert P.work_payload("m", "r", json.dumps({"round": bad_round}))[0] == "r/m/0"                        # not a round number: round 0
    assert P.work_payload("m", "r", '{"b": 1, "a": 2}') == P.work_payload("m", "r", '{"a": 2, "b": 1}')        # deterministic


def test_what_each_stage_enqueues(tmp_path):
    p = P.Pipeline.create(str(tmp_path / "p"), "mod", 2, 3)
    q = p.queue()
    assert p.start_oracle(5) == "oracle/mod/0" and q.queued_ids() == ["oracle/mod/0"]
    assert json.loads(q.get("oracle/mod/0").payload_json) == {"module": "mod", "role": "oracle", "round": 0}
    p.record_oracle(False, 6)
    ids = p.start_implementers(7)
    assert ids == ["implementer/mod/0/0", "implementer/mod/0/1"]
    assert [json.loads(q.get(i).payload_json) for i in ids] == [{"candidate": str(k), "module": "mod", "role": "implementer", "round": 0} for k in range(2)]
    p.submit_candidate(cand(1, "fast", b"\x00\xffz"), 8)
    sub = json.loads(q.get("pipeline/mod/0/submit_candidate/1").payload_json)
    assert (sub["op"], sub["angle"], sub["candidate"], sub["patch"]) == ("submit_candidate", "fast", "1", [0, 255, 122])
    assert p.start_review(9) == "reviewer/mod/0"
    assert p.record_verdict(P.Verdict.reject_all(["d1", "d2"]), 10) == "Implement"
    assert json.loads(q.get("pipeline/mod/0/record_verdict").payload_json)["verdict"] == {"RejectAll": {"defects": ["d1", "d2"]}}
    assert p.start_review(11) == "reviewer/mod/1"                                                              # the round is in the id
    assert P.Verdict.pick("3").to_json() == '{"Pick":"3"}' and json.loads(P.Verdict.reject_all([]).to_json()) == {"RejectAll": {"defects": []}}
    assert all(t == "task.enqueued" for t in q.event_types())                                                  # the pipeline only enqueues; workers claim


# ------------------------------------------------------------------------------ planted marker
@pytest.mark.parametrize("patch, planted", [
    (b"", False), (b"diff --git a b", False), (MARK, True), (b"xx" + MARK + b"yy", True), (MARK[:-1], False), (MARK[1:], False),
    (MARK.lower(), False), (MARK[:8] + b"_" + MARK[8:], False), (MARK + MARK, True), (MARK[:-1] + MARK, True), (b"\x00\xff" + MARK + b"\x00", True),
    (b"PLANTED_BAD_PATC" + b"PLANTED_BAD_PATCH", True), (b"PLANTED BAD PATCH", False),
])
def test_planted_marker(patch, planted):
    assert P.is_planted_bad(patch) is planted


def test_random_patches_agree_with_substring_search():
    rng = random.Random(0)
    for _ in range(300):
        parts = [rng.choice([MARK, MARK[:rng.randint(0, 16)], bytes(rng.randrange(256) for _ in range(rng.randint(0, 6))), b"PLANTED_"]) for _ in range(rng.randint(0, 4))]
        patch = b"".join(parts)
        assert P.is_planted_bad(patch) == (MARK in patch)


# ------------------------------------------------------------------------------ review / merge gate
def model_review(cands, ok):
    defects = []
    for c, passed in zip(cands, ok):
        if MARK in c[1]:
            defects.append(f"candidate {c[0]} is planted-bad")
        elif not passed:
            defects.append(f"candidate {c[0]} tests failed")
        else:
            return ("pick", c[0])
    return ("reject", defects or ["no candidates"])


def model_merge(verdict, cands, ok):
    if len(cands) != len(ok) or verdict[0] != "pick":
        return "Other"
    for c, passed in zip(cands, ok):
        if c[0] == verdict[1]:
            return "PlantedBad" if MARK in c[1] else ("ok" if passed else "CandidateFailed")
    return "NoCandidate"


def test_review_rule():
    good, bad = b"fine", b"x" + MARK
    v = P.review([cand(5, patch=good), cand(2, patch=good)], [True, True])
    assert v.is_pick and v.candidate == "5"                                                                    # slice order, not id order
    v = P.review([cand(0, patch=bad), cand(1, patch=good), cand(2, patch=good)], [True, False, True])
    assert v.is_pick and v.candidate == "2"
    v = P.review([cand(0, patch=bad), cand(1, patch=bad)], [True, True])
    assert not v.is_pick and v.defects == ["candidate 0 is planted-bad", "candidate 1 is planted-bad"]        # never a planted one
    v = P.review([cand(0), cand(1)], [False, False])
    assert not v.is_pick and v.defects == ["candidate 0 tests failed", "candidate 1 tests failed"]
    v = P.review([], [])
    assert not v.is_pick and v.defects                                                                         # nothing to pick is still a rejection with a reason
    assert err(lambda: P.review([cand(0)], [])).kind == "Other" and err(lambda: P.review([], [True])).kind == "Other"


def test_merge_gate():
    cs = [cand(0, patch=b"ok"), cand(1, patch=MARK), cand(2, patch=b"ok")]
    P.merge_allowed(P.Verdict.pick("0"), cs, [True, True, False])
    assert err(lambda: P.merge_allowed(P.Verdict.pick("1"), cs, [True, True, False])).kind == "PlantedBad"
    assert err(lambda: P.merge_allowed(P.Verdict.pick("1"), cs, [True, False, False])).kind == "PlantedBad"    # planted outranks failing
    assert err(lambda: P.merge_allowed(P.Verdict.pick("2"), cs, [True, True, False])).kind == "CandidateFailed"
    assert err(lambda: P.merge_allowed(P.Verdict.pick("9"), cs, [True, True, True])).kind == "NoCandidate"
    assert err(lambda: P.merge_allowed(P.Verdict.reject_all(["x"]), cs, [True, True, True])).kind == "Other"
    assert err(lambda: P.merge_allowed(P.Verdict.pick("0"), cs, [True])).kind == "Other"


def test_random_reviews_and_merges_agree_with_the_model():
    rng = random.Random(1)
    for _ in range(300):
        n = rng.randint(0, 5)
        raw = [(str(rng.randint(0, 6)), rng.choice([b"ok", b"a" + MARK, b""])) for _ in range(n)]
        ok = [rng.random() < 0.5 for _ in range(n)]
        v = P.review([P.Candidate(i, "a", p) for i, p in raw], ok)
        want = model_review(raw, ok)
        assert (("pick", v.candidate) if v.is_pick else ("reject", v.defects)) == want
        pick = ("pick", str(rng.randint(0, 6)))
        ok2 = ok if rng.random() < 0.85 else ok + [True]
        outcome = model_merge(pick, raw, ok2)
        call = lambda: P.merge_allowed(P.Verdict.pick(pick[1]), [P.Candidate(i, "a", p) for i, p in raw], ok2)
        if outcome == "ok":
            call()
        else:
            assert err(call).kind == outcome
        if v.is_pick and len({i for i, _ in raw}) == n:
            P.merge_allowed(v, [P.Candidate(i, "a", p) for i, p in raw], ok)                                   # what review picks, the gate lets through


# ------------------------------------------------------------------------------ stages
def test_happy_path_and_refusals_along_it(tmp_path):
    p = P.Pipeline.create(str(tmp_path / "p"), "m")
    wrong = lambda call: err(call).kind == "WrongStage"
    merge = lambda: p.record_merge("m", "15.2", "abc", 3, 0, ["fv-1"], 9)
    assert all(wrong(c) for c in (lambda: p.record_oracle(False, 0), lambda: p.submit_candidate(cand(0), 0), lambda: p.start_review(0),
                                  lambda: p.record_verdict(P.Verdict.pick("0"), 0), merge))
    e = err(lambda: p.record_oracle(False, 0))
    assert "Oracle" in str(e) and "Interface" in str(e)                                                        # names the stage it wanted and the one it is at
    assert err(lambda: p.start_implementers(0)).kind == "StubNotFailed"
    p.start_oracle(1)
    assert p.stage == "Oracle" and wrong(lambda: p.start_oracle(1)) and err(lambda: p.start_implementers(1)).kind == "StubNotFailed"
    assert err(lambda: p.record_oracle(True, 2)).kind == "StubPassed" and (p.stage, p.stub_failed) == ("Oracle", False)   # a stub that passes proves nothing
    p.record_oracle(False, 3)
    assert (p.stage, p.stub_failed) == ("StubMustFail", True) and wrong(lambda: p.submit_candidate(cand(0), 3)) and wrong(lambda: p.record_oracle(False, 3))
    p.start_implementers(4)
    assert p.stage == "Implement" and all(wrong(c) for c in (lambda: p.start_oracle(4), lambda: p.record_oracle(False, 4), lambda: p.start_implementers(4),
                                                             lambda: p.record_verdict(P.Verdict.pick("0"), 4), merge))
    assert err(lambda: p.submit_candidate(cand(3), 5)).kind == "NoCandidate" and err(lambda: p.submit_candidate(P.Candidate("x", "a", b""), 5)).kind == "NoCandidate"
    p.submit_candidate(cand(1, "one", b"v1"), 5)
    p.submit_candidate(cand(0, "zero", MARK), 5)                                                               # a planted patch may be submitted
    p.submit_candidate(cand(1, "uno", b"v2"), 6)
    assert [(c.id, c.angle, c.patch) for c in p.candidates] == [("1", "uno", b"v2"), ("0", "zero", MARK)]      # first-submit order, last write wins
    p.start_review(7)
    assert p.stage == "Review" and wrong(lambda: p.submit_candidate(cand(2), 7)) and wrong(lambda: p.start_review(7))
    assert err(lambda: p.record_verdict(P.Verdict.pick("2"), 8)).kind == "NoCandidate" and p.stage == "Review"  # never submitted
    assert err(lambda: p.record_verdict(P.Verdict.pick("0"), 8)).kind == "PlantedBad" and p.stage == "Review"
    assert p.record_verdict(P.Verdict.pick("1"), 8) == "Merged" and wrong(lambda: p.record_verdict(P.Verdict.pick("1"), 8))
    err(lambda: p.record_merge("other", "15.2", "abc", 3, 0, [], 9))
    merge()
    assert p.stage == "Merged" and [c.id for c in p.candidates] == ["1", "0"]


@pytest.mark.parametrize("max_rounds", [1, 2, 3])
def test_rejected_rounds_retry_then_block(tmp_path, max_rounds):
    p = P.Pipeline.create(str(tmp_path / "p"), "m", 2, max_rounds)
    to_implement(p)
    for r in range(max_rounds):
        p.submit_candidate(cand(0), r)
        p.start_review(r)                                                                                      # a review with nothing new is allowed too
        stage = p.record_verdict(P.Verdict.reject_all([f"round {r}"]), r)
        assert stage == ("Blocked" if r == max_rounds - 1 else "Implement") and p.round == r + 1
        assert p.candidates == []                                                                              # the rejected patches are dropped
        if stage == "Implement":
            assert p.queue().queued_ids()[-2:] == [f"implementer/m/{r + 1}/0", f"implementer/m/{r + 1}/1"]     # the next round's work is already queued
    for call in (lambda: p.start_oracle(9), lambda: p.start_implementers(9), lambda: p.start_review(9), lambda: p.submit_candidate(cand(0), 9),
                 lambda: p.record_verdict(P.Verdict.pick("0"), 9), lambda: p.record_merge("m", "1", "c", 0, 0, [], 9)):
        assert err(call).kind == "WrongStage"
    assert P.Pipeline.open(str(tmp_path / "p"), "m", 2, max_rounds).stage == "Blocked"


# ------------------------------------------------------------------------------ model under random operations
class Model:
    def __init__(self, n, max_rounds):
        self.n, self.max, self.stage, self.round, self.stub, self.cands = n, max_rounds, "Interface", 0, False, []

    def apply(self, op, arg):
        s = self.stage
        if op == "start_oracle":
            if s != "Interface":
                return "WrongStage"
            self.stage = "Oracle"
        elif op == "record_oracle":
            if s != "Oracle":
                return "WrongStage"
            if arg:
                return "StubPassed"
            self.stage, self.stub = "StubMustFail", True
        elif op == "start_implementers":
            if not self.stub:
                return "StubNotFailed"
            if s != "StubMustFail":
                return "WrongStage"
            self.stage = "Implement"
        elif op == "submit":
            if s != "Implement":
                return "WrongStage"
            cid, patch = arg
            if not (cid.isdigit() and int(cid) < self.n):
                return "NoCandidate"
            for i, c in enumerate(self.cands):
                if c[0] == cid:
                    self.cands[i] = (cid, patch)
                    break
            else:
                self.cands.append((cid, patch))
        elif op == "start_review":
            if s != "Implement":
                return "WrongStage"
            self.stage = "Review"
        elif op == "pick":
            if s != "Review":
                return "WrongStage"
            hit = [c for c in self.cands if c[0] == arg]
            if not hit:
                return "NoCandidate"
            if MARK in hit[0][1]:
                return "PlantedBad"
            self.stage = "Merged"
        elif op == "reject":
            if s != "Review":
                return "WrongStage"
            self.round, self.cands = self.round + 1, []
            self.stage = "Blocked" if self.round >= self.max else "Implement"
        return "ok"


@pytest.mark.parametrize("seed", range(8))
def test_random_operations_match_the_model_and_replay(tmp_path, seed):
    rng = random.Random(seed)
    n, max_rounds = rng.choice([1, 2, 3]), rng.choice([1, 2, 3])
    d = str(tmp_path / "p")
    p, m = P.Pipeline.create(d, "mod", n, max_rounds), Model(n, max_rounds)
    order = ["start_oracle", "record_oracle", "start_implementers", "submit", "submit", "start_review", "pick", "reject"]
    for step in range(120):
        op = order[min(len(order) - 1, rng.randrange(len(order) + 2))] if rng.random() < 0.5 else rng.choice(order)
        arg = None
        if op == "record_oracle":
            arg = rng.random() < 0.3
            call = lambda: p.record_oracle(arg, step)
        elif op == "submit":
            arg = (str(rng.randint(0, 3)), rng.choice([b"ok", MARK + b"!", b""]))
            call = lambda: p.submit_candidate(P.Candidate(arg[0], "angle", arg[1]), step)
        elif op == "pick":
            arg = str(rng.randint(0, 3))
            call = lambda: p.record_verdict(P.Verdict.pick(arg), step)
        elif op == "reject":
            call = lambda: p.record_verdict(P.Verdict.reject_all(["no"]), step)
        else:
            call = {"start_oracle": lambda: p.start_oracle(step), "start_implementers": lambda: p.start_implementers(step), "start_review": lambda: p.start_review(step)}[op]
        want = m.apply(op, arg)
        if want == "ok":
            call()
        else:
            assert err(call).kind == want, (op, arg, m.stage)
        if step % 30 == 29:
            p = P.Pipeline.open(d, "mod", n, max_rounds)                                                       # replayed from the queue's log alone
        assert (p.stage, p.round, p.stub_failed) == (m.stage, m.round, m.stub)
        assert [(c.id, c.patch) for c in p.candidates] == m.cands
