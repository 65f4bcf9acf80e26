"""Behaviour list of the kill switch and its tripwires (C++ ``native.monitors``; reference
harness/monitors/tests/{boundaries,fault,graders,held_out,iface,kernel,kill,now,open,plant,
properties,self_check}.rs): every boundary trips the same freeze, the first freeze keeps its
time and reason, later violations are still appended, the freeze file is the state (a
corrupt one fails the open and is left alone), the file format of the reference, injected
time, and a Python model under random operations with reopens."""
import json
import os
import random
import time

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

M = native.monitors
KIND = {"kernel": "Message", "graders": "GraderHashMismatch", "held_out": "HeldOutAccess", "monitors": "MonitorSelfCheck"}
REASON = {"kernel": "kernel escape", "graders": "grader hash mismatch", "held_out": "held-out access blocked", "monitors": "monitor self-check failed"}
ON_DISK = {"kernel": "Kernel", "graders": "Graders", "held_out": "HeldOut", "monitors": "Monitors"}
NOT_FROZEN = {"frozen": False, "frozen_at": None, "reason": None, "violations": []}


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    return e.value


def mon(tmp_path, graders=None, name="freeze.json"):
    return M.Monitors(str(tmp_path / name), graders or {})


def real_trip(m, boundary, detail, now):
    return {"kernel": m.note_kernel_escape, "held_out": m.note_held_out_access, "monitors": m.note_self_check}[boundary](detail, now)


# ------------------------------------------------------------------------------ open
def test_open_without_a_file_is_not_frozen_and_creates_nothing(tmp_path):
    m = M.Monitors(str(tmp_path / "a" / "b" / "freeze.json"))
    assert not m.frozen() and m.snapshot() == NOT_FROZEN and not (tmp_path / "a").exists()
    assert M.BOUNDARIES == ["kernel", "graders", "held_out", "monitors"]
    assert sorted(n for n in dir(M.Monitors) if not n.startswith("_")) == \
        ["frozen", "kill", "note_grader_hash", "note_held_out_access", "note_kernel_escape", "note_self_check", "plant", "snapshot"]   # no way to thaw


@pytest.mark.parametrize("body", ['{"frozen": tr', "", "nope", "[1]", "null", '{"reason": "x", "violations": []}', '{"frozen": "yes", "violations": []}',
                                  '{"frozen": true}', '{"frozen": true, "violations": [{"boundary": "Nowhere", "at_ms": 1, "detail": ""}]}',
                                  '{"frozen": true, "violations": [{"boundary": "Kernel"}]}', '{"frozen": true, "frozen_at": -4, "violations": []}'])
def test_a_corrupt_freeze_file_fails_the_open_and_is_left_alone(tmp_path, body):
    (tmp_path / "freeze.json").write_text(body)
    e = err(lambda: mon(tmp_path))
    assert e.kind == "Message" and str(e) not in REASON.values()                               # not reported as some boundary's violation
    assert (tmp_path / "freeze.json").read_text() == body
    (tmp_path / "d.json").mkdir()
    err(lambda: mon(tmp_path, name="d.json"))                                                  # a directory there fails too


def test_hand_written_snapshots_load(tmp_path):
    (tmp_path / "freeze.json").write_text('{"frozen": false, "frozen_at": null, "reason": null, "violations": []}')
    assert not mon(tmp_path).frozen()
    (tmp_path / "short.json").write_text('{"frozen": false, "violations": []}')                # an absent time and reason read as none
    assert mon(tmp_path, name="short.json").snapshot() == NOT_FROZEN
    (tmp_path / "hand.json").write_text(json.dumps({"frozen": True, "frozen_at": 7, "reason": "hand", "extra": [1], "violations": [
        {"boundary": "HeldOut", "at_ms": 6, "detail": "agent-3", "more": 1}, {"boundary": "kernel", "at_ms": 7, "detail": ""}]}))
    m = mon(tmp_path, name="hand.json")
    assert m.frozen() and m.snapshot() == {"frozen": True, "frozen_at": 7, "reason": "hand", "violations": [
        {"boundary": "held_out", "detail": "agent-3", "at_ms": 6}, {"boundary": "kernel", "detail": "", "at_ms": 7}]}
    assert mon(tmp_path, name="hand.json").snapshot() == m.snapshot()                          # two opens agree


# ------------------------------------------------------------------------------ tripwires
def test_grader_hashes_are_compared_exactly(tmp_path):
    m = mon(tmp_path, {"g1": "abcDEF", "g2": "0123"})
    m.note_grader_hash("g1", "abcDEF", 1)
    m.note_grader_hash("g2", "0123", 2)
    assert not m.frozen() and not (tmp_path / "freeze.json").exists()                          # matching hashes never freeze or write
    for n, (grader, sha) in enumerate([("g1", "abcdef"), ("g1", "abcDEF "), ("g1", ""), ("g3", "abcDEF"), ("", "")]):
        fresh = mon(tmp_path, {"g1": "abcDEF", "g2": "0123"}, f"g{n}.json")
        assert err(fresh.note_grader_hash, grader, sha, 5).kind == "GraderHashMismatch" and fresh.frozen()
        assert fresh.snapshot()["violations"] == [{"boundary": "graders", "detail": grader, "at_ms": 5}]
    assert err(mon(tmp_path, {}, "empty.json").note_grader_hash, "g1", "x", 1).kind == "GraderHashMismatch"     # nothing configured: nothing matches
    one = mon(tmp_path, {"g1": "aa", "g2": "bb"}, "one.json")
    one.note_grader_hash("g1", "aa", 1)
    assert err(one.note_grader_hash, "g2", "aa", 2).kind == "GraderHashMismatch"               # one good grader does not excuse another
    one.note_grader_hash("g1", "aa", 3)                                                        # a match is still fine after the freeze
    assert len(one.snapshot()["violations"]) == 1


@pytest.mark.parametrize("boundary", ["kernel", "held_out", "monitors"])
@pytest.mark.parametrize("detail", ["cap-net-raw", "", "ünï ☃ who"])
def test_every_attempt_trips_whatever_the_detail(tmp_path, boundary, detail):
    m = mon(tmp_path)
    e = err(real_trip, m, boundary, detail, 11)
    assert e.kind == KIND[boundary] and str(e) == REASON[boundary]
    assert m.frozen() and m.snapshot() == {"frozen": True, "frozen_at": 11, "reason": REASON[boundary], "violations": [{"boundary": boundary, "detail": detail, "at_ms": 11}]}
    on_disk = json.loads((tmp_path / "freeze.json").read_text())
    assert on_disk == {"frozen": True, "frozen_at": 11, "reason": REASON[boundary], "violations": [{"boundary": ON_DISK[boundary], "at_ms": 11, "detail": detail}]}
    assert err(real_trip, m, boundary, detail, 12).kind == KIND[boundary]                      # again: still an error, still frozen, appended
    assert [v["at_ms"] for v in m.snapshot()["violations"]] == [11, 12] and m.snapshot()["frozen_at"] == 11


def test_plant_takes_the_same_path_as_a_real_violation(tmp_path):
    for b in M.BOUNDARIES:
        planted, real = mon(tmp_path, name=f"p-{b}.json"), mon(tmp_path, name=f"r-{b}.json")
        e = err(planted.plant, b, "x", 3)
        assert e.kind == KIND[b]
        if b == "graders":
            err(real.note_grader_hash, "x", "nope", 3)
        else:
            err(real_trip, real, b, "x", 3)
        assert planted.snapshot() == real.snapshot()
        assert (tmp_path / f"p-{b}.json").read_text() == (tmp_path / f"r-{b}.json").read_text()
    for unknown in ("Kernel", "HeldOut", "held-out", "", "all"):
        m = mon(tmp_path, name="u.json")
        assert err(m.plant, unknown, "x", 1).kind == "UnknownBoundary" and not m.frozen()      # the file's spelling is not the API's


# ------------------------------------------------------------------------------ kill
def test_operator_kill(tmp_path):
    m = M.Monitors(str(tmp_path / "deep" / "er" / "freeze.json"))
    t0 = time.monotonic()
    m.kill("operator said so", 0)                                                              # time zero is a legal time
    assert time.monotonic() - t0 < 2
    assert m.snapshot() == {"frozen": True, "frozen_at": 0, "reason": "operator said so", "violations": []}     # a kill is not a violation
    assert json.loads((tmp_path / "deep" / "er" / "freeze.json").read_text()) == {"frozen": True, "frozen_at": 0, "reason": "operator said so", "violations": []}
    assert err(m.kill, "again", 5).kind == "AlreadyFrozen" and m.snapshot()["frozen_at"] == 0 and m.snapshot()["reason"] == "operator said so"
    late = mon(tmp_path, name="late.json")
    err(late.plant, "kernel", "cap", 1)
    assert err(late.kill, "late", 2).kind == "AlreadyFrozen" and late.snapshot()["reason"] == "kernel escape"
    big = mon(tmp_path, name="big.json")
    big.kill("end of time", 2 ** 64 - 1)
    assert mon(tmp_path, name="big.json").snapshot()["frozen_at"] == 2 ** 64 - 1


def test_the_first_freeze_keeps_its_time_and_reason(tmp_path):
    m = mon(tmp_path, {"g": "aa"})
    err(m.note_kernel_escape, "a", 100)
    err(m.note_held_out_access, "b", 50)                                                       # even an earlier timestamp does not replace it
    err(m.note_grader_hash, "g", "bb", 200)
    err(m.note_self_check, "c", 300)
    snap = m.snapshot()
    assert (snap["frozen_at"], snap["reason"]) == (100, "kernel escape")
    assert [(v["boundary"], v["detail"], v["at_ms"]) for v in snap["violations"]] == [("kernel", "a", 100), ("held_out", "b", 50), ("graders", "g", 200), ("monitors", "c", 300)]
    copy = m.snapshot()
    copy["violations"].clear()
    assert len(m.snapshot()["violations"]) == 4                                                # a snapshot is a copy
    again = mon(tmp_path, {})
    assert again.snapshot() == snap and again.frozen()                                         # the file is the state
    os.remove(tmp_path / "freeze.json")
    assert m.frozen() and not mon(tmp_path).frozen()                                           # a live instance stays frozen; only a new one reads the disk
    err(m.note_self_check, "d", 400)
    assert mon(tmp_path).frozen() and len(mon(tmp_path).snapshot()["violations"]) == 5         # and its next violation writes the file back


# ------------------------------------------------------------------------------ model
@pytest.mark.parametrize("seed", range(6))
def test_random_operations_match_a_model_across_reopens(tmp_path, seed):
    rng = random.Random(seed)
    graders = {"g1": "h1", "g2": "h2"}
    m = mon(tmp_path, graders)
    state = dict(NOT_FROZEN, violations=[])
    for now in range(1, 80):
        op = rng.choice(["grader", "grader", "held_out", "kernel", "monitors", "plant", "kill", "reopen"] if rng.random() < 0.4 else ["grader", "reopen"])
        want = None

        def trip(b, detail):
            state["violations"].append({"boundary": b, "detail": detail, "at_ms": now})
            if not state["frozen"]:
                state.update(frozen=True, frozen_at=now, reason=REASON[b])
            return KIND[b]
        if op == "grader":
            g, h = rng.choice(["g1", "g2", "g3"]), rng.choice(["h1", "h2"])
            call = lambda: m.note_grader_hash(g, h, now)
            if graders.get(g) != h:
                want = trip("graders", g)
        elif op in ("held_out", "kernel", "monitors"):
            d = rng.choice(["", "x", "yy"])
            call, want = (lambda: real_trip(m, op, d, now)), trip(op, d)
        elif op == "plant":
            b = rng.choice(M.BOUNDARIES + ["bogus"])
            call = lambda: m.plant(b, "p", now)
            want = "UnknownBoundary" if b == "bogus" else trip(b, "p")
        elif op == "kill":
            call = lambda: m.kill("op", now)
            if state["frozen"]:
                want = "AlreadyFrozen"
            else:
                state.update(frozen=True, frozen_at=now, reason="op")
        else:
            m = mon(tmp_path, graders)
            call = lambda: None
        if want is None:
            call()
        else:
            assert err(call).kind == want
        assert m.frozen() == state["frozen"] and m.snapshot() == state
        if (tmp_path / "freeze.json").exists():
            disk = json.loads((tmp_path / "freeze.json").read_text())
            assert disk["frozen"] and [v["boundary"] for v in disk["violations"]] == [ON_DISK[v["boundary"]] for v in state["violations"]]
        else:
            assert not state["frozen"]
