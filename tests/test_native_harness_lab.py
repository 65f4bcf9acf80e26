"""Ledger, lab kernel, eval gate and monitors (C++), against the contracts of the reference's
harness/ledger, harness/kernel, harness/eval-gate and harness/monitors crates."""
import hashlib
import json

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

LG, K, EG, MON = native.ledger, native.kernel, native.eval_gate, native.monitors


def _kind(e):
    return e.value.kind


def _rec(eid, hyp, role="researcher", rung=None, **kw):
    r = {"experiment_id": eid, "hypothesis": hyp, "prediction": "loss goes down", "config_hash": "c" * 8,
         "results": None, "delta_rci": None, "replication": None, "gpu_hours": None, "author_role": role,
         "rung": rung, "created_at": "2026-01-01T00:00:00Z", "closed_at": None, "supersedes": None}
    r.update(kw)
    return json.dumps(r)


def test_ledger_append_only_query_language_and_search(tmp_path):
    path = str(tmp_path / "ledger.jsonl")
    l = LG.Ledger(path)
    l.append(_rec("e1", "CHECK:muon Muon lr transfer holds across width", rung=1))
    l.append(_rec("e2", "PREREG:muon wider model keeps the optimum", role="engineer", rung=1))
    l.append(_rec("e3", "delta rule gates help long context", results={"passed": False}))
    l.append(_rec("e4", "fp8 matches bf16", replication={"status": "failed", "n": 3, "notes": None}))
    with pytest.raises(NativeError) as e:
        l.append(_rec("e1", "again"))
    assert _kind(e) == "Duplicate"
    with pytest.raises(NativeError) as e:
        l.append(_rec("e5", "x", supersedes="missing"))
    assert _kind(e) == "NotFound"
    l.append(_rec("e5", "fp8 matches bf16 after fix", supersedes="e4"))
    assert len(l) == 5 and json.loads(l.get("e2"))["author_role"] == "engineer"
    ids = lambda rows: [json.loads(r)["experiment_id"] for r in rows]
    assert ids(l.query("all")) == ["e1", "e2", "e3", "e4", "e5"]
    assert ids(l.query("rung=1 AND author_role=engineer")) == ["e2"]
    assert ids(l.query("kind=check")) == ["e1"] and ids(l.query("kind=prereg")) == ["e2"]
    assert ids(l.query('hypothesis~"fp8 matches" AND rung=none')) == ["e4", "e5"]
    for bad in ("SELECT * FROM records", "colour=red", 'hypothesis~"open', "rung=x", "a= AND "):
        with pytest.raises(NativeError):
            l.query(bad)
    hits = l.search_similar("does fp8 match bf16", 2)
    assert [h[0] for h in hits] == ["e4", "e5"] or [h[0] for h in hits] == ["e5", "e4"]
    assert hits[0][1] > 0.3 and l.search_similar("x", 0) == []
    assert ids(l.list_negatives()) == ["e3", "e4"]
    assert ids(LG.Ledger(path).query("*")) == ["e1", "e2", "e3", "e4", "e5"]      # durable


def test_lab_kernel_budgets_depth_jobs_fetch_and_promotion(tmp_path):
    mirror = tmp_path / "mirror"
    (mirror / "arxiv.org" / "abs").mkdir(parents=True)
    (mirror / "arxiv.org" / "abs" / "1234").write_bytes(b"paper")
    (tmp_path / "secret").write_bytes(b"no")
    k = K.Kernel(str(tmp_path / "ledger.jsonl"), str(mirror), str(tmp_path / "log"))
    root = k.spawn("director", "run the lab", K.Quota(1000, 100, 50), "prog")
    assert (root.id, root.depth, root.parent) == ("a-1", 0, None)
    text = (tmp_path / "log" / "agents" / "a-1" / "instructions.txt").read_text()
    assert text.startswith(K.KERNEL_INVARIANT) and text.endswith("run the lab")
    child = k.spawn("researcher", "x", K.Quota(400, 40, 10), "prog", root.id)
    assert child.depth == 1 and k.remaining(root.id).tokens == 600
    with pytest.raises(NativeError) as e:
        k.spawn("researcher", "x", K.Quota(700, 0, 0), "prog", root.id)
    assert _kind(e) == "QuotaRefused"
    a = child
    for _ in range(2):
        a = k.spawn("subagent", "x", K.Quota(0, 0, 0), "prog", a.id)
    assert a.depth == 3
    with pytest.raises(NativeError) as e:
        k.spawn("subagent", "x", K.Quota(0, 0, 0), "prog", a.id)
    assert _kind(e) == "SpawnDepth"
    with pytest.raises(NativeError) as e:
        k.spawn("overlord", "x", K.Quota(), "prog")
    assert _kind(e) == "RoleNotSpawnable"
    empty = k.spawn("engineer", "x", K.Quota(), "prog")
    with pytest.raises(NativeError) as e:
        k.submit_job(empty.id, 0, [], K.Quota(1, 0, 0))
    assert _kind(e) == "BudgetExhausted"
    # mailboxes
    mid = k.send(root.id, child.id, "hello", 5)
    msg = k.recv(child.id)
    assert (msg.id, msg.sender, msg.body, msg.created_ms) == (mid, root.id, "hello", 5) and k.recv(child.id) is None
    with pytest.raises(NativeError) as e:
        k.send(root.id, "a-99", "x", 1)
    assert _kind(e) == "AgentNotFound"
    # rung > 0 needs CHECK + PREREG rows for the job's first tag
    assert k.submit_job(child.id, 0, [], K.Quota(10, 0, 0)) == "j-1"
    with pytest.raises(NativeError) as e:
        k.submit_job(child.id, 2, ["muon"], K.Quota(10, 0, 0))
    assert _kind(e) == "RungNotCleared"
    k.ledger_append(_rec("e1", "CHECK:muon sanity"))
    k.ledger_append(_rec("e2", "PREREG:muon prediction"))
    assert k.submit_job(child.id, 2, ["muon"], K.Quota(10, 0, 0)) == "j-2"
    assert k.remaining(child.id).tokens == 380
    assert len(k.ledger_query("kind=check")) == 1
    # fetch: mirror hosts only, no traversal
    assert k.fetch("https://arxiv.org/abs/1234?v=2") == b"paper"
    for url in ("http://arxiv.org/abs/1234", "https://evil.example/abs/1234", "https://arxiv.org/../secret",
                "https://arxiv.org/abs/none"):
        with pytest.raises(NativeError) as e:
            k.fetch(url)
        assert _kind(e) == "NotMirrored"
    assert K.is_mirror_url("https://GitHub.com:443/x") and not K.is_mirror_url("https://github.com.evil/x")
    # genome patch: smoke -> gate -> canary 24 h -> rolled out / reverted
    p = k.propose_patch(child.id, "good diff", "why", "genome")
    assert [k.promote_genome(p, 0), k.promote_genome(p, 1), k.promote_genome(p, 2)] == \
        ["smoke_passed", "gate_passed", "canary"]
    assert k.promote_genome(p, 2 + K.CANARY_MS - 1) == "canary"
    assert k.promote_genome(p, 2 + K.CANARY_MS) == "rolled_out"
    bad = k.propose_patch(child.id, "FAIL_GATE", "why", "genome")
    assert [k.promote_genome(bad, 0), k.promote_genome(bad, 1)] == ["smoke_passed", "refused"]
    with pytest.raises(NativeError) as e:
        k.promote_genome(bad, 2)
    assert _kind(e) == "PromoteRefused"
    rev = k.propose_patch(child.id, "FAIL_CANARY", "why", "recipe")
    for t in (0, 1, 2):
        k.promote_genome(rev, t)
    assert k.promote_genome(rev, 2 + K.CANARY_MS) == "reverted"
    # weights need two distinct human signatures
    with pytest.raises(NativeError) as e:
        k.promote_weights("ckpt-1", [("alice", b"s"), ("alice", b"t"), ("bob", b"")])
    assert _kind(e) == "NoQuorum"
    assert k.promote_weights("ckpt-1", [("alice", b"s"), ("bob", b"t")]) == "serving"
    assert k.promote_weights("ckpt-FAIL_EVALS", []) == "refused"
    t = k.escalate(child.id, "grader looks wrong", "evidence")
    assert k.ticket(t) == ("grader looks wrong", "evidence", child.id)
    # agents and the id counter survive a restart
    k2 = K.Kernel(str(tmp_path / "ledger.jsonl"), str(mirror), str(tmp_path / "log"))
    assert k2.remaining(child.id).tokens == 380
    assert k2.spawn("reviewer", "x", K.Quota(), "prog").id == "a-" + str(int(empty.id[2:]) + 1)


def _suite(root, suite, items, written, compute=7):
    d = root / suite / "pending"
    d.mkdir(parents=True, exist_ok=True)
    (d / "items.jsonl").write_text("".join(json.dumps(i) + "\n" for i in items))
    (d / "meta.json").write_text(json.dumps({"written_ms": written, "compute_ms": compute}))


def test_eval_gate_scores_only_and_rotation(tmp_path):
    root = tmp_path / "suites"
    root.mkdir()
    g = EG.EvalGate(str(root), "h1")
    items = [{"id": "b", "prompt": "2+2", "answer": "4", "weight_milli": 600},
             {"id": "a", "prompt": "cap of fr", "answer": "paris", "weight_milli": 400}]
    for s, kind in (("aime", "NotHeldOut"), ("nope", "UnknownSuite")):
        with pytest.raises(NativeError) as e:
            g.suite_hash(s)
        assert _kind(e) == kind
    with pytest.raises(NativeError) as e:
        g.rotate("re_bench", 10, 100)
    assert _kind(e) == "RotationRefused"
    _suite(root, "re_bench", items, written=50)
    with pytest.raises(NativeError):
        g.rotate("re_bench", 60, 100)            # items must postdate the cutoff
    with pytest.raises(NativeError):
        g.rotate("re_bench", 200, 100)           # cutoff in the future
    h = g.rotate("re_bench", 40, 100)
    canon = "".join(json.dumps(i, sort_keys=True, separators=(",", ":")) + "\n"
                    for i in sorted(items, key=lambda i: i["id"]))
    assert h == hashlib.sha256(canon.encode()).hexdigest() == g.suite_hash("re_bench")
    assert not (root / "re_bench" / "pending").exists()
    (root / "subjects" / "checkpoint").mkdir(parents=True)
    (root / "subjects" / "checkpoint" / "ck1.json").write_text(json.dumps({"a": "paris", "b": "5"}))
    s = g.request("checkpoint", "ck1", "re_bench")
    assert (s.rci_milli, s.n_items, s.compute_ms, s.harness_version, s.suite_hash) == (400, 2, 7, "h1", h)
    assert not any(hasattr(s, f) for f in ("items", "prompt", "answer"))
    for subj in ("../ck1", "missing", ""):
        with pytest.raises(NativeError) as e:
            g.request("checkpoint", subj, "re_bench")
        assert _kind(e) == "SubjectNotFound"
    # rotation only every 90 days; the retired generation goes to history
    _suite(root, "re_bench", items[:1], written=EG.ROTATION_MS)
    with pytest.raises(NativeError) as e:
        g.rotate("re_bench", 100, 100 + EG.ROTATION_MS - 1)
    assert _kind(e) == "RotationRefused"
    h2 = g.rotate("re_bench", 100, 100 + EG.ROTATION_MS)
    assert h2 != h and json.loads((root / "re_bench" / "history.jsonl").read_text())["suite_hash"] == h
    assert g.request("checkpoint", "ck1", "re_bench").rci_milli == 0
    assert EG.is_held_out_suite("speedrun") and not EG.is_held_out_suite("gpqa")


def test_monitors_trip_freeze_and_persist(tmp_path):
    path = str(tmp_path / "state" / "freeze.json")
    m = MON.Monitors(path, {"g1": "aa"})
    m.note_grader_hash("g1", "aa", 1)
    assert not m.frozen()
    with pytest.raises(NativeError) as e:
        m.note_grader_hash("g1", "bb", 2)
    assert _kind(e) == "GraderHashMismatch" and m.frozen()
    with pytest.raises(NativeError) as e:
        m.note_held_out_access("a-3", 3)
    assert _kind(e) == "HeldOutAccess"
    snap = m.snapshot()
    assert snap["frozen_at"] == 2 and snap["reason"] == "grader hash mismatch"
    assert [v["boundary"] for v in snap["violations"]] == ["graders", "held_out"]
    with pytest.raises(NativeError) as e:
        m.kill("manual", 4)
    assert _kind(e) == "AlreadyFrozen"
    again = MON.Monitors(path, {})
    assert again.frozen() and len(again.snapshot()["violations"]) == 2
    with pytest.raises(NativeError) as e:
        again.plant("nowhere", "x", 5)
    assert _kind(e) == "UnknownBoundary"
    fresh = MON.Monitors(str(tmp_path / "f2.json"))
    fresh.kill("operator", 9)
    assert fresh.snapshot()["reason"] == "operator"
    for fn, kind in ((fresh.note_kernel_escape, "Message"), (fresh.note_self_check, "MonitorSelfCheck")):
        with pytest.raises(NativeError) as e:
            fn("x", 10)
        assert _kind(e) == kind
    assert MON.BOUNDARIES == ["kernel", "graders", "held_out", "monitors"]
