"""Lease queue, CAS, mesh and pipeline (C++), against the contracts of the reference's
harness/leases, harness/cas, harness/mesh and harness/pipeline crates."""
import json

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

L, C, MESH, P = native.leases, native.cas, native.mesh, native.pipeline


def _kind(exc):
    return exc.value.kind


# ----------------------------------------------------------------------------- leases
def test_queue_fifo_lease_heartbeat_expiry_and_replay(tmp_path):
    d = str(tmp_path / "q")
    q = L.Queue.create(d)
    with pytest.raises(NativeError):
        L.Queue.create(d)
    q.enqueue("a", json.dumps({"x": 1}), 10)
    q.enqueue("b", "{}", 11)
    with pytest.raises(NativeError) as e:
        q.enqueue("a", "{}", 12)
    assert _kind(e) == "Duplicate"
    lease = q.claim("w1", 100)
    assert (lease.task_id, lease.attempt, lease.expires_at) == ("a", 1, 100 + 30_000)
    assert q.get("a").state == "Leased" and q.get("a").worker_id == "w1"
    hb = q.heartbeat("a", "w1", 1, 20_000)
    assert hb.expires_at == 50_000
    with pytest.raises(NativeError) as e:
        q.heartbeat("a", "w2", 1, 20_001)
    assert _kind(e) == "NotHolder"
    with pytest.raises(NativeError) as e:
        q.heartbeat("a", "w1", 7, 20_001)
    assert _kind(e) == "StaleAttempt"
    # deadline passes: the task goes to the back of the queue, the next claim is attempt 2
    assert q.expire_due(50_000) == ["a"]
    assert q.queued_ids() == ["b", "a"]
    l2 = q.claim("w2", 50_001)
    assert l2.task_id == "b"
    l3 = q.claim("w2", 50_002)
    assert (l3.task_id, l3.attempt) == ("a", 2)
    # the zombie of attempt 1 can do nothing
    with pytest.raises(NativeError) as e:
        q.complete("a", "w1", 1, b"stale", 50_003)
    assert _kind(e) == "StaleAttempt"
    q.complete("a", "w2", 2, b"result", 50_004)
    q.fail("b", "w2", 1, "boom", 50_005)
    assert q.get_output("a", 2) == b"result" and q.get_output("a", 1) is None
    assert q.get("a").state == "Completed" and q.get("b").state == "Failed"
    assert q.claim("w3", 60_000) is None
    assert L.Queue.checkpoint_branch("a", 2) == "task/a/attempt/2"
    types = q.event_types()
    assert types[:3] == ["task.enqueued", "task.enqueued", "task.claimed"]
    assert types[-3:] == ["task.output", "task.completed", "task.failed"]
    # replay rebuilds the same tables
    r = L.Queue.open(d)
    assert r.get("a").state == "Completed" and r.get("a").attempt == 2
    assert r.get("a").output_hash == q.get("a").output_hash and r.queued_ids() == []
    with pytest.raises(NativeError) as e:
        r.get_output("nope", 1)
    assert _kind(e) == "NotFound"


def test_claim_if_skips_without_events_and_ttl_config(tmp_path):
    q = L.Queue.create(str(tmp_path / "q"), L.QueueConfig(1000, 0))
    assert L.QueueConfig(1000, 0).lease_ttl_ms() == 1000          # max(missed, 1)
    q.enqueue("cpu", json.dumps({"requires": {"gpus": 0}}), 0)
    q.enqueue("gpu", json.dumps({"requires": {"gpus": 4}}), 0)
    n = q.log_len()
    lease = q.claim_if("w", 5, lambda t: json.loads(t.payload_json)["requires"]["gpus"] == 4)
    assert lease.task_id == "gpu" and lease.expires_at == 1005
    assert q.log_len() == n + 1 and q.queued_ids() == ["cpu"]
    assert q.claim_if("w", 6, lambda t: False) is None and q.log_len() == n + 1


# -------------------------------------------------------------------------------- cas
def test_cas_replication_pins_gc_and_corruption(tmp_path):
    backs = [str(tmp_path / f"b{i}") for i in range(3)]
    for b in backs:
        (tmp_path / b.split("/")[-1]).mkdir()
    with pytest.raises(NativeError) as e:
        C.Store.create(str(tmp_path / "s0"), backs[:1])
    assert _kind(e) == "TooFewBackends"
    s = C.Store.create(str(tmp_path / "s"), backs)
    d1, d2 = s.put(b"hello"), s.put(b"world")
    assert len(d1) == 64 and s.replica_count(d1) == 3 and s.get(d1) == b"hello"
    s.pin(d1, "kernel.current")
    with pytest.raises(NativeError) as e:
        s.pin(d2, "kernel.current")
    assert _kind(e) == "DuplicatePin"
    with pytest.raises(NativeError) as e:
        s.pin("0" * 64, "x")
    assert _kind(e) == "NotFound"
    rep = s.gc()
    assert rep.blobs_removed == 1 and rep.bytes_freed == 15 and s.replica_count(d2) == 0
    # one bad replica is skipped, only bad replicas -> DigestMismatch, none -> NotFound
    (tmp_path / "b0" / d1).write_bytes(b"garbage")
    assert s.get(d1) == b"hello"
    for i in (1, 2):
        (tmp_path / f"b{i}" / d1).write_bytes(b"junk")
    with pytest.raises(NativeError) as e:
        s.get(d1)
    assert _kind(e) == "DigestMismatch"
    with pytest.raises(NativeError) as e:
        s.get(d2)
    assert _kind(e) == "NotFound"
    # pins are replayed from the log
    again = C.Store.open(str(tmp_path / "s"), backs)
    assert again.pins == {"kernel.current": d1}
    again.unpin("kernel.current")
    assert C.Store.open(str(tmp_path / "s"), backs).pins == {}
    assert again.event_types() == ["cas.put", "cas.put", "cas.pin", "cas.gc", "cas.unpin"]
    # a put that reaches fewer than two backends fails
    lone = C.Store.create(str(tmp_path / "s2"), [backs[0], str(tmp_path / "missing")])
    with pytest.raises(NativeError) as e:
        lone.put(b"x")
    assert _kind(e) == "UnderReplicated"


# ------------------------------------------------------------------------------- mesh
def test_mesh_pull_by_capability_freeze_and_watch_ring(tmp_path):
    with pytest.raises(NativeError) as e:
        MESH.LocalMesh.start(2, str(tmp_path / "m2"))
    assert _kind(e) == "TooFewNodes"
    lm = MESH.LocalMesh.start(4, str(tmp_path / "m"))
    ring = [(w.watcher, w.watchee) for w in lm.get(0).watches]
    assert ring[:4] == [("1", "0"), ("2", "0"), ("2", "1"), ("3", "1")] and len(ring) == 8
    q = L.Queue.create(str(tmp_path / "q"))
    q.enqueue("big", json.dumps({"requires": {"gpus": 4, "providers": ["a"]}}), 0)
    q.enqueue("small", json.dumps({"requires": {"cpus": 1}}), 0)
    q.enqueue("any", "{}", 0)
    lm.get(0).advertise(MESH.Capabilities(gpus=1, cpus=8), 1)
    lm.get(1).advertise(MESH.Capabilities(gpus=8, cpus=8, providers=["a", "b"]), 1)
    assert lm.get(0).pull(q, 2).task_id == "small"      # FIFO among what fits
    assert lm.get(1).pull(q, 3).task_id == "big"
    assert lm.get(0).pull(q, 4).task_id == "any"
    assert lm.get(0).pull(q, 5) is None
    lm.tick(6)
    assert sorted(a.node for a in lm.get(3).adverts) == ["0", "1"]
    # freeze: bad signature refused; a partitioned node honours it after heal
    with pytest.raises(NativeError) as e:
        lm.get(0).freeze(MESH.Freeze("stop", "key-0", b"nope"))
    assert _kind(e) == "BadSignature"
    lm.partition([3])
    lm.get(0).freeze(MESH.Freeze("stop", "key-0", b"stop"))
    lm.tick(7)
    assert lm.get(1).is_frozen() and not lm.get(3).is_frozen()
    lm.heal()
    lm.tick(8)
    assert lm.get(3).is_frozen()
    with pytest.raises(NativeError) as e:
        lm.get(3).pull(q, 9)
    assert _kind(e) == "Frozen"
    # persisted across a restart; untrusted nodes cannot pull
    assert MESH.Mesh.open(str(tmp_path / "m" / "3"), "3", "key-3").is_frozen()
    guest = MESH.Mesh.create(str(tmp_path / "guest"), "g", "kg", False)
    with pytest.raises(NativeError) as e:
        guest.pull(q, 10)
    assert _kind(e) == "Untrusted"
    assert not MESH.caps_satisfy(MESH.Capabilities(kvm=False), json.dumps({"requires": {"kvm": True}}))
    assert not MESH.caps_satisfy(MESH.Capabilities(), json.dumps({"requires": 3}))


# --------------------------------------------------------------------------- pipeline
def test_pipeline_stub_must_fail_rounds_planted_patch_and_replay(tmp_path):
    d = str(tmp_path / "p")
    p = P.Pipeline.create(d, "kernels")
    with pytest.raises(NativeError) as e:
        p.start_implementers(0)
    assert _kind(e) == "StubNotFailed"
    assert p.start_oracle(1) == "oracle/kernels/0" and p.stage == "Oracle"
    with pytest.raises(NativeError) as e:
        p.record_oracle(True, 2)
    assert _kind(e) == "StubPassed" and p.stage == "Oracle"
    p.record_oracle(False, 3)
    assert p.stage == "StubMustFail" and p.stub_failed
    ids = p.start_implementers(4)
    assert ids == [f"implementer/kernels/0/{i}" for i in range(3)]
    bad = P.Candidate("0", "fast", b"diff PLANTED_BAD_PATCH here")
    ok = P.Candidate("1", "simple", b"diff good")
    with pytest.raises(NativeError) as e:
        p.submit_candidate(P.Candidate("9", "x", b""), 5)
    assert _kind(e) == "NoCandidate"
    p.submit_candidate(bad, 5)
    p.submit_candidate(ok, 6)
    p.submit_candidate(ok, 7)                      # resubmission: fresh task id
    assert p.queue().get("pipeline/kernels/0/submit_candidate/1#1") is not None
    v = P.review(p.candidates, [True, True])
    assert v.is_pick and v.candidate == "1"
    rej = P.review(p.candidates, [True, False])
    assert not rej.is_pick and rej.defects == ["candidate 0 is planted-bad", "candidate 1 tests failed"]
    with pytest.raises(NativeError) as e:
        P.merge_allowed(P.Verdict.pick("0"), p.candidates, [True, True])
    assert _kind(e) == "PlantedBad"
    with pytest.raises(NativeError) as e:
        P.merge_allowed(P.Verdict.pick("1"), p.candidates, [True, False])
    assert _kind(e) == "CandidateFailed"
    p.start_review(8)
    with pytest.raises(NativeError) as e:
        p.record_verdict(P.Verdict.pick("0"), 9)
    assert _kind(e) == "PlantedBad"
    assert p.record_verdict(P.Verdict.reject_all(["meh"]), 9) == "Implement" and p.round == 1
    assert p.candidates == []
    p.submit_candidate(P.Candidate("2", "third", b"ok"), 10)
    p.start_review(11)
    assert p.record_verdict(P.Verdict.pick("2"), 12) == "Merged"
    with pytest.raises(NativeError):
        p.record_merge("other", "15.2", "abc", 3, 0, [], 13)
    p.record_merge("kernels", "15.2", "abc123", 12, 0, ["fv-1"], 13)
    again = P.Pipeline.open(d, "kernels")
    assert again.stage == "Merged" and again.round == 1 and again.stub_failed
    assert [c.id for c in again.candidates] == ["2"] and again.candidates[0].patch == b"ok"
    # three rejected rounds block the module
    b = P.Pipeline.create(str(tmp_path / "b"), "m", 1, 2)
    b.start_oracle(0); b.record_oracle(False, 0); b.start_implementers(0)
    for _ in range(2):
        b.start_review(1)
        stage = b.record_verdict(P.Verdict.reject_all([]), 1)
    assert stage == "Blocked" and P.Pipeline.open(str(tmp_path / "b"), "m", 1, 2).stage == "Blocked"
    assert P.is_planted_bad(b"xxPLANTED_BAD_PATCHyy") and not P.is_planted_bad(b"PLANTED")
    tid, payload = P.work_payload("m", "oracle", json.dumps({"round": 2}))
    assert tid == "oracle/m/2" and json.loads(payload) == {"round": 2, "module": "m", "role": "oracle"}
