"""Behaviour lists of the lease queue and the content-addressed store (C++ ``native.leases`` and
``native.cas``; reference harness/leases/tests/*.rs and harness/cas/tests/*.rs): FIFO claims,
lease expiry and attempts, what a zombie worker may not do, terminal states, conditional
claims, replay; replication, pins, garbage collection, corrupt and lost replicas. Each ends
with random operations checked against a dictionary model, before and after a reopen."""
import hashlib
import json
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

L, C = native.leases, native.cas
TTL = 30_000


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


# ------------------------------------------------------------------------------ lease queue
def queue(tmp_path, name="q", **cfg):
    return L.Queue.create(str(tmp_path / name), L.QueueConfig(**cfg) if cfg else L.QueueConfig())


def test_queue_directory_and_defaults(tmp_path):
    assert L.DEFAULT_HEARTBEAT_PERIOD_MS * L.MISSED_HEARTBEATS == L.QueueConfig().lease_ttl_ms() == TTL
    q = queue(tmp_path)
    assert q.dir == str(tmp_path / "q") and q.log_len() == 0 and q.queued_ids() == [] and q.claim("w", 0) is None and q.get("x") is None
    err(lambda: queue(tmp_path))
    (tmp_path / "file").write_text("x")
    err(lambda: L.Queue.create(str(tmp_path / "file")))
    err(lambda: L.Queue.open(str(tmp_path / "missing")))
    assert L.Queue.open(str(tmp_path / "q")).queued_ids() == []
    for i, garbage in enumerate(("not json\n", '{"type": "task.enqueued"}\n')):                              # a complete line that is not an event
        d = tmp_path / f"bad{i}"
        queue(tmp_path, d.name).enqueue("a", "{}", 0)
        (d / "log" / "events.jsonl").write_text(garbage)
        err(lambda: L.Queue.open(str(d)))
    torn = queue(tmp_path, "torn")
    torn.enqueue("a", "{}", 0)
    with open(tmp_path / "torn" / "log" / "events.jsonl", "a") as f:
        f.write('{"type": "task.claim')                                                                    # a torn last line is dropped
    again = L.Queue.open(str(tmp_path / "torn"))
    assert again.queued_ids() == ["a"] and again.claim("w", 1).attempt == 1


def test_claims_are_fifo_with_attempt_numbers_and_expiry(tmp_path):
    q = queue(tmp_path)
    for i, t in enumerate("abc"):
        q.enqueue(t, json.dumps({"n": i}), i)
    t = q.get("a")
    assert (t.state, t.attempt, t.worker_id, json.loads(t.payload_json)) == ("Queued", 0, None, {"n": 0})
    assert err(lambda: q.enqueue("a", "{}", 9)).kind == "Duplicate"
    leases = [q.claim("w1", 100 + i) for i in range(3)]
    assert [(x.task_id, x.attempt, x.expires_at) for x in leases] == [("a", 1, 100 + TTL), ("b", 1, 101 + TTL), ("c", 1, 102 + TTL)]
    assert q.claim("w2", 200) is None and err(lambda: q.enqueue("b", "{}", 9)).kind == "Duplicate"       # leased ids stay taken
    assert q.event_types() == ["task.enqueued"] * 3 + ["task.claimed"] * 3


def test_heartbeats_extend_and_only_the_holder_of_the_current_attempt_may_send_them(tmp_path):
    q = queue(tmp_path)
    q.enqueue("a", "{}", 0)
    q.claim("w1", 0)
    assert q.heartbeat("a", "w1", 1, 10_000).expires_at == 10_000 + TTL
    assert err(lambda: q.heartbeat("a", "w2", 1, 10_001)).kind == "NotHolder"
    assert err(lambda: q.heartbeat("a", "w1", 2, 10_001)).kind == "StaleAttempt"
    assert err(lambda: q.heartbeat("nope", "w1", 1, 10_001)).kind == "NotFound"
    assert q.expire_due(10_000 + TTL - 1) == [] and q.get("a").state == "Leased"                          # before the deadline nothing moves
    assert q.event_types()[-1] == "task.heartbeat"


def test_expired_leases_requeue_behind_the_queue_and_zombies_are_refused(tmp_path):
    q = queue(tmp_path)
    for t in "ab":
        q.enqueue(t, "{}", 0)
    q.claim("w1", 0)
    q.enqueue("c", "{}", 1)
    assert q.expire_due(TTL) == ["a"] and q.queued_ids() == ["b", "c", "a"]
    assert [q.claim("w2", TTL + 1).task_id for _ in range(2)] == ["b", "c"]
    again = q.claim("w1", TTL + 2)                                                                         # the same worker may reclaim
    assert (again.task_id, again.attempt) == ("a", 2) and L.Queue.checkpoint_branch("a", 2) == "task/a/attempt/2"
    assert err(lambda: q.heartbeat("a", "w1", 1, TTL + 3)).kind == "StaleAttempt"
    assert err(lambda: q.complete("a", "w1", 1, b"late", TTL + 3)).kind == "StaleAttempt"
    assert q.get_output("a", 1) is None                                                                    # a refused completion writes nothing
    q.complete("a", "w1", 2, b"fresh", TTL + 4)
    assert q.get_output("a", 2) == b"fresh" and q.get("a").output_hash == hashlib.sha256(b"fresh").hexdigest()
    implicit = queue(tmp_path, "q2")
    implicit.enqueue("x", "{}", 0)
    implicit.claim("w1", 0)
    got = implicit.claim("w2", TTL)                                                                        # a claim expires due leases first
    assert (got.task_id, got.attempt) == ("x", 2) and implicit.event_types()[-2:] == ["task.expired", "task.claimed"]


def test_completed_and_failed_are_terminal(tmp_path):
    q = queue(tmp_path)
    for t in "ab":
        q.enqueue(t, "{}", 0)
    q.claim("w", 0)
    q.claim("w", 0)
    assert err(lambda: q.complete("a", "other", 1, b"x", 1)).kind == "NotHolder"
    assert err(lambda: q.complete("zz", "w", 1, b"x", 1)).kind == "NotFound"
    q.complete("a", "w", 1, b"", 1)
    assert q.get("a").output_hash == hashlib.sha256(b"").hexdigest() and q.get_output("a", 1) == b""
    err(lambda: q.complete("a", "w", 1, b"again", 2))
    assert err(lambda: q.fail("b", "w", 9, "why", 2)).kind == "StaleAttempt" and err(lambda: q.fail("zz", "w", 1, "why", 2)).kind == "NotFound"
    q.fail("b", "w", 1, "boom", 3)
    assert (q.get("a").state, q.get("b").state) == ("Completed", "Failed") and q.queued_ids() == [] and q.expire_due(10 ** 9) == []
    for t in "ab":
        assert err(lambda: q.enqueue(t, "{}", 4)).kind == "Duplicate"                                      # finished ids are not reusable
    assert q.event_types()[-3:] == ["task.output", "task.completed", "task.failed"]
    assert err(lambda: q.get_output("zz", 1)).kind == "NotFound" and q.get_output("b", 1) is None


def test_conditional_claims_skip_without_reordering(tmp_path):
    q = queue(tmp_path)
    for i, gpus in enumerate((0, 4, 0, 8)):
        q.enqueue(f"t{i}", json.dumps({"gpus": gpus}), i)
    needs = lambda n: (lambda t: json.loads(t.payload_json)["gpus"] == n)
    assert q.claim_if("w", 10, lambda t: False) is None and q.queued_ids() == ["t0", "t1", "t2", "t3"]
    before = q.log_len()
    assert q.claim_if("w", 10, needs(8)).task_id == "t3" and q.log_len() == before + 1                     # skipped tasks leave no events
    assert q.claim_if("w", 11, needs(0)).task_id == "t0" and q.queued_ids() == ["t1", "t2"]
    assert q.claim("w", 12).task_id == "t1"                                                                # plain claims still see FIFO order
    assert q.claim_if("w", 13, needs(8)) is None                                                           # a held lease is not claimable
    assert q.claim_if("w2", 10 + TTL, lambda t: t.id == "t3").attempt == 2                                 # expiry runs before matching
    empty = queue(tmp_path, "e")
    assert empty.claim_if("w", 0, lambda t: True) is None


def _model_step(rng, q, m, now):
    """One random operation on the queue ``q`` and the model ``m`` (id -> dict); returns nothing,
    asserts the same answers."""
    op = rng.choice(["enqueue", "claim", "heartbeat", "complete", "fail", "expire"])
    ids = list(m["tasks"])
    if op == "enqueue":
        tid = f"t{rng.randint(0, 12)}"
        if tid in m["tasks"]:
            assert err(lambda: q.enqueue(tid, "{}", now)).kind == "Duplicate"
        else:
            q.enqueue(tid, "{}", now)
            m["tasks"][tid] = dict(state="Queued", attempt=0, worker=None, exp=None)
            m["order"].append(tid)
        return
    def expire():                                                                                          # in the order the tasks were first enqueued
        due = [t for t in m["tasks"] if m["tasks"][t]["state"] == "Leased" and m["tasks"][t]["exp"] <= now]
        for t in due:
            m["tasks"][t].update(state="Queued", worker=None, exp=None)
            m["order"].append(t)
        return due
    if op == "expire":
        assert q.expire_due(now) == expire()
    elif op == "claim":
        expire()
        w = rng.choice(["w1", "w2"])
        got = q.claim(w, now)
        if not m["order"]:
            assert got is None
        else:
            tid = m["order"].pop(0)
            t = m["tasks"][tid]
            t.update(state="Leased", attempt=t["attempt"] + 1, worker=w, exp=now + TTL)
            assert (got.task_id, got.attempt, got.expires_at) == (tid, t["attempt"], t["exp"])
    elif ids:
        tid, w = rng.choice(ids), rng.choice(["w1", "w2"])
        t = m["tasks"][tid]
        att = t["attempt"] if rng.random() < 0.8 else t["attempt"] + 1
        ok = t["state"] == "Leased" and t["worker"] == w and att == t["attempt"]
        call = {"heartbeat": lambda: q.heartbeat(tid, w, att, now), "complete": lambda: q.complete(tid, w, att, tid.encode(), now),
                "fail": lambda: q.fail(tid, w, att, "r", now)}[op]
        if ok:
            call()
            if op == "heartbeat":
                t["exp"] = now + TTL
            else:
                t.update(state="Completed" if op == "complete" else "Failed", exp=None)
        else:
            err(call)


@pytest.mark.parametrize("seed", range(6))
def test_random_operations_match_a_dictionary_model_across_a_reopen(tmp_path, seed):
    rng = random.Random(seed)
    q = queue(tmp_path)
    m = dict(tasks={}, order=[])
    now = 0
    for step in range(150):
        now += rng.choice([1, 10, 5_000, 20_000])
        _model_step(rng, q, m, now)
        if step % 50 == 49:
            q = L.Queue.open(str(tmp_path / "q"))
        assert q.queued_ids() == m["order"]
        for tid, t in m["tasks"].items():
            got = q.get(tid)
            assert (got.state, got.attempt) == (t["state"], t["attempt"]) and (got.worker_id if t["state"] == "Leased" else None) == (t["worker"] if t["state"] == "Leased" else None)
            if t["state"] == "Completed":
                assert q.get_output(tid, t["attempt"]) == tid.encode()


# ------------------------------------------------------------------------------ content-addressed store
def store(tmp_path, n=3, name="s", min_replicas=2):
    backs = []
    for i in range(n):
        b = tmp_path / f"{name}-b{i}"
        b.mkdir(exist_ok=True)
        backs.append(str(b))
    return C.Store.create(str(tmp_path / name), backs, min_replicas), backs


def test_store_creation_rules(tmp_path):
    assert C.MIN_REPLICAS == 2
    for n in (0, 1):
        e = err(lambda: C.Store.create(str(tmp_path / f"few{n}"), [str(tmp_path)] * n))
        assert e.kind == "TooFewBackends" and not (tmp_path / f"few{n}").exists()
    assert err(lambda: C.Store.create(str(tmp_path / "three"), [str(tmp_path)] * 2, 3)).kind == "TooFewBackends"
    s, backs = store(tmp_path)
    assert s.event_types() == [] and s.pins == {}
    err(lambda: C.Store.create(str(tmp_path / "s"), backs))
    (tmp_path / "file").write_text("x")
    err(lambda: C.Store.create(str(tmp_path / "file"), backs))
    err(lambda: C.Store.open(str(tmp_path / "missing"), backs))
    assert err(lambda: C.Store.open(str(tmp_path / "s"), backs[:1])).kind == "TooFewBackends"
    assert C.Store.open(str(tmp_path / "s"), backs).pins == {}
    (tmp_path / "s" / "log" / "events.jsonl").write_text("garbage\n")
    err(lambda: C.Store.open(str(tmp_path / "s"), backs))


def test_digests_and_replication(tmp_path):
    s, backs = store(tmp_path)
    assert s.put(b"") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert s.put(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    big = bytes(range(256)) * 4096
    d = s.put(big)
    assert d == hashlib.sha256(big).hexdigest() == d.lower() and s.get(d) == big and s.replica_count(d) == 3
    assert s.put(big) == d and s.replica_count(d) == 3                                                     # the same bytes again: same digest
    assert err(lambda: s.get("0" * 64)).kind == "NotFound" and s.replica_count("0" * 64) == 0
    two, _ = store(tmp_path, 2, "two")
    assert two.replica_count(two.put(b"x")) == 2


def test_pins_and_garbage_collection(tmp_path):
    s, backs = store(tmp_path)
    d1, d2, d3 = s.put(b"one"), s.put(b"two!"), s.put(b"")
    s.pin(d1, "a")
    s.pin(d1, "b")                                                                                         # two names, one blob
    assert err(lambda: s.pin(d2, "a")).kind == "DuplicatePin" and err(lambda: s.pin("f" * 64, "c")).kind == "NotFound"
    assert err(lambda: s.unpin("nobody")).kind == "NotFound"
    before = s.event_types()
    rep = s.gc()
    assert (rep.blobs_removed, rep.bytes_freed) == (2, 3 * 4) and s.get(d1) == b"one" and s.replica_count(d2) == 0    # the empty blob counts; bytes are summed over replicas
    assert s.event_types() == before + ["cas.gc"]
    s.unpin("a")
    assert s.gc().blobs_removed == 0 and s.get(d1) == b"one"                                               # still pinned under "b"
    s.unpin("b")
    assert s.gc().blobs_removed == 1 and err(lambda: s.get(d1)).kind == "NotFound"
    s.pin(s.put(b"new"), "a")                                                                              # a freed name can be used again
    assert s.event_types()[:5] == ["cas.put", "cas.put", "cas.put", "cas.pin", "cas.pin"]
    nothing = s.gc()
    assert nothing.blobs_removed == 0 and s.event_types()[-1] != "cas.gc" or nothing.blobs_removed == 0     # an empty sweep is not news


def test_corrupt_and_lost_replicas(tmp_path):
    s, backs = store(tmp_path)
    d = s.put(b"payload")
    s.pin(d, "keep")
    (tmp_path / "s-b0" / d).write_bytes(b"flipped")
    assert s.get(d) == b"payload"                                                                          # never the wrong bytes
    (tmp_path / "s-b1" / d).unlink()
    assert s.get(d) == b"payload" and s.replica_count(d) in (1, 2)
    (tmp_path / "s-b2" / d).write_bytes(b"also bad")
    assert err(lambda: s.get(d)).kind == "DigestMismatch"
    for b in backs:
        p = tmp_path / b.split("/")[-1] / d
        if p.exists():
            p.unlink()
    assert err(lambda: s.get(d)).kind == "NotFound"
    fresh, fb = store(tmp_path, 3, "f")
    d2 = fresh.put(b"x")
    fresh.pin(d2, "p")
    import shutil

    shutil.rmtree(fb[0])                                                                                   # a whole backend disappears
    again = C.Store.open(str(tmp_path / "f"), fb)
    assert again.get(d2) == b"x" and again.pins == {"p": d2}


def test_writes_need_two_live_backends(tmp_path):
    good = tmp_path / "g"
    good.mkdir()
    lone = C.Store.create(str(tmp_path / "lone"), [str(good), str(tmp_path / "absent")])
    assert err(lambda: lone.put(b"x")).kind == "UnderReplicated"
    assert lone.gc().blobs_removed in (0, 1)                                                               # what the failed put left behind is swept
    assert list(good.iterdir()) == []
    ok = C.Store.create(str(tmp_path / "ok"), [str(good), str(tmp_path / "absent"), str(tmp_path)])
    assert ok.replica_count(ok.put(b"y")) == 2                                                             # two of three is enough


@pytest.mark.parametrize("seed", range(5))
def test_random_store_operations_match_a_model_across_a_reopen(tmp_path, seed):
    rng = random.Random(seed)
    s, backs = store(tmp_path)
    blobs, pins = {}, {}
    for step in range(120):
        op = rng.choice(["put", "put", "pin", "unpin", "gc", "get"])
        if op == "put":
            data = bytes([rng.randint(0, 5)]) * rng.randint(0, 4)
            d = s.put(data)
            assert d == hashlib.sha256(data).hexdigest()
            blobs[d] = data
        elif op == "pin":
            name = f"n{rng.randint(0, 4)}"
            d = rng.choice(sorted(blobs) + ["a" * 64])
            if d not in blobs:                                                                             # the blob is looked up before the name
                assert err(lambda: s.pin(d, name)).kind == "NotFound"
            elif name in pins:
                assert err(lambda: s.pin(d, name)).kind == "DuplicatePin"
            else:
                s.pin(d, name)
                pins[name] = d
        elif op == "unpin":
            name = f"n{rng.randint(0, 4)}"
            if name in pins:
                s.unpin(name)
                del pins[name]
            else:
                assert err(lambda: s.unpin(name)).kind == "NotFound"
        elif op == "gc":
            dead = [d for d in blobs if d not in pins.values()]
            rep = s.gc()
            assert rep.blobs_removed == len(dead) and rep.bytes_freed == 3 * sum(len(blobs[d]) for d in dead)
            for d in dead:
                del blobs[d]
        else:
            for d, data in blobs.items():
                assert s.get(d) == data
        if step % 40 == 39:
            s = C.Store.open(str(tmp_path / "s"), backs)
        assert s.pins == pins
