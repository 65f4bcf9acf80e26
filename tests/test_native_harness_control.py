"""Raft control plane, provider guards and release roll-out (C++), against the contracts of the
reference's harness/raft, harness/providers and harness/ops crates."""
import hashlib
import json

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

R, PV, O, C = native.raft, native.providers, native.ops, native.cas


def _kind(e):
    return e.value.kind


def test_raft_election_majority_partition_and_restart(tmp_path):
    with pytest.raises(NativeError) as e:
        R.LocalGroup.start(2, str(tmp_path / "g2"))
    assert _kind(e) == "TooFewVoters"
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    assert g.leader() == -1
    g.tick(0)
    lead = g.leader()
    assert lead == 0 and g.get(0).term == 1                 # ties go to the smallest id
    L = g.get(lead)
    with pytest.raises(NativeError) as e:
        g.get(1).set_kernel_version("x")
    assert _kind(e) == "NotLeader"
    L.set_kernel_version("1.0")
    assert all(g.get(i).state()["kernel_version"] == "1.0" for i in range(3))
    # workers never vote; ephemeral nodes cannot be voters; untrusted refused
    L.add_worker(R.NodeInfo("w1", "tcp://w1", always_on=False))
    with pytest.raises(NativeError) as e:
        L.add_voter(R.NodeInfo("w2", "", always_on=False))
    assert _kind(e) == "EphemeralVoter"
    with pytest.raises(NativeError) as e:
        L.add_voter(R.NodeInfo("v9", "", trusted=False))
    assert _kind(e) == "Untrusted"
    with pytest.raises(NativeError) as e:
        L.add_worker(R.NodeInfo("w1", "", always_on=False))
    assert _kind(e) == "Duplicate"
    with pytest.raises(NativeError) as e:
        L.remove_node("1")
    assert _kind(e) == "TooFewVoters"
    # role leases
    lease = L.claim_role("coordinator", "1", 1000)
    assert lease == {"role": "coordinator", "holder": "1", "attempt": 1, "expires_at": 31000}
    with pytest.raises(NativeError) as e:
        L.claim_role("coordinator", "2", 2000)
    assert _kind(e) == "NotClaimable"
    with pytest.raises(NativeError) as e:
        L.heartbeat_role("coordinator", "2", 2000)
    assert _kind(e) == "NotHolder"
    assert L.heartbeat_role("coordinator", "1", 5000)["expires_at"] == 35000
    assert L.expire_roles(34999) == [] and L.expire_roles(35000) == ["coordinator"]
    assert L.claim_role("coordinator", "2", 35001)["attempt"] == 2
    gen, blob = L.commit_token(b"refresh-1")
    assert (gen, blob) == (1, b"refresh-1") and L.commit_token(b"r2")[0] == 2
    # a minority leader cannot commit; the majority side elects a new leader with a higher term
    n_before = L.log_len
    g.partition([0])
    with pytest.raises(NativeError) as e:
        L.set_kernel_version("lost")
    assert _kind(e) == "NotLeader" and L.log_len == n_before
    g.tick(40000)
    new = g.leader()
    assert new == 1 and g.get(1).term == 2 and not g.get(0).is_leader()
    g.get(1).set_kernel_version("2.0")
    assert g.get(0).state()["kernel_version"] == "1.0"       # isolated: not replicated to
    g.heal()
    g.tick(40001)
    assert g.get(0).state()["kernel_version"] == "2.0" and g.get(0).term == 2
    # crash + restart: durable state comes back, node is a follower until it hears the leader
    g.crash(2)
    with pytest.raises(NativeError):
        g.get(2)
    g.get(1).set_kernel_version("2.1")
    g.restart(2)
    assert g.get(2).state()["kernel_version"] == "2.0" and not g.get(2).is_leader()
    g.tick(40002)
    assert g.get(2).state()["kernel_version"] == "2.1"
    st = g.get(2).state()
    assert [m.id for m in st["membership"]] == ["0", "1", "2", "w1"] and st["token"] == (2, b"r2")
    # bootstrap of a single node and reopen from disk
    one = R.Cluster.bootstrap(str(tmp_path / "solo"), R.NodeInfo("a", "x"))
    assert one.is_leader()
    one.set_kernel_version("k")
    again = R.Cluster.open(str(tmp_path / "solo"), "a")
    assert again.state()["kernel_version"] == "k" and not again.is_leader()


def test_provider_response_validation_aimd_failover_and_broker(tmp_path):
    ok = json.dumps({"choices": [{"finish_reason": "stop", "message": {"content": "hi"}}]}).encode()
    assert json.loads(PV.validate_response(ok))["choices"][0]["finish_reason"] == "stop"
    cases = {
        b"rate_limit": "RateLimitText", b"RATE_LIMIT": "RateLimitText",
        b'{"error": "Rate_Limit"}': "RateLimitText", b"not json": "MalformedJson", b"[1]": "MalformedJson",
        b'{"choices": []}': "EmptyCompletion", b"{}": "EmptyCompletion",
        json.dumps({"choices": [{"finish_reason": "length", "tool_calls": [
            {"function": {"name": "f", "arguments": '{"a": 1'}}]}]}).encode(): "TruncatedToolCall",
        json.dumps({"choices": [{"finish_reason": "length", "message": {"tool_calls": [
            {"function": {"name": "f"}}]}}]}).encode(): "TruncatedToolCall",
    }
    for body, kind in cases.items():
        with pytest.raises(NativeError) as e:
            PV.validate_response(body)
        assert _kind(e) == kind, body
    fine = json.dumps({"choices": [{"finish_reason": "length", "tool_calls": [
        {"function": {"name": "f", "arguments": '{"a": 1}'}}]}]}).encode()
    PV.validate_response(fine)
    a = PV.Aimd(PV.AimdConfig(min_window=2, max_window=5))
    assert a.window == 2
    for _ in range(5):
        a.on_success(10)
    assert a.window == 5
    a.on_success(30001)          # slow success shrinks like a 429
    assert a.window == 2
    a.on_success(1); a.on_outage()
    assert a.window == 2
    b = PV.Aimd(PV.AimdConfig(decrease=1.0, max_window=8))
    for _ in range(3):
        b.on_success(1)
    b.on_429()
    assert b.window == 3         # at least one step down
    f = PV.Failover(["p0", "p1"])
    assert f.current() == "p0" and f.wait_backoff_ms() == 100
    f.mark_down("p0")
    assert f.current() == "p1" and f.wait_backoff_ms() == 200
    f.mark_down("p1")
    with pytest.raises(NativeError) as e:
        f.current()
    assert _kind(e) == "NoProvider" and f.wait_backoff_ms() == 400
    f.mark_up("p0")
    assert f.current() == "p0"
    with pytest.raises(NativeError):
        f.mark_down("nope")
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    with pytest.raises(NativeError) as e:
        PV.broker_refresh(g.get(1), "anthropic", 60_000, b"blob", 5)
    assert _kind(e) == "NotBroker"
    (gen, blob), tok = PV.broker_refresh(g.get(0), "anthropic", 60_000, b"blob", 5)
    assert gen == 1 and tok.token == hashlib.sha256(b"blob").hexdigest() and tok.expires_at == 60_005
    assert g.get(2).state()["token"] == (1, b"blob")       # committed before the token was issued


def _release(version, artifact, signers):
    return O.Release(version, hashlib.sha256(artifact).hexdigest(), "c0ffee", signers)


def test_ops_rollout_quorum_shadow_promote_and_rollback(tmp_path):
    backs = []
    for i in range(2):
        (tmp_path / f"b{i}").mkdir()
        backs.append(str(tmp_path / f"b{i}"))
    store = C.Store.create(str(tmp_path / "cas"), backs)
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    lead = g.get(0)
    ops = O.Ops.create(str(tmp_path / "ops"))
    art = b"kernel-v1"
    weak = _release("1.0", art, [("alice", b"sig"), ("alice", b"sig2"), ("bob", b"")])
    assert not O.has_quorum(weak)
    with pytest.raises(NativeError) as e:
        ops.propose(weak, art, store, 1)
    assert _kind(e) == "NoQuorum" and ops.state.startswith("refused:need 2 human signatures, have 1")
    good = _release("1.0", art, [("alice", b"s"), ("bob", b"t")])
    with pytest.raises(NativeError) as e:
        ops.propose(good, b"tampered", store, 2)
    assert _kind(e) == "DigestMismatch"
    ops.propose(good, art, store, 3)
    assert ops.state == "proposed" and store.pins == {"kernel.shadow": good.digest}
    with pytest.raises(NativeError) as e:
        ops.apply_one("0", 4)
    assert _kind(e) == "WrongState"
    ops.start_shadow(store, 5)
    ops.shadow_pass(6)
    with pytest.raises(NativeError) as e:
        ops.apply_one("shadow", 7)
    assert _kind(e) == "WrongState"
    with pytest.raises(NativeError) as e:
        ops.promote(lead, store, 7)
    assert _kind(e) == "WrongState"
    for i, node in enumerate(("0", "1", "2")):
        ops.apply_one(node, 8 + i)
        assert ops.state == f"rolling:{node}"
    ops.promote(lead, store, 20)
    assert ops.state == "current" and lead.state()["kernel_version"] == "1.0"
    assert store.pins == {"kernel.current": good.digest}
    text = ops.cli(["status"], lead)
    assert text.splitlines()[:4] == ["kernel_version: 1.0", "state: current", "release: 1.0", "nodes:"]
    assert "  0 applied=1.0 healthy=true role=live" in text
    js = json.loads(ops.cli(["--json", "status"], lead))
    assert js["state"] == "current" and len(js["nodes"]) == 3
    with pytest.raises(NativeError):
        ops.cli(["frobnicate"], lead)
    # second release, an unhealthy node triggers the automatic rollback
    art2 = b"kernel-v2"
    r2 = _release("2.0", art2, [("alice", b"s"), ("carol", b"u")])
    ops.propose(r2, art2, store, 30)
    ops.start_shadow(store, 31)
    ops.shadow_pass(32)
    ops.apply_one("0", 33)
    ops.mark_unhealthy("0", "oom", lead, store, 34)
    assert ops.state == "rolled_back:oom" and lead.state()["kernel_version"] == "1.0"
    assert store.pins == {"kernel.current": good.digest}
    # promote v2, then roll back from current: previous digest becomes current again
    ops.propose(r2, art2, store, 40)
    ops.start_shadow(store, 41); ops.shadow_pass(42)
    for node in ("0", "1", "2"):
        ops.apply_one(node, 43)
    ops.promote(lead, store, 44)
    assert store.pins == {"kernel.current": r2.digest, "kernel.previous": good.digest}
    ops.rollback("regression", lead, store, 45)
    assert lead.state()["kernel_version"] == "1.0" and store.pins == {"kernel.current": good.digest}
    again = O.Ops.open(str(tmp_path / "ops"))
    assert again.state == "rolled_back:regression" and again.kernel_version == "1.0"
    assert again.event_types()[:3] == ["ops.refuse", "ops.propose", "ops.shadow"]
    # shadow failure
    ops.propose(r2, art2, store, 50)
    ops.start_shadow(store, 51)
    ops.shadow_fail("diverged", store, 52)
    assert ops.state == "rolled_back:diverged" and "kernel.shadow" not in store.pins


def test_harness_command_line(tmp_path, capsys):
    from prometheus_b200.native import harness

    assert harness.main([]) == 0 and "usage: harness" in capsys.readouterr().out
    assert harness.main(["frobnicate"]) == 1 and "unknown command" in capsys.readouterr().err
    assert harness.main(["status"]) == 1
    capsys.readouterr()
    args = ["--ops-dir", str(tmp_path / "ops"), "--raft-dir", str(tmp_path / "raft")]
    assert harness.main(["status"] + args) == 0
    text = capsys.readouterr().out
    assert text.startswith("kernel_version:") and "nodes:" in text
    assert harness.main(["--json", "status"] + args) == 0          # reopened from the same directories
    js = json.loads(capsys.readouterr().out)
    assert js["state"] == "idle" and len(js["nodes"]) == 3
