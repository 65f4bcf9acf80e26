"""Behaviour list of kernel releases (C++ ``native.ops``; reference
harness/ops/tests/{cli,create_open,properties,propose,quorum,replay,rollback,rollout,shadow,
status}.rs): what counts as a human quorum, a release that is refused never touches the
store or the running kernel, shadow before roll-out, one node at a time, promotion only when
every live node applied, automatic and manual rollback, replay from the log. The quorum
rule and the state machine are compared with Python models on random inputs."""
import hashlib
import json
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

O, C, R = native.ops, native.cas, native.raft
GOOD = [("alice", b"s"), ("bob", b"t")]


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    return e.value


def release(version, artifact, signers=GOOD, digest=None):
    return O.Release(version, digest or hashlib.sha256(artifact).hexdigest(), "c0ffee", signers)


@pytest.fixture
def world(tmp_path):
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    backs = []
    for i in range(2):
        (tmp_path / f"b{i}").mkdir()
        backs.append(str(tmp_path / f"b{i}"))
    return O.Ops.create(str(tmp_path / "ops")), C.Store.create(str(tmp_path / "cas"), backs), g.get(0), tmp_path


def fresh_store(tmp_path, name):
    backs = []
    for i in range(2):
        (tmp_path / f"{name}-b{i}").mkdir()
        backs.append(str(tmp_path / f"{name}-b{i}"))
    return C.Store.create(str(tmp_path / name), backs)


def ready(ops, store, version, artifact, t):
    rel = release(version, artifact)
    ops.propose(rel, artifact, store, t)
    ops.start_shadow(store, t + 1)
    ops.shadow_pass(t + 2)
    return rel


def to_current(ops, store, lead, version, artifact, t):
    rel = ready(ops, store, version, artifact, t)
    for n in ("0", "1", "2"):
        ops.apply_one(n, t + 3)
    ops.promote(lead, store, t + 4)
    return rel


# ------------------------------------------------------------------------------ quorum
def model_quorum(signers, quorum):
    return len({who for who, sig in signers if sig}) >= quorum


def test_quorum_rule():
    assert O.DEFAULT_QUORUM == 2 and (O.PIN_CURRENT, O.PIN_PREVIOUS, O.PIN_SHADOW) == ("kernel.current", "kernel.previous", "kernel.shadow")
    q = lambda signers, n=2: O.has_quorum(release("v", b"", signers), n)
    assert q(GOOD) and q(GOOD + [("carol", b"u")]) and not q([("alice", b"s")]) and not q([])
    assert not q([("alice", b"s"), ("alice", b"other")])                                       # one human signing twice is one human
    assert not q([("alice", b"s"), ("bob", b"")]) and not q([("alice", b""), ("bob", b"")])   # an empty signature is no signature
    assert q([("alice", b""), ("alice", b"s"), ("bob", b"t"), ("bob", b"")])
    assert q([], 0) and q(GOOD, 1) and not q(GOOD, 3) and q(GOOD + [("carol", b"u")], 3)
    rng = random.Random(0)
    for _ in range(300):
        signers = [(rng.choice(["a", "b", "c", "d"]), rng.choice([b"", b"x", b"y"])) for _ in range(rng.randint(0, 6))]
        n = rng.randint(0, 4)
        assert q(signers, n) == model_quorum(signers, n), (signers, n)


# ------------------------------------------------------------------------------ create / open
def test_create_and_open(tmp_path):
    ops = O.Ops.create(str(tmp_path / "ops"))
    assert ops.state == "idle" and ops.event_types() == [] and (tmp_path / "ops" / "log" / "events.jsonl").exists()
    err(O.Ops.create, str(tmp_path / "ops"))
    err(O.Ops.open, str(tmp_path / "missing"))
    assert O.Ops.open(str(tmp_path / "ops")).state == "idle"


# ------------------------------------------------------------------------------ propose
def test_a_refused_release_touches_nothing(world):
    ops, store, lead, _ = world
    assert err(ops.propose, release("1.0", b"k", digest="0" * 64), b"k", store, 1).kind == "DigestMismatch"
    assert err(ops.propose, release("1.0", b"k", [("alice", b"s"), ("alice", b"t")]), b"k", store, 2).kind == "NoQuorum"
    assert ops.state.startswith("refused:") and store.pins == {} and store.event_types() == []  # nothing was put, nothing pinned
    assert lead.state()["kernel_version"] == "0"
    assert err(ops.start_shadow, store, 3).kind == "WrongState" and err(ops.rollback, "why", lead, store, 3).kind == "WrongState"
    rel = release("1.0", b"k")
    ops.propose(rel, b"k", store, 4)                                                           # a refusal does not block a later, valid proposal
    assert ops.state == "proposed" and store.pins == {"kernel.shadow": rel.digest} and store.get(rel.digest) == b"k"
    assert lead.state()["kernel_version"] == "0"                                               # still nothing running changed
    assert err(ops.propose, release("1.1", b"k2"), b"k2", store, 5).kind == "WrongState"


def test_known_digests_and_custom_quorums(world, tmp_path):
    ops, store, _lead, _ = world
    rel = release("1.0", b"abc")
    assert rel.digest == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    ops.propose(rel, b"abc", store, 1)
    store2 = fresh_store(tmp_path, "cas2")
    O.Ops.create(str(tmp_path / "e")).propose(release("1.0", b""), b"", store2, 1)             # an empty artifact with its own digest is fine
    assert store2.get("e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855") == b""
    three = O.Ops.create(str(tmp_path / "three"), 3)
    assert err(three.propose, release("1.0", b"k"), b"k", fresh_store(tmp_path, "cas3"), 1).kind == "NoQuorum"
    one = O.Ops.create(str(tmp_path / "one"), 1)
    one.propose(release("1.0", b"k", [("alice", b"s")]), b"k", fresh_store(tmp_path, "cas1"), 1)
    assert one.state == "proposed" and O.Ops.open(str(tmp_path / "one"), 1).state == "proposed"


# ------------------------------------------------------------------------------ shadow / roll-out
def test_shadow_comes_before_any_live_node(world):
    ops, store, lead, _ = world
    assert err(ops.start_shadow, store, 0).kind == "WrongState" and err(ops.shadow_pass, 0).kind == "WrongState" and err(ops.shadow_fail, "x", store, 0).kind == "WrongState"
    rel = release("1.0", b"k")
    ops.propose(rel, b"k", store, 1)
    assert err(ops.apply_one, "0", 2).kind == "WrongState" and err(ops.shadow_pass, 2).kind == "WrongState"
    ops.start_shadow(store, 3)
    assert ops.state == "shadowing" and store.pins == {"kernel.shadow": rel.digest} and lead.state()["kernel_version"] == "0"
    assert err(ops.start_shadow, store, 4).kind == "WrongState" and err(ops.apply_one, "0", 4).kind == "WrongState"
    ops.shadow_pass(5)
    assert err(ops.apply_one, "shadow", 6).kind == "WrongState" and err(ops.apply_one, "9", 6).kind == "NotFound"
    assert lead.state()["kernel_version"] == "0"
    failed, store2 = O.Ops.create(str(world[3] / "ops2")), fresh_store(world[3], "cas-f")
    failed.propose(release("1.0", b"other"), b"other", store2, 1)
    failed.start_shadow(store2, 2)
    failed.shadow_fail("diverged", store2, 3)
    assert failed.state == "rolled_back:diverged" and "kernel.shadow" not in store2.pins


def test_one_node_at_a_time_and_promotion_only_when_all_applied(world):
    ops, store, lead, _ = world
    rel = ready(ops, store, "1.0", b"k", 1)
    ops.apply_one("1", 5)
    js = json.loads(ops.status_json(lead))
    applied = {n["id"]: n["applied"] for n in js["nodes"] if n.get("role", "live") == "live"}
    assert applied["1"] == "1.0" and applied["0"] != "1.0" and applied["2"] != "1.0" and lead.state()["kernel_version"] == "0"
    ops.apply_one("1", 6)                                                                      # applying again changes nothing
    assert err(ops.promote, lead, store, 7).kind == "WrongState"                               # not every live node has it yet
    ops.apply_one("0", 8)
    assert err(ops.promote, lead, store, 9).kind == "WrongState"
    ops.apply_one("2", 10)
    ops.promote(lead, store, 11)
    assert ops.state == "current" and lead.state()["kernel_version"] == "1.0" and store.pins == {"kernel.current": rel.digest}
    assert err(ops.mark_unhealthy, "9", "x", lead, store, 12).kind == "NotFound"


# ------------------------------------------------------------------------------ rollback
def test_rollbacks(world):
    ops, store, lead, tmp = world
    assert err(ops.rollback, "nothing to undo", lead, store, 0).kind == "WrongState"
    first = to_current(ops, store, lead, "1.0", b"k1", 10)
    ready(ops, store, "2.0", b"k2", 20)
    ops.apply_one("0", 24)
    ops.mark_unhealthy("0", "oom", lead, store, 25)                                            # an unhealthy node during roll-out undoes it
    assert ops.state == "rolled_back:oom" and lead.state()["kernel_version"] == "1.0" and store.pins == {"kernel.current": first.digest}
    assert err(ops.rollback, "again", lead, store, 26).kind == "WrongState"
    second = to_current(ops, store, lead, "2.0", b"k2", 30)                                    # a rollback is followed by a new release
    assert store.pins == {"kernel.current": second.digest, "kernel.previous": first.digest} and lead.state()["kernel_version"] == "2.0"
    ops.rollback("regression", lead, store, 40)
    assert ops.state == "rolled_back:regression" and lead.state()["kernel_version"] == "1.0" and store.pins == {"kernel.current": first.digest}
    ready(ops, store, "3.0", b"k3", 50)
    ops.rollback("changed our minds", lead, store, 55)                                         # mid roll-out: the candidate goes, the kernel stays
    assert "kernel.shadow" not in store.pins and lead.state()["kernel_version"] == "1.0"
    again = O.Ops.open(str(tmp / "ops"))
    assert again.state == "rolled_back:changed our minds" and again.kernel_version == "1.0" and again.event_types() == ops.event_types()


def test_replay_in_the_middle_of_a_roll_out(world):
    ops, store, lead, tmp = world
    ready(ops, store, "1.0", b"k", 1)
    ops.apply_one("2", 5)
    again = O.Ops.open(str(tmp / "ops"))
    assert again.state == ops.state and json.loads(again.status_json(lead)) == json.loads(ops.status_json(lead))
    again.apply_one("0", 6)
    again.apply_one("1", 7)
    again.promote(lead, store, 8)
    assert again.state == "current" and lead.state()["kernel_version"] == "1.0"


# ------------------------------------------------------------------------------ status / cli
def test_status_and_cli(world):
    ops, store, lead, _ = world
    idle = json.loads(ops.status_json(lead))
    assert idle["state"] == "idle" and idle["kernel_version"] == "0" and len(idle["nodes"]) >= 3
    assert "kernel_version: 0" in ops.status_text(lead) and "state: idle" in ops.status_text(lead)
    assert ops.cli(["status"], lead) == ops.status_text(lead)
    assert json.loads(ops.cli(["--json", "status"], lead)) == idle == json.loads(ops.cli(["status", "--json"], lead))   # the flag may come first or last
    for bad in (["frobnicate"], [], ["--json"], ["status", "extra"]):
        err(ops.cli, bad, lead)
    rel = release("1.0", b"k")
    ops.propose(rel, b"k", store, 1)
    ops.start_shadow(store, 2)
    js = json.loads(ops.status_json(lead))
    assert js["state"] == "shadowing" and js["state"] == js["state"].lower() and any(n.get("role") == "shadow" for n in js["nodes"])
    assert sum(1 for n in js["nodes"] if n.get("role") == "live") == 3                         # the shadow node is not one of the live ones


# ------------------------------------------------------------------------------ model
@pytest.mark.parametrize("seed", range(8))
def test_random_operations_match_a_model_of_the_state_machine(tmp_path, seed):
    rng = random.Random(seed)
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    lead = g.get(0)
    backs = []
    for i in range(2):
        (tmp_path / f"b{i}").mkdir()
        backs.append(str(tmp_path / f"b{i}"))
    store, ops = C.Store.create(str(tmp_path / "cas"), backs), O.Ops.create(str(tmp_path / "ops"))
    state, kernel, applied, cand, cur, prev, n_rel, passed = "idle", "0", set(), None, None, None, 0, False
    OPEN = ("proposed", "shadowing", "rolling")

    def digest(v):
        return hashlib.sha256(v.encode()).hexdigest()

    def undo():
        """What a rollback does in the model; returns the error kind, if any."""
        nonlocal state, kernel, cur, prev
        if state in OPEN:
            state = "rolled_back"
        elif state == "current" and prev is not None:
            state, kernel, cur, prev = "rolled_back", prev, prev, None
        elif state == "current":
            return "either"                                                                    # a first release has nothing to go back to
        else:
            return "WrongState"

    for t in range(150):
        op = rng.choice(["propose", "propose_bad", "shadow", "pass", "fail", "apply", "apply", "promote", "unhealthy", "rollback", "reopen"])
        want = None
        if op in ("propose", "propose_bad"):
            n_rel += 1
            v = f"{n_rel}.0"
            signers = GOOD if op == "propose" else [("alice", b"s")]
            call = lambda: ops.propose(release(v, v.encode(), signers), v.encode(), store, t)
            if state in OPEN:
                want = "WrongState"
            elif op == "propose_bad":
                want, state = "NoQuorum", "refused"
            else:
                state, cand, applied, passed = "proposed", v, set(), False
        elif op == "shadow":
            call = lambda: ops.start_shadow(store, t)
            want, state = (None, "shadowing") if state == "proposed" else ("WrongState", state)
        elif op in ("pass", "fail"):
            call = (lambda: ops.shadow_pass(t)) if op == "pass" else (lambda: ops.shadow_fail("bad", store, t))
            if state != "shadowing":
                want = "WrongState"
            elif op == "pass":
                passed = True
            else:
                state = "rolled_back"
        elif op == "apply":
            node = rng.choice(["0", "1", "2"])
            call = lambda: ops.apply_one(node, t)
            if state == "rolling" or (state == "shadowing" and passed):
                state = "rolling"
                applied.add(node)
            else:
                want = "WrongState"
        elif op == "promote":
            call = lambda: ops.promote(lead, store, t)
            if state != "rolling" or len(applied) < 3:
                want = "WrongState"
            else:
                state, kernel, prev, cur = "current", cand, cur, cand
        elif op == "unhealthy":
            node = rng.choice(["0", "1", "2"])
            call = lambda: ops.mark_unhealthy(node, "sick", lead, store, t)                    # an unhealthy live node is a rollback with a reason
            want = undo()
        elif op == "rollback":
            call = lambda: ops.rollback("manual", lead, store, t)
            want = undo()
        else:
            ops = O.Ops.open(str(tmp_path / "ops"))
            call = lambda: None
        if want is None:
            call()
        elif want == "either":
            try:
                call()
                state, kernel = ops.state.split(":")[0], lead.state()["kernel_version"]
                cur = cur if "kernel.current" in store.pins else None
            except NativeError as e:
                assert e.kind == "WrongState"
        else:
            assert err(call).kind == want, (op, state, t)
        assert ops.state.split(":")[0] == state, (op, t, ops.state, state)
        assert lead.state()["kernel_version"] == kernel
        pins = store.pins
        assert pins.get("kernel.current") == (digest(cur) if cur else None)
        assert ("kernel.shadow" in pins) == (state in OPEN)
