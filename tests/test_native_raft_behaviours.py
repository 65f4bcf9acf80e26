"""Behaviour list of the replicated control state (C++ ``native.raft``; reference
harness/raft/tests/{bootstrap,crash,election,kernel,membership,partition,properties,roles,
token}.rs): bootstrap and reopen, who may vote, the floor of three voters, role leases on
injected time, token generations, elections, partitions and crashes. A Python model of the
leader's state is driven with the same random operations and compared on every node."""
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

R = native.raft
TTL = 30_000


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    return e.value


def node(i, always_on=True, trusted=True):
    return R.NodeInfo(str(i), f"local:{i}", always_on=always_on, trusted=trusted)


def members(c):
    return [(m.id, m.always_on, m.trusted) for m in c.state()["membership"]]


@pytest.fixture
def group(tmp_path):
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    return g


# ------------------------------------------------------------------------------ bootstrap
def test_bootstrap_and_reopen(tmp_path):
    assert R.MIN_VOTERS == 3 and R.ClusterConfig().lease_ttl_ms() == TTL and R.ClusterConfig(100, 0).lease_ttl_ms() == 100   # no missed beats allowed: one period
    c = R.Cluster.bootstrap(str(tmp_path / "solo"), node("a"))
    assert c.is_leader() and c.this_id == "a"
    assert c.state() | {"membership": None} == {"membership": None, "coordinator": None, "token_broker": None, "kernel_version": "0", "token": None}
    assert members(c) == [("a", True, True)]
    err(R.Cluster.bootstrap, str(tmp_path / "solo"), node("a"))
    assert err(R.Cluster.bootstrap, str(tmp_path / "e"), node("e", always_on=False)).kind == "EphemeralVoter"
    assert err(R.Cluster.bootstrap, str(tmp_path / "u"), node("u", trusted=False)).kind == "Untrusted"
    err(R.Cluster.open, str(tmp_path / "missing"), "a")
    c.set_kernel_version("1.2")
    assert c.commit_token(b"tok") == (1, b"tok")
    c.add_voter(node("b"))
    assert [m[0] for m in members(c)] == ["a", "b"]
    assert err(c.set_kernel_version, "1.3").kind == "NotLeader"                                # two voters, one of them absent: no majority
    again = R.Cluster.open(str(tmp_path / "solo"), "a")
    assert again.state()["kernel_version"] == "1.2" and tuple(again.state()["token"]) == (1, b"tok")
    assert [m[0] for m in members(again)] == ["a", "b"] and not again.is_leader()             # leadership is not durable


def test_start_needs_three_voters(tmp_path):
    for n in (0, 1, 2):
        assert err(R.LocalGroup.start, n, str(tmp_path / f"g{n}")).kind == "TooFewVoters"
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    assert g.leader() == -1                                                                    # nobody leads before the first tick
    g.tick(0)
    assert g.leader() == 0 and [g.get(i).is_leader() for i in range(3)] == [True, False, False] and g.get(0).term == 1
    g.tick(1)
    g.tick(10 ** 9)
    assert g.leader() == 0 and g.get(0).term == 1                                              # a stable group does not re-elect


# ------------------------------------------------------------------------------ membership
def test_followers_refuse_every_write(group):
    f = group.get(1)
    for call in (lambda: f.add_voter(node(9)), lambda: f.add_worker(node(9, always_on=False)), lambda: f.remove_node("2"), lambda: f.set_kernel_version("x"),
                 lambda: f.claim_role("coordinator", "1", 0), lambda: f.heartbeat_role("coordinator", "1", 0), lambda: f.commit_token(b"t")):
        assert err(call).kind == "NotLeader"
    assert f.log_len == group.get(0).log_len


def test_who_may_join_and_the_floor_of_three_voters(group):
    L = group.get(0)
    L.add_worker(node("w", always_on=False))
    L.add_worker(node("guest", always_on=False, trusted=False))                                # an untrusted worker may join; it can hold no role
    assert err(L.add_voter, node("e", always_on=False)).kind == "EphemeralVoter" and err(L.add_voter, node("u", trusted=False)).kind == "Untrusted"
    assert err(L.add_worker, node("big")).kind == "Other"                                      # an always-on node joins as a voter
    for dup in (node("w", always_on=False), node("1", always_on=False)):
        assert err(L.add_worker, dup).kind == "Duplicate"
    assert err(L.add_voter, node("w")).kind == "Duplicate" and err(L.add_voter, node("2")).kind == "Duplicate"
    assert err(L.remove_node, "nobody").kind == "NotFound"
    for v in ("1", "2"):
        assert err(L.remove_node, v).kind == "TooFewVoters"                                    # never below three once three were reached
    L.remove_node("w")                                                                         # workers do not count toward the floor
    L.add_voter(node(3))
    L.remove_node("3")
    assert err(L.remove_node, "2").kind == "TooFewVoters"
    assert [m[0] for m in members(L)] == ["0", "1", "2", "guest"]
    assert all(members(group.get(i)) == members(L) for i in range(3))
    assert err(L.claim_role, "coordinator", "guest", 0).kind == "Untrusted" and err(L.claim_role, "coordinator", "ghost", 0).kind == "NotFound"


# ------------------------------------------------------------------------------ roles / token / kernel
def test_role_leases_run_on_injected_time(group):
    L = group.get(0)
    assert L.claim_role("coordinator", "1", 1_000) == {"role": "coordinator", "holder": "1", "attempt": 1, "expires_at": 1_000 + TTL}
    assert L.claim_role("token_broker", "1", 1_000)["attempt"] == 1                            # a separate role; one node may hold both
    assert err(L.claim_role, "coordinator", "2", 1_000 + TTL - 1).kind == "NotClaimable" and err(L.claim_role, "coordinator", "1", 2_000).kind == "NotClaimable"
    assert err(L.heartbeat_role, "coordinator", "2", 2_000).kind == "NotHolder" and err(L.claim_role, "janitor", "1", 0).kind == "Other"
    assert L.heartbeat_role("coordinator", "1", 20_000)["expires_at"] == 20_000 + TTL
    assert L.expire_roles(1_000 + TTL - 1) == [] and L.expire_roles(1_000 + TTL) == ["token_broker"]
    assert err(L.heartbeat_role, "token_broker", "1", 31_001).kind == "NotHolder"              # a vacant role has no holder
    assert L.claim_role("token_broker", "2", 31_001)["attempt"] == 2
    took = L.claim_role("coordinator", "2", 20_000 + TTL)                                      # an expired lease can be taken without an expiry sweep
    assert (took["holder"], took["attempt"]) == ("2", 2)
    assert L.expire_roles(10 ** 12) == ["coordinator", "token_broker"] and L.expire_roles(10 ** 12) == []
    assert all(group.get(i).state()["coordinator"] is None for i in range(3))


def test_tokens_and_kernel_version_replicate_and_survive_a_restart(group):
    L = group.get(0)
    assert L.commit_token(b"first") == (1, b"first") and L.commit_token(b"\x00\xff") == (2, b"\x00\xff")
    L.set_kernel_version("1.0")
    L.set_kernel_version("1.1")
    for i in range(3):
        s = group.get(i).state()
        assert s["kernel_version"] == "1.1" and tuple(s["token"]) == (2, b"\x00\xff")
    group.crash(1)
    assert err(group.get, 1).kind == "NotFound" and err(group.crash, 1).kind == "NotFound" and err(group.restart, 0).kind
    L.commit_token(b"third")
    n0, n2 = group.get(0).log_len, group.get(2).log_len
    group.restart(1)
    assert tuple(group.get(1).state()["token"]) == (2, b"\x00\xff") and (group.get(0).log_len, group.get(2).log_len) == (n0, n2)
    group.tick(1)
    assert tuple(group.get(1).state()["token"]) == (3, b"third")


# ------------------------------------------------------------------------------ elections / partitions / crashes
def test_partitions(group):
    L = group.get(0)
    L.set_kernel_version("1.0")
    n = L.log_len
    assert err(group.partition, [5]).kind == "NotFound"
    group.partition([1, 2])                                                                    # the leader alone: no majority, no commit
    assert err(L.set_kernel_version, "lost").kind == "NotLeader" and L.log_len == n
    group.heal()
    group.partition([2])                                                                       # leader plus one follower is a majority of three
    group.tick(1)
    L.set_kernel_version("1.1")
    assert [group.get(i).state()["kernel_version"] for i in range(3)] == ["1.1", "1.1", "1.0"]
    group.heal()
    group.tick(2)
    assert group.get(2).state()["kernel_version"] == "1.1"
    group.partition([0])
    group.tick(40_000)
    assert group.leader() == 1 and group.get(1).term == 2 and sum(group.get(i).is_leader() for i in range(3)) == 1
    group.get(1).set_kernel_version("2.0")
    assert group.get(0).state()["kernel_version"] == "1.1"
    group.heal()
    group.tick(40_001)
    assert [group.get(i).state()["kernel_version"] for i in range(3)] == ["2.0"] * 3 and group.get(0).term == 2 and not group.get(0).is_leader()


def test_a_crashed_leader_is_replaced_and_the_state_survives(group):
    L = group.get(0)
    L.add_worker(node("w", always_on=False))
    L.set_kernel_version("3.3")
    L.commit_token(b"t")
    L.claim_role("coordinator", "1", 40_000)
    group.crash(0)
    group.tick(50_000)
    lead = group.get(group.leader())
    assert group.leader() == 1 and lead.term == 2
    s = lead.state()
    assert s["kernel_version"] == "3.3" and tuple(s["token"]) == (1, b"t") and s["coordinator"]["holder"] == "1" and [m[0] for m in members(lead)] == ["0", "1", "2", "w"]
    group.crash(2)                                                                             # two of three gone: nobody can lead
    group.tick(100_000)
    assert err(lead.set_kernel_version, "x").kind == "NotLeader"
    group.restart(0)
    group.restart(2)
    group.tick(150_000)
    assert group.leader() >= 0 and sum(group.get(i).is_leader() for i in range(3)) == 1
    group.get(group.leader()).set_kernel_version("3.4")
    assert [group.get(i).state()["kernel_version"] for i in range(3)] == ["3.4"] * 3


# ------------------------------------------------------------------------------ model
class Model:
    def __init__(self):
        self.members = {str(i): (True, True) for i in range(3)}                                # id -> (always_on, trusted); insertion ordered
        self.roles = {"coordinator": None, "token_broker": None}
        self.attempt = {"coordinator": 0, "token_broker": 0}
        self.kernel, self.token, self.reached = "0", None, True

    def voters(self):
        return [m for m, (on, _) in self.members.items() if on]

    def add(self, nid, always_on, trusted, as_voter):
        if nid in self.members:
            return "Duplicate"
        if as_voter and not always_on:
            return "EphemeralVoter"
        if as_voter and not trusted:
            return "Untrusted"
        if not as_voter and always_on:
            return "Other"
        self.members[nid] = (always_on, trusted)

    def remove(self, nid):
        if nid not in self.members:
            return "NotFound"
        if self.members[nid][0] and len(self.voters()) - 1 < 3:
            return "TooFewVoters"
        del self.members[nid]
        for r, held in self.roles.items():                                                     # a removed node keeps no role
            if held and held["holder"] == nid:
                self.roles[r] = None

    def claim(self, role, nid, now):
        if nid not in self.members:
            return "NotFound"
        if not self.members[nid][1]:
            return "Untrusted"
        held = self.roles[role]
        if held and held["expires_at"] > now:
            return "NotClaimable"
        self.attempt[role] += 1
        self.roles[role] = {"role": role, "holder": nid, "attempt": self.attempt[role], "expires_at": now + TTL}

    def heartbeat(self, role, nid, now):
        held = self.roles[role]
        if not held or held["holder"] != nid:
            return "NotHolder"
        held["expires_at"] = now + TTL

    def expire(self, now):
        out = [r for r in ("coordinator", "token_broker") if self.roles[r] and self.roles[r]["expires_at"] <= now]
        for r in out:
            self.roles[r] = None
        return out


@pytest.mark.parametrize("seed", range(8))
def test_random_leader_operations_match_the_model_on_every_node(tmp_path, seed):
    rng = random.Random(seed)
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    L, m, now = g.get(0), Model(), 0
    for step in range(120):
        now += rng.choice([1, 1_000, 14_000, 31_000])
        op = rng.choice(["add_voter", "add_worker", "remove", "claim", "claim", "heartbeat", "heartbeat", "expire", "kernel", "token"])
        nid = rng.choice(["0", "1", "2", "3", "4", "w1", "w2", "ghost"])
        role = rng.choice(["coordinator", "token_broker"])
        want = None
        if op in ("add_voter", "add_worker"):
            if op == "add_voter" and len(m.voters()) >= 5:
                nid = "0"                                                                      # three running nodes are a majority of at most five voters
            on, tr = rng.random() < 0.6, rng.random() < 0.8
            want = m.add(nid, on, tr, op == "add_voter")
            call = lambda: getattr(L, op)(R.NodeInfo(nid, "", always_on=on, trusted=tr))
        elif op == "remove":
            if nid in ("0", "1", "2") and len(m.voters()) > 3:
                nid = "3" if "3" in m.members else "ghost"                                       # the three running nodes stay, so a majority stays
            want, call = m.remove(nid), lambda: L.remove_node(nid)
        elif op == "claim":
            want, call = m.claim(role, nid, now), lambda: L.claim_role(role, nid, now)
        elif op == "heartbeat":
            want, call = m.heartbeat(role, nid, now), lambda: L.heartbeat_role(role, nid, now)
        elif op == "expire":
            expected = m.expire(now)
            assert L.expire_roles(now) == expected
            call = lambda: None
        elif op == "kernel":
            m.kernel = f"v{step}"
            call = lambda: L.set_kernel_version(f"v{step}")
        else:
            m.token = ((m.token[0] if m.token else 0) + 1, bytes([step]))
            call = lambda: L.commit_token(bytes([step]))
        if want is None:
            try:
                call()
            except NativeError as e:
                raise AssertionError((op, nid, step, dict(m.members), str(e)))
        else:
            assert err(call).kind == want, (op, nid, role, step)
        for i in range(3):
            s = g.get(i).state()
            assert [(x.id, x.always_on, x.trusted) for x in s["membership"]] == [(k, *v) for k, v in m.members.items()]
            assert s["kernel_version"] == m.kernel and (tuple(s["token"]) if s["token"] else None) == m.token
            assert s["coordinator"] == m.roles["coordinator"] and s["token_broker"] == m.roles["token_broker"]
    g.crash(1)
    g.restart(1)
    assert g.get(1).state()["kernel_version"] == m.kernel                                       # and all of it was on disk
