"""Behaviour list of the host-side chaos world (C++ ``native.chaos``; reference
harness/chaos/tests/{clock,create_open,disk,gates,invariants,kill,partition,replay,soak,
properties}.rs). Every fault is simulated on event-log replicas on disk: injected time,
replica layout, partitions (one-way and two-way), full and corrupt disks, kills and the
recovery replay, lost and replaced nodes, the lost-task and duplicate-output invariants, the
gate scripts. A Python model of the world is driven with the same random operations."""
import json
import os
import random
import time

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

C = native.chaos


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def world(tmp_path, n=3, procs=4, seed=0, name="w"):
    return C.World.create(str(tmp_path / name), n, procs, seed)


# ------------------------------------------------------------------------------ layout / clock
def test_layout_names_and_open(tmp_path):
    assert (C.MIN_REPLICAS, C.D0_KILLS, C.CLOCK_SKEW_MS, C.SOAK_MS) == (2, 1000, 30_000, 72 * 3600 * 1000)
    for n in (0, 1):
        assert err(lambda: world(tmp_path, n, name=f"few{n}")).kind == "TooFewReplicas"
    w = world(tmp_path, 2)
    assert w.replicas() == ["0", "1"] and w.processes() == ["coordinator", "worker-0", "worker-1", "worker-2"]
    assert w.replica_dir("1") == str(tmp_path / "w" / "replicas" / "1") and sorted(os.listdir(tmp_path / "w" / "replicas")) == ["0", "1"]
    assert all(os.path.getsize(os.path.join(w.replica_dir(r), "events.jsonl")) == 0 for r in w.replicas())
    err(lambda: world(tmp_path, 2))
    err(lambda: C.World.open(str(tmp_path / "missing"), 2))
    assert err(lambda: C.World.open(str(tmp_path / "w"), 1)).kind == "TooFewReplicas"
    assert C.World.open(str(tmp_path / "w"), 2).replicas() == ["0", "1"]
    none = world(tmp_path, 3, 0, name="noproc")
    assert none.processes() == [] and none.replicas() == ["0", "1", "2"]                       # no processes, still three replicas
    assert world(tmp_path, 2, 1, name="one").processes() == ["coordinator"]
    default = C.World.create(str(tmp_path / "default"))
    assert len(default.replicas()) == 2 and len(default.processes()) == 4


def test_time_is_injected(tmp_path):
    w = world(tmp_path)
    assert w.now() == 0
    w.advance(5)
    w.advance(0)
    w.advance(10 ** 9)
    assert w.now() == 5 + 10 ** 9
    w.enqueue_task("t", 123)
    assert w.now() == 5 + 10 ** 9                                                              # the caller's timestamp is data, not the clock
    rec = json.loads(open(os.path.join(w.replica_dir("0"), "events.jsonl")).readline())
    assert rec["payload"] == {"now": 123, "task_id": "t"} and rec["timestamp"] == "1970-01-01T00:00:00Z" and rec["node_id"] == "0"
    w.inject(C.Fault("clock_skew", "0", delta_ms=30_000))
    w.inject(C.Fault("clock_skew", "1", delta_ms=-30_000))
    for over in (30_001, -30_001, 10 ** 12):
        assert err(lambda: w.inject(C.Fault("clock_skew", "0", delta_ms=over))).kind == "ClockSkewBound"
    assert err(lambda: w.inject(C.Fault("clock_skew", "9", delta_ms=1))).kind == "NoReplica"
    assert err(lambda: w.inject(C.Fault("clock_skew", "9", delta_ms=10 ** 9))).kind == "NoReplica"      # the replica is checked first
    assert w.replica_event_types("2") == ["chaos.enqueued", "chaos.fault", "chaos.fault"]                # refused faults are not recorded


# ------------------------------------------------------------------------------ partitions / disks
def test_partitions_block_replication_in_the_stated_direction(tmp_path):
    w = world(tmp_path)
    lens = lambda: [w.log_len(r) for r in w.replicas()]
    w.inject(C.Fault("partition", "0", "1"))                                                   # two-way; enqueues originate at 0, completions at 1
    w.enqueue_task("a", 0)
    w.complete_task("a", 1, b"x", 0)
    assert lens() == [1 + 1, 1 + 1, 1 + 2] and w.invariants().hold()                           # the task is complete on some replica: not lost
    w.inject(C.Fault("heal_partition", "1", "0"))                                              # healing names the pair in either order
    w.enqueue_task("b", 1)
    assert lens() == [4, 4, 5]
    w.inject(C.Fault("partition", "1", "0", True))                                             # one-way: 1 -> 0 is cut, 0 -> 1 still delivers
    w.enqueue_task("c", 2)
    w.complete_task("c", 1, b"x", 2)
    assert lens() == [4 + 2, 4 + 3, 5 + 3]
    for bad in (C.Fault("partition", "0", "7"), C.Fault("partition", "7", "0"), C.Fault("heal_partition", "0", "7")):
        assert err(lambda: w.inject(bad)).kind == "NoReplica"
    assert w.invariants().lost_tasks == 1                                                      # only "b" is still open


def test_full_and_corrupt_disks(tmp_path):
    w = world(tmp_path)
    w.enqueue_task("a", 0)
    w.inject(C.Fault("disk_full", "2"))
    w.enqueue_task("b", 1)
    assert [w.log_len(r) for r in w.replicas()] == [3, 3, 2]                                   # the fault itself was still written there
    w.inject(C.Fault("disk_corrupt", "1"))
    assert open(os.path.join(w.replica_dir("1"), "events.jsonl"), "rb").read() == b"{broken hash chain\n"
    assert err(lambda: w.log_len("1")).kind == "Disk"
    w.enqueue_task("c", 2)
    w.complete_task("c", 1, b"x", 3)                                                           # completions fall back to the first writeable replica
    assert w.log_len("0") == 6 and w.invariants().lost_tasks == 2
    w.recover()                                                                                # skips the corrupt replica
    assert w.replica_event_types("0")[-1] == "chaos.recover" and err(lambda: w.log_len("1")).kind == "Disk"
    err(lambda: C.World.open(str(tmp_path / "w"), 3))                                          # a broken chain on disk fails the open
    for kind in ("disk_full", "disk_corrupt", "node_loss"):
        assert err(lambda: w.inject(C.Fault(kind, "9"))).kind == "NoReplica"
    assert err(lambda: w.inject(C.Fault("node_replace", "9", "10"))).kind == "NoReplica"


# ------------------------------------------------------------------------------ kill / recover / replace
def test_kill_drops_every_handle_until_recovery_replays_the_disk(tmp_path):
    w = world(tmp_path)
    w.enqueue_task("a", 0)
    for unknown in ("nobody", "worker-3", "", "0"):
        assert err(lambda: w.inject(C.Fault("kill", unknown))).kind == "NoProcess"
    w.inject(C.Fault("kill", "worker-2"))                                                      # any process name kills the world's handles
    assert err(lambda: w.enqueue_task("b", 1)).kind == "Other" and err(lambda: w.complete_task("a", 1, b"x", 1)).kind == "Other"
    assert [w.log_len(r) for r in w.replicas()] == [2, 2, 2] and w.invariants().lost_tasks == 1 and w.invariants().duplicated_outputs == 0
    w.recover()
    w.complete_task("a", 1, b"x", 2)
    assert w.invariants().hold() and all(w.replica_event_types(r) == ["chaos.enqueued", "chaos.fault", "chaos.recover", "chaos.completed"] for r in w.replicas())
    w.recover()                                                                                # recovering a healthy world only records it
    assert w.log_len("0") == 5
    again = C.World.open(str(tmp_path / "w"), 3)
    assert again.invariants().hold() and [again.log_len(r) for r in again.replicas()] == [5, 5, 5] and again.now() == 0


def test_lost_and_replaced_nodes(tmp_path):
    w = world(tmp_path)
    w.enqueue_task("a", 0)
    w.inject(C.Fault("node_loss", "0"))
    w.enqueue_task("b", 1)                                                                     # the origin moves to the next writeable replica
    assert [w.log_len(r) for r in w.replicas()] == [2, 3, 3]
    w.inject(C.Fault("node_replace", "1", "n1"))
    assert w.replicas() == ["0", "1", "2", "n1"] and w.log_len("n1") == 0
    w.enqueue_task("c", 2)
    w.complete_task("c", 1, b"x", 2)
    assert [w.log_len(r) for r in w.replicas()] == [2, 4, 6, 2]
    w.inject(C.Fault("node_replace", "2", "n1"))                                               # an existing id is not created twice
    assert w.replicas() == ["0", "1", "2", "n1"]
    w.recover()                                                                                # lost nodes come back from their disks
    w.enqueue_task("d", 3)
    assert [w.replica_event_types(r)[-2:] for r in w.replicas()] == [["chaos.recover", "chaos.enqueued"]] * 4


# ------------------------------------------------------------------------------ invariants
def test_invariants(tmp_path):
    w = world(tmp_path, 2)
    assert w.invariants().hold() and (w.invariants().lost_tasks, w.invariants().duplicated_outputs) == (0, 0)
    w.enqueue_task("a", 0)
    w.enqueue_task("a", 0)                                                                     # the same id twice is one task
    w.enqueue_task("b", 0)
    assert w.invariants().lost_tasks == 2 and not w.invariants().hold()
    w.complete_task("a", 1, b"x", 1)
    w.complete_task("a", 2, b"x", 1)                                                           # another attempt is not a duplicate
    assert (w.invariants().lost_tasks, w.invariants().duplicated_outputs) == (1, 0)
    w.complete_task("a", 2, b"y", 1)
    w.complete_task("a", 2, b"y", 1)
    assert w.invariants().duplicated_outputs == 2 and not w.invariants().hold()
    w.complete_task("ghost", 1, b"", 1)                                                        # never enqueued: nothing to lose
    w.complete_task("b", 1, b"\xff\xfe", 1)
    assert w.invariants().lost_tasks == 0
    pre = world(tmp_path, 2, name="pre")
    pre.enqueue_task("stale", 0)
    failed = err(lambda: C.run_gate(pre, "D3"))                                                # a gate fails on what it finds, even if it was there before
    assert failed.kind == "Invariant" and "lost_tasks=1" in str(failed)


# ------------------------------------------------------------------------------ gates
def test_gate_scripts(tmp_path):
    spec = {g: [json.loads(f.to_json()) for f in C.faults_for(g)] for g in ("D0", "D1", "D2", "D3", "D4", "D5")}
    assert spec["D0"] == [{"kill": {"process": "coordinator"}}]
    assert spec["D1"] == [{"kill": {"process": "coordinator"}}, {"partition": {"from": "0", "to": "1", "asymmetric": False}}]
    assert spec["D2"] == [{"partition": {"from": "0", "to": "1", "asymmetric": True}}, {"clock_skew": {"replica": "0", "delta_ms": 30_000}},
                          {"clock_skew": {"replica": "1", "delta_ms": -30_000}}, {"node_loss": {"replica": "0"}}]
    assert spec["D3"] == [{"job_preempt": {"job": "job-0"}}, {"walltime_kill": {"job": "job-0"}}, "hung_squeue"]
    assert spec["D4"] == ["broker_death", "token_expiry", {"outage": {"provider": "xai"}}]
    assert spec["D5"] == [{"outage": {"provider": "xai"}}, {"outage": {"provider": "openai"}}]             # every hosted provider
    kinds = {next(iter(f)) if isinstance(f, dict) else f for f in map(lambda x: json.loads(x.to_json()), C.faults_for("Soak"))}
    assert {"kill", "partition", "clock_skew", "node_loss", "outage", "broker_death", "hung_squeue"} <= kinds and kinds <= set(C.FAULT_KINDS)
    assert err(lambda: C.faults_for("D6")).kind and err(lambda: C.run_gate(world(tmp_path, name="bad"), "nope")).kind
    a, b = world(tmp_path, 2, 4, 7, "a"), world(tmp_path, 2, 4, 7, "b")
    ra, rb = C.run_gate(a, "D0"), C.run_gate(b, "D0")
    assert ra.faults_applied == rb.faults_applied == 1000 and ra.recovered and ra.invariants.hold()
    assert [a.replica_event_types(r) for r in a.replicas()] == [b.replica_event_types(r) for r in b.replicas()]   # the same seed, the same history
    assert a.replica_event_types("0").count("chaos.fault") == 1000 and a.replica_event_types("0").count("chaos.recover") >= 1000


def test_soak_runs_on_injected_time(tmp_path):
    w = world(tmp_path, 3, 4, 5)
    t0 = time.monotonic()
    rep = C.run_soak(w, C.SOAK_MS, 5)
    assert time.monotonic() - t0 < 30 and w.now() >= C.SOAK_MS                                 # three days pass without sleeping
    assert rep.gate == "Soak" and rep.recovered and rep.invariants.hold() and rep.faults_applied >= len(C.faults_for("Soak"))
    short = world(tmp_path, 2, 4, 1, "short")
    assert C.run_soak(short, 60_000, 1).invariants.hold() and short.now() >= 60_000


# ------------------------------------------------------------------------------ model under random operations
class Model:
    def __init__(self, n, procs):
        self.ids = [str(i) for i in range(n)]
        self.procs = (["coordinator"] + [f"worker-{i}" for i in range(procs - 1)]) if procs else []
        self.events = {r: [] for r in self.ids}
        self.open_, self.full, self.corrupt, self.lost = {r: True for r in self.ids}, set(), set(), set()
        self.cut, self.enq, self.done = set(), [], {}

    def can_write(self, r):
        return self.open_[r] and r not in self.full and r not in self.corrupt and r not in self.lost

    def origin(self, prefer):
        if len(self.ids) > prefer and self.can_write(self.ids[prefer]):
            return self.ids[prefer]
        return next((r for r in self.ids if self.can_write(r)), None)

    def write(self, origin, kind, task=None):
        for r in self.ids:
            if self.can_write(r) and (r == origin or (origin, r) not in self.cut):
                self.events[r].append((kind, task))

    def enqueue(self, t):
        o = self.origin(0)
        if o is None:
            return "Other"
        self.write(o, "chaos.enqueued", t)
        self.enq.append(t)

    def complete(self, t, attempt):
        o = self.origin(1) if len(self.ids) > 1 and self.can_write(self.ids[1]) else self.origin(0)
        if o is None:
            return "Other"
        self.write(o, "chaos.completed", t)
        self.done[(t, attempt)] = self.done.get((t, attempt), 0) + 1

    def inject(self, kind, a="", b="", asym=False, delta=0):
        if kind == "kill" and a not in self.procs:
            return "NoProcess"
        if kind in ("partition", "heal_partition") and (a not in self.ids or b not in self.ids):
            return "NoReplica"
        if kind in ("disk_full", "disk_corrupt", "clock_skew", "node_loss", "node_replace") and a not in self.ids:
            return "NoReplica"
        if kind == "clock_skew" and abs(delta) > 30_000:
            return "ClockSkewBound"
        for r in self.ids:
            if self.can_write(r):
                self.events[r].append(("chaos.fault", None))
        if kind == "kill":
            self.open_ = {r: False for r in self.ids}
        elif kind == "partition":
            self.cut.add((a, b))
            if not asym:
                self.cut.add((b, a))
        elif kind == "heal_partition":
            self.cut -= {(a, b), (b, a)}
        elif kind == "disk_full":
            self.full.add(a)
        elif kind == "disk_corrupt":
            self.open_[a] = False
            self.corrupt.add(a)
            self.events[a] = []
        elif kind == "node_loss":
            self.lost.add(a)
            self.open_[a] = False
        elif kind == "node_replace":
            self.lost.add(a)
            self.open_[a] = False
            if b not in self.ids:
                self.ids.append(b)
                self.events[b], self.open_[b] = [], True

    def recover(self):
        for r in self.ids:
            if r in self.corrupt:
                continue
            self.open_[r] = True
            self.lost.discard(r)
            self.events[r].append(("chaos.recover", None))

    def invariants(self):
        completed = {t for r in self.ids if r not in self.corrupt and r not in self.lost for k, t in self.events[r] if k == "chaos.completed"}
        return len({t for t in self.enq if t not in completed}), sum(c - 1 for c in self.done.values())


@pytest.mark.parametrize("seed", range(10))
def test_random_operations_match_the_model(tmp_path, seed):
    rng = random.Random(seed)
    n = rng.choice([2, 3, 4])
    w, m = world(tmp_path, n, 3, seed), Model(n, 3)
    for step in range(90):
        op = rng.choice(["enqueue", "enqueue", "complete", "complete", "fault", "fault", "recover"])
        rid = lambda: rng.choice(m.ids + ["77"])
        if op == "enqueue":
            t = f"t{rng.randint(0, 15)}"
            want, call = m.enqueue(t), lambda: w.enqueue_task(t, step)
        elif op == "complete":
            t, att = f"t{rng.randint(0, 15)}", rng.randint(1, 2)
            want, call = m.complete(t, att), lambda: w.complete_task(t, att, b"out", step)
        elif op == "recover":
            want, call = m.recover(), lambda: w.recover()
        else:
            kind = rng.choice(["kill", "partition", "partition", "heal_partition", "disk_full", "disk_corrupt", "clock_skew", "node_loss", "node_replace", "outage", "token_expiry", "hung_squeue"])
            if kind == "kill":
                args = dict(a=rng.choice(m.procs + ["ghost"]))
            elif kind in ("partition", "heal_partition"):
                args = dict(a=rid(), b=rid(), asym=kind == "partition" and rng.random() < 0.5)
            elif kind == "clock_skew":
                args = dict(a=rid(), delta=rng.choice([-30_001, -30_000, 0, 5, 30_000, 30_001]))
            elif kind == "node_replace":
                args = dict(a=rid(), b=rng.choice(["n0", "n1", "0"]))
            elif kind in ("outage",):
                args = dict(a="xai")
            elif kind in ("token_expiry", "hung_squeue"):
                args = {}
            else:
                args = dict(a=rid())
            fault = C.Fault(kind, args.get("a", ""), args.get("b", ""), args.get("asym", False), args.get("delta", 0))
            want, call = m.inject(kind, **args), lambda: w.inject(fault)
        if want is None:
            call()
        else:
            assert err(call).kind == want, (op, step)
        assert w.replicas() == m.ids
        for r in m.ids:
            if r in m.corrupt:
                assert err(lambda: w.log_len(r)).kind == "Disk"
                continue
            assert w.log_len(r) == len(m.events[r]), (r, step, op)
            if m.open_[r]:
                assert w.replica_event_types(r) == [k for k, _ in m.events[r]], (r, step, op)
            else:
                err(lambda: w.replica_event_types(r))                                                      # no handle until recovery
        inv = w.invariants()
        assert (inv.lost_tasks, inv.duplicated_outputs) == m.invariants()
