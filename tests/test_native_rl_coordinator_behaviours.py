"""Behaviour list of the RL coordinator (C++ ``native.coordinator``), one case per documented rule:
construction checks and their order, the deterministic initial split, the FIFO queue with its
stale-prefix drop, publish / sync versioning, the five rebalance rules and parity halts
(reference rl/coordinator/tests/{construction,enqueue,publish_sync,rebalance,stale_drop,
staleness,parity,properties}.rs). The last test drives the C++ and a small Python model of the
same rules with the same random operations and compares every answer."""
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

CO = native.coordinator


def cfg(**kw):
    base = dict(max_staleness=CO.MAX_STALENESS, rollout_numer=CO.DEFAULT_ROLLOUT_NUMER,
                rollout_denom=CO.DEFAULT_ROLLOUT_DENOM, parity_threshold=0.25, queue_high=8,
                min_rollout_racks=1, min_trainer_racks=1)
    base.update(kw)
    return CO.CoordinatorConfig(**base)


def racks(n, gpus=8):
    return [(f"r{i:02d}", gpus) for i in range(n)]


def batch(bid, pid="p", version=0, n=1, routing=False):
    return CO.RolloutBatch(bid, pid, version, n_samples=n, routing_present=routing)


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


# ------------------------------------------------------------------------------ construction
@pytest.mark.parametrize("config, fleet, kind, text", [
    (dict(), [], "EmptyFleet", None),
    (dict(), [("a", 8), ("b", 8), ("a", 4)], "DuplicateRack", "a"),
    (dict(), [("a", 8), ("b", 0), ("c", 8)], "Message", "gpu"),
    (dict(), [("solo", 0)], "Message", "gpu"),                       # zero GPUs before NotEnoughRacks
    (dict(), [("x", 0), ("x", 8)], "DuplicateRack", "x"),            # duplicate before zero GPUs
    (dict(rollout_denom=0), racks(4), "BadSplit", None),
    (dict(rollout_numer=101, rollout_denom=100), racks(4), "BadSplit", None),
    (dict(min_rollout_racks=2, min_trainer_racks=2), racks(3), "NotEnoughRacks", None),
    (dict(rollout_denom=0), [], "EmptyFleet", None),                 # empty fleet before BadSplit
])
def test_construction_checks_and_their_order(config, fleet, kind, text):
    e = err(lambda: CO.Coordinator(cfg(**config), fleet))
    assert e.kind == kind
    if text:
        assert text in str(e).lower()


@pytest.mark.parametrize("config, fleet, rollout_ids, split", [
    (dict(), racks(4), ["r00", "r01"], (16, 16)),
    (dict(), [("r03", 8), ("r01", 8), ("r02", 8), ("r00", 8)], ["r00", "r01"], (16, 16)),
    (dict(min_rollout_racks=2), racks(3, 10), ["r00", "r01"], (20, 10)),          # floor overshoots target 19
    (dict(), [("d", 1), ("c", 10), ("b", 10), ("a", 1)], ["a", "b"], (11, 11)),
    (dict(), [("a", 100), ("b", 1)], ["a"], (100, 1)),
    (dict(rollout_numer=100, min_rollout_racks=0, min_trainer_racks=0), racks(4), ["r00", "r01", "r02", "r03"], (32, 0)),
    (dict(rollout_numer=100), racks(4), ["r00", "r01", "r02"], (24, 8)),
    (dict(rollout_numer=0), racks(3), ["r00"], (8, 16)),
    (dict(rollout_numer=100, min_trainer_racks=2), racks(4, 1), ["r00", "r01"], (2, 2)),
    (dict(), racks(5, 1), ["r00", "r01", "r02"], (3, 2)),
])
def test_initial_assignment_is_a_lexicographic_prefix(config, fleet, rollout_ids, split):
    c = CO.Coordinator(cfg(**config), fleet)
    assert c.split_gpus() == split and c.n_rollout_racks() == len(rollout_ids)
    assert c.n_trainer_racks() == len(fleet) - len(rollout_ids)
    for rid, _ in fleet:
        if rid in rollout_ids:
            assert c.rack_role(rid) == "rollout" and c.rack_version(rid) == 0
        else:
            assert c.rack_role(rid) == "trainer"
            e = err(lambda: c.rack_version(rid))
            assert e.kind == "NotRollout" and rid in str(e)
    assert c.trainer_version() == 0 and c.state() == "running" and not c.halted() and c.queue_depth() == 0


def test_zero_max_staleness_is_allowed_and_unknown_rack_is_not_found():
    c = CO.Coordinator(cfg(max_staleness=0), racks(4))
    assert c.trainer_version() == 0 and c.state() == "running"
    e = err(lambda: c.rack_role("nope"))
    assert e.kind == "RackNotFound" and "nope" in str(e)


# ------------------------------------------------------------------------------ enqueue
def test_queue_is_fifo_and_returns_batches_unchanged():
    c = CO.Coordinator(cfg(), racks(4))
    assert c.consume_batch() is None
    c.enqueue_batch(batch("b0", "shared", 0, 16, True))
    c.enqueue_batch(batch("b1", "shared", 0, 3, False))            # n_samples need not be the group size
    assert c.queue_depth() == 2
    a, b = c.consume_batch(), c.consume_batch()
    assert (a.id, a.prompt_id, a.n_samples, a.routing_present) == ("b0", "shared", 16, True)
    assert (b.id, b.prompt_id, b.n_samples, b.routing_present) == ("b1", "shared", 3, False)
    assert c.consume_batch() is None and c.queue_depth() == 0


def test_enqueue_validation_and_its_order():
    c = CO.Coordinator(cfg(), racks(4))
    assert err(lambda: c.enqueue_batch(batch("b", "p", 0, 0))).kind == "EmptyGroup"
    assert err(lambda: c.enqueue_batch(batch("", "", 0, 0))).kind == "EmptyGroup"     # empty group wins over empty ids
    e = err(lambda: c.enqueue_batch(batch("", "p")))
    assert e.kind == "Message" and "id" in str(e).lower()
    e = err(lambda: c.enqueue_batch(batch("b", "")))
    assert e.kind == "Message" and "prompt" in str(e).lower()
    e = err(lambda: c.enqueue_batch(batch("", "")))
    assert e.kind == "Message" and "id" in str(e).lower() and "prompt" not in str(e).lower().replace("prompt_id", "")
    assert c.queue_depth() == 0


def test_duplicate_ids_only_while_queued_and_versions_unchecked_at_enqueue():
    c = CO.Coordinator(cfg(), racks(4))
    c.enqueue_batch(batch("dup"))
    e = err(lambda: c.enqueue_batch(batch("dup")))
    assert e.kind == "DuplicateBatch" and "dup" in str(e)
    assert c.consume_batch().id == "dup"
    c.enqueue_batch(batch("dup"))                                   # a consumed id may come back
    assert c.queue_depth() == 1 and c.consume_batch().id == "dup"
    c.enqueue_batch(batch("ahead", version=7))                      # not validated here ...
    assert err(lambda: c.consume_batch()).kind == "FromTheFuture"   # ... but on consume
    assert c.queue_depth() == 1


# ------------------------------------------------------------------------------ publish / sync
def test_publish_is_strictly_the_next_version_and_leaves_racks_alone():
    c = CO.Coordinator(cfg(), racks(4))
    for bad in (0, 2, 5):
        assert err(lambda: c.publish_weights(bad)).kind == "NotNextVersion"
    c.publish_weights(1)
    assert c.trainer_version() == 1 and c.rack_version("r00") == 0 and c.rack_version("r01") == 0
    for bad in (1, 3):
        assert err(lambda: c.publish_weights(bad)).kind == "NotNextVersion"
    c.publish_weights(2)
    assert c.trainer_version() == 2


def test_version_zero_batches_are_valid_before_any_publish():
    c = CO.Coordinator(cfg(), racks(4))
    c.enqueue_batch(batch("v0"))
    assert c.consume_batch().policy_version == 0
    c.sync_rack("r00", 0)                                           # sync of 0 at trainer version 0
    assert c.rack_version("r00") == 0


def test_sync_rules():
    c = CO.Coordinator(cfg(), racks(4))
    c.publish_weights(1)
    e = err(lambda: c.sync_rack("r00", 0))
    assert e.kind == "Unpublished" and "0" in str(e)
    e = err(lambda: c.sync_rack("r00", 2))
    assert e.kind == "Unpublished" and "2" in str(e)
    c.sync_rack("r00", 1)
    assert c.rack_version("r00") == 1 and c.rack_version("r01") == 0     # only that rack
    assert err(lambda: c.sync_rack("ghost", 1)).kind == "RackNotFound"
    assert err(lambda: c.sync_rack("ghost", 9)).kind == "RackNotFound"   # before Unpublished
    assert err(lambda: c.sync_rack("r03", 1)).kind == "NotRollout"
    for v in (2, 3):
        c.publish_weights(v)
        for r in ("r00", "r01"):
            c.sync_rack(r, v)
            assert c.rack_version(r) == v
    assert err(lambda: c.rack_version("ghost")).kind == "RackNotFound"


# ------------------------------------------------------------------------------ staleness
def test_staleness_function():
    assert CO.staleness(0, 0) == 0 and CO.staleness(7, 7) == 0
    assert CO.staleness(9, 4) == 5
    assert err(lambda: CO.staleness(3, 4)).kind == "FromTheFuture"
    assert CO.staleness(CO.MAX_STALENESS, 0) == CO.MAX_STALENESS


def _at_version(c, v):
    for i in range(c.trainer_version() + 1, v + 1):
        c.publish_weights(i)


def test_stale_prefix_drop_boundaries():
    c = CO.Coordinator(cfg(max_staleness=2), racks(4))
    c.enqueue_batch(batch("keep", version=0))
    _at_version(c, 2)
    assert c.consume_batch().id == "keep"                           # staleness == max is kept
    c.enqueue_batch(batch("gone", version=0))
    _at_version(c, 3)
    assert c.consume_batch() is None and c.queue_depth() == 0      # one past max is dropped


def test_only_a_stale_prefix_is_dropped():
    c = CO.Coordinator(cfg(max_staleness=1), racks(4))
    _at_version(c, 1)
    c.enqueue_batch(batch("s0", version=0))
    c.enqueue_batch(batch("s1", version=0))
    c.enqueue_batch(batch("fresh", version=1))
    c.enqueue_batch(batch("late_stale", version=0))
    _at_version(c, 2)
    assert c.consume_batch().id == "fresh"                          # s0, s1 dropped on the way
    assert c.queue_depth() == 1
    assert c.consume_batch() is None and c.queue_depth() == 0      # the trailing stale one goes next


def test_future_batch_leaves_the_queue_unchanged():
    c = CO.Coordinator(cfg(max_staleness=0), racks(4))
    c.enqueue_batch(batch("stale", version=0))
    c.enqueue_batch(batch("future", version=9))
    _at_version(c, 2)
    assert err(lambda: c.consume_batch()).kind == "FromTheFuture"
    assert c.queue_depth() == 2                                     # the stale prefix was not dropped either
    c2 = CO.Coordinator(cfg(max_staleness=0), racks(4))
    _at_version(c2, 1)
    c2.enqueue_batch(batch("old", version=0))
    c2.enqueue_batch(batch("match", version=1))
    assert c2.consume_batch().id == "match"                         # only the matching version survives


# ------------------------------------------------------------------------------ rebalance
def test_rule_one_empty_queue_prefers_rollout_lowest_trainer_first():
    c = CO.Coordinator(cfg(rollout_numer=50), racks(4))
    assert c.split_gpus() == (16, 16)
    assert c.rebalance() == ("r02", "rollout")
    assert c.rack_role("r02") == "rollout" and c.rack_version("r02") == 0 and c.rack_role("r03") == "trainer"
    assert (c.n_rollout_racks(), c.n_trainer_racks()) == (3, 1)


def test_rule_two_backlog_moves_the_lowest_rollout_rack_to_training():
    c = CO.Coordinator(cfg(rollout_numer=50, queue_high=2), racks(4))
    c.enqueue_batch(batch("a"))
    c.enqueue_batch(batch("b"))
    assert c.rebalance() == ("r00", "trainer")
    assert c.rack_role("r00") == "trainer" and err(lambda: c.rack_version("r00")).kind == "NotRollout"
    assert c.queue_depth() == 2


def test_queue_high_zero_never_fires_rule_two_and_floors_block():
    c = CO.Coordinator(cfg(rollout_numer=50, queue_high=0), racks(4))
    for i in range(5):
        c.enqueue_batch(batch(f"b{i}"))
    assert c.rebalance() is None and c.n_rollout_racks() == 2 and c.queue_depth() == 5
    c2 = CO.Coordinator(cfg(), racks(2))
    assert (c2.n_rollout_racks(), c2.n_trainer_racks()) == (1, 1) and c2.rebalance() is None


def test_rules_three_and_four_follow_the_gpu_target():
    c = CO.Coordinator(cfg(), racks(4))                              # target 20, holds 16
    c.enqueue_batch(batch("only"))
    assert c.rebalance() == ("r02", "rollout") and c.split_gpus() == (24, 8) and c.queue_depth() == 1
    c2 = CO.Coordinator(cfg(rollout_numer=50), racks(4))
    assert c2.rebalance() == ("r02", "rollout") and c2.split_gpus() == (24, 8)     # rule 1 overshoots
    c2.enqueue_batch(batch("q"))
    assert c2.rebalance() == ("r00", "trainer") and c2.n_rollout_racks() == 2      # rule 4 peels one back
    c3 = CO.Coordinator(cfg(rollout_numer=50), racks(4))
    c3.enqueue_batch(batch("q"))
    assert c3.rebalance() is None                                   # at target, queue below high


def test_flip_back_to_rollout_resets_the_rack_version_and_keeps_the_queue():
    c = CO.Coordinator(cfg(rollout_numer=50, queue_high=1), racks(4))
    c.publish_weights(1)
    c.sync_rack("r00", 1)
    c.enqueue_batch(batch("keep", "prompt-x", 1, 4, True))
    assert c.rebalance() == ("r00", "trainer")
    got = c.consume_batch()
    assert (got.id, got.prompt_id, got.routing_present) == ("keep", "prompt-x", True)
    assert c.rebalance() == ("r00", "rollout") and c.rack_version("r00") == 0


def test_empty_queue_over_target_oscillates():
    c = CO.Coordinator(cfg(rollout_numer=50), racks(4))
    moves = [c.rebalance()[1] for _ in range(3)]
    assert moves == ["rollout", "trainer", "rollout"]


# ------------------------------------------------------------------------------ parity
def test_parity_report_threshold_and_halt():
    c = CO.Coordinator(cfg(parity_threshold=0.25), racks(4))
    assert c.run_parity(0, []) == (0, 0.0, 0)
    assert err(lambda: c.run_parity(1, [])).kind == "Unpublished"
    for bad in (float("nan"), float("inf"), float("-inf")):
        assert err(lambda: c.run_parity(0, [(bad, -1.0)])).kind == "InvalidLogprob"
        assert err(lambda: c.run_parity(0, [(-1.0, bad)])).kind == "InvalidLogprob"
    assert not c.halted()
    v, worst, n = c.run_parity(0, [(-1.0, -1.25), (-3.0, -2.9)])
    assert (v, n) == (0, 2) and worst == 0.25 and not c.halted()    # equal to the threshold does not halt
    e = err(lambda: c.run_parity(0, [(-1.0, -1.0), (-2.0, -2.5)]))
    assert e.kind == "ParityHalt" and c.halted() and c.state() == "halted"
    for call in (lambda: c.enqueue_batch(batch("x")), c.consume_batch, c.rebalance, lambda: c.publish_weights(1),
                 lambda: c.sync_rack("r00", 0), lambda: c.run_parity(0, [])):
        assert err(call).kind == "Halted"
    # reads still answer
    assert c.trainer_version() == 0 and c.split_gpus() == (16, 16) and c.queue_depth() == 0
    assert c.rack_role("r00") == "rollout" and c.n_rollout_racks() == 2 and c.rack_version("r00") == 0


# ------------------------------------------------------------------------------ model check
class _Model:
    """The documented rules, written directly; errors are returned as their kind."""

    def __init__(self, c, fleet):
        self.c = c
        order = sorted(fleet)
        total = sum(g for _, g in order)
        self.target = total * c["rollout_numer"] // c["rollout_denom"]
        self.gpus = dict(order)
        self.role, run, n_roll = {}, 0, 0
        for i, (rid, g) in enumerate(order):
            left_after = len(order) - i - 1
            if run + g <= self.target and left_after >= c["min_trainer_racks"]:
                self.role[rid] = "rollout"
                run += g
                n_roll += 1
            else:
                break
        for rid, _ in order:
            if rid not in self.role:
                if n_roll < c["min_rollout_racks"]:
                    self.role[rid] = "rollout"
                    n_roll += 1
                else:
                    self.role[rid] = "trainer"
        self.version = {r: 0 for r in self.role}
        self.trainer, self.queue = 0, []

    def n(self, role):
        return sum(1 for r in self.role.values() if r == role)

    def rollout_gpus(self):
        return sum(self.gpus[r] for r, role in self.role.items() if role == "rollout")

    def enqueue(self, bid, ver):
        if any(b == bid for b, _ in self.queue):
            return "DuplicateBatch"
        self.queue.append((bid, ver))

    def consume(self):
        drop = 0
        for _b, ver in self.queue:
            if ver > self.trainer:
                return "FromTheFuture"
            if self.trainer - ver > self.c["max_staleness"]:
                drop += 1
            else:
                break
        # a future batch anywhere behind the stale prefix but before the first kept one is seen
        # by the loop above; beyond the first kept batch nothing is scanned
        self.queue = self.queue[drop:]
        return self.queue.pop(0)[0] if self.queue else None

    def publish(self, v):
        if v != self.trainer + 1:
            return "NotNextVersion"
        self.trainer = v

    def sync(self, rid, v):
        if rid not in self.role:
            return "RackNotFound"
        if self.role[rid] != "rollout":
            return "NotRollout"
        if v != self.trainer:
            return "Unpublished"
        self.version[rid] = v

    def _to_rollout(self):
        if self.n("trainer") - 1 < self.c["min_trainer_racks"]:
            return None
        rid = min(r for r, role in self.role.items() if role == "trainer")
        self.role[rid], self.version[rid] = "rollout", 0
        return (rid, "rollout")

    def _to_trainer(self):
        if self.n("rollout") - 1 < self.c["min_rollout_racks"]:
            return None
        rid = min(r for r, role in self.role.items() if role == "rollout")
        self.role[rid] = "trainer"
        return (rid, "trainer")

    def rebalance(self):
        depth, high = len(self.queue), self.c["queue_high"]
        if depth == 0:
            got = self._to_rollout()
            if got:
                return got
        if high > 0 and depth >= high:
            got = self._to_trainer()
            if got:
                return got
        if self.rollout_gpus() < self.target:
            got = self._to_rollout()
            if got:
                return got
        if self.rollout_gpus() > self.target:
            got = self._to_trainer()
            if got:
                return got
        return None


def _native(call):
    try:
        return call()
    except NativeError as e:
        return e.kind


@pytest.mark.parametrize("seed", range(12))
def test_random_operation_sequences_match_the_rule_model(seed):
    rng = random.Random(seed)
    c = dict(max_staleness=rng.randint(0, 3), rollout_numer=rng.choice([0, 35, 50, 65, 100]), rollout_denom=100,
             parity_threshold=0.25, queue_high=rng.choice([0, 1, 2, 4]), min_rollout_racks=rng.randint(0, 2),
             min_trainer_racks=rng.randint(0, 2))
    n = rng.randint(max(2, c["min_rollout_racks"] + c["min_trainer_racks"]), 6)
    fleet = [(f"k{rng.randint(0, 99):02d}-{i}", rng.choice([1, 4, 8, 16])) for i in range(n)]
    co, mo = CO.Coordinator(CO.CoordinatorConfig(**c), fleet), _Model(c, fleet)
    next_id = 0
    for _step in range(200):
        op = rng.choice(["enqueue", "enqueue", "consume", "publish", "sync", "rebalance", "rebalance"])
        if op == "enqueue":
            bid = f"b{next_id if rng.random() < 0.9 else max(0, next_id - 1)}"
            next_id += 1
            ver = max(0, mo.trainer - rng.randint(0, 4)) if rng.random() < 0.95 else mo.trainer + 1
            got, want = _native(lambda: co.enqueue_batch(batch(bid, "p", ver))), mo.enqueue(bid, ver)
        elif op == "consume":
            got = _native(lambda: co.consume_batch())
            got = got.id if hasattr(got, "id") else got
            want = mo.consume()
        elif op == "publish":
            v = mo.trainer + (1 if rng.random() < 0.8 else rng.choice([0, 2]))
            got, want = _native(lambda: co.publish_weights(v)), mo.publish(v)
        elif op == "sync":
            rid = rng.choice([r for r, _ in fleet] + ["ghost"])
            v = mo.trainer if rng.random() < 0.8 else mo.trainer + 1
            got, want = _native(lambda: co.sync_rack(rid, v)), mo.sync(rid, v)
        else:
            got, want = _native(lambda: co.rebalance()), mo.rebalance()
        assert got == want, (seed, _step, op, got, want)
        assert co.queue_depth() == len(mo.queue) and co.trainer_version() == mo.trainer
        assert co.n_rollout_racks() == mo.n("rollout") and co.split_gpus()[0] == mo.rollout_gpus()
        for rid, role in mo.role.items():
            assert co.rack_role(rid) == role
            if role == "rollout":
                assert co.rack_version(rid) == mo.version[rid]
