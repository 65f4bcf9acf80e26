"""Behaviour list of the elastic controller, one test per behaviour (names follow the reference's
control/tests/{collectives,fail,heal,health,new,straggler,sdc,spike}.rs): membership, gradient
accumulation that holds the tokens per step, the collective watchdog on an injected clock,
health events, spare healing at a step boundary, the checksum vote and the spike policy."""
import pytest

from prometheus_b200 import native

K = native.control


def ctl(live=4, spares=0, tokens=4096, micro=512, **kw):
    specs = [K.ReplicaSpec(f"r{i}", f"rack{i}") for i in range(live)]
    specs += [K.ReplicaSpec(f"s{i}", f"rack{live + i}", True) for i in range(spares)]
    return K.Controller(K.ElasticConfig(tokens, micro, **kw), specs)


def kind_of(fn, *a):
    with pytest.raises(native.NativeError) as e:
        fn(*a)
    return e.value.kind


# ---------------------------------------------------------------- construction
def test_new_rejects_empty_replicas():
    with pytest.raises(native.NativeError):
        K.Controller(K.ElasticConfig(1024, 128), [])


def test_new_rejects_all_spares():
    with pytest.raises(native.NativeError):
        K.Controller(K.ElasticConfig(1024, 128), [K.ReplicaSpec("s", "a", True)])


def test_new_rejects_duplicate_replica_id_live_and_spare():
    with pytest.raises(native.NativeError):
        K.Controller(K.ElasticConfig(1024, 128), [K.ReplicaSpec("a", "x"), K.ReplicaSpec("a", "y", True)])


def test_new_rejects_zero_microbatch_tokens():
    with pytest.raises(native.NativeError):
        K.Controller(K.ElasticConfig(1024, 0), [K.ReplicaSpec("a", "x")])


def test_new_accepts_one_live_zero_spare():
    c = K.Controller(K.ElasticConfig(1024, 128), [K.ReplicaSpec("a", "x")])
    assert c.n_live() == 1 and c.grad_accumulation() == 8


def test_initial_live_set_is_non_spares_in_spec_order():
    c = ctl(3, 2)
    assert c.live_replicas() == ["r0", "r1", "r2"]
    assert str(c.replica_state("s0")).endswith("Spare")


def test_four_live_accum_is_two_and_effective_equals_product():
    c = ctl(4)
    assert c.grad_accumulation() == 2 and c.effective_tokens_per_step() == 2 * 4 * 512


def test_uneven_tokens_uses_ceil_accum():
    c = ctl(3, tokens=4097)
    assert c.grad_accumulation() == 3 and c.effective_tokens_per_step() >= 4097


def test_tokens_per_step_zero_accum_zero():
    assert ctl(2, tokens=0).grad_accumulation() == 0


def test_replica_state_unknown_is_not_found():
    assert kind_of(ctl().replica_state, "nope") == "ReplicaNotFound"


# --------------------------------------------------------------------- failing
def test_fail_live_sets_dead_drops_n_live_raises_accum():
    c = ctl(4)
    c.fail_replica("r1")
    assert str(c.replica_state("r1")).endswith("Dead") and c.n_live() == 3 and c.grad_accumulation() == 3


def test_two_fails_raise_accum_to_hold_tokens():
    c = ctl(4)
    c.fail_replica("r0")
    c.fail_replica("r3")
    assert c.grad_accumulation() == 4 and c.effective_tokens_per_step() >= 4096


def test_fail_last_live_is_no_live_replicas_and_does_not_change_state():
    c = ctl(1)
    assert kind_of(c.fail_replica, "r0") == "NoLiveReplicas"
    assert str(c.replica_state("r0")).endswith("Live")


def test_fail_unknown_is_replica_not_found():
    assert kind_of(ctl().fail_replica, "zz") == "ReplicaNotFound"


def test_fail_spare_and_fail_already_dead_are_not_live():
    c = ctl(3, 1)
    assert kind_of(c.fail_replica, "s0") == "NotLive"
    c.fail_replica("r0")
    assert kind_of(c.fail_replica, "r0") == "NotLive"


def test_tokens_invariant_after_each_fail_until_one_left():
    c = ctl(6, tokens=6000, micro=100)
    for i in range(5):
        c.fail_replica(f"r{i}")
        assert c.effective_tokens_per_step() >= 6000
        assert (c.grad_accumulation() - 1) * c.n_live() * 100 < 6000       # the smallest that holds them


# ------------------------------------------------------------------- straggler
def test_step_over_the_timeout_drains_and_at_the_timeout_does_not():
    c = ctl(3, straggler_timeout_ms=100)
    c.observe_step_time("r0", 1, 100)
    assert "r0" in c.live_replicas()
    c.observe_step_time("r0", 2, 101)
    assert "r0" not in c.live_replicas()
    assert kind_of(c.observe_step_time, "r0", 3, 5) == "NotLive"


# ----------------------------------------------------------------- collectives
def test_tick_past_watchdog_without_end_drains():
    c = ctl(3, collective_watchdog_ms=50)
    c.begin_collective("ar", "r1", 1000)
    c.tick(1051)
    assert "r1" not in c.live_replicas() and c.open_collectives() == 0


def test_end_before_deadline_leaves_live():
    c = ctl(3, collective_watchdog_ms=50)
    c.begin_collective("ar", "r1", 1000)
    c.end_collective("ar", "r1", 1020)
    c.tick(5000)
    assert "r1" in c.live_replicas()


def test_elapsed_equal_watchdog_does_not_drain_and_clock_before_begin_is_ignored():
    c = ctl(3, collective_watchdog_ms=50)
    c.begin_collective("ar", "r1", 1000)
    c.tick(1050)
    c.tick(900)
    assert "r1" in c.live_replicas()


def test_tick_with_no_open_collective_and_unmatched_end_are_ok():
    c = ctl(2)
    c.tick(10 ** 9)
    c.end_collective("never-began", "r0", 5)
    assert c.n_live() == 2


def test_begin_unknown_spare_and_duplicate():
    c = ctl(2, 1)
    assert kind_of(c.begin_collective, "ar", "zz", 0) == "ReplicaNotFound"
    assert kind_of(c.begin_collective, "ar", "s0", 0) == "NotLive"
    c.begin_collective("ar", "r0", 0)
    assert kind_of(c.begin_collective, "ar", "r0", 1) == "Message"


def test_one_replica_times_out_other_stays_live():
    c = ctl(3, collective_watchdog_ms=10)
    c.begin_collective("ar", "r0", 0)
    c.begin_collective("ar", "r1", 95)
    c.tick(100)
    assert c.live_replicas() == ["r1", "r2"]


def test_watchdog_of_last_live_is_no_live_replicas_no_change():
    c = ctl(1, collective_watchdog_ms=10)
    c.begin_collective("ar", "r0", 0)
    assert kind_of(c.tick, 100) == "NoLiveReplicas"
    assert c.live_replicas() == ["r0"]


# ---------------------------------------------------------------------- health
@pytest.mark.parametrize("kind", ["Xid", "Ecc", "Nvlink", "NicFlap", "Thermal", "WatchdogTimeout"])
def test_every_health_kind_drains_like_fail_replica(kind):
    c = ctl(3)
    c.report_health(K.HealthEvent("r2", "r2", getattr(K.HealthKind, kind), 7, "x"))
    assert "r2" not in c.live_replicas() and c.health_events() == 1 and c.grad_accumulation() == 4


def test_health_errors():
    c = ctl(1, 1)
    ev = lambda who: K.HealthEvent(who, who, K.HealthKind.Xid)        # noqa: E731
    assert kind_of(c.report_health, ev("zz")) == "ReplicaNotFound"
    assert kind_of(c.report_health, ev("s0")) == "NotLive"
    assert kind_of(c.report_health, ev("r0")) == "NoLiveReplicas"
    assert c.live_replicas() == ["r0"]


# --------------------------------------------------------------------- healing
def test_heal_spare_sets_healing_n_live_unchanged_then_rejoin_lowers_accum():
    c = ctl(3, 1)
    c.fail_replica("r0")
    assert c.grad_accumulation() == 4
    c.heal_spare("s0", "r1")
    assert str(c.replica_state("s0")).endswith("Healing") and c.n_live() == 2 and c.heal_source("s0") == "r1"
    c.offer_weight_copy("s0", "r1", [K.WeightShard("embed", b"abc")])
    c.rejoin("s0", 10)
    assert c.n_live() == 3 and c.grad_accumulation() == 3
    assert [(s.name, bytes(s.bytes)) for s in c.healed_weight_shards("s0")] == [("embed", b"abc")]


def test_heal_errors():
    c = ctl(2, 2)
    assert kind_of(c.heal_spare, "r0", "r1") == "NotSpare"
    assert kind_of(c.heal_spare, "zz", "r1") == "ReplicaNotFound"
    assert kind_of(c.heal_spare, "s0", "zz") == "ReplicaNotFound"
    assert kind_of(c.heal_spare, "s0", "s1") == "NotLive"
    assert kind_of(c.rejoin, "s0", 1) in ("NotSpare", "NoHealInProgress", "NotStepBoundary")
    assert kind_of(c.rejoin, "r0", 1) == "NotSpare"
    c.heal_spare("s0", "r0")
    assert kind_of(c.heal_spare, "s0", "r0") == "NotSpare"
    c.rejoin("s0", 3)
    assert kind_of(c.rejoin, "s0", 4) == "NotSpare"


def test_offer_copies_bytes_and_rejects_bad_shards():
    c = ctl(2, 1)
    assert kind_of(c.offer_weight_copy, "s0", "r0", [K.WeightShard("w", b"1")]) == "NoHealInProgress"
    c.heal_spare("s0", "r0")
    assert kind_of(c.offer_weight_copy, "s0", "r1", [K.WeightShard("w", b"1")]) == "HealSourceMismatch"
    assert kind_of(c.offer_weight_copy, "s0", "r0", [K.WeightShard("", b"1")]) == "EmptyWeightShardName"
    c.offer_weight_copy("s0", "r0", [K.WeightShard("a", b"1"), K.WeightShard("b", b"22")])
    assert kind_of(c.offer_weight_copy, "s0", "r0", [K.WeightShard("a", b"3")]) == "DuplicateWeightShard"
    assert c.n_live() == 2                                   # offering does not change membership
    c.rejoin("s0", 5)
    assert [s.name for s in c.healed_weight_shards("s0")] == ["a", "b"]


# ------------------------------------------------------------------------- SDC
def test_sdc_majority_quarantines_the_offenders_rack_and_reports():
    c = ctl(4, sdc_period_steps=10)
    for r, h in zip(("r0", "r1", "r2", "r3"), ("aa", "aa", "bb", "aa")):
        c.report_shard_hash(r, "w0", h, 10)
    assert kind_of(c.check_sdc, 10) == "HashMismatch"
    assert str(c.replica_state("r2")).endswith("Quarantined") and c.n_live() == 3


def test_sdc_off_period_steps_and_all_equal_are_quiet_and_missing_hash_is_an_error():
    c = ctl(3, sdc_period_steps=10)
    c.check_sdc(7)                                           # not a probe step
    for r in ("r0", "r1", "r2"):
        c.report_shard_hash(r, "w0", "aa", 10)
    c.check_sdc(10)
    assert c.n_live() == 3
    c.report_shard_hash("r0", "w0", "aa", 20)
    assert kind_of(c.check_sdc, 20) == "MissingHash"


def test_sdc_never_quarantines_the_last_live_rack():
    specs = [K.ReplicaSpec("a", "one"), K.ReplicaSpec("b", "one")]
    c = K.Controller(K.ElasticConfig(1024, 128, 5), specs)
    c.report_shard_hash("a", "w", "x", 5)
    c.report_shard_hash("b", "w", "y", 5)
    assert kind_of(c.check_sdc, 5) == "HashMismatch"
    assert c.n_live() == 2


# ---------------------------------------------------------------------- spikes
def test_spike_policy_rolls_back_skips_and_pages_inside_the_window():
    c = ctl(2, page_window_steps=100)
    first = c.on_loss_spike(500, "shard-9", "ckpt-a")
    assert (first.rollback_checkpoint_id, first.skipped_shard, first.page) == ("ckpt-a", "shard-9", False)
    assert c.on_loss_spike(560, "shard-11", "ckpt-b").page and c.pages() == 1
    assert not c.on_loss_spike(800, "shard-12", "ckpt-c").page
    assert c.skipped_shards() == ["shard-9", "shard-11", "shard-12"]
