"""Behaviour list of the serving-fork rules (``prometheus_b200.fork``; reference
tests/test_sglang_fork.py and sglang-fork/__init__.py): recurrence buckets under a budget,
latent chunk bounds, the decode-mode truth table, the KV tier ladder, routing capture for
replay, prefix groups of sub-agents and test-time-training hooks."""
import dataclasses
import itertools

import pytest

from prometheus_b200 import fork as F


def test_constants_and_enums():
    assert F.RECURRENCE_BUCKETS == (1, 2, 4, 8, 16) and F.RECURRENCE_MAX == 16
    assert (F.LATENT_CHUNK_MIN, F.LATENT_CHUNK_MAX, F.SUBAGENT_DEPTH_MAX) == (4, 64, 3)
    assert [t.value for t in F.KV_TIER_ORDER] == ["hbm", "grace", "nvme", "distributed"] == [t.value for t in F.KvTier]
    assert [m.value for m in F.DecodeMode] == ["verbal", "latent"] and str(F.DecodeMode.LATENT) == "latent"
    assert issubclass(F.ForkError, ValueError)
    plan, chunk = F.bucket_recurrence(3, 16), F.validate_latent_chunk(8)
    assert plan.kv_shared is True and chunk.mode is F.DecodeMode.LATENT
    for obj in (plan, chunk, F.capture_routing(0, 0, (1,), 1), F.schedule_prefix_group("p", ("c",), 1), F.register_ttt("t", "l")):
        with pytest.raises(dataclasses.FrozenInstanceError):
            setattr(obj, dataclasses.fields(obj)[0].name, None)


@pytest.mark.parametrize("r, budget, want", [(3, 16, 4), (1, 16, 1), (16, 8, 8), (5, 4, 4), (2, 16, 2), (4, 16, 4), (7, 16, 8),
                                             (9, 16, 16), (8, 8, 8), (16, 16, 16), (16, 1, 1), (1, 1, 1), (6, 5, 5), (20, 16, 16),
                                             (4, 32, 4), (100, 100, 16), (17, 3, 3)])
def test_recurrence_rounds_up_to_a_bucket_then_caps(r, budget, want):
    plan = F.bucket_recurrence(r, budget)
    assert (plan.r, plan.budget, plan.kv_shared) == (want, budget, True) and isinstance(plan.r, int)


def test_recurrence_rule_on_a_grid():
    for r, budget in itertools.product(range(1, 40), range(1, 40)):
        up = next((b for b in (1, 2, 4, 8, 16) if b >= r), 16)
        got = F.bucket_recurrence(r, budget).r
        assert got == min(up, budget, 16) and 1 <= got <= min(budget, 16)
        if r in (1, 2, 4, 8, 16) and budget >= r:
            assert got == r                                                             # exact buckets stay
    for r, budget in ((0, 16), (-1, 16), (-16, 16), (4, 0), (4, -1), (4, -8), (0, 0), (-1, -1)):
        with pytest.raises(F.ForkError):
            F.bucket_recurrence(r, budget)


def test_latent_chunk_bounds():
    for n in (4, 5, 32, 63, 64):
        assert F.validate_latent_chunk(n) == F.LatentChunk(n, F.DecodeMode.LATENT)
    for n in (3, 0, -4, 65, 1000):
        with pytest.raises(F.ForkError):
            F.validate_latent_chunk(n)
    for n in range(-5, 80):
        ok = 4 <= n <= 64
        try:
            F.validate_latent_chunk(n)
            assert ok
        except F.ForkError:
            assert not ok


@pytest.mark.parametrize("in_think, halt, want", [(True, False, "latent"), (True, True, "verbal"), (False, False, "verbal"), (False, True, "verbal")])
def test_decode_mode_truth_table(in_think, halt, want):
    assert F.decode_mode(in_think, halt).value == want


def test_kv_tiers_walk_colder_and_waiting_sessions_go_one_step():
    assert F.next_kv_tier(F.KvTier.HBM) is F.KvTier.GRACE and F.next_kv_tier(F.KvTier.GRACE) is F.KvTier.NVME
    assert F.next_kv_tier(F.KvTier.NVME) is F.KvTier.DISTRIBUTED and F.next_kv_tier(F.KvTier.DISTRIBUTED) is None
    assert F.next_kv_tier("hbm") is F.KvTier.GRACE
    with pytest.raises(F.ForkError):
        F.next_kv_tier("tape")
    seen, t = [], F.KvTier.HBM
    while t is not None:
        seen.append(t)
        t = F.next_kv_tier(t)
    assert tuple(seen) == F.KV_TIER_ORDER
    assert F.swap_waiting_session(True) is F.KvTier.HBM and F.swap_waiting_session(False) is F.KvTier.GRACE
    assert {F.swap_waiting_session(d) for d in (True, False)}.isdisjoint({F.KvTier.NVME, F.KvTier.DISTRIBUTED})


def test_routing_capture():
    rec = F.capture_routing(7, 3, [5, 0, 9], 3)
    assert rec == F.RoutingRecord(7, 3, (5, 0, 9)) and isinstance(rec.expert_ids, tuple)      # order kept, zero is an id
    assert F.capture_routing(0, 0, (4,), 1).expert_ids == (4,)
    bad = [((1, 1), 2), ((1, -1), 2), ((-3,), 1), ((1, 2, 3), 2), ((1,), 2), ((), 0), ((1,), 0), ((1,), -1), ((), 1)]
    for ids, top_k in bad:
        with pytest.raises(F.ForkError):
            F.capture_routing(0, 0, ids, top_k)
    for ids in itertools.permutations(range(4), 3):
        assert F.capture_routing(1, 2, ids, 3).expert_ids == ids


def test_prefix_groups():
    g = F.schedule_prefix_group("parent", ["c2", "c1", "c3"], 2)
    assert g == F.PrefixGroup("parent", ("c2", "c1", "c3"), 2)                            # child order kept
    for depth in (1, 2, 3):
        assert F.schedule_prefix_group("p", ("c",), depth).depth == depth
    bad = [("", ("c",), 1), ("p", (), 1), ("p", ("a", "p"), 1), ("p", ("c",), 0), ("p", ("c",), 4), ("p", ("c",), -1), ("p", ("c",), 100)]
    for parent, kids, depth in bad:
        with pytest.raises(F.ForkError):
            F.schedule_prefix_group(parent, kids, depth)


def test_ttt_hooks():
    assert F.register_ttt("task-1", "lora-9") == F.TttHook("task-1", "lora-9")
    for t, l in (("", "l"), ("t", ""), ("", "")):
        with pytest.raises(F.ForkError):
            F.register_ttt(t, l)
