"""Behaviour list of the multi-agent bookkeeping (C++ ``native.multiagent``): configuration
checks and their order, the topology CDF, rosters, spawn validation order, the shared scratch
pad, private inboxes with latent-memo dropout, credit records, the token budget and the
distillation gate (reference rl/multiagent/tests/{new,topology,roster,spawn,scratch,messages,
credit,tokens,distill,properties}.rs)."""
import math

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

MA = native.multiagent
T = list(MA.TOPOLOGIES)
SINGLE, ORCH, PAR, PROP, AUTH = "single", "orchestrator_subs", "parallel_aggregate", "proposer_solver", "author_reviewer"


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def spawned(topology=ORCH, n_subs=2, budget=100, **cfg):
    m = MA.Multiagent(MA.MultiConfig(**cfg)) if cfg else MA.Multiagent()
    return m, m.spawn_episode("e1", "task", topology, n_subs, budget)


# ------------------------------------------------------------------------------ configuration
def test_topology_names_and_production_weights():
    assert T == [SINGLE, ORCH, PAR, PROP, AUTH] and MA.MAX_N_SUBS == 99
    assert [MA.topology_weight(t) for t in T] == [50, 20, 15, 10, 5]
    MA.Multiagent(MA.MultiConfig())                                  # the defaults are valid


@pytest.mark.parametrize("kw", [
    dict(weights=[50, 20, 15, 10, 4]),                               # sums to 99
    dict(weights=[50, 20, 15, 10, 6]),                               # 101
    dict(weights=[2 ** 32 - 1, 1, 50, 50, 0]),                       # wraps in 32 bits: still not 100
    dict(weights=[49, 21, 15, 10, 5]),                               # single below its floor
    dict(latent_keep_denom=0, latent_keep_numer=0),
    dict(latent_keep_denom=0, latent_keep_numer=5),
    dict(latent_keep_numer=101, latent_keep_denom=100),
    dict(default_n_subs=0),
    dict(default_n_subs=100),
])
def test_bad_configurations_are_bad_mix(kw):
    assert err(lambda: MA.Multiagent(MA.MultiConfig(**kw))).kind == "BadMix"


@pytest.mark.parametrize("kw", [
    dict(weights=[50, 50, 0, 0, 0]), dict(weights=[100, 0, 0, 0, 0]), dict(weights=[60, 0, 40, 0, 0]),
    dict(weights=[51, 19, 15, 10, 5]), dict(latent_keep_numer=100, latent_keep_denom=100),
    dict(latent_keep_numer=0, latent_keep_denom=7), dict(default_n_subs=1), dict(default_n_subs=99),
])
def test_edge_configurations_are_accepted(kw):
    MA.Multiagent(MA.MultiConfig(**kw))


# ------------------------------------------------------------------------------ topology draws
def test_production_cdf_boundaries_wrap_and_histogram():
    bounds = {0: SINGLE, 49: SINGLE, 50: ORCH, 69: ORCH, 70: PAR, 84: PAR, 85: PROP, 94: PROP, 95: AUTH, 99: AUTH}
    for d, want in bounds.items():
        assert MA.topology_from_draw(d) == want
        assert MA.topology_from_draw(d + 100) == want and MA.topology_from_draw(d + 10 ** 9 * 100) == want
    draws = [MA.topology_from_draw(d) for d in range(10000)]
    assert [draws.count(t) for t in T] == [5000, 2000, 1500, 1000, 500]


def test_instance_mix_drives_sample_topology_only():
    m = MA.Multiagent(MA.MultiConfig(weights=[60, 0, 40, 0, 0]))
    got = [m.sample_topology(d) for d in range(10000)]
    assert [got.count(t) for t in T] == [6000, 0, 4000, 0, 0]       # zero-weight buckets are skipped
    assert m.sample_topology(59) == SINGLE and m.sample_topology(60) == PAR and m.sample_topology(160) == PAR
    assert MA.topology_from_draw(60) == ORCH                        # the free function ignores the instance
    d = MA.Multiagent()
    assert [d.sample_topology(x) for x in range(100)] == [MA.topology_from_draw(x) for x in range(100)]
    both = MA.Multiagent(MA.MultiConfig(weights=[50, 50, 0, 0, 0]))
    assert {both.sample_topology(x) for x in range(100)} == {SINGLE, ORCH}
    assert err(lambda: both.topology_of("nobody")).kind == "UnknownEpisode"      # sampling created nothing


# ------------------------------------------------------------------------------ rosters
def test_rosters_of_every_topology():
    assert MA.roster(SINGLE, 0) == [("solo", "solo")]
    assert MA.roster(ORCH, 2) == [("orchestrator", "orchestrator"), ("sub-00", "sub_agent"), ("sub-01", "sub_agent")]
    assert MA.roster(ORCH, 10)[-1][0] == "sub-09" and MA.roster(ORCH, 99)[-1][0] == "sub-98"
    assert len(MA.roster(ORCH, 99)) == 100
    assert MA.roster(PAR, 1) == [("attempt-00", "attempt"), ("aggregator", "aggregator")]
    assert MA.roster(PAR, 10)[-2][0] == "attempt-09" and MA.roster(PAR, 10)[-1][0] == "aggregator"
    assert MA.roster(PROP, 0) == [("proposer", "proposer"), ("solver", "solver")]
    assert MA.roster(AUTH, 0) == [("author", "author"), ("reviewer", "reviewer")]
    for aid, _role in MA.roster(ORCH, 3) + MA.roster(PAR, 3):
        assert aid.isascii() and "‐" not in aid and " " not in aid


@pytest.mark.parametrize("topology, n", [(SINGLE, 1), (PROP, 1), (AUTH, 2), (ORCH, 0), (ORCH, 100), (PAR, 0), (PAR, 100)])
def test_bad_widths(topology, n):
    assert err(lambda: MA.roster(topology, n)).kind == "BadWidth"


# ------------------------------------------------------------------------------ spawn
def test_spawn_returns_the_roster_and_an_empty_state():
    m = MA.Multiagent(MA.MultiConfig(default_n_subs=5))
    ros = m.spawn_episode("e", "t", ORCH, 3, 10)                     # the call's width, not the default
    assert [a for a, _ in ros] == ["orchestrator", "sub-00", "sub-01", "sub-02"] and m.agents("e") == ros
    assert m.topology_of("e") == ORCH and m.scratch_read("e") == "" and m.credit("e") == [] and m.tokens_used("e") == 0
    for a, _ in ros:
        assert m.inbox("e", a) == [] and m.tokens_used_by("e", a) == 0
    for i, (t, n) in enumerate([(SINGLE, 0), (PAR, 2), (PROP, 0), (AUTH, 0)]):
        assert m.spawn_episode(f"x{i}", "t", t, n, 1) == MA.roster(t, n)


def test_spawn_validation_order():
    m = MA.Multiagent()
    assert err(lambda: m.spawn_episode("", "", SINGLE, 5, 0)).kind == "EmptyId"        # episode id first of all
    assert err(lambda: m.spawn_episode("e", "", SINGLE, 0, 1)).kind == "EmptyId"
    m.spawn_episode("e", "t", SINGLE, 0, 1)
    assert err(lambda: m.spawn_episode("e", "", SINGLE, 0, 1)).kind == "EmptyId"       # empty task before duplicate
    assert err(lambda: m.spawn_episode("e", "t", SINGLE, 7, 0)).kind == "DuplicateEpisode"
    assert err(lambda: m.spawn_episode("f", "t", SINGLE, 7, 0)).kind == "BadWidth"     # width before budget
    e = err(lambda: m.spawn_episode("f", "t", SINGLE, 0, 0))
    assert e.kind == "Message" and "budget" in str(e).lower()
    assert err(lambda: m.topology_of("f")).kind == "UnknownEpisode"                    # failed spawns create nothing
    m.spawn_episode("E", "t", PROP, 0, 1)                                              # ids are case-sensitive
    assert m.topology_of("E") == PROP and m.topology_of("e") == SINGLE


def test_every_keyed_method_names_an_unknown_episode_first():
    m = MA.Multiagent()
    m.spawn_episode("other", "t", SINGLE, 0, 5)
    calls = [lambda: m.agents("nope"), lambda: m.topology_of("nope"), lambda: m.scratch_read("nope"),
             lambda: m.scratch_append("nope", "ghost", "x"), lambda: m.inbox("nope", "ghost"),
             lambda: m.send_message("nope", MA.Message("ghost", "ghost", "x"), 0),
             lambda: m.record_credit("nope", "ghost", ["ghost"]), lambda: m.credit("nope"),
             lambda: m.charge_tokens("nope", "ghost", 0), lambda: m.tokens_used("nope"),
             lambda: m.tokens_used_by("nope", "ghost")]
    for call in calls:
        assert err(call).kind == "UnknownEpisode"


# ------------------------------------------------------------------------------ scratch pad
def test_scratch_is_one_shared_string_in_call_order():
    m, _ = spawned()
    m.scratch_append("e1", "sub-00", "a")
    m.scratch_append("e1", "orchestrator", "")
    m.scratch_append("e1", "sub-01", "b")
    m.scratch_append("e1", "sub-00", "c")
    assert m.scratch_read("e1") == "abc"                             # no separator, empty text allowed
    for ghost in ("Sub-00", "solo", "ghost"):                       # case-sensitive; another topology's id
        assert err(lambda: m.scratch_append("e1", ghost, "")).kind == "UnknownAgent"
    m.spawn_episode("e2", "t", SINGLE, 0, 5)
    m.scratch_append("e2", "solo", "z")
    assert m.scratch_read("e1") == "abc" and m.scratch_read("e2") == "z"


# ------------------------------------------------------------------------------ messages
def test_inboxes_are_private_and_fifo():
    m, _ = spawned()
    for text in ("one", "", "three"):
        m.send_message("e1", MA.Message("orchestrator", "sub-00", text), 0)
    m.send_message("e1", MA.Message("sub-00", "sub-00", "self"), 0)
    assert [x.text for x in m.inbox("e1", "sub-00")] == ["one", "", "three", "self"]
    assert m.inbox("e1", "sub-01") == [] and m.inbox("e1", "orchestrator") == []     # the sender keeps no copy
    assert err(lambda: m.inbox("e1", "ghost")).kind == "UnknownAgent"
    m.spawn_episode("e2", "t", ORCH, 2, 5)
    assert m.inbox("e2", "sub-00") == []                                              # no crossing between episodes


def test_message_validation_order_and_no_delivery_on_failure():
    m, _ = spawned(budget=1)
    e = err(lambda: m.send_message("e1", MA.Message("ghost-a", "ghost-b", "x"), 0))
    assert e.kind == "UnknownAgent" and "ghost-a" in str(e)
    e = err(lambda: m.send_message("e1", MA.Message("orchestrator", "ghost-b", "x"), 0))
    assert e.kind == "UnknownAgent" and "ghost-b" in str(e)
    assert err(lambda: m.send_message("e1", MA.Message("ghost", "sub-00", "x"), 0)).kind == "UnknownAgent"
    assert m.inbox("e1", "sub-00") == []
    m.charge_tokens("e1", "sub-00", 1)
    m.send_message("e1", MA.Message("sub-00", "sub-01", "still fine"), 0)             # the budget is not consulted
    assert len(m.inbox("e1", "sub-01")) == 1


def test_latent_memo_dropout_uses_the_instance_ratio():
    m, _ = spawned(latent_keep_numer=3, latent_keep_denom=10)
    memo = [0.25, -1.5]
    for draw, kept in ((0, True), (2, True), (3, False), (9, False), (12, True), (13, False)):
        got = m.send_message("e1", MA.Message("orchestrator", "sub-00", "m", memo), draw)
        assert (got.latent_memo == memo) if kept else (got.latent_memo is None)
        tail = m.inbox("e1", "sub-00")[-1]
        assert tail.latent_memo == got.latent_memo and tail.text == "m" and tail.sender == "orchestrator"
    for draw in (0, 5, 99):                                          # nothing to keep: stays None
        assert m.send_message("e1", MA.Message("orchestrator", "sub-01", "n"), draw).latent_memo is None
    always, _ = spawned(latent_keep_numer=7, latent_keep_denom=7)
    never, _ = spawned(latent_keep_numer=0, latent_keep_denom=7)
    for draw in range(20):
        assert always.send_message("e1", MA.Message("orchestrator", "sub-00", "", memo), draw).latent_memo == memo
        assert never.send_message("e1", MA.Message("orchestrator", "sub-00", "", memo), draw).latent_memo is None


# ------------------------------------------------------------------------------ credit
def test_credit_records_append_as_given():
    m, _ = spawned()
    assert m.credit("e1") == []
    m.record_credit("e1", "orchestrator", [])
    m.record_credit("e1", "orchestrator", ["sub-00", "sub-00", "orchestrator"])      # duplicates and the parent itself
    m.record_credit("e1", "sub-01", ["sub-00"])
    assert m.credit("e1") == [("orchestrator", []), ("orchestrator", ["sub-00", "sub-00", "orchestrator"]), ("sub-01", ["sub-00"])]
    e = err(lambda: m.record_credit("e1", "ghost", ["also-ghost"]))
    assert e.kind == "UnknownAgent" and "ghost" in str(e) and "also" not in str(e)   # parent before used
    e = err(lambda: m.record_credit("e1", "orchestrator", ["sub-00", "g1", "g2"]))
    assert e.kind == "UnknownAgent" and "g1" in str(e)                                # first unknown in order
    m.spawn_episode("e2", "t", SINGLE, 0, 5)
    assert err(lambda: m.record_credit("e1", "solo", [])).kind == "UnknownAgent"      # another episode's agent
    assert m.credit("e2") == [] and len(m.credit("e1")) == 3


# ------------------------------------------------------------------------------ tokens
def test_token_budget_is_per_episode_and_exact():
    m, _ = spawned(budget=100)
    assert m.charge_tokens("e1", "sub-00", 0) == 0 and m.tokens_used("e1") == 0
    assert m.charge_tokens("e1", "sub-00", 60) == 60
    assert m.charge_tokens("e1", "sub-01", 40) == 100                # returns the episode total; equal is allowed
    assert m.charge_tokens("e1", "orchestrator", 0) == 100           # nothing at the limit is fine
    assert err(lambda: m.charge_tokens("e1", "orchestrator", 1)).kind == "BudgetExceeded"
    assert (m.tokens_used("e1"), m.tokens_used_by("e1", "sub-00"), m.tokens_used_by("e1", "sub-01"),
            m.tokens_used_by("e1", "orchestrator")) == (100, 60, 40, 0)
    assert err(lambda: m.charge_tokens("e1", "ghost", 0)).kind == "UnknownAgent"
    assert err(lambda: m.tokens_used_by("e1", "ghost")).kind == "UnknownAgent"
    fresh, _ = spawned(budget=5)
    assert err(lambda: fresh.charge_tokens("e1", "sub-00", 6)).kind == "BudgetExceeded" and fresh.tokens_used("e1") == 0
    big, _ = spawned(budget=2 ** 64 - 1)
    big.charge_tokens("e1", "sub-00", 2 ** 63)
    assert err(lambda: big.charge_tokens("e1", "sub-00", 2 ** 63)).kind == "BudgetExceeded"    # the sum wraps
    assert big.tokens_used("e1") == 2 ** 63
    m.spawn_episode("e2", "t", ORCH, 2, 10)
    assert m.tokens_used("e2") == 0 and m.charge_tokens("e2", "sub-00", 10) == 10


# ------------------------------------------------------------------------------ distillation gate
def test_distill_back_only_on_a_strict_win():
    m = MA.Multiagent()                                              # no episode needed, nothing mutated
    assert m.distill_back("task", 123, 0.9, 0.5) == ("task", 123)
    assert m.distill_back("task", 123, 0.5, 0.5) is None and m.distill_back("task", 123, 0.4, 0.5) is None
    assert m.distill_back("task", 1, -0.5, -1.0) == ("task", 1) and m.distill_back("task", 1, -1.0, -0.5) is None
    assert m.distill_back("task", 1, 0.0, -0.0) is None and m.distill_back("task", 1, -0.0, 0.0) is None
    assert m.distill_back("t", 1, math.nextafter(0.5, 1.0), 0.5) == ("t", 1)
    for multi, single in ((math.nan, 0.0), (0.0, math.nan), (math.inf, 0.0), (0.0, -math.inf), (math.nan, math.nan)):
        assert err(lambda: m.distill_back("t", 1, multi, single)).kind == "InvalidReward"
    assert err(lambda: m.topology_of("task")).kind == "UnknownEpisode"
