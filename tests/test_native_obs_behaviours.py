"""Observability behaviour list (names follow the reference's obs/tests/{registry,events,hashes,
metrics,metric_log,tracer,spike,spike_faults,dashboard}.rs), against the C++ module."""
import hashlib
import json
import math
import random

import pytest

from prometheus_b200 import native

O = native.obs


def kind_of(fn, *a, **k):
    with pytest.raises(native.NativeError) as e:
        fn(*a, **k)
    return e.value.kind


# ------------------------------------------------------------------- registry
def test_register_then_get_list_status_and_parent():
    r = O.RunRegistry()
    assert r.list() == []
    r.register(O.RunRecord("a", "pretrain"))
    child = O.RunRecord("b", "rl")
    child.parent_run_id = "a"
    r.register(child)
    assert [x.run_id for x in r.list()] == ["a", "b"] and r.get("b").parent_run_id == "a"
    before = r.get("a")
    r.set_status("a", "completed")
    after = r.get("a")
    assert after.status == "completed" and (after.kind, after.created_at, after.config_hash) == \
        (before.kind, before.created_at, before.config_hash)
    assert [x.status for x in r.list()][0] == "completed"
    assert kind_of(r.get, "zz") == "UnknownRun" and kind_of(r.set_status, "zz", "running") == "UnknownRun"


def test_duplicate_register_errors_and_does_not_replace():
    r = O.RunRegistry()
    r.register(O.RunRecord("a", "pretrain"))
    assert kind_of(r.register, O.RunRecord("a", "other")) == "DuplicateRun"
    assert r.get("a").kind == "pretrain"


# --------------------------------------------------------------------- events
def test_event_chain_genesis_seq_prev_hash_order_and_per_run():
    r = O.RunRegistry()
    r.register(O.RunRecord("a", "k"))
    r.register(O.RunRecord("b", "k"))
    assert r.events("a") == []
    e1 = r.append_event("a", "start", "{}")
    e2 = r.append_event("a", "step", '{"x":1}')
    b1 = r.append_event("b", "start", "{}")
    assert (e1.seq, e1.prev_hash) == (1, O.GENESIS_HASH) and (e2.seq, e2.prev_hash) == (2, e1.hash)
    assert (b1.seq, b1.prev_hash) == (1, O.GENESIS_HASH)
    assert [e.seq for e in r.events("a")] == [1, 2]
    assert "T" in e1.timestamp and e1.timestamp.endswith("Z")
    assert kind_of(r.events, "zz") == "UnknownRun" and kind_of(r.append_event, "zz", "t", "{}") == "UnknownRun"


def test_payload_hash_tracks_payload_not_event_type():
    r = O.RunRegistry()
    r.register(O.RunRecord("a", "k"))
    x = r.append_event("a", "one", '{"v":1}', "t")
    y = r.append_event("a", "two", '{"v":1}', "t")
    z = r.append_event("a", "two", '{"v":2}', "t")
    assert x.payload_hash == y.payload_hash != z.payload_hash


# --------------------------------------------------------------------- hashes
def test_payload_hash_goldens_key_order_and_utf8():
    assert O.payload_hash("{}") == hashlib.sha256(b"{}").hexdigest()
    assert O.payload_hash('{"b":1,"a":2}') == O.payload_hash('{"a":2,"b":1}') == \
        hashlib.sha256(b'{"a":2,"b":1}').hexdigest()
    assert O.payload_hash('{"s":"\\u00e9"}') == hashlib.sha256('{"s":"é"}'.encode()).hexdigest()
    assert O.payload_hash('{"a":1}') != O.payload_hash('{"a":2}')


def test_event_hash_is_pipe_concatenation_with_plain_decimal_seq():
    ph = O.payload_hash("{}")
    h = O.event_hash(12, "p" * 64, ph, "2026-01-01T00:00:00Z", "step")
    assert h == hashlib.sha256(f"12|{'p' * 64}|{ph}|2026-01-01T00:00:00Z|step".encode()).hexdigest()
    assert len(h) == 64 and h == h.lower() and all(c in "0123456789abcdef" for c in h)


# -------------------------------------------------------------------- metrics
def test_metrics_series_kinds_and_labels():
    m = O.Metrics()
    assert m.get("nope") is None
    m.inc("c", {}, 0)
    assert m.get("c") == 0
    m.inc("c", {"a": "1", "b": "2"}, 2)
    m.inc("c", {"b": "2", "a": "1"}, 3)                  # key order does not split a series
    assert m.get("c", {"a": "1", "b": "2"}) == 5 and m.get("c") == 0
    m.set("g", {}, 1.0)
    m.set("g", {}, 4.0)
    assert m.get("g") == 4.0
    m.observe("h", {}, 1.5)
    m.observe("h", {}, 2.5)
    assert m.get("h") == 4.0 and m.count("h") == 2
    assert kind_of(m.set, "c", {"x": "y"}, 1.0) == "KindMismatch"       # the kind is per name
    assert kind_of(m.observe, "g", {}, 1.0) == "KindMismatch"
    assert kind_of(m.inc, "h", {}, 1) == "KindMismatch"


def test_property_independent_names_do_not_interfere():
    rng = random.Random(3)
    m, want = O.Metrics(), {}
    for _ in range(300):
        n = f"n{rng.randrange(8)}"
        v = rng.randrange(5)
        m.inc(n, {}, v)
        want[n] = want.get(n, 0) + v
    assert all(m.get(n) == v for n, v in want.items())


# ----------------------------------------------------------------- metric log
def test_metric_log_series_rules():
    log = O.MetricLog()
    assert kind_of(log.series, "x") == "EmptyHistory"
    log.record("x", {}, 5, 1.0)
    log.record("x", {}, 2, 2.0)
    log.record("x", {}, 5, 3.0)                          # same step: the last write wins
    log.record("x", {"rank": "1"}, 1, 9.0)               # labels, even empty ones, are their own series
    log.record("y", {}, 1, 7.0)
    assert log.series("x") == [(2, 2.0), (5, 3.0)] and log.series("x", {"rank": "1"}) == [(1, 9.0)]
    assert log.series("y") == [(1, 7.0)]
    assert kind_of(log.series, "z") == "UnknownMetric"
    assert kind_of(log.series, "y", {"rank": "1"}) == "UnknownMetric"
    log.record("x", {}, 6, math.nan)                      # non-finite values are accepted
    assert math.isnan(log.series("x")[-1][1])


def test_property_last_write_wins_and_sort():
    rng = random.Random(5)
    log, want = O.MetricLog(), {}
    for _ in range(200):
        s, v = rng.randrange(40), rng.random()
        log.record("m", {}, s, v)
        want[s] = v
    assert log.series("m") == sorted(want.items())


# --------------------------------------------------------------------- tracer
def test_tracer_current_nesting_lifo_and_foreign_spans():
    t, u = O.Tracer(), O.Tracer()
    assert t.current() is None
    t.set_now_ms(0.0)
    a = t.start("a")
    b = t.start("b")
    assert t.current() == "b" and u.current() is None
    assert kind_of(t.end, a) == "Other"                  # LIFO only
    with pytest.raises(native.NativeError):
        u.end(b)                                          # a span of another tracer
    t.set_now_ms(12.0)
    assert t.end(b) == 12.0 and t.current() == "a"
    # a span that is dropped without end() stays on the stack under later ones
    c = t.start("c")
    del c
    assert t.current() == "c" and t.depth() == 2


# ---------------------------------------------------------------------- spikes
def _log(**kw):
    kw = {"page_window_steps": 10, "relative_threshold": 0.5, "baseline_window": 3,
          "last_checkpoint_step": 7, **kw}
    return O.SpikeLog(**kw)


def test_warmup_sliding_window_and_nonpositive_baseline():
    s = _log()
    assert s.spikes() == [] and s.skipped_shards() == []
    assert [s.observe(i, v, "sh", "r") for i, v in enumerate([1.0, 1e9, 1.0])] == [[], [], []]
    # window of 3 slides: the baseline for the 4th sample is the mean of the last three
    acts = s.observe(3, 1e12, "sh", "r")
    assert acts and acts[0].event.baseline == pytest.approx((1.0 + 1e9 + 1.0) / 3)
    z = _log()
    for i in range(3):
        z.observe(i, 0.0, "sh", "r")
    assert z.observe(3, 100.0, "sh", "r") == []           # a zero baseline never spikes


def test_page_window_is_inclusive_and_uses_any_prior_spike():
    s = _log(baseline_window=1, page_window_steps=10)
    s.observe(0, 1.0, "a", "r")
    first = s.observe(1, 10.0, "a", "r")
    assert [a.kind for a in first] == ["log", "skip_shard", "rollback"] and first[2].checkpoint_step == 7
    s.observe(2, 1.0, "a", "r")
    assert [a.kind for a in s.observe(11, 10.0, "b", "r")][-1] == "page"          # 11 - 1 == window
    s.observe(12, 1.0, "a", "r")
    assert [a.kind for a in s.observe(22, 10.0, "c", "r")][-1] != "page"          # 22 - 11 > window
    assert len(s.spikes()) == len(s.skipped_shards()) == 3


def test_window_one_baseline_is_the_previous_sample_and_constant_loss_never_spikes():
    s = _log(baseline_window=1)
    s.observe(0, 2.0, "a", "r")
    acts = s.observe(1, 4.0, "a", "r")
    assert acts[0].event.baseline == 2.0
    c = _log()
    assert all(c.observe(i, 3.0, "a", "r") == [] for i in range(50))


def test_bad_spike_config_and_non_finite_losses():
    assert kind_of(_log(relative_threshold=0.0).observe, 0, 1.0, "a", "r") == "BadSpikeConfig"
    assert kind_of(_log(relative_threshold=-1.0).observe, 0, 1.0, "a", "r") == "BadSpikeConfig"
    assert kind_of(_log(baseline_window=0).observe, 0, 1.0, "a", "r") == "BadSpikeConfig"
    s = _log(baseline_window=2)
    s.observe(0, 1.0, "a", "r")
    for bad in (math.nan, math.inf, -math.inf):
        assert kind_of(s.observe, 1, bad, "a", "r") == "BadSpikeConfig"
    # the bad samples took no warm-up slot: one more finite sample completes the window
    assert s.observe(1, 1.0, "a", "r") == [] and s.observe(2, 10.0, "a", "r") != []
    assert len(s.spikes()) == 1


# ------------------------------------------------------------------ dashboard
def test_snapshot_panels_order_points_and_errors():
    log = O.MetricLog()
    empty = json.loads(O.snapshot(O.Dashboard("d", "t", []), log, [], "now"))
    assert empty["panels"] == []
    assert kind_of(O.snapshot, O.Dashboard("d", "t", [O.Panel("p", "x", "m")]), log, [], "now") == "EmptyHistory"
    table = json.loads(O.snapshot(O.Dashboard("d", "t", [O.Panel("p", "x", "m", "table")]), log, [], "now"))
    assert table["panels"][0]["points"] == []
    log.record("m", {}, 1, 1.0)
    log.record("m", {"rank": "0"}, 2, 5.0)                # labelled series are not read by a snapshot
    dash = O.Dashboard("d", "t", [O.Panel("a", "x", "m"), O.Panel("b", "x", "", "table"),
                                  O.Panel("c", "x", "m", "gauge")])
    snap = json.loads(O.snapshot(dash, log, [], "now"))
    assert [p["panel_id"] if "panel_id" in p else p.get("id") for p in snap["panels"]] == ["a", "b", "c"]
    assert snap["panels"][0]["points"] == [{"step": 1, "value": 1.0}] == snap["panels"][2]["points"]
    assert json.loads(json.dumps(snap)) == snap
