"""C++ controller (elastic DP, SDC vote, watchdog, spike policy, rungs, scaling fit) and
observability. All failures are injected on the host with an injected clock."""
import hashlib
import json
import math

import pytest

from prometheus_b200 import native

K = native.control
O = native.obs


def _ctl(n=4, spares=1, **kw):
    cfg = K.ElasticConfig(tokens_per_step=4096, microbatch_tokens=256, sdc_period_steps=10,
                          straggler_timeout_ms=1000, collective_watchdog_ms=500, **kw)
    specs = [K.ReplicaSpec(f"r{i}", f"rack{i // 2}") for i in range(n)]
    specs += [K.ReplicaSpec(f"s{i}", "rack9", spare=True) for i in range(spares)]
    return K.Controller(cfg, specs)


def test_grad_accumulation_grows_when_replicas_drop():
    c = _ctl()
    assert c.n_live() == 4 and c.grad_accumulation() == 4 and c.effective_tokens_per_step() == 4096
    c.fail_replica("r3")
    assert c.grad_accumulation() == 6 and c.effective_tokens_per_step() == 3 * 256 * 6
    assert c.replica_state("r3") == K.ReplicaState.Dead
    with pytest.raises(native.NativeError) as e:
        c.fail_replica("r3")
    assert e.value.kind == "NotLive"
    with pytest.raises(native.NativeError) as e:
        c.fail_replica("nope")
    assert e.value.kind == "ReplicaNotFound"
    c.fail_replica("r2")
    c.fail_replica("r1")
    with pytest.raises(native.NativeError) as e:
        c.fail_replica("r0")
    assert e.value.kind == "NoLiveReplicas"


def test_straggler_health_and_watchdog_drain():
    c = _ctl()
    c.observe_step_time("r0", 1, 900)
    assert c.n_live() == 4
    c.observe_step_time("r0", 2, 1001)
    assert c.replica_state("r0") == K.ReplicaState.Dead
    c.report_health(K.HealthEvent("r1", "rank3", K.HealthKind.Xid, 5, "xid 79"))
    assert c.live_replicas() == ["r2", "r3"] and c.health_events() == 1
    c.begin_collective("allreduce", "r2", 1000)
    c.begin_collective("allreduce", "r3", 1000)
    with pytest.raises(native.NativeError):
        c.begin_collective("allreduce", "r2", 1001)
    c.end_collective("allreduce", "r3", 1100)
    c.tick(1400)
    assert c.n_live() == 2
    c.tick(1501)           # r2's collective has been open for more than 500 ms
    assert c.live_replicas() == ["r3"] and c.open_collectives() == 0


def test_spare_healing_installs_weights_at_step_boundary():
    c = _ctl()
    with pytest.raises(native.NativeError) as e:
        c.heal_spare("r0", "r1")
    assert e.value.kind == "NotSpare"
    c.heal_spare("s0", "r1")
    assert c.replica_state("s0") == K.ReplicaState.Healing and c.heal_source("s0") == "r1"
    with pytest.raises(native.NativeError) as e:
        c.offer_weight_copy("s0", "r2", [K.WeightShard("w", b"x")])
    assert e.value.kind == "HealSourceMismatch"
    c.offer_weight_copy("s0", "r1", [K.WeightShard("embed", b"abc")])
    with pytest.raises(native.NativeError) as e:
        c.offer_weight_copy("s0", "r1", [K.WeightShard("embed", b"zzz")])
    assert e.value.kind == "DuplicateWeightShard"
    with pytest.raises(native.NativeError) as e:
        c.healed_weight_shards("s0")
    assert e.value.kind == "WeightCopyNotInstalled"
    c.rejoin("s0", 100)
    assert c.n_live() == 5 and c.grad_accumulation() == 4
    assert [(s.name, s.bytes) for s in c.healed_weight_shards("s0")] == [("embed", b"abc")]


def test_sdc_majority_vote_quarantines_the_rack():
    c = _ctl()
    for r in ("r0", "r1", "r2", "r3"):
        c.report_shard_hash(r, "layers.0", "aa" if r != "r2" else "bb", 10)
    c.check_sdc(7)          # not a check step
    with pytest.raises(native.NativeError) as e:
        c.check_sdc(10)
    assert e.value.kind == "HashMismatch" and "r2" in str(e.value)
    assert c.replica_state("r2") == K.ReplicaState.Quarantined
    assert c.replica_state("r3") == K.ReplicaState.Quarantined      # same rack
    assert c.live_replicas() == ["r0", "r1"]
    with pytest.raises(native.NativeError) as e:
        c.report_shard_hash("r2", "layers.0", "aa", 20)
    assert e.value.kind == "Quarantined"
    c.report_shard_hash("r0", "layers.0", "aa", 20)
    with pytest.raises(native.NativeError) as e:
        c.check_sdc(20)
    assert e.value.kind == "MissingHash"


def test_loss_spike_policy_pages_inside_window():
    c = _ctl(page_window_steps=100)
    a = c.on_loss_spike(500, "shard-7", "ckpt-400")
    assert (a.rollback_checkpoint_id, a.skipped_shard, a.page) == ("ckpt-400", "shard-7", False)
    assert c.on_loss_spike(550, "shard-9", "ckpt-500").page is True
    assert c.on_loss_spike(700, "shard-1", "ckpt-600").page is False
    assert c.skipped_shards() == ["shard-7", "shard-9", "shard-1"] and c.pages() == 1


def test_rung_run_checkpoint_resume():
    spec = K.rung_0_spec()
    cfg = K.RungConfig(spec, token_budget=1000, tokens_per_step=300, tokenizer_hash="t", seed=3)
    run = K.RungRun(cfg)
    reports = [run.step(2.0 - 0.1 * i) for i in range(3)]
    assert [r.tokens_seen for r in reports] == [300, 600, 900] and not run.done()
    ck = run.checkpoint()
    resumed = K.RungRun.resume(cfg, ck)
    last = resumed.step(1.5)
    assert last.tokens_seen == 1000 and last.done and resumed.remaining_tokens() == 0
    with pytest.raises(native.NativeError) as e:
        resumed.step(1.0)
    assert e.value.kind == "AlreadyDone"
    with pytest.raises(native.NativeError) as e:
        K.RungRun.resume(K.RungConfig(spec, 1000, 300, "other", 3), ck)
    assert e.value.kind == "TokenizerChanged"
    with pytest.raises(native.NativeError) as e:
        K.RungRun(K.RungConfig(K.rung_spec(1), 1000, 300, "t", 3))
    assert e.value.kind == "NotRung0"
    with pytest.raises(native.NativeError) as e:
        run.step(float("nan"))
    assert e.value.kind == "NonFiniteLoss"


def test_scaling_fit_recovers_power_law():
    a, alpha = 50.0, 0.05
    obs = []
    for i in (1, 2, 3):
        s = K.rung_spec(i)
        c = 6.0 * s.active_params * s.tokens
        obs.append(K.RungObservation(s, a * c ** (-alpha)))
    f = K.fit(obs)
    assert f.a == pytest.approx(a, rel=1e-6) and f.alpha == pytest.approx(alpha, rel=1e-6)
    pred = f.predict_flagship()
    assert pred == pytest.approx(a * (6.0 * 4e11 * 1.8e14) ** (-alpha), rel=1e-6)
    assert K.should_stop(1.0, 1.05) and not K.should_stop(1.0, 1.049)
    with pytest.raises(native.NativeError) as e:
        K.fit(obs[:1])
    assert e.value.kind == "NeedTwoRungs"
    with pytest.raises(native.NativeError) as e:
        K.fit([K.RungObservation(K.rung_spec(0), 1.0), obs[0]])
    assert e.value.kind == "Rung0NotUsed"
    held = K.predict_held_out(obs[:2], K.rung_spec(3))
    assert held == pytest.approx(a * (6.0 * 4e10 * 6e12) ** (-alpha), rel=1e-6)


# ----------------------------------------------------------------------- obs
def test_metrics_kinds_and_values():
    m = O.Metrics()
    m.inc("steps", {"job": "a"}, 1)
    m.inc("steps", {"job": "a"}, 2)
    m.set("lr", {}, 0.1)
    m.observe("latency", {}, 5.0)
    m.observe("latency", {}, 7.0)
    assert m.get("steps", {"job": "a"}) == 3 and m.get("lr") == 0.1
    assert m.get("latency") == 12.0 and m.count("latency") == 2 and m.get("nope") is None
    with pytest.raises(native.NativeError) as e:
        m.set("steps", {}, 1.0)
    assert e.value.kind == "KindMismatch"


def test_tracer_is_lifo_with_injected_clock():
    t = O.Tracer()
    t.set_now_ms(100.0)
    outer = t.start("step")
    inner = t.start("forward")
    assert t.current() == "forward" and t.depth() == 2
    with pytest.raises(native.NativeError):
        t.end(outer)
    t.set_now_ms(130.0)
    assert t.end(inner) == 30.0
    t.set_now_ms(150.0)
    assert t.end(outer) == 50.0 and t.current() is None


def test_run_registry_hash_chain():
    r = O.RunRegistry()
    r.register(O.RunRecord("run1", "pretrain"))
    with pytest.raises(native.NativeError) as e:
        r.register(O.RunRecord("run1", "pretrain"))
    assert e.value.kind == "DuplicateRun"
    e1 = r.append_event("run1", "start", json.dumps({"b": 1, "a": [1, 2]}), "2026-01-01T00:00:00Z")
    e2 = r.append_event("run1", "step", json.dumps({"loss": 1.5}), "2026-01-01T00:00:01Z")
    assert e1.seq == 1 and e1.prev_hash == "0" * 64 and e2.prev_hash == e1.hash
    ph = hashlib.sha256(b'{"a":[1,2],"b":1}').hexdigest()
    assert e1.payload_hash == ph
    want = hashlib.sha256(f"1|{'0' * 64}|{ph}|2026-01-01T00:00:00Z|start".encode()).hexdigest()
    assert e1.hash == want and r.verify("run1")
    assert json.loads(e2.to_json())["payload"] == {"loss": 1.5}
    r.set_status("run1", "running")
    assert r.get("run1").status == "running" and len(r.events("run1")) == 2
    with pytest.raises(native.NativeError):
        r.append_event("ghost", "x", "{}")
    assert O.rfc3339_utc(0) == "1970-01-01T00:00:00Z"


def test_spike_log_actions():
    s = O.SpikeLog(page_window_steps=50, relative_threshold=0.5, baseline_window=4,
                   last_checkpoint_step=90)
    for i in range(4):
        assert s.observe(i, 2.0, "sh", "run") == []
    assert s.observe(5, 2.5, "sh", "run") == []
    acts = s.observe(6, 4.0, "shard-x", "run")
    assert [a.kind for a in acts] == ["log", "skip_shard", "rollback"]
    assert acts[0].event.baseline == pytest.approx((2 + 2 + 2 + 2.5) / 4)
    assert acts[1].shard_id == "shard-x" and acts[2].checkpoint_step == 90
    acts = s.observe(20, 9.0, "shard-y", "run")
    assert [a.kind for a in acts][-1] == "page" and "step=20" in acts[-1].message
    assert [k.shard_id for k in s.skipped_shards()] == ["shard-x", "shard-y"]
    with pytest.raises(native.NativeError):
        s.observe(21, math.inf, "", "")


def test_metric_log_sink_and_snapshot(tmp_path):
    log = O.MetricLog()
    with pytest.raises(native.NativeError) as e:
        log.series("train.loss")
    assert e.value.kind == "EmptyHistory"
    log.open_sink(str(tmp_path / "metrics.jsonl"))
    for step, v in [(2, 1.5), (1, 2.0), (3, 1.2)]:
        log.record("train.loss", {}, step, v)
    log.close_sink()
    assert log.series("train.loss") == [(1, 2.0), (2, 1.5), (3, 1.2)]
    lines = [json.loads(l) for l in (tmp_path / "metrics.jsonl").read_text().splitlines()]
    assert lines[0] == {"labels": {}, "name": "train.loss", "step": 2, "value": 1.5}
    dash = O.Dashboard("d", "Training", [O.Panel("p1", "loss", "train.loss"), O.Panel("p2", "log", "", "log")])
    snap = json.loads(O.snapshot(dash, log, [], "2026-01-01T00:00:00Z"))
    assert snap["panels"][0]["points"][0] == {"step": 1, "value": 2.0} and snap["panels"][1]["points"] == []
    with pytest.raises(native.NativeError) as e:
        O.snapshot(O.Dashboard("d", "t", [O.Panel("p", "x", "missing")]), log, [], "")
    assert e.value.kind == "UnknownMetric"
