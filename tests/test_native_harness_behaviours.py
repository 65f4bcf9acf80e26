"""One behaviour per test for the control-plane crates' C++ equivalents: raft (membership,
leases, partitions, durability), providers (response validation, AIMD window, failover, token
broker), ops (quorum, shadow, roll-out, rollback), ledger (append-only rules, query language),
lab kernel (quotas, spawn depth, mailboxes, rung gate, mirror fetch, promotion), eval gate and
monitors. Names follow the reference's harness/*/tests files."""
import hashlib
import json

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

R, PV, O, C = native.raft, native.providers, native.ops, native.cas
LG, K, EG, MON = native.ledger, native.kernel, native.eval_gate, native.monitors


def kind_of(fn, *a, **k):
    with pytest.raises(NativeError) as e:
        fn(*a, **k)
    return e.value.kind


@pytest.fixture
def group(tmp_path):
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    g.tick(0)
    return g


# ------------------------------------------------------------------------- raft
def test_group_of_two_voters_is_refused(tmp_path):
    assert kind_of(R.LocalGroup.start, 2, str(tmp_path / "g2")) == "TooFewVoters"


def test_no_leader_before_the_first_tick_then_smallest_id_wins(tmp_path):
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    assert g.leader() == -1
    g.tick(0)
    assert g.leader() == 0 and g.get(0).term == 1


def test_followers_refuse_writes(group):
    assert kind_of(group.get(1).set_kernel_version, "x") == "NotLeader"


def test_a_committed_write_reaches_every_node(group):
    group.get(0).set_kernel_version("1.0")
    assert [group.get(i).state()["kernel_version"] for i in range(3)] == ["1.0"] * 3


def test_workers_join_but_ephemeral_or_untrusted_nodes_cannot_vote(group):
    L = group.get(0)
    L.add_worker(R.NodeInfo("w1", "tcp://w1", always_on=False))
    assert kind_of(L.add_voter, R.NodeInfo("w2", "", always_on=False)) == "EphemeralVoter"
    assert kind_of(L.add_voter, R.NodeInfo("v9", "", trusted=False)) == "Untrusted"
    assert kind_of(L.add_worker, R.NodeInfo("w1", "", always_on=False)) == "Duplicate"


def test_removing_a_voter_below_three_is_refused(group):
    assert kind_of(group.get(0).remove_node, "1") == "TooFewVoters"


def test_role_lease_claim_heartbeat_expiry_and_reclaim(group):
    L = group.get(0)
    assert L.claim_role("coordinator", "1", 1000) == {"role": "coordinator", "holder": "1", "attempt": 1,
                                                      "expires_at": 31000}
    assert kind_of(L.claim_role, "coordinator", "2", 2000) == "NotClaimable"
    assert kind_of(L.heartbeat_role, "coordinator", "2", 2000) == "NotHolder"
    assert L.heartbeat_role("coordinator", "1", 5000)["expires_at"] == 35000
    assert L.expire_roles(34999) == [] and L.expire_roles(35000) == ["coordinator"]
    assert L.claim_role("coordinator", "2", 35001)["attempt"] == 2


def test_token_generations_count_up(group):
    L = group.get(0)
    assert L.commit_token(b"a") == (1, b"a") and L.commit_token(b"b")[0] == 2


def test_minority_leader_cannot_commit_and_majority_elects_a_higher_term(group):
    L = group.get(0)
    n = L.log_len
    group.partition([0])
    assert kind_of(L.set_kernel_version, "lost") == "NotLeader" and L.log_len == n
    group.tick(40000)
    assert group.leader() == 1 and group.get(1).term == 2 and not group.get(0).is_leader()


def test_healed_partition_catches_up(group):
    group.get(0).set_kernel_version("1.0")
    group.partition([0])
    group.tick(40000)
    group.get(1).set_kernel_version("2.0")
    assert group.get(0).state()["kernel_version"] == "1.0"
    group.heal()
    group.tick(40001)
    assert group.get(0).state()["kernel_version"] == "2.0" and group.get(0).term == 2


def test_crashed_node_restarts_from_disk_as_a_follower(group):
    group.get(0).set_kernel_version("1.0")
    group.crash(2)
    with pytest.raises(NativeError):
        group.get(2)
    group.get(0).set_kernel_version("1.1")
    group.restart(2)
    assert group.get(2).state()["kernel_version"] == "1.0" and not group.get(2).is_leader()
    group.tick(1)
    assert group.get(2).state()["kernel_version"] == "1.1"


def test_single_node_bootstrap_and_reopen(tmp_path):
    one = R.Cluster.bootstrap(str(tmp_path / "solo"), R.NodeInfo("a", "x"))
    assert one.is_leader()
    one.set_kernel_version("k")
    again = R.Cluster.open(str(tmp_path / "solo"), "a")
    assert again.state()["kernel_version"] == "k" and not again.is_leader()


# -------------------------------------------------------------------- providers
OK_BODY = json.dumps({"choices": [{"finish_reason": "stop", "message": {"content": "hi"}}]}).encode()


def test_valid_response_passes_through():
    assert json.loads(PV.validate_response(OK_BODY))["choices"][0]["finish_reason"] == "stop"


@pytest.mark.parametrize("body,kind", [
    (b"rate_limit", "RateLimitText"), (b"RATE_LIMIT", "RateLimitText"), (b'{"error": "Rate_Limit"}', "RateLimitText"),
    (b"not json", "MalformedJson"), (b"[1]", "MalformedJson"),
    (b'{"choices": []}', "EmptyCompletion"), (b"{}", "EmptyCompletion")])
def test_bad_response_bodies(body, kind):
    assert kind_of(PV.validate_response, body) == kind


def test_truncated_tool_call_is_caught_only_when_the_arguments_do_not_parse():
    def body(args):
        return json.dumps({"choices": [{"finish_reason": "length", "tool_calls": [
            {"function": {"name": "f", "arguments": args}}]}]}).encode()
    assert kind_of(PV.validate_response, body('{"a": 1')) == "TruncatedToolCall"
    PV.validate_response(body('{"a": 1}'))


def test_aimd_grows_by_one_and_shrinks_on_429_slow_success_and_outage():
    a = PV.Aimd(PV.AimdConfig(min_window=2, max_window=5))
    assert a.window == 2
    for _ in range(5):
        a.on_success(10)
    assert a.window == 5
    a.on_success(30001)
    assert a.window == 2
    a.on_success(1)
    a.on_outage()
    assert a.window == 2


def test_aimd_decrease_takes_at_least_one_step():
    b = PV.Aimd(PV.AimdConfig(decrease=1.0, max_window=8))
    for _ in range(3):
        b.on_success(1)
    b.on_429()
    assert b.window == 3


def test_failover_order_backoff_doubling_and_recovery():
    f = PV.Failover(["p0", "p1"])
    assert f.current() == "p0" and f.wait_backoff_ms() == 100
    f.mark_down("p0")
    assert f.current() == "p1" and f.wait_backoff_ms() == 200
    f.mark_down("p1")
    assert kind_of(f.current) == "NoProvider" and f.wait_backoff_ms() == 400
    f.mark_up("p0")
    assert f.current() == "p0"
    with pytest.raises(NativeError):
        f.mark_down("nope")


def test_only_the_leader_brokers_tokens_and_commits_before_issuing(group):
    assert kind_of(PV.broker_refresh, group.get(1), "anthropic", 60_000, b"blob", 5) == "NotBroker"
    (gen, blob), tok = PV.broker_refresh(group.get(0), "anthropic", 60_000, b"blob", 5)
    assert gen == 1 and tok.token == hashlib.sha256(b"blob").hexdigest() and tok.expires_at == 60_005
    assert group.get(2).state()["token"] == (1, b"blob")


# -------------------------------------------------------------------------- ops
def _release(version, artifact, signers):
    return O.Release(version, hashlib.sha256(artifact).hexdigest(), "c0ffee", signers)


@pytest.fixture
def rollout(tmp_path, group):
    backs = []
    for i in range(2):
        (tmp_path / f"b{i}").mkdir()
        backs.append(str(tmp_path / f"b{i}"))
    store = C.Store.create(str(tmp_path / "cas"), backs)
    return O.Ops.create(str(tmp_path / "ops")), store, group.get(0), tmp_path


def test_quorum_needs_two_distinct_non_empty_signatures(rollout):
    ops, store, _lead, _ = rollout
    weak = _release("1.0", b"k", [("alice", b"sig"), ("alice", b"sig2"), ("bob", b"")])
    assert not O.has_quorum(weak)
    assert kind_of(ops.propose, weak, b"k", store, 1) == "NoQuorum"
    assert ops.state.startswith("refused:need 2 human signatures, have 1")


def test_artifact_digest_must_match_the_release(rollout):
    ops, store, _lead, _ = rollout
    good = _release("1.0", b"k", [("alice", b"s"), ("bob", b"t")])
    assert kind_of(ops.propose, good, b"tampered", store, 2) == "DigestMismatch"


def test_stages_cannot_be_skipped(rollout):
    ops, store, lead, _ = rollout
    good = _release("1.0", b"k", [("alice", b"s"), ("bob", b"t")])
    ops.propose(good, b"k", store, 3)
    assert ops.state == "proposed" and store.pins == {"kernel.shadow": good.digest}
    assert kind_of(ops.apply_one, "0", 4) == "WrongState"
    ops.start_shadow(store, 5)
    ops.shadow_pass(6)
    assert kind_of(ops.apply_one, "shadow", 7) == "WrongState"
    assert kind_of(ops.promote, lead, store, 7) == "WrongState"


def _to_current(ops, store, lead, version, art, t0):
    rel = _release(version, art, [("alice", b"s"), ("bob", b"t")])
    ops.propose(rel, art, store, t0)
    ops.start_shadow(store, t0 + 1)
    ops.shadow_pass(t0 + 2)
    for node in ("0", "1", "2"):
        ops.apply_one(node, t0 + 3)
    ops.promote(lead, store, t0 + 4)
    return rel


def test_roll_out_one_node_at_a_time_then_promote(rollout):
    ops, store, lead, _ = rollout
    rel = _to_current(ops, store, lead, "1.0", b"k1", 10)
    assert ops.state == "current" and lead.state()["kernel_version"] == "1.0"
    assert store.pins == {"kernel.current": rel.digest}


def test_status_text_and_json(rollout):
    ops, store, lead, _ = rollout
    _to_current(ops, store, lead, "1.0", b"k1", 10)
    text = ops.cli(["status"], lead)
    assert text.splitlines()[:4] == ["kernel_version: 1.0", "state: current", "release: 1.0", "nodes:"]
    assert "  0 applied=1.0 healthy=true role=live" in text
    js = json.loads(ops.cli(["--json", "status"], lead))
    assert js["state"] == "current" and len(js["nodes"]) == 3
    with pytest.raises(NativeError):
        ops.cli(["frobnicate"], lead)


def test_unhealthy_node_during_roll_out_rolls_back_automatically(rollout):
    ops, store, lead, _ = rollout
    first = _to_current(ops, store, lead, "1.0", b"k1", 10)
    r2 = _release("2.0", b"k2", [("alice", b"s"), ("carol", b"u")])
    ops.propose(r2, b"k2", store, 30)
    ops.start_shadow(store, 31)
    ops.shadow_pass(32)
    ops.apply_one("0", 33)
    ops.mark_unhealthy("0", "oom", lead, store, 34)
    assert ops.state == "rolled_back:oom" and lead.state()["kernel_version"] == "1.0"
    assert store.pins == {"kernel.current": first.digest}


def test_rollback_from_current_restores_the_previous_digest_and_persists(rollout):
    ops, store, lead, tmp = rollout
    first = _to_current(ops, store, lead, "1.0", b"k1", 10)
    second = _to_current(ops, store, lead, "2.0", b"k2", 40)
    assert store.pins == {"kernel.current": second.digest, "kernel.previous": first.digest}
    ops.rollback("regression", lead, store, 50)
    assert lead.state()["kernel_version"] == "1.0" and store.pins == {"kernel.current": first.digest}
    again = O.Ops.open(str(tmp / "ops"))
    assert again.state == "rolled_back:regression" and again.kernel_version == "1.0"
    assert again.event_types()[:2] == ["ops.propose", "ops.shadow"]


def test_shadow_failure_unpins_the_candidate(rollout):
    ops, store, _lead, _ = rollout
    rel = _release("1.0", b"k1", [("alice", b"s"), ("bob", b"t")])
    ops.propose(rel, b"k1", store, 1)
    ops.start_shadow(store, 2)
    ops.shadow_fail("diverged", store, 3)
    assert ops.state == "rolled_back:diverged" and "kernel.shadow" not in store.pins


# ----------------------------------------------------------------------- ledger
def _rec(eid, hyp, role="researcher", rung=None, **kw):
    r = {"experiment_id": eid, "hypothesis": hyp, "prediction": "loss goes down", "config_hash": "c" * 8,
         "results": None, "delta_rci": None, "replication": None, "gpu_hours": None, "author_role": role,
         "rung": rung, "created_at": "2026-01-01T00:00:00Z", "closed_at": None, "supersedes": None}
    r.update(kw)
    return json.dumps(r)


@pytest.fixture
def ledger(tmp_path):
    l = LG.Ledger(str(tmp_path / "ledger.jsonl"))
    l.append(_rec("e1", "CHECK:muon Muon lr transfer holds across width", rung=1))
    l.append(_rec("e2", "PREREG:muon wider model keeps the optimum", role="engineer", rung=1))
    l.append(_rec("e3", "delta rule gates help long context", results={"passed": False}))
    l.append(_rec("e4", "fp8 matches bf16", replication={"status": "failed", "n": 3, "notes": None}))
    return l


def ids(rows):
    return [json.loads(r)["experiment_id"] for r in rows]


def test_ledger_is_append_only(ledger):
    assert kind_of(ledger.append, _rec("e1", "again")) == "Duplicate"
    assert kind_of(ledger.append, _rec("e5", "x", supersedes="missing")) == "NotFound"
    ledger.append(_rec("e5", "fp8 matches bf16 after fix", supersedes="e4"))
    assert len(ledger) == 5 and json.loads(ledger.get("e2"))["author_role"] == "engineer"


def test_ledger_query_language(ledger):
    assert ids(ledger.query("all")) == ["e1", "e2", "e3", "e4"]
    assert ids(ledger.query("rung=1 AND author_role=engineer")) == ["e2"]
    assert ids(ledger.query("kind=check")) == ["e1"] and ids(ledger.query("kind=prereg")) == ["e2"]
    assert ids(ledger.query('hypothesis~"fp8 matches" AND rung=none')) == ["e4"]


@pytest.mark.parametrize("bad", ["SELECT * FROM records", "colour=red", 'hypothesis~"open', "rung=x", "a= AND "])
def test_ledger_rejects_anything_outside_the_query_language(ledger, bad):
    with pytest.raises(NativeError):
        ledger.query(bad)


def test_ledger_similarity_search_negatives_and_durability(ledger, tmp_path):
    hits = ledger.search_similar("does fp8 match bf16", 1)
    assert hits[0][0] == "e4" and hits[0][1] > 0.3 and ledger.search_similar("x", 0) == []
    assert ids(ledger.list_negatives()) == ["e3", "e4"]
    assert ids(LG.Ledger(str(tmp_path / "ledger.jsonl")).query("*")) == ["e1", "e2", "e3", "e4"]


# ------------------------------------------------------------------- lab kernel
@pytest.fixture
def lab(tmp_path):
    mirror = tmp_path / "mirror"
    (mirror / "arxiv.org" / "abs").mkdir(parents=True)
    (mirror / "arxiv.org" / "abs" / "1234").write_bytes(b"paper")
    (tmp_path / "secret").write_bytes(b"no")
    k = K.Kernel(str(tmp_path / "ledger.jsonl"), str(mirror), str(tmp_path / "log"))
    root = k.spawn("director", "run the lab", K.Quota(1000, 100, 50), "prog")
    child = k.spawn("researcher", "x", K.Quota(400, 40, 10), "prog", root.id)
    return k, root, child, tmp_path


def test_spawn_ids_depth_and_the_invariant_in_the_instructions(lab):
    k, root, child, tmp = lab
    assert (root.id, root.depth, root.parent) == ("a-1", 0, None) and child.depth == 1
    text = (tmp / "log" / "agents" / "a-1" / "instructions.txt").read_text()
    assert text.startswith(K.KERNEL_INVARIANT) and text.endswith("run the lab")


def test_child_quota_is_carved_out_of_the_parent(lab):
    k, root, _child, _ = lab
    assert k.remaining(root.id).tokens == 600
    assert kind_of(k.spawn, "researcher", "x", K.Quota(700, 0, 0), "prog", root.id) == "QuotaRefused"


def test_spawn_depth_is_capped_at_three_and_roles_are_checked(lab):
    k, _root, child, _ = lab
    a = child
    for _ in range(2):
        a = k.spawn("subagent", "x", K.Quota(0, 0, 0), "prog", a.id)
    assert a.depth == 3
    assert kind_of(k.spawn, "subagent", "x", K.Quota(0, 0, 0), "prog", a.id) == "SpawnDepth"
    assert kind_of(k.spawn, "overlord", "x", K.Quota(), "prog") == "RoleNotSpawnable"


def test_an_agent_without_budget_cannot_submit(lab):
    k, _root, _child, _ = lab
    empty = k.spawn("engineer", "x", K.Quota(), "prog")
    assert kind_of(k.submit_job, empty.id, 0, [], K.Quota(1, 0, 0)) == "BudgetExhausted"


def test_mailboxes_deliver_once_in_order(lab):
    k, root, child, _ = lab
    mid = k.send(root.id, child.id, "hello", 5)
    msg = k.recv(child.id)
    assert (msg.id, msg.sender, msg.body, msg.created_ms) == (mid, root.id, "hello", 5) and k.recv(child.id) is None
    assert kind_of(k.send, root.id, "a-99", "x", 1) == "AgentNotFound"


def test_rung_above_zero_needs_check_and_prereg_rows(lab):
    k, _root, child, _ = lab
    assert k.submit_job(child.id, 0, [], K.Quota(10, 0, 0)) == "j-1"
    assert kind_of(k.submit_job, child.id, 2, ["muon"], K.Quota(10, 0, 0)) == "RungNotCleared"
    k.ledger_append(_rec("e1", "CHECK:muon sanity"))
    assert kind_of(k.submit_job, child.id, 2, ["muon"], K.Quota(10, 0, 0)) == "RungNotCleared"
    k.ledger_append(_rec("e2", "PREREG:muon prediction"))
    assert k.submit_job(child.id, 2, ["muon"], K.Quota(10, 0, 0)) == "j-2"
    assert k.remaining(child.id).tokens == 380 and len(k.ledger_query("kind=check")) == 1


@pytest.mark.parametrize("url", ["http://arxiv.org/abs/1234", "https://evil.example/abs/1234",
                                 "https://arxiv.org/../secret", "https://arxiv.org/abs/none"])
def test_fetch_serves_only_mirrored_https_pages(lab, url):
    k = lab[0]
    assert k.fetch("https://arxiv.org/abs/1234?v=2") == b"paper"
    assert kind_of(k.fetch, url) == "NotMirrored"


def test_mirror_host_matching_is_exact():
    assert K.is_mirror_url("https://GitHub.com:443/x") and not K.is_mirror_url("https://github.com.evil/x")


def test_genome_patch_goes_smoke_gate_canary_then_rolls_out_after_24h(lab):
    k, _root, child, _ = lab
    p = k.propose_patch(child.id, "good diff", "why", "genome")
    assert [k.promote_genome(p, t) for t in (0, 1, 2)] == ["smoke_passed", "gate_passed", "canary"]
    assert k.promote_genome(p, 2 + K.CANARY_MS - 1) == "canary"
    assert k.promote_genome(p, 2 + K.CANARY_MS) == "rolled_out"


def test_gate_failure_refuses_and_canary_failure_reverts(lab):
    k, _root, child, _ = lab
    bad = k.propose_patch(child.id, "FAIL_GATE", "why", "genome")
    assert [k.promote_genome(bad, 0), k.promote_genome(bad, 1)] == ["smoke_passed", "refused"]
    assert kind_of(k.promote_genome, bad, 2) == "PromoteRefused"
    rev = k.propose_patch(child.id, "FAIL_CANARY", "why", "recipe")
    for t in (0, 1, 2):
        k.promote_genome(rev, t)
    assert k.promote_genome(rev, 2 + K.CANARY_MS) == "reverted"


def test_weights_need_two_human_signatures_and_passing_evals(lab):
    k = lab[0]
    assert kind_of(k.promote_weights, "ckpt-1", [("alice", b"s"), ("alice", b"t"), ("bob", b"")]) == "NoQuorum"
    assert k.promote_weights("ckpt-1", [("alice", b"s"), ("bob", b"t")]) == "serving"
    assert k.promote_weights("ckpt-FAIL_EVALS", []) == "refused"


def test_escalation_tickets_and_restart_keeps_agents_and_the_id_counter(lab):
    k, _root, child, tmp = lab
    t = k.escalate(child.id, "grader looks wrong", "evidence")
    assert k.ticket(t) == ("grader looks wrong", "evidence", child.id)
    k2 = K.Kernel(str(tmp / "ledger.jsonl"), str(tmp / "mirror"), str(tmp / "log"))
    assert k2.remaining(child.id).tokens == 400
    assert k2.spawn("reviewer", "x", K.Quota(), "prog").id == "a-3"


# -------------------------------------------------------------------- eval gate
ITEMS = [{"id": "b", "prompt": "2+2", "answer": "4", "weight_milli": 600},
         {"id": "a", "prompt": "cap of fr", "answer": "paris", "weight_milli": 400}]


def _suite(root, suite, items, written, compute=7):
    d = root / suite / "pending"
    d.mkdir(parents=True, exist_ok=True)
    (d / "items.jsonl").write_text("".join(json.dumps(i) + "\n" for i in items))
    (d / "meta.json").write_text(json.dumps({"written_ms": written, "compute_ms": compute}))


@pytest.fixture
def gate(tmp_path):
    root = tmp_path / "suites"
    root.mkdir()
    return EG.EvalGate(str(root), "h1"), root


def test_only_held_out_suites_are_served(gate):
    g, _ = gate
    assert kind_of(g.suite_hash, "aime") == "NotHeldOut" and kind_of(g.suite_hash, "nope") == "UnknownSuite"
    assert EG.is_held_out_suite("speedrun") and not EG.is_held_out_suite("gpqa")


def test_rotation_needs_pending_items_written_after_a_past_cutoff(gate):
    g, root = gate
    assert kind_of(g.rotate, "re_bench", 10, 100) == "RotationRefused"
    _suite(root, "re_bench", ITEMS, written=50)
    with pytest.raises(NativeError):
        g.rotate("re_bench", 60, 100)
    with pytest.raises(NativeError):
        g.rotate("re_bench", 200, 100)


def test_suite_hash_is_over_the_canonical_sorted_items(gate):
    g, root = gate
    _suite(root, "re_bench", ITEMS, written=50)
    h = g.rotate("re_bench", 40, 100)
    canon = "".join(json.dumps(i, sort_keys=True, separators=(",", ":")) + "\n"
                    for i in sorted(ITEMS, key=lambda i: i["id"]))
    assert h == hashlib.sha256(canon.encode()).hexdigest() == g.suite_hash("re_bench")
    assert not (root / "re_bench" / "pending").exists()


def test_requests_return_scores_only(gate):
    g, root = gate
    _suite(root, "re_bench", ITEMS, written=50)
    h = g.rotate("re_bench", 40, 100)
    (root / "subjects" / "checkpoint").mkdir(parents=True)
    (root / "subjects" / "checkpoint" / "ck1.json").write_text(json.dumps({"a": "paris", "b": "5"}))
    s = g.request("checkpoint", "ck1", "re_bench")
    assert (s.rci_milli, s.n_items, s.compute_ms, s.harness_version, s.suite_hash) == (400, 2, 7, "h1", h)
    assert not any(hasattr(s, f) for f in ("items", "prompt", "answer"))
    for subj in ("../ck1", "missing", ""):
        assert kind_of(g.request, "checkpoint", subj, "re_bench") == "SubjectNotFound"


def test_rotation_at_most_every_ninety_days_and_history_kept(gate):
    g, root = gate
    _suite(root, "re_bench", ITEMS, written=50)
    h = g.rotate("re_bench", 40, 100)
    _suite(root, "re_bench", ITEMS[:1], written=EG.ROTATION_MS)
    assert kind_of(g.rotate, "re_bench", 100, 100 + EG.ROTATION_MS - 1) == "RotationRefused"
    h2 = g.rotate("re_bench", 100, 100 + EG.ROTATION_MS)
    assert h2 != h and json.loads((root / "re_bench" / "history.jsonl").read_text())["suite_hash"] == h


# --------------------------------------------------------------------- monitors
def test_grader_hash_mismatch_freezes_and_later_events_are_recorded(tmp_path):
    m = MON.Monitors(str(tmp_path / "state" / "freeze.json"), {"g1": "aa"})
    m.note_grader_hash("g1", "aa", 1)
    assert not m.frozen()
    assert kind_of(m.note_grader_hash, "g1", "bb", 2) == "GraderHashMismatch" and m.frozen()
    assert kind_of(m.note_held_out_access, "a-3", 3) == "HeldOutAccess"
    snap = m.snapshot()
    assert snap["frozen_at"] == 2 and snap["reason"] == "grader hash mismatch"
    assert [v["boundary"] for v in snap["violations"]] == ["graders", "held_out"]
    assert kind_of(m.kill, "manual", 4) == "AlreadyFrozen"


def test_freeze_survives_a_restart(tmp_path):
    path = str(tmp_path / "freeze.json")
    m = MON.Monitors(path, {"g1": "aa"})
    with pytest.raises(NativeError):
        m.note_grader_hash("g1", "bb", 2)
    again = MON.Monitors(path, {})
    assert again.frozen() and len(again.snapshot()["violations"]) == 1
    assert kind_of(again.plant, "nowhere", "x", 5) == "UnknownBoundary"


def test_operator_kill_and_the_other_tripwires(tmp_path):
    fresh = MON.Monitors(str(tmp_path / "f2.json"))
    fresh.kill("operator", 9)
    assert fresh.snapshot()["reason"] == "operator"
    assert kind_of(fresh.note_kernel_escape, "x", 10) == "Message"
    assert kind_of(fresh.note_self_check, "x", 10) == "MonitorSelfCheck"
    assert MON.BOUNDARIES == ["kernel", "graders", "held_out", "monitors"]
