"""RL coordinator, multi-agent bookkeeping, sandbox pool, exact verifiers and reward models
(C++), against the contracts of the reference's rl/* and verifiers crates."""
import hashlib
import json
import math

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

CO, MA, EN, VE, RW = native.coordinator, native.multiagent, native.envs, native.verifiers, native.rewards


def _kind(e):
    return e.value.kind


def test_coordinator_split_staleness_parity_and_rebalance():
    cfg = CO.CoordinatorConfig(queue_high=2)
    for racks, kind in (([], "EmptyFleet"), ([("a", 8), ("a", 8)], "DuplicateRack"), ([("a", 0), ("b", 8)], "Message"),
                        ([("a", 8)], "NotEnoughRacks")):
        with pytest.raises(NativeError) as e:
            CO.Coordinator(cfg, racks)
        assert _kind(e) == kind
    c = CO.Coordinator(cfg, [(f"r{i}", 8) for i in range(10)])
    assert c.split_gpus() == (48, 32) and c.n_rollout_racks() == 6       # floor(80 * 65 / 100) = 52
    assert c.rack_role("r0") == "rollout" and c.rack_role("r9") == "trainer" and c.rack_version("r0") == 0
    with pytest.raises(NativeError) as e:
        c.rack_version("r9")
    assert _kind(e) == "NotRollout"
    # versions advance one at a time; racks sync only to the published version
    with pytest.raises(NativeError) as e:
        c.publish_weights(2)
    assert _kind(e) == "NotNextVersion"
    c.publish_weights(1)
    with pytest.raises(NativeError) as e:
        c.sync_rack("r0", 0)
    assert _kind(e) == "Unpublished"
    c.sync_rack("r0", 1)
    assert c.rack_version("r0") == 1
    # queue: duplicates / empties rejected, too-stale heads dropped on consume
    c.enqueue_batch(CO.RolloutBatch("b0", "p0", 0))
    c.enqueue_batch(CO.RolloutBatch("b1", "p1", 1))
    with pytest.raises(NativeError) as e:
        c.enqueue_batch(CO.RolloutBatch("b1", "p1", 1))
    assert _kind(e) == "DuplicateBatch"
    with pytest.raises(NativeError) as e:
        c.enqueue_batch(CO.RolloutBatch("b2", "p", 1, n_samples=0))
    assert _kind(e) == "EmptyGroup"
    for v in range(2, 6):
        c.publish_weights(v)
    assert CO.staleness(5, 1) == 4
    got = c.consume_batch()                        # b0 is 5 versions old: dropped; b1 is 4: kept
    assert got.id == "b1" and c.queue_depth() == 0 and c.consume_batch() is None
    c.enqueue_batch(CO.RolloutBatch("future", "p", 9))
    with pytest.raises(NativeError) as e:
        c.consume_batch()
    assert _kind(e) == "FromTheFuture"
    # rebalance: empty queue -> one trainer rack joins the rollouts (lowest id first)
    c2 = CO.Coordinator(cfg, [(f"r{i}", 8) for i in range(10)])
    assert c2.rebalance() == ("r6", "rollout")
    c2.enqueue_batch(CO.RolloutBatch("x0", "p", 0))
    c2.enqueue_batch(CO.RolloutBatch("x1", "p", 0))
    assert c2.rebalance() == ("r0", "trainer")     # backlog at queue_high -> more trainer
    # parity: drift above the threshold halts everything, and it sticks
    rep = c2.run_parity(0, [(-1.0, -1.0005), (-2.0, -2.0)])
    assert rep[0] == 0 and abs(rep[1] - 5e-4) < 1e-12 and rep[2] == 2
    with pytest.raises(NativeError) as e:
        c2.run_parity(0, [(-1.0, float("nan"))])
    assert _kind(e) == "InvalidLogprob"
    with pytest.raises(NativeError) as e:
        c2.run_parity(0, [(-1.0, -1.5)])
    assert _kind(e) == "ParityHalt" and c2.state() == "halted"
    for call in (lambda: c2.publish_weights(1), lambda: c2.consume_batch(), lambda: c2.rebalance()):
        with pytest.raises(NativeError) as e:
            call()
        assert _kind(e) == "Halted"


def test_multiagent_topologies_budget_memos_and_distill():
    draws = [MA.topology_from_draw(d) for d in range(100)]
    assert [draws.count(t) for t in MA.TOPOLOGIES] == [50, 20, 15, 10, 5]
    assert MA.topology_from_draw(149) == MA.topology_from_draw(49) == "single" and MA.topology_from_draw(50) == "orchestrator_subs"
    assert MA.roster("parallel_aggregate", 2) == [("attempt-00", "attempt"), ("attempt-01", "attempt"), ("aggregator", "aggregator")]
    for topo, n in (("single", 1), ("orchestrator_subs", 0), ("proposer_solver", 3), ("parallel_aggregate", 100)):
        with pytest.raises(NativeError) as e:
            MA.roster(topo, n)
        assert _kind(e) == "BadWidth"
    with pytest.raises(NativeError) as e:
        MA.Multiagent(MA.MultiConfig(weights=[40, 30, 15, 10, 5]))       # single must keep >= 50
    assert _kind(e) == "BadMix"
    m = MA.Multiagent()
    ros = m.spawn_episode("e1", "task", "orchestrator_subs", 2, 100)
    assert [a for a, _ in ros] == ["orchestrator", "sub-00", "sub-01"]
    with pytest.raises(NativeError) as e:
        m.spawn_episode("e1", "task", "single", 0, 10)
    assert _kind(e) == "DuplicateEpisode"
    with pytest.raises(NativeError):
        m.spawn_episode("e2", "task", "single", 0, 0)
    m.scratch_append("e1", "sub-00", "note;")
    assert m.scratch_read("e1") == "note;"
    kept = m.send_message("e1", MA.Message("orchestrator", "sub-00", "go", [0.5, 1.0]), 49)
    dropped = m.send_message("e1", MA.Message("orchestrator", "sub-01", "go", [0.5]), 50)
    assert kept.latent_memo == [0.5, 1.0] and dropped.latent_memo is None
    assert [x.text for x in m.inbox("e1", "sub-00")] == ["go"] and m.inbox("e1", "orchestrator") == []
    with pytest.raises(NativeError) as e:
        m.send_message("e1", MA.Message("ghost", "sub-00", "x"), 0)
    assert _kind(e) == "UnknownAgent"
    m.record_credit("e1", "orchestrator", ["sub-00"])
    assert m.credit("e1") == [("orchestrator", ["sub-00"])]
    assert m.charge_tokens("e1", "sub-00", 60) == 60 and m.charge_tokens("e1", "sub-01", 40) == 100
    with pytest.raises(NativeError) as e:
        m.charge_tokens("e1", "orchestrator", 1)
    assert _kind(e) == "BudgetExceeded" and m.tokens_used_by("e1", "sub-00") == 60
    assert m.distill_back("t", 100, 0.9, 0.5) == ("t", 100) and m.distill_back("t", 100, 0.5, 0.5) is None
    with pytest.raises(NativeError):
        m.distill_back("t", 100, float("inf"), 0.5)


def test_sandbox_pool_views_tools_and_tamper_flags():
    pool = EN.Pool(EN.PoolConfig(capacity=20, offline_pages={"https://docs.local/a": (b"<p>hi</p>", 10),
                                                             "https://docs.local/new": (b"late", 99)},
                                 web_cutoff_unix_s=50))
    for img, kind in ((EN.Image("bad", env={"AWS_KEY": "x"}), "CredentialInSandbox"),
                      (EN.Image("bad", hidden_tests={"/work/t.py": b"x"}), "HiddenTestsVisible"),
                      (EN.Image("bad", agent_files={"/grader/t.py": b"x"}), "HiddenTestsVisible")):
        with pytest.raises(NativeError) as e:
            pool.register_image(img)
        assert _kind(e) == kind
    pool.register_image(EN.Image("img", {"/work/a.txt": b"alpha"}, {"/grader/test.py": b"assert 1"}, {"LANG": "C"}))
    snap = pool.snapshot_from_image("img")
    group = pool.fork_group(snap)
    assert len(group) == EN.GRPO_GROUP == 16 and pool.live_count() == 16
    with pytest.raises(NativeError) as e:
        pool.fork_group(snap, 5)
    assert _kind(e) == "PoolExhausted"
    a, b = group[0], group[1]
    call = lambda sb, tool, **payload: pool.call(sb, "c1", tool, json.dumps(payload), None, 7)
    assert call(a, "shell", command="echo hi there").stdout == b"hi there\n"
    assert call(a, "shell", command="echo new > /work/b.txt").ok and call(a, "shell", command="cat /work/b.txt").stdout == b"new\n"
    assert not call(b, "shell", command="cat /work/b.txt").ok          # forks are isolated
    assert call(a, "python", code="print(open('/work/a.txt').read())").stdout == b"alpha\n"
    assert call(a, "python", code="print(2 + 3 * 4)").stdout == b"14\n" and call(a, "python", code='print("x")').stdout == b"x\n"
    assert call(a, "editor", path="/work/c.txt", content="C").ok and call(a, "editor", path="/work/c.txt").stdout == b"C"
    assert call(a, "notes", content="memo").ok and pool.agent_view(a)["/notes/memo.txt"] == b"memo"
    assert call(a, "browser", url="https://docs.local/a").stdout == b"<p>hi</p>"
    assert call(a, "browser", url="https://docs.local/new").stderr == "page after cutoff"
    assert call(a, "lean", code="theorem t : True := trivial").ok and not call(a, "lean", code="sorry").ok
    # the grader area is invisible to the agent, and writes to it are blocked and recorded
    assert "/grader/test.py" not in pool.agent_view(a) and pool.grader_view(a)["/grader/test.py"] == b"assert 1"
    assert not call(a, "shell", command="cat /grader/test.py").ok
    for tool, payload in (("shell", {"command": "echo pass > /grader/test.py"}),
                          ("editor", {"path": "/grader/x", "content": "y"}),
                          ("python", {"code": "open('/grader/test.py', 'w').write('')"})):
        with pytest.raises(NativeError) as e:
            pool.call(a, "evil", tool, json.dumps(payload), None, 9)
        assert _kind(e) == "TestFileWrite"
    assert [(f.path, f.call_id, f.now_ms) for f in pool.tamper_flags][0] == ("/grader/test.py", "evil", 9)
    assert len(pool.tamper_flags) == 3
    for tool, payload, kind in (("shell", {"command": "curl http://x"}, "EgressDenied"),
                                ("python", {"code": "import requests"}, "LiveInternet"),
                                ("browser", {"url": "https://live.example"}, "EgressDenied"),
                                ("shell", {"command": "sleep 100"}, "Timeout"),
                                ("shell", {"command": "nvidia-smi"}, "Backend")):
        with pytest.raises(NativeError) as e:
            pool.call(a, "c", tool, json.dumps(payload), 30, 0)
        assert _kind(e) == kind
    pool.kill(b)
    child = call(a, "spawn").child_sandbox
    assert pool.agent_view(child)["/work/b.txt"] == b"new\n" and pool.live_count() == 16
    with pytest.raises(NativeError) as e:
        call(b, "shell", command="echo x")
    assert _kind(e) == "SandboxDead"


def test_exact_verifiers():
    eq = VE.math_equivalent
    assert eq("$\\frac{1}{2}$", "0.5") and eq("\\left( 1 + 2 \\right) * 3", "9") and eq("2/4", "\\frac{1}{2}")
    assert eq("x+1", " x + 1 ") and not eq("x+1", "1+x") and not eq("1/3", "0.333") and not eq("1/0", "2/0")
    assert VE.math_canonicalize(" $ a \\left( b \\right) $ ") == "a(b)"
    assert VE.tiny_kernel_check("true", " trivial ") and not VE.tiny_kernel_check("id", "fun y => y")
    with pytest.raises(NativeError) as e:
        VE.tiny_kernel_check("riemann", "obvious")
    assert _kind(e) == "Lean"
    g = [[1, 2], [3, 4]]
    assert VE.grid_pass_at_2(g, [[[0, 0], [0, 0]], g]) and not VE.grid_pass_at_2(g, [[[1, 2], [3, 5]]])
    with pytest.raises(NativeError) as e:
        VE.grid_pass_at_2(g, [g, g, g])
    assert _kind(e) == "TooManyGrids"
    with pytest.raises(NativeError) as e:
        VE.grid_pass_at_2(g, [[[1, 2], [3]]])
    assert _kind(e) == "BadGrid"
    assert abs(VE.relative_log_score(0.8, 0.5, True) - math.log(0.8 / 0.5)) < 1e-12
    assert abs(VE.relative_log_score(0.8, 0.5, False) - math.log(0.2 / 0.5)) < 1e-12
    assert VE.relative_log_score(0.0, 0.5, True) == pytest.approx(math.log(1e-12) - math.log(0.5))
    with pytest.raises(NativeError) as e:
        VE.relative_log_score(1.2, 0.5, True)
    assert _kind(e) == "BadProbability"
    # hidden tests + mutants in a sandbox
    pool = EN.Pool()
    image = EN.Image("task", {"/work/solution.txt": b"todo"}, {"/grader/expected": b"42"})
    task = VE.CodeTask(image, json.dumps({"code": "print(open('/work/solution.txt').read())"}), b"42\n",
                       mutants=[("m1", {"/work/solution.txt": b"41"})])
    assert VE.verify_sandboxed(pool, task, {"/work/solution.txt": b"42"}) == (1.0, True)
    assert VE.verify_sandboxed(pool, task, {"/work/solution.txt": b"7"}) == (0.0, False)
    with pytest.raises(NativeError) as e:
        VE.verify_sandboxed(pool, task, {"/grader/expected": b"x"})
    assert _kind(e) == "TestFileWrite"
    weak = VE.CodeTask(image, json.dumps({"code": "print(1)"}), b"1\n", mutants=[("m1", {"/work/solution.txt": b"41"})])
    with pytest.raises(NativeError) as e:
        VE.verify_sandboxed(pool, weak, {})
    assert _kind(e) == "WeakTests"
    bare = VE.CodeTask(image, json.dumps({"code": "print(open('/work/solution.txt').read())"}), b"42\n")
    with pytest.raises(NativeError) as e:
        VE.verify_sandboxed(pool, bare, {"/work/solution.txt": b"42"})
    assert _kind(e) == "Unverifiable"
    assert pool.live_count() == 0


def test_reward_models():
    rubric = [RW.Criterion("clarity", "is it clear?", 1.0), RW.Criterion("rigor", "is it rigorous?", 3.0)]
    replies = {("g1", "clarity"): "1.0", ("g1", "rigor"): "0.5", ("g2", "clarity"): "0.5", ("g2", "rigor"): " 0.5 "}
    seen = []

    def judge(prompt):
        lines = prompt.split("\n")
        seen.append(prompt)
        return replies[(lines[0].split(":")[1], lines[1].split(":")[1])]

    scores = RW.rubric_score(rubric, ["g1", "g2"], judge, "the answer")
    assert scores == [("g1", 0.625), ("g2", 0.5)] and seen[0] == "grader:g1\ncriterion:clarity\nis it clear?\n\nthe answer"
    assert RW.rubric_combine([0.625, 0.5]) == pytest.approx(0.5625 * 0.875)
    assert RW.rubric_combine([0.7, 0.7]) == pytest.approx(0.7)
    for bad, kind in (("seven", "Unverifiable"), ("1.5", "BadScore")):
        with pytest.raises(NativeError) as e:
            RW.rubric_score(rubric, ["g"], lambda p: bad, "x")
        assert _kind(e) == kind
    with pytest.raises(NativeError) as e:
        RW.rubric_score([], ["g"], judge, "x")
    assert _kind(e) == "EmptyRubric"
    with pytest.raises(NativeError) as e:
        RW.rubric_score([RW.Criterion("c", "p", 0.0)], ["g"], judge, "x")
    assert _kind(e) == "BadWeight"
    clean = RW.TrajectoryView(visible_passed=True, hidden_passed=True)
    hack = RW.TrajectoryView(visible_passed=True, hidden_passed=False, wrote_test_file=True)
    assert not clean.is_confirmed_hack() and hack.kinds() == ["test_write", "visible_pass_hidden_fail"]
    RW.tamper_pair_keep(clean, hack)
    for pos, neg in ((hack, hack), (clean, clean)):
        with pytest.raises(NativeError) as e:
            RW.tamper_pair_keep(pos, neg)
        assert _kind(e) == "UnconfirmedPair"
    RW.rescore_keep(0.9, 0.2)
    with pytest.raises(NativeError):
        RW.rescore_keep(0.2, 0.2)
    assert RW.tamper_verify(hack) == (0.0, False, ["tampering"]) and RW.tamper_verify(clean) == (1.0, True, [])
    assert RW.held_out_recall([hack, RW.TrajectoryView(special_cased=True), clean, hack]) == 0.75
    with pytest.raises(NativeError) as e:
        RW.refuse_exact("sandboxed_tests")
    assert _kind(e) == "ExactVerifier"
