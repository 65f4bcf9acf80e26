"""Behaviour list of the sandbox pool (C++ ``native.envs``; reference rl/envs/tests/{config,
egress,faults,fork,gpu,isolation,register,subagent,tools,firecracker}.rs): image registration
rules, fork capacity, isolation between forks, the agent / grader views, blocked writes and
their tamper records, egress and offline pages, tool timeouts, the GPU wall-time budget and the
microVM backend's boot checks."""
import hashlib
import json
import os

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

EN = native.envs


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def booted(capacity=64, n=1, **cfg):
    pool = EN.Pool(EN.PoolConfig(capacity=capacity, **cfg))
    pool.register_image(EN.Image("img", {"/work/a.txt": b"alpha", "/work/data.txt": b"1 2 3"},
                                 {"/grader/test_a.py": b"assert 1", "/grader/sub/test_b.py": b"assert 2"}, {"LANG": "C"}))
    snap = pool.snapshot_from_image("img")
    return pool, snap, pool.fork_group(snap, n)


def call(pool, sb, tool, timeout=None, now=0, call_id="c", **payload):
    return pool.call(sb, call_id, tool, json.dumps(payload), timeout, now)


# ------------------------------------------------------------------------------ constants / images
def test_constants():
    assert EN.GRPO_GROUP == 16 and EN.FORK_BUDGET_MS == 200 and EN.GRADER_ROOT == "/grader"
    assert sorted(EN.TOOLS) == ["browser", "editor", "lean", "notes", "python", "shell", "spawn"]


@pytest.mark.parametrize("key", ["AWS_ACCESS_KEY_ID", "aws_secret", "GITHUB_TOKEN", "db_password", "SSH_AUTH_SOCK",
                                 "MY_SECRET", "Api_Credential"])
def test_credential_like_variables_are_refused_at_registration(key):
    pool = EN.Pool()
    e = err(lambda: pool.register_image(EN.Image("bad", env={key: "x"})))
    assert e.kind == "CredentialInSandbox" and key in str(e)
    assert err(lambda: pool.snapshot_from_image("bad")).kind == "UnknownImage"      # nothing was registered


def test_ordinary_variables_and_clean_images_register():
    pool = EN.Pool()
    assert pool.register_image(EN.Image("ok", {"/work/x": b"1"}, {"/grader/t": b"2"}, {"LANG": "C", "PATH": "/bin", "HOME": "/work"})) == "ok"
    assert pool.register_image(EN.Image("empty")) == "empty"
    assert pool.snapshot_from_image("ok") != pool.snapshot_from_image("ok")         # each snapshot has its own id


def test_hidden_tests_live_under_the_grader_root_and_agent_files_do_not():
    pool = EN.Pool()
    for img in (EN.Image("b1", hidden_tests={"/work/test.py": b"x"}), EN.Image("b2", hidden_tests={"/graderx/test.py": b"x"}),
                EN.Image("b3", agent_files={"/grader/leak.py": b"x"}), EN.Image("b4", agent_files={"/grader": b"x"})):
        assert err(lambda: pool.register_image(img)).kind == "HiddenTestsVisible"


# ------------------------------------------------------------------------------ forks and capacity
def test_a_group_of_sixteen_identical_forks_then_the_pool_is_full():
    pool, snap, _ = booted(capacity=17, n=1)
    group = pool.fork_group(snap)
    assert len(group) == 16 and len(set(group)) == 16 and pool.live_count() == 17
    views = [pool.agent_view(sb) for sb in group]
    assert all(v == views[0] for v in views) and views[0]["/work/a.txt"] == b"alpha"
    e = err(lambda: pool.fork_group(snap, 1))
    assert e.kind == "PoolExhausted" and "17" in str(e)
    assert pool.live_count() == 17                                                    # a refused fork creates nothing


def test_capacity_counts_live_sandboxes_only():
    pool, snap, (first,) = booted(capacity=2)
    assert err(lambda: pool.fork_group(snap, 2)).kind == "PoolExhausted"
    second = pool.fork_group(snap, 1)[0]
    pool.kill(first)
    assert pool.live_count() == 1
    third = pool.fork_group(snap, 1)[0]                                               # the freed slot is reusable
    assert len({first, second, third}) == 3 and pool.live_count() == 2
    fresh = EN.Pool(EN.PoolConfig(capacity=3))
    fresh.register_image(EN.Image("i"))
    assert err(lambda: fresh.fork_group(fresh.snapshot_from_image("i"), 4)).kind == "PoolExhausted"


def test_fork_pair_gives_two_distinct_isolated_sandboxes():
    pool, snap, _ = booted()
    a, b = pool.fork_pair(snap)
    assert a != b
    assert call(pool, a, "editor", path="/work/only_a.txt", content="A").ok
    assert call(pool, a, "shell", command="echo changed > /work/a.txt").ok
    assert "/work/only_a.txt" not in pool.agent_view(b) and pool.agent_view(b)["/work/a.txt"] == b"alpha"
    assert pool.agent_view(a)["/work/a.txt"] == b"changed\n"
    later = pool.fork_group(snap, 1)[0]
    assert pool.agent_view(later)["/work/a.txt"] == b"alpha"                          # the snapshot is untouched too


def test_snapshot_of_a_running_sandbox_carries_its_changes():
    pool, _snap, (sb,) = booted()
    call(pool, sb, "editor", path="/work/new.txt", content="N")
    snap2 = pool.snapshot(sb)
    child = pool.fork_group(snap2, 1)[0]
    assert pool.agent_view(child)["/work/new.txt"] == b"N" and pool.grader_view(child)["/grader/test_a.py"] == b"assert 1"


def test_unknown_ids():
    pool, snap, (sb,) = booted()
    assert err(lambda: pool.fork_group("snap-404", 1)).kind == "UnknownSnapshot"
    assert err(lambda: pool.fork_pair("snap-404")).kind == "UnknownSnapshot"
    assert err(lambda: pool.snapshot_from_image("nope")).kind == "UnknownImage"
    for fn in (lambda: pool.kill("sb-404"), lambda: pool.snapshot("sb-404"), lambda: pool.agent_view("sb-404"),
               lambda: pool.grader_view("sb-404"), lambda: call(pool, "sb-404", "shell", command="echo x")):
        assert err(fn).kind == "UnknownSandbox"
    pool.kill(sb)
    for fn in (lambda: pool.kill(sb), lambda: pool.snapshot(sb), lambda: call(pool, sb, "shell", command="echo x")):
        assert err(fn).kind == "SandboxDead"
    assert err(lambda: call(pool, pool.fork_group(snap, 1)[0], "teleport")).kind == "BadToolRequest"


# ------------------------------------------------------------------------------ views and tampering
def test_agent_view_hides_the_grader_area():
    pool, _snap, (sb,) = booted()
    agent, grader = pool.agent_view(sb), pool.grader_view(sb)
    assert not any(p.startswith("/grader") for p in agent)
    assert {p for p in grader if p.startswith("/grader")} == {"/grader/test_a.py", "/grader/sub/test_b.py"}
    assert {p: v for p, v in grader.items() if not p.startswith("/grader")} == agent
    assert not call(pool, sb, "shell", command="cat /grader/test_a.py").ok
    assert not call(pool, sb, "editor", path="/grader/test_a.py").ok
    assert b"assert" not in call(pool, sb, "python", code="print(open('/grader/test_a.py').read())").stdout


@pytest.mark.parametrize("tool, payload, path", [
    ("editor", {"path": "/grader/test_a.py", "content": "assert True"}, "/grader/test_a.py"),
    ("shell", {"command": "echo pass > /grader/new_test.py"}, "/grader/new_test.py"),
    ("python", {"code": "open('/grader/test_a.py', 'w').write('')"}, "/grader/test_a.py"),
])
def test_writes_into_the_grader_area_are_blocked_and_recorded(tool, payload, path):
    pool, _snap, (sb,) = booted()
    before = pool.grader_view(sb)
    e = err(lambda: call(pool, sb, tool, now=1234, call_id="evil-1", **payload))
    assert e.kind == "TestFileWrite" and path in str(e)
    assert pool.grader_view(sb) == before
    (flag,) = pool.tamper_flags
    assert (flag.sandbox, flag.path, flag.call_id, flag.now_ms) == (sb, path, "evil-1", 1234)
    assert call(pool, sb, "editor", path="/work/fine.txt", content="ok").ok and len(pool.tamper_flags) == 1


# ------------------------------------------------------------------------------ tools
def test_shell_python_editor_notes_and_lean():
    pool, _snap, (sb,) = booted()
    assert call(pool, sb, "shell", command="echo a  b").stdout == b"a b\n"
    assert call(pool, sb, "shell", command="cat /work/a.txt").stdout == b"alpha"
    assert not call(pool, sb, "shell", command="cat /work/missing").ok and not call(pool, sb, "shell", command="").ok
    assert call(pool, sb, "python", code="print(1 + 2 * 3)").stdout == b"7\n"
    assert call(pool, sb, "python", code="print('hi')").stdout == b"hi\n"
    assert call(pool, sb, "python", code="print(open('/work/data.txt').read())").stdout == b"1 2 3\n"
    assert call(pool, sb, "editor", path="/work/e.txt", content="body").ok
    got = call(pool, sb, "editor", path="/work/e.txt")
    assert got.stdout == b"body" and got.stdout_hash == hashlib.sha256(b"body").hexdigest() and got.tool == "editor"
    assert call(pool, sb, "notes", content="remember").ok and any(p.startswith("/notes/") for p in pool.agent_view(sb))
    assert call(pool, sb, "lean", code="theorem t : True := trivial").ok
    assert not call(pool, sb, "lean", code="theorem t : False := sorry").ok
    r = call(pool, sb, "shell", command="echo x", call_id="my-call")
    assert r.call_id == "my-call" and r.child_sandbox is None


def test_unknown_commands_fail_closed():
    pool, _snap, (sb,) = booted()
    before = pool.agent_view(sb)
    for cmd in ("rm -rf /", "make all", "pip install x"):
        r = call(pool, sb, "shell", command=cmd)
        assert not r.ok and r.stdout == b"" and r.stdout_hash == hashlib.sha256(b"").hexdigest()
    assert pool.agent_view(sb) == before
    assert err(lambda: call(pool, sb, "shell", command="nvidia-smi")).kind == "Backend"      # no GPU configured


def test_timeouts_come_from_the_request_or_the_pool_default():
    pool, _snap, (sb,) = booted(default_timeout_s=5)
    assert call(pool, sb, "shell", command="sleep 5").ok                               # at the limit is fine
    assert err(lambda: call(pool, sb, "shell", command="sleep 6")).kind == "Timeout"   # pool default
    assert call(pool, sb, "shell", command="sleep 30", timeout=30).ok                  # the request's own limit
    assert err(lambda: call(pool, sb, "shell", command="sleep 3", timeout=2)).kind == "Timeout"


# ------------------------------------------------------------------------------ egress
def test_network_tools_and_imports_fail_closed():
    pool, _snap, (sb,) = booted()
    for cmd in ("curl https://example.com", "wget https://example.com", "nc 1.1.1.1 80", "ssh host"):
        assert err(lambda: call(pool, sb, "shell", command=cmd)).kind == "EgressDenied"
    for code in ("import requests", "import urllib.request", "import socket"):
        assert err(lambda: call(pool, sb, "python", code=code)).kind in ("LiveInternet", "EgressDenied")


def test_the_browser_serves_only_offline_pages_up_to_the_cutoff():
    pages = {"https://docs.local/old": (b"old page", 10), "https://docs.local/at": (b"edge", 50), "https://docs.local/new": (b"new", 51)}
    pool, _snap, (sb,) = booted(offline_pages=pages, web_cutoff_unix_s=50)
    assert call(pool, sb, "browser", url="https://docs.local/old").stdout == b"old page"
    assert call(pool, sb, "browser", url="https://docs.local/at").stdout == b"edge"   # at the cutoff still served
    late = call(pool, sb, "browser", url="https://docs.local/new")
    assert not late.ok and b"new" not in late.stdout
    assert err(lambda: call(pool, sb, "browser", url="https://live.example/")).kind in ("EgressDenied", "LiveInternet")
    for url in ("", "file:///etc/passwd", "not a url"):
        assert not call(pool, sb, "browser", url=url).ok                              # no page, no exception


# ------------------------------------------------------------------------------ sub-agents
def test_spawn_forks_a_child_with_the_parents_files():
    pool, _snap, (sb,) = booted(capacity=2)
    call(pool, sb, "editor", path="/work/state.txt", content="S")
    r = call(pool, sb, "spawn", call_id="parent-call")
    assert r.ok and r.child_sandbox and r.child_sandbox != sb and r.call_id == "parent-call"
    assert pool.agent_view(r.child_sandbox)["/work/state.txt"] == b"S" and pool.live_count() == 2
    assert err(lambda: call(pool, sb, "spawn")).kind == "PoolExhausted"              # at capacity


# ------------------------------------------------------------------------------ GPU wall time
def test_gpu_work_needs_a_configured_device_and_stays_inside_its_budget():
    none, _snap, (sb,) = booted()
    assert err(lambda: call(none, sb, "shell", command="python train.py --device cuda")).kind == "Backend"
    assert err(lambda: call(none, sb, "python", code="print(1)", gpu=True)).kind == "Backend"
    pool, _snap, (sb,) = booted(gpu_walltime_s=10)
    assert call(pool, sb, "python", code="print(1)", gpu=True, work_s=4).ok
    assert call(pool, sb, "python", code="print(1)", gpu=True, work_s=6).ok            # 10 of 10 used
    assert err(lambda: call(pool, sb, "python", code="print(1)", gpu=True, work_s=1)).kind == "GpuTimeLimit"
    other = pool.fork_group(_snap, 1)[0]
    assert err(lambda: call(pool, other, "python", code="print(1)", gpu=True, work_s=11)).kind == "GpuTimeLimit"
    assert call(pool, other, "python", code="print(1)", gpu=True, work_s=10).ok        # budgets are per sandbox
    assert call(pool, sb, "python", code="print(2)").ok                                # CPU work is unaffected


# ------------------------------------------------------------------------------ microVM backend
def test_microvm_backend_records_its_paths_and_refuses_to_boot_without_images(tmp_path):
    kernel, rootfs = tmp_path / "vmlinux", tmp_path / "rootfs.ext4"
    kvm = tmp_path / "kvm"
    kvm.write_bytes(b"")
    pool = EN.Pool.firecracker(str(tmp_path / "fc.sock"), str(kernel), str(rootfs), EN.PoolConfig(), str(kvm))
    assert pool.backend == "firecracker" and EN.Pool().backend == "in_process"
    assert tuple(pool.firecracker_paths) == (str(tmp_path / "fc.sock"), str(kernel), str(rootfs))
    pool.register_image(EN.Image("img", {"/work/a": b"1"}))
    e = err(lambda: pool.snapshot_from_image("img"))
    assert e.kind == "Backend" and "kernel" in str(e)
    kernel.write_bytes(b"k")
    e = err(lambda: pool.snapshot_from_image("img"))
    assert e.kind == "Backend" and "rootfs" in str(e)
    rootfs.write_bytes(b"r")
    snap = pool.snapshot_from_image("img")
    assert len(pool.fork_group(snap)) == 16
    assert err(lambda: pool.fork_group("snap-none", 1)).kind == "UnknownSnapshot"
    missing = str(tmp_path / "no-kvm")
    assert err(lambda: EN.Pool.firecracker("s", str(kernel), str(rootfs), EN.PoolConfig(), missing)).kind == "Backend"
    assert os.path.exists(kvm)
