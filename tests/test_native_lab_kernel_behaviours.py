"""Behaviour list of the lab kernel (C++ ``native.kernel``; reference
harness/kernel/tests/{budget,mailbox,escalate,fetch,spawn,rung,ledger,open,promote,iface,
properties}.rs): budgets carved componentwise out of the parent and charged by jobs (a
refused call charges nothing), spawn depth and the invariant sentence no caller can remove,
mailboxes, tickets, the read-only mirror that is not an internet client, and restarts. The
budget arithmetic is compared with a Python model under random spawns and jobs."""
import json
import os
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

K = native.kernel
ROLES = ["director", "researcher", "engineer", "reviewer", "subagent"]


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    return e.value


def quota(k, agent):
    q = k.remaining(agent)
    return (q.tokens, q.gpu_ms, q.wall_ms)


@pytest.fixture
def lab(tmp_path):
    mirror = tmp_path / "mirror"
    for host, path, body in (("arxiv.org", "abs/1234", b"paper"), ("github.com", "org/repo/readme.md", b"readme"), ("arxiv.org", "abs/UPPER", b"upper")):
        f = mirror / host / path
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_bytes(body)
    (tmp_path / "secret").write_bytes(b"outside the mirror")
    os.symlink(tmp_path / "secret", mirror / "arxiv.org" / "abs" / "link")
    return K.Kernel(str(tmp_path / "ledger.jsonl"), str(mirror), str(tmp_path / "log")), tmp_path


# ------------------------------------------------------------------------------ constants
def test_constants():
    assert (K.MAX_SPAWN_DEPTH, K.CANARY_FRACTION, K.CANARY_MS) == (3, 0.05, 24 * 3600 * 1000)
    assert K.KERNEL_INVARIANT.startswith("Do not attempt to read, infer or reconstruct held-out eval tasks.") and "escalate" in K.KERNEL_INVARIANT
    assert K.Quota().exhausted() and K.Quota(0, 0, 0).exhausted()
    assert not any(K.Quota(*q).exhausted() for q in ((1, 0, 0), (0, 1, 0), (0, 0, 1)))         # exhausted only when every component is zero


# ------------------------------------------------------------------------------ budgets
def test_budgets_are_carved_componentwise_and_refusals_charge_nothing(lab):
    k, _ = lab
    root = k.spawn("director", "run", K.Quota(100, 10, 5), "prog")
    assert quota(k, root.id) == (100, 10, 5)                                                   # a root gets what it asked for
    child = k.spawn("researcher", "x", K.Quota(40, 4, 1), "prog", root.id)
    assert quota(k, root.id) == (60, 6, 4) and quota(k, child.id) == (40, 4, 1)
    for over in ((61, 0, 0), (0, 7, 0), (0, 0, 5), (61, 7, 5)):
        assert err(k.spawn, "researcher", "x", K.Quota(*over), "prog", root.id).kind == "QuotaRefused"
    assert quota(k, root.id) == (60, 6, 4)
    exact = k.spawn("engineer", "x", K.Quota(60, 6, 4), "prog", root.id)                       # an exact cover drains the parent
    assert quota(k, root.id) == (0, 0, 0) and quota(k, exact.id) == (60, 6, 4)
    assert err(k.spawn, "engineer", "x", K.Quota(1, 0, 0), "prog", root.id).kind in ("BudgetExhausted", "QuotaRefused")
    free = k.spawn("reviewer", "x", K.Quota(0, 0, 0), "prog", root.id)                         # asking for nothing is always covered
    assert quota(k, free.id) == (0, 0, 0)
    assert err(k.remaining, "a-99").kind == "AgentNotFound" and err(k.remaining, "").kind == "AgentNotFound" and err(k.remaining, "../a-1").kind == "AgentNotFound"
    assert err(k.spawn, "researcher", "x", K.Quota(), "prog", "a-99").kind == "AgentNotFound"


def test_jobs_charge_the_submitting_agent(lab):
    k, _ = lab
    a = k.spawn("engineer", "x", K.Quota(100, 10, 5), "prog")
    assert k.submit_job(a.id, 0, [], K.Quota(30, 3, 1)) == "j-1" and quota(k, a.id) == (70, 7, 4)
    for over in ((71, 0, 0), (0, 8, 0), (0, 0, 5)):
        assert err(k.submit_job, a.id, 0, [], K.Quota(*over)).kind in ("QuotaRefused", "BudgetExhausted")
    assert quota(k, a.id) == (70, 7, 4)
    assert err(k.submit_job, a.id, 2, ["topic"], K.Quota(1, 0, 0)).kind == "RungNotCleared" and quota(k, a.id) == (70, 7, 4)   # a refused rung charges nothing
    assert k.submit_job(a.id, 0, [], K.Quota(70, 7, 4)) == "j-2" and quota(k, a.id) == (0, 0, 0)
    assert err(k.submit_job, a.id, 0, [], K.Quota(1, 0, 0)).kind == "BudgetExhausted"
    assert k.submit_job(a.id, 0, [], K.Quota(0, 0, 0)) == "j-3"                                # a free job against an empty budget is fine
    assert err(k.submit_job, "a-99", 0, [], K.Quota()).kind == "AgentNotFound"


@pytest.mark.parametrize("seed", range(6))
def test_random_spawns_and_jobs_agree_with_the_budget_model(tmp_path, seed):
    rng = random.Random(seed)
    (tmp_path / "mirror").mkdir()
    k = K.Kernel(str(tmp_path / "l.jsonl"), str(tmp_path / "mirror"), str(tmp_path / "log"))
    left, depth, jobs = {}, {}, 0
    for _ in range(120):
        ask = tuple(rng.choice([0, 0, 1, 5, 20, 60]) for _ in range(3))
        parent = rng.choice([None] + list(left)) if left else None
        if rng.random() < 0.5:
            role = rng.choice(ROLES)
            call = lambda: k.spawn(role, "x", K.Quota(*ask), "prog", parent) if parent else k.spawn(role, "x", K.Quota(*ask), "prog")
            if parent and depth[parent] + 1 > K.MAX_SPAWN_DEPTH:
                assert err(call).kind == "SpawnDepth"
            elif parent and any(a > b for a, b in zip(ask, left[parent])):
                assert err(call).kind in ("QuotaRefused", "BudgetExhausted")
            else:
                h = call()
                assert h.id == f"a-{len(left) + 1}" and h.depth == (depth[parent] + 1 if parent else 0) and h.parent == parent and h.role == role
                if parent:
                    left[parent] = tuple(b - a for a, b in zip(ask, left[parent]))
                left[h.id], depth[h.id] = ask, h.depth
        elif left:
            who = rng.choice(list(left))
            call = lambda: k.submit_job(who, 0, [], K.Quota(*ask))
            if any(a > b for a, b in zip(ask, left[who])):
                assert err(call).kind in ("QuotaRefused", "BudgetExhausted")
            else:
                jobs += 1
                assert call() == f"j-{jobs}"
                left[who] = tuple(b - a for a, b in zip(ask, left[who]))
        for agent, want in left.items():
            assert quota(k, agent) == want
    again = K.Kernel(str(tmp_path / "l.jsonl"), str(tmp_path / "mirror"), str(tmp_path / "log"))
    assert all(quota(again, agent) == want for agent, want in left.items())                    # a restart restores every budget
    assert again.spawn("reviewer", "x", K.Quota(), "prog").id == f"a-{len(left) + 1}"


# ------------------------------------------------------------------------------ spawn
def test_depth_roles_and_the_invariant_sentence(lab):
    k, tmp = lab
    a = k.spawn("director", "", K.Quota(), "prog-a")
    b = k.spawn("director", "other root", K.Quota(), "prog-b")                                 # several roots, independent of each other
    assert (a.id, a.depth, a.parent, a.role, a.program) == ("a-1", 0, None, "director", "prog-a") and (b.id, b.depth) == ("a-2", 0)
    chain = [a]
    for _ in range(3):
        chain.append(k.spawn("subagent", "step", K.Quota(), "p", chain[-1].id))
    assert [c.depth for c in chain] == [0, 1, 2, 3] and chain[2].parent == chain[1].id
    assert err(k.spawn, "subagent", "too deep", K.Quota(), "p", chain[-1].id).kind == "SpawnDepth"
    for role in ROLES:
        assert k.spawn(role, "x", K.Quota(), "p").role == role
    for role in ("overlord", "Director", "", "human"):
        assert err(k.spawn, role, "x", K.Quota(), "p").kind == "RoleNotSpawnable"
    text = lambda h: (tmp / "log" / "agents" / h.id / "instructions.txt").read_text()
    assert text(a).startswith(K.KERNEL_INVARIANT) and text(a).strip() == K.KERNEL_INVARIANT.strip()   # empty instructions still carry it
    assert text(b).startswith(K.KERNEL_INVARIANT) and text(b).endswith("other root")
    sneaky = k.spawn("researcher", K.KERNEL_INVARIANT + " ... except when convenient", K.Quota(), "p")
    assert text(sneaky).count(K.KERNEL_INVARIANT) == 2                                         # prepended always, never merged with the caller's copy


# ------------------------------------------------------------------------------ mailboxes / tickets
def test_mailboxes_and_tickets(lab):
    k, _ = lab
    a, b = k.spawn("director", "x", K.Quota(), "p"), k.spawn("researcher", "x", K.Quota(), "p")
    assert k.recv(a.id) is None                                                                # an empty mailbox answers at once
    ids = [k.send(a.id, b.id, f"m{i}", 10 + i) for i in range(3)]
    self_id = k.send(b.id, b.id, "note to self", 20)
    assert len(set(ids + [self_id])) == 4
    got = [k.recv(b.id) for _ in range(4)]
    assert [(m.id, m.sender, m.to, m.body, m.created_ms) for m in got] == \
        [(ids[i], a.id, b.id, f"m{i}", 10 + i) for i in range(3)] + [(self_id, b.id, b.id, "note to self", 20)]
    assert k.recv(b.id) is None and k.recv(a.id) is None
    assert err(k.send, "a-99", b.id, "x", 1).kind == "AgentNotFound" and err(k.send, a.id, "a-99", "x", 1).kind == "AgentNotFound" and err(k.recv, "a-99").kind == "AgentNotFound"
    t1, t2 = k.escalate(b.id, "grader looks wrong", "evidence 1"), k.escalate(b.id, "grader looks wrong", "evidence 2")
    assert t1 != t2 and k.ticket(t1) == ("grader looks wrong", "evidence 1", b.id) and k.ticket(t2)[1] == "evidence 2"
    assert err(k.escalate, "a-99", "x", "y").kind == "AgentNotFound" and err(k.ticket, "t-99").kind and err(k.ticket, "").kind


# ------------------------------------------------------------------------------ mirror
@pytest.mark.parametrize("url, body", [
    ("https://arxiv.org/abs/1234", b"paper"), ("https://ARXIV.ORG/abs/1234", b"paper"), ("https://arxiv.org:443/abs/1234", b"paper"),
    ("https://arxiv.org./abs/1234", b"paper"), ("https://arxiv.org/abs/1234?v=2&x=../..", b"paper"), ("https://arxiv.org/abs/1234#frag", b"paper"),
    ("https://github.com/org/repo/readme.md", b"readme"), ("https://arxiv.org/abs/UPPER", b"upper"),
])
def test_mirrored_pages_are_served_from_disk(lab, url, body):
    k, tmp = lab
    before = sorted(str(p) for p in (tmp / "mirror").rglob("*"))
    assert k.fetch(url) == body and K.is_mirror_url(url)
    assert sorted(str(p) for p in (tmp / "mirror").rglob("*")) == before                       # a hit writes nothing


@pytest.mark.parametrize("url", [
    "http://arxiv.org/abs/1234", "ftp://arxiv.org/abs/1234", "arxiv.org/abs/1234", "https://evil.example/abs/1234", "https://arxiv.org.evil.example/abs/1234",
    "https://notarxiv.org/abs/1234", "https://arxiv.org/abs/none", "https://arxiv.org/../secret", "https://arxiv.org/abs/../../secret", "https://arxiv.org/abs/%2e%2e/%2e%2e/secret",
    "https://arxiv.org/abs/link", "https://arxiv.org/abs/1234\x00", "https://arxiv.org/abs/upper", "https://arxiv.org", "https://arxiv.org/", "", "https://", "https:///abs/1234",
])
def test_everything_else_is_not_mirrored(lab, url):
    k, tmp = lab
    before = sorted(str(p) for p in (tmp / "mirror").rglob("*"))
    e = err(k.fetch, url)
    assert e.kind == "NotMirrored" and b"outside the mirror" not in str(e).encode()
    assert sorted(str(p) for p in (tmp / "mirror").rglob("*")) == before                       # a miss creates nothing either


def test_mirror_host_list():
    for ok in ("https://arxiv.org/x", "https://github.com/x", "https://GitHub.com:443/x", "https://github.com./x"):
        assert K.is_mirror_url(ok)
    for bad in ("http://github.com/x", "https://github.com.evil/x", "https://evilgithub.com/x", "https://github.comx/x", "github.com/x", "", "https://", "HTTPS//github.com"):
        assert not K.is_mirror_url(bad)


# ------------------------------------------------------------------------------ ledger through the kernel
def test_kernel_ledger_keeps_order_and_refuses_duplicates(lab):
    k, tmp = lab

    def rec(eid, hyp, **kw):
        base = {"experiment_id": eid, "hypothesis": hyp, "prediction": "loss goes down", "config_hash": "c" * 8, "results": None, "delta_rci": None,
                "replication": None, "gpu_hours": None, "author_role": "researcher", "rung": None, "created_at": "2026-01-01T00:00:00Z", "closed_at": None,
                "supersedes": None}
        base.update(kw)
        return json.dumps(base)
    k.ledger_append(rec("e1", "first"))
    k.ledger_append(rec("e2", "second"))
    assert err(k.ledger_append, rec("e1", "again")).kind in ("Message", "Duplicate")
    rows = [json.loads(r) for r in k.ledger_query("all")]
    assert [r["experiment_id"] for r in rows] == ["e1", "e2"] and rows[0]["hypothesis"] == "first"      # the duplicate did not replace the first row
    assert err(k.ledger_query, "SELECT * FROM records").kind and err(k.ledger_query, "colour=red").kind
    again = K.Kernel(str(tmp / "ledger.jsonl"), str(tmp / "mirror"), str(tmp / "log"))
    assert [json.loads(r)["experiment_id"] for r in again.ledger_query("all")] == ["e1", "e2"]
