"""Behaviour list of the worker mesh (C++ ``native.mesh``; reference
harness/mesh/tests/{create_open,local_mesh,watches,gossip,pull,freeze,partition,untrusted}.rs):
the watcher ring, gossip of adverts only on ticks and only across connected nodes, pulls that
scan past tasks a node cannot run, the signed freeze and how it spreads across a healed
partition, untrusted nodes. ``caps_satisfy`` and the gossip are compared with Python models
under random inputs."""
import json
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

M, L = native.mesh, native.leases


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def caps(**kw):
    return M.Capabilities(**kw)


def task(q, tid, requires=None, now=0):
    q.enqueue(tid, json.dumps({} if requires is None else {"requires": requires}), now)


def satisfies(c, payload):
    """Python model: every stated requirement must be met; a malformed ``requires`` fits nothing."""
    req = payload.get("requires")
    if req is None:
        return True
    if not isinstance(req, dict):
        return False
    return (c["gpus"] >= req.get("gpus", 0) and c["cpus"] >= req.get("cpus", 0) and (c["kvm"] or not req.get("kvm", False))
            and all(p in c["providers"] for p in req.get("providers", [])))


# ------------------------------------------------------------------------------ create / open / start
def test_create_open_and_start_rules(tmp_path):
    assert (M.MIN_RING, M.MIN_WATCHERS) == (3, 2)
    m = M.Mesh.create(str(tmp_path / "n"), "a", "key-a")
    assert not m.is_frozen() and m.adverts == [] and (tmp_path / "n").is_dir()
    err(lambda: M.Mesh.create(str(tmp_path / "n"), "a", "key-a"))
    err(lambda: M.Mesh.open(str(tmp_path / "missing"), "a", "key-a"))
    assert not M.Mesh.open(str(tmp_path / "n"), "a", "key-a").is_frozen()
    for n in (0, 1, 2):
        assert err(lambda: M.LocalMesh.start(n, str(tmp_path / f"few{n}"))).kind == "TooFewNodes"
    lm = M.LocalMesh.start(3, str(tmp_path / "three"))
    assert sorted(p.name for p in (tmp_path / "three").iterdir()) == ["0", "1", "2"]            # one directory per slot
    assert all(not lm.get(i).is_frozen() for i in range(3))
    with pytest.raises((NativeError, IndexError)):
        lm.get(3)


@pytest.mark.parametrize("n", [3, 4, 5, 6])
def test_watcher_ring(tmp_path, n):
    lm = M.LocalMesh.start(n, str(tmp_path / "m"))
    ring = [(w.watcher, w.watchee) for w in lm.get(0).watches]
    assert len(ring) == n * M.MIN_WATCHERS and all(a != b for a, b in ring)
    for node in map(str, range(n)):
        assert sum(1 for _, e in ring if e == node) == 2 and sum(1 for w, _ in ring if w == node) == 2
        assert sorted(w for w, e in ring if e == node) == sorted({str((int(node) + 1) % n), str((int(node) + 2) % n)})   # the next two on the ring
    assert all([(w.watcher, w.watchee) for w in lm.get(i).watches] == ring for i in range(n))
    lm.partition([0])
    lm.tick(1)
    assert [(w.watcher, w.watchee) for w in lm.get(1).watches] == ring                          # isolation does not shrink the ring


# ------------------------------------------------------------------------------ gossip
def test_adverts_travel_only_on_ticks_and_only_between_connected_nodes(tmp_path):
    lm = M.LocalMesh.start(4, str(tmp_path / "m"))
    ad = lm.get(0).advertise(caps(gpus=2, cpus=4, kvm=True, providers=["x"]), 5)
    assert (ad.node, ad.key, ad.at, ad.caps.gpus, ad.caps.cpus, ad.caps.kvm, list(ad.caps.providers)) == ("0", "key-0", 5, 2, 4, True, ["x"])
    assert [a.node for a in lm.get(0).adverts] == ["0"] and lm.get(1).adverts == []
    lm.tick(6)
    assert all([a.node for a in lm.get(i).adverts] == ["0"] for i in range(4))
    lm.get(0).advertise(caps(gpus=8), 7)                                                        # a second advert replaces the first
    lm.tick(8)
    assert all([(a.node, a.caps.gpus, a.at) for a in lm.get(i).adverts] == [("0", 8, 7)] for i in range(4))
    lm.partition([3])
    lm.get(3).advertise(caps(gpus=1), 9)
    lm.get(1).advertise(caps(cpus=2), 9)
    lm.tick(10)
    assert sorted(a.node for a in lm.get(0).adverts) == ["0", "1"] and sorted(a.node for a in lm.get(3).adverts) == ["0", "3"]
    lm.tick(11)
    assert sorted(a.node for a in lm.get(2).adverts) == ["0", "1"]                              # ticking alone does not heal
    lm.heal()
    assert sorted(a.node for a in lm.get(2).adverts) == ["0", "1"]                              # nor healing without a tick
    lm.tick(12)
    assert all(sorted(a.node for a in lm.get(i).adverts) == ["0", "1", "3"] for i in range(4))
    lm.partition([0, 1])
    lm.partition([2])                                                                           # a new partition replaces the old one
    lm.get(0).advertise(caps(gpus=3), 13)
    lm.tick(14)
    assert [a.caps.gpus for a in lm.get(1).adverts if a.node == "0"] == [3] and [a.caps.gpus for a in lm.get(2).adverts if a.node == "0"] == [8]


@pytest.mark.parametrize("seed", range(4))
def test_random_gossip_matches_a_model(tmp_path, seed):
    rng = random.Random(seed)
    n = rng.choice([3, 4, 5])
    lm = M.LocalMesh.start(n, str(tmp_path / "m"))
    view = [dict() for _ in range(n)]                                                           # node -> {advertiser: (at, gpus)}
    isolated = set()
    for now in range(1, 60):
        op = rng.choice(["advertise", "advertise", "tick", "tick", "partition", "heal"])
        if op == "advertise":
            i, g = rng.randrange(n), rng.randint(0, 9)
            lm.get(i).advertise(caps(gpus=g), now)
            view[i][str(i)] = (now, g)
        elif op == "partition":
            isolated = set(rng.sample(range(n), rng.randint(0, n - 1)))
            lm.partition(sorted(isolated))
        elif op == "heal":
            isolated = set()
            lm.heal()
        else:
            lm.tick(now)
            group = [i for i in range(n) if i not in isolated]
            merged = {}
            for i in group:
                for k, v in view[i].items():
                    if k not in merged or v[0] > merged[k][0]:
                        merged[k] = v
            for i in group:
                view[i] = dict(merged)
        for i in range(n):
            assert {a.node: (a.at, a.caps.gpus) for a in lm.get(i).adverts} == view[i]


# ------------------------------------------------------------------------------ pull
def test_pull_claims_what_the_node_can_run_in_queue_order(tmp_path):
    lm = M.LocalMesh.start(3, str(tmp_path / "m"))
    q = L.Queue.create(str(tmp_path / "q"))
    assert lm.get(0).pull(q, 0) is None
    task(q, "gpu", {"gpus": 1})
    assert lm.get(0).pull(q, 1) is None and q.get("gpu").state == "Queued"                     # no advert yet: zero GPUs, one CPU
    lm.get(0).advertise(caps(gpus=0, cpus=2), 1)
    lm.get(1).advertise(caps(gpus=1, cpus=2, kvm=True, providers=["a", "b"]), 1)
    assert lm.get(0).pull(q, 2) is None
    lease = lm.get(1).pull(q, 3)
    assert (lease.task_id, lease.worker_id, lease.attempt) == ("gpu", "1", 1)                   # the worker is the node id
    for tid, req in (("g2", {"gpus": 2}), ("kvm", {"kvm": True}), ("cpu4", {"cpus": 4}), ("prov", {"providers": ["a", "c"]}), ("fit", {"cpus": 2}), ("any", None)):
        task(q, tid, req, 4)
    before = q.log_len()
    assert lm.get(0).pull(q, 5).task_id == "fit" and q.log_len() == before + 1                  # scanned past four misfits, wrote one event
    assert lm.get(0).pull(q, 6).task_id == "any" and lm.get(0).pull(q, 7) is None
    assert lm.get(1).pull(q, 8).task_id == "kvm" and lm.get(1).pull(q, 9) is None
    assert q.queued_ids() == ["g2", "cpu4", "prov"]                                             # nobody fits these; their order is kept
    lm.get(1).advertise(caps(gpus=2, cpus=4, providers=["c", "a"]), 10)
    assert [lm.get(1).pull(q, 11 + i).task_id for i in range(3)] == ["g2", "cpu4", "prov"]


@pytest.mark.parametrize("seed", range(5))
def test_caps_satisfy_and_pull_agree_with_the_model(tmp_path, seed):
    rng = random.Random(seed)
    lm = M.LocalMesh.start(3, str(tmp_path / "m"))
    q = L.Queue.create(str(tmp_path / "q"))
    mine = dict(gpus=rng.randint(0, 3), cpus=rng.randint(1, 4), kvm=rng.random() < 0.5, providers=rng.sample(["a", "b", "c"], rng.randint(0, 3)))
    lm.get(0).advertise(caps(**mine), 0)
    payloads = []
    for i in range(25):
        req = {}
        if rng.random() < 0.5:
            req["gpus"] = rng.randint(0, 3)
        if rng.random() < 0.5:
            req["cpus"] = rng.randint(0, 5)
        if rng.random() < 0.4:
            req["kvm"] = rng.random() < 0.5
        if rng.random() < 0.4:
            req["providers"] = rng.sample(["a", "b", "c"], rng.randint(0, 2))
        payload = rng.choice([{"requires": req}, {"requires": req, "other": 1}, {}, {"requires": 3}, {"requires": "gpu"}]) if rng.random() < 0.3 else {"requires": req}
        payloads.append(payload)
        q.enqueue(f"t{i}", json.dumps(payload), 0)
        assert M.caps_satisfy(caps(**mine), json.dumps(payload)) == satisfies(mine, payload)
    want = [f"t{i}" for i, p in enumerate(payloads) if satisfies(mine, p)]
    got = []
    while (lease := lm.get(0).pull(q, 1)) is not None:
        got.append(lease.task_id)
    assert got == want and q.queued_ids() == [f"t{i}" for i, p in enumerate(payloads) if not satisfies(mine, p)]


# ------------------------------------------------------------------------------ freeze
def test_freeze_needs_a_good_signature_and_stops_work_for_good(tmp_path):
    lm = M.LocalMesh.start(3, str(tmp_path / "m"))
    q = L.Queue.create(str(tmp_path / "q"))
    task(q, "t")
    node = lm.get(0)
    for bad in (b"nope", b"", b"stop "):
        assert err(lambda: node.freeze(M.Freeze("stop", "key-0", bad))).kind == "BadSignature" and not node.is_frozen()
    node.freeze(M.Freeze("stop", "key-0", b"stop"))
    node.freeze(M.Freeze("stop", "key-0", b"stop"))                                             # again: no error
    assert node.is_frozen()
    assert err(lambda: node.pull(q, 1)).kind == "Frozen" and err(lambda: node.advertise(caps(), 1)).kind == "Frozen"
    assert q.get("t").state == "Queued"
    assert M.Mesh.open(str(tmp_path / "m" / "0"), "0", "key-0").is_frozen()                     # survives a restart
    other = M.Mesh.create(str(tmp_path / "solo"), "s", "ks")
    other.freeze(M.Freeze("", "ks", b""))                                                       # the empty payload signs as empty
    assert other.is_frozen()


def test_freeze_spreads_on_ticks_and_reaches_a_partitioned_node_after_healing(tmp_path):
    lm = M.LocalMesh.start(4, str(tmp_path / "m"))
    q = L.Queue.create(str(tmp_path / "q"))
    task(q, "t")
    lm.partition([2])
    lm.tick(1)
    assert not any(lm.get(i).is_frozen() for i in range(4))                                     # ticking a split mesh freezes nobody
    lm.get(0).freeze(M.Freeze("halt", "key-0", b"halt"))
    assert not lm.get(1).is_frozen()
    lm.tick(2)
    assert [lm.get(i).is_frozen() for i in range(4)] == [True, True, False, True]
    assert lm.get(2).pull(q, 3).task_id == "t"                                                  # the cut-off node still works
    lm.heal()
    assert not lm.get(2).is_frozen()
    lm.tick(4)
    assert lm.get(2).is_frozen() and err(lambda: lm.get(2).pull(q, 5)).kind == "Frozen"
    back = M.LocalMesh.start(3, str(tmp_path / "m2"))
    back.partition([1])
    back.get(1).freeze(M.Freeze("x", "key-1", b"x"))                                            # frozen while alone
    back.tick(1)
    assert [back.get(i).is_frozen() for i in range(3)] == [False, True, False]
    back.heal()
    back.tick(2)
    assert all(back.get(i).is_frozen() for i in range(3))


def test_untrusted_nodes_may_advertise_but_never_pull(tmp_path):
    q = L.Queue.create(str(tmp_path / "q"))
    guest = M.Mesh.create(str(tmp_path / "g"), "g", "kg", False)
    assert err(lambda: guest.pull(q, 0)).kind == "Untrusted"                                    # even with nothing to pull
    task(q, "t")
    assert guest.advertise(caps(gpus=8), 1).node == "g"
    assert err(lambda: guest.pull(q, 2)).kind == "Untrusted" and q.get("t").state == "Queued"
    assert err(lambda: M.Mesh.open(str(tmp_path / "g"), "g", "kg", False).pull(q, 3)).kind == "Untrusted"
