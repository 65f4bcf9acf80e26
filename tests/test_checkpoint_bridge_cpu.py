"""Trainer <-> native checkpoint bridge on CPU, with a stand-in for the GPU trainer that has
the same flat-buffer layout."""
import types

import pytest
import torch

from prometheus_b200 import checkpoint, model


def _fake_trainer(seed):
    g = torch.Generator().manual_seed(seed)
    W = types.SimpleNamespace
    weights = {
        "layers.0.q": W(name="layers.0.q", shape=(4, 6), group="muon", off=0),
        "layers.0.o": W(name="layers.0.o", shape=(6, 4), group="muon", off=24),
        "embed": W(name="embed", shape=(8, 4), group="adam", off=0),
        "final_norm": W(name="final_norm", shape=(4,), group="vec", off=0),
    }
    r = lambda n: torch.randn(n, generator=g)
    tr = W(weights=weights, cfg=model.tiny_config(), device=torch.device("cpu"), world=1, rank=0,
           sym=None, step_count=7,
           muon_master=r(48), muon_mom=r(48), adam_master=r(32), adam_m=r(32), adam_v=r(32).abs(),
           vec_master=r(4), vec_m=r(4), vec_v=r(4).abs(),
           muon_lp=torch.zeros(48, dtype=torch.bfloat16), adam_lp=torch.zeros(32, dtype=torch.bfloat16))
    return tr


def test_capture_apply_roundtrip_and_manifest(tmp_path):
    a, b = _fake_trainer(0), _fake_trainer(1)
    ck = checkpoint.capture(a, loader_state={"epoch": 1, "cursor": 5}, created_at="2026-01-01T00:00:00Z")
    m = ck.manifest
    assert m.step == 7 and len(m.checkpoint_id) == 64
    assert [w.name for w in m.weights] == list(a.weights) + ["rng.torch.cpu.0"]   # generator bytes ride along
    assert {o.name: o.kind for o in m.optimizer} == {
        "layers.0.q.mom": "muon", "layers.0.o.mom": "muon", "embed.m": "adamw", "embed.v": "adamw",
        "final_norm.m": "adamw", "final_norm.v": "adamw"}
    # same state -> same id; different state -> different id
    assert checkpoint.capture(a, created_at="x").manifest.checkpoint_id == m.checkpoint_id
    assert checkpoint.capture(b).manifest.checkpoint_id != m.checkpoint_id
    saver = checkpoint.TrainerCheckpointer(str(tmp_path / "s"))
    cid = saver.save_persistent(a, wait=True, loader_state={"epoch": 1, "cursor": 5})
    assert cid == m.checkpoint_id
    assert saver.restore(b, cid) == {"cursor": 5, "epoch": 1}
    for name in ("muon_master", "muon_mom", "adam_master", "adam_m", "adam_v", "vec_master", "vec_m",
                 "vec_v"):
        assert torch.equal(getattr(a, name), getattr(b, name)), name
    assert b.step_count == 7
    assert torch.equal(b.muon_lp, a.muon_master.to(torch.bfloat16))
    # the generator state itself is restored, not only its hash: the next draws repeat
    torch.manual_seed(1234)
    ck2 = checkpoint.capture(a)
    first = torch.rand(4)
    torch.manual_seed(99)
    checkpoint.apply(b, ck2)
    assert torch.equal(torch.rand(4), first)
    # in-memory path
    c = _fake_trainer(2)
    saver.save_memory(a)
    saver.restore(c)
    assert torch.equal(c.adam_v, a.adam_v)


def test_apply_rejects_other_model_and_bad_sizes():
    a = _fake_trainer(0)
    ck = checkpoint.capture(a)
    other = _fake_trainer(0)
    other.cfg = model.with_overrides(model.tiny_config(), vocab_size=512)
    with pytest.raises(ValueError):
        checkpoint.apply(other, ck)
    short = _fake_trainer(0)
    short.weights["embed"].shape = (9, 4)
    short.adam_master = torch.zeros(36)
    with pytest.raises(ValueError):
        checkpoint.apply(short, ck)


def _free_port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_rank_restore_worker(rank, world, port, root, out):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a = _fake_trainer(0)                   # every rank holds the same (already complete) state
        a.world, a.rank, a.pg = world, rank, None
        saver = checkpoint.TrainerCheckpointer(root if rank == 0 else None)   # only rank 0 has the store
        mem_id = saver.save_memory(a)
        b = _fake_trainer(5 + rank)
        b.world, b.rank, b.pg = world, rank, None
        saver.restore(b)                       # newest in-memory replica lives on rank 0 only
        same_mem = all(torch.equal(getattr(a, n), getattr(b, n))
                       for n in ("muon_master", "muon_mom", "adam_m", "adam_v", "vec_master"))
        cid = saver.save_persistent(a, wait=True, loader_state={"cursor": 3})
        c = _fake_trainer(9 + rank)
        c.world, c.rank, c.pg = world, rank, None
        loader = saver.restore(c, cid)         # rank 1's own store is empty: it must still succeed
        same_disk = torch.equal(a.adam_master, c.adam_master) and c.step_count == a.step_count
        try:
            saver.restore(c, "f" * 64)
            raised = False
        except RuntimeError:
            raised = True                      # rank 0's error reaches every rank; nobody hangs
        out.put((rank, mem_id == cid, same_mem, same_disk, loader, raised))
    finally:
        dist.destroy_process_group()


def test_two_rank_restore_reaches_every_rank(tmp_path):
    """Only rank 0 keeps replicas and reads the store; a rollback or a resume must still restore
    every rank, and a failed restore must fail everywhere instead of leaving ranks in a barrier."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_two_rank_restore_worker, args=(r, 2, port, str(tmp_path / "s"), out))
             for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert got == [(r, True, True, True, {"cursor": 3}, True) for r in range(2)]
