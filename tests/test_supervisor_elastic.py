"""Run supervision on the host: watchdog status -> drained replica -> higher gradient
accumulation; checksum vote over replicated state; tracer / metric wiring; and gloo CPU ranks
in which one rank leaves between steps and a flipped byte in one rank's copy is voted out."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from prometheus_b200 import native, supervisor
from prometheus_b200.elastic import ElasticMembership


def _sup(world=4, rank=0, **kw):
    base = dict(world=world, rank=rank, tokens_per_step=4096, microbatch_tokens=512, sdc_period_steps=2,
                nvtx=False)
    base.update(kw)
    return supervisor.RunSupervisor(**base)


def test_device_timeout_status_drains_the_replica_and_raises_grad_accumulation():
    s = _sup()
    assert s.grad_accumulation() == 2 and len(s.live()) == 4          # 4096 / (4 * 512)
    out = s.after_step(1, 100.0, status_code=0)
    assert out["state"] == "Live" and out["grad_accumulation"] == 2
    out = s.after_step(2, 100.0, status_code=2, replica="r3")         # PB_TIMEOUT_FLAG latched on r3
    assert "r3" not in out["live"] and out["grad_accumulation"] == 3  # ceil(4096 / (3 * 512))
    assert s.controller.health_events() == 1
    assert str(s.controller.replica_state("r3")).endswith("Dead")      # drained for good
    # a replica that leaves is dead, and the survivors carry its share
    assert s.replica_left("r2")["grad_accumulation"] == 4


def test_single_replica_timeout_is_reported_but_cannot_be_drained():
    s = _sup(world=1)
    out = s.after_step(1, 5.0, status_code=2)
    assert out["live"] == ["r0"] and s.last_health_error and "no live replicas" in s.last_health_error


def test_collective_bracket_and_watchdog_tick():
    s = _sup(collective_watchdog_ms=50)
    with s.collective("grad_sync"):
        assert s.controller.open_collectives() == 1
    assert s.controller.open_collectives() == 0
    # a collective that never ends is seen by tick() once its budget is over
    s.controller.begin_collective("grad_sync", "r1", 1000)
    s.controller.tick(1000 + 49)
    assert "r1" in s.live()
    s.controller.tick(1000 + 51)
    assert "r1" not in s.live()


def test_checksum_matches_between_forms_and_detects_a_flipped_bit():
    t = torch.randn(1000)
    a = supervisor.checksum64(t)
    assert a == supervisor.checksum64(t.clone()) and 0 <= a < 2 ** 64
    u = t.clone()
    u.view(torch.int32)[123] ^= 1 << 7
    assert supervisor.checksum64(u) != a
    swapped = t.clone()
    swapped[[0, 1]] = swapped[[1, 0]]                 # position-weighted: a swap is seen too
    assert supervisor.checksum64(swapped) != a
    assert supervisor.checksum64(t.to(torch.bfloat16).view(torch.int32)) == \
        supervisor.checksum64(t.to(torch.bfloat16).clone().view(torch.int32))
    with pytest.raises(ValueError):
        supervisor.checksum64(torch.zeros(3, dtype=torch.bfloat16))


def test_sdc_vote_quarantines_the_odd_replica():
    s = _sup(world=4)
    good = torch.arange(64, dtype=torch.float32)
    bad = good.clone()
    bad.view(torch.uint8)[17] ^= 0x10                  # one flipped bit in rank 2's host copy
    per_rank = [good, good, bad, good]
    hashes = [{"vec.master": f"{supervisor.checksum64(t):016x}"} for t in per_rank]
    assert s.sdc_due(2) and not s.sdc_due(3)
    gone = s.sdc_probe(2, {"vec.master": good}, exchange=lambda local: hashes)
    assert gone == ["r2"] and "r2" not in s.live()
    assert str(s.controller.replica_state("r2")).endswith("Quarantined")
    # nothing else is voted out when all agree
    assert s.sdc_probe(4, {"vec.master": good}, exchange=lambda local: [hashes[0]] * 4) == []


def test_phases_and_metrics_reach_the_native_objects(tmp_path):
    sink = tmp_path / "metrics.jsonl"
    s = _sup(metric_sink=str(sink))
    with s.phase("step"):
        with s.phase("forward_backward"):
            assert s.tracer.current() == "forward_backward" and s.tracer.depth() == 2
    assert s.tracer.depth() == 0 and set(s.phase_ms) == {"step", "forward_backward"}
    s.record(3, {"train.loss": 2.5, "train.mfu": 0.5, "comm.exposed_ms": 1.25, "skip": None},
             {"preset": "tiny"})
    s.record(3, supervisor.moe_load_stats(torch.tensor([[0.5, 0.25, 0.125, 0.125]])))
    assert s.metrics.get("train.mfu", {"preset": "tiny"}) == 0.5
    assert s.metrics.get("moe.load.max", {}) == 2.0 and s.metrics.get("moe.load.mean", {}) == 1.0
    assert s.log.series("comm.exposed_ms", {"preset": "tiny"}) == [(3, 1.25)]
    s.close()
    text = sink.read_text()
    assert "train.loss" in text and "comm.exposed_ms" in text


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _elastic_worker(rank, world, port, out):
    """Data-parallel SGD on a linear model over gloo. Rank 2 leaves after step 2 (between
    steps); the survivors learn of it from the store, raise their gradient accumulation so the
    batch per optimizer step is unchanged, and finish on a group of their own. At step 4 rank 1
    holds a copy of the replicated weight with one flipped bit; the vote quarantines it."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        store = dist.distributed_c10d._get_default_store()
        micro, total = 2, 12                          # samples per micro-batch / per optimizer step
        sup = supervisor.RunSupervisor(world=world, rank=rank, tokens_per_step=total,
                                       microbatch_tokens=micro, sdc_period_steps=4, nvtx=False)
        mem = ElasticMembership(store, rank, world, sup)
        g = torch.Generator().manual_seed(0)
        X, Y = torch.randn(6, total, 4, generator=g), torch.randn(6, total, 1, generator=g)
        w = torch.zeros(4, 1)
        accum_seen, quarantined = [], []
        for step in range(1, 7):
            info = mem.refresh(step)
            live, accum, group = info["live"], info["grad_accumulation"], info["group"]
            accum_seen.append(accum)
            if rank not in live:
                break
            me = live.index(rank)
            # this rank's share of the step's batch: `accum` micro-batches
            mine = slice(me * accum * micro, (me + 1) * accum * micro)
            grad = torch.zeros_like(w)
            for k in range(accum):
                xs = X[step - 1, mine][k * micro:(k + 1) * micro]
                ys = Y[step - 1, mine][k * micro:(k + 1) * micro]
                grad += 2 * xs.t() @ (xs @ w - ys) / total
            with sup.collective("grad_sync"):
                dist.all_reduce(grad, group=group)
            w = w - 0.05 * grad
            sup.after_step(step, 10.0)
            mem.heartbeat(step)
            if sup.sdc_due(step):
                probe = w.clone()
                if rank == 1:
                    probe.view(torch.int32)[0] ^= 1 << 3      # silent corruption of one copy
                every = [None] * len(live)
                dist.all_gather_object(every, {"w": f"{supervisor.checksum64(probe):016x}"}, group=group)
                full = [None] * world
                for r, h in zip(live, every):
                    full[r] = h
                quarantined = sup.sdc_probe(step, {"w": probe}, exchange=lambda local: full)
            leaving = (rank == 2 and step == 2) or sup.me in quarantined
            if leaving:
                mem.leave(step)                        # announced before the step's last meeting
            if group is not None:
                dist.barrier(group=group)
            else:
                dist.barrier()
            if leaving:
                break                                  # between steps, nothing in flight
        out.put((rank, accum_seen, w.flatten().tolist(), quarantined, sup.live()))
    finally:
        dist.destroy_process_group()


def test_gloo_ranks_a_rank_leaves_and_a_corrupt_copy_is_voted_out():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_elastic_worker, args=(r, 3, port, out)) for r in range(3)]
    for p in procs:
        p.start()
    got = {r: rest for r, *rest in (out.get(timeout=180) for _ in procs)}
    for p in procs:
        p.join(60)
    # 12 samples per step, micro-batches of 2: 3 ranks -> 2 micro-batches each; 2 ranks -> 3
    # each; after the vote at step 4 rank 0 is alone and runs all 6
    assert got[0][0] == [2, 2, 3, 3, 6, 6] and got[1][0] == [2, 2, 3, 3]
    assert got[2][0] == [2, 2]
    # the survivors hold identical weights, equal to plain SGD on the whole batch every step
    g = torch.Generator().manual_seed(0)
    X, Y = torch.randn(6, 12, 4, generator=g), torch.randn(6, 12, 1, generator=g)
    w = torch.zeros(4, 1)
    for s in range(6):
        w = w - 0.05 * (2 * X[s].t() @ (X[s] @ w - Y[s]) / 12)
    assert torch.allclose(torch.tensor(got[0][1]), w.flatten(), rtol=1e-5, atol=1e-6)
    # the flipped bit in rank 1's copy: with two live replicas and two different hashes there
    # is no majority and the first reporter's value stands, so r1 is quarantined on both ranks
    assert got[0][2] == ["r1"] and got[1][2] == ["r1"] and got[0][3] == ["r0"]
