"""Parallelism on CPU: mesh arithmetic, FSDP shard math, schedules, ring attention, the
delta-state hand-off, and two-process gloo runs of the pipeline and the CP paths."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from prometheus_b200 import kernels, model
from prometheus_b200 import parallel as P
from prometheus_b200.parallel import cp, fsdp


def test_mesh_and_coords():
    spec = P.tiny_mesh()
    assert spec.n_devices == 8 and P.device_ids(spec) == tuple(range(8))
    assert [P.coord_of(d, spec) for d in (0, 1, 2, 5, 7)] == \
        [(0, 0, 0, 0), (0, 0, 1, 0), (0, 1, 0, 0), (1, 0, 1, 0), (1, 1, 1, 0)]
    with pytest.raises(P.MeshError):
        P.validate_mesh(P.MeshSpec(1, 2, 4, 1, 1))
    with pytest.raises(P.MeshError):
        P.coord_of(8, spec)
    assert P.fsdp_partition(P.ParamKind.ROUTED_EXPERT).axes == (None,)
    assert P.fsdp_partition(P.ParamKind.ATTENTION).axes == ("fsdp",)
    assert P.box_mesh(8, cp=8).cp == 8 and P.context_parallel_on(131072, 4096)


def test_pipeline_stage_layers_balances_recurrent_tail():
    r = P.pipeline_stage_layers(8, 2, 2, 4)
    assert (r[0].start, r[-1].end) == (0, 8) and r[0].end == r[1].start
    cost = lambda a: sum(4 if i >= 6 else 1 for i in range(a.start, a.end))  # noqa: E731
    assert abs(cost(r[0]) - cost(r[1])) <= 4
    assert [(-a.start + a.end) for a in P.pipeline_stage_layers(6, 3, 0, 1)] == [2, 2, 2]
    with pytest.raises(P.MeshError):
        P.pipeline_stage_layers(2, 3, 0, 1)


def test_fsdp_shard_gather_reduce_scatter():
    x = torch.arange(7 * 3, dtype=torch.float32).reshape(7, 3)
    shards = [P.fsdp_shard(x, 3, 0, r) for r in range(3)]
    assert [s.shape[0] for s in shards] == [3, 2, 2]
    assert torch.equal(P.fsdp_all_gather(shards, 0), x)
    with pytest.raises(P.MeshError):
        P.fsdp_shard(x, 8, 0, 0)
    parts = [torch.randn(6, 4, generator=torch.Generator().manual_seed(i)).bfloat16() for i in range(4)]
    acc = parts[0].float()
    for p in parts[1:]:
        acc = acc + p.float()
    got = P.fsdp_reduce_scatter(parts, 0, 2)
    assert got.dtype == torch.bfloat16 and torch.equal(got, acc[4:5].bfloat16())
    ints = [torch.tensor([2**31 - 1, 1], dtype=torch.int32)] * 2
    assert P.fsdp_reduce_scatter(ints, 0, 1).dtype == torch.int32
    with pytest.raises(P.MeshError):
        P.fsdp_reduce_scatter([torch.ones(2, dtype=torch.bool)] * 2, 0, 0)
    gpu, grace = P.zero3_views(x, P.ParamKind.DENSE, 2, 0, 1)
    assert gpu.dtype == torch.bfloat16 and grace.dtype == torch.float32 and grace.shape == (3, 3)
    full, _ = P.zero3_views(x, P.ParamKind.ROUTED_EXPERT, 2, 0, 1)
    assert full.shape == (7, 3)
    with pytest.raises(P.MeshError):
        P.zero3_views(x, "dense", 2, 0, 1)
    assert fsdp.plan_ownership([10, 3], 4)[3] == [(8, 10), (3, 3)]


def test_schedule_and_in_process_pipeline():
    sched = P.pipeline_forward_schedule(3, 2)
    assert sched == ((0, None), (1, 0), (2, 1), (None, 2))
    calls = []
    fns = [lambda x, s=s: (calls.append(s), x + 10 ** s)[1] for s in range(3)]
    out = P.circular_pipeline([1, 2], fns)
    assert out == (112, 113) and calls == [0, 0, 1, 1, 2, 2]
    with pytest.raises(P.MeshError):
        P.circular_pipeline([], fns)
    with pytest.raises(P.MeshError):
        P.spmd_circular_pipeline([torch.zeros(1)], 2, lambda s, x: x)


def test_ring_attention_matches_dense_and_schedule():
    assert P.cp_ring_schedule(4, 1) == (1, 0, 3, 2)
    q = torch.randn(2, 24, 4, 8, generator=torch.Generator().manual_seed(0))
    k = torch.randn(2, 24, 2, 8, generator=torch.Generator().manual_seed(1))
    v = torch.randn(2, 24, 2, 8, generator=torch.Generator().manual_seed(2))
    torch.testing.assert_close(P.ring_attention(q, k, v, 3), model.gqa_attention(q, k, v),
                               rtol=1e-5, atol=1e-5)
    with pytest.raises(P.MeshError):
        P.cp_split_seq(q, 5, 0)
    assert P.cp_split_seq(q, 4, 3).shape[1] == 6


def test_delta_state_handoff_equals_serial_scan():
    b, s, h, d, n = 1, 256, 2, 16, 4
    g = torch.Generator().manual_seed(0)
    k = torch.nn.functional.normalize(torch.randn(b, s, h, d, generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(b, s, h, d, generator=g), dim=-1)
    v = torch.randn(b, s, h, d, generator=g)
    beta = torch.rand(b, s, h, generator=g)
    o_ref, s_ref = kernels.delta_rule_recurrent(q, k, v, beta)
    maps = [cp.slice_affine_map(P.cp_split_seq(k, n, r), P.cp_split_seq(v, n, r),
                                P.cp_split_seq(beta, n, r), chunk=16) for r in range(n)]
    incoming = P.delta_state_handoff(maps)
    outs = []
    for r in range(n):
        o, st = kernels.chunked_delta_rule(P.cp_split_seq(q, n, r), P.cp_split_seq(k, n, r),
                                           P.cp_split_seq(v, n, r), P.cp_split_seq(beta, n, r),
                                           incoming[r], kernels.LinearAttnConfig(chunk=16))
        outs.append(o)
    torch.testing.assert_close(torch.cat(outs, 1), o_ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(st, s_ref, rtol=1e-4, atol=1e-4)
    full = maps[0]
    for m in maps[1:]:
        full = P.compose_affine(full, m)
    torch.testing.assert_close(full[1], s_ref, rtol=1e-4, atol=1e-4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # pipeline: stage s multiplies by (s + 2)
        mbs = [torch.full((3,), float(i + 1)) for i in range(4)]
        res = P.spmd_circular_pipeline(mbs, world, lambda s, x: x * (s + 2))
        want = [m * 2 * 3 for m in mbs]
        ok_pp = all(torch.equal(a, b) for a, b in zip(res, want))
        # ring attention: each rank folds its block, compare with the dense result
        g = torch.Generator().manual_seed(0)
        q = torch.randn(1, 8 * world, 2, 4, generator=g)
        k = torch.randn(1, 8 * world, 2, 4, generator=g)
        v = torch.randn(1, 8 * world, 2, 4, generator=g)
        mine = cp.ring_attention_distributed(P.cp_split_seq(q, world, rank),
                                             P.cp_split_seq(k, world, rank),
                                             P.cp_split_seq(v, world, rank))
        dense = P.cp_split_seq(model.gqa_attention(q, k, v), world, rank)
        ok_cp = torch.allclose(mine, dense, rtol=1e-5, atol=1e-5)
        # delta hand-off over all_gather
        kk = torch.nn.functional.normalize(torch.randn(1, 32 * world, 1, 8, generator=g), dim=-1)
        vv = torch.randn(1, 32 * world, 1, 8, generator=g)
        bb = torch.rand(1, 32 * world, 1, generator=g)
        local = cp.slice_affine_map(P.cp_split_seq(kk, world, rank), P.cp_split_seq(vv, world, rank),
                                    P.cp_split_seq(bb, world, rank), chunk=16)
        s_in = cp.delta_state_handoff_distributed(local)
        _, s_ref = kernels.delta_rule_recurrent(kk[:, :32 * rank], kk[:, :32 * rank],
                                                vv[:, :32 * rank], bb[:, :32 * rank])
        ok_ds = torch.allclose(s_in, s_ref, rtol=1e-4, atol=1e-4)
        out.put((rank, ok_pp, ok_cp, ok_ds))
    finally:
        dist.destroy_process_group()


def test_two_process_gloo_pipeline_ring_and_handoff():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert got == [(0, True, True, True), (1, True, True, True)]


def _pp_train_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        layers = [torch.nn.Linear(6, 6) for _ in range(world)]         # same weights on every rank
        mbs = [torch.randn(5, 6, generator=torch.Generator().manual_seed(10 + i)) for i in range(3)]
        tgt = [torch.randn(5, 6, generator=torch.Generator().manual_seed(20 + i)) for i in range(3)]
        loss_fn = lambda y, m: ((y - tgt[m]) ** 2).mean()               # noqa: E731
        mine = layers[rank]
        total = P.spmd_pipeline_train(mbs, world, lambda s, x: torch.tanh(mine(x)), loss_fn)
        # the unsplit model on one process
        ref = [torch.nn.Linear(6, 6) for _ in range(world)]
        for a, b in zip(ref, layers):
            a.load_state_dict(b.state_dict())
        want = 0.0
        for m, x in enumerate(mbs):
            h = x
            for l in ref:
                h = torch.tanh(l(h))
            loss = loss_fn(h, m)
            loss.backward()
            want = want + loss.item()
        ok_grad = torch.allclose(mine.weight.grad, ref[rank].weight.grad, rtol=1e-5, atol=1e-6) and \
            torch.allclose(mine.bias.grad, ref[rank].bias.grad, rtol=1e-5, atol=1e-6)
        ok_loss = total is None if rank < world - 1 else abs(float(total) - want) < 1e-5
        out.put((rank, ok_grad, ok_loss))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_pipeline_backward_matches_the_unsplit_model(world):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_train_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert got == [(r, True, True) for r in range(world)]


def test_pipeline_train_single_stage_and_errors():
    lin = torch.nn.Linear(3, 3)
    xs = [torch.randn(2, 3) for _ in range(2)]
    total = P.spmd_pipeline_train(xs, 1, lambda s, x: lin(x), lambda y, m: y.sum())
    assert lin.weight.grad is not None and torch.isfinite(total)
    with pytest.raises(P.MeshError):
        P.spmd_pipeline_train(xs, 2, lambda s, x: x, lambda y, m: y.sum())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_zigzag_split_chain_and_balance(world):
    """The zig-zag layout on the CPU definitions: rank r holds half-slices r and 2 world - 1 - r;
    the delta-rule states entering every half-slice, folded in chain order from the half-slice
    maps, reproduce the serial scan when the per-rank outputs are put back in sequence order; and
    the causal-attention work per rank is the same for every rank."""
    from prometheus_b200.parallel.cp import zigzag_positions, zigzag_slice

    b, h, d = 1, 2, 16
    half = 32
    s = 2 * world * half
    g = torch.Generator().manual_seed(world)
    k = torch.nn.functional.normalize(torch.randn(b, s, h, d, generator=g), dim=-1)
    q = torch.nn.functional.normalize(torch.randn(b, s, h, d, generator=g), dim=-1)
    v = torch.randn(b, s, h, d, generator=g)
    beta = torch.rand(b, s, h, generator=g)
    o_ref, _ = kernels.delta_rule_recurrent(q, k, v, beta)
    # every chain position's map, as the owning rank would build it from its local tensors
    maps = [None] * (2 * world)
    local = {}
    for r in range(world):
        lq, lk, lv, lb = (zigzag_slice(t, world, r) for t in (q, k, v, beta))
        assert lq.shape[1] == 2 * half
        local[r] = (lq, lk, lv, lb)
        for which, pos in enumerate(zigzag_positions(world, r)):
            sl = slice(which * half, (which + 1) * half)
            maps[pos] = cp.slice_affine_map(lk[:, sl], lv[:, sl], lb[:, sl], chunk=16)
            torch.testing.assert_close(lq[:, sl], q[:, pos * half:(pos + 1) * half])
    incoming = P.delta_state_handoff(maps)                       # fold over the 2 x world positions
    out = torch.empty_like(o_ref)
    for r in range(world):
        lq, lk, lv, lb = local[r]
        for which, pos in enumerate(zigzag_positions(world, r)):
            sl = slice(which * half, (which + 1) * half)
            o, _ = kernels.chunked_delta_rule(lq[:, sl], lk[:, sl], lv[:, sl], lb[:, sl], incoming[pos],
                                              kernels.LinearAttnConfig(chunk=16))
            out[:, pos * half:(pos + 1) * half] = o
    torch.testing.assert_close(out, o_ref, rtol=1e-4, atol=1e-4)
    # causal work in units of half-slice blocks: position p attends p + 1/2 blocks
    work = [sum(p + 0.5 for p in zigzag_positions(world, r)) for r in range(world)]
    assert len(set(work)) == 1 and work[0] == 2 * world
    assert sorted(p for r in range(world) for p in zigzag_positions(world, r)) == list(range(2 * world))
    with pytest.raises(P.MeshError):
        zigzag_slice(q[:, :s - 1], world, 0)
