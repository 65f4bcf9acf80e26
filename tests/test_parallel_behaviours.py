"""Behaviour list of the host definitions of the parallel layouts (``prometheus_b200.parallel``;
reference tests/test_parallel.py, test_parallel_fsdp.py, test_parallel_schedule.py and
parallel/{__init__,fsdp,schedule}.py): mesh arithmetic, the ZeRO-3 shard / gather /
reduce-scatter semantics that the device kernels implement (array-split bounds, left fold in
rank order in the accumulation type), balanced pipeline stages and the tick schedule."""
import itertools

import numpy as np
import pytest
import torch

from prometheus_b200 import parallel as P
from prometheus_b200.parallel import fsdp as F
from prometheus_b200.parallel import schedule as S


# ------------------------------------------------------------------------------ mesh
def test_mesh_constants_and_coordinates():
    f, t = P.flagship_mesh(), P.tiny_mesh()
    assert (f.dp, f.fsdp, f.ep, f.pp, f.cp) == (115, 72, 72, 12, 1) and f.n_devices == 115 * 12 * 72
    assert (t.dp, t.fsdp, t.ep, t.pp, t.cp) == (2, 2, 2, 2, 1) and t.n_devices == 8 and P.device_ids(t) == tuple(range(8))
    assert [a.value for a in P.Axis] == ["dp", "fsdp", "ep", "pp", "cp"] and issubclass(P.MeshError, ValueError)
    seen = {P.coord_of(d, t) for d in range(8)}
    assert seen == set(itertools.product(range(2), range(2), range(2), range(1)))       # a bijection
    assert P.coord_of(0, t) == (0, 0, 0, 0) and P.coord_of(1, t) == (0, 0, 1, 0) and P.coord_of(2, t) == (0, 1, 0, 0) and P.coord_of(4, t) == (1, 0, 0, 0)
    with_cp = P.MeshSpec(dp=1, fsdp=2, ep=2, pp=1, cp=4)
    assert [P.coord_of(d, with_cp)[3] for d in range(8)] == [0, 1, 2, 3] * 2             # context ranks are innermost
    for bad in (-1, 8):
        with pytest.raises(P.MeshError):
            P.coord_of(bad, t)
    for spec in (P.MeshSpec(0, 2, 2, 2, 1), P.MeshSpec(2, 2, 3, 2, 1), P.MeshSpec(2, 2, 2, 2, 0)):
        with pytest.raises(P.MeshError):
            P.validate_mesh(spec)
    box = P.box_mesh(8, cp=2)
    assert (box.dp, box.fsdp, box.ep, box.pp, box.cp) == (1, 4, 4, 1, 2) and box.n_devices == 8
    for n, cp in ((0, 1), (8, 3), (8, 0)):
        with pytest.raises(P.MeshError):
            P.box_mesh(n, cp=cp)


def test_partition_rule_and_context_parallel_switch():
    for kind in P.ParamKind:
        want = (None,) if kind is P.ParamKind.ROUTED_EXPERT else ("fsdp",)
        assert P.fsdp_partition(kind).axes == want
    assert not P.context_parallel_on(16384, 16384) and P.context_parallel_on(16385, 16384)


# ------------------------------------------------------------------------------ shard
@pytest.mark.parametrize("shape, n, axis", [((10,), 3, 0), ((7, 5), 4, 0), ((7, 5), 2, -1), ((3, 9, 2), 4, 1), ((6, 6), 6, 1), ((5,), 1, 0)])
def test_shard_uses_array_split_bounds(shape, n, axis):
    x = np.arange(int(np.prod(shape)), dtype=np.int32).reshape(shape)
    before = x.copy()
    pieces = np.array_split(x, n, axis=axis)
    for r in range(n):
        got = F.fsdp_shard(x, n, axis, r)
        assert np.array_equal(got.numpy(), pieces[r]) and got.dtype == torch.int32
    assert np.array_equal(x, before)
    back = F.fsdp_all_gather([F.fsdp_shard(x, n, axis, r) for r in range(n)], axis)
    assert np.array_equal(back.numpy(), x)                                               # shard then gather is the identity


def test_shard_keeps_bits():
    x = torch.tensor([0.0, -0.0, float("nan"), 1.5])
    got = F.fsdp_shard(x, 1, 0, 0)
    assert got.view(torch.int32).tolist() == x.view(torch.int32).tolist()                # signed zero and NaN payload survive
    bf = torch.arange(10, dtype=torch.float32).to(torch.bfloat16)
    assert F.fsdp_shard(bf, 3, 0, 0).dtype == torch.bfloat16 and F.fsdp_shard(bf, 3, 0, 0).tolist() == [0.0, 1.0, 2.0, 3.0]
    assert F.split_bounds(10, 3, 0) == (0, 4) and F.split_bounds(10, 3, 1) == (4, 7) and F.split_bounds(10, 3, 2) == (7, 10)


@pytest.mark.parametrize("args", [(0, 0, 0), (-1, 0, 0), (2, 0, 2), (2, 0, -1), (2, 1, 0), (2, -2, 0), (5, 0, 0), (True, 0, 0), (2, 0.0, 0), (2, 0, 1.0)])
def test_shard_argument_errors(args):
    with pytest.raises(P.MeshError):
        F.fsdp_shard(np.zeros(4), *args)                                                 # 4 elements: n = 5 would leave a rank empty


def test_shard_of_scalars_and_empty_axes():
    for x, n, axis in ((np.float32(1.0), 1, 0), (np.zeros((0, 3)), 1, 0), (np.zeros((3, 0)), 2, 1)):
        with pytest.raises(P.MeshError):
            F.fsdp_shard(x, n, axis, 0)


# ------------------------------------------------------------------------------ gather
def test_gather_is_concatenation_with_checks():
    a, b = torch.arange(6.0).reshape(2, 3), torch.arange(3.0).reshape(1, 3)
    assert F.fsdp_all_gather([a, b], 0).shape == (3, 3) and F.fsdp_all_gather((a, a), -1).shape == (2, 6)
    one = F.fsdp_all_gather([a], 0)
    assert torch.equal(one, a)
    for shards, axis in (([], 0), ([a, b.double()], 0), ([a, b], 1), ([a, a[0]], 0), ([a, a], 2), ([a, a], -3)):
        with pytest.raises(P.MeshError):
            F.fsdp_all_gather(shards, axis)
    with pytest.raises(P.MeshError):
        F.fsdp_all_gather(None, 0)


# ------------------------------------------------------------------------------ reduce-scatter
def test_reduce_scatter_is_a_left_fold_in_rank_order():
    big, small = np.float32(2 ** 24), np.float32(1.0)                                    # (big + 1) + 1 loses both ones; big + (1 + 1) would not
    parts = [np.array([big, 0, 0], np.float32), np.array([small, 0, 0], np.float32), np.array([small, 0, 0], np.float32)]
    got = F.fsdp_reduce_scatter(parts, 0, 0)
    assert got.tolist() == [float(np.float32(np.float32(big + small) + small))] == [float(big)]
    rev = F.fsdp_reduce_scatter(parts[::-1], 0, 0)
    assert rev.tolist() == [float(big) + 2.0]                                            # order is part of the definition
    x = [np.array([1.0, 2.0, 3.0, 4.0], np.float32) * (r + 1) for r in range(4)]
    assert F.fsdp_reduce_scatter(x, 0, 1).tolist() == [20.0] and F.fsdp_reduce_scatter(x[:2], 0, 1).tolist() == [9.0, 12.0]     # a sum, not a mean


def test_reduce_scatter_accumulation_types():
    h = [torch.tensor([2048.0, 1.0, 0.0], dtype=torch.float16), torch.tensor([1.0, 1.0, 0.0], dtype=torch.float16), torch.tensor([1.0, 1.0, 0.0], dtype=torch.float16)]
    got = F.fsdp_reduce_scatter(h, 0, 0)
    assert got.dtype == torch.float16 and got.tolist() == [2050.0]                       # summed in fp32 (fp16 would stick at 2048), cast once
    bf = [torch.tensor([256.0, 0, 0, 0, 0], dtype=torch.bfloat16)] + [torch.tensor([1.0, 0, 0, 0, 0], dtype=torch.bfloat16)] * 4
    assert F.fsdp_reduce_scatter(bf, 0, 0).tolist() == [260.0] and F.fsdp_reduce_scatter(bf, 0, 0).dtype == torch.bfloat16
    d = [torch.tensor([1e16, 0.0, 0.0], dtype=torch.float64), torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64), torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64)]
    assert F.fsdp_reduce_scatter(d, 0, 0).tolist() == [1e16]                             # float64 stays float64: ones are lost one at a time
    for dt in (torch.int8, torch.int32, torch.int64, torch.uint8):
        parts = [torch.tensor([100, 1], dtype=dt), torch.tensor([27, 1], dtype=dt)]
        got = F.fsdp_reduce_scatter(parts, 0, 0)
        assert got.dtype == dt and got.tolist() == [127]
    z = F.fsdp_reduce_scatter([torch.tensor([-0.0])], 0, 0)
    assert z.view(torch.int32).tolist() == torch.tensor([-0.0]).view(torch.int32).tolist()


def test_reduce_scatter_argument_errors():
    a = torch.zeros(4)
    for partials, axis, rank in (([], 0, 0), ([a, a.double()], 0, 0), ([a, torch.zeros(5)], 0, 0), ([a, a], 1, 0), ([a, a], 0, 2),
                                 ([a, a], 0, -1), ([torch.zeros(1)] * 2, 0, 0), ([torch.zeros(2, dtype=torch.bool)] * 2, 0, 0),
                                 ([torch.zeros(2, dtype=torch.complex64)] * 2, 0, 0)):
        with pytest.raises(P.MeshError):
            F.fsdp_reduce_scatter(partials, axis, rank)
    assert F.fsdp_reduce_scatter((a, a), 0, 1).shape == (2,)


@pytest.mark.parametrize("n, axis", [(2, 0), (3, 1), (4, -1)])
def test_reduce_scatter_matches_numpy_left_fold(n, axis):
    rng = np.random.default_rng(n)
    parts = [rng.standard_normal((6, 8)).astype(np.float32) for _ in range(n)]
    acc = parts[0].copy()
    for p in parts[1:]:
        acc = acc + p
    for r in range(n):
        got = F.fsdp_reduce_scatter(parts, axis, r)
        assert np.array_equal(got.numpy(), np.array_split(acc, n, axis=axis)[r])


# ------------------------------------------------------------------------------ ZeRO-3 views
def test_zero3_views_shard_first_then_cast():
    x = torch.arange(12, dtype=torch.float32).reshape(4, 3) + 0.1234567
    for kind in (P.ParamKind.ATTENTION, P.ParamKind.DENSE, P.ParamKind.SHARED_EXPERT, P.ParamKind.OTHER):
        bf, master = F.zero3_views(x, kind, 2, 0, 1)
        assert bf.dtype == torch.bfloat16 and master.dtype == torch.float32 and bf.shape == master.shape == (2, 3)
        assert torch.equal(master, x[2:]) and torch.equal(bf, x[2:].to(torch.bfloat16))
    bf, master = F.zero3_views(x, P.ParamKind.ROUTED_EXPERT, 2, 0, 1)
    assert torch.equal(master, x) and bf.shape == (4, 3)                                 # experts are not sharded on this axis
    whole_bf, whole = F.zero3_views(x, P.ParamKind.DENSE, 1, 0, 0)
    assert torch.equal(whole, x) and torch.equal(whole_bf, x.to(torch.bfloat16))
    uneven = F.zero3_views(torch.arange(10.0), P.ParamKind.DENSE, 3, -1, 2)[1]
    assert uneven.tolist() == [7.0, 8.0, 9.0]
    for bad in (lambda: F.zero3_views(x, "dense", 2, 0, 0), lambda: F.zero3_views(x.long(), P.ParamKind.DENSE, 2, 0, 0),
                lambda: F.zero3_views(x, P.ParamKind.DENSE, 5, 0, 0), lambda: F.zero3_views(x, P.ParamKind.DENSE, 2, 0, 2)):
        with pytest.raises(P.MeshError):
            bad()


def test_ownership_plan_is_contiguous_and_balanced():
    plan = F.plan_ownership([10, 3, 1], 4)
    assert len(plan) == 4
    for c, count in enumerate([10, 3, 1]):
        spans = [plan[r][c] for r in range(4)]
        assert spans[0][0] == 0 and spans[-1][1] == count and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


# ------------------------------------------------------------------------------ pipeline
def test_stage_layers_balance_cost_with_a_recurrent_tail():
    even = P.pipeline_stage_layers(8, 4, 0, 1)
    assert [(s.start, s.end) for s in even] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    tail = P.pipeline_stage_layers(8, 2, 2, 4)                                           # costs 1 x 6 + 4 x 2 = 14: the split sits late
    assert [(s.start, s.end) for s in tail] == [(0, 6), (6, 8)] or tail[0].end >= 6
    for n_layers, n_pp, core, rec in ((12, 3, 4, 3), (96, 12, 8, 3), (5, 5, 5, 2), (7, 1, 3, 9)):
        stages = P.pipeline_stage_layers(n_layers, n_pp, core, rec)
        assert stages[0].start == 0 and stages[-1].end == n_layers and len(stages) == n_pp
        assert all(a.end == b.start and a.end > a.start for a, b in zip(stages, stages[1:])) and stages[-1].end > stages[-1].start
    for bad in ((0, 1, 0, 1), (4, 0, 0, 1), (4, 5, 0, 1), (4, 2, 5, 1), (4, 2, -1, 1), (4, 2, 1, 0)):
        with pytest.raises(P.MeshError):
            P.pipeline_stage_layers(*bad)


def test_tick_schedule():
    assert S.pipeline_forward_schedule(3, 2) == ((0, None), (1, 0), (2, 1), (None, 2))
    assert S.pipeline_forward_schedule(1, 1) == ((0,),) and S.pipeline_forward_schedule(1, 3) == ((0, None, None), (None, 0, None), (None, None, 0))
    assert S.pipeline_forward_schedule(2, 1) == ((0,), (1,))
    for m, s in itertools.product(range(1, 6), range(1, 5)):
        ticks = S.pipeline_forward_schedule(m, s)
        assert len(ticks) == m + s - 1
        for t, row in enumerate(ticks):
            assert row == tuple((t - j) if 0 <= t - j < m else None for j in range(s))
        for j in range(s):
            assert [row[j] for row in ticks if row[j] is not None] == list(range(m))     # every stage sees every microbatch once, in order
    for bad in ((0, 1), (1, 0), (-1, 2)):
        with pytest.raises(P.MeshError):
            S.pipeline_forward_schedule(*bad)


def test_in_process_pipeline_composes_stages_in_tick_order():
    calls = []

    def stage(j):
        def fn(x):
            calls.append((j, int(x[0])))
            return x * 10 + j
        return fn

    mbs = [np.array([1]), np.array([2]), np.array([3])]
    out = S.circular_pipeline(mbs, [stage(1), stage(2)])
    assert [int(o[0]) for o in out] == [112, 212, 312]
    assert calls == [(1, 1), (1, 2), (2, 11), (1, 3), (2, 21), (2, 31)]                  # tick-major, stage order inside a tick
    w = [np.random.default_rng(i).standard_normal((4, 4)).astype(np.float32) for i in range(3)]
    xs = [np.random.default_rng(10 + i).standard_normal((2, 4)).astype(np.float32) for i in range(4)]
    got = S.circular_pipeline(xs, [lambda x, m=m: x @ m for m in w])
    for x, g in zip(xs, got):
        assert np.array_equal(g, ((x @ w[0]) @ w[1]) @ w[2])                             # bitwise: same operations in the same order
    shapes = S.circular_pipeline([np.zeros((2, 3))], [lambda x: x.reshape(3, 2), lambda x: x.sum(0), lambda x: x[None, None]])
    assert shapes[0].shape == (1, 1, 2)                                                  # stages may change shape and rank
    assert S.circular_pipeline([5], [lambda x: x + 1]) == (6,)
    for mb, fns in (([], [lambda x: x]), ([1], [])):
        with pytest.raises(P.MeshError):
            S.circular_pipeline(mb, fns)

    def boom(x):
        raise KeyError("stage fell over")

    with pytest.raises(KeyError):
        S.circular_pipeline([1, 2], [lambda x: x, boom])                                 # the stage's own exception, not wrapped
