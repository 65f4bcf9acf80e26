"""Behaviour list of the host definitions of context parallelism (``prometheus_b200.parallel.cp``;
reference tests/test_parallel_cp.py, parallel/cp.py): the ring schedule, equal sequence
splits, ring attention against a float64 one-shot softmax (causal and not, any scale, grouped
KV heads), finite-difference gradients, the affine hand-off of the delta-rule state across
slices, and the zig-zag layout this framework adds."""
import itertools
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import kernels as K
from prometheus_b200 import parallel as P
from prometheus_b200.parallel import cp as C


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def one_shot(q, k, v, causal, scale=None):
    q, k, v = (t.double().numpy() for t in (q, k, v))
    g = q.shape[2] // k.shape[2]
    k, v = np.repeat(k, g, 2), np.repeat(v, g, 2)
    s = np.einsum("bqhd,bkhd->bhqk", q, k) * (1 / math.sqrt(q.shape[-1]) if scale is None else scale)
    if causal:
        mask = np.arange(k.shape[1])[None, :] > np.arange(q.shape[1])[:, None]
        s = np.where(mask[None, None], -np.inf, s)
    w = np.exp(s - s.max(-1, keepdims=True))
    w /= w.sum(-1, keepdims=True)
    return np.einsum("bhqk,bkhd->bqhd", w, v)


# ------------------------------------------------------------------------------ schedule / split
def test_ring_schedule():
    assert C.cp_ring_schedule(4, 1) == (1, 0, 3, 2) and C.cp_ring_schedule(1, 0) == (0,) and C.cp_ring_schedule(3, 0) == (0, 2, 1)
    for n in range(1, 9):
        for r in range(n):
            sched = C.cp_ring_schedule(n, r)
            assert sched[0] == r and sorted(sched) == list(range(n))                    # own block first, every block once
            assert all(sched[t] == (r - t) % n for t in range(n))
        step = [C.cp_ring_schedule(n, r) for r in range(n)]
        for t in range(n):
            assert sorted(s[t] for s in step) == list(range(n))                         # at every step each block is held by one rank
    for n, r in ((0, 0), (-1, 0), (4, 4), (4, -1), (True, 0), (4, 1.0), (2.0, 0)):
        with pytest.raises(P.MeshError):
            C.cp_ring_schedule(n, r)


def test_sequence_split():
    x = torch.arange(2 * 12 * 3).reshape(2, 12, 3)
    for n in (1, 2, 3, 4, 6, 12):
        parts = [C.cp_split_seq(x, n, r) for r in range(n)]
        assert torch.equal(torch.cat(parts, 1), x) and all(p.shape == (2, 12 // n, 3) for p in parts)
    assert C.cp_split_seq(x, 1, 0) is x or torch.equal(C.cp_split_seq(x, 1, 0), x)
    assert torch.equal(C.cp_split_seq(x, 3, 1, axis=-2), C.cp_split_seq(x, 3, 1, axis=1))
    assert torch.equal(C.cp_split_seq(x, 3, 2, axis=2), x[:, :, 2:3]) and torch.equal(C.cp_split_seq(x, 2, 1, axis=0), x[1:])
    for dt in (torch.float16, torch.bfloat16, torch.float64, torch.int32):
        assert C.cp_split_seq(x.to(dt), 2, 0).dtype == dt
    assert torch.equal(C.cp_split_seq(np.arange(8).reshape(1, 8), 4, 3), torch.tensor([[6, 7]]))
    for n, r, axis in ((0, 0, 1), (5, 0, 1), (24, 0, 1), (4, 4, 1), (4, -1, 1), (2, 0, 3), (2, 0, -4), (2.0, 0, 1), (2, 0, True)):
        with pytest.raises(P.MeshError):
            C.cp_split_seq(x, n, r, axis=axis)


# ------------------------------------------------------------------------------ ring attention
@pytest.mark.parametrize("causal, n, heads, kv_heads", list(itertools.product([True, False], [1, 2, 4], [4], [4, 1])))
def test_ring_attention_equals_the_one_shot_softmax(causal, n, heads, kv_heads):
    q, k, v = rnd(2, 16, heads, 8, seed=1), rnd(2, 16, kv_heads, 8, seed=2), rnd(2, 16, kv_heads, 6, seed=3)
    got = C.ring_attention(q, k, v, n, causal=causal)
    assert got.shape == (2, 16, heads, 6) and got.dtype == torch.float32
    np.testing.assert_allclose(got.numpy(), one_shot(q, k, v, causal), rtol=1e-4, atol=1e-5)


def test_ring_attention_details():
    q, k, v = rnd(1, 8, 2, 4, seed=4), rnd(1, 8, 2, 4, seed=5), rnd(1, 8, 2, 4, seed=6)
    for scale in (0.1, 1.0, 2.5):
        np.testing.assert_allclose(C.ring_attention(q, k, v, 4, scale=scale).numpy(), one_shot(q, k, v, True, scale), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(C.ring_attention(q, k, v, 2).numpy(), C.ring_attention(q, k, v, 2, scale=0.5).numpy(), rtol=1e-6)   # default 1 / sqrt(d)
    base = C.ring_attention(q, k, v, 4)
    k2, v2 = k.clone(), v.clone()
    k2[:, 6:] += 5.0
    v2[:, 6:] -= 3.0
    moved = C.ring_attention(q, k2, v2, 4)
    assert torch.equal(moved[:, :6], base[:, :6]) and not torch.allclose(moved[:, 6:], base[:, 6:])     # future blocks never reach earlier queries
    for dt in (torch.float16, torch.float64):
        assert C.ring_attention(q.to(dt), k.to(dt), v.to(dt), 2).dtype == torch.float32
    tiny_q = torch.tensor([[[[1.0, 0.0]], [[0.0, 1.0]]]])                                               # (1, 2, 1, 2)
    tiny_v = torch.tensor([[[[1.0]], [[3.0]]]])
    out = C.ring_attention(tiny_q, tiny_q, tiny_v, 2, scale=1.0)
    w = math.exp(1.0) / (math.exp(0.0) + math.exp(1.0))
    np.testing.assert_allclose(out.reshape(-1).numpy(), [1.0, (1 - w) * 1.0 + w * 3.0], rtol=1e-6)


def test_one_rank_of_the_ring_and_its_argument_errors():
    q, k, v = rnd(1, 12, 2, 4, seed=7), rnd(1, 12, 2, 4, seed=8), rnd(1, 12, 2, 4, seed=9)
    whole = one_shot(q, k, v, True)
    ks, vs = [C.cp_split_seq(k, 3, r) for r in range(3)], [C.cp_split_seq(v, 3, r) for r in range(3)]
    for r in range(3):
        got = C.ring_attention_rank(C.cp_split_seq(q, 3, r), ks, vs, r)
        np.testing.assert_allclose(got.numpy(), whole[:, 4 * r:4 * r + 4], rtol=1e-4, atol=1e-5)
    qs = C.cp_split_seq(q, 3, 0)
    for bad in (lambda: C.ring_attention_rank(qs, [], [], 0), lambda: C.ring_attention_rank(qs, ks, vs[:2], 0), lambda: C.ring_attention_rank(qs, ks, vs, 3),
                lambda: C.ring_attention_rank(qs, ks, vs, -1), lambda: C.ring_attention_rank(qs, [ks[0], ks[1], ks[2][:, :3]], vs, 0),
                lambda: C.ring_attention(q, k, v, 5), lambda: C.ring_attention(q, k, v, 0)):
        with pytest.raises(P.MeshError):
            bad()


def test_ring_attention_gradient_against_finite_differences():
    q, k, v = (rnd(1, 6, 1, 3, seed=s).double() for s in (10, 11, 12))
    g = rnd(1, 6, 1, 3, seed=13).double()
    leaves = [t.clone().float().requires_grad_(True) for t in (q, k, v)]
    (C.ring_attention(*leaves, 3) * g.float()).sum().backward()
    h = 1e-5
    for which, leaf in enumerate(leaves):
        base = [q, k, v]
        flat = base[which].reshape(-1)
        for idx in range(0, flat.numel(), 5):
            old = float(flat[idx])
            flat[idx] = old + h
            up = float((torch.tensor(one_shot(*base, True)) * g).sum())
            flat[idx] = old - h
            down = float((torch.tensor(one_shot(*base, True)) * g).sum())
            flat[idx] = old
            assert float(leaf.grad.reshape(-1)[idx]) == pytest.approx((up - down) / (2 * h), rel=2e-3, abs=2e-4)


# ------------------------------------------------------------------------------ delta-rule state hand-off
def test_slice_maps_compose_to_the_state_of_the_whole_prefix():
    n, chunk = 4, 8
    k = torch.nn.functional.normalize(rnd(2, 16 * n, 2, 8, seed=14), dim=-1)
    v, beta = rnd(2, 16 * n, 2, 6, seed=15), torch.sigmoid(rnd(2, 16 * n, 2, seed=16))
    maps = [C.slice_affine_map(C.cp_split_seq(k, n, r), C.cp_split_seq(v, n, r), C.cp_split_seq(beta, n, r), chunk=chunk) for r in range(n)]
    states = C.delta_state_handoff(maps)
    assert states[0].abs().max() == 0
    for r in range(1, n):
        _, want = K.delta_rule_recurrent(k[:, :16 * r], k[:, :16 * r], v[:, :16 * r], beta[:, :16 * r])
        torch.testing.assert_close(states[r], want, rtol=1e-4, atol=1e-5)
    s0 = rnd(2, 2, 8, 6, seed=17) * 0.1
    with_start = C.delta_state_handoff(maps, s0)
    _, want = K.delta_rule_recurrent(k[:, :32], k[:, :32], v[:, :32], beta[:, :32], s0)
    torch.testing.assert_close(with_start[2], want, rtol=1e-4, atol=1e-5)
    both = C.compose_affine(maps[0], maps[1])                                            # composition is the map of the joined slice
    joined = C.slice_affine_map(k[:, :32], v[:, :32], beta[:, :32], chunk=chunk)
    torch.testing.assert_close(both[0], joined[0], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(both[1], joined[1], rtol=1e-4, atol=1e-5)
    left = C.compose_affine(C.compose_affine(maps[0], maps[1]), maps[2])
    right = C.compose_affine(maps[0], C.compose_affine(maps[1], maps[2]))
    torch.testing.assert_close(left[1], right[1], rtol=1e-4, atol=1e-5)                  # associative: any grouping of ranks works
    with pytest.raises(P.MeshError):
        C.delta_state_handoff([])
    with pytest.raises(P.MeshError):
        C.slice_affine_map(k[:, :12], v[:, :12], beta[:, :12], chunk=8)


# ------------------------------------------------------------------------------ zig-zag layout
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_zigzag_layout_balances_causal_work(world):
    pairs = [C.zigzag_positions(world, r) for r in range(world)]
    assert sorted(i for p in pairs for i in p) == list(range(2 * world))                 # a permutation of the 2W half-slices
    assert all(a + b == 2 * world - 1 for a, b in pairs)                                 # early half paired with its mirror
    work = [(a + 1) + (b + 1) for a, b in pairs]                                         # key blocks a causal query half-slice sees
    assert len(set(work)) == 1 and work[0] == 2 * world + 1
    x = torch.arange(2 * world * 3).reshape(1, 2 * world * 3)
    got = torch.cat([C.zigzag_slice(x, world, r) for r in range(world)], 1)
    assert sorted(got.reshape(-1).tolist()) == x.reshape(-1).tolist()
    for r, (a, b) in enumerate(pairs):
        piece = C.zigzag_slice(x, world, r)
        assert piece[0, :3].tolist() == list(range(3 * a, 3 * a + 3)) and piece[0, 3:].tolist() == list(range(3 * b, 3 * b + 3))
