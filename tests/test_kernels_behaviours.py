"""Behaviour list of the numeric primitives on the host (``prometheus_b200.kernels``; reference
tests/test_kernels.py and kernels/__init__.py): the chunked delta rule against a float64
per-token recurrence written here, its causality / linearity / state-carry properties and
finite-difference gradients, FP8 e4m3 block quantisation bit patterns and error bounds, the
straight-through FP8 linear, and expert dispatch / combine layouts with their VJPs."""
import dataclasses

import numpy as np
import pytest
import torch

from prometheus_b200 import kernels as K


def rand(*shape, seed=0, dtype=torch.float32):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=dtype)


def delta_inputs(b=1, s=6, h=2, dk=4, dv=3, seed=0):
    q, k = rand(b, s, h, dk, seed=seed), rand(b, s, h, dk, seed=seed + 1)
    k = k / k.norm(dim=-1, keepdim=True)
    v = rand(b, s, h, dv, seed=seed + 2)
    beta = torch.sigmoid(rand(b, s, h, seed=seed + 3))
    return q, k, v, beta


def recurrence64(q, k, v, beta, s0=None):
    """S_t = S_{t-1} + beta_t k_t (v_t - S_{t-1}^T k_t)^T ; o_t = S_t^T q_t, in float64 NumPy."""
    q, k, v, beta = (np.asarray(t, dtype=np.float64) for t in (q, k, v, beta))
    b, s, h, dk = q.shape
    dv = v.shape[-1]
    S = np.zeros((b, h, dk, dv)) if s0 is None else np.asarray(s0, dtype=np.float64).copy()
    out = np.zeros((b, s, h, dv))
    for t in range(s):
        for bi in range(b):
            for hi in range(h):
                kt, vt, bt = k[bi, t, hi], v[bi, t, hi], beta[bi, t, hi]
                S[bi, hi] += bt * np.outer(kt, vt - S[bi, hi].T @ kt)
                out[bi, t, hi] = S[bi, hi].T @ q[bi, t, hi]
    return out, S


# ------------------------------------------------------------------------------ constants / types
def test_constants_and_records():
    assert (K.DEFAULT_CHUNK, K.DEFAULT_FP8_BLOCK, K.MAX_RACKS, K.FP8_E4M3_MAX) == (64, 128, 4, 448.0)
    assert [d.value for d in K.DType] == ["fp32", "bf16", "fp8", "nvfp4"] and str(K.DType.FP8) == "fp8"
    assert K.LinearAttnConfig().chunk == 64 and issubclass(K.KernelError, ValueError)
    meta = K.Fp8Meta(torch.zeros(1, 4, dtype=torch.int8), torch.ones(1, 1))
    assert (meta.block, meta.dtype, meta.block2d) == (128, K.DType.FP8, False)
    d = K.DispatchMeta(torch.zeros(1, 1, dtype=torch.long), torch.ones(1, 1), torch.zeros(1, dtype=torch.long), 1)
    assert d.max_racks == 4
    for obj in (K.LinearAttnConfig(), meta, d):
        with pytest.raises(dataclasses.FrozenInstanceError):
            setattr(obj, dataclasses.fields(obj)[0].name, None)


# ------------------------------------------------------------------------------ delta rule
@pytest.mark.parametrize("seq, chunk", [(1, 64), (7, 3), (64, 64), (65, 64), (100, 32), (12, 1)])
def test_chunked_delta_rule_matches_the_float64_recurrence(seq, chunk):
    q, k, v, beta = delta_inputs(2, seq, 2, 4, 3, seed=seq)
    s0 = rand(2, 2, 4, 3, seed=99) * 0.1
    want_o, want_s = recurrence64(q, k, v, beta, s0)
    o, s = K.chunked_delta_rule(q, k, v, beta, s0, K.LinearAttnConfig(chunk=chunk))
    assert o.shape == v.shape and s.shape == (2, 2, 4, 3) and o.dtype == torch.float32
    np.testing.assert_allclose(o.numpy(), want_o, rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(s.numpy(), want_s, rtol=2e-4, atol=2e-5)
    o_np, s_np = K.chunked_delta_rule(q.numpy(), k.numpy(), v.numpy(), beta.numpy(), s0.numpy(), K.LinearAttnConfig(chunk=chunk))
    torch.testing.assert_close(o_np, o)                                                 # arrays are accepted too
    torch.testing.assert_close(s_np, s)


def test_delta_rule_hand_values():
    e0, e1 = [1.0, 0.0], [0.0, 1.0]
    q = torch.tensor([[[e0], [e1]]])
    v = torch.tensor([[[[1.0, 2.0]], [[3.0, 4.0]]]])
    out, state = K.chunked_delta_rule(q, q.clone(), v, torch.ones(1, 2, 1))             # orthonormal keys, beta 1: a key-value store
    torch.testing.assert_close(out, v)
    torch.testing.assert_close(state, torch.tensor([[[[1.0, 2.0], [3.0, 4.0]]]]))
    out, state = K.chunked_delta_rule(torch.tensor([[[e0]]]), torch.tensor([[[e0]]]), torch.tensor([[[[2.0, 4.0]]]]), torch.tensor([[[0.5]]]))
    torch.testing.assert_close(out, torch.tensor([[[[1.0, 2.0]]]]))                     # beta one half writes half the value
    out, state = K.chunked_delta_rule(torch.tensor([[[e0]]]), torch.tensor([[[e1]]]), torch.zeros(1, 1, 1, 2), torch.ones(1, 1, 1),
                                      state=torch.eye(2)[None, None])
    torch.testing.assert_close(state, torch.tensor([[[[1.0, 0.0], [0.0, 0.0]]]]))      # writing zero under key e1 erases that row
    torch.testing.assert_close(out, torch.tensor([[[[1.0, 0.0]]]]))


def test_delta_rule_properties():
    q, k, v, beta = delta_inputs(1, 10, 2, 4, 3, seed=5)
    o, s = K.chunked_delta_rule(q, k, v, beta, config=K.LinearAttnConfig(4))
    o0, s0 = K.chunked_delta_rule(q, k, v, beta, torch.zeros(1, 2, 4, 3), K.LinearAttnConfig(4))
    torch.testing.assert_close(o, o0)                                                   # no state is a zero state
    torch.testing.assert_close(s, s0)
    v2 = v.clone()
    v2[:, 7:] += 5.0                                                                    # the future does not reach the past
    o2, _ = K.chunked_delta_rule(q, k, v2, beta, config=K.LinearAttnConfig(4))
    torch.testing.assert_close(o2[:, :7], o[:, :7])
    assert not torch.allclose(o2[:, 7:], o[:, 7:])
    oa, sa = K.chunked_delta_rule(q[:, :6], k[:, :6], v[:, :6], beta[:, :6], config=K.LinearAttnConfig(4))
    ob, sb = K.chunked_delta_rule(q[:, 6:], k[:, 6:], v[:, 6:], beta[:, 6:], sa, K.LinearAttnConfig(4))
    torch.testing.assert_close(torch.cat([oa, ob], 1), o, rtol=1e-5, atol=1e-6)         # carrying the state = one shot
    torch.testing.assert_close(sb, s, rtol=1e-5, atol=1e-6)
    o3, s3 = K.chunked_delta_rule(q, k, 3.0 * v, beta, config=K.LinearAttnConfig(4))
    torch.testing.assert_close(o3, 3.0 * o, rtol=1e-5, atol=1e-6)                       # linear in v
    _, s4 = K.chunked_delta_rule(q * 7.0 + 1.0, k, v, beta, config=K.LinearAttnConfig(4))
    torch.testing.assert_close(s4, s)                                                   # the state never sees q
    for c in (1, 2, 5, 64):
        oc, sc = K.chunked_delta_rule(q, k, v, beta, config=K.LinearAttnConfig(c))
        torch.testing.assert_close(oc, o, rtol=1e-5, atol=1e-6)


def test_delta_rule_gradients_against_finite_differences():
    q, k, v, beta = (t.double() for t in delta_inputs(1, 5, 1, 3, 2, seed=11))
    s0 = rand(1, 1, 3, 2, seed=12).double() * 0.1
    go, gs = rand(1, 5, 1, 2, seed=13).double(), rand(1, 1, 3, 2, seed=14).double()

    def scalar(*xs):
        o, s = recurrence64(*xs)
        return float((o * go.numpy()).sum() + (s * gs.numpy()).sum())

    (_, _), res = K.chunked_delta_rule_fwd(q.float(), k.float(), v.float(), beta.float(), s0.float(), K.LinearAttnConfig(2))
    grads = K.chunked_delta_rule_bwd(res, (go.float(), gs.float()))
    args = [t.numpy().copy() for t in (q, k, v, beta, s0)]
    h = 1e-5
    for which, g in enumerate(grads):
        flat = args[which].reshape(-1)
        for idx in range(0, flat.size, max(1, flat.size // 6)):
            old = flat[idx]
            flat[idx] = old + h
            up = scalar(*args)
            flat[idx] = old - h
            down = scalar(*args)
            flat[idx] = old
            assert g.reshape(-1)[idx].item() == pytest.approx((up - down) / (2 * h), rel=2e-3, abs=2e-4)
    only_out = K.chunked_delta_rule_bwd(res, (go.float(), None))                        # a missing cotangent is zero
    with_zero = K.chunked_delta_rule_bwd(res, (go.float(), torch.zeros(1, 1, 3, 2)))
    for a, b in zip(only_out, with_zero):
        torch.testing.assert_close(a, b)


def test_delta_rule_autograd_equals_the_explicit_vjp():
    q, k, v, beta = delta_inputs(2, 9, 2, 4, 4, seed=21)
    s0 = rand(2, 2, 4, 4, seed=22) * 0.1
    go, gs = rand(2, 9, 2, 4, seed=23), rand(2, 2, 4, 4, seed=24)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, beta, s0)]
    o, s = K.chunked_delta_rule(*leaves, K.LinearAttnConfig(4))
    auto = torch.autograd.grad([o, s], leaves, [go, gs])
    (_, _), res = K.chunked_delta_rule_fwd(q, k, v, beta, s0, K.LinearAttnConfig(4))
    for a, b in zip(auto, K.chunked_delta_rule_bwd(res, (go, gs))):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_delta_rule_argument_errors():
    q, k, v, beta = delta_inputs(1, 3, 1, 4, 4)
    bad = [lambda: K.chunked_delta_rule(q[..., :3], k, v, beta), lambda: K.chunked_delta_rule(q, k, v, beta[:, :2]),
           lambda: K.chunked_delta_rule(q, k, v, beta, state=torch.zeros(1, 1, 3, 3)), lambda: K.chunked_delta_rule(q[0], k[0], v[0], beta[0]),
           lambda: K.chunked_delta_rule(q, k, v[:, :2], beta), lambda: K.chunked_delta_rule(q, k, v, beta, config=K.LinearAttnConfig(0)),
           lambda: K.chunked_delta_rule_fwd(q, k, v, beta, None, K.LinearAttnConfig(-1))]
    neg = beta.clone()
    neg[0, 0, 0] = -0.1
    bad.append(lambda: K.chunked_delta_rule(q, k, v, neg))
    for call in bad:
        with pytest.raises(K.KernelError):
            call()


# ------------------------------------------------------------------------------ fp8
def test_fp8_bit_patterns():
    meta = K.fp8_quantize(torch.tensor([[0.0, 1.0, 2.0, -2.0]]), block=4)               # amax 2: scaled values 0, 224, 448, -448
    torch.testing.assert_close(meta.scale, torch.tensor([[2.0 / 448.0]]))
    assert meta.q.view(torch.int8).tolist() == [[0, 118, 126, -2]] and meta.block == 4
    torch.testing.assert_close(K.fp8_dequantize(meta), torch.tensor([[0.0, 1.0, 2.0, -2.0]]))
    full = K.fp8_quantize(torch.tensor([[448.0, 224.0, 0.0]]), block=3)
    assert full.scale.tolist() == [[1.0]] and full.q.view(torch.uint8).tolist() == [[126, 118, 0]]
    zeros = K.fp8_quantize(torch.zeros(3, 16), block=8)
    assert zeros.scale.tolist() == [[1.0, 1.0]] * 3 and K.fp8_dequantize(zeros).abs().max() == 0
    made = K.Fp8Meta(q=torch.zeros(2, 4, dtype=torch.int8), scale=torch.ones(2, 1), block=4)
    assert K.fp8_dequantize(made).tolist() == [[0.0] * 4] * 2


def test_fp8_round_trip_error_is_bounded_per_block():
    x = rand(4, 32, seed=30)
    meta = K.fp8_quantize(x, block=8)
    dq = K.fp8_dequantize(meta)
    amax = x.abs().reshape(4, 4, 8).amax(-1)
    torch.testing.assert_close(meta.scale, amax / 448.0)
    err = (x - dq).abs().reshape(4, 4, 8).amax(-1)
    assert bool((err <= amax * 2.0 ** -4 + 1e-8).all())                                 # three mantissa bits: half an ulp of 2^-3
    odd = rand(2, 10, seed=31)                                                           # a ragged last block
    m2 = K.fp8_quantize(odd, block=8)
    assert m2.q.shape == (2, 10) and m2.scale.shape == (2, 2) and K.fp8_dequantize(m2).shape == (2, 10)
    torch.testing.assert_close(m2.scale[:, 1], odd[:, 8:].abs().amax(-1) / 448.0)
    for call in (lambda: K.fp8_quantize(x, block=0), lambda: K.fp8_quantize(torch.tensor(1.0)), lambda: K.fp8_quantize_2d(rand(2, 3, 4))):
        with pytest.raises(K.KernelError):
            call()


def test_fp8_two_dimensional_blocks():
    w = rand(10, 12, seed=32)
    meta = K.fp8_quantize_2d(w, block=4)
    assert meta.block2d and meta.scale.shape == (3, 3)
    tiles = torch.nn.functional.pad(w, (0, 0, 0, 2)).reshape(3, 4, 3, 4).abs().amax((1, 3))
    torch.testing.assert_close(meta.scale, tiles / 448.0)
    assert (w - K.fp8_dequantize(meta)).abs().max() <= w.abs().max() * 2.0 ** -4


def test_fp8_linear_is_the_product_of_the_dequantised_operands():
    x, w = rand(6, 16, seed=33), rand(5, 16, seed=34)
    y = K.fp8_linear(x, w, 8)
    want = K.fp8_dequantize(K.fp8_quantize(x, block=8)) @ K.fp8_dequantize(K.fp8_quantize(w, block=8)).T
    torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-5)
    assert (y - x @ w.T).abs().max() < 0.35 * (x @ w.T).abs().max()                     # close to the exact product, not equal
    assert not torch.equal(y, x @ w.T)
    yb = K.fp8_linear(x.reshape(2, 3, 16), w, 8)                                         # leading dimensions pass through
    torch.testing.assert_close(yb.reshape(6, 5), y)
    ident = K.fp8_linear(torch.tensor([[1.0, 2.0]]), torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), 2)
    torch.testing.assert_close(ident, torch.tensor([[1.0, 2.0, 3.0]]))
    for call in (lambda: K.fp8_linear(x, rand(5, 15), 8), lambda: K.fp8_linear(x[0, 0], w, 8), lambda: K.fp8_linear(x, w[0], 8)):
        with pytest.raises(K.KernelError):
            call()


def test_fp8_linear_gradient_is_straight_through_on_the_quantised_operands():
    x, w, g = rand(4, 16, seed=35), rand(3, 16, seed=36), rand(4, 3, seed=37)
    xq = K.fp8_dequantize(K.fp8_quantize(x, block=8))
    wq = K.fp8_dequantize(K.fp8_quantize(w, block=8))
    xs, ws = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    K.fp8_linear(xs, ws, 8).backward(g)
    torch.testing.assert_close(xs.grad, g @ wq, rtol=1e-5, atol=1e-5)                   # not g @ w
    torch.testing.assert_close(ws.grad, g.T @ xq, rtol=1e-5, atol=1e-5)
    assert not torch.allclose(xs.grad, g @ w, rtol=1e-6, atol=1e-7)
    y, res = K.fp8_linear_fwd(x, w, 8)
    gx, gw = K.fp8_linear_bwd(res, g)
    torch.testing.assert_close(gx, xs.grad)
    torch.testing.assert_close(gw, ws.grad)
    eps = 1e-4                                                                           # a finite difference of the rounding itself is (mostly) zero
    bumped = K.fp8_linear(x + eps * torch.ones_like(x), w, 8)
    assert (bumped - y).abs().max() < 0.5 and not torch.allclose((bumped - y) / eps, (torch.ones_like(x) @ wq.T), rtol=0.05, atol=0.05)


# ------------------------------------------------------------------------------ dispatch / combine
def meta_of(ids, probs, racks, n_experts, max_racks=K.MAX_RACKS):
    return K.DispatchMeta(torch.tensor(ids), torch.tensor(probs, dtype=torch.float32), torch.tensor(racks), n_experts, max_racks)


def test_dispatch_layout_and_padding():
    tokens = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    meta = meta_of([[0], [1], [0]], [[1.0], [1.0], [1.0]], [0, 1], 2)
    out, res = K.ep_dispatch(tokens, meta)
    assert out.tolist() == [[[1.0, 2.0], [5.0, 6.0]], [[3.0, 4.0], [0.0, 0.0]]]         # token order inside an expert, zero padding
    assert res.max_per_expert == 2 and res.token_index.tolist() == [[0, 2], [1, -1]]
    torch.testing.assert_close(K.ep_combine(out, meta, res), tokens)


def test_combine_weights_by_the_router_probabilities():
    tokens = rand(7, 5, seed=40)
    g = torch.Generator().manual_seed(41)
    ids = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(7)])
    probs = torch.rand(7, 2, generator=g)
    probs = probs / probs.sum(1, keepdim=True)
    meta = K.DispatchMeta(ids, probs, torch.arange(4) % 3, 4)
    out, res = K.ep_dispatch(tokens, meta)
    counts = torch.bincount(ids.reshape(-1), minlength=4)
    assert out.shape == (4, int(counts.max()), 5)
    torch.testing.assert_close(K.ep_combine(out, meta, res), tokens, rtol=1e-5, atol=1e-6)          # probabilities sum to one
    half = K.DispatchMeta(ids, probs * 0.5, meta.racks, 4)
    torch.testing.assert_close(K.ep_combine(out, half, res), 0.5 * tokens, rtol=1e-5, atol=1e-6)
    doubled = out * torch.arange(1, 5).float()[:, None, None]                             # expert e multiplies by e + 1
    want = torch.stack([sum(probs[t, j] * (ids[t, j] + 1) * tokens[t] for j in range(2)) for t in range(7)])
    torch.testing.assert_close(K.ep_combine(doubled, meta, res), want, rtol=1e-5, atol=1e-6)


def test_rack_span_limit():
    one = torch.ones(1, 3)
    with pytest.raises(K.KernelError):
        K.ep_dispatch(one, meta_of([[0, 1, 2, 3, 4]], [[0.2] * 5], [0, 1, 2, 3, 4], 5))
    for racks, max_racks in (([0, 1, 2, 3], 4), ([0, 0, 1, 2, 3], 4)):                   # exactly the limit; duplicates count once
        n = len(racks)
        meta = meta_of([list(range(n))], [[1.0 / n] * n], racks, n, max_racks)
        out, res = K.ep_dispatch(one, meta)
        torch.testing.assert_close(K.ep_combine(out, meta, res), one)
    with pytest.raises(K.KernelError):
        K.ep_dispatch(one, meta_of([[0, 1]], [[0.5, 0.5]], [0, 1], 2, max_racks=1))


def test_dispatch_argument_errors():
    tokens = torch.ones(3, 4)
    bad = [meta_of([[0], [1]], [[1.0], [1.0]], [0, 1], 2), meta_of([[0], [1], [0]], [[1.0], [1.0]], [0, 1], 2),
           meta_of([[0], [1], [0]], [[1.0], [1.0], [1.0]], [0], 2), meta_of([[9], [0], [0]], [[1.0]] * 3, [0, 1], 2),
           meta_of([[-1], [0], [0]], [[1.0]] * 3, [0, 1], 2)]
    for meta in bad:
        with pytest.raises(K.KernelError):
            K.ep_dispatch(tokens, meta)
    with pytest.raises(K.KernelError):
        K.ep_dispatch(torch.ones(3), bad[0])
    meta = meta_of([[0], [1], [0]], [[1.0]] * 3, [0, 1], 2)
    out, res = K.ep_dispatch(tokens, meta)
    with pytest.raises(K.KernelError):
        K.ep_combine(out[:, :1], meta, res)


def test_dispatch_and_combine_vjps_are_the_transposed_scatters():
    tokens = rand(5, 3, seed=50)
    ids = torch.tensor([[0, 2], [1, 2], [0, 1], [2, 0], [1, 0]])
    probs = torch.rand(5, 2, generator=torch.Generator().manual_seed(51))
    meta = K.DispatchMeta(ids, probs, torch.tensor([0, 1, 2]), 3)
    t = tokens.clone().requires_grad_(True)
    out, res = K.ep_dispatch(t, meta)
    g = rand(*out.shape, seed=52)
    (auto,) = torch.autograd.grad(out, t, g)
    want = torch.zeros_like(tokens)
    for e in range(3):
        for slot, tok in enumerate(res.token_index[e].tolist()):
            if tok >= 0:
                want[tok] += g[e, slot]
    torch.testing.assert_close(auto, want)
    _, r2 = K.ep_dispatch_fwd(tokens, meta)
    torch.testing.assert_close(K.ep_dispatch_bwd(r2, g), want)
    eo = out.detach().clone().requires_grad_(True)
    y = K.ep_combine(eo, meta, res)
    gy = rand(*y.shape, seed=53)
    (gauto,) = torch.autograd.grad(y, eo, gy)
    _, r3 = K.ep_combine_fwd(out.detach(), meta, res)
    torch.testing.assert_close(K.ep_combine_bwd(r3, gy), gauto)
    for e in range(3):                                                                   # padding slots get no gradient
        for slot, tok in enumerate(res.token_index[e].tolist()):
            if tok < 0:
                assert gauto[e, slot].abs().max() == 0
