"""Behaviour list of the model primitives on the host (``prometheus_b200.model``; reference
tests/test_model.py and model/__init__.py): configuration numbers and checks, the layer
pattern, RMSNorm, rotary embeddings (partial, full, two-dimensional), delta-rule linear
attention, the compressed-KV softmax attention, the routed mixture with its rack limit, the
latent adapter, parameter trees and the forward pass. Oracles are float64 NumPy restatements."""
import dataclasses
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import model as M


def rnd(*shape, seed=0):
    return np.random.default_rng(seed).standard_normal(shape)


def t32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32)


# ------------------------------------------------------------------------------ configuration
def test_flagship_and_tiny_numbers():
    f, t = M.flagship_config(), M.tiny_config()
    assert (f.d_model, f.n_layers, f.n_dense, f.n_moe, f.n_linear_attn, f.n_mla) == (12288, 96, 3, 93, 72, 24)
    assert (f.n_routed_experts, f.n_shared_experts, f.top_k, f.expert_hidden, f.mtp_heads, f.core_block_layers) == (512, 2, 20, 4096, 2, 8)
    assert (f.recurrence_train_mean, f.recurrence_max, f.vocab_size, f.max_context, f.max_racks) == (3.0, 16, 256000, 16384, 4)
    assert (t.d_model, t.n_layers, t.n_dense, t.n_moe, t.n_linear_attn, t.n_mla) == (128, 8, 1, 7, 6, 2)
    assert (t.n_routed_experts, t.n_shared_experts, t.top_k, t.expert_hidden, t.vocab_size, t.max_context) == (8, 2, 2, 256, 256, 128)
    assert (t.prelude_layers, t.coda_layers, t.core_block_layers, t.adapter_hidden) == (3, 3, 2, 128)
    for c in (f, t):
        M.validate_config(c)
        assert c.n_linear_attn == 3 * c.n_mla and c.n_dense + c.n_moe == c.n_layers
    assert [k.value for k in M.AttentionKind][:2] == ["linear", "mla"] and [k.value for k in M.FfnKind] == ["dense", "moe"]


@pytest.mark.parametrize("kw", [dict(n_linear_attn=5, n_mla=3), dict(n_dense=2), dict(n_linear_attn=7), dict(top_k=9), dict(n_layers=0, n_dense=0, n_moe=0,
                                n_linear_attn=0, n_mla=0), dict(d_model=0), dict(vocab_size=0), dict(n_shared_experts=-1), dict(mtp_heads=-1),
                                dict(prelude_layers=4, coda_layers=3)])
def test_invalid_configurations(kw):
    with pytest.raises(M.ConfigError):
        M.validate_config(dataclasses.replace(M.tiny_config(), **kw))


def test_layer_pattern():
    t = M.tiny_config()
    assert [M.attention_kind(i, t).value for i in range(8)] == ["linear", "linear", "linear", "mla"] * 2
    assert [M.ffn_kind(i, t).value for i in range(8)] == ["dense"] + ["moe"] * 7
    f = M.flagship_config()
    assert M.attention_kind(0, f) is M.AttentionKind.LINEAR and M.attention_kind(3, f) is M.AttentionKind.MLA and M.attention_kind(95, f) is M.AttentionKind.MLA
    assert sum(M.attention_kind(i, f) is M.AttentionKind.MLA for i in range(96)) == 24
    assert [M.ffn_kind(i, f).value for i in (0, 2, 3, 95)] == ["dense", "dense", "moe", "moe"]
    for bad in (-1, 8):
        with pytest.raises(M.AttentionKindError):
            M.attention_kind(bad, t)
        with pytest.raises(M.ConfigError):
            M.ffn_kind(bad, t)


# ------------------------------------------------------------------------------ RMSNorm
def test_rms_norm():
    x, w = rnd(3, 5, 16, seed=1), rnd(16, seed=2)
    want = x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-6) * w
    np.testing.assert_allclose(M.rms_norm(t32(x), t32(w)).numpy(), want, rtol=1e-5, atol=1e-6)
    assert M.rms_norm(torch.zeros(2, 8), torch.ones(8)).abs().max() == 0
    unit = M.rms_norm(t32(x), torch.ones(16))
    np.testing.assert_allclose((unit ** 2).mean(-1).numpy(), 1.0, rtol=1e-4)
    np.testing.assert_allclose(M.rms_norm(t32(7.0 * x), t32(w)).numpy(), want, rtol=1e-4, atol=1e-5)   # scale of the input drops out
    xt = torch.tensor(x[0, 0], dtype=torch.float64, requires_grad=True)
    wt = torch.tensor(w, dtype=torch.float64)
    M.rms_norm(xt, wt).sum().backward()
    h = 1e-6
    d = rnd(16, seed=3)
    f = lambda v: float((v / np.sqrt((v ** 2).mean() + 1e-6) * w).sum())
    assert float((xt.grad.numpy() * d).sum()) == pytest.approx((f(x[0, 0] + h * d) - f(x[0, 0] - h * d)) / (2 * h), rel=1e-3, abs=1e-5)


# ------------------------------------------------------------------------------ rotary embeddings
def np_rope(x, pos, partial, base=10000.0):
    x = np.asarray(x, dtype=np.float64)
    d = x.shape[-1]
    n_pairs = d // 2
    n_rot = max(1, n_pairs // 2) if partial else n_pairs
    out = x.copy()
    inv = base ** (-2.0 * np.arange(n_rot) / (2 * n_rot))
    ang = np.asarray(pos, dtype=np.float64)[:, None] * inv                               # (seq, n_rot)
    ang = ang[None, :, None, :] if x.ndim == 4 else ang[None, :, :]
    ev, od = x[..., 0:2 * n_rot:2], x[..., 1:2 * n_rot:2]
    out[..., 0:2 * n_rot:2] = ev * np.cos(ang) - od * np.sin(ang)
    out[..., 1:2 * n_rot:2] = ev * np.sin(ang) + od * np.cos(ang)
    return out


def test_rope_partial_and_full():
    q, k = rnd(2, 6, 3, 16, seed=4), rnd(2, 6, 3, 16, seed=5)
    pos = np.arange(6)
    for partial in (True, False):
        rq, rk = M.rope(t32(q), t32(k), torch.arange(6), partial=partial)
        np.testing.assert_allclose(rq.numpy(), np_rope(q, pos, partial), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(rk.numpy(), np_rope(k, pos, partial), rtol=1e-4, atol=1e-5)
    rq, _ = M.rope(t32(q), t32(k), torch.arange(6), partial=True)
    assert torch.equal(rq[..., 8:], t32(q)[..., 8:])                                      # the second half is passed through
    assert torch.equal(rq[:, 0], t32(q)[:, 0])                                            # position zero is the identity
    full, _ = M.rope(t32(q), t32(k), torch.arange(6), partial=False)
    pair = lambda x: x[..., 0::2] ** 2 + x[..., 1::2] ** 2
    np.testing.assert_allclose(pair(full).numpy(), pair(t32(q)).numpy(), rtol=1e-4, atol=1e-5)    # a rotation keeps pair norms
    a, b = M.rope(t32(q[:, :, 0]), t32(k[:, :, 0]), torch.arange(6), partial=False)       # 3-D input: no head axis
    np.testing.assert_allclose(a.numpy(), np_rope(q[:, :, 0], pos, False), rtol=1e-4, atol=1e-5)
    shift, _ = M.rope(t32(q), t32(k), torch.arange(6) + 11, partial=False)                # relative: scores depend on the offset only
    base_scores = np.einsum("bqhd,bkhd->bhqk", *(x.numpy() for x in M.rope(t32(q), t32(k), torch.arange(6), partial=False)))
    shifted = np.einsum("bqhd,bkhd->bhqk", *(x.numpy() for x in M.rope(t32(q), t32(k), torch.arange(6) + 11, partial=False)))
    np.testing.assert_allclose(shifted, base_scores, rtol=1e-3, atol=1e-3)


def test_rope_two_dimensional():
    q, k = rnd(1, 6, 2, 8, seed=6), rnd(1, 6, 2, 8, seed=7)
    row, col = np.array([0, 0, 0, 1, 1, 1]), np.array([0, 1, 2, 0, 1, 2])
    rq, rk = M.rope_2d(t32(q), t32(k), torch.tensor(row), torch.tensor(col))
    want = np.concatenate([np_rope(q[..., :4], row, False), np_rope(q[..., 4:], col, False)], -1)
    np.testing.assert_allclose(rq.numpy(), want, rtol=1e-4, atol=1e-5)
    assert torch.equal(rq[:, 0], t32(q)[:, 0])                                            # cell (0, 0) is untouched
    with pytest.raises(ValueError):
        M.rope_2d(t32(q[..., :7]), t32(k[..., :7]), torch.tensor(row), torch.tensor(col))


# ------------------------------------------------------------------------------ linear attention
def np_delta(q, k, v, s0=None):
    q, k, v = (np.asarray(x, dtype=np.float64) for x in (q, k, v))
    norm = lambda x: x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-6)
    q, k = norm(q), norm(k)
    b, s, h, d = q.shape
    S = np.zeros((b, h, d, d)) if s0 is None else np.asarray(s0, dtype=np.float64).copy()
    out = np.zeros_like(v)
    for t in range(s):
        for i in range(b):
            for j in range(h):
                kt = k[i, t, j]
                S[i, j] += np.outer(kt, v[i, t, j] - S[i, j].T @ kt)
                out[i, t, j] = S[i, j].T @ q[i, t, j]
    return out, S


def test_linear_attention_is_the_delta_rule_on_normalised_keys():
    q, k, v = rnd(2, 9, 2, 8, seed=8), rnd(2, 9, 2, 8, seed=9), rnd(2, 9, 2, 8, seed=10)
    o, s = M.linear_attention(t32(q), t32(k), t32(v))
    wo, ws = np_delta(q, k, v)
    np.testing.assert_allclose(o.numpy(), wo, rtol=2e-3, atol=2e-4)
    np.testing.assert_allclose(s.numpy(), ws, rtol=2e-3, atol=2e-4)
    v2 = v.copy()
    v2[:, 6:] += 3.0
    o2, _ = M.linear_attention(t32(q), t32(k), t32(v2))
    assert torch.equal(o2[:, :6], o[:, :6]) or torch.allclose(o2[:, :6], o[:, :6], atol=1e-6)         # causal
    oa, sa = M.linear_attention(t32(q[:, :5]), t32(k[:, :5]), t32(v[:, :5]))
    ob, sb = M.linear_attention(t32(q[:, 5:]), t32(k[:, 5:]), t32(v[:, 5:]), state=sa)
    torch.testing.assert_close(torch.cat([oa, ob], 1), o, rtol=1e-4, atol=1e-5)                       # chunks chained through the state
    torch.testing.assert_close(sb, s, rtol=1e-4, atol=1e-5)
    o3, s3 = M.linear_attention(t32(q[:, :, 0]), t32(k[:, :, 0]), t32(v[:, :, 0]))                   # 3-D input: one head, squeezed back
    assert o3.shape == (2, 9, 8) and s3.shape == (2, 8, 8)
    torch.testing.assert_close(o3, o[:, :, 0], rtol=1e-4, atol=1e-5)
    gated, _ = M.linear_attention(t32(q), t32(k), t32(v), beta=torch.full((2, 9, 2), 0.5))
    assert not torch.allclose(gated, o)
    with pytest.raises(ValueError):
        M.linear_attention(t32(q), t32(k[:, :8]), t32(v))
    with pytest.raises(ValueError):
        M.linear_attention(t32(q), t32(k), t32(v), state=torch.zeros(2, 2, 4, 4))


# ------------------------------------------------------------------------------ softmax attention
def np_softmax_attention(q, k, v):
    scores = np.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(q.shape[-1])
    sq, sk = q.shape[1], k.shape[1]
    mask = np.arange(sk)[None, :] > (np.arange(sq)[:, None] + (sk - sq))
    scores = np.where(mask[None, None], -1e9, scores)
    w = np.exp(scores - scores.max(-1, keepdims=True))
    w /= w.sum(-1, keepdims=True)
    return np.einsum("bhqk,bkhd->bqhd", w, v)


def test_compressed_kv_attention():
    q, ckv, rk = rnd(2, 5, 3, 12, seed=11), rnd(2, 5, 8, seed=12), rnd(2, 5, 4, seed=13)
    got = M.mla_attention(t32(q), t32(ckv), t32(rk), qk_norm=False)
    kk = np.broadcast_to(np.concatenate([ckv, rk], -1)[:, :, None], (2, 5, 3, 12))
    vv = np.broadcast_to(ckv[:, :, None], (2, 5, 3, 8))
    np.testing.assert_allclose(got.numpy(), np_softmax_attention(q, kk, vv), rtol=1e-4, atol=1e-5)
    assert got.shape == (2, 5, 3, 8)                                                      # values are the compressed part only
    normed = M.mla_attention(t32(q), t32(ckv), t32(rk))
    rms = lambda x: x / np.sqrt((x ** 2).mean(-1, keepdims=True) + 1e-6)
    np.testing.assert_allclose(normed.numpy(), np_softmax_attention(rms(q), rms(kk), vv), rtol=1e-4, atol=1e-5)
    ckv2 = ckv.copy()
    ckv2[:, 3:] += 2.0
    later = M.mla_attention(t32(q), t32(ckv2), t32(rk), qk_norm=False)
    torch.testing.assert_close(later[:, :3], got[:, :3])                                  # causal
    for bad in ((t32(q[:, :, 0]), t32(ckv), t32(rk)), (t32(q), t32(ckv[..., :7]), t32(rk)), (t32(q), t32(rnd(2, 5, 2, 8)), t32(rk))):
        with pytest.raises(ValueError):
            M.mla_attention(*bad)


def test_grouped_query_attention():
    q, k, v = rnd(1, 6, 4, 8, seed=14), rnd(1, 6, 2, 8, seed=15), rnd(1, 6, 2, 8, seed=16)
    got = M.gqa_attention(t32(q), t32(k), t32(v))
    np.testing.assert_allclose(got.numpy(), np_softmax_attention(q, np.repeat(k, 2, 2), np.repeat(v, 2, 2)), rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        M.gqa_attention(t32(q), t32(rnd(1, 6, 3, 8)), t32(rnd(1, 6, 3, 8)))


# ------------------------------------------------------------------------------ mixture of experts
def np_moe(x, wr, routed, shared, top_k):
    x = np.asarray(x, dtype=np.float64)
    silu = lambda z: z / (1 + np.exp(-z))
    ffn = lambda z, g, u, d: (silu(z @ g) * (z @ u)) @ d
    probs = 1 / (1 + np.exp(-(x @ wr)))
    out = np.zeros_like(x)
    ids = np.zeros((x.shape[0], top_k), dtype=np.int64)
    for t in range(x.shape[0]):
        order = np.argsort(-probs[t], kind="stable")[:top_k]
        ids[t] = order
        gates = probs[t, order] / max(probs[t, order].sum(), 1e-9)
        for e, g in zip(order, gates):
            out[t] += g * ffn(x[t], routed[0][e], routed[1][e], routed[2][e])
        for j in range(shared[0].shape[0]):
            out[t] += ffn(x[t], shared[0][j], shared[1][j], shared[2][j])
    return out, probs, ids


def test_moe_is_top_k_sigmoid_gates_plus_shared_experts():
    d, h, e = 8, 6, 4
    x, wr = rnd(5, d, seed=17), rnd(d, e, seed=18)
    routed = [0.3 * rnd(e, d, h, seed=19), 0.3 * rnd(e, d, h, seed=20), 0.3 * rnd(e, h, d, seed=21)]
    shared = [0.3 * rnd(2, d, h, seed=22), 0.3 * rnd(2, d, h, seed=23), 0.3 * rnd(2, h, d, seed=24)]
    out, probs, ids = M.moe(t32(x), router_weight=t32(wr), routed_weights=[t32(w) for w in routed], shared_weights=[t32(w) for w in shared], top_k=2)
    wo, wp, wi = np_moe(x, wr, routed, shared, 2)
    np.testing.assert_allclose(out.numpy(), wo, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(probs.numpy(), wp, rtol=1e-5)
    assert np.array_equal(ids.numpy(), wi) and ids.dtype == torch.int32
    assert all(len(set(r)) == 2 and 0 <= min(r) and max(r) < e for r in ids.tolist())
    batched, _, bids = M.moe(t32(x).reshape(1, 5, d), router_weight=t32(wr), routed_weights=[t32(w) for w in routed],
                             shared_weights=[t32(w) for w in shared], top_k=2)
    torch.testing.assert_close(batched.reshape(5, d), out)
    assert bids.shape == (1, 5, 2)
    bias = torch.tensor([0.0, 0.0, 0.0, 100.0])                                           # the bias picks, the gates ignore it
    _, _, forced = M.moe(t32(x), router_weight=t32(wr), routed_weights=[t32(w) for w in routed], shared_weights=[t32(w) for w in shared],
                         top_k=2, router_bias=bias)
    assert all(3 in r for r in forced.tolist())


def test_rack_limit_binds_the_choice():
    scores = torch.tensor([[0.9, 0.1, 0.8, 0.2, 0.7, 0.3, 0.6, 0.4]])                     # 8 experts on 8 racks when the limit is 8
    free = M._node_limited_topk(scores, 4, 8)
    assert free.tolist() == [[0, 2, 4, 6]]
    two = M._node_limited_topk(scores, 4, 2)                                              # racks {0..3} and {4..7}: both used, plain top-4
    assert sorted(two.tolist()[0]) == [0, 2, 4, 6]
    racks = M._expert_to_rack(8, 2)
    assert racks.tolist() == [0, 0, 0, 0, 1, 1, 1, 1] and M._expert_to_rack(6, 4).tolist() == [0, 0, 1, 2, 2, 3]
    tie = M._node_limited_topk(torch.ones(1, 5), 3, 8)
    assert tie.tolist() == [[0, 1, 2]]                                                    # ties go to the lower index


# ------------------------------------------------------------------------------ adapter / parameters / forward
def test_latent_adapter_shape_and_unit_scale():
    x = t32(rnd(2, 3, 16, seed=25))
    y = M.latent_adapter(x, hidden=16)
    assert y.shape == x.shape and y.dtype == torch.float32
    np.testing.assert_allclose((y ** 2).mean(-1).numpy(), 1.0, rtol=5e-3)              # small outputs: the epsilon of the norm shows


def test_parameter_tree_and_counts():
    c = M.tiny_config()
    p = M.init_params(c, 0)
    flat = M.flatten_params(p)
    assert M.param_count(p) == sum(v.numel() for v in flat.values()) and 5e6 < M.param_count(p) < 2e7
    assert all(v.dtype == torch.float32 for v in flat.values())
    again = M.flatten_params(M.init_params(c, 0))
    assert all(torch.equal(flat[k], again[k]) for k in flat)                              # same seed, same tree
    other = M.flatten_params(M.init_params(c, 1))
    assert any(not torch.equal(flat[k], other[k]) for k in flat)
    back = M.flatten_params(M.unflatten_params(flat))
    assert list(back) == list(flat) and all(torch.equal(back[k], flat[k]) for k in flat)
    lin = {k.split(".", 2)[2] for k in flat if k.startswith("layers.0.")}
    mla = {k.split(".", 2)[2] for k in flat if k.startswith("layers.3.")}
    assert lin != mla and any("kv" in k.lower() for k in mla - lin)                       # the two attention kinds carry different leaves


def test_forward_shapes_thoughts_and_recurrence():
    c = M.tiny_config()
    p = M.init_params(c, 0)
    tokens = torch.randint(0, c.vocab_size, (2, 12), generator=torch.Generator().manual_seed(1))
    out = M.forward(tokens, p, c, r=1)
    assert out.logits.shape == (2, 12, c.vocab_size) and len(out.mtp_logits) == c.mtp_heads and bool(torch.isfinite(out.logits).all())
    same = M.forward(tokens, p, c, r=1)
    assert torch.equal(out.logits, same.logits)
    r2 = M.forward(tokens, p, c, r=2)
    assert not torch.allclose(r2.logits, out.logits)                                      # the core block ran twice
    one = M.forward(tokens[:, :1], p, c, r=1)
    assert one.logits.shape == (2, 1, c.vocab_size)
    changed = tokens.clone()
    changed[:, 8:] = (changed[:, 8:] + 1) % c.vocab_size
    later = M.forward(changed, p, c, r=1)
    torch.testing.assert_close(later.logits[:, :8], out.logits[:, :8], rtol=1e-4, atol=1e-5)      # causal end to end
    with pytest.raises((IndexError, ValueError, RuntimeError)):
        M.forward(torch.full((1, 4), c.vocab_size), p, c, r=1)
