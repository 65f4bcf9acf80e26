"""Behaviour list of the optimizer and loss arithmetic (``prometheus_b200.train``; reference
tests/test_train.py, tests/test_mup_muon.py and train/__init__.py): configuration checks, the
Muon / AdamW split, the precision map, Newton-Schulz orthogonalisation, the two Muon step
forms, QK-clip, AdamW with 1-based bias correction, the warmup-stable-decay schedule and the
loss terms. Oracles are float64 NumPy restatements written here."""
import dataclasses
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import train as T

NS = (3.4445, -4.7750, 2.0315)


def np_ns(g, steps):
    g = np.asarray(g, dtype=np.float64)
    t = g.shape[0] > g.shape[1]
    x = g.T if t else g
    fro = np.linalg.norm(x)
    x = x / fro if fro > 1e-7 else np.zeros_like(x)
    a, b, c = NS
    for _ in range(steps):
        gram = x @ x.T
        x = a * x + (b * gram + c * gram @ gram) @ x
    return x.T if t else x


def rnd(*shape, seed=0):
    return np.random.default_rng(seed).standard_normal(shape)


# ------------------------------------------------------------------------------ configuration
def test_flagship_and_tiny_constants():
    f, t = T.flagship_train_config(), T.tiny_train_config()
    assert (f.peak_lr, f.muon_lr, f.adamw_lr, f.adamw_eps, f.adamw_wd) == (2e-4, 2e-2, 2e-4, 1e-8, 0.1)
    assert (f.muon_momentum, f.muon_ns_steps, f.warmup_steps, f.stable_steps, f.decay_steps) == (0.95, 5, 2000, 500000, 100000)
    assert (f.z_loss_weight, f.softcap, f.qk_clip, f.grad_clip, f.n_layers) == (1e-3, 30.0, 100.0, 1.0, 96)
    assert (t.warmup_steps, t.stable_steps, t.decay_steps, t.fp8_block, t.n_layers) == (2, 8, 4, 16, 8) and t.muon_ns_steps == 5
    assert [k.value for k in T.ParamKind][:2] == ["muon_2d", "adamw"] or {k.name for k in T.ParamKind} >= {"MUON_2D", "ADAMW"}
    assert {k.name for k in T.PrecisionKind} >= {"FP8_LINEAR", "BF16_STABLE"}
    for c in (f, t):
        T.validate_train_config(c)
    with pytest.raises(dataclasses.FrozenInstanceError):
        f.peak_lr = 1.0


@pytest.mark.parametrize("kw", [dict(peak_lr=0.0), dict(muon_lr=-1e-3), dict(adamw_lr=0.0), dict(warmup_steps=0, stable_steps=0, decay_steps=0),
                                dict(bf16_tail_layers=9)])
def test_invalid_train_configurations(kw):
    with pytest.raises(T.TrainConfigError):
        T.validate_train_config(dataclasses.replace(T.tiny_train_config(), **kw))
    T.validate_train_config(dataclasses.replace(T.tiny_train_config(), bf16_tail_layers=8))     # the whole stack may be the tail


# ------------------------------------------------------------------------------ parameter split / precision
def test_only_two_dimensional_hidden_weights_go_to_muon():
    m = np.zeros((4, 4))
    for name in ("layers.0.attn.W_q", "layers.3.ffn.w_up", "head.proj"):
        assert T.classify_param(name, m) is T.ParamKind.MUON_2D
    for name in ("embed.table", "layers.0.norm1.scale", "layers.0.attn.bias_q", "latent.sigma_head", "final_NORM.w"):
        assert T.classify_param(name, m) is T.ParamKind.ADAMW                            # by name, whatever the shape
    assert T.classify_param("layers.0.ffn.w", np.zeros(4)) is T.ParamKind.ADAMW
    assert T.classify_param("layers.0.moe.routed_up", np.zeros((2, 4, 4))) is T.ParamKind.ADAMW  # 3-D is not "2-D"
    assert T.classify_param("x", torch.zeros(3, 5)) is T.ParamKind.MUON_2D


def test_precision_map():
    c = T.tiny_train_config()                                                            # 8 layers, the last two stay bf16
    assert T.precision_for("layers.0.attn.W_q", c) is T.PrecisionKind.FP8_LINEAR
    assert T.precision_for("layers.5.ffn.w_down", c) is T.PrecisionKind.FP8_LINEAR
    for name in ("layers.6.attn.W_q", "layers.7.ffn.w_up"):
        assert T.precision_for(name, c) is T.PrecisionKind.BF16_STABLE
    for name in ("layers.1.moe.router.w", "layers.1.norm1.scale", "embed.table", "latent_adapter.w_in", "layers.2.attn.softmax_scale"):
        assert T.precision_for(name, c) is T.PrecisionKind.BF16_STABLE
    kinds = {T.precision_for(n, c) for n in ("a", "layers.0.x", "embed", "layers.7.x")}
    assert kinds <= {T.PrecisionKind.FP8_LINEAR, T.PrecisionKind.BF16_STABLE}            # never the fp32 master kind


# ------------------------------------------------------------------------------ Newton-Schulz
def test_newton_schulz_matches_the_float64_iteration():
    for shape in ((4, 4), (3, 7), (9, 2), (16, 16)):
        g = rnd(*shape, seed=sum(shape))
        for steps in (1, 3, 5):
            got = T.newton_schulz(g, steps)
            assert got.shape == shape and got.dtype == torch.float32
            np.testing.assert_allclose(got.numpy(), np_ns(g, steps), rtol=2e-3, atol=2e-4)
    for bad in (0, 2, 4, -1):
        with pytest.raises(ValueError):
            T.newton_schulz(rnd(3, 3), bad)
    for bad in (rnd(3), rnd(2, 2, 2, 2)):
        with pytest.raises(ValueError):
            T.newton_schulz(bad, 5)


def test_newton_schulz_properties():
    g = rnd(32, 8, seed=3)
    o = T.newton_schulz(g, 5).double().numpy()
    sv = np.linalg.svd(o, compute_uv=False)
    assert 0.6 < sv.min() and sv.max() < 1.25                                            # roughly orthonormal columns
    np.testing.assert_allclose(T.newton_schulz(7.5 * g, 5).numpy(), T.newton_schulz(g, 5).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(T.newton_schulz(-g, 5).numpy(), -T.newton_schulz(g, 5).numpy(), rtol=1e-5, atol=1e-6)   # an odd map
    assert T.newton_schulz(np.zeros((3, 5)), 5).abs().max() == 0
    stack = np.stack([rnd(4, 6, seed=i) for i in range(3)])
    batched = T.newton_schulz(stack, 5)
    for i in range(3):
        np.testing.assert_allclose(batched[i].numpy(), T.newton_schulz(stack[i], 5).numpy(), rtol=1e-5, atol=1e-6)
    u, _, vt = np.linalg.svd(g, full_matrices=False)
    assert np.abs(o - u @ vt).max() < 0.35                                               # near the polar factor


# ------------------------------------------------------------------------------ Muon
def test_muon_update_is_nesterov_then_orthogonalise_with_the_jordan_scale():
    g, m = rnd(8, 4, seed=1), rnd(8, 4, seed=2)
    delta, new_m = T.muon_update(g, m, lr=0.02, momentum_coeff=0.95, ns_steps=5)
    want_m = 0.95 * m + g
    np.testing.assert_allclose(new_m.numpy(), want_m, rtol=1e-5, atol=1e-6)
    want = 0.02 * math.sqrt(max(1.0, 8 / 4)) * np_ns(g + 0.95 * want_m, 5)
    np.testing.assert_allclose(delta.numpy(), want, rtol=3e-3, atol=3e-5)
    wide, _ = T.muon_update(g.T, m.T, lr=0.02, momentum_coeff=0.95, ns_steps=5)
    np.testing.assert_allclose(wide.numpy(), 0.02 * np_ns((g + 0.95 * want_m).T, 5), rtol=3e-3, atol=3e-5)     # no scale when wide
    zero_delta, kept = T.muon_update(np.zeros((4, 4)), m[:4], lr=0.02, momentum_coeff=0.9, ns_steps=5)
    np.testing.assert_allclose(kept.numpy(), 0.9 * m[:4], rtol=1e-5, atol=1e-6)                     # momentum decays, and still drives the step
    assert zero_delta.abs().max() > 0
    for bad in ((g, m[:4]), (g[0], m[0])):
        with pytest.raises(ValueError):
            T.muon_update(*bad, lr=0.02, momentum_coeff=0.9, ns_steps=5)


@pytest.mark.parametrize("rows, cols", [(1, 1), (4, 16), (16, 4), (128, 128), (2048, 5632)])
def test_rms_scale_depends_on_the_longer_side(rows, cols):
    assert T.muon_rms_scale(rows, cols) == pytest.approx(0.2 * math.sqrt(max(rows, cols)))
    assert T.muon_rms_scale(rows, cols) == T.muon_rms_scale(cols, rows)


def test_rms_scale_and_lr_transfer_argument_errors():
    for bad in ((0, 4), (4, 0), (-1, 4), (1.5, 4), (True, 4), ("4", 4)):
        with pytest.raises(ValueError):
            T.muon_rms_scale(*bad)
    for lr, w, bw in ((2e-2, 512, 4096), (1.0, 1, 1), (0.0, 8, 8)):
        assert T.transferred_muon_lr(lr, width=w, base_width=bw) == lr                   # transfers unchanged
    for kw in (dict(base_lr=-1.0, width=8, base_width=8), dict(base_lr=math.nan, width=8, base_width=8), dict(base_lr=0.1, width=0, base_width=8),
               dict(base_lr=0.1, width=8, base_width=-2), dict(base_lr="0.1", width=8, base_width=8), dict(base_lr=0.1, width=8.0, base_width=8)):
        with pytest.raises(ValueError):
            T.transferred_muon_lr(**kw)


def test_transfer_step_is_rms_matched_with_decoupled_decay():
    p, g, m = rnd(6, 10, seed=4), rnd(6, 10, seed=5), rnd(6, 10, seed=6)
    kw = dict(lr=0.02, momentum_coeff=0.95, ns_steps=5, weight_decay=0.1)
    new_p, new_m = T.muon_transfer_step(p, g, m, **kw)
    want_m = 0.95 * m + g
    orth = np_ns(g + 0.95 * want_m, 5)
    np.testing.assert_allclose(new_m.numpy(), want_m, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(new_p.numpy(), p - 0.02 * (0.2 * math.sqrt(10) * orth + 0.1 * p), rtol=3e-3, atol=3e-5)
    no_wd, _ = T.muon_transfer_step(p, g, m, **{**kw, "weight_decay": 0.0})
    np.testing.assert_allclose((new_p - no_wd).numpy(), -0.02 * 0.1 * p, rtol=1e-4, atol=1e-7)     # decay does not pass through Newton-Schulz
    decay_only, _ = T.muon_transfer_step(p, np.zeros_like(g), np.zeros_like(m), **kw)
    np.testing.assert_allclose(decay_only.numpy(), p * (1 - 0.02 * 0.1), rtol=1e-6)
    held, moved = T.muon_transfer_step(p, g, m, **{**kw, "lr": 0.0})
    np.testing.assert_allclose(held.numpy(), p, rtol=1e-7)
    np.testing.assert_allclose(moved.numpy(), want_m, rtol=1e-5, atol=1e-6)              # momentum still advances
    plain, pm = T.muon_transfer_step(p, g, m, **{**kw, "momentum_coeff": 0.0})
    np.testing.assert_allclose(pm.numpy(), g, rtol=1e-7)
    np.testing.assert_allclose(plain.numpy(), p - 0.02 * (0.2 * math.sqrt(10) * np_ns(g, 5) + 0.1 * p), rtol=3e-3, atol=3e-5)
    before = (p.copy(), g.copy(), m.copy())
    T.muon_transfer_step(p, g, m, **kw)
    assert all(np.array_equal(a, b) for a, b in zip(before, (p, g, m)))                  # inputs untouched
    p2, m2 = T.muon_transfer_step(new_p, g, new_m, **kw)                                 # momentum carries over steps
    np.testing.assert_allclose(m2.numpy(), 0.95 * want_m + g, rtol=1e-5, atol=1e-6)
    assert not np.allclose(p2.numpy(), new_p.numpy())


@pytest.mark.parametrize("kw", [dict(lr=math.nan), dict(lr="x"), dict(weight_decay=-0.1), dict(weight_decay=math.inf), dict(ns_steps=4),
                                dict(ns_steps=0), dict(ns_steps=5.0), dict(ns_steps=True)])
def test_transfer_step_argument_errors(kw):
    p = rnd(4, 4)
    base = dict(lr=0.02, momentum_coeff=0.95, ns_steps=5, weight_decay=0.1)
    with pytest.raises(ValueError):
        T.muon_transfer_step(p, p, p, **{**base, **kw})
    for shapes in ((p, p[:2], p), (p[0], p[0], p[0]), (np.zeros((0, 4)),) * 3):
        with pytest.raises(ValueError):
            T.muon_transfer_step(*shapes, **base)


# ------------------------------------------------------------------------------ QK-clip / AdamW / schedule
def test_qk_clip_caps_the_largest_logit():
    q, k = 5.0 * rnd(6, 8, seed=7), 5.0 * rnd(9, 8, seed=8)
    mx = np.abs(q @ k.T).max()
    q2, k2 = T.qk_clip(q, k, mx / 4)
    assert float((q2 @ k2.T).abs().max()) == pytest.approx(mx / 4, rel=1e-4)
    s = math.sqrt(1 / 4)
    np.testing.assert_allclose(q2.numpy(), q * s, rtol=1e-5)
    np.testing.assert_allclose(k2.numpy(), k * s, rtol=1e-5)                             # split evenly between q and k
    q3, k3 = T.qk_clip(q, k, mx * 2)
    np.testing.assert_allclose(q3.numpy(), q, rtol=1e-6)                                 # below the cap nothing changes
    qb, kb = T.qk_clip(np.stack([q, 0.1 * q]), np.stack([k, 0.1 * k]), mx / 4)           # one scale for the whole batch
    assert float((qb @ kb.transpose(-1, -2)).abs().max()) == pytest.approx(mx / 4, rel=1e-4)
    for cap in (0.0, -1.0):
        with pytest.raises(ValueError):
            T.qk_clip(q, k, cap)
    with pytest.raises(ValueError):
        T.qk_clip(q, k[:, :4], 1.0)


def test_adamw_is_decoupled_with_one_based_bias_correction():
    p, g = rnd(5, seed=9), rnd(5, seed=10)
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, wd=0.1)
    p1, m1, v1 = T.adamw_update(p, g, np.zeros(5), np.zeros(5), step=1, **kw)
    m, v = 0.1 * g, 0.01 * g * g
    want = p * (1 - 1e-2 * 0.1) - 1e-2 * (m / 0.1) / (np.sqrt(v / 0.01) + 1e-8)
    np.testing.assert_allclose(p1.numpy(), want, rtol=1e-5)
    np.testing.assert_allclose(m1.numpy(), m, rtol=1e-6)
    np.testing.assert_allclose(v1.numpy(), v, rtol=1e-6)
    p2, m2, v2 = T.adamw_update(p1, g, m1, v1, step=2, **kw)
    mm, vv = 0.9 * m + 0.1 * g, 0.99 * v + 0.01 * g * g
    want2 = p1.numpy() * (1 - 1e-3) - 1e-2 * (mm / (1 - 0.81)) / (np.sqrt(vv / (1 - 0.9801)) + 1e-8)
    np.testing.assert_allclose(p2.numpy(), want2, rtol=1e-5)
    same_m = T.adamw_update(p1, g, m1, v1, step=1, **kw)[0]
    assert not np.allclose(same_m.numpy(), p2.numpy())                                   # the step number matters
    nowd = T.adamw_update(p, g, np.zeros(5), np.zeros(5), step=1, **{**kw, "wd": 0.0})[0]
    np.testing.assert_allclose((p1 - nowd).numpy(), -1e-3 * p, rtol=1e-4, atol=1e-9)     # decay acts on the weights, not on the gradient
    for bad in (0, -1):
        with pytest.raises(ValueError):
            T.adamw_update(p, g, m, v, step=bad, **kw)


def test_warmup_stable_decay_schedule():
    c = T.tiny_train_config()                                                            # 2 + 8 + 4 steps
    peak = c.peak_lr
    got = [T.wsd_lr(s, c) for s in range(1, 17)]
    want = [peak * 0.5, peak] + [peak] * 8 + [peak * 0.75, peak * 0.5, peak * 0.25, 0.0] + [0.0, 0.0]
    assert got == pytest.approx(want)
    f = T.flagship_train_config()
    assert T.wsd_lr(1, f) == pytest.approx(f.peak_lr / 2000) and T.wsd_lr(2000, f) == f.peak_lr and T.wsd_lr(502000, f) == f.peak_lr
    assert T.wsd_lr(552000, f) == pytest.approx(f.peak_lr / 2) and T.wsd_lr(602000, f) == 0.0 and T.wsd_lr(10 ** 7, f) == 0.0
    no_warm = dataclasses.replace(c, warmup_steps=0)
    assert T.wsd_lr(1, no_warm) == peak
    for bad in (0, -3):
        with pytest.raises(ValueError):
            T.wsd_lr(bad, c)


# ------------------------------------------------------------------------------ losses
def test_soft_cap():
    x = np.array([-1000.0, -30.0, 0.0, 3.0, 30.0, 1000.0])
    np.testing.assert_allclose(T.soft_cap(x, 30.0).numpy(), 30 * np.tanh(x / 30), rtol=1e-6)
    assert float(T.soft_cap(1e9, 30.0)) == pytest.approx(30.0) and float(T.soft_cap(0.01, 30.0)) == pytest.approx(0.01, rel=1e-4)
    for cap in (0.0, -5.0):
        with pytest.raises(ValueError):
            T.soft_cap(x, cap)


def test_masked_cross_entropy():
    lg = rnd(2, 4, 7, seed=11)
    tg = np.random.default_rng(12).integers(0, 7, (2, 4))
    mask = np.array([[1, 1, 0, 1], [0, 0, 1, 1]], dtype=np.float32)
    ls = lg - lg.max(-1, keepdims=True)
    nll = -(np.take_along_axis(ls, tg[..., None], -1)[..., 0] - np.log(np.exp(ls).sum(-1)))
    assert float(T.cross_entropy(lg, tg, mask)) == pytest.approx(float((nll * mask).sum() / mask.sum()), rel=1e-5)
    assert float(T.cross_entropy(lg, tg, np.zeros((2, 4)))) == 0.0
    assert float(T.cross_entropy(lg, tg, 2 * mask)) == pytest.approx(float((nll * mask).sum() / mask.sum()), rel=1e-5)   # a weighted mean
    for bad in ((lg, tg[:, :3], mask), (lg, tg, mask[:, :3]), (lg[0], tg, mask)):
        with pytest.raises(ValueError):
            T.cross_entropy(*bad)


def test_mtp_head_i_predicts_the_token_i_plus_one_ahead():
    tokens = np.array([[3, 1, 4, 1, 5]])
    mask = np.ones((1, 5), dtype=np.float32)
    v = 6

    def one_hot_logits(offset):
        lg = np.full((1, 5, v), -20.0)
        for t in range(5 - offset):
            lg[0, t, tokens[0, t + offset]] = 20.0
        return lg

    perfect = T.mtp_loss([one_hot_logits(1), one_hot_logits(2)], tokens, mask)
    assert float(perfect) < 1e-6
    swapped = T.mtp_loss([one_hot_logits(2), one_hot_logits(1)], tokens, mask)
    assert float(swapped) > 5.0
    h0 = T.cross_entropy(one_hot_logits(2)[:, :4], tokens[:, 1:], mask[:, 1:])
    h1 = T.cross_entropy(one_hot_logits(1)[:, :3], tokens[:, 2:], mask[:, 2:])
    assert float(swapped) == pytest.approx(float((h0 + h1) / 2), rel=1e-5)               # the mean over heads
    holes = np.array([[1, 1, 0, 1, 1]], dtype=np.float32)                                # both ends of a pair must be unmasked
    got = T.mtp_loss([rnd(1, 5, v, seed=13)], tokens, holes)
    want = T.cross_entropy(rnd(1, 5, v, seed=13)[:, :4], tokens[:, 1:], holes[:, 1:] * holes[:, :4])
    assert float(got) == pytest.approx(float(want), rel=1e-6)
    assert float(T.mtp_loss([], tokens, mask)) == 0.0 and float(T.mtp_loss([rnd(1, 1, v)], tokens[:, :1], mask[:, :1])) == 0.0
    capped = T.mtp_loss([10 * rnd(1, 5, v, seed=14)], tokens, mask, cap=30.0)
    manual = T.cross_entropy(T.soft_cap(10 * rnd(1, 5, v, seed=14)[:, :4], 30.0), tokens[:, 1:], mask[:, 1:])
    assert float(capped) == pytest.approx(float(manual), rel=1e-6)


def test_z_loss_and_total():
    probs = rnd(3, 5, 8, seed=15)
    lse = np.log(np.exp(probs).sum(-1))
    assert float(T.z_loss(probs)) == pytest.approx(float((lse ** 2).mean()), rel=1e-5)
    assert float(T.z_loss(np.zeros((0, 8)))) == 0.0
    c = T.tiny_train_config()
    assert float(T.total_loss(2.0, 0.5, 40.0, c)) == pytest.approx(2.0 + 0.5 + 1e-3 * 40.0)
    assert float(T.total_loss(2.0, 0.5, 40.0, dataclasses.replace(c, z_loss_weight=0.0))) == pytest.approx(2.5)
