"""Behaviour list of the latent-reasoning losses (``prometheus_b200.latent``; reference
tests/test_latent.py and model/latent.py): configuration checks in their order, the PonderNet
halting distribution with its pinned last slot, the geometric prior, halting loss and KL, the
masked trajectory CE, the four-term Stage-B loss, Jacobi sweeps with truncated backpropagation
and the noisy latent policy. Oracles are float64 NumPy restatements written here."""
import dataclasses
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import latent as L

EPS = 1e-6


def np_ponder(lam):
    lam = np.clip(np.asarray(lam, dtype=np.float64), EPS, 1 - EPS)
    lam[-1] = 1.0
    surv = np.concatenate([[1.0], np.cumprod(1 - lam[:-1])])
    return lam, lam * surv


def np_log_softmax(x):
    x = np.asarray(x, dtype=np.float64)
    m = x.max(-1, keepdims=True)
    return x - m - np.log(np.exp(x - m).sum(-1, keepdims=True))


def cfg(**kw):
    return dataclasses.replace(L.LatentConfig(), **kw)


# ------------------------------------------------------------------------------ constants / config
def test_constants_and_defaults():
    assert (L.CHUNK_MIN_THOUGHTS, L.CHUNK_MAX_THOUGHTS, L.COMPRESSION_TOKENS_PER_THOUGHT) == (4, 64, 8)
    assert (L.DEFAULT_JACOBI_SWEEPS, L.TRUNCATED_SWEEPS, L.TRUNCATED_RECURRENCE, L.DEFAULT_MAX_THOUGHTS) == (4, 2, 4, 16)
    assert (L.DEFAULT_ALPHA_TRAJ, L.DEFAULT_GAMMA_HALT, L.DEFAULT_BETA_KL, L.DEFAULT_LAMBDA_PRIOR) == (1.0, 1.0, 0.01, 0.2)
    assert (L.HALT_EPS, L.SIGMA_MIN, L.SIGMA_MAX) == (1e-6, 1e-4, 0.1)
    c = L.LatentConfig()
    assert (c.max_thoughts, c.chunk_min, c.chunk_max, c.jacobi_sweeps, c.truncated_sweeps) == (16, 4, 64, 4, 2)
    assert (c.alpha_traj, c.gamma_halt, c.beta_kl, c.lambda_prior, c.sigma_min, c.sigma_max) == (1.0, 1.0, 0.01, 0.2, 1e-4, 0.1)
    assert issubclass(L.LatentError, ValueError)
    with pytest.raises(dataclasses.FrozenInstanceError):
        c.max_thoughts = 1
    L.validate_latent_config(c)


@pytest.mark.parametrize("kw", [dict(max_thoughts=0), dict(alpha_traj=0.0, gamma_halt=0.0, beta_kl=0.0), dict(sigma_min=0.05, sigma_max=0.05),
                                dict(chunk_min=4, chunk_max=4), dict(chunk_min=64, chunk_max=64), dict(jacobi_sweeps=1, truncated_sweeps=1),
                                dict(jacobi_sweeps=8, truncated_sweeps=8), dict(lambda_prior=1e-9), dict(lambda_prior=1 - 1e-9)])
def test_valid_configurations(kw):
    L.validate_latent_config(cfg(**kw))


@pytest.mark.parametrize("kw, text", [
    (dict(max_thoughts=-1), "max_thoughts"), (dict(chunk_min=3), "chunk"), (dict(chunk_max=65), "chunk"), (dict(chunk_min=10, chunk_max=9), "chunk"),
    (dict(alpha_traj=-0.1), "alpha_traj"), (dict(alpha_traj=math.nan), "alpha_traj"), (dict(gamma_halt=-1.0), "gamma_halt"),
    (dict(gamma_halt=math.inf), "gamma_halt"), (dict(beta_kl=-1e-9), "beta_kl"), (dict(beta_kl=math.nan), "beta_kl"),
    (dict(lambda_prior=0.0), "lambda_prior"), (dict(lambda_prior=1.0), "lambda_prior"), (dict(lambda_prior=-0.2), "lambda_prior"),
    (dict(lambda_prior=math.nan), "lambda_prior"), (dict(jacobi_sweeps=0), "jacobi_sweeps"), (dict(truncated_sweeps=0), "truncated_sweeps"),
    (dict(truncated_sweeps=5), "truncated_sweeps"), (dict(sigma_min=0.0), "sigma"), (dict(sigma_min=-1.0), "sigma"),
    (dict(sigma_min=0.2, sigma_max=0.1), "sigma"), (dict(sigma_max=math.inf), "sigma"), (dict(sigma_min=math.nan), "sigma"),
])
def test_invalid_configurations_name_the_field(kw, text):
    with pytest.raises(L.LatentError, match=text):
        L.validate_latent_config(cfg(**kw))


def test_checks_run_in_a_fixed_order():
    with pytest.raises(L.LatentError, match="max_thoughts"):
        L.validate_latent_config(cfg(max_thoughts=-1, chunk_min=1, sigma_min=-1.0))
    with pytest.raises(L.LatentError, match="chunk"):
        L.validate_latent_config(cfg(chunk_min=1, alpha_traj=-1.0))
    with pytest.raises(L.LatentError, match="alpha_traj"):
        L.validate_latent_config(cfg(alpha_traj=-1.0, gamma_halt=-1.0, lambda_prior=2.0))
    with pytest.raises(L.LatentError, match="lambda_prior"):
        L.validate_latent_config(cfg(lambda_prior=2.0, jacobi_sweeps=0))
    with pytest.raises(L.LatentError, match="jacobi_sweeps"):
        L.validate_latent_config(cfg(jacobi_sweeps=0, sigma_min=-1.0))


# ------------------------------------------------------------------------------ halting
def test_ponder_distribution():
    p = L.ponder_distribution([0.5, 0.5, 0.1])
    np.testing.assert_allclose(p.numpy(), [0.5, 0.25, 0.25], rtol=1e-6)                # the last slot takes what is left
    rng = np.random.default_rng(0)
    for n in (1, 2, 5, 17):
        lam = rng.random(n)
        got = L.ponder_distribution(lam).double().numpy()
        np.testing.assert_allclose(got, np_ponder(lam)[1], rtol=1e-5, atol=1e-7)
        assert abs(got.sum() - 1.0) < 1e-5 and (got >= 0).all()
    assert L.ponder_distribution([0.3]).tolist() == [1.0]
    clipped = L.ponder_distribution([0.0, 1.0, 0.5]).double().numpy()                   # clipped to [eps, 1 - eps] before the pin
    np.testing.assert_allclose(clipped, np_ponder([0.0, 1.0, 0.5])[1], rtol=1e-4, atol=1e-9)
    assert clipped[0] > 0 and clipped[2] > 0
    for bad in ([], [[0.5, 0.5]], 0.5, [0.5, math.nan], [math.inf]):
        with pytest.raises(L.LatentError):
            L.ponder_distribution(bad)


def test_geometric_prior():
    g = L.geometric_prior(4, 0.2)
    raw = 0.2 * 0.8 ** np.arange(4)
    np.testing.assert_allclose(g, raw / raw.sum(), rtol=1e-12)
    assert g.dtype == np.float64 and abs(g.sum() - 1) < 1e-12 and np.all(np.diff(g) < 0)
    assert L.geometric_prior(1, 0.7).tolist() == [1.0]
    for n, lam in ((0, 0.2), (-1, 0.2), (3, 0.0), (3, 1.0), (3, -0.1), (3, math.nan)):
        with pytest.raises(L.LatentError):
            L.geometric_prior(n, lam)


def test_halt_from_logits():
    out = L.halt_from_logits([0.0, 0.0, -3.0])
    np.testing.assert_allclose(out.lambdas.numpy(), [0.5, 0.5, 1.0], rtol=1e-6)
    np.testing.assert_allclose(out.p.numpy(), [0.5, 0.25, 0.25], rtol=1e-6)
    assert float(out.expected_depth) == pytest.approx(0 * 0.5 + 1 * 0.25 + 2 * 0.25)
    x = np.array([2.0, -1.0, 0.3, 5.0, -80.0, 123.0])
    got = L.halt_from_logits(x)
    lam, p = np_ponder(1 / (1 + np.exp(-np.clip(x, -80, 80))))
    np.testing.assert_allclose(got.p.double().numpy(), p, rtol=1e-4, atol=1e-9)
    assert float(got.expected_depth) == pytest.approx(float((p * np.arange(6)).sum()), rel=1e-4)
    for bad in ([], [[0.0]], [math.nan], [0.0, math.inf]):
        with pytest.raises(L.LatentError):
            L.halt_from_logits(bad)


def test_halt_loss_and_kl():
    p = torch.tensor([0.5, 0.25, 0.25])
    assert float(L.halt_loss(p, 1)) == pytest.approx(-math.log(0.25 + EPS), rel=1e-6)
    assert float(L.halt_loss(p, -3)) == pytest.approx(-math.log(0.5 + EPS), rel=1e-6)   # clamped into range
    assert float(L.halt_loss(p, 99)) == pytest.approx(-math.log(0.25 + EPS), rel=1e-6)
    prior = L.geometric_prior(5, 0.3)
    assert abs(float(L.halt_kl(prior, 0.3))) < 1e-6
    away = np.array([0.9, 0.025, 0.025, 0.025, 0.025])
    want = float((away * (np.log(away + EPS) - np.log(prior + EPS))).sum())
    assert float(L.halt_kl(away, 0.3)) == pytest.approx(want, rel=1e-5) and want > 0
    for call in (lambda: L.halt_loss([], 0), lambda: L.halt_kl([], 0.2), lambda: L.halt_kl([0.5, 0.5], 0.0), lambda: L.halt_kl([0.5, math.nan], 0.2),
                 lambda: L.halt_loss([[0.5]], 0)):
        with pytest.raises(L.LatentError):
            call()


# ------------------------------------------------------------------------------ trajectory / answer CE
def test_thought_decode_ce():
    rng = np.random.default_rng(1)
    lg = rng.standard_normal((5, 7))
    ids = np.array([0, 6, 3, 3, 1])
    ce = -np_log_softmax(lg)[np.arange(5), ids]
    for mask in ([1, 1, 1, 1, 1], [1, 0, 1, 0, 0], [True, False, False, True, True], [0.0, 2.0, 0.0, 0.0, -1.0]):
        keep = np.asarray(mask) != 0
        assert float(L.thought_decode_ce(lg, ids, mask)) == pytest.approx(float(ce[keep].mean()), rel=1e-5)
    assert float(L.thought_decode_ce(lg, ids, [0] * 5)) == 0.0
    for bad in (lambda: L.thought_decode_ce(lg, [0, 1, 2, 3, 7], [1] * 5), lambda: L.thought_decode_ce(lg, [0, 1, 2, 3, -1], [1] * 5),
                lambda: L.thought_decode_ce(lg, ids[:4], [1] * 5), lambda: L.thought_decode_ce(lg, ids, [1] * 4),
                lambda: L.thought_decode_ce(lg[0], ids, [1] * 5), lambda: L.thought_decode_ce(np.zeros((0, 7)), [], []),
                lambda: L.thought_decode_ce(lg, ids[None], [1] * 5)):
        with pytest.raises(L.LatentError):
            bad()
    t = torch.tensor(lg, dtype=torch.float64, requires_grad=True)
    L.thought_decode_ce(t, ids, [1, 1, 0, 0, 1]).backward()
    soft = np.exp(np_log_softmax(lg))
    onehot = np.eye(7)[ids]
    want = (soft - onehot) * (np.array([1, 1, 0, 0, 1])[:, None] / 3.0)
    np.testing.assert_allclose(t.grad.numpy(), want, rtol=1e-6, atol=1e-9)


def test_answer_ce_at_depths():
    lg = np.random.default_rng(2).standard_normal((4, 6))
    got = L.answer_ce_at_depths(lg, 2).double().numpy()
    np.testing.assert_allclose(got, -np_log_softmax(lg)[:, 2], rtol=1e-5)
    for bad in (lambda: L.answer_ce_at_depths(lg, 6), lambda: L.answer_ce_at_depths(lg, -1), lambda: L.answer_ce_at_depths(lg[0], 0),
                lambda: L.answer_ce_at_depths(np.zeros((0, 6)), 0)):
        with pytest.raises(L.LatentError):
            bad()


def test_stage_b_loss_is_four_weighted_terms():
    rng = np.random.default_rng(3)
    k, v = 3, 6
    halt, ans, th = rng.standard_normal(k + 1), rng.standard_normal((k + 1, v)), rng.standard_normal((k, v))
    ids, mask = np.array([1, 5, 0]), np.array([1, 0, 1])
    c = cfg(alpha_traj=0.5, gamma_halt=2.0, beta_kl=0.1, lambda_prior=0.3)
    out = L.stage_b_loss(halt, ans, th, ids, mask, 4, 2, c)
    lam, p = np_ponder(1 / (1 + np.exp(-halt)))
    task = float((p * -np_log_softmax(ans)[:, 4]).sum())
    traj = float((-np_log_softmax(th)[np.arange(k), ids])[mask != 0].mean())
    hl = -math.log(p[2] + EPS)
    prior = L.geometric_prior(k + 1, 0.3)
    kl = float((p * (np.log(p + EPS) - np.log(prior + EPS))).sum())
    assert float(out.l_task) == pytest.approx(task, rel=1e-4) and float(out.l_traj) == pytest.approx(traj, rel=1e-4)
    assert float(out.l_halt) == pytest.approx(hl, rel=1e-4) and float(out.l_kl) == pytest.approx(kl, rel=1e-3, abs=1e-6)
    assert float(out.total) == pytest.approx(task + 0.5 * traj + 2.0 * hl + 0.1 * kl, rel=1e-4)
    assert float(out.expected_depth) == pytest.approx(float((p * np.arange(k + 1)).sum()), rel=1e-4)
    zero = L.stage_b_loss(halt, ans, th, ids, mask, 4, 2, cfg(alpha_traj=0.0, gamma_halt=0.0, beta_kl=0.0))
    assert float(zero.total) == pytest.approx(task, rel=1e-4)
    k0 = L.stage_b_loss([0.3], ans[:1], np.zeros((0, v)), [], [], 4, 0, c)               # no thoughts: no trajectory term
    assert float(k0.l_traj) == 0.0 and float(k0.l_task) == pytest.approx(float(-np_log_softmax(ans[:1])[0, 4]), rel=1e-5)


def test_stage_b_argument_errors():
    halt, ans, th = np.zeros(3), np.zeros((3, 4)), np.zeros((2, 4))
    with pytest.raises(L.LatentError, match="max_thoughts"):
        L.stage_b_loss(np.zeros((2, 2)), ans, th, [0, 0], [1, 1], 0, 0, cfg(max_thoughts=-1))     # the configuration is checked first
    for args in ((np.zeros((3, 1)), ans, th), (np.zeros(0), ans, th), (halt, ans[:2], th), (halt, ans, th[:1]), (halt, np.zeros(3), th)):
        with pytest.raises(L.LatentError):
            L.stage_b_loss(*args, [0, 0], [1, 1], 0, 0, cfg())
    with pytest.raises(L.LatentError):
        L.stage_b_loss(halt, ans, th, [0], [1, 1], 0, 0, cfg())
    with pytest.raises(L.LatentError):
        L.stage_b_loss(halt, ans, th, [0, 0], [1, 1], 9, 0, cfg())


# ------------------------------------------------------------------------------ Jacobi sweeps
def test_jacobi_sweeps_update_all_thoughts_together():
    x = torch.arange(6.0).reshape(3, 2)
    assert torch.equal(L.jacobi_sweeps(x, lambda t: t, 4, 2), x)
    target = torch.tensor([[1.0, -1.0]] * 3)
    out = L.jacobi_sweeps(x, lambda t: 0.5 * t + 0.5 * target, 12, 2)                   # a contraction converges to its fixed point
    assert (out - target).abs().max() < 2e-3
    shifted = L.jacobi_sweeps(x, lambda t: torch.roll(t, 1, 0), 1, 1)                   # every row sees the previous sweep's values
    assert torch.equal(shifted, torch.roll(x, 1, 0))
    a = L.jacobi_sweeps(x, lambda t: 0.9 * t + 1.0, 5, 1)
    b = L.jacobi_sweeps(x, lambda t: 0.9 * t + 1.0, 5, 5)
    assert torch.equal(a, b)                                                             # truncation changes gradients, not values
    for args in ((x[0], 2, 1), (torch.zeros(0, 2), 2, 1), (torch.zeros(2, 0), 2, 1), (x, 0, 1), (x, 2, 0), (x, 2, 3)):
        with pytest.raises(L.LatentError):
            L.jacobi_sweeps(args[0], lambda t: t, args[1], args[2])
    with pytest.raises(L.LatentError):
        L.jacobi_sweeps(x, lambda t: t[:2], 2, 1)


def test_gradient_flows_only_through_the_last_sweeps():
    w = torch.tensor(0.5, requires_grad=True)
    x = torch.ones(2, 2)
    for sweeps, trunc in ((4, 4), (4, 2), (4, 1), (3, 3)):
        (g,) = torch.autograd.grad(L.jacobi_sweeps(x, lambda t: w * t, sweeps, trunc).sum(), w)
        # value entering the window is w^(sweeps - trunc), held constant; inside it d/dw w^trunc
        assert float(g) == pytest.approx(4 * 0.5 ** (sweeps - trunc) * trunc * 0.5 ** (trunc - 1))


# ------------------------------------------------------------------------------ noisy latent policy
def test_clamp_sigma_and_noisy_latent():
    c = cfg()
    assert L.clamp_sigma([1e-6, 0.05, 3.0], c).tolist() == pytest.approx([1e-4, 0.05, 0.1])
    for bad in ([], [math.nan], [math.inf]):
        with pytest.raises(L.LatentError):
            L.clamp_sigma(bad, c)
    with pytest.raises(L.LatentError, match="sigma"):
        L.clamp_sigma([0.1], cfg(sigma_min=-1.0))
    mu, sg, ep = [0.5, -1.0, 2.0], [0.05, 5.0, 1e-9], [1.0, -2.0, 0.5]
    out = L.noisy_latent(mu, sg, ep, c)
    s = np.clip(sg, 1e-4, 0.1)
    z = np.array(mu) + s * np.array(ep)
    np.testing.assert_allclose(out.z.numpy(), z, rtol=1e-6)
    np.testing.assert_allclose(out.sigma.numpy(), s, rtol=1e-6)
    want = float((-0.5 * (np.array(ep) ** 2 + 2 * np.log(s) + math.log(2 * math.pi))).sum())
    assert float(out.log_density) == pytest.approx(want, rel=1e-5)
    assert float(L.gaussian_log_density(out.z, out.mu, out.sigma)) == pytest.approx(want, rel=1e-4)
    for args in (([], [], []), (mu, sg[:2], ep), (mu, sg, ep[:1]), ([math.nan, 0, 0], sg, ep), (mu, sg, [0, 0, math.inf])):
        with pytest.raises(L.LatentError):
            L.noisy_latent(*args, c)


def test_noisy_latent_density_gradient_in_z():
    mu, sg = torch.tensor([0.2, -0.4], dtype=torch.float64), torch.tensor([0.05, 0.08], dtype=torch.float64)
    z = torch.tensor([0.25, -0.5], dtype=torch.float64, requires_grad=True)
    L.gaussian_log_density(z, mu, sg).backward()
    np.testing.assert_allclose(z.grad.numpy(), (-(z.detach() - mu) / sg ** 2).numpy(), rtol=1e-10)


def test_random_vectors_follow_the_restatements():
    rng = np.random.default_rng(9)
    for _ in range(20):
        n = int(rng.integers(1, 9))
        x = rng.standard_normal(n) * 3
        got = L.halt_from_logits(x)
        lam, p = np_ponder(1 / (1 + np.exp(-x)))
        np.testing.assert_allclose(got.p.double().numpy(), p, rtol=2e-4, atol=1e-8)
        k = int(rng.integers(0, n))
        assert float(L.halt_loss(got.p, k)) == pytest.approx(-math.log(p[k] + EPS), rel=2e-4, abs=1e-6)
        prior = L.geometric_prior(n, 0.2)
        assert float(L.halt_kl(got.p, 0.2)) == pytest.approx(float((p * (np.log(p + EPS) - np.log(prior + EPS))).sum()), rel=2e-3, abs=2e-5)
