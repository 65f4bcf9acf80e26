"""Behaviour list of the RL objective (``prometheus_b200.rl_loss``; reference tests/test_rl_loss.py
and rl/loss/__init__.py): configuration checks, Dr.GRPO advantages, dynamic sampling, sequence
ratios, clip-higher, truncated importance sampling, the overlong penalty, Gaussian latent
densities, routing-replay tables and the group loss, which is also compared with a scalar
restatement on generated groups."""
import dataclasses
import itertools
import math
import random

import pytest

from prometheus_b200 import rl_loss as R

BAD = (math.nan, math.inf, -math.inf)


def S(new, old, reward, version=5, lat=((), ()), n_tokens=None, routing=()):
    return R.Sample(tuple(new), tuple(old), tuple(lat[0]), tuple(lat[1]), reward,
                    n_tokens if n_tokens is not None else len(new), version, tuple(routing))


# ------------------------------------------------------------------------------ constants / config
def test_constants_and_frozen_records():
    assert (R.GROUP_SIZE, R.MAX_STALENESS, R.DEFAULT_CLIP_EPS_LOW, R.DEFAULT_CLIP_EPS_HIGH) == (16, 4, 0.2, 0.28)
    assert issubclass(R.LossError, ValueError)
    for obj in (R.RoutingTrace(0, 0, (1,)), S([-1.0], [-1.0], 0.0), R.Group("p", ()), R.LossConfig(),
                R.LossBreakdown(0.0, 0.0, 0.0, 0.0, 0, 0.0)):
        with pytest.raises(dataclasses.FrozenInstanceError):
            setattr(obj, dataclasses.fields(obj)[0].name, None)


def test_config_defaults_and_custom_values():
    c = R.make_config()
    assert c == R.LossConfig() and (c.clip_eps_low, c.clip_eps_high, c.latent_clip_eps_low, c.latent_clip_eps_high) == (0.2, 0.28, 0.2, 0.28)
    assert (c.loss_normalizer, c.overlong_cache, c.overlong_penalty, c.max_staleness, c.tis_clip, c.kl_coeff) == (1.0, 0, 0.0, 4, 1.0, 0.0)
    d = R.make_config(clip_eps_low=0.0, clip_eps_high=0.5, latent_clip_eps_low=0.1, latent_clip_eps_high=0.0, loss_normalizer=4096.0,
                      overlong_cache=128, overlong_penalty=0.01, max_staleness=2, tis_clip=2.0)
    assert (d.clip_eps_low, d.clip_eps_high, d.loss_normalizer, d.overlong_cache, d.max_staleness, d.tis_clip) == (0.0, 0.5, 4096.0, 128, 2, 2.0)
    for k in (1, 2, 3, 4):
        assert R.make_config(max_staleness=k).max_staleness == k


@pytest.mark.parametrize("kwargs", [
    dict(clip_eps_low=-0.1), dict(clip_eps_high=-0.1), dict(latent_clip_eps_low=-1e-9), dict(latent_clip_eps_high=-1.0),
    dict(loss_normalizer=0.0), dict(loss_normalizer=-1.0), dict(loss_normalizer=math.nan), dict(loss_normalizer=math.inf),
    dict(overlong_cache=-1), dict(overlong_penalty=-0.1), dict(max_staleness=0), dict(max_staleness=5), dict(max_staleness=-1),
    dict(tis_clip=0.99), dict(tis_clip=math.nan), dict(tis_clip=math.inf), dict(kl_coeff=0.1), dict(kl_coeff=-0.1),
])
def test_config_rejects(kwargs):
    with pytest.raises(R.LossError):
        R.make_config(**kwargs)


# ------------------------------------------------------------------------------ advantages
def test_mean_centering_has_no_division_by_the_deviation():
    assert R.mean_center((1.0, 3.0, 5.0)) == (-2.0, 0.0, 2.0)
    assert R.mean_center((10.0, 30.0, 50.0)) == (-20.0, 0.0, 20.0)                    # scales with the rewards
    assert R.mean_center((7.0,)) == (0.0,)
    rng = random.Random(0)
    for _ in range(20):
        r = tuple(rng.uniform(-5, 5) for _ in range(rng.randint(1, 16)))
        assert abs(math.fsum(R.mean_center(r))) < 1e-12
    with pytest.raises(R.LossError):
        R.mean_center(())
    for bad in BAD:
        with pytest.raises(R.LossError):
            R.mean_center((1.0, bad))


def test_all_equal_is_exact_equality():
    assert R.all_equal_reward((1.0, 1.0, 1.0)) and R.all_equal_reward((0.5,)) and not R.all_equal_reward((1.0, 1.0 + 1e-12))
    assert not R.all_equal_reward((0.0, 1.0))
    with pytest.raises(R.LossError):
        R.all_equal_reward(())


def test_dynamic_sampling_drops_groups_without_signal():
    same = R.Group("same", (S([-1], [-1], 1.0), S([-1], [-1], 1.0)))
    mixed = R.Group("mixed", (S([-1], [-1], 1.0), S([-1], [-1], 0.0)))
    single = R.Group("single", (S([-1], [-1], 3.0),))
    assert [g.prompt_id for g in R.drop_zero_advantage_groups((same, mixed, single, mixed))] == ["mixed", "mixed"]
    assert R.drop_zero_advantage_groups(()) == ()
    for groups in ((R.Group("empty", ()),), (mixed, R.Group("empty", ()), same)):
        with pytest.raises(R.LossError):
            R.drop_zero_advantage_groups(groups)


# ------------------------------------------------------------------------------ ratios / clipping
def test_sequence_ratio_is_the_exponential_of_the_summed_difference():
    assert R.sequence_ratio((-1.0, -2.0), (-1.0, -2.0)) == 1.0
    assert R.sequence_ratio((math.log(2.0),), (0.0,)) == pytest.approx(2.0)
    one, many = R.sequence_ratio((-1.0,), (-1.1,)), R.sequence_ratio((-1.0,) * 10, (-1.1,) * 10)
    assert many == pytest.approx(one ** 10)                                            # no length normalisation by default
    assert R.sequence_ratio((-1.0,) * 10, (-1.1,) * 10, length_normalize=True) == pytest.approx(one)
    for new, old in (((), ()), ((-1.0,), ()), ((-1.0, -2.0), (-1.0,))):
        with pytest.raises(R.LossError):
            R.sequence_ratio(new, old)
    for bad in BAD:
        for new, old in (((bad,), (-1.0,)), ((-1.0,), (bad,))):
            with pytest.raises(R.LossError):
                R.sequence_ratio(new, old)


def test_clip_higher_leaves_more_room_upward():
    assert R.clip_higher(2.0, 0.2, 0.28) == 1.28 and R.clip_higher(0.1, 0.2, 0.28) == 0.8
    assert R.clip_higher(1.1, 0.2, 0.28) == 1.1 and R.clip_higher(0.8, 0.2, 0.28) == 0.8 and R.clip_higher(1.28, 0.2, 0.28) == 1.28
    assert R.clip_higher(5.0, 0.0, 0.0) == 1.0
    for bad in BAD:
        with pytest.raises(R.LossError):
            R.clip_higher(bad, 0.2, 0.28)
    for lo, hi in ((-0.1, 0.2), (0.2, -0.1)):
        with pytest.raises(R.LossError):
            R.clip_higher(1.0, lo, hi)


def test_staleness():
    assert R.staleness(5, 5) == 0 and R.staleness(5, 1) == 4 and R.staleness(0, 0) == 0
    with pytest.raises(R.LossError):
        R.staleness(3, 4)


def test_truncated_importance_weights():
    assert R.truncated_is((-1.0,), (-3.0,), 0, 2.0) == 1.0                              # fresh: one, whatever the log-probs
    assert R.truncated_is((), (-1.0, -2.0), 0, 1.0) == 1.0                              # and nothing is even looked at
    assert R.truncated_is((-1.0,), (-3.0,), 2, 2.0) == 2.0                              # e^2 clipped at 2
    assert R.truncated_is((-1.0,), (-1.5,), 1, 2.0) == pytest.approx(math.exp(0.5))
    assert R.truncated_is((-2.0,), (-1.0,), 3, 2.0) == pytest.approx(math.exp(-1.0))    # below one is never raised
    assert R.truncated_is((-1.0,), (-3.0,), 1, 1.0) == 1.0 and R.truncated_is((-3.0,), (-1.0,), 1, 1.0) == pytest.approx(math.exp(-2.0))
    for k, clip in ((-1, 2.0), (1, 0.99)):
        with pytest.raises(R.LossError):
            R.truncated_is((-1.0,), (-1.0,), k, clip)


def test_overlong_penalty_is_linear_past_the_cache():
    assert R.overlong_soft_penalty(10, 10, 0.5) == 0.0 and R.overlong_soft_penalty(3, 10, 0.5) == 0.0
    assert R.overlong_soft_penalty(14, 10, 0.25) == 1.0 and R.overlong_soft_penalty(4, 0, 0.5) == 2.0
    for args in ((-1, 0, 0.1), (1, -1, 0.1), (1, 0, -0.1)):
        with pytest.raises(R.LossError):
            R.overlong_soft_penalty(*args)


# ------------------------------------------------------------------------------ latent densities
def test_gaussian_log_density():
    base = -0.5 * math.log(2 * math.pi)
    assert R.gaussian_log_density((0.0,), (0.0,), (1.0,)) == pytest.approx(base)
    assert R.gaussian_log_density((1.0, -2.0), (0.0, 0.5), (1.0, 2.0)) == pytest.approx(
        R.gaussian_log_density((1.0,), (0.0,), (1.0,)) + R.gaussian_log_density((-2.0,), (0.5,), (2.0,)))
    z, mu, sg, h = 0.7, 0.2, 1.3, 1e-6                                                  # d/dz log N = -(z - mu) / sigma^2
    num = (R.gaussian_log_density((z + h,), (mu,), (sg,)) - R.gaussian_log_density((z - h,), (mu,), (sg,))) / (2 * h)
    assert num == pytest.approx(-(z - mu) / sg ** 2, rel=1e-6)
    for args in (((), (), ()), ((1.0,), (1.0, 2.0), (1.0,)), ((1.0,), (1.0,), ())):
        with pytest.raises(R.LossError):
            R.gaussian_log_density(*args)
    for bad in BAD:
        for args in (((bad,), (0.0,), (1.0,)), ((0.0,), (bad,), (1.0,)), ((0.0,), (0.0,), (bad,))):
            with pytest.raises(R.LossError):
                R.gaussian_log_density(*args)
    for sigma in (0.0, -1.0):
        with pytest.raises(R.LossError):
            R.gaussian_log_density((0.0,), (0.0,), (sigma,))


def test_latent_ratio():
    assert R.latent_ratio((), ()) == 1.0
    assert R.latent_ratio((-0.5, -0.5), (-0.6, -0.7)) == R.sequence_ratio((-0.5, -0.5), (-0.6, -0.7))
    for new, old in (((-1.0,), ()), ((), (-1.0,)), ((-1.0,), (-1.0, -2.0)), ((math.nan,), (-1.0,))):
        with pytest.raises(R.LossError):
            R.latent_ratio(new, old)


# ------------------------------------------------------------------------------ routing replay
def test_routing_table():
    traces = [R.RoutingTrace(t, l, (t * 10 + l, 0)) for t in range(3) for l in range(2)]
    random.Random(1).shuffle(traces)
    table = R.routing_table(traces, 3, 2, 2)
    assert table == tuple(tuple((t * 10 + l, 0) for l in range(2)) for t in range(3))
    assert R.routing_table([R.RoutingTrace(0, 0, (7,))], 1, 1, 1) == (((7,),),)
    for dims in ((0, 1, 1), (1, 0, 1), (1, 1, 0), (-1, 1, 1)):
        with pytest.raises(R.LossError):
            R.routing_table([], *dims)
    ordered = sorted(traces, key=lambda t: (t.token_index, t.layer_index))
    for bad in (ordered + [ordered[0]], ordered[:-1], ordered[:-1] + [R.RoutingTrace(2, 1, (1,))],
                ordered[:-1] + [R.RoutingTrace(2, 1, (1, -1))], ordered[:-1] + [R.RoutingTrace(3, 1, (1, 1))]):
        with pytest.raises(R.LossError):
            R.routing_table(bad, 3, 2, 2)


# ------------------------------------------------------------------------------ the group loss
def m_loss(group, cfg, trainer_version):
    """Scalar restatement: sum over samples of tis * clip(ratio) * advantage for tokens and for
    latents (own clip), plus the overlong penalty, over the normaliser."""
    rewards = [s.reward for s in group.samples]
    if max(rewards) == min(rewards):
        return dict(pg=0.0, tis=0.0, overlong=0.0, latent=0.0, n_kept=0, total=0.0)
    mean = math.fsum(rewards) / len(rewards)
    pg = lat = ol = tis = 0.0
    for s in group.samples:
        adv = s.reward - mean
        k = trainer_version - s.policy_version
        d = math.fsum(a - b for a, b in zip(s.token_logp_trainer, s.token_logp_rollout))
        ratio = math.exp(d / len(s.token_logp_trainer) if cfg.length_normalize else d)
        w = 1.0 if k == 0 else min(math.exp(d), cfg.tis_clip)
        pg += w * min(max(ratio, 1 - cfg.clip_eps_low), 1 + cfg.clip_eps_high) * adv
        if s.latent_logp_trainer:
            lr = math.exp(math.fsum(a - b for a, b in zip(s.latent_logp_trainer, s.latent_logp_rollout)))
            lat += w * min(max(lr, 1 - cfg.latent_clip_eps_low), 1 + cfg.latent_clip_eps_high) * adv
        ol += cfg.overlong_penalty * max(0, s.n_tokens - cfg.overlong_cache)
        tis += w
    n = cfg.loss_normalizer
    return dict(pg=pg / n, tis=tis / len(group.samples), overlong=ol / n, latent=lat / n, n_kept=len(group.samples),
                total=(pg + lat + ol) / n)


def same(out, want):
    for k, v in want.items():
        assert getattr(out, k) == pytest.approx(v, rel=1e-5, abs=1e-6), k


def test_equal_rewards_give_zeros():
    g = R.Group("p", tuple(S([-1.0, -2.0], [-1.5, -2.5], 1.0) for _ in range(4)))
    assert R.gspo_dapo_loss(g, R.make_config(overlong_penalty=0.5), 5) == R.LossBreakdown(0.0, 0.0, 0.0, 0.0, 0, 0.0)


def test_on_policy_group_is_the_sum_of_advantages_and_has_no_kl_term():
    g = R.Group("p", (S([-1.0], [-1.0], 1.0), S([-2.0], [-2.0], 0.0), S([-3.0], [-3.0], 2.0)))
    out = R.gspo_dapo_loss(g, R.make_config(), 5)
    assert out.pg == pytest.approx(0.0, abs=1e-6) and out.tis == pytest.approx(1.0) and out.n_kept == 3 and out.total == pytest.approx(out.pg)
    far = R.Group("p", (S([-1.0], [-9.0], 1.0), S([-9.0], [-1.0], 0.0)))
    got = R.gspo_dapo_loss(far, R.make_config(), 5)                                     # far from the rollout policy: only clipping acts
    assert got.total == pytest.approx(1.28 * 0.5 + 0.8 * -0.5) and not hasattr(got, "kl")


def test_overlong_latent_normaliser_and_staleness_terms():
    cfg = R.make_config(loss_normalizer=4.0, overlong_cache=2, overlong_penalty=0.1, tis_clip=2.0, latent_clip_eps_low=0.05, latent_clip_eps_high=0.05)
    g = R.Group("p", (S([-1.0, -1.0, -1.0], [-1.2, -1.2, -1.2], 1.0, version=5, lat=((-0.5,), (-1.5,))),
                      S([-2.0, -2.0], [-1.0, -1.0], 0.0, version=3, lat=((-1.0,), (-0.9,))),
                      S([-1.0], [-3.0], 0.5, version=4)))
    out = R.gspo_dapo_loss(g, cfg, 5)
    same(out, m_loss(g, cfg, 5))
    assert out.overlong == pytest.approx(0.1 * 1 / 4.0)
    double = R.gspo_dapo_loss(g, dataclasses.replace(cfg, loss_normalizer=8.0), 5)
    assert double.total == pytest.approx(out.total / 2) and double.tis == pytest.approx(out.tis)
    clip_one = R.gspo_dapo_loss(g, dataclasses.replace(cfg, tis_clip=1.0), 5)           # every stale weight above one becomes one
    same(clip_one, m_loss(g, dataclasses.replace(cfg, tis_clip=1.0), 5))
    no_latent = R.Group("p", tuple(dataclasses.replace(s, latent_logp_trainer=(), latent_logp_rollout=()) for s in g.samples))
    assert R.gspo_dapo_loss(no_latent, cfg, 5).latent == 0.0


def test_routing_traces_do_not_change_the_loss_and_sixteen_samples_work():
    rng = random.Random(4)
    samples = tuple(S([rng.uniform(-3, -1) for _ in range(3)], [rng.uniform(-3, -1) for _ in range(3)], float(i % 3)) for i in range(R.GROUP_SIZE))
    plain = R.gspo_dapo_loss(R.Group("p", samples), R.make_config(), 5)
    routed = tuple(dataclasses.replace(s, routing=(R.RoutingTrace(0, 0, (1, 2)),)) for s in samples)
    assert R.gspo_dapo_loss(R.Group("p", routed), R.make_config(), 5) == plain and plain.n_kept == 16


def test_group_validation():
    ok = S([-1.0], [-1.0], 1.0)
    cfg = R.make_config()
    bad_groups = [R.Group("p", ()), R.Group("", (ok, S([-1.0], [-1.0], 0.0))), R.Group("p", (ok, S([], [], 0.0))),
                  R.Group("p", (ok, S([-1.0, -2.0], [-1.0], 0.0))), R.Group("p", (ok, S([-1.0], [-1.0], 0.0, lat=((-1.0,), ())))),
                  R.Group("p", (ok, S([-1.0], [-1.0], math.nan))), R.Group("p", (ok, S([-1.0], [-1.0], math.inf)))]
    for g in bad_groups:
        with pytest.raises(R.LossError):
            R.gspo_dapo_loss(g, cfg, 5)
    edge = R.Group("p", (ok, S([-1.0], [-1.0], 0.0, version=1)))
    R.gspo_dapo_loss(edge, cfg, 5)                                                      # staleness 4 == max is fine
    with pytest.raises(R.LossError):
        R.gspo_dapo_loss(R.Group("p", (ok, S([-1.0], [-1.0], 0.0, version=0))), cfg, 5)
    with pytest.raises(R.LossError):
        R.gspo_dapo_loss(R.Group("p", (ok, S([-1.0], [-1.0], 0.0, version=6))), cfg, 5)  # from the future


@pytest.mark.parametrize("seed", range(10))
def test_generated_groups_match_the_scalar_restatement(seed):
    rng = random.Random(seed)
    cfg = R.make_config(clip_eps_low=rng.choice([0.0, 0.1, 0.2]), clip_eps_high=rng.choice([0.1, 0.28, 0.5]),
                        latent_clip_eps_low=rng.choice([0.05, 0.2]), latent_clip_eps_high=rng.choice([0.05, 0.28]),
                        loss_normalizer=rng.choice([1.0, 3.0, 64.0]), overlong_cache=rng.randint(0, 4),
                        overlong_penalty=rng.choice([0.0, 0.05]), max_staleness=rng.randint(1, 4), tis_clip=rng.choice([1.0, 1.5, 3.0]),
                        length_normalize=rng.random() < 0.3)
    samples = []
    for _ in range(rng.randint(2, 8)):
        n = rng.randint(1, 6)
        old = [rng.uniform(-3.0, -0.1) for _ in range(n)]
        new = [o + rng.uniform(-0.4, 0.4) for o in old]
        nl = rng.choice([0, 0, 2])
        lo = [rng.uniform(-2.0, -0.1) for _ in range(nl)]
        ln = [o + rng.uniform(-0.3, 0.3) for o in lo]
        samples.append(S(new, old, rng.choice([0.0, 0.5, 1.0]), version=5 - rng.randint(0, cfg.max_staleness), lat=(ln, lo),
                         n_tokens=n + rng.randint(0, 3)))
    g = R.Group("p", tuple(samples))
    same(R.gspo_dapo_loss(g, cfg, 5), m_loss(g, cfg, 5))
