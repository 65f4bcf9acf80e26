"""GSPO/DAPO objective pieces against hand computations."""
import math

import pytest
import torch

from prometheus_b200 import rl_loss as R


def _sample(new, old, reward, version=5, lat=((), ()), n_tokens=None):
    return R.Sample(tuple(new), tuple(old), tuple(lat[0]), tuple(lat[1]), reward,
                    n_tokens if n_tokens is not None else len(new), version)


def test_pieces():
    assert R.mean_center((1.0, 2.0, 3.0)) == (-1.0, 0.0, 1.0)
    assert R.sequence_ratio((-1.0, -2.0), (-1.5, -2.5)) == pytest.approx(math.e)
    assert R.sequence_ratio((-1.0, -2.0), (-1.5, -2.5), length_normalize=True) == pytest.approx(math.exp(0.5))
    assert R.clip_higher(2.0, 0.2, 0.28) == 1.28 and R.clip_higher(0.1, 0.2, 0.28) == 0.8
    assert R.truncated_is((-1.0,), (-3.0,), 0, 2.0) == 1.0
    assert R.truncated_is((-1.0,), (-3.0,), 2, 2.0) == 2.0
    assert R.overlong_soft_penalty(12, 10, 0.5) == 1.0 and R.overlong_soft_penalty(5, 10, 0.5) == 0.0
    assert R.latent_ratio((), ()) == 1.0
    assert R.gaussian_log_density((0.0,), (0.0,), (1.0,)) == pytest.approx(-0.5 * math.log(2 * math.pi))
    with pytest.raises(R.LossError):
        R.staleness(3, 4)
    with pytest.raises(R.LossError):
        R.make_config(kl_coeff=0.1)
    with pytest.raises(R.LossError):
        R.latent_ratio((1.0,), ())
    groups = (R.Group("a", (_sample([-1], [-1], 1.0), _sample([-1], [-1], 1.0))),
              R.Group("b", (_sample([-1], [-1], 1.0), _sample([-1], [-1], 0.0))))
    assert [g.prompt_id for g in R.drop_zero_advantage_groups(groups)] == ["b"]


def test_routing_table():
    tr = [R.RoutingTrace(t, l, (t, l)) for t in range(2) for l in range(2)]
    assert R.routing_table(tr, 2, 2, 2)[1][0] == (1, 0)
    with pytest.raises(R.LossError):
        R.routing_table(tr[:3], 2, 2, 2)
    with pytest.raises(R.LossError):
        R.routing_table(tr + [tr[0]], 2, 2, 2)


def test_group_loss_hand_value():
    cfg = R.make_config(loss_normalizer=2.0, overlong_cache=1, overlong_penalty=0.1, tis_clip=1.5)
    g = R.Group("p", (
        _sample([-1.0, -1.0], [-1.2, -1.2], 1.0, version=5, lat=((-0.5,), (-0.6,))),
        _sample([-2.0, -2.0], [-1.0, -1.0], 0.0, version=3),
    ))
    out = R.gspo_dapo_loss(g, cfg, trainer_version=5)
    r0, r1 = math.exp(0.4), math.exp(-2.0)
    c0, c1 = min(r0, 1.28), max(r1, 0.8)
    w0, w1 = 1.0, min(r1, 1.5)
    pg = (c0 * 0.5 * w0 + c1 * -0.5 * w1)
    lat = min(math.exp(0.1), 1.28) * 0.5 * w0
    ol = 0.1 + 0.1
    assert out.pg == pytest.approx(pg / 2) and out.latent == pytest.approx(lat / 2)
    assert out.overlong == pytest.approx(ol / 2) and out.tis == pytest.approx((w0 + w1) / 2)
    assert out.total == pytest.approx((pg + lat + ol) / 2) and out.n_kept == 2
    same = R.Group("q", (_sample([-1], [-1], 1.0), _sample([-1], [-1], 1.0)))
    assert R.gspo_dapo_loss(same, cfg, 5).total == 0.0
    with pytest.raises(R.LossError):
        R.gspo_dapo_loss(g, cfg, trainer_version=9)


def test_tensor_logps_are_differentiable_and_pessimistic_min():
    new = torch.tensor([-1.0, -1.0], requires_grad=True)
    g = R.Group("p", (R.Sample(new, torch.tensor([-1.05, -1.05]), (), (), 1.0, 2, 1),
                      _sample([-1.0], [-1.0], 0.0, version=1)))
    out = R.gspo_dapo_loss(g, R.make_config(), 1)
    out.total.backward()
    assert new.grad.abs().sum() > 0
    big = torch.tensor([-0.1, -0.1])
    g2 = R.Group("p", (R.Sample(big, torch.tensor([-2.0, -2.0]), (), (), 0.0, 2, 1),
                       _sample([-1.0], [-1.0], 1.0, version=1)))
    plain = R.gspo_dapo_loss(g2, R.make_config(), 1).pg
    pess = R.gspo_dapo_loss(g2, R.make_config(pessimistic=True), 1).pg
    assert float(pess) < float(plain)      # negative advantage with a huge ratio is not clipped away


def test_batched_loss_equals_the_sum_of_group_losses_and_drops_flat_groups():
    """Many groups in one packed batch: per-group totals equal the one-group calls, a group with
    equal rewards contributes exactly nothing, and the gradient flows to the trainer log-probs
    of the kept samples only."""
    g = torch.Generator().manual_seed(0)
    cfg = R.make_config(loss_normalizer=3.0, overlong_cache=3, overlong_penalty=0.05, tis_clip=2.0)
    groups, leaves = [], []
    for gi in range(5):
        samples = []
        for si in range(4):
            n = int(torch.randint(2, 7, (1,), generator=g))
            new = (-torch.rand(n, generator=g)).requires_grad_(True)
            old = new.detach() + 0.1 * torch.randn(n, generator=g)
            lat_n = (-torch.rand(2, generator=g)).requires_grad_(True) if si % 2 else ()
            lat_o = (lat_n.detach() + 0.05) if si % 2 else ()
            reward = 1.0 if gi == 3 else float(torch.rand((), generator=g))      # group 3: all equal
            samples.append(R.Sample(new, old, lat_n, lat_o, reward, n, 7 - (si % 3)))
            leaves.append((gi, new))
        groups.append(R.Group(f"p{gi}", tuple(samples)))
    packed = R.pack_groups(groups, 7, cfg)
    out = R.batched_loss(packed, cfg)
    singles = [R.gspo_dapo_loss(grp, cfg, 7) for grp in groups]
    for gi, s in enumerate(singles):
        assert float(out["per_group"][gi]) == pytest.approx(float(s.total), rel=1e-5, abs=1e-7)
    assert float(out["per_group"][3]) == 0.0 and int(out["n_kept"]) == 16
    assert float(out["total"]) == pytest.approx(sum(float(s.total) for s in singles), rel=1e-5)
    out["total"].backward()
    for gi, leaf in leaves:
        if gi == 3:
            assert leaf.grad is None or float(leaf.grad.abs().sum()) == 0.0
    assert any(float(leaf.grad.abs().sum()) > 0 for gi, leaf in leaves if gi != 3)
    with pytest.raises(R.LossError):
        R.pack_groups([], 7, cfg)
    with pytest.raises(R.LossError):
        R.pack_groups([R.Group("", groups[0].samples)], 7, cfg)
