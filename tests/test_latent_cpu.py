"""Latent reasoning on CPU: halting distribution, Stage-B loss terms, truncated Jacobi
gradient, noisy policy density, layout planner, segment decoder, latent-slot solve."""
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import latent as L


def test_ponder_distribution_and_prior():
    p = L.ponder_distribution([0.5, 0.5, 0.2])
    np.testing.assert_allclose(p.numpy(), [0.5, 0.25, 0.25], rtol=1e-6)
    assert p.sum().item() == pytest.approx(1.0)
    g = L.geometric_prior(3, 0.5)
    np.testing.assert_allclose(g, np.array([0.5, 0.25, 0.125]) / 0.875)
    h = L.halt_from_logits(torch.zeros(3))
    assert h.expected_depth.item() == pytest.approx(0.25 + 2 * 0.25)
    assert h.lambdas[-1].item() == 1.0
    assert L.halt_loss(p, 99).item() == pytest.approx(-math.log(0.25 + 1e-6))
    assert L.halt_kl(torch.as_tensor(g, dtype=torch.float32), 0.5).item() == pytest.approx(0.0, abs=1e-5)
    with pytest.raises(L.LatentError):
        L.geometric_prior(0, 0.5)
    with pytest.raises(L.LatentError):
        L.ponder_distribution([])


def test_stage_b_loss_composition():
    torch.manual_seed(0)
    k, vocab = 3, 7
    halt = torch.randn(k + 1)
    ans = torch.randn(k + 1, vocab)
    th = torch.randn(k, vocab)
    ids = torch.tensor([1, 2, 3])
    mask = torch.tensor([1.0, 0.0, 1.0])
    cfg = L.LatentConfig()
    out = L.stage_b_loss(halt, ans, th, ids, mask, 4, 2, cfg)
    p = L.halt_from_logits(halt).p
    task = (p * -torch.log_softmax(ans, -1)[:, 4]).sum()
    ce = -torch.log_softmax(th, -1)[[0, 2], [1, 3]].mean()
    assert out.l_task.item() == pytest.approx(task.item(), rel=1e-6)
    assert out.l_traj.item() == pytest.approx(ce.item(), rel=1e-6)
    total = task + cfg.alpha_traj * ce + cfg.gamma_halt * L.halt_loss(p, 2) + cfg.beta_kl * L.halt_kl(p, 0.2)
    assert out.total.item() == pytest.approx(total.item(), rel=1e-6)
    obj = L.stage_b_objective(halt, ans, th, ids, mask, 4, 2, cfg, torch.ones(2, 3), torch.zeros(2, 3),
                              align_weight=0.5)
    assert obj.total.item() == pytest.approx(out.total.item() + 0.5, rel=1e-6)
    k0 = L.stage_b_loss(torch.zeros(1), torch.randn(1, vocab), None, None, None, 0, 0, cfg)
    assert k0.l_traj.item() == 0.0
    with pytest.raises(L.LatentError):
        L.stage_b_loss(halt, ans[:2], th, ids, mask, 4, 2, cfg)
    with pytest.raises(L.LatentError):
        L.validate_latent_config(L.LatentConfig(truncated_sweeps=9))


def test_jacobi_truncation_blocks_gradient():
    w = torch.tensor([[0.5, 0.1], [0.0, 0.3]], requires_grad=True)
    x0 = torch.ones(3, 2, requires_grad=True)

    def run(trunc):
        out = L.jacobi_sweeps(x0, lambda t: torch.tanh(t @ w), 4, trunc)
        return torch.autograd.grad(out.sum(), [x0, w], allow_unused=True)

    gx_full, gw_full = run(4)
    gx_cut, gw_cut = run(2)
    assert gx_full.abs().sum() > 0 and gx_cut is None       # cut: no gradient reaches the input
    assert not torch.allclose(gw_full, gw_cut)
    a = L.jacobi_sweeps(x0, lambda t: torch.tanh(t @ w), 4, 4)
    b = L.jacobi_sweeps(x0, lambda t: torch.tanh(t @ w), 4, 1)
    torch.testing.assert_close(a, b)                          # value does not depend on the cut
    with pytest.raises(L.LatentError):
        L.jacobi_sweeps(x0, lambda t: t[:, :1], 2, 1)


def test_noisy_latent_density():
    cfg = L.LatentConfig()
    out = L.noisy_latent([0.0, 1.0], [5.0, 1e-9], [1.0, -1.0], cfg)
    np.testing.assert_allclose(out.sigma.numpy(), [0.1, 1e-4], rtol=1e-6)
    np.testing.assert_allclose(out.z.numpy(), [0.1, 1.0 - 1e-4], rtol=1e-6)
    ref = sum(-0.5 * (e * e + 2 * math.log(s) + math.log(2 * math.pi)) for e, s in ((1.0, 0.1), (-1.0, 1e-4)))
    assert out.log_density.item() == pytest.approx(ref, rel=1e-4)


def test_think_layout_and_tools():
    cfg = L.LatentConfig()
    lay = L.plan_think_layout([4, 8, 4], [7], cfg)
    assert [s.kind.value for s in lay] == ["latent", "anchor", "latent", "anchor", "latent"]
    lay2 = L.insert_discrete_tool(lay, 0, [11, 12])
    assert [s.kind.value for s in lay2] == ["latent", "anchor", "tool", "latent", "anchor", "latent"]
    lay3 = L.insert_discrete_tool(lay2, 2, [5])
    assert lay3[-1].kind is L.SpanKind.TOOL
    with pytest.raises(L.LatentError):
        L.plan_think_layout([2], [7], cfg)
    with pytest.raises(L.LatentError):
        L.insert_discrete_tool(lay, 3, [1])


def test_segment_decoder_and_tied_head():
    d, vocab = 4, 6
    torch.manual_seed(0)
    h, u = torch.randn(d), torch.randn(vocab, d)
    one = L.decode_thought_segment(h, 1, u)
    torch.testing.assert_close(one, h @ u.T)
    dec = L.SegmentDecoder(torch.randn(d, d) * 0.3, torch.randn(d, d) * 0.3, torch.zeros(d))
    many = L.decode_thought_segment(h, 3, u, dec, final_norm=torch.ones(d))
    assert many.shape == (3, vocab)
    s1 = torch.tanh(h @ dec.w_in)
    n1 = s1 * torch.rsqrt((s1 * s1).mean() + 1e-6)
    torch.testing.assert_close(many[0], n1 @ u.T)
    with pytest.raises(L.LatentError):
        L.decode_thought_segment(h, 2, u)


def test_latent_slot_jacobi_matches_sequential_feedback():
    """With K + 1 sweeps the Jacobi solve equals feeding hidden states back one by one."""
    torch.manual_seed(0)
    b, s, d, k, start = 2, 9, 5, 3, 4
    embeds = torch.randn(b, s, d)
    wa, wb = torch.randn(d, d) * 0.4, torch.randn(d, d) * 0.4

    def fwd(e):     # a causal toy model: cumulative mean then a nonlinearity
        c = torch.cumsum(e, 1) / torch.arange(1, s + 1)[None, :, None]
        return torch.tanh(c @ wa)

    adapter = lambda x: x @ wb  # noqa: E731
    seq = embeds.clone()
    for j in range(k):
        hid = fwd(seq)
        seq[:, start + j] = adapter(hid[:, start + j - 1])
    want = fwd(seq)
    got, _ = L.latent_slot_forward(embeds, fwd, adapter, start, k, n_sweeps=k + 1)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    approx, _ = L.latent_slot_forward(embeds, fwd, adapter, start, k, n_sweeps=2)
    assert not torch.allclose(approx, want)
    e2 = embeds.clone().requires_grad_(True)
    hid, _ = L.latent_slot_forward(e2, fwd, adapter, start, k, n_sweeps=4, truncated_sweeps=4)
    hid.sum().backward()
    assert e2.grad.abs().sum() > 0
