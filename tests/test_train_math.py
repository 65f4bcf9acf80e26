"""Optimizer / loss math against hand goldens (values from the reference's
tests/test_train.py:53-75 and tests/test_mup_muon.py:67-79) and an fp32 restatement."""
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import model, train

GOLDEN_NS_G = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])


def test_newton_schulz_golden():
    got = train.newton_schulz(GOLDEN_NS_G, steps=5)
    assert got[0, 0].item() == pytest.approx(-0.46751821, rel=1e-5, abs=1e-5)
    assert got[2, 1].item() == pytest.approx(0.24543214, rel=1e-5, abs=1e-5)
    assert got.sum().item() == pytest.approx(1.4456556, rel=1e-5, abs=1e-5)


def test_newton_schulz_scale_invariance_and_zero():
    g = torch.randn(6, 3, generator=torch.Generator().manual_seed(4))
    a = train.newton_schulz(g, 5)
    torch.testing.assert_close(train.newton_schulz(2.5 * g, 5), a, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(train.newton_schulz(-g, 5), -a, rtol=1e-5, atol=1e-5)
    assert train.newton_schulz(torch.zeros(3, 4), 5).abs().max().item() == 0.0
    with pytest.raises(ValueError):
        train.newton_schulz(g, 4)


def test_newton_schulz_batched_matches_loop():
    g = torch.randn(3, 5, 7, generator=torch.Generator().manual_seed(1))
    b = train.newton_schulz(g, 5)
    for i in range(3):
        torch.testing.assert_close(b[i], train.newton_schulz(g[i], 5), rtol=1e-5, atol=1e-6)


def test_muon_update_golden():
    g = torch.tensor([[0.5, -0.25], [0.1, 0.8], [-0.3, 0.4]])
    delta, m = train.muon_update(g, torch.zeros_like(g), lr=0.02, momentum_coeff=0.95, ns_steps=5)
    assert delta[0, 0].item() == pytest.approx(0.01596472, rel=1e-4, abs=1e-6)
    assert delta.sum().item() == pytest.approx(0.036446046, rel=1e-4, abs=1e-6)
    assert m.sum().item() == pytest.approx(1.25, rel=1e-6)


def test_muon_transfer_step_golden():
    p = torch.tensor([[0.5, -0.25], [0.1, 0.8], [-0.3, 0.4]])
    g = torch.tensor([[0.2, -0.1], [0.0, 0.3], [-0.4, 0.05]])
    m = torch.tensor([[0.1, 0.2], [-0.3, 0.0], [0.4, -0.2]])
    new_p, new_m = train.muon_transfer_step(p, g, m, lr=0.02, momentum_coeff=0.95, ns_steps=5,
                                            weight_decay=0.1)
    assert new_p[0, 0].item() == pytest.approx(0.4941366910934448, rel=1e-5)
    assert new_p.sum().item() == pytest.approx(1.2451510429382324, rel=1e-5)
    assert new_m[0, 0].item() == pytest.approx(0.29500001668930054, rel=1e-6)
    assert train.muon_rms_scale(3, 2) == pytest.approx(0.2 * math.sqrt(3))
    assert train.transferred_muon_lr(0.02, width=4096, base_width=256) == 0.02


def test_adamw_golden():
    p, m, v = train.adamw_update(torch.tensor([1.0]), torch.tensor([0.5]), torch.zeros(1),
                                 torch.zeros(1), lr=2e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                 wd=0.1, step=1)
    assert p.item() == pytest.approx(0.99978, rel=1e-6)
    assert m.item() == pytest.approx(0.05, rel=1e-6)
    assert v.item() == pytest.approx(0.0125, rel=1e-6)


def test_softcap_golden():
    got = train.soft_cap(torch.tensor([0.0, 30.0, 60.0, -15.0]), 30.0)
    np.testing.assert_allclose(got.numpy(), [0.0, 22.847826, 28.920828, -13.863516], rtol=1e-5)


def test_cross_entropy_masked_and_empty():
    logits = torch.randn(2, 5, 11, generator=torch.Generator().manual_seed(0))
    tgt = torch.randint(0, 11, (2, 5), generator=torch.Generator().manual_seed(1))
    mask = torch.ones(2, 5)
    ref = torch.nn.functional.cross_entropy(logits.reshape(-1, 11), tgt.reshape(-1))
    assert train.cross_entropy(logits, tgt, mask).item() == pytest.approx(ref.item(), rel=1e-5)
    assert train.cross_entropy(logits, tgt, torch.zeros(2, 5)).item() == 0.0


def test_wsd_schedule():
    cfg = train.tiny_train_config()
    assert train.wsd_lr(1, cfg) == pytest.approx(cfg.peak_lr * 0.5)
    assert train.wsd_lr(2, cfg) == pytest.approx(cfg.peak_lr)
    assert train.wsd_lr(10, cfg) == pytest.approx(cfg.peak_lr)
    assert train.wsd_lr(12, cfg) == pytest.approx(cfg.peak_lr * 0.5)
    assert train.wsd_lr(14, cfg) == 0.0
    with pytest.raises(ValueError):
        train.wsd_lr(0, cfg)


def test_qk_clip():
    q = torch.tensor([[1.0, 1.0]])
    k = torch.tensor([[1.5, 1.5]])
    qc, kc = train.qk_clip(q, k, 1.5)
    assert qc[0, 0].item() == pytest.approx(0.70710677, rel=1e-5)
    assert (qc @ kc.T).abs().max().item() == pytest.approx(1.5, rel=1e-5)


def test_classify_and_precision():
    assert train.classify_param("layers.0.W_q", torch.zeros(4, 2, 2)) is train.ParamKind.ADAMW
    assert train.classify_param("layers.0.ffn_up", torch.zeros(4, 2)) is train.ParamKind.MUON_2D
    assert train.classify_param("embed", torch.zeros(4, 2)) is train.ParamKind.ADAMW
    assert train.muon_matrix_view("layers.0.W_q", (64, 4, 16)) == (1, 64, 64)
    assert train.muon_matrix_view("layers.0.W_o", (4, 16, 64)) == (1, 64, 64)
    assert train.muon_matrix_view("layers.0.routed_up", (8, 64, 32)) == (8, 64, 32)
    assert train.muon_matrix_view("layers.0.W_beta", (64, 4)) is None
    cfg = train.tiny_train_config()
    assert train.precision_for("layers.7.ffn_up", cfg) is train.PrecisionKind.BF16_STABLE
    assert train.precision_for("layers.0.ffn_up", cfg) is train.PrecisionKind.FP8_LINEAR
    assert train.precision_for("layers.0.router", cfg) is train.PrecisionKind.BF16_STABLE


def test_train_step_reduces_loss_on_fixed_batch():
    cfg = model.tiny_config()
    tcfg = train.tiny_train_config()
    params = model.init_params(cfg, 0)
    opt = train.init_opt_state(params, tcfg, muon_all_matrices=True)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, cfg.vocab_size, (2, 32), generator=g)
    batch = train.Batch(tokens=tokens, loss_mask=torch.ones(2, 32), positions=torch.arange(32))
    losses = []
    for step in range(1, 7):
        out = train.train_step(params, opt, batch, cfg, tcfg, step=step, muon_transfer=True,
                               muon_weight_decay=0.0, muon_all_matrices=True)
        params, opt = out.params, out.opt_state
        losses.append(out.loss.total.item())
    assert losses[-1] < losses[0]
    assert math.isfinite(out.grad_norm.item())


def test_train_step_reference_flags():
    cfg = model.tiny_config()
    tcfg = train.tiny_train_config()
    params = model.init_params(cfg, 1)
    opt = train.init_opt_state(params, tcfg)
    tokens = torch.randint(0, cfg.vocab_size, (1, 16), generator=torch.Generator().manual_seed(2))
    batch = train.Batch(tokens=tokens, loss_mask=torch.ones(1, 16), positions=torch.arange(16))
    with pytest.raises(ValueError, match="muon_transfer"):
        train.train_step(params, opt, batch, cfg, tcfg, step=1, muon_transfer=1)
    with pytest.raises(ValueError, match="muon_weight_decay"):
        train.train_step(params, opt, batch, cfg, tcfg, step=1, muon_transfer=True,
                         muon_weight_decay=-1.0)
    out = train.train_step(params, opt, batch, cfg, tcfg, step=1)
    assert out.step == 1 and out.lr == pytest.approx(tcfg.peak_lr * 0.5)
    assert "momentum" in out.opt_state["layers"][0]["ffn_gate"]
    assert "m" in out.opt_state["layers"][0]["W_q"]


def test_router_bias_rules_probs_and_count():
    """The reference rule (mean router probability of the last MoE layer) and the assignment-count
    rule move ``router_bias`` by the same step size and can disagree in sign per expert."""
    import torch

    from prometheus_b200 import train as T

    params = {"layers": [{"router_bias": torch.zeros(4)}]}
    probs = torch.tensor([[[0.4, 0.3, 0.2, 0.1], [0.4, 0.3, 0.2, 0.1]]])       # expert 1 above the mean 0.25
    ids = torch.tensor([[[0, 2], [0, 3]]])                                   # ... but never assigned
    by_probs = T._update_router_bias(params, ids, 4, u=0.5, router_probs=probs, rule="probs")
    by_count = T._update_router_bias(params, ids, 4, u=0.5, router_probs=probs, rule="count")
    assert by_probs["layers"][0]["router_bias"].tolist() == [-0.5, -0.5, 0.5, 0.5]
    assert by_count["layers"][0]["router_bias"].tolist() == [-0.5, 0.5, 0.0, 0.0]
    assert params["layers"][0]["router_bias"].tolist() == [0.0] * 4              # input untouched
    import pytest
    with pytest.raises(ValueError):
        T._update_router_bias(params, ids, 4, rule="other")
