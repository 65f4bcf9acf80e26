"""Behaviour list of the depth recurrence and its truncated backpropagation
(``prometheus_b200.model.forward``; reference tests/test_model_recurrence_grad.py,
model/__init__.py:866-881,932-970): the forward value never depends on the gradient window, a
window shorter than the iteration count changes the gradient, a window at least as long as
the count is the full gradient, prepended thoughts, and argument checks. A scalar toy with the
same cut is differentiated by hand as the oracle."""
import pytest
import torch

from prometheus_b200 import model as M

CFG = M.tiny_config()
PARAMS = M.init_params(CFG, 0)
TOKENS = torch.randint(0, CFG.vocab_size, (1, 8), generator=torch.Generator().manual_seed(0))


def run(r, trunc, z=False):
    leaves = {k: v.clone().requires_grad_(True) for k, v in M.flatten_params(PARAMS).items()}
    out = M.forward(TOKENS, M.unflatten_params(leaves), CFG, r=r, truncated_recurrence=trunc)
    (out.z_loss if z else out.logits.square().mean()).backward()
    core = f"layers.{CFG.prelude_layers}."
    return out, {k: v.grad for k, v in leaves.items() if k.startswith(core) and v.grad is not None}


def test_default_window_and_argument_checks():
    assert M.TRUNCATED_RECURRENCE == 4
    for bad in (0, -1, True, 2.0, "2", None):
        with pytest.raises(M.ConfigError):
            M.forward(TOKENS, PARAMS, CFG, r=2, truncated_recurrence=bad)
    for bad_r in (0, -3):
        with pytest.raises(M.ConfigError):
            M.forward(TOKENS, PARAMS, CFG, r=bad_r)
    with pytest.raises(ValueError):
        M.forward(TOKENS[0], PARAMS, CFG, r=1)
    with pytest.raises(M.ConfigError):
        M.forward(torch.zeros(1, CFG.max_context + 1, dtype=torch.long), PARAMS, CFG, r=1)
    sampled = M.forward(TOKENS, PARAMS, CFG)
    assert 1 <= sampled.r_used <= CFG.recurrence_max and sampled.r_used == M.forward(TOKENS, PARAMS, CFG).r_used   # a function of the tokens


@pytest.mark.parametrize("r", [1, 2, 3, 5])
def test_forward_value_does_not_depend_on_the_window(r):
    with torch.no_grad():
        base = M.forward(TOKENS, PARAMS, CFG, r=r, truncated_recurrence=1)
        for trunc in (2, 4, 9):
            other = M.forward(TOKENS, PARAMS, CFG, r=r, truncated_recurrence=trunc)
            assert torch.equal(other.logits, base.logits) and torch.equal(other.z_loss, base.z_loss) and other.r_used == r
            assert all(torch.equal(a, b) for a, b in zip(other.mtp_logits, base.mtp_logits))


@pytest.mark.parametrize("r, short", [(2, 1), (3, 1), (3, 2), (5, 2)])
def test_a_short_window_changes_the_gradient_of_the_core_block(r, short):
    _, g_full = run(r, r)
    _, g_short = run(r, short)
    assert g_full.keys() == g_short.keys()
    assert any(not torch.allclose(g_full[k], g_short[k], rtol=1e-4, atol=1e-7) for k in g_full)
    _, z_full = run(r, r, z=True)
    _, z_short = run(r, short, z=True)
    moved = [k for k in z_full if not torch.allclose(z_full[k], z_short[k], rtol=1e-4, atol=1e-9)]
    assert moved                                                                         # the router z-loss is cut too


@pytest.mark.parametrize("r", [1, 2, 3])
def test_a_window_at_least_as_long_as_r_is_the_full_gradient(r):
    _, a = run(r, r)
    _, b = run(r, r + 3)
    assert all(torch.equal(a[k], b[k]) for k in a)


def test_the_injected_prelude_output_keeps_its_gradient():
    """Only the carry is detached at the cut: the prelude still gets gradient through the
    re-injection of its output inside the window."""
    leaves = {k: v.clone().requires_grad_(True) for k, v in M.flatten_params(PARAMS).items()}
    out = M.forward(TOKENS, M.unflatten_params(leaves), CFG, r=3, truncated_recurrence=1)
    out.logits.square().mean().backward()
    assert leaves["embed"].grad is not None and float(leaves["embed"].grad.abs().max()) > 0
    pre = [v.grad for k, v in leaves.items() if k.startswith("layers.0.") and v.grad is not None]
    assert pre and any(float(g.abs().max()) > 0 for g in pre)


def test_scalar_toy_with_the_same_cut_matches_its_hand_derivative():
    """h_0 = f(x); h_{t+1} = w * (h_t + x): with the carry detached before the last ``k``
    iterations, d h_r / d w is the derivative of the unrolled last k steps with the entering
    carry held constant."""
    def toy(w, x, r, trunc):
        h = w * x
        effective = min(trunc, r)
        cut = r - effective
        for i in range(r - 1):
            if cut > 0 and i == cut - 1:
                h = h.detach()
            h = w * (h + x)
        return h

    x = torch.tensor(0.7)
    for r, trunc in ((3, 1), (4, 2), (3, 3), (2, 5)):
        w = torch.tensor(0.9, requires_grad=True)
        (g,) = torch.autograd.grad(toy(w, x, r, trunc), w)
        effective = min(trunc, r)
        cut = r - effective
        wv, xv = 0.9, 0.7
        if cut == 0:
            h, dh = wv * xv, xv                                     # full unroll
            steps = r - 1
        else:
            h = wv * xv
            for _ in range(cut - 1):
                h = wv * (h + xv)
            dh, steps = 0.0, r - cut                                # constant entering the window
        for _ in range(steps):
            h, dh = wv * (h + xv), (h + xv) + wv * dh
        assert float(g) == pytest.approx(dh, rel=1e-5)


def test_thoughts_are_prepended_and_dropped_from_the_outputs():
    th = torch.randn(1, 3, CFG.d_model, generator=torch.Generator().manual_seed(2)) * 0.1
    with torch.no_grad():
        plain = M.forward(TOKENS, PARAMS, CFG, r=2)
        with_th = M.forward(TOKENS, PARAMS, CFG, r=2, thoughts=th)
        empty = M.forward(TOKENS, PARAMS, CFG, r=2, thoughts=torch.zeros(1, 0, CFG.d_model))
    assert with_th.logits.shape == plain.logits.shape and with_th.router_probs.shape == plain.router_probs.shape
    assert not torch.allclose(with_th.logits, plain.logits) and torch.equal(empty.logits, plain.logits)
    for bad in (torch.zeros(2, 3, CFG.d_model), torch.zeros(1, 3, CFG.d_model + 1), torch.zeros(3, CFG.d_model)):
        with pytest.raises(ValueError):
            M.forward(TOKENS, PARAMS, CFG, r=1, thoughts=bad)
