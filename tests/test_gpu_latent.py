"""Latent Jacobi step kernels and latent-slot training in the engine (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def test_jacobi_step_matches_fp32_forward_and_backward():
    from prometheus_b200.ops import latent as LK

    B, S, d, ah, start, k = 3, 40, 256, 384, 9, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    r = lambda *s, sc=1.0: (torch.randn(*s, device="cuda", generator=g) * sc)
    hidden, embeds = r(B, S, d).to(BF16), r(B, S, d).to(BF16)
    w1, w2 = r(ah, d, sc=0.06).to(BF16), r(d, ah, sc=0.06).to(BF16)
    nw = (1.0 + 0.1 * r(d)).float()
    go = r(B, S, d).to(BF16)
    leaves = [t.clone().requires_grad_(True) for t in (hidden, embeds, w1, w2, nw)]
    out = LK.jacobi_step(*leaves, start, k)
    out.backward(go)
    ref_leaves = [t.detach().float().requires_grad_(True) for t in (hidden, embeds, w1, w2, nw)]
    ref = LK.jacobi_step_ref(*ref_leaves, start, k)
    ref.backward(go.float())
    assert torch.equal(out[:, :start], embeds[:, :start]) and torch.equal(out[:, start + k:], embeds[:, start + k:])
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()
    assert rel(out, ref) < 1e-2
    for name, a, b in zip(("hidden", "embeds", "w1", "w2", "norm"), leaves, ref_leaves):
        assert rel(a.grad, b.grad) < 3e-2, name
    assert leaves[0].grad[:, start + k - 1:].abs().max() == 0          # only the k source rows get gradient
    assert leaves[1].grad[:, start:start + k].abs().max() == 0         # slot embeddings are overwritten
    with pytest.raises(ValueError):
        LK.jacobi_step(hidden, embeds, w1, w2, nw, 0, k)
    with pytest.raises(ValueError):
        LK.jacobi_step(hidden, embeds, w1, w2, nw, S - 3, k)


def test_engine_latent_slots_match_generic_solver_and_train():
    from test_gpu_engine import small_hybrid

    from prometheus_b200 import engine, latent, model, train
    from prometheus_b200.ops import functional as ops

    cfg = small_hybrid()
    tcfg = train.train_config_for(cfg, warmup_steps=2, stable_steps=100, decay_steps=10)
    tr = engine.Trainer(cfg, tcfg, seed=3, micro_batch=2)
    tokens = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda",
                           generator=torch.Generator(device="cuda").manual_seed(1))
    start, k, sweeps = 40, 8, 3
    tr.set_latent_slots(start, k, sweeps)
    B, S, d = 2, 128, cfg.d_model
    with torch.no_grad():
        got = tr.forward_hidden_latent(tokens).reshape(B, S, d)
        embeds = tr.p["embed"][tokens.reshape(-1).long()].reshape(B, S, d)

        def adapter(x):
            a = torch.nn.functional.silu(x.float() @ tr.p["adapter_w1"].float().t()) @ tr.p["adapter_w2"].float().t()
            return model.rms_norm(a, tr.p["adapter_norm"].float())

        want, _ = latent.latent_slot_forward(
            embeds, lambda e: tr.forward_hidden(tokens, inputs_embeds=e.to(BF16)).reshape(B, S, d), adapter,
            start, k, n_sweeps=sweeps)
    rel = ((got.float() - want.float()).norm() / want.float().norm()).item()
    assert rel < 3e-2, rel
    plain = tr.forward_hidden(tokens).reshape(B, S, d)
    assert (got[:, :start].float() - plain[:, :start].float()).abs().max() < 1e-2     # causal: the prefix is untouched
    assert (got[:, start + k:].float() - plain[:, start + k:].float()).abs().max() > 1e-2

    mask = torch.ones(2, 128, device="cuda")
    mask[:, start:start + k] = 0
    tr.set_latent_slots(start, k, sweeps, truncated_sweeps=2)
    w1_before = tr.p["adapter_w1"].clone()
    losses = [tr.step(tokens, loss_mask=mask)["loss"].item() for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses
    assert not torch.equal(w1_before, tr.p["adapter_w1"])               # the adapter is being trained
    ops.check_status("cuda")
    tr.set_latent_slots(0, 0)
    assert tr.latent_slots is None
