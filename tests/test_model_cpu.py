"""Model forward on CPU: config validation, layer pattern, truncated-recurrence gradient
cut, thought prepending, MoE equivalence with the per-token formulation."""
import pytest
import torch

from prometheus_b200 import model


def test_configs_validate_and_pattern():
    for fn in (model.tiny_config, model.flagship_config, *model.BASELINE_CONFIGS.values()):
        model.validate_config(fn())
    cfg = model.tiny_config()
    kinds = [model.attention_kind(i, cfg).value for i in range(8)]
    assert kinds == ["linear"] * 3 + ["mla"] + ["linear"] * 3 + ["mla"]
    assert model.ffn_kind(0, cfg) is model.FfnKind.DENSE and model.ffn_kind(1, cfg) is model.FfnKind.MOE
    d = model.config_dense_1p3b()
    assert model.attention_kind(3, d) is model.AttentionKind.GQA
    with pytest.raises(model.AttentionKindError):
        model.attention_kind(8, cfg)
    with pytest.raises(model.ConfigError):
        model.validate_config(model.with_overrides(cfg, n_dense=2))
    with pytest.raises(model.ConfigError):
        model.validate_config(model.with_overrides(cfg, top_k=9))


def test_param_counts():
    cfg = model.config_tiny_fp32()
    p = model.init_params(cfg, 0)
    flat = model.flatten_params(p)
    assert flat["layers.0.W_q"].shape == (256, 4, 64)
    assert "layers.3.W_beta" in flat
    assert model.param_count(p) == sum(t.numel() for t in flat.values())
    back = model.unflatten_params(flat)
    assert back["layers"][2]["router"].shape == (256, 8)


def test_forward_shapes_and_thoughts():
    cfg = model.tiny_config()
    p = model.init_params(cfg, 0)
    tok = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(0))
    out = model.forward(tok, p, cfg, r=2)
    assert out.logits.shape == (2, 12, 256) and len(out.mtp_logits) == 2
    assert out.router_probs.shape == (2, 12, 8) and out.expert_ids.shape == (2, 12, 2)
    th = torch.randn(2, 3, cfg.d_model, generator=torch.Generator().manual_seed(1))
    out2 = model.forward(tok, p, cfg, r=1, thoughts=th)
    assert out2.logits.shape == (2, 12, 256)
    with pytest.raises(model.ConfigError):
        model.forward(torch.full((1, 4), 999), p, cfg, r=1)


def test_truncated_recurrence_cuts_gradient():
    cfg = model.tiny_config()
    p = model.init_params(cfg, 0)
    tok = torch.randint(0, 256, (1, 8), generator=torch.Generator().manual_seed(0))

    def grad_of(trunc):
        leaves = {k: v.clone().requires_grad_(True) for k, v in model.flatten_params(p).items()}
        tree = model.unflatten_params(leaves)
        out = model.forward(tok, tree, cfg, r=3, truncated_recurrence=trunc)
        out.logits.square().mean().backward()
        return out.logits.detach(), leaves["layers.3.W_q"].grad.clone()

    full_logits, g_full = grad_of(4)
    cut_logits, g_cut = grad_of(1)
    torch.testing.assert_close(full_logits, cut_logits)      # forward value unchanged
    assert not torch.allclose(g_full, g_cut)                 # gradient differs through the cut


def test_moe_matches_per_token_formulation():
    torch.manual_seed(0)
    d, e, h, k, n = 16, 6, 8, 2, 10
    x = torch.randn(n, d)
    wr = torch.randn(d, e) * 0.3
    wg, wu, wd = torch.randn(e, d, h) * 0.2, torch.randn(e, d, h) * 0.2, torch.randn(e, h, d) * 0.2
    sg, su, sd = torch.randn(1, d, h) * 0.2, torch.randn(1, d, h) * 0.2, torch.randn(1, h, d) * 0.2
    out, probs, ids = model.moe(x, router_weight=wr, routed_weights=(wg, wu, wd),
                                shared_weights=(sg, su, sd), top_k=k, max_racks=8)
    pr = torch.sigmoid(x @ wr)
    top = torch.argsort(-pr, dim=-1, stable=True)[:, :k]
    assert (ids.long() == top).all()
    ref = torch.zeros(n, d)
    for t in range(n):
        sc = pr[t, top[t]]
        gates = sc / sc.sum()
        for j in range(k):
            ee = top[t, j]
            ref[t] += gates[j] * ((torch.nn.functional.silu(x[t] @ wg[ee]) * (x[t] @ wu[ee])) @ wd[ee])
        ref[t] += (torch.nn.functional.silu(x[t] @ sg[0]) * (x[t] @ su[0])) @ sd[0]
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)


def test_node_limited_topk_binds():
    scores = torch.tensor([[0.9, 0.1, 0.8, 0.2, 0.7, 0.3, 0.6, 0.4]])
    ids = model._node_limited_topk(scores, 3, 1)   # 8 experts -> racks of 1? max_racks=1
    racks = model._expert_to_rack(8, 1)
    assert len(set(racks[ids[0].long()].tolist())) == 1
    ids4 = model._node_limited_topk(scores, 3, 4)
    assert ids4[0].tolist() == [0, 2, 4]


def test_rope_properties():
    q = torch.randn(1, 6, 2, 8, generator=torch.Generator().manual_seed(0))
    pos = torch.arange(6)
    q1, k1 = model.rope(q, q, pos, partial=False)
    torch.testing.assert_close(q1.norm(dim=-1), q.norm(dim=-1))
    torch.testing.assert_close(q1[:, 0], q[:, 0])
    qp, _ = model.rope(q, q, pos, partial=True)
    torch.testing.assert_close(qp[..., 4:], q[..., 4:])
    a, b = model.rope_2d(q, q, pos, pos)
    assert a.shape == q.shape


def test_gqa_attention_matches_sdpa():
    q = torch.randn(2, 10, 4, 8, generator=torch.Generator().manual_seed(0))
    k = torch.randn(2, 10, 2, 8, generator=torch.Generator().manual_seed(1))
    v = torch.randn(2, 10, 2, 8, generator=torch.Generator().manual_seed(2))
    got = model.gqa_attention(q, k, v)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.repeat_interleave(2, 2).transpose(1, 2),
        v.repeat_interleave(2, 2).transpose(1, 2), is_causal=True).transpose(1, 2)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)


def test_forward_matches_the_independent_numpy_restatement():
    """model.forward against the float64 per-token / per-head / per-expert statement of the same
    definitions (reference: prometheus/verify/_torch_forward.py is the V1 oracle of its model)."""
    import numpy as np

    from prometheus_b200.verify.independent_forward import forward_logits

    cases = [model.tiny_config(),                                   # delta + MLA, dense + MoE, recurrence
             model.with_overrides(model.tiny_config(), softmax_kind="gqa", n_kv_heads=2)]
    for cfg in cases:
        params = model.init_params(cfg, 0)
        tok = torch.randint(0, cfg.vocab_size, (2, 20), generator=torch.Generator().manual_seed(3))
        for r in (1, 2):
            with torch.no_grad():
                got = model.forward(tok, params, cfg, r=r).logits.numpy()
            want = forward_logits(tok, params, cfg, r=r)
            assert np.abs(got - want).max() < 2e-5, (cfg.softmax_kind, r)
