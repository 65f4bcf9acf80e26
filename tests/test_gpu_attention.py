"""tcgen05 causal GQA attention (forward, dQ, dK/dV) against the fp32 formula."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def _rand(b, s, hq, hkv, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(b, s, hq, 128, device="cuda", generator=g) * scale).to(BF16)
    k = (torch.randn(b, s, hkv, 128, device="cuda", generator=g) * scale).to(BF16)
    v = torch.randn(b, s, hkv, 128, device="cuda", generator=g).to(BF16)
    return q, k, v


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-20)).item()


@pytest.mark.parametrize("b,s,hq,hkv", [(1, 128, 1, 1), (2, 512, 4, 2), (1, 1024, 16, 4), (1, 320, 2, 1)])
def test_attention_forward_and_backward_match_fp32(b, s, hq, hkv):
    from prometheus_b200.ops import attention

    q, k, v = _rand(b, s, hq, hkv, 1)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    out, rowmax = attention.causal_gqa(q, k, v, return_max_logit=True)
    go = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), go)

    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention.causal_gqa_ref(qf, kf, vf)
    rq, rk, rv = torch.autograd.grad(ref, (qf, kf, vf), go.float())
    assert _rel(out, ref) < 1e-2
    assert _rel(dq, rq) < 2e-2 and _rel(dk, rk) < 2e-2 and _rel(dv, rv) < 2e-2

    kk = kf.detach().transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    logits = qf.detach().transpose(1, 2) @ kk.transpose(-1, -2) / math.sqrt(128)
    mask = torch.ones(s, s, dtype=torch.bool, device="cuda").tril()
    want_max = logits.masked_fill(~mask, float("-inf")).amax(-1)
    torch.testing.assert_close(rowmax, want_max, atol=2e-3, rtol=1e-3)


def test_attention_large_logits_exercise_the_rescale_path():
    """Scores that keep growing along the keys force the running maximum to be raised
    repeatedly (more than 2^8 between blocks), so the tensor-memory rescale of O runs."""
    from prometheus_b200.ops import attention

    b, s, hq, hkv = 1, 768, 2, 2
    q, k, v = _rand(b, s, hq, hkv, 3)
    ramp = torch.linspace(0.0, 6.0, s, device="cuda").view(1, s, 1, 1)
    k = (k.float() + ramp * q.float().mean(dim=(1,), keepdim=True).sign()).to(BF16)
    q = (q.float() * 3.0).to(BF16)
    out = attention.causal_gqa(q, k, v)
    ref = attention.causal_gqa_ref(q.float(), k.float(), v.float())
    assert torch.isfinite(out.float()).all()
    assert _rel(out, ref) < 1.5e-2


def test_attention_is_deterministic_and_matches_library_kernel():
    import torch.nn.functional as F

    from prometheus_b200.ops import attention

    q, k, v = _rand(2, 1024, 8, 2, 5)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    go = torch.randn(2, 1024, 8, 128, device="cuda").to(BF16)
    runs = []
    for _ in range(2):
        o = attention.causal_gqa(q, k, v)
        runs.append((o,) + torch.autograd.grad(o, (q, k, v), go))
    for a, b_ in zip(*runs):
        assert torch.equal(a, b_)
    o2 = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                        is_causal=True, enable_gqa=True).transpose(1, 2)
    g2 = torch.autograd.grad(o2, (q, k, v), go)
    assert _rel(runs[0][0], o2) < 1e-2
    for mine, lib in zip(runs[0][1:], g2):
        assert _rel(mine, lib) < 2e-2


@pytest.mark.parametrize("q_off,s_loc,s_kv", [(512, 256, 1024), (0, 512, 640), (768, 256, 1024)])
def test_offset_attention_equals_a_slice_of_the_full_sequence(q_off, s_loc, s_kv):
    """A query slice at a global offset against the whole prefix (the context-parallel case):
    output and dq of the slice, and dk / dv of every key row (zero where nothing sees it)."""
    from prometheus_b200.ops import attention

    q, k, v = _rand(2, 1024, 4, 2, 11)
    k, v = k[:, :s_kv].contiguous(), v[:, :s_kv].contiguous()
    ql = q[:, q_off:q_off + s_loc].contiguous().requires_grad_()
    kl, vl = k.clone().requires_grad_(), v.clone().requires_grad_()
    out = attention.causal_gqa_offset(ql, kl, vl, q_off)
    go = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), go)

    s_all = max(s_kv, q_off + s_loc)
    qf = torch.zeros(2, s_all, 4, 128, device="cuda")
    qf[:, q_off:q_off + s_loc] = q[:, q_off:q_off + s_loc].float()
    qf.requires_grad_()
    kf = torch.zeros(2, s_all, 2, 128, device="cuda"); kf[:, :s_kv] = k.float(); kf.requires_grad_()
    vf = torch.zeros(2, s_all, 2, 128, device="cuda"); vf[:, :s_kv] = v.float(); vf.requires_grad_()
    ref = attention.causal_gqa_ref(qf, kf, vf)
    gof = torch.zeros_like(ref)
    gof[:, q_off:q_off + s_loc] = go.float()
    rq, rk, rv = torch.autograd.grad(ref, (qf, kf, vf), gof)
    assert _rel(out, ref[:, q_off:q_off + s_loc]) < 1e-2
    assert _rel(dq, rq[:, q_off:q_off + s_loc]) < 2e-2
    assert _rel(dk, rk[:, :s_kv]) < 2e-2 and _rel(dv, rv[:, :s_kv]) < 2e-2
    unseen = q_off + s_loc
    if unseen < s_kv:
        assert dk[:, unseen:].abs().max() == 0 and dv[:, unseen:].abs().max() == 0
    with pytest.raises(ValueError):
        attention.causal_gqa_offset(ql, kl, vl, q_off + 128)
