"""Numeric primitives on CPU: chunked WY delta rule vs the per-token recurrence, hand
goldens (reference tests/test_kernels.py:279-316), FP8 round trip, dispatch/combine."""
import pytest
import torch

from prometheus_b200 import kernels


def _rand(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("seq,chunk", [(5, 64), (64, 16), (70, 32), (128, 64)])
def test_chunked_matches_recurrent(seq, chunk):
    b, h, dk, dv = 2, 3, 8, 6
    q, k = _rand(b, seq, h, dk, seed=1), _rand(b, seq, h, dk, seed=2)
    k = k / k.norm(dim=-1, keepdim=True)
    v = _rand(b, seq, h, dv, seed=3)
    beta = torch.sigmoid(_rand(b, seq, h, seed=4))
    s0 = _rand(b, h, dk, dv, seed=5) * 0.1
    o_ref, s_ref = kernels.delta_rule_recurrent(q, k, v, beta, s0)
    o, s = kernels.chunked_delta_rule(q, k, v, beta, s0, kernels.LinearAttnConfig(chunk=chunk))
    torch.testing.assert_close(o, o_ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s, s_ref, rtol=1e-4, atol=1e-4)


def test_delta_goldens():
    q = torch.tensor([[[[1.0, 0.0]], [[0.0, 1.0]]]])
    v = torch.tensor([[[[1.0, 2.0]], [[3.0, 4.0]]]])
    out, state = kernels.chunked_delta_rule(q, q.clone(), v, torch.ones(1, 2, 1))
    torch.testing.assert_close(out, v)
    torch.testing.assert_close(state, torch.tensor([[[[1.0, 2.0], [3.0, 4.0]]]]))
    out, state = kernels.chunked_delta_rule(
        torch.tensor([[[[1.0, 0.0]]]]), torch.tensor([[[[1.0, 0.0]]]]),
        torch.tensor([[[[2.0, 4.0]]]]), torch.tensor([[[0.5]]]))
    torch.testing.assert_close(out, torch.tensor([[[[1.0, 2.0]]]]))
    torch.testing.assert_close(state, torch.tensor([[[[1.0, 2.0], [0.0, 0.0]]]]))
    out, state = kernels.chunked_delta_rule(
        torch.tensor([[[[1.0, 0.0]]]]), torch.tensor([[[[0.0, 1.0]]]]),
        torch.tensor([[[[0.0, 0.0]]]]), torch.tensor([[[1.0]]]), state=torch.eye(2)[None, None])
    torch.testing.assert_close(out, torch.tensor([[[[1.0, 0.0]]]]))
    torch.testing.assert_close(state, torch.tensor([[[[1.0, 0.0], [0.0, 0.0]]]]))


def test_delta_explicit_vjp_matches_autograd_of_recurrence():
    b, s, h, d = 1, 20, 2, 4
    q, k, v = _rand(b, s, h, d, seed=1), _rand(b, s, h, d, seed=2), _rand(b, s, h, d, seed=3)
    k = k / k.norm(dim=-1, keepdim=True)
    beta = torch.sigmoid(_rand(b, s, h, seed=4))
    s0 = _rand(b, h, d, d, seed=5) * 0.1
    go, gs = _rand(b, s, h, d, seed=6), _rand(b, h, d, d, seed=7)
    (_, _), res = kernels.chunked_delta_rule_fwd(q, k, v, beta, s0, kernels.LinearAttnConfig(8))
    grads = kernels.chunked_delta_rule_bwd(res, (go, gs))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, beta, s0)]
    o, ns = kernels.delta_rule_recurrent(*leaves)
    ref = torch.autograd.grad([o, ns], leaves, [go, gs])
    for g, r in zip(grads, ref):
        torch.testing.assert_close(g, r, rtol=1e-3, atol=1e-4)


def test_fp8_roundtrip_and_scales():
    x = _rand(4, 300, seed=1) * 3
    meta = kernels.fp8_quantize(x, block=128)
    assert meta.scale.shape == (4, 3) and meta.q.dtype == torch.int8
    back = kernels.fp8_dequantize(meta)
    assert (back - x).abs().max() <= x.abs().max() * 0.07
    # amax of every block is representable exactly (scale = amax / 448)
    xb = torch.nn.functional.pad(x, (0, 84)).reshape(4, 3, 128)
    bb = torch.nn.functional.pad(back, (0, 84)).reshape(4, 3, 128)
    torch.testing.assert_close(bb.abs().amax(-1), xb.abs().amax(-1), rtol=1e-6, atol=0)
    z = kernels.fp8_quantize(torch.zeros(2, 128))
    assert (z.scale == 1).all() and (kernels.fp8_dequantize(z) == 0).all()


def test_fp8_e4m3_bit_goldens():
    # 448 is the largest finite e4m3 value (0x7E), 2^-9 the smallest subnormal (0x01)
    x = torch.tensor([[448.0, -448.0, 1.0, 2.0 ** -9 * 448.0 / 448.0, 0.0]])
    meta = kernels.fp8_quantize(x, block=5)
    bits = meta.q.view(torch.uint8)[0].tolist()
    assert bits[0] == 0x7E and bits[1] == 0xFE and bits[2] == 0x38 and bits[4] == 0x00


def test_fp8_2d_blocks_and_linear_ste():
    w = _rand(200, 260, seed=2)
    m = kernels.fp8_quantize_2d(w, block=128)
    assert m.scale.shape == (2, 3)
    assert (kernels.fp8_dequantize(m) - w).abs().max() <= w.abs().max() * 0.07
    x = _rand(6, 260, seed=3).requires_grad_(True)
    wl = w.clone().requires_grad_(True)
    y = kernels.fp8_linear(x, wl, 128)
    y.sum().backward()
    xh = kernels.fp8_dequantize(kernels.fp8_quantize(x.detach(), block=128))
    wh = kernels.fp8_dequantize(kernels.fp8_quantize(w, block=128))
    torch.testing.assert_close(y.detach(), xh @ wh.T)
    torch.testing.assert_close(x.grad, torch.ones(6, 200) @ wh)
    torch.testing.assert_close(wl.grad, torch.ones(200, 6) @ xh)


def test_dispatch_combine_roundtrip_and_order():
    n, d, e, k = 7, 5, 4, 2
    tokens = _rand(n, d, seed=1)
    ids = torch.tensor([[0, 1], [1, 2], [0, 3], [2, 3], [1, 0], [3, 2], [0, 1]])
    probs = torch.rand(n, k, generator=torch.Generator().manual_seed(2))
    meta = kernels.DispatchMeta(ids, probs, torch.zeros(e, dtype=torch.int64), e, 4)
    disp, res = kernels.ep_dispatch(tokens, meta)
    assert disp.shape == (e, res.max_per_expert, d)
    # slot order inside an expert = increasing token index
    assert res.token_index[0].tolist()[:4] == [0, 2, 4, 6]
    out = kernels.ep_combine(disp, meta, res)
    torch.testing.assert_close(out, tokens * probs.sum(-1, keepdim=True))
    g = _rand(e, res.max_per_expert, d, seed=3)
    gt = kernels.ep_dispatch_bwd(res, g)
    t2 = tokens.clone().requires_grad_(True)
    d2, _ = kernels.ep_dispatch(t2, meta)
    (d2 * g).sum().backward()
    torch.testing.assert_close(gt, t2.grad)


def test_dispatch_rejects_rack_span_and_bad_ids():
    tokens = _rand(2, 3)
    meta = kernels.DispatchMeta(torch.tensor([[0, 3], [1, 2]]), torch.ones(2, 2),
                                torch.tensor([0, 1, 2, 3]), 4, max_racks=1)
    with pytest.raises(kernels.KernelError):
        kernels.ep_dispatch(tokens, meta)
    bad = kernels.DispatchMeta(torch.tensor([[0, 9], [1, 2]]), torch.ones(2, 2),
                               torch.zeros(4, dtype=torch.int64), 4)
    with pytest.raises(kernels.KernelError):
        kernels.ep_dispatch(tokens, bad)


def test_compile_cache(tmp_path):
    c = kernels.CompileCache(tmp_path / "cc")
    art, hit = c.get_or_compile(b"prog", lambda p: b"bin:" + p)
    assert (art, hit) == (b"bin:prog", False)
    assert c.get_or_compile(b"prog", lambda p: 1 / 0) == (b"bin:prog", True)
    assert c.store(b"prog", b"bin:prog") == kernels.program_hash(b"prog")
    with pytest.raises(kernels.CacheError):
        c.store(b"prog", b"other")
    (tmp_path / "cc" / kernels.program_hash(b"torn")).write_bytes(b"CC01\x00")
    assert c.lookup(b"torn") is None
    blob = (tmp_path / "cc" / kernels.program_hash(b"prog")).read_bytes()
    assert blob[:4] == b"CC01" and int.from_bytes(blob[4:12], "big") == 8


def test_affine_scan_delta_matches_recurrent():
    from prometheus_b200.ops import delta

    b, s, h, dk, dv = 2, 100, 2, 8, 6
    q, k = _rand(b, s, h, dk, seed=1), _rand(b, s, h, dk, seed=2)
    k = k / k.norm(dim=-1, keepdim=True)
    v = _rand(b, s, h, dv, seed=3)
    beta = torch.sigmoid(_rand(b, s, h, seed=4))
    s0 = _rand(b, h, dk, dv, seed=5) * 0.1
    o_ref, s_ref = kernels.delta_rule_recurrent(q, k, v, beta, s0)
    o, st = delta.delta_rule_scan(q, k, v, beta, s0, chunk=16)
    torch.testing.assert_close(o, o_ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(st, s_ref, rtol=1e-4, atol=1e-4)
