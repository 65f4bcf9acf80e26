"""FP8 quantisers and the block-scaled tcgen05 GEMM against fp32 PyTorch (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _r(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(BF16)


def test_quantisers_match_the_reference_rule():
    from prometheus_b200 import kernels
    from prometheus_b200.ops import fp8

    x = _r(300, 512, seed=1, scale=3.0)
    x[5, 128:256] = 0                                   # an all-zero block keeps scale 1
    q, s = fp8.quantize_rows(x)
    # oracle on the CPU: there amax / 448 is a true division, as in the reference (on the GPU
    # PyTorch turns division by a scalar into a multiply by its rounded reciprocal)
    ref = kernels.fp8_quantize(x.float().cpu(), block=128)
    assert s.shape == (4, 300)
    assert torch.equal(s.t().cpu(), ref.scale)
    assert s[1, 5].item() == 1.0
    assert torch.equal(q.view(torch.int8).cpu(), ref.q)
    torch.testing.assert_close(fp8.dequantize_rows(q, s).cpu(), kernels.fp8_dequantize(ref))
    w = _r(200, 384, seed=2, scale=0.05)
    qw, sw = fp8.quantize_blocks(w)
    refw = kernels.fp8_quantize_2d(w.float().cpu(), block=128)
    assert sw.shape == (2, 3)
    assert torch.equal(sw.cpu(), refw.scale)
    assert torch.equal(qw.view(torch.int8).cpu(), refw.q)
    torch.testing.assert_close(fp8.dequantize_blocks(qw, sw).cpu(), kernels.fp8_dequantize(refw))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 200, 384), (1024, 1408, 2048), (77, 2048, 256)])
def test_fp8_gemm_equals_dequantised_matmul(M, N, K):
    from prometheus_b200.ops import fp8
    from prometheus_b200.ops import functional as ops

    x, w = _r(M, K, seed=1), _r(N, K, seed=2, scale=0.05)
    xq, sx = fp8.quantize_rows(x)
    wq, sw = fp8.quantize_blocks(w)
    got = fp8.gemm_fp8(xq, sx, wq, sw)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    ref = fp8.dequantize_rows(xq, sx) @ fp8.dequantize_blocks(wq, sw).t()
    err = (got.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item(), err          # bf16 output rounding only
    # and the quantisation error itself is what one expects of e4m3 (a few percent)
    exact = x.float() @ w.float().t()
    rel = (got.float() - exact).norm().item() / exact.norm().item()
    assert rel < 0.06, rel


def test_fp8_linear_and_grouped_gemm():
    from prometheus_b200 import kernels
    from prometheus_b200.ops import fp8, moe
    from prometheus_b200.ops import functional as ops

    x = _r(4, 96, 256, seed=1).requires_grad_(True)
    w = _r(384, 256, seed=2, scale=0.05).requires_grad_(True)
    y = fp8.fp8_linear(x, w)
    y.float().square().sum().backward()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = kernels.fp8_linear(xr, wr, 128, weight_2d=True)
    yr.square().sum().backward()
    assert (y.float() - yr).abs().max().item() <= 2e-2 * yr.abs().max().item()
    # straight-through gradients on the quantised operands, like the oracle: g w^ and g^T x^;
    # what is left is bf16 rounding of the products and of the incoming gradient (2 y)
    for a, b in ((x.grad, xr.grad), (w.grad, wr.grad)):
        rel = (a.float() - b).norm().item() / b.norm().item()
        assert rel < 0.02, rel
    # the weight image the backward multiplies by: quantise -> dequantise, rounded to bf16
    wq_, sw_ = fp8.quantize_blocks(w.detach())
    assert torch.equal(fp8.fakequant_blocks(w.detach()), fp8.dequantize_blocks(wq_, sw_).to(BF16))
    w3 = _r(3, 256, 384, seed=9, scale=0.05)
    q3, s3 = fp8.quantize_blocks(w3)
    assert torch.equal(fp8.fakequant_blocks(w3), fp8.dequantize_blocks(q3, s3).to(BF16))
    # grouped: rows of expert e use weight e
    T, E, k, K, N = 500, 4, 2, 256, 256
    ids = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    pl = moe.place(ids.contiguous(), E)
    xp = moe.permute(_r(T, K, seed=3), pl)
    wg = _r(E, N, K, seed=4, scale=0.05)
    xq, sx = fp8.quantize_rows(xp)
    wq, sw = fp8.quantize_blocks(wg)
    got = fp8.gemm_fp8(xq, sx, wq, sw, mblk_group=pl.mblk_group)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    off, tot = pl.expert_off.cpu().tolist(), pl.totals.cpu().tolist()
    xd, wd = fp8.dequantize_rows(xq, sx), fp8.dequantize_blocks(wq, sw)
    for e in range(E):
        seg = slice(off[e], off[e] + tot[e])
        ref = xd[seg] @ wd[e].t()
        assert (got[seg].float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()


def test_swiglu_quantize_and_dequantize_kernels():
    """The fused SwiGLU + row quantiser equals SwiGLU followed by the row quantiser (bitwise:
    it quantises the bf16 values it writes), rows beyond a device-side count stay untouched,
    and the bf16 dequantiser returns exactly scale * e4m3 value."""
    from prometheus_b200.ops import fp8
    from prometheus_b200.ops import functional as ops

    g = torch.Generator(device="cuda").manual_seed(0)
    for M, H in ((300, 128), (257, 1408), (64, 512)):
        gu = (torch.randn(M, 2 * H, device="cuda", generator=g) * 2).bfloat16()
        h_ref = ops.swiglu(gu)
        q_ref, s_ref = fp8.quantize_rows(h_ref)
        none, q0, s0 = fp8.swiglu_quantize(gu, keep_bf16=False)
        h, q, s = fp8.swiglu_quantize(gu)
        assert none is None and torch.equal(q0, q) and torch.equal(s0, s)
        assert torch.equal(h, h_ref) and torch.equal(q, q_ref) and torch.equal(s, s_ref), (M, H)
        # against plain fp32 PyTorch
        want = torch.nn.functional.silu(gu[:, :H].float()) * gu[:, H:].float()
        assert (h.float() - want).abs().max() <= 1e-2 * want.abs().max()
        deq = fp8.dequantize_rows_bf16(q, s)
        ref = fp8.dequantize_rows(q, s)
        assert torch.equal(deq.float(), ref.bfloat16().float())
        assert (deq.float() - h.float()).abs().max() <= 0.07 * h.float().abs().max()
        # device-side row count
        used = torch.tensor([M // 2], dtype=torch.int32, device="cuda")
        h2, q2, s2 = fp8.swiglu_quantize(gu, used)
        assert torch.equal(h2[: M // 2], h_ref[: M // 2]) and torch.equal(q2[: M // 2], q_ref[: M // 2])
        assert torch.equal(s2[:, : M // 2], s_ref[:, : M // 2])
        d2 = fp8.dequantize_rows_bf16(q, s, used)
        assert torch.equal(d2[: M // 2], deq[: M // 2])


@pytest.mark.parametrize("rows,d", [(300, 2048), (64, 1024), (1000, 256)])
def test_rmsnorm_emits_the_fp8_rows_the_gemm_reads(rows, d):
    """add + RMSNorm with the fused e4m3 output: y and h as without it, q and scales bitwise equal
    to the stand-alone row quantiser run over y, and the FP8 linear that takes them equal to the
    one that quantises for itself (forward and both gradients)."""
    from prometheus_b200.ops import fp8
    from prometheus_b200.ops import functional as ops

    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    r = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).float()
    x[3] = 0
    r[3] = 0                                              # an all-zero row: scale 1, bytes 0
    y0, h0 = ops.add_rmsnorm(x, r, w)
    y1, h1, qs = ops.add_rmsnorm(x, r, w, emit_fp8=True)
    assert qs is not None and torch.equal(y0, y1) and torch.equal(h0, h1)
    q_ref, s_ref = fp8.quantize_rows(y0)
    assert torch.equal(qs[0], q_ref) and torch.equal(qs[1], s_ref)
    wl = (torch.randn(256, d, device="cuda", generator=g) * 0.05).bfloat16()
    outs = []
    for pre in (None, qs):
        yl = y0.clone().requires_grad_(True)
        wp = wl.clone().requires_grad_(True)
        o = fp8.fp8_linear(yl, wp, pre)
        o.float().square().sum().backward()
        outs.append((o, yl.grad, wp.grad))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
