"""sm_100a kernels against plain PyTorch fp32 references of the same op (needs a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16 = torch.bfloat16


def _r(*shape, seed=0, scale=1.0, dtype=BF16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


def _close(got, ref, tol=2e-2):
    """Three bounds, so that neither a wrong row of small magnitude nor a dropped tail tile can
    hide behind the largest element: (1) max abs error against the largest reference element,
    (2) every row (last axis) on its own: error norm <= 4 tol x that row's norm + tol x the norm
    of a typical row, (3) cosine of the flattened tensors >= 1 - tol^2."""
    got, ref = got.float(), ref.float()
    assert got.shape == ref.shape, f"shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), "non-finite values"
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err:.4g} vs scale {scale:.4g}"
    if ref.ndim >= 1 and ref.shape[-1] > 1:
        g2, r2 = got.reshape(-1, ref.shape[-1]), ref.reshape(-1, ref.shape[-1])
        row_err = (g2 - r2).norm(dim=1)
        row_ref = r2.norm(dim=1)
        typical = ref.pow(2).mean().sqrt().item() * math.sqrt(ref.shape[-1]) + 1e-6
        over = row_err - (4 * tol * row_ref + tol * typical)
        worst = int(over.argmax())
        assert over[worst].item() <= 0, (f"row {worst}: err {row_err[worst].item():.4g}, row norm "
                                         f"{row_ref[worst].item():.4g}, typical row {typical:.4g}")
    denom = got.norm().item() * ref.norm().item()
    if denom > 0:
        cos = (got * ref).sum().item() / denom
        assert cos >= 1 - tol * tol, f"cosine {cos:.6f}"


def test_kernel_library_is_loaded_in_tree():
    from prometheus_b200.ops import _lib

    _lib.load()
    assert "prometheus_b200/_lib/libpb200_kernels.so" in open("/proc/self/maps").read()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (384, 512, 1024),
                                   (200, 328, 264), (4096, 2048, 2048)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from prometheus_b200.ops import functional as ops

    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need the MN extent to be a multiple of 8")
    a = _r(K, M, seed=1) if a_mn else _r(M, K, seed=1)
    b = _r(K, N, seed=2) if b_mn else _r(N, K, seed=2)
    c = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = ops.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn)
    _close(c, ref)
    ops.check_status("cuda")


def test_gemm_batched_epilogue_variants():
    from prometheus_b200.ops import functional as ops

    a, b = _r(3, 256, 192, seed=1), _r(3, 320, 192, seed=2)
    d = _r(3, 256, 320, seed=3)
    c = ops.gemm(a, b, d=d, alpha=0.5, beta=-2.0)
    _close(c, ops.gemm_ref(a, b, d=d, alpha=0.5, beta=-2.0))
    acc = torch.randn(256, 320, device="cuda")
    ref = acc + ops.gemm_ref(a[0], b[0])
    ops.gemm(a[0], b[0], out=acc, d=acc, beta=1.0)
    _close(acc, ref)
    c32 = ops.gemm(a, b, out_dtype=torch.float32)
    assert c32.dtype == torch.float32
    _close(c32, ops.gemm_ref(a, b), tol=5e-3)
    ops.check_status("cuda")


def test_gemm_limited_grid_and_many_tiles():
    from prometheus_b200.ops import functional as ops

    a, b = _r(2048, 512, seed=1), _r(1536, 512, seed=2)
    _close(ops.gemm(a, b, max_ctas=16), ops.gemm_ref(a, b))
    ops.check_status("cuda")


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [
    (4096, 2560, 320, False, False),      # 16 x 10 pair tiles, K not a multiple of 64
    (2304 + 72, 2048 + 136, 512, False, False),   # ragged last row block (odd CTA all out of range) and column block
    (2048, 5632, 1024, True, True),       # weight-gradient layout
    (4096, 2048, 768, False, True),       # input-gradient layout
    (3072, 3072, 256, True, False),
])
def test_gemm_cta_pair_kernel(M, N, K, a_mn, b_mn):
    """Products with at least one full wave of 256 x 256 tiles run on the two-CTA kernel
    (tcgen05.mma.cta_group::2); same products on the single-CTA kernel for comparison."""
    from prometheus_b200.ops import functional as ops
    from prometheus_b200.ops._lib import call

    a = _r(K, M, seed=1) if a_mn else _r(M, K, seed=1)
    b = _r(K, N, seed=2) if b_mn else _r(N, K, seed=2)
    ref = ops.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn)
    c = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ops.check_status("cuda")
    _close(c, ref)
    try:
        call("pb_gemm_set_variant", 8)       # every product on the single-CTA kernel
        c1 = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    finally:
        call("pb_gemm_set_variant", 0)
    _close(c, c1, 2e-3)


def test_gemm_cta_pair_batched_epilogue_variants():
    from prometheus_b200.ops import functional as ops

    a, b = _r(10, 768, 192, seed=1), _r(10, 768, 192, seed=2)       # 3 x 3 x 10 = 90 pair tiles
    d = _r(10, 768, 768, seed=3)
    c = ops.gemm(a, b, d=d, alpha=0.5, beta=-2.0)
    _close(c, ops.gemm_ref(a, b, d=d, alpha=0.5, beta=-2.0))
    c32 = ops.gemm(a, b, out_dtype=torch.float32)
    _close(c32, ops.gemm_ref(a, b), tol=5e-3)
    big_a, big_b = _r(4096, 256, seed=4), _r(2560, 256, seed=5)
    acc = torch.randn(4096, 2560, device="cuda")
    ref = acc + ops.gemm_ref(big_a, big_b)
    ops.gemm(big_a, big_b, out=acc, d=acc, beta=1.0)
    _close(acc, ref)
    # a row stride that rules out the TMA store (direct-store epilogue)
    odd = torch.empty(4096, 2563, device="cuda", dtype=torch.bfloat16)[:, :2560]
    ops.gemm(big_a, big_b, out=odd)
    _close(odd, ops.gemm_ref(big_a, big_b))
    ops.check_status("cuda")


@pytest.mark.parametrize("rows,d", [(37, 256), (1000, 2048), (64, 384), (5, 128)])
def test_rmsnorm_fwd_bwd(rows, d):
    from prometheus_b200.ops import functional as ops

    x = _r(rows, d, seed=1).requires_grad_(True)
    res = _r(rows, d, seed=2).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).requires_grad_(True)
    y, h = ops.add_rmsnorm(x, res, w)
    gy, gh = _r(rows, d, seed=3), _r(rows, d, seed=4)
    (y.float() * gy.float()).sum().add((h.float() * gh.float()).sum()).backward()
    xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, res, w))
    yr, hr = ops.rmsnorm_ref(xr, wr, res=rr)
    # the kernel rounds h to bf16 before normalising
    _close(h, hr, 1e-2)
    _close(y, yr, 2e-2)
    ((yr * gy.float()).sum() + (hr * gh.float()).sum()).backward()
    _close(x.grad, xr.grad, 3e-2)
    _close(res.grad, rr.grad, 3e-2)
    _close(w.grad, wr.grad, 3e-2)
    y1 = ops.rmsnorm(x.detach(), w.detach())
    _close(y1, ops.rmsnorm_ref(x.detach(), w.detach()), 2e-2)


def test_rope_matches_model_and_inverts():
    from prometheus_b200 import model
    from prometheus_b200.ops import functional as ops

    B, S, H, D = 2, 300, 3, 128
    x = _r(B, S, H, D, seed=1)
    y = ops.rope_(x, seq_len=S)
    ref, _ = model.rope(x.float(), x.float(), torch.arange(S, device="cuda"), partial=False)
    _close(y, ref, 1e-2)
    xg = x.clone().requires_grad_(True)
    g = _r(B, S, H, D, seed=2)
    (ops.rope_(xg, seq_len=S).float() * g.float()).sum().backward()
    xr = x.float().requires_grad_(True)
    (model.rope(xr, xr, torch.arange(S, device="cuda"), partial=False)[0] * g.float()).sum().backward()
    _close(xg.grad, xr.grad, 1e-2)
    # large positions keep full precision (no fast-math sincos)
    pos = torch.full((B * S,), 131071, dtype=torch.int32, device="cuda")
    y2 = ops.rope_(x, seq_len=S, pos=pos)
    ref2, _ = model.rope(x.float(), x.float(), torch.full((S,), 131071.0, device="cuda"), partial=False)
    _close(y2, ref2, 1e-2)


def test_swiglu_fwd_bwd():
    from prometheus_b200.ops import functional as ops

    gu = _r(77, 2 * 512, seed=1).requires_grad_(True)
    g = _r(77, 512, seed=2)
    out = ops.swiglu(gu)
    (out.float() * g.float()).sum().backward()
    gr = gu.detach().float().requires_grad_(True)
    ref = ops.swiglu_ref(gr)
    (ref * g.float()).sum().backward()
    _close(out, ref)
    _close(gu.grad, gr.grad)


def test_l2norm_fwd_bwd():
    from prometheus_b200.ops import functional as ops

    x = _r(50, 4, 128, seed=1).requires_grad_(True)
    g = _r(50, 4, 128, seed=2)
    y = ops.l2norm(x)
    (y.float() * g.float()).sum().backward()
    xr = x.detach().float().requires_grad_(True)
    yr = xr / xr.norm(dim=-1, keepdim=True).clamp(min=1e-6)
    (yr * g.float()).sum().backward()
    _close(y, yr)
    _close(x.grad, xr.grad, 3e-2)


def test_linear_multi_and_inplace_rope_equal_the_separate_ops():
    """Three projections of one input with the input gradients summed in the GEMM epilogues, rotary
    embedding written over the projection outputs: values and all gradients against fp32."""
    from prometheus_b200 import model
    from prometheus_b200.ops import functional as ops

    T, S, d, H, Hkv, D = 600, 300, 256, 4, 2, 128
    x = _r(T, d, seed=1).requires_grad_(True)
    ws = [_r(H * D, d, seed=2, scale=0.1).requires_grad_(True), _r(Hkv * D, d, seed=3, scale=0.1).requires_grad_(True),
          _r(Hkv * D, d, seed=4, scale=0.1).requires_grad_(True)]
    gs = [_r(T, H * D, seed=5), _r(T, Hkv * D, seed=6), _r(T, Hkv * D, seed=7)]
    q, k, v = ops.linear_multi(x, ws)
    q = ops.rope2d_(q, H, seq_len=S)
    k = ops.rope2d_(k, Hkv, seq_len=S)
    sum((o.float() * g.float()).sum() for o, g in zip((q, k, v), gs)).backward()

    xr = x.detach().float().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    pos = torch.arange(S, device="cuda")
    qr = model.rope((xr @ wr[0].t()).view(T // S, S, H, D), (xr @ wr[0].t()).view(T // S, S, H, D), pos, partial=False)[0]
    kr = model.rope((xr @ wr[1].t()).view(T // S, S, Hkv, D), (xr @ wr[1].t()).view(T // S, S, Hkv, D), pos, partial=False)[0]
    vr = xr @ wr[2].t()
    outs_r = (qr.reshape(T, H * D), kr.reshape(T, Hkv * D), vr)
    sum((o * g.float()).sum() for o, g in zip(outs_r, gs)).backward()
    for got, want in zip((q, k, v), outs_r):
        _close(got, want)
    _close(x.grad, xr.grad, 4e-2)
    for w, r in zip(ws, wr):
        _close(w.grad, r.grad, 4e-2)


def test_l2norm_inplace_over_a_projection_output():
    """The in-place form on the output of a linear layer: values and the gradients of the
    layer's input and weight equal the out-of-place composition; D = 64 takes the generic kernel."""
    from prometheus_b200.ops import functional as ops

    for heads, D in ((4, 128), (8, 64)):
        x = _r(300, 256, seed=1).requires_grad_(True)
        w = _r(heads * D, 256, seed=2, scale=0.1).requires_grad_(True)
        g = _r(300, heads, D, seed=3)
        y = ops.l2norm_(ops.linear(x, w), D).view(300, heads, D)
        (y.float() * g.float()).sum().backward()
        xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        pr = (xr @ wr.t()).view(300, heads, D)
        yr = pr / pr.norm(dim=-1, keepdim=True).clamp(min=1e-6)
        (yr * g.float()).sum().backward()
        _close(y, yr)
        _close(x.grad, xr.grad, 4e-2)
        _close(w.grad if w.grad is not None else w.main_grad, wr.grad, 4e-2)


@pytest.mark.parametrize("cap", [30.0, 0.0])
def test_softcap_ce_fused(cap):
    from prometheus_b200.ops import functional as ops

    rows, d, V = 300, 256, 4096
    h = _r(rows, d, seed=1).requires_grad_(True)
    U = _r(V, d, seed=2, scale=0.3).requires_grad_(True)
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    wt = (torch.rand(rows, device="cuda") > 0.2).float() / rows
    loss = ops.softcap_cross_entropy(h, U, tgt, wt, cap, chunk_rows=128)
    loss.backward()
    hr, Ur = h.detach().float().requires_grad_(True), U.detach().float().requires_grad_(True)
    ref = ops.softcap_cross_entropy_ref(hr, Ur, tgt, wt, cap)
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 2e-2 * abs(ref.item())
    _close(h.grad, hr.grad, 5e-2)
    _close(U.grad, Ur.grad, 5e-2)


def test_optimizer_kernels():
    from prometheus_b200 import train
    from prometheus_b200.ops import _lib
    from prometheus_b200.ops._lib import call, ptr, stream_ptr

    n = 100_003
    g = torch.randn(n, device="cuda")
    scratch = torch.empty(_lib.query("pb_sumsq_nparts", n) + 8, device="cuda")
    out = torch.zeros(1, device="cuda")
    call("pb_sumsq_f32", ptr(g), n, ptr(scratch), ptr(out), 0, stream_ptr())
    assert out.item() == pytest.approx((g.double() ** 2).sum().item(), rel=1e-5)
    p, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    lp = torch.empty(n, dtype=BF16, device="cuda")
    gn = (g ** 2).sum().reshape(1)
    clip = 1.0
    s = clip / (gn.sqrt() + 1e-6)
    rp, rm, rv = train.adamw_update(p, g * s, m, v, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                    wd=0.1, step=3)
    call("pb_adamw", ptr(p), ptr(g), ptr(m), ptr(v), ptr(lp), n, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3,
         ptr(gn), clip, 1.0, stream_ptr())
    torch.testing.assert_close(p, rp, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(m, rm, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(v, rv, rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(lp.float(), rp, rtol=1e-2, atol=1e-3)
    # Muon prepare: momentum + normalised Nesterov
    r, c = 64, 96
    gm, mom = torch.randn(r * c, device="cuda"), torch.randn(r * c, device="cuda")
    x0 = torch.empty(r * c, dtype=BF16, device="cuda")
    new_m = 0.95 * mom + gm
    nes = gm + 0.95 * new_m
    call("pb_muon_prepare", ptr(gm), ptr(mom), ptr(x0), r * c, 0.95, None, 0.0, 1.0, ptr(scratch),
         stream_ptr())
    torch.testing.assert_close(mom, new_m, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(x0.float(), nes / nes.norm(), rtol=1e-2, atol=1e-3)


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """A device-side wait on a flag nobody sets returns a status code within its budget."""
    from prometheus_b200.ops import _lib
    from prometheus_b200.ops._lib import call, ptr, stream_ptr

    if not hasattr(_lib.load(), "pb_wait_flag_probe"):
        pytest.skip("probe not built")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    call("pb_wait_flag_probe", ptr(flag), 1, 2_000_000, ptr(status), stream_ptr())
    torch.cuda.synchronize()
    assert status.item() == 2


@pytest.mark.parametrize("B,S,H", [(1, 64, 1), (1, 128, 2), (2, 448, 3), (1, 200, 2)])
def test_delta_rule_fused_matches_recurrence(B, S, H):
    from prometheus_b200 import kernels
    from prometheus_b200.ops import functional as ops

    D = 128
    q = torch.nn.functional.normalize(_r(B, S, H, D, seed=1).float(), dim=-1).to(BF16)
    k = torch.nn.functional.normalize(_r(B, S, H, D, seed=2).float(), dim=-1).to(BF16)
    v = _r(B, S, H, D, seed=3)
    beta = torch.sigmoid(_r(B, S, H, seed=4).float()).to(BF16)
    s0 = _r(B, H, D, D, seed=5, scale=0.05, dtype=torch.float32)
    go = _r(B, S, H, D, seed=6)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, beta)]
    s0l = s0.clone().requires_grad_(True)
    out, st = kernels.chunked_delta_rule(*leaves, s0l)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    (out.float() * go.float()).sum().add(st.sum() * 0.01).backward()
    ref_leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v, beta)]
    s0r = s0.clone().requires_grad_(True)
    o_ref, s_ref = kernels.delta_rule_recurrent(*ref_leaves, s0r)
    (o_ref * go.float()).sum().add(s_ref.sum() * 0.01).backward()
    _close(out, o_ref, 3e-2)
    _close(st, s_ref, 3e-2)
    for name, a, b in zip("qkvb", leaves, ref_leaves):
        _close(a.grad, b.grad, 6e-2)
    _close(s0l.grad, s0r.grad, 6e-2)
    ops.check_status("cuda")


@pytest.mark.parametrize("B,S,H,seg", [(1, 1024, 2, 4), (1, 512, 1, 2), (2, 768, 1, 3)])
def test_delta_rule_segmented_walk_equals_single_pass(B, S, H, seg):
    """Sequences cut into segments (summary walk -> sequential fold -> segmented walk) against
    the single-pass walk of the same kernels and against the fp32 per-token recurrence, forward,
    final state and every gradient, with an initial state and a final-state gradient."""
    from prometheus_b200 import kernels
    from prometheus_b200.ops import functional as ops
    from prometheus_b200.ops.delta import delta_rule_fused, scan_segments

    assert scan_segments(16, 256) == 8 and scan_segments(128, 64) == 1 and scan_segments(1, 8) == 1
    assert scan_segments(64, 64) == 1 and scan_segments(32, 128) == 4
    D = 128
    q = torch.nn.functional.normalize(_r(B, S, H, D, seed=1).float(), dim=-1).to(BF16)
    k = torch.nn.functional.normalize(_r(B, S, H, D, seed=2).float(), dim=-1).to(BF16)
    v = _r(B, S, H, D, seed=3)
    beta = torch.sigmoid(_r(B, S, H, seed=4).float()).to(BF16)
    s0 = _r(B, H, D, D, seed=5, scale=0.05, dtype=torch.float32)
    go = _r(B, S, H, D, seed=6)

    def run(n_seg):
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, beta)]
        s0l = s0.clone().requires_grad_(True)
        out, st = delta_rule_fused(*leaves, s0l, n_seg=n_seg)
        (out.float() * go.float()).sum().add(st.sum() * 0.01).backward()
        torch.cuda.synchronize()
        ops.check_status("cuda")
        return [out, st] + [t.grad for t in leaves] + [s0l.grad]

    one, cut = run(1), run(seg)
    for name, a, b in zip(("out", "state", "dq", "dk", "dv", "dbeta", "ds0"), cut, one):
        err = (a.float() - b.float()).norm().item()
        assert err <= 1.5e-2 * (b.float().norm().item() + 1e-6), (name, err)
    ref_leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v, beta)]
    s0r = s0.clone().requires_grad_(True)
    o_ref, s_ref = kernels.delta_rule_recurrent(*ref_leaves, s0r)
    (o_ref * go.float()).sum().add(s_ref.sum() * 0.01).backward()
    _close(cut[0], o_ref, 3e-2)
    _close(cut[1], s_ref, 3e-2)
    for a, b in zip(cut[2:6], ref_leaves):
        _close(a, b.grad, 6e-2)
    _close(cut[6], s0r.grad, 6e-2)


def test_delta_prep_bwd_kernel_matches_fp32_oracle():
    """The fused chunk-local backward against the same algebra in batched fp32 PyTorch."""
    from prometheus_b200.ops import delta as dl
    from prometheus_b200.ops import functional as ops
    from prometheus_b200.ops._lib import call, ptr, stream_ptr

    B, S, H, D = 2, 192, 3, 128
    n = S // 64
    G = B * H * n
    q = torch.nn.functional.normalize(_r(B, S, H, D, seed=1).float(), dim=-1).to(BF16)
    k = torch.nn.functional.normalize(_r(B, S, H, D, seed=2).float(), dim=-1).to(BF16)
    v = _r(B, S, H, D, seed=3)
    beta = torch.sigmoid(_r(B, S, H, seed=4).float()).to(BF16)
    w, uh = torch.empty(G, 64, 128, dtype=BF16, device="cuda"), torch.empty(G, 64, 128, dtype=BF16, device="cuda")
    m, ap, t = (torch.empty(G, 64, 64, dtype=BF16, device="cuda") for _ in range(3))
    st = ptr(ops.status_word("cuda"))
    call("pb_delta_prep_fwd", ptr(q), ptr(k), ptr(v), ptr(beta), 0, ptr(w), ptr(uh), ptr(m), ptr(ap),
         ptr(t), B, S, H, H * D, st, 0, stream_ptr())
    # forward operands against their definition
    kc, vc, qc = (dl._to_chunks(x, n).float() for x in (k, v, q))
    bc = beta.float().reshape(B, n, 64, H).permute(0, 3, 1, 2).reshape(G, 64)
    a = torch.tril(kc @ kc.transpose(-1, -2), diagonal=-1) * bc[:, :, None]
    eye = torch.eye(64, device="cuda")
    t_ref = torch.linalg.solve_triangular(eye + a, eye.expand(G, 64, 64).contiguous(), upper=False)
    _close(t, t_ref, 2e-2)
    _close(ap, t_ref * bc[:, None, :], 2e-2)
    _close(w, (t_ref * bc[:, None, :]) @ kc, 2e-2)
    _close(uh, (t_ref * bc[:, None, :]) @ vc, 2e-2)
    _close(m, torch.tril(qc @ kc.transpose(-1, -2)), 2e-2)
    d_w, ndu, d_qs, d_ks = (_r(G, 64, 128, seed=10 + i, scale=0.5) for i in range(4))
    d_m = _r(G, 64, 64, seed=20, scale=0.5)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    db = torch.empty_like(beta)
    call("pb_delta_prep_bwd", ptr(q), ptr(k), ptr(v), ptr(beta), 0, ptr(ap), ptr(t), ptr(d_w),
         ptr(ndu), ptr(d_m), ptr(d_qs), ptr(d_ks), ptr(dq), ptr(dk), ptr(dv), ptr(db), B, S, H, H * D,
         st, 0, stream_ptr())
    torch.cuda.synchronize()
    ops.check_status("cuda")
    rq, rk, rv, rb = dl.delta_prep_backward_ref(q, k, v, beta, ap, t, d_w, ndu, d_m, d_qs, d_ks)
    _close(dq, rq, 3e-2)
    _close(dk, rk, 3e-2)
    _close(dv, rv, 3e-2)
    _close(db, rb, 3e-2)


def test_debug_bounds_build_records_and_skips_a_bad_index():
    """The -DPB_DEBUG_BOUNDS library: an index that comes from data and leaves its range is
    recorded as (kernel, index, limit) and the access is skipped; the kernel finishes and the
    context stays usable. Both injected indices stay inside real allocations, so nothing could
    fault even without the check. Runs in a child interpreter (the library is chosen at load)."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    code = r'''
import torch
from prometheus_b200.ops import _lib, functional as ops
from prometheus_b200.ops._lib import call, ptr, stream_ptr
assert _lib.load().pb_debug_bounds_enabled() == 1
assert _lib.debug_bounds_read() is None
# 1. soft-cap CE: a target outside the vocabulary (row 0 of 4: the element it names is in row 1)
V, rows = 1024, 4
logits = torch.randn(rows, V, device="cuda").bfloat16()
targets = torch.tensor([V + 3, 5, 6, 7], dtype=torch.int32, device="cuda")
wt = torch.ones(rows, device="cuda")
loss = torch.empty(rows, device="cuda")
call("pb_softcap_ce", ptr(logits), ptr(targets), ptr(wt), ptr(loss), None, rows, V, 30.0, 0, stream_ptr())
rec = _lib.debug_bounds_read()
assert rec["hits"] >= 1                                      # every thread of the row's block saw it
assert {k: rec[k] for k in ("file", "kernel", "index", "limit")} == \
    {"file": "elementwise", "kernel": 1, "index": V + 3, "limit": V}, rec
assert torch.isfinite(loss).all()
assert _lib.debug_bounds_read() is None                      # reading clears the record
# 2. MoE combine: a routed row beyond the stated row count (but inside the buffer)
T, k, d = 8, 2, 64
y = torch.randn(256, d, device="cuda").bfloat16()
row_of = torch.arange(T * k, dtype=torch.int32, device="cuda")
row_of[5] = 200
gates = torch.ones(T, k, device="cuda")
out = torch.empty(T, d, device="cuda", dtype=torch.bfloat16)
call("pb_moe_combine", ptr(y), ptr(row_of), ptr(gates), None, T, k, d, ptr(out), 128, stream_ptr())
rec = _lib.debug_bounds_read()
assert rec["file"] == "moe" and rec["kernel"] == 3 and rec["index"] == 200 and rec["limit"] == 128, rec
want = y[4].float()                                          # token 2 = rows 4 and (skipped) 200
assert torch.allclose(out[2].float(), want, atol=1e-2)
# the checked library computes the same results as the normal one on valid inputs
x = torch.randn(64, 256, device="cuda").bfloat16(); w = torch.ones(256, device="cuda")
assert torch.isfinite(ops.rmsnorm(x, w).float()).all()
print("DEBUG_BOUNDS_OK")
'''
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PB200_DEBUG_BOUNDS="1", PYTHONPATH=str(root))
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300,
                         cwd=root)
    assert res.returncode == 0 and "DEBUG_BOUNDS_OK" in res.stdout, (res.stdout + res.stderr)[-3000:]
