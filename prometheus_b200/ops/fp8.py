"""Block-scaled FP8 (e4m3) linear algebra on the GPU: quantisers + the tcgen05 FP8 GEMM.

``quantize_rows`` (activations, 1 x 128 blocks) and ``quantize_blocks`` (weights, 128 x 128
blocks) produce e4m3 bytes and fp32 scales with the reference's rule (scale = amax / 448, 1 for
an all-zero block; kernels/__init__.py ``fp8_quantize`` of the reference). ``gemm_fp8``
multiplies them with the scales applied to each 128-deep partial product, which equals
dequantise-then-matmul in exact arithmetic. ``fp8_linear`` is the differentiable layer: FP8
forward, straight-through bf16 backward (the reference's ``fp8_linear`` contract).
"""
from __future__ import annotations

import torch

from ._lib import call, ptr, stream_ptr

Tensor = torch.Tensor
BF16 = torch.bfloat16


def quantize_rows(x: Tensor, rows_used: Tensor | None = None):
    """x [M, K] bf16 (K % 128 == 0) -> (q [M, K] uint8 holding e4m3, scales [K / 128, M] fp32).
    ``rows_used`` (a device int32): only the first that many rows are touched."""
    M, K = x.shape
    assert x.dtype == BF16 and K % 128 == 0 and x.stride(1) == 1
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((K // 128, M), dtype=torch.float32, device=x.device)
    if rows_used is None:
        call("pb_fp8_quant_rows", ptr(x), x.stride(0), M, K, ptr(q), ptr(s), stream_ptr())
    else:
        call("pb_fp8_quant_rows_dyn", ptr(x), x.stride(0), M, K, ptr(q), ptr(s), ptr(rows_used),
             stream_ptr())
    return q, s


def swiglu_quantize(gu: Tensor, rows_used: Tensor | None = None, keep_bf16: bool = True):
    """gu [M, 2H] bf16 (gate | up, H % 128 == 0) -> (h [M, H] bf16, q [M, H] e4m3 bytes, scales
    [H / 128, M] fp32) in one pass: ``h = silu(gate) * up`` and the 1 x 128 block quantisation
    of those bf16 values, i.e. ``swiglu`` followed by ``quantize_rows`` without the second read.
    ``rows_used`` (a device int32): only the first that many rows are touched. ``keep_bf16=False``
    skips the bf16 copy (``h`` comes back as ``None``)."""
    M, two_h = gu.shape
    H = two_h // 2
    assert gu.dtype == BF16 and gu.is_contiguous() and H % 128 == 0
    h = torch.empty((M, H), dtype=BF16, device=gu.device) if keep_bf16 else None
    q = torch.empty((M, H), dtype=torch.uint8, device=gu.device)
    s = torch.empty((H // 128, M), dtype=torch.float32, device=gu.device)
    call("pb_swiglu_quant", ptr(gu), ptr(h), M, H, ptr(q), ptr(s), ptr(rows_used), stream_ptr())
    return h, q, s


def quantize_blocks(w: Tensor):
    """w [N, K] or [E, N, K] bf16 -> (q same shape uint8, scales [(E,) ceil(N/128), K/128])."""
    assert w.dtype == BF16 and w.is_contiguous() and w.shape[-1] % 128 == 0
    K = w.shape[-1]
    rows = w.numel() // K
    if w.ndim == 3:
        assert w.shape[1] % 128 == 0, "grouped weights need 128-aligned rows per expert"
    q = torch.empty(w.shape, dtype=torch.uint8, device=w.device)
    nb = (rows + 127) // 128
    s = torch.empty((nb, K // 128), dtype=torch.float32, device=w.device)
    call("pb_fp8_quant_blocks", ptr(w), K, rows, K, ptr(q), ptr(s), stream_ptr())
    if w.ndim == 3:
        s = s.view(w.shape[0], w.shape[1] // 128, K // 128)
    return q, s


def fakequant_blocks(w: Tensor) -> Tensor:
    """bf16 image of ``w`` after 128 x 128 block quantisation to e4m3 and back: the weight the FP8
    GEMM really multiplied by. The backward of an FP8 linear differentiates against it."""
    assert w.dtype == BF16 and w.is_contiguous() and w.shape[-1] % 128 == 0
    K = w.shape[-1]
    rows = w.numel() // K
    if w.ndim == 3:
        assert w.shape[1] % 128 == 0, "grouped weights need 128-aligned rows per expert"
    out = torch.empty_like(w)
    call("pb_fp8_fakequant_blocks", ptr(w), K, rows, K, ptr(out), stream_ptr())
    return out


def dequantize_rows(q: Tensor, s: Tensor) -> Tensor:
    return q.view(torch.float8_e4m3fn).float() * s.t().repeat_interleave(128, dim=1)


def dequantize_blocks(q: Tensor, s: Tensor) -> Tensor:
    n = q.shape[-2]
    full = s.repeat_interleave(128, dim=-2)[..., :n, :].repeat_interleave(128, dim=-1)
    return q.view(torch.float8_e4m3fn).float() * full


def dequantize_rows_bf16(q: Tensor, s: Tensor, rows_used: Tensor | None = None) -> Tensor:
    """(q [M, K] e4m3 bytes, s [K / 128, >= M] fp32) -> bf16 [M, K] on the GPU: the values an FP8
    product really multiplied, which its straight-through backward differentiates against.
    ``rows_used`` (a device int32): only the first that many rows are written."""
    M, K = q.shape
    assert q.dtype == torch.uint8 and q.is_contiguous() and s.stride(1) == 1 and s.shape[1] >= M
    y = torch.empty((M, K), dtype=BF16, device=q.device)
    call("pb_fp8_dequant_rows", ptr(q), ptr(s), s.stride(0), M, K, ptr(y), ptr(rows_used), stream_ptr())
    return y


def gemm_fp8(aq: Tensor, sa: Tensor, bq: Tensor, sb: Tensor, *, mblk_group: Tensor | None = None,
             max_ctas: int = 0, out: Tensor | None = None, arrived: Tensor | None = None,
             expect: Tensor | None = None, budget_ns: int = 0) -> Tensor:
    """C [M, N] bf16 = (aq, sa) @ (bq, sb)^T. bq [N, K], or [E, N, K] with ``mblk_group`` (one
    int32 per 128-row block of aq naming its expert, negative = skip that block). ``out``: a
    contiguous bf16 [M, N] destination (e.g. a symmetric-memory buffer peers read).
    ``arrived`` / ``expect`` (int32 per 128-row block): fused expert-parallel dispatch, aq / sa are
    a receive buffer peers are still filling and a block is consumed once ``arrived >= expect``
    (waits bounded by ``budget_ns``)."""
    from .functional import status_word

    M, K = aq.shape
    groups = bq.shape[0] if bq.ndim == 3 else 1
    N = bq.shape[-2]
    assert bq.shape[-1] == K and (groups == 1 or mblk_group is not None)
    assert sa.shape[1] == M and sa.is_contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=BF16, device=aq.device)
    else:
        assert out.shape == (M, N) and out.dtype == BF16 and out.is_contiguous()
    if arrived is not None:
        call("pb_gemm_fp8_grouped_arrive", ptr(aq), ptr(sa), ptr(bq), ptr(sb), ptr(out), M, N, K, groups,
             N, ptr(mblk_group), ptr(arrived), ptr(expect), int(budget_ns), ptr(status_word(aq.device)),
             stream_ptr())
        return out
    call("pb_gemm_fp8_blockscaled", ptr(aq), ptr(sa), ptr(bq), ptr(sb), ptr(out), M, N, K, groups, N,
         ptr(mblk_group), ptr(status_word(aq.device)), int(max_ctas), stream_ptr())
    return out


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, pre=None):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if pre is not None and pre[0].shape == x2.shape and pre[1].shape == (x2.shape[1] // 128, x2.shape[0]):
            xq, sx = pre             # quantised by the producer of x (fused into its kernel)
        else:
            xq, sx = quantize_rows(x2)
        wq, sw = quantize_blocks(w)
        # the backward differentiates y = x^ w^^T, the product that was computed: it needs the
        # quantised activations (kept as e4m3 + scales: half the bytes of x) and the quantised
        # weight (re-made from w when the backward runs)
        ctx.save_for_backward(xq, sx, w)
        ctx.w_ref = w
        ctx.xshape = x.shape
        return gemm_fp8(xq, sx, wq, sw).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .functional import gemm

        xq, sx, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, fakequant_blocks(w.contiguous()), b_mn=True).reshape(ctx.xshape)     # g w^
        dw = None
        if ctx.needs_input_grad[1]:
            xh = dequantize_rows_bf16(xq, sx)                                                   # x^
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                gemm(dy2, xh, a_mn=True, b_mn=True, out=mg, d=mg, beta=1.0)
            else:
                dw = gemm(dy2, xh, a_mn=True, b_mn=True)
        return dx, dw, None


def fp8_linear(x: Tensor, w: Tensor, xq=None) -> Tensor:
    """y = q(x) @ q(w)^T with 1 x 128 activation blocks and 128 x 128 weight blocks (w stored
    (out, in)). Straight-through gradients on the quantised operands, ``gx = g w^``,
    ``gw = g^T x^`` (reference kernels/__init__.py:849-944), as bf16 products; fp32
    ``main_grad`` accumulation as ``linear``.
    ``xq``: ``(q, scales)`` of ``x`` when its producer already wrote them
    (``functional.add_rmsnorm(..., emit_fp8=True)``); the row quantiser is then skipped."""
    return _Fp8LinearFn.apply(x, w, xq)
