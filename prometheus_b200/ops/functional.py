"""Autograd wrappers around the sm_100a kernels (bf16 activations, fp32 statistics)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import call, ptr, stream_ptr

Tensor = torch.Tensor
BF16 = torch.bfloat16

_status_buf: dict[int, Tensor] = {}
_scratch: dict[tuple, Tensor] = {}


def status_word(device) -> Tensor:
    """Per-device int32 the kernels latch a non-zero code into when a bounded wait runs out."""
    idx = torch.device(device).index or 0
    if idx not in _status_buf:
        _status_buf[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_buf[idx]


def check_status(device) -> None:
    """Raise if any kernel on ``device`` recorded a timed-out wait (synchronises)."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"a device-side bounded wait timed out (code {code})")


def scratch(device, nfloats: int, tag: str = "") -> Tensor:
    """Reusable fp32 scratch buffer (grown on demand, one per device and tag)."""
    key = (torch.device(device).index or 0, tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
def gemm(a: Tensor, b: Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Tensor | None = None,
         out_dtype=BF16, d: Tensor | None = None, alpha: float = 1.0, beta: float = 0.0,
         max_ctas: int = 0) -> Tensor:
    """``C = alpha * A @ B^T + beta * D`` on the tcgen05 kernel.

    A is logically (.., M, K): stored (.., M, K) or, with ``a_mn``, (.., K, M).
    B is logically (.., N, K): stored (.., N, K) or, with ``b_mn``, (.., K, N).
    Leading batch axes (at most one after flattening) must match. ``out`` may be given
    (bf16 or fp32); ``d`` has the shape and dtype class of the output.
    """
    assert a.dtype == BF16 and b.dtype == BF16 and a.is_cuda
    if a.ndim == 2:
        a3, b3 = a[None], b[None]
    else:
        a3, b3 = a.reshape(-1, *a.shape[-2:]), b.reshape(-1, *b.shape[-2:])
    batch = a3.shape[0]
    assert b3.shape[0] == batch
    if a3.stride(-1) != 1 or (batch > 1 and a3.stride(0) % 8) or a3.stride(1) % 8:
        a3 = a3.contiguous()
    if b3.stride(-1) != 1 or (batch > 1 and b3.stride(0) % 8) or b3.stride(1) % 8:
        b3 = b3.contiguous()
    M, K = (a3.shape[2], a3.shape[1]) if a_mn else (a3.shape[1], a3.shape[2])
    N, Kb = (b3.shape[2], b3.shape[1]) if b_mn else (b3.shape[1], b3.shape[2])
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
        c3 = out
    else:
        c3 = out.reshape(batch, M, N) if out.ndim != 3 else out
        assert c3.stride(-1) == 1
    out_f32 = c3.dtype == torch.float32
    assert out_f32 or c3.dtype == BF16
    d3 = None
    if d is not None:
        d3 = d.reshape(batch, M, N) if d.ndim != 3 else d
        assert d3.stride(-1) == 1 and d3.dtype in (BF16, torch.float32)
    st = status_word(a.device)
    call("pb_gemm_bf16", ptr(a3), ptr(b3), ptr(c3), ptr(d3), M, N, K, batch,
         a3.stride(1), b3.stride(1), c3.stride(1), d3.stride(1) if d3 is not None else 0,
         a3.stride(0), b3.stride(0), c3.stride(0), d3.stride(0) if d3 is not None else 0,
         int(a_mn), int(b_mn), int(out_f32), int(d3 is not None and d3.dtype == torch.float32),
         float(alpha), float(beta), ptr(st), int(max_ctas), stream_ptr())
    if a.ndim == 2:
        return c3[0] if out is c3 else out
    return c3.reshape(*a.shape[:-2], M, N)


def gemm_ref(a, b, *, a_mn=False, b_mn=False, d=None, alpha=1.0, beta=0.0):
    af = a.float().transpose(-1, -2) if a_mn else a.float()
    bf = b.float().transpose(-1, -2) if b_mn else b.float()
    c = alpha * (af @ bf.transpose(-1, -2))
    return c if d is None else c + beta * d.float()


class _LinearFn(torch.autograd.Function):
    """y = x @ W^T, W stored (out, in). The weight gradient is accumulated in fp32 into
    ``W.main_grad`` when that attribute exists (the trainer's flat gradient buffer) and
    ``None`` is returned for it; otherwise a bf16 gradient tensor is returned."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        # the output is allocated here and returned as it is for 2-D inputs (not as a view of
        # another tensor), so that a following in-place op (l2norm_) is legal for autograd
        y = torch.empty((x2.shape[0], w.shape[0]), dtype=BF16, device=x.device)
        gemm(x2, w, out=y)
        ctx.save_for_backward(x2, w)
        ctx.w_ref = w
        ctx.xshape = x.shape
        return y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.xshape)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, d=mg, beta=1.0)
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw


def linear(x: Tensor, w: Tensor) -> Tensor:
    return _LinearFn.apply(x, w)


class _LinearMultiFn(torch.autograd.Function):
    """Several projections of one input (q, k, v of an attention layer): the forward is one GEMM per
    weight, the backward adds the input gradients up inside the GEMM epilogues
    (``dx = dy0 W0``, then ``dx = dy1 W1 + dx``, ...) instead of leaving autograd to sum separate
    tensors with elementwise kernels. Weight gradients as in ``_LinearFn``."""

    @staticmethod
    def forward(ctx, x, *ws):
        x2 = x.reshape(-1, x.shape[-1])
        outs = []
        for w in ws:
            y = torch.empty((x2.shape[0], w.shape[0]), dtype=BF16, device=x.device)
            gemm(x2, w, out=y)
            outs.append(y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0]))
        ctx.save_for_backward(x2, *ws)
        ctx.w_refs = ws
        ctx.xshape = x.shape
        return tuple(outs)

    @staticmethod
    def backward(ctx, *dys):
        x2, *ws = ctx.saved_tensors
        dx = None
        dws = []
        for i, (dy, w) in enumerate(zip(dys, ws)):
            if dy is None:
                dws.append(None)
                continue
            dy2 = dy.reshape(-1, dy.shape[-1])
            if not dy2.is_contiguous():
                dy2 = dy2.contiguous()
            if ctx.needs_input_grad[0]:
                if dx is None:
                    dx = gemm(dy2, w, b_mn=True)
                else:
                    gemm(dy2, w, b_mn=True, out=dx, d=dx, beta=1.0)
            dw = None
            if ctx.needs_input_grad[1 + i]:
                mg = getattr(ctx.w_refs[i], "main_grad", None)
                if mg is not None:
                    gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, d=mg, beta=1.0)
                else:
                    dw = gemm(dy2, x2, a_mn=True, b_mn=True)
            dws.append(dw)
        if dx is not None:
            dx = dx.reshape(ctx.xshape)
        return (dx, *dws)


def linear_multi(x: Tensor, ws) -> tuple:
    """``tuple(x @ W^T for W in ws)`` with the input gradients accumulated in the GEMM epilogues."""
    return _LinearMultiFn.apply(x, *ws)


# ---------------------------------------------------------------------------
# RMSNorm (+ residual)
# ---------------------------------------------------------------------------
def _accumulate_param_grad(p: Tensor, g: Tensor):
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        mg.add_(g.reshape(mg.shape))
        return None
    return g.to(p.dtype)


class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps, fp8_out=None):
        """``fp8_out``: a list that receives ``(q, scales)``, the e4m3 image of ``y`` in the operand
        layout of the block-scaled GEMM, written by the same kernel (d a multiple of 256, <= 2048)."""
        shape = x.shape
        d = shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        r2 = res.reshape(-1, d).contiguous() if res is not None else None
        h = torch.empty_like(x2) if res is not None else x2
        if fp8_out is not None and d % 256 == 0 and d <= 2048:
            q = torch.empty((rows, d), dtype=torch.uint8, device=x.device)
            sc = torch.empty((d // 128, rows), dtype=torch.float32, device=x.device)
            call("pb_rmsnorm_fwd_fp8", ptr(x2), ptr(r2), ptr(w), ptr(y), ptr(h) if res is not None else None,
                 ptr(rstd), ptr(q), ptr(sc), rows, d, float(eps), stream_ptr())
            fp8_out.append((q, sc))
        else:
            call("pb_rmsnorm_fwd", ptr(x2), ptr(r2), ptr(w), ptr(y), ptr(h) if res is not None else None,
                 ptr(rstd), rows, d, float(eps), stream_ptr())
        ctx.save_for_backward(h, w, rstd)
        ctx.w_ref = w
        ctx.has_res = res is not None
        ctx.shape = shape
        if res is not None:
            return y.reshape(shape), h.reshape(shape)
        return y.reshape(shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        h, w, rstd = ctx.saved_tensors
        rows, d = h.shape
        dy2 = dy.reshape(rows, d).contiguous()
        dres = dh.reshape(rows, d).contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        nparts = _lib.query("pb_rmsnorm_bwd_nparts", rows, d)
        part = scratch(h.device, nparts * d, "rms")
        dw = torch.empty(d, dtype=torch.float32, device=h.device)
        call("pb_rmsnorm_bwd", ptr(dy2), ptr(h), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(dw),
             ptr(part), 0, rows, d, stream_ptr())
        dx = dx.reshape(ctx.shape)
        gw = _accumulate_param_grad(ctx.w_ref, dw) if ctx.needs_input_grad[2] else None
        return dx, (dx if ctx.has_res else None), gw, None, None


def rmsnorm(x: Tensor, w: Tensor, eps: float = 1e-6) -> Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w (x bf16, w fp32)."""
    return _RmsNormFn.apply(x, None, w, eps)[0]


def add_rmsnorm(x: Tensor, res: Tensor, w: Tensor, eps: float = 1e-6, emit_fp8: bool = False):
    """h = x + res; y = rmsnorm(h). Returns (y, h) from one kernel. With ``emit_fp8`` the kernel
    also writes the e4m3 rows and 1 x 128 scales of ``y`` (what ``fp8.quantize_rows(y)`` would
    produce, without the extra pass over ``y``) and ``(y, h, (q, scales))`` comes back;
    the third element is ``None`` where the fused kernel does not cover the width."""
    if not emit_fp8:
        return _RmsNormFn.apply(x, res, w, eps)
    got: list = []
    y, h = _RmsNormFn.apply(x, res, w, eps, got)
    return y, h, (got[0] if got else None)


def rmsnorm_ref(x, w, eps=1e-6, res=None):
    h = x.float() if res is None else (x.float() + res.float())
    y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return (y, h) if res is not None else y


# ---------------------------------------------------------------------------
# RoPE (in place on a fresh copy), SwiGLU, L2 norm
# ---------------------------------------------------------------------------
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, seq_len, base, rot_pairs):
        x = x.contiguous().clone()
        tokens = x.numel() // (x.shape[-1] * x.shape[-2])
        ctx.args = (tokens, x.shape[-2], x.shape[-1], rot_pairs, seq_len, base)
        ctx.pos = pos
        call("pb_rope", ptr(x), ptr(pos), tokens, x.shape[-2], x.shape[-1], rot_pairs, seq_len,
             float(base), 0, stream_ptr())
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        tokens, heads, D, rot_pairs, seq_len, base = ctx.args
        call("pb_rope", ptr(g), ptr(ctx.pos), tokens, heads, D, rot_pairs, seq_len, float(base), 1,
             stream_ptr())
        return g, None, None, None, None


def rope_(x: Tensor, *, seq_len: int, pos: Tensor | None = None, base: float = 10000.0,
          partial: bool = False) -> Tensor:
    """Interleaved-pair rotary embedding of x (.., seq, heads, D); positions default to the
    index along the sequence axis, or ``pos`` (int32, one per token)."""
    n_pairs = x.shape[-1] // 2
    rot = n_pairs if not partial else max(1, n_pairs // 2)
    return _RopeFn.apply(x, pos, seq_len, base, rot)


class _RopeInplaceFn(torch.autograd.Function):
    """Rotary embedding written over a fresh projection output ``(tokens, heads * D)`` (and, in the
    backward, over the incoming gradient): no copies. Same kernel as ``rope_``."""

    @staticmethod
    def forward(ctx, x, heads, pos, seq_len, base, rot_pairs):
        if not x.is_contiguous() or x.dim() != 2 or x.shape[1] % heads:
            raise ValueError("rope2d_ needs a contiguous (tokens, heads * D) tensor")
        ctx.mark_dirty(x)
        D = x.shape[1] // heads
        ctx.args = (x.shape[0], heads, D, rot_pairs, seq_len, base)
        ctx.pos = pos
        call("pb_rope", ptr(x), ptr(pos), x.shape[0], heads, D, rot_pairs, seq_len, float(base), 0,
             stream_ptr())
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        tokens, heads, D, rot_pairs, seq_len, base = ctx.args
        call("pb_rope", ptr(g), ptr(ctx.pos), tokens, heads, D, rot_pairs, seq_len, float(base), 1,
             stream_ptr())
        return g, None, None, None, None, None


def rope2d_(x: Tensor, heads: int, *, seq_len: int, pos: Tensor | None = None, base: float = 10000.0,
            partial: bool = False) -> Tensor:
    """In-place rotary embedding of a projection output ``(tokens, heads * D)``; returns ``x``."""
    n_pairs = (x.shape[-1] // heads) // 2
    rot = n_pairs if not partial else max(1, n_pairs // 2)
    return _RopeInplaceFn.apply(x, heads, pos, seq_len, base, rot)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        H = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * H).contiguous()
        out = torch.empty((g2.shape[0], H), dtype=gu.dtype, device=gu.device)
        call("pb_swiglu_fwd", ptr(g2), ptr(out), g2.shape[0], H, stream_ptr())
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.reshape(*gu.shape[:-1], H)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        H = g2.shape[1] // 2
        d2 = dout.reshape(-1, H).contiguous()
        dgu = torch.empty_like(g2)
        call("pb_swiglu_bwd", ptr(d2), ptr(g2), ptr(dgu), g2.shape[0], H, stream_ptr())
        return dgu.reshape(ctx.shape)


def swiglu(gu: Tensor) -> Tensor:
    """silu(gu[..., :H]) * gu[..., H:] for a fused gate|up projection."""
    return _SwigluFn.apply(gu)


def swiglu_ref(gu):
    H = gu.shape[-1] // 2
    g, u = gu[..., :H].float(), gu[..., H:].float()
    return torch.nn.functional.silu(g) * u


class _L2NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        x = x.contiguous().clone()
        D = x.shape[-1]
        nvec = x.numel() // D
        inv = torch.empty(nvec, dtype=torch.float32, device=x.device)
        call("pb_l2norm_fwd", ptr(x), ptr(inv), nvec, D, float(eps), stream_ptr())
        ctx.save_for_backward(x, inv)
        return x

    @staticmethod
    def backward(ctx, g):
        xn, inv = ctx.saved_tensors
        g = g.contiguous().clone()
        D = xn.shape[-1]
        call("pb_l2norm_bwd", ptr(g), ptr(xn), ptr(inv), xn.numel() // D, D, stream_ptr())
        return g, None


def l2norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    """x / max(|x|, eps) along the last axis."""
    return _L2NormFn.apply(x, eps)


class _L2NormInplaceFn(torch.autograd.Function):
    """The same normalisation written over its input, for a tensor that nothing else reads: the
    fresh output of a projection whose backward needs only its own input and weight. The
    gradient is transformed in place as well (it is the fresh output of the consumer's
    backward). Saves the two device-to-device copies of the out-of-place form."""

    @staticmethod
    def forward(ctx, x, D, eps):
        if not x.is_contiguous():
            raise ValueError("l2norm_ needs a contiguous tensor")
        ctx.mark_dirty(x)
        nvec = x.numel() // D
        inv = torch.empty(nvec, dtype=torch.float32, device=x.device)
        call("pb_l2norm_fwd", ptr(x), ptr(inv), nvec, D, float(eps), stream_ptr())
        ctx.save_for_backward(x, inv)
        ctx.D = D
        return x

    @staticmethod
    def backward(ctx, g):
        xn, inv = ctx.saved_tensors
        g = g.contiguous()
        call("pb_l2norm_bwd", ptr(g), ptr(xn), ptr(inv), xn.numel() // ctx.D, ctx.D, stream_ptr())
        return g, None, None


def l2norm_(x: Tensor, head_dim: int, eps: float = 1e-6) -> Tensor:
    """In-place ``l2norm`` over consecutive groups of ``head_dim`` elements of a contiguous tensor
    (``(tokens, heads * head_dim)`` straight out of a projection). Returns ``x``."""
    if x.shape[-1] % head_dim:
        raise ValueError("last dimension must be a multiple of head_dim")
    return _L2NormInplaceFn.apply(x, head_dim, eps)


# ---------------------------------------------------------------------------
# soft-cap + cross-entropy over the vocabulary, fused with the unembedding GEMMs
# ---------------------------------------------------------------------------
class _SoftcapCeFn(torch.autograd.Function):
    """loss = sum_rows wt[row] * CE(softcap(h @ U^T), target). Rows are processed in chunks:
    logits chunk (bf16) -> fused CE kernel rewrites it as d(loss)/d(logits) -> dh and dU
    GEMMs, so full-vocabulary fp32 logits never exist and the backward is free."""

    @staticmethod
    def forward(ctx, h, U, targets, wt, cap, chunk_rows):
        rows, d = h.shape
        V = U.shape[0]
        dev = h.device
        loss_rows = torch.empty(rows, dtype=torch.float32, device=dev)
        need_h, need_U = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        write_grad = int(need_h or need_U)
        dh = torch.empty_like(h) if need_h else None
        mg = getattr(U, "main_grad", None)
        dU = None
        if need_U and mg is None:
            dU = torch.zeros((V, d), dtype=torch.float32, device=dev)
        acc = mg if mg is not None else dU
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            hc = h[r0:r1]
            logits = gemm(hc, U)
            call("pb_softcap_ce", ptr(logits), ptr(targets[r0:r1]), ptr(wt[r0:r1]),
                 ptr(loss_rows[r0:r1]), None, r1 - r0, V, float(cap), write_grad, stream_ptr())
            if need_h:
                gemm(logits, U, b_mn=True, out=dh[r0:r1])
            if need_U:
                gemm(logits, hc, a_mn=True, b_mn=True, out=acc, d=acc, beta=1.0)
            del logits
        ctx.save_for_backward(dh, dU)
        ctx.U_ref = U
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, g):
        dh, dU = ctx.saved_tensors
        # The trainer always calls backward with g == 1 (the loss is the root); a general
        # upstream factor is applied to the returned tensors only.
        gh = (dh * g.to(dh.dtype)) if dh is not None else None
        gU = None
        if dU is not None:
            gU = (dU * g).to(ctx.U_ref.dtype)
        return gh, gU, None, None, None, None


def softcap_cross_entropy(h: Tensor, U: Tensor, targets: Tensor, wt: Tensor, cap: float,
                          chunk_rows: int = 4096) -> Tensor:
    """Sum over rows of ``wt * CE(cap * tanh(h @ U^T / cap), targets)``.

    h: (rows, d) bf16; U: (vocab, d) bf16; targets int32; wt fp32 carries the loss mask and
    the 1/denominator. When U has a ``main_grad`` buffer its gradient is accumulated there
    during the forward (scaled as if the upstream gradient were 1)."""
    return _SoftcapCeFn.apply(h, U, targets, wt, cap, chunk_rows)


def softcap_cross_entropy_ref(h, U, targets, wt, cap):
    logits = h.float() @ U.float().T
    if cap > 0:
        logits = cap * torch.tanh(logits / cap)
    nll = torch.nn.functional.cross_entropy(logits, targets.long(), reduction="none")
    return (nll * wt.float()).sum()
