"""Delta-rule attention on the GPU.

``delta_rule`` is the entry used by ``kernels.chunked_delta_rule`` for CUDA bf16
inputs. The chunk-local WY operands are state independent, and the state
recurrence across chunks is affine in the state,

    S_{i+1} = (I - K_i^T W_i) S_i + K_i^T U^_i  =  P_i S_i + R_i,

so the chunk-boundary states come from a log-depth scan over affine maps
``(P_b, R_b) o (P_a, R_a) = (P_b P_a, P_b R_a + R_b)`` instead of a serial loop:
a handful of large batched products instead of hundreds of tiny launches. The
same composition is what context parallelism exchanges between ranks
(``prometheus_b200.parallel.cp``). Outputs follow in one batched pass:
``O_i = Q_i S_i + tril(Q_i K_i^T)(U^_i - W_i S_i)``.
"""
from __future__ import annotations

import torch

Tensor = torch.Tensor


def chunk_affine_maps(k: Tensor, w: Tensor, uhat: Tensor):
    """(P, R) per chunk: P = I - K^T W (Dk x Dk), R = K^T U^ (Dk x Dv)."""
    kt = k.transpose(-1, -2)
    dk = k.shape[-1]
    eye = torch.eye(dk, dtype=k.dtype, device=k.device)
    return eye - kt @ w, kt @ uhat


def affine_inclusive_scan(p: Tensor, r: Tensor):
    """Inclusive scan of affine maps along axis -3 (the chunk axis), Hillis-Steele.
    p: (..., N, Dk, Dk), r: (..., N, Dk, Dv). Element i of the result maps the state
    entering chunk 0 to the state leaving chunk i."""
    n = p.shape[-3]
    d = 1
    while d < n:
        p_hi, p_lo = p[..., d:, :, :], p[..., :-d, :, :]
        r_hi, r_lo = r[..., d:, :, :], r[..., :-d, :, :]
        new_r = p_hi @ r_lo + r_hi
        new_p = p_hi @ p_lo
        p = torch.cat([p[..., :d, :, :], new_p], dim=-3)
        r = torch.cat([r[..., :d, :, :], new_r], dim=-3)
        d *= 2
    return p, r


def delta_rule_scan(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, s0: Tensor | None,
                    chunk: int = 64):
    """fp32 chunk-parallel delta rule built from batched matmuls (differentiable).
    q, k: (B,S,H,Dk); v: (B,S,H,Dv); beta: (B,S,H). Returns (out (B,S,H,Dv), state)."""
    from ..kernels import wy_chunk_operands

    b, s, h, dk = q.shape
    dv = v.shape[-1]
    c = int(chunk)
    pad = (-s) % c
    if pad:
        q = torch.nn.functional.pad(q, (0, 0, 0, 0, 0, pad))
        k = torch.nn.functional.pad(k, (0, 0, 0, 0, 0, pad))
        v = torch.nn.functional.pad(v, (0, 0, 0, 0, 0, pad))
        beta = torch.nn.functional.pad(beta, (0, 0, 0, pad))
    n = (s + pad) // c

    def chunks(x):
        return x.reshape(b, n, c, h, x.shape[-1]).permute(0, 3, 1, 2, 4)

    qc, kc, vc = chunks(q), chunks(k), chunks(v)
    bc = beta.reshape(b, n, c, h).permute(0, 3, 1, 2)
    w, uhat = wy_chunk_operands(kc, vc, bc)
    p, r = chunk_affine_maps(kc, w, uhat)
    pacc, racc = affine_inclusive_scan(p, r)
    if s0 is None:
        s0 = torch.zeros((b, h, dk, dv), dtype=q.dtype, device=q.device)
    after = pacc @ s0[:, :, None] + racc                       # state leaving each chunk
    before = torch.cat([s0[:, :, None], after[:, :, :-1]], 2)  # state entering each chunk
    u = uhat - w @ before
    qk = torch.tril(qc @ kc.transpose(-1, -2))
    out = qc @ before + qk @ u
    out = out.permute(0, 2, 3, 1, 4).reshape(b, n * c, h, dv)[:, :s]
    return out, after[:, :, -1]


class _DeltaScanFn(torch.autograd.Function):
    """Delta rule with recomputation: only the bf16 inputs are kept for the backward, which
    re-runs the chunk-parallel scan under autograd (no per-token or per-level state saved)."""

    @staticmethod
    def forward(ctx, q, k, v, beta, state, chunk):
        with torch.no_grad():
            out, st = delta_rule_scan(q.float(), k.float(), v.float(), beta.float(),
                                      None if state is None else state.float(), chunk)
        ctx.save_for_backward(q, k, v, beta, state)
        ctx.chunk = chunk
        return out.to(q.dtype), st

    @staticmethod
    def backward(ctx, go, gs):
        q, k, v, beta, state = ctx.saved_tensors
        leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v, beta)]
        s0 = None if state is None else state.detach().float().requires_grad_(True)
        with torch.enable_grad():
            out, st = delta_rule_scan(*leaves, s0, ctx.chunk)
            outs, grads = [out], [go.float()]
            if gs is not None:
                outs.append(st)
                grads.append(gs.float())
            wrt = leaves + ([s0] if s0 is not None else [])
            gr = torch.autograd.grad(outs, wrt, grads, allow_unused=True)
        gq, gk, gv, gb = (g.to(t.dtype) if g is not None else None
                          for g, t in zip(gr[:4], (q, k, v, beta)))
        gst = gr[4] if s0 is not None else None
        return gq, gk, gv, gb, gst, None


class _BmmNT(torch.autograd.Function):
    """Batched ``a @ b^T`` on the tcgen05 GEMM (bf16 in/out), with its two gradient GEMMs."""

    @staticmethod
    def forward(ctx, a, b, fp32_out=False):
        from .functional import gemm

        ctx.save_for_backward(a, b)
        return gemm(a, b, out_dtype=torch.float32 if fp32_out else torch.bfloat16)

    @staticmethod
    def backward(ctx, g):
        from .functional import gemm

        a, b = ctx.saved_tensors
        g = g.to(torch.bfloat16).contiguous()
        return gemm(g, b, b_mn=True), gemm(g, a, a_mn=True, b_mn=True), None


class _BmmNN(torch.autograd.Function):
    """Batched ``a @ b`` on the tcgen05 GEMM (b consumed MN-major, no transpose copy)."""

    @staticmethod
    def forward(ctx, a, b):
        from .functional import gemm

        ctx.save_for_backward(a, b)
        return gemm(a, b, b_mn=True)

    @staticmethod
    def backward(ctx, g):
        from .functional import gemm

        a, b = ctx.saved_tensors
        g = g.contiguous()
        return gemm(g, b), gemm(a, g, a_mn=True, b_mn=True)


def _to_chunks(x: Tensor, n: int) -> Tensor:
    """[B, n*64, H, D] -> per-chunk [B*H*n, 64, D] (chunk g = (b*H + h)*n + i)."""
    b, s, h, d = x.shape
    return x.reshape(b, n, 64, h, d).permute(0, 3, 1, 2, 4).reshape(b * h * n, 64, d).contiguous()


def _from_chunks(x: Tensor, b: int, h: int, n: int) -> Tensor:
    d = x.shape[-1]
    return x.reshape(b, h, n, 64, d).permute(0, 2, 3, 1, 4).reshape(b, n * 64, h, d)


def scan_segments(n_seq: int, n_chunks: int, ctas: int = 148) -> int:
    """Segments per sequence for the state walk, chosen by a cost model in units of one chunk
    step of one CTA wave. The single-pass walk costs ``waves(n_seq) * n_chunks``. With ``seg``
    segments the summary launch has two CTAs per segment and does about 0.6 of a chunk step
    per chunk (three of the six products, no stores), the segmented walk one step per chunk,
    and the two extra launches plus the fold about 24 steps of start-up (tensor-memory
    allocation, first loads, state load / store: measured at about ten chunk steps per launch):

        waves(2 n_seq seg) * 0.6 n_chunks / seg  +  waves(n_seq seg) * n_chunks / seg  +  24

    The smallest power of two (at least four chunks per segment) that beats the single pass
    by a fifth is taken; 1 means the plain single-pass walk."""
    def waves(c):
        return -(-c // ctas)

    best, best_cost = 1, float(waves(n_seq) * n_chunks)
    seg = 2
    while n_chunks % seg == 0 and n_chunks // seg >= 4:
        per = n_chunks / seg
        cost = waves(2 * n_seq * seg) * 0.6 * per + waves(n_seq * seg) * per + 24.0
        if cost < 0.8 * best_cost and cost < best_cost:
            best, best_cost = seg, cost
        seg *= 2
    return best


class _DeltaFusedFn(torch.autograd.Function):
    """Delta rule, head dim 128, chunk 64, sequence a multiple of 64, on three kernels: the
    chunk-local WY operands (``pb_delta_prep_fwd``), the forward state walk and the backward
    state walk. q, k, v are read in place from their ``[B, S, H, 128]`` layout and the output
    is written in that layout. The chunk-local part of the backward is batched tcgen05 GEMMs.

    The walk is affine in the state, ``S_out = P S_in + R`` per run of chunks. When the batch
    has too few sequences to fill the GPU (``scan_segments`` > 1), or when the sequence is
    split over the ranks of a context-parallel group (``cp``), each segment's ``(P, R)`` comes
    from a summary walk without outputs (two CTAs per segment), a small sequential kernel folds
    them into the state entering every segment -- with the cross-rank hand-off in the middle
    under ``cp`` -- and one segmented walk produces the outputs: two passes of 1 / n_seg the
    length instead of one full-length pass. The backward does the same with ``P^T``."""

    @staticmethod
    def forward(ctx, q, k, v, beta, s0, cp=None, n_seg=None):
        from ._lib import call, ptr, stream_ptr
        from .functional import status_word

        b, s, h, d = q.shape
        n = s // 64
        g = b * h * n
        bh = b * h
        dev = q.device
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        beta = beta.contiguous()
        bf = torch.bfloat16
        w = torch.empty((g, 64, 128), dtype=bf, device=dev)
        uhat = torch.empty_like(w)
        m = torch.empty((g, 64, 64), dtype=bf, device=dev)
        ap = torch.empty_like(m)
        t = torch.empty_like(m)
        status = ptr(status_word(dev))
        call("pb_delta_prep_fwd", ptr(q), ptr(k), ptr(v), ptr(beta),
             1 if beta.dtype == torch.float32 else 0, ptr(w), ptr(uhat), ptr(m), ptr(ap), ptr(t),
             b, s, h, h * d, status, 0, stream_ptr())
        out = torch.empty_like(q)
        u = torch.empty_like(w)
        sb = torch.empty((g, 128, 128), dtype=bf, device=dev)
        sfin = torch.empty((bh, 128, 128), dtype=torch.float32, device=dev)
        s0c = None if s0 is None else s0.reshape(bh, d, d).float().contiguous()
        seg = int(n_seg) if n_seg else scan_segments(bh, n)
        p_map = None
        if seg == 1 and cp is None:
            call("pb_delta_scan_fwd", ptr(w), ptr(uhat), ptr(q), ptr(k), ptr(m), ptr(out), ptr(u),
                 ptr(sb), ptr(s0c), ptr(sfin), bh, n, h, h * d, status, stream_ptr())
        else:
            f32 = dict(dtype=torch.float32, device=dev)
            r_map = torch.empty((bh * seg, 128, 128), **f32)
            p_map = torch.empty_like(r_map)
            call("pb_delta_scan_summary_fwd", ptr(w), ptr(uhat), ptr(k), ptr(r_map), ptr(p_map),
                 bh, n, seg, h, h * d, status, stream_ptr())
            if cp is not None:
                # this rank's whole slice as one map, exchanged; what comes back is the state
                # entering the slice
                r_tot, p_tot = torch.empty((bh, 128, 128), **f32), torch.empty((bh, 128, 128), **f32)
                call("pb_delta_compose", ptr(p_map), ptr(r_map), None, None, ptr(r_tot), ptr(p_tot),
                     bh, seg, 0, stream_ptr())
                s0c = cp.handoff(p_tot, r_tot).reshape(bh, d, d).contiguous()
                ctx.p_tot = p_tot
            s_in = torch.empty_like(r_map)
            call("pb_delta_compose", ptr(p_map), ptr(r_map), ptr(s0c), ptr(s_in), ptr(sfin), None,
                 bh, seg, 0, stream_ptr())
            call("pb_delta_scan_fwd_seg", ptr(w), ptr(uhat), ptr(q), ptr(k), ptr(m), ptr(out), ptr(u),
                 ptr(sb), ptr(s_in), None, bh, n, seg, h, h * d, status, stream_ptr())
        ctx.save_for_backward(q, k, v, beta, w, m, ap, t, u, sb, p_map)
        ctx.has_s0 = s0 is not None
        ctx.seg, ctx.cp = seg, cp
        return out, sfin.reshape(b, h, d, d)

    @staticmethod
    def backward(ctx, d_out, d_sfin):
        from ._lib import call, ptr, stream_ptr
        from .functional import gemm, status_word

        q, k, v, beta, w, m, ap, t, u, sb, p_map = ctx.saved_tensors
        b, s, h, d = q.shape
        n = s // 64
        bh = b * h
        dev = q.device
        seg, cp = ctx.seg, ctx.cp
        d_out = d_out.contiguous()
        ndu = torch.empty_like(u)          # the kernel writes -dU
        dsb = torch.empty_like(sb)
        ds0 = torch.empty((bh, 128, 128), dtype=torch.float32, device=dev)
        dfin = None if d_sfin is None else d_sfin.reshape(bh, d, d).float().contiguous()
        status = ptr(status_word(dev))
        if p_map is None:
            call("pb_delta_scan_bwd", ptr(w), ptr(q), ptr(k), ptr(m), ptr(d_out), ptr(ndu), ptr(dsb),
                 ptr(dfin), ptr(ds0), bh, n, h, h * d, status, stream_ptr())
        else:
            g_map = torch.empty_like(p_map)
            call("pb_delta_scan_summary_bwd", ptr(w), ptr(q), ptr(k), ptr(m), ptr(d_out), ptr(g_map),
                 bh, n, seg, h, h * d, status, stream_ptr())
            if cp is not None:
                g_tot = torch.empty((bh, 128, 128), dtype=torch.float32, device=dev)
                call("pb_delta_compose", ptr(p_map), ptr(g_map), None, None, ptr(g_tot), None,
                     bh, seg, 1, stream_ptr())
                dfin = cp.handoff(ctx.p_tot, g_tot, reverse=True).reshape(bh, d, d).contiguous()
            g_in = torch.empty_like(p_map)
            call("pb_delta_compose", ptr(p_map), ptr(g_map), ptr(dfin), ptr(g_in), ptr(ds0), None,
                 bh, seg, 1, stream_ptr())
            call("pb_delta_scan_bwd_seg", ptr(w), ptr(q), ptr(k), ptr(m), ptr(d_out), ptr(ndu),
                 ptr(dsb), ptr(g_in), None, bh, n, seg, h, h * d, status, stream_ptr())
        doc = _to_chunks(d_out, n)
        d_w = gemm(ndu, sb)                                   # dW = -dU S^T
        d_m = gemm(doc, u)                                    # dM = dO U^T (masked in the kernel)
        d_qs = gemm(doc, sb)                                  # walk's dQ = dO S^T
        d_ks = gemm(u, dsb)                                   # walk's dK = U dS'^T
        d_q, d_k, d_v = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        d_beta = torch.empty_like(beta)
        call("pb_delta_prep_bwd", ptr(q), ptr(k), ptr(v), ptr(beta),
             1 if beta.dtype == torch.float32 else 0, ptr(ap), ptr(t), ptr(d_w), ptr(ndu), ptr(d_m),
             ptr(d_qs), ptr(d_ks), ptr(d_q), ptr(d_k), ptr(d_v), ptr(d_beta), b, s, h, h * d,
             status, 0, stream_ptr())
        return (d_q, d_k, d_v, d_beta, (ds0.reshape(b, h, d, d) if ctx.has_s0 else None), None, None)


def delta_prep_backward_ref(q, k, v, beta, ap, t, d_w, ndu, d_m, d_qs, d_ks):
    """The chunk-local backward in batched fp32 PyTorch (oracle for ``pb_delta_prep_bwd``).
    Per-chunk operands ``[G, 64, .]``; q, k, v, beta token-major. Returns dq, dk, dv, dbeta."""
    b, s, h, d = q.shape
    n = s // 64
    g = b * h * n
    qc, kc, vc = (_to_chunks(x, n).float() for x in (q, k, v))
    bc = beta.float().reshape(b, n, 64, h).permute(0, 3, 1, 2).reshape(g, 64)
    ap, t, d_w, ndu = ap.float(), t.float(), d_w.float(), ndu.float()
    d_m = torch.tril(d_m.float())
    dap = d_w @ kc.transpose(-1, -2) - ndu @ vc.transpose(-1, -2)
    d_k = d_ks.float() + ap.transpose(-1, -2) @ d_w
    d_v = -(ap.transpose(-1, -2) @ ndu)
    d_beta = (dap * t).sum(dim=-2)
    d_a = -(t.transpose(-1, -2) @ (dap @ ap.transpose(-1, -2)))
    gk = torch.tril(kc @ kc.transpose(-1, -2), diagonal=-1)
    d_beta = d_beta + (d_a * gk).sum(dim=-1)
    d_g = torch.tril(d_a * bc[:, :, None], diagonal=-1)
    d_k = d_k + (d_g + d_g.transpose(-1, -2)) @ kc + d_m.transpose(-1, -2) @ qc
    d_q = d_qs.float() + d_m @ kc
    d_beta = d_beta.reshape(b, h, n, 64).permute(0, 2, 3, 1).reshape(b, s, h)
    return (_from_chunks(d_q, b, h, n), _from_chunks(d_k, b, h, n), _from_chunks(d_v, b, h, n),
            d_beta)


def delta_rule_fused(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, state: Tensor | None,
                     cp=None, n_seg: int | None = None):
    """bf16, head dim 128, chunk 64 (sequences are zero-padded to a multiple of 64: padded
    tokens have beta = 0 and k = 0, so they leave the state untouched). ``cp``: a
    ``parallel.cp.DeltaCpContext`` when the sequence is split over ranks (``state`` is then
    ignored: the incoming state is what the earlier ranks hand over). ``n_seg`` overrides the
    number of segments per sequence (default: ``scan_segments``)."""
    s = q.shape[1]
    pad = (-s) % 64
    if pad:
        q = torch.nn.functional.pad(q, (0, 0, 0, 0, 0, pad))
        k = torch.nn.functional.pad(k, (0, 0, 0, 0, 0, pad))
        v = torch.nn.functional.pad(v, (0, 0, 0, 0, 0, pad))
        beta = torch.nn.functional.pad(beta, (0, 0, 0, pad))
    out, sfin = _DeltaFusedFn.apply(q, k, v, beta, state, cp, n_seg)
    return (out[:, :s] if pad else out), sfin


class UnsupportedGeometry(ValueError):
    """A CUDA call whose shape the tcgen05 kernels do not cover, made without
    ``allow_fallback=True``."""


def delta_rule(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, state: Tensor | None = None,
               chunk: int = 64, allow_fallback: bool = False):
    """CUDA entry: bf16 in, bf16 out, fp32 state. Head dim 128 with chunk 64 runs the fused
    tcgen05 path. Other geometries raise ``UnsupportedGeometry`` unless ``allow_fallback`` is
    set, in which case the chunk-parallel PyTorch scan with recomputation runs (test-sized
    models only)."""
    if q.shape[-1] == 128 and v.shape[-1] == 128 and chunk == 64:
        return delta_rule_fused(q, k, v, beta, state)
    if not allow_fallback:
        raise UnsupportedGeometry(
            f"delta_rule: no tcgen05 kernel for head dims {q.shape[-1]}/{v.shape[-1]} with chunk "
            f"{chunk}; pass allow_fallback=True for the PyTorch scan")
    return _DeltaScanFn.apply(q, k, v, beta, state, chunk)
