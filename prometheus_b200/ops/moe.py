"""Mixture-of-experts FFN on the GPU: routing kernel, stable expert-grouped row placement,
grouped tcgen05 GEMMs (forward, data gradient, per-expert weight gradient), SwiGLU, combine.

``moe_ffn`` is the single-rank (all experts local) layer; ``prometheus_b200.parallel.ep``
adds the dispatch/combine across expert-parallel ranks around the same grouped GEMMs.

Semantics follow the reference's ``moe`` (model/__init__.py:485-598 of the reference):
sigmoid router scores, stable top-k on ``score + router_bias`` (the bias steers selection
only), gates = selected scores / max(sum, 1e-9), routed experts are SwiGLU MLPs; the
per-token weight gather of the reference is replaced by grouping tokens per expert.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import call, ptr, stream_ptr

Tensor = torch.Tensor
BF16 = torch.bfloat16


@dataclass
class Placement:
    """Where every (token, slot) pair lives in the expert-grouped buffers."""

    row_of: Tensor       # [T * k] int32
    expert_off: Tensor   # [E + 1] int32, 128-aligned segment starts
    totals: Tensor       # [E] int32 rows in use per expert
    k_len: Tensor        # [E] int32 padded segment length
    mblk_group: Tensor   # [rows / 128] int32 expert of each 128-row block (-1: unused)
    rows: int            # allocated rows (upper bound, multiple of 128)
    n_experts: int
    top_k: int


def route(logits: Tensor, bias: Tensor | None, top_k: int):
    """logits [T, E] fp32 -> (probs [T, E] fp32, ids [T, k] int32, gates [T, k] fp32)."""
    T, E = logits.shape
    dev = logits.device
    probs = torch.empty((T, E), dtype=torch.float32, device=dev)
    ids = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    gates = torch.empty((T, top_k), dtype=torch.float32, device=dev)
    call("pb_moe_route", ptr(logits), ptr(bias), T, E, top_k, ptr(probs), ptr(ids), ptr(gates),
         stream_ptr())
    return probs, ids, gates


def place(ids: Tensor, n_experts: int) -> Placement:
    """Stable grouping of the (token, slot) pairs by expert (no host synchronisation: buffer
    sizes are the worst case, pairs + 127 padding rows per expert)."""
    T, k = ids.shape
    n_pairs = T * k
    dev = ids.device
    rows = (n_pairs + n_experts * 127 + 127) // 128 * 128
    nblocks = _lib.query("pb_moe_sort_nblocks", n_pairs, k)
    i32 = dict(dtype=torch.int32, device=dev)
    scratch = torch.empty(nblocks * n_experts, **i32)
    pl = Placement(row_of=torch.empty(n_pairs, **i32), expert_off=torch.empty(n_experts + 1, **i32),
                   totals=torch.empty(n_experts, **i32), k_len=torch.empty(n_experts, **i32),
                   mblk_group=torch.empty(rows // 128, **i32), rows=rows, n_experts=n_experts,
                   top_k=k)
    call("pb_moe_sort", ptr(ids), n_pairs, k, n_experts, ptr(scratch), ptr(pl.row_of),
         ptr(pl.expert_off), ptr(pl.totals), ptr(pl.k_len), ptr(pl.mblk_group), rows // 128,
         stream_ptr())
    return pl


def permute(x: Tensor, pl: Placement, scale: Tensor | None = None) -> Tensor:
    """[T, d] token rows -> [rows, d] expert-grouped rows (padding rows zero)."""
    T, d = x.shape
    out = torch.empty((pl.rows, d), dtype=BF16, device=x.device)
    call("pb_moe_permute", ptr(x), ptr(pl.row_of), ptr(scale), T * pl.top_k, pl.top_k, d, x.stride(0),
         ptr(out), ptr(pl.expert_off), ptr(pl.totals), pl.n_experts, stream_ptr())
    return out


def combine(y: Tensor, pl: Placement, gates: Tensor | None, T: int, add: Tensor | None = None) -> Tensor:
    d = y.shape[1]
    out = torch.empty((T, d), dtype=BF16, device=y.device)
    call("pb_moe_combine", ptr(y), ptr(pl.row_of), ptr(gates), ptr(add), T, pl.top_k, d, ptr(out),
         y.shape[0], stream_ptr())
    return out


def grouped_gemm(a: Tensor, w: Tensor, pl: Placement, *, b_mn: bool = False,
                 out: Tensor | None = None) -> Tensor:
    """C[rows of expert e] = A[rows] @ W[e]^T (``b_mn``: @ W[e]); a [rows, K], w [E, N, K]
    (``b_mn``: [E, K, N]). ``out``: a contiguous bf16 [rows, N] destination."""
    from .functional import status_word

    R, K = a.shape
    E = w.shape[0]
    N = w.shape[2] if b_mn else w.shape[1]
    if out is None:
        out = torch.empty((R, N), dtype=BF16, device=a.device)
    else:
        assert out.shape == (R, N) and out.dtype == BF16 and out.is_contiguous()
    rc_w = w.stride(1)
    call("pb_gemm_bf16_grouped", ptr(a), ptr(w), ptr(out), R, N, K, E, a.stride(0), rc_w, N,
         w.stride(0), 1 if b_mn else 0, ptr(pl.mblk_group), ptr(status_word(a.device)), 0,
         stream_ptr())
    return out


def grouped_wgrad(a: Tensor, b: Tensor, pl: Placement, out: Tensor, accumulate: bool) -> Tensor:
    """out[e] (+)= A[rows_e]^T @ B[rows_e]; a [rows, M], b [rows, N], out [E, M, N] fp32 or bf16.
    Experts without rows keep their previous contents (zero them first when not accumulating)."""
    from .functional import status_word

    R, M = a.shape
    N = b.shape[1]
    E = out.shape[0]
    f32 = out.dtype == torch.float32
    if not accumulate:
        out.zero_()
    call("pb_gemm_bf16_grouped_wgrad", ptr(a), ptr(b), ptr(out), ptr(out), M, N, R, E, a.stride(0),
         b.stride(0), N, M * N, 1 if f32 else 0, 1 if f32 else 0, 1.0, ptr(pl.expert_off),
         ptr(pl.k_len), ptr(status_word(a.device)), 0, stream_ptr())
    return out


def _acc_grad(w: Tensor, shape3, fn):
    """Weight gradient into ``w.main_grad`` (fp32 accumulate) when present, else returned."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        fn(mg.view(shape3), True)
        return None
    return fn(torch.empty(shape3, dtype=BF16, device=w.device), False).view(w.shape)


class _MoeFfnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_w, router_bias, w_gu_p, w_down_p, top_k, n_shared, shapes, fp8=False):
        from .functional import gemm

        w_gu = w_gu_p.view(shapes[0]) if shapes is not None else w_gu_p
        w_down = w_down_p.view(shapes[1]) if shapes is not None else w_down_p
        T, d = x.shape
        E, two_h, _ = w_gu.shape          # routed + shared
        h = two_h // 2
        logits = gemm(x, router_w, out_dtype=torch.float32)
        probs, ids_r, gates_r = route(logits, router_bias, top_k)
        if n_shared:
            # shared experts: every token, gate 1, appended as extra slots
            extra = torch.arange(E - n_shared, E, dtype=torch.int32, device=x.device)
            ids = torch.cat([ids_r, extra.expand(T, n_shared)], dim=1).contiguous()
            gates = torch.cat([gates_r, torch.ones((T, n_shared), dtype=torch.float32,
                                                   device=x.device)], dim=1).contiguous()
        else:
            ids, gates = ids_r, gates_r
        pl = place(ids, E)
        xp = permute(x, pl)
        empty = x.new_empty(0)
        # FP8 products keep their quantised inputs (e4m3 + scales) for the backward, which
        # differentiates the product that was really computed: g w^ and g^T x^
        q_gu = bool(fp8) and d % 128 == 0 and w_gu.shape[1] % 128 == 0
        q_dn = bool(fp8) and h % 128 == 0 and w_down.shape[1] % 128 == 0
        if q_gu:
            from . import fp8 as F8

            xq, sx = F8.quantize_rows(xp)
            wq, sw = F8.quantize_blocks(w_gu.contiguous())
            gu = F8.gemm_fp8(xq, sx, wq, sw, mblk_group=pl.mblk_group)
            x_saved = (xq, sx)
        else:
            gu = grouped_gemm(xp, w_gu, pl)
            x_saved = (xp, empty)
        if q_dn:
            # SwiGLU and the e4m3 rows of its output in one pass
            from . import fp8 as F8

            _none, hq, sh = F8.swiglu_quantize(gu, keep_bf16=False)
            wq, sw = F8.quantize_blocks(w_down.contiguous())
            y = F8.gemm_fp8(hq, sh, wq, sw, mblk_group=pl.mblk_group)
            h_saved = (hq, sh)
        else:
            hs = torch.empty((pl.rows, h), dtype=BF16, device=x.device)
            call("pb_swiglu_fwd", ptr(gu), ptr(hs), pl.rows, h, stream_ptr())
            y = grouped_gemm(hs, w_down, pl)
            h_saved = (hs, empty)
        out = combine(y, pl, gates, T)
        ctx.save_for_backward(x, router_w, w_gu, w_down, probs, ids_r, gates, x_saved[0], x_saved[1], gu,
                              h_saved[0], h_saved[1], y)
        ctx.q_gu, ctx.q_dn = q_gu, q_dn
        ctx.pl = pl
        ctx.refs = (router_w, w_gu_p, w_down_p)
        ctx.top_k = top_k
        ctx.mark_non_differentiable(ids_r)
        return out, probs, ids_r, logits

    @staticmethod
    def backward(ctx, d_out, d_probs, _di, d_logits=None):
        from .functional import gemm

        x, router_w, w_gu, w_down, probs, ids, gates, xs0, xs1, gu, hs0, hs1, y = ctx.saved_tensors
        router_ref, gu_ref, down_ref = ctx.refs
        if ctx.q_gu or ctx.q_dn:
            from . import fp8 as F8
        # operands of the straight-through backward: the quantised ones where the forward was FP8
        # (each made just before its use, so that only one pair is alive at a time)
        hs = F8.dequantize_rows_bf16(hs0, hs1) if ctx.q_dn else hs0
        wd_b = F8.fakequant_blocks(w_down.contiguous()) if ctx.q_dn else w_down
        pl = ctx.pl
        T, d = x.shape
        E_all, two_h, _ = w_gu.shape
        E = router_w.shape[0]
        h = two_h // 2
        k = pl.top_k                       # routed + shared slots
        k_r = ctx.top_k
        d_out = d_out.contiguous()
        dgates = torch.empty((T, k), dtype=torch.float32, device=x.device)
        call("pb_moe_combine_bwd", ptr(y), ptr(d_out), ptr(pl.row_of), T * k, k, d, ptr(dgates),
             stream_ptr())
        dyp = permute(d_out, pl, scale=gates.reshape(-1))
        dh = grouped_gemm(dyp, wd_b, pl, b_mn=True)
        g_down = _acc_grad(down_ref, w_down.shape, lambda o, acc: grouped_wgrad(dyp, hs, pl, o, acc))
        del hs, wd_b
        dgu = torch.empty_like(gu)
        call("pb_swiglu_bwd", ptr(dh), ptr(gu), ptr(dgu), pl.rows, h, stream_ptr())
        xp = F8.dequantize_rows_bf16(xs0, xs1) if ctx.q_gu else xs0
        wg_b = F8.fakequant_blocks(w_gu.contiguous()) if ctx.q_gu else w_gu
        g_gu = _acc_grad(gu_ref, w_gu.shape, lambda o, acc: grouped_wgrad(dgu, xp, pl, o, acc))
        dxp = grouped_gemm(dgu, wg_b, pl, b_mn=True)
        del xp, wg_b
        dlogits = torch.empty((T, E), dtype=torch.float32, device=x.device)
        dg_r = dgates if k_r == k else dgates[:, :k_r].contiguous()
        g_r = gates if k_r == k else gates[:, :k_r].contiguous()
        call("pb_moe_route_bwd", ptr(dg_r), ptr(g_r), ptr(probs), ptr(ids), T, E, k_r, ptr(dlogits),
             stream_ptr())
        if d_probs is not None:
            dlogits = dlogits + d_probs * probs * (1.0 - probs)
        if d_logits is not None:
            dlogits = dlogits + d_logits
        dl = dlogits.to(BF16)
        # dx = sum over slots of dxp rows + dlogits @ router_w
        dx_r = gemm(dl, router_w, b_mn=True)
        dx = combine(dxp, pl, None, T, add=dx_r)
        mg = getattr(router_ref, "main_grad", None)
        g_router = None
        if mg is not None:
            gemm(dl, x, a_mn=True, b_mn=True, out=mg.view(router_w.shape), d=mg.view(router_w.shape),
                 beta=1.0)
        else:
            g_router = gemm(dl, x, a_mn=True, b_mn=True)
        return dx, g_router, None, g_gu, g_down, None, None, None, None


def moe_ffn(x: Tensor, router_w: Tensor, router_bias: Tensor | None, w_gu: Tensor, w_down: Tensor,
            top_k: int, n_shared: int = 0, shapes=None, fp8: bool = False, return_logits: bool = False):
    """Routed (+ shared) expert FFN. x [T, d] bf16; router_w [E, d]; w_gu [E + n_shared, 2h, d]
    (gate rows then up rows per expert; the shared experts last); w_down [E + n_shared, d, h].
    ``shapes`` gives those two 3-D shapes when the weights are passed as flat 2-D parameters.
    ``fp8``: forward expert products in block-scaled FP8; the backward is straight-through on the
    quantised operands (``g w^``, ``g^T x^``) as bf16 products.
    Returns (out [T, d], probs [T, E] fp32, ids [T, k] int32); out and probs are differentiable.
    ``return_logits`` appends the router logits [T, E] fp32 (differentiable: the router z-loss)."""
    res = _MoeFfnFn.apply(x, router_w, router_bias, w_gu, w_down, int(top_k), int(n_shared), shapes,
                          bool(fp8))
    return res if return_logits else res[:3]


def moe_ffn_ref(x, router_w, router_bias, w_gu, w_down, top_k, n_shared=0):
    """fp32 PyTorch statement of the same layer (oracle for the tests)."""
    xf = x.float()
    if n_shared:
        E = router_w.shape[0]
        routed, probs, ids = moe_ffn_ref(x, router_w, router_bias, w_gu[:E], w_down[:E], top_k)
        hh = w_gu.shape[1] // 2
        for j in range(E, E + n_shared):
            gu = xf @ w_gu[j].float().t()
            routed = routed + (torch.nn.functional.silu(gu[:, :hh]) * gu[:, hh:]) @ w_down[j].float().t()
        return routed, probs, ids
    probs = torch.sigmoid(xf @ router_w.float().t())
    sel = probs if router_bias is None else probs + router_bias.float()
    ids = torch.argsort(-sel, dim=-1, stable=True)[:, :top_k]
    top = torch.gather(probs, 1, ids)
    gates = top / top.sum(-1, keepdim=True).clamp_min(1e-9)
    h = w_gu.shape[1] // 2
    out = torch.zeros_like(xf)
    for s in range(top_k):
        wg = w_gu.float()[ids[:, s]]                       # [T, 2h, d]
        gu = torch.einsum("td,thd->th", xf, wg)
        hs = torch.nn.functional.silu(gu[:, :h]) * gu[:, h:]
        out = out + gates[:, s:s + 1] * torch.einsum("th,tdh->td", hs, w_down.float()[ids[:, s]])
    return out, probs, ids.to(torch.int32)
