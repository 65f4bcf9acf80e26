"""Causal softmax attention with grouped KV heads (the GQA layers of the hybrid).

On a GPU with head dim 128 this runs the package's own tcgen05 kernels
(``csrc/kernels/attention.cu``): a flash-style forward with the scores and the output
accumulator in tensor memory, and a two-kernel deterministic backward (dQ; dK/dV). q, k, v
are read in place from their ``(B, S, H, 128)`` layout. Other geometries and the CPU use the
plain fp32 formula, which is also the oracle of the tests
(reference: model/__init__.py softmax attention with a causal mask, scale 1/sqrt(d)).
"""
from __future__ import annotations

import math

import torch
from torch import Tensor


def causal_gqa_ref(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None) -> Tensor:
    """fp32 oracle. q: (B, S, Hq, D); k, v: (B, S, Hkv, D) -> (B, S, Hq, D) in q's dtype."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    logits = qf @ kf.transpose(-1, -2) * scale
    mask = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
    logits = logits.masked_fill(~mask, float("-inf"))
    return (torch.softmax(logits, dim=-1) @ vf).transpose(1, 2).to(q.dtype)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, want_max):
        from ._lib import call, ptr, stream_ptr
        from .functional import status_word

        b, s, hq, d = q.shape
        hkv = k.shape[2]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = torch.empty_like(q)
        lse2 = torch.empty((b, hq, s), dtype=torch.float32, device=q.device)
        rowmax = torch.empty_like(lse2) if want_max else None
        call("pb_attn_fwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse2), ptr(rowmax), b, s, hq, hkv,
             hq * d, hkv * d, hq * d, float(scale), ptr(status_word(q.device)), stream_ptr())
        ctx.save_for_backward(q, k, v, out, lse2)
        ctx.scale = float(scale)
        if want_max:
            ctx.mark_non_differentiable(rowmax)
            return out, rowmax
        return out, None

    @staticmethod
    def backward(ctx, d_out, _d_max):
        from ._lib import call, ptr, stream_ptr
        from .functional import status_word

        q, k, v, out, lse2 = ctx.saved_tensors
        b, s, hq, d = q.shape
        hkv = k.shape[2]
        d_out = d_out.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty_like(lse2)
        call("pb_attn_bwd", ptr(q), ptr(k), ptr(v), ptr(out), ptr(d_out), ptr(lse2), ptr(delta),
             ptr(dq), ptr(dk), ptr(dv), b, s, hq, hkv, hq * d, hkv * d, hq * d, ctx.scale,
             ptr(status_word(q.device)), stream_ptr())
        return dq, dk, dv, None, None


class _AttnCpFn(torch.autograd.Function):
    """Local queries at global offset ``q_off`` against the keys / values of the whole prefix."""

    @staticmethod
    def forward(ctx, q, k, v, q_off, scale):
        from ._lib import call, ptr, stream_ptr
        from .functional import status_word

        b, s, hq, d = q.shape
        skv, hkv = k.shape[1], k.shape[2]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = torch.empty_like(q)
        lse2 = torch.empty((b, hq, s), dtype=torch.float32, device=q.device)
        call("pb_attn_fwd_cp", ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse2), None, b, s, skv, int(q_off), hq,
             hkv, hq * d, hkv * d, hq * d, float(scale), ptr(status_word(q.device)), stream_ptr())
        ctx.save_for_backward(q, k, v, out, lse2)
        ctx.geom = (int(q_off), float(scale))
        return out

    @staticmethod
    def backward(ctx, d_out):
        from ._lib import call, ptr, stream_ptr
        from .functional import status_word

        q, k, v, out, lse2 = ctx.saved_tensors
        q_off, scale = ctx.geom
        b, s, hq, d = q.shape
        skv, hkv = k.shape[1], k.shape[2]
        d_out = d_out.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty_like(lse2)
        call("pb_attn_bwd_cp", ptr(q), ptr(k), ptr(v), ptr(out), ptr(d_out), ptr(lse2), ptr(delta), ptr(dq),
             ptr(dk), ptr(dv), b, s, skv, q_off, hq, hkv, hq * d, hkv * d, hq * d, scale,
             ptr(status_word(q.device)), stream_ptr())
        return dq, dk, dv, None, None


def causal_gqa_offset(q: Tensor, k: Tensor, v: Tensor, q_off: int, scale: float | None = None) -> Tensor:
    """Causal attention of a query slice that starts at global position ``q_off`` against keys and
    values that start at position 0: q ``(B, S, Hq, 128)``, k / v ``(B, S_kv, Hkv, 128)`` with
    ``S_kv >= q_off + S``. ``S`` and ``q_off`` multiples of 256, ``S_kv`` of 128 (the
    context-parallel layer pads). Gradients: ``dq`` for the slice, ``dk`` / ``dv`` for every key
    row (zero for rows no query of the slice sees)."""
    if not _fused_ok(q, k):
        raise ValueError("causal_gqa_offset needs bf16 CUDA tensors with head dim 128")
    if q.shape[1] % 256 or q_off % 256 or k.shape[1] % 128 or k.shape[1] < q_off + q.shape[1]:
        raise ValueError("causal_gqa_offset: S and q_off must be multiples of 256, S_kv of 128, S_kv >= q_off + S")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    return _AttnCpFn.apply(q, k, v, int(q_off), float(scale))


def _fused_ok(q: Tensor, k: Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and k.shape[-1] == 128
            and q.shape[2] % k.shape[2] == 0)


class UnsupportedGeometry(ValueError):
    """A CUDA call whose shape the tcgen05 kernel does not cover, made without
    ``allow_fallback=True``."""


def causal_gqa(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None,
               return_max_logit: bool = False, allow_fallback: bool = False):
    """q: (B, S, Hq, D); k, v: (B, S, Hkv, D) -> (B, S, Hq, D).

    With ``return_max_logit`` also returns the largest scaled logit per (batch, head, row),
    the statistic QK-clip needs (reference: train/__init__.py qk_clip).

    On a GPU the tcgen05 kernel covers bf16 with head dim 128; any other CUDA geometry raises
    ``UnsupportedGeometry`` unless ``allow_fallback`` is set (then the library kernel or the
    fp32 formula runs: test-sized models only). CPU tensors always use the fp32 formula."""
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if not _fused_ok(q, k):
        if q.is_cuda and not allow_fallback:
            raise UnsupportedGeometry(
                f"causal_gqa: no tcgen05 kernel for dtype {q.dtype}, head dim {d}, heads "
                f"{q.shape[2]}/{k.shape[2]}; pass allow_fallback=True for the library form")
        if q.is_cuda and not return_max_logit:
            # head dims other than 128 (test-sized models): the library kernel, not the
            # O(S^2)-memory formula
            o = torch.nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                enable_gqa=True, scale=scale)
            return o.transpose(1, 2).contiguous()
        out = causal_gqa_ref(q, k, v, scale)
        if not return_max_logit:
            return out
        hq, hkv = q.shape[2], k.shape[2]
        kf = k.float().transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
        logits = q.float().transpose(1, 2) @ kf.transpose(-1, -2) * scale
        s = q.shape[1]
        mask = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
        return out, logits.masked_fill(~mask, float("-inf")).amax(dim=-1)
    s = q.shape[1]
    pad = (-s) % 256
    if pad:   # padded keys come after every real query, so the causal mask hides them
        q, k, v = (torch.nn.functional.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
    out, rowmax = _AttnFn.apply(q, k, v, scale, return_max_logit)
    if pad:
        out = out[:, :s]
        rowmax = None if rowmax is None else rowmax[..., :s]
    return (out, rowmax) if return_max_logit else out
