"""Latent Jacobi step on the GPU: one sweep's update of the input embeddings.

``jacobi_step(hidden, embeds, w1, w2, norm_w, slot_start, k)`` returns the embeddings of the
next sweep: slot ``j`` receives ``rmsnorm(silu(h W1^T) W2^T) * norm_w`` of the hidden state
at the position just before it, every other position keeps its embedding. The two products
run on the tcgen05 GEMM; the gather, the SiLU and the fused copy + normalise + scatter are
``csrc/kernels/latent.cu``. Differentiable in ``hidden``, ``embeds`` and the three weights
(weights in the engine's ``(out, in)`` bf16 layout; ``norm_w`` fp32).
Oracle: ``latent.latent_slot_embeddings`` with ``model._apply_latent_adapter``.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from ._lib import call, ptr, stream_ptr
from .functional import _accumulate_param_grad, linear, scratch


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, start, k):
        b, s, d = src.shape
        src = src.contiguous()
        rows = torch.empty((b * k, d), dtype=src.dtype, device=src.device)
        call("pb_latent_gather", ptr(src), ptr(rows), b, s, d, start, k, stream_ptr())
        ctx.geom = (b, s, d, start, k)
        return rows

    @staticmethod
    def backward(ctx, d_rows):
        b, s, d, start, k = ctx.geom
        d_src = torch.zeros((b, s, d), dtype=d_rows.dtype, device=d_rows.device)
        call("pb_latent_scatter", ptr(d_rows.contiguous()), ptr(d_src), b, s, d, start, k, stream_ptr())
        return d_src, None, None


class _SiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        y = torch.empty_like(x)
        call("pb_silu_fwd", ptr(x), ptr(y), x.numel(), stream_ptr())
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        call("pb_silu_bwd", ptr(dy.contiguous()), ptr(x), ptr(dx), x.numel(), stream_ptr())
        return dx


class _NormScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, embeds, start, k, eps):
        b, s, d = embeds.shape
        a, embeds = a.contiguous(), embeds.contiguous()
        out = torch.empty_like(embeds)
        rstd = torch.empty(b * k, dtype=torch.float32, device=a.device)
        call("pb_latent_norm_scatter", ptr(a), ptr(w), ptr(embeds), ptr(out), ptr(rstd), b, s, d,
             start, k, float(eps), stream_ptr())
        ctx.save_for_backward(a, w, rstd)
        ctx.w_ref = w
        ctx.geom = (b, s, d, start, k)
        return out

    @staticmethod
    def backward(ctx, d_out):
        a, w, rstd = ctx.saved_tensors
        b, s, d, start, k = ctx.geom
        d_out = d_out.contiguous()
        rows = b * k
        dy = torch.empty((rows, d), dtype=d_out.dtype, device=d_out.device)
        call("pb_latent_gather", ptr(d_out), ptr(dy), b, s, d, start, k, stream_ptr())
        da = torch.empty_like(a)
        nparts = _lib.query("pb_rmsnorm_bwd_nparts", rows, d)
        part = scratch(a.device, nparts * d, "rms")
        dw = torch.empty(d, dtype=torch.float32, device=a.device)
        call("pb_rmsnorm_bwd", ptr(dy), ptr(a), ptr(w), ptr(rstd), None, ptr(da), ptr(dw), ptr(part),
             0, rows, d, stream_ptr())
        d_emb = None
        if ctx.needs_input_grad[2]:
            d_emb = d_out.clone()
            d_emb[:, start:start + k].zero_()
        gw = _accumulate_param_grad(ctx.w_ref, dw) if ctx.needs_input_grad[1] else None
        return da, gw, d_emb, None, None, None


def jacobi_step(hidden: Tensor, embeds: Tensor, w1: Tensor, w2: Tensor, norm_w: Tensor,
                slot_start: int, k: int, eps: float = 1e-6) -> Tensor:
    """hidden, embeds: (B, S, d) bf16; w1: (adapter_hidden, d), w2: (d, adapter_hidden) bf16."""
    if slot_start < 1 or slot_start + k > embeds.shape[1]:
        raise ValueError("latent slots outside the sequence")
    rows = _GatherFn.apply(hidden, slot_start - 1, k)
    a = linear(_SiluFn.apply(linear(rows, w1)), w2)
    return _NormScatterFn.apply(a, norm_w, embeds, slot_start, k, eps)


def jacobi_step_ref(hidden, embeds, w1, w2, norm_w, slot_start: int, k: int, eps: float = 1e-6):
    """fp32 oracle of :func:`jacobi_step` (same weight layout)."""
    src = hidden.float()[:, slot_start - 1:slot_start - 1 + k]
    a = torch.nn.functional.silu(src @ w1.float().t()) @ w2.float().t()
    a = a * torch.rsqrt(a.square().mean(-1, keepdim=True) + eps) * norm_w.float()
    out = embeds.float().clone()
    out[:, slot_start:slot_start + k] = a
    return out
