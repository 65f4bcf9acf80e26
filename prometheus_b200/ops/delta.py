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


def delta_rule(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, state: Tensor | None = None,
               chunk: int = 64):
    """CUDA entry: bf16 in, bf16 out, fp32 state."""
    return _DeltaScanFn.apply(q, k, v, beta, state, chunk)
