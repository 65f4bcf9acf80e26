"""Numeric primitives: chunked delta rule, block-scaled FP8, expert dispatch/combine.

Public API parity with the reference ``kernels/__init__.py``:
``chunked_delta_rule[_fwd/_bwd]`` (:592-719), ``fp8_quantize/dequantize`` (:747-812),
``fp8_linear[_fwd/_bwd]`` (:849-944), ``ep_dispatch/ep_combine[_fwd/_bwd]``
(:1169-1324), ``Fp8Meta``, ``DispatchMeta``, ``LinearAttnConfig``, ``KernelError``.

Differences that are deliberate:

* the delta rule is the true chunked WY/UT-transform algorithm (the reference's
  chunking is only a traversal order): per chunk ``A = diag(b) tril(K K^T, -1)``,
  ``T = (I + A)^-1``, ``W = T b K``, ``U^ = T b V``, then the sequential part
  ``U = U^ - W S``, ``O = Q S + tril(Q K^T) U`` (diagonal included: the read is
  post-update), ``S += K^T U``. Only chunk-boundary states are kept; the
  backward recomputes inside chunks.
* FP8 rounding is the hardware's round-to-nearest-even (``cvt.rn.satfinite``);
  the reference's table quantiser breaks exact ties toward the smaller
  magnitude. Weights may use 128x128 scale tiles (``fp8_quantize_2d``).
* on CUDA bf16 inputs the same functions run the hand-written sm_100a kernels
  (``prometheus_b200.ops``); this file's torch code is their fp32 oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any

import torch

from .compile_cache import CacheError, CompileCache, program_hash  # noqa: F401  (re-export)

Tensor = torch.Tensor


class KernelError(ValueError):
    """Shape, dtype, or routing invariant failed before the kernel ran."""


class DType(str, Enum):
    FP32 = "fp32"
    BF16 = "bf16"
    FP8 = "fp8"
    NVFP4 = "nvfp4"

    def __str__(self) -> str:
        return self.value


DEFAULT_CHUNK = 64
DEFAULT_FP8_BLOCK = 128
MAX_RACKS = 4
FP8_E4M3_MAX = 448.0


@dataclass(frozen=True)
class LinearAttnConfig:
    """Chunked delta-rule knobs. ``chunk`` does not change the mathematical result."""

    chunk: int = DEFAULT_CHUNK
    eps: float = 1e-6


@dataclass(frozen=True)
class Fp8Meta:
    """Per-block scales for an FP8 packed tensor. ``q`` is the e4m3 payload viewed as int8;
    ``scale`` has one fp32 value per ``block`` elements of the contracting (last) axis, or
    per ``block x block`` tile when ``block2d`` is set."""

    q: Tensor
    scale: Tensor
    block: int = DEFAULT_FP8_BLOCK
    dtype: DType = DType.FP8
    block2d: bool = False
    shape: tuple | None = None


@dataclass(frozen=True)
class DispatchMeta:
    """Who goes where for one MoE all-to-all. ``expert_ids``/``probs``: (tokens, top_k);
    ``racks``: rack id per expert. Dispatch refuses a token spanning > ``max_racks`` racks."""

    expert_ids: Tensor
    probs: Tensor
    racks: Tensor
    n_experts: int
    max_racks: int = MAX_RACKS


@dataclass(frozen=True)
class _DeltaResidual:
    q: Tensor
    k: Tensor
    v: Tensor
    beta: Tensor
    state0: Tensor
    chunk: int


@dataclass(frozen=True)
class _DispatchResidual:
    token_index: Tensor  # (n_experts, max_per_expert), -1 padded
    k_index: Tensor
    max_per_expert: int
    n_tokens: int | None = None


def _f32(x: Any) -> Tensor:
    t = torch.as_tensor(x)
    return t if t.dtype == torch.float32 else t.float()


# ---------------------------------------------------------------------------
# delta rule
# ---------------------------------------------------------------------------
def _validate_delta(q, k, v, beta, state):
    q, k, v, beta = _f32(q), _f32(k), _f32(v), _f32(beta)
    if q.ndim != 4:
        raise KernelError(f"q must be (batch, seq, heads, dim), got {tuple(q.shape)}")
    if k.shape != q.shape:
        raise KernelError(f"k shape {tuple(k.shape)} != q shape {tuple(q.shape)}")
    if v.ndim != 4 or v.shape[:3] != q.shape[:3]:
        raise KernelError(f"v shape {tuple(v.shape)} incompatible with q {tuple(q.shape)}")
    if tuple(beta.shape) != tuple(q.shape[:3]):
        raise KernelError(f"beta shape {tuple(beta.shape)} != {tuple(q.shape[:3])}")
    if beta.device.type == "cpu" and not beta.requires_grad and bool((beta < 0).any()):
        raise KernelError("beta must be in (0, 1]")            # host tensors only: no device sync
    b, _, h, dk = q.shape
    dv = v.shape[-1]
    if state is None:
        s0 = torch.zeros((b, h, dk, dv), dtype=torch.float32, device=q.device)
    else:
        s0 = _f32(state)
        if tuple(s0.shape) != (b, h, dk, dv):
            raise KernelError(f"state shape {tuple(s0.shape)} != {(b, h, dk, dv)}")
    return q, k, v, beta, s0


def delta_rule_recurrent(q, k, v, beta, state=None):
    """Per-token recurrence (the definition; O(seq) sequential steps). Oracle for tests."""
    q, k, v, beta, s = _validate_delta(q, k, v, beta, state)
    outs = []
    for t in range(q.shape[1]):
        kt, vt, qt, bt = k[:, t], v[:, t], q[:, t], beta[:, t]
        pred = torch.einsum("bhd,bhde->bhe", kt, s)
        s = s + torch.einsum("bhd,bhe->bhde", kt, bt[..., None] * (vt - pred))
        outs.append(torch.einsum("bhd,bhde->bhe", qt, s))
    out = torch.stack(outs, dim=1) if outs else torch.zeros_like(v)
    return out, s


def wy_chunk_operands(k: Tensor, v: Tensor, beta: Tensor):
    """Per-chunk WY operands, independent of the running state.

    k: (..., C, Dk), v: (..., C, Dv), beta: (..., C). Returns (W, Uhat) with
    ``W = T diag(b) K`` and ``Uhat = T diag(b) V``, ``T = (I + diag(b) tril(K K^T, -1))^-1``.
    """
    c = k.shape[-2]
    kk = k @ k.transpose(-1, -2)
    a = torch.tril(kk, diagonal=-1) * beta[..., :, None]
    eye = torch.eye(c, dtype=k.dtype, device=k.device)
    t = torch.linalg.solve_triangular(eye + a, eye.expand_as(a).contiguous(), upper=False)
    w = t @ (k * beta[..., None])
    u = t @ (v * beta[..., None])
    return w, u


def _chunked_delta_torch(q, k, v, beta, s0, chunk: int):
    """Chunked WY-form scan in plain torch ops (differentiable). All fp32.
    q, k: (B,S,H,Dk); v: (B,S,H,Dv); beta: (B,S,H); s0: (B,H,Dk,Dv)."""
    b, s, h, dk = q.shape
    dv = v.shape[-1]
    if s == 0:
        return torch.zeros_like(v), s0
    c = int(chunk)
    pad = (-s) % c
    if pad:
        # padded tokens carry beta = 0: they write nothing into the state
        zq = torch.zeros((b, pad, h, dk), dtype=q.dtype, device=q.device)
        zv = torch.zeros((b, pad, h, dv), dtype=q.dtype, device=q.device)
        q, k, v = torch.cat([q, zq], 1), torch.cat([k, zq], 1), torch.cat([v, zv], 1)
        beta = torch.cat([beta, torch.zeros((b, pad, h), dtype=q.dtype, device=q.device)], 1)
    n = (s + pad) // c

    def chunks(x):  # (B, S, H, D) -> (B, H, N, C, D)
        return x.reshape(b, n, c, h, x.shape[-1]).permute(0, 3, 1, 2, 4)

    qc, kc, vc = chunks(q), chunks(k), chunks(v)
    bc = beta.reshape(b, n, c, h).permute(0, 3, 1, 2)
    w, uhat = wy_chunk_operands(kc, vc, bc)
    qk = torch.tril(qc @ kc.transpose(-1, -2))
    state = s0
    outs = []
    for i in range(n):
        u = uhat[:, :, i] - w[:, :, i] @ state
        outs.append(qc[:, :, i] @ state + qk[:, :, i] @ u)
        state = state + kc[:, :, i].transpose(-1, -2) @ u
    out = torch.stack(outs, dim=2)  # (B,H,N,C,Dv)
    out = out.permute(0, 2, 3, 1, 4).reshape(b, n * c, h, dv)[:, :s]
    return out, state


def chunked_delta_rule(q, k, v, beta, state=None, config: LinearAttnConfig | None = None, *,
                       initial_state=None, allow_fallback: bool = False):
    """Gated delta-rule linear attention.

    q, k: (batch, seq, heads, dim_k); v: (batch, seq, heads, dim_v); beta: (batch, seq,
    heads) write gate. state: (batch, heads, dim_k, dim_v), zeros if None. Returns
    (output shaped like v, next_state). q and k are used as given (no L2 normalisation,
    no 1/sqrt(d) scale). CUDA bf16 inputs run the fused sm_100a kernels (head dim 128,
    chunk 64; another geometry raises unless ``allow_fallback``); CPU and fp32 inputs run
    the fp32 torch implementation of the same chunked algorithm.
    """
    cfg = LinearAttnConfig() if config is None else config
    if cfg.chunk < 1:
        raise KernelError(f"chunk must be >= 1, got {cfg.chunk}")
    if state is None:
        state = initial_state
    if isinstance(q, Tensor) and q.is_cuda and q.dtype == torch.bfloat16:
        from .ops import delta as _delta_op

        return _delta_op.delta_rule(q, k, v, beta, state, chunk=int(cfg.chunk),
                                    allow_fallback=allow_fallback)
    qf, kf, vf, bf, s0 = _validate_delta(q, k, v, beta, state)
    return _chunked_delta_torch(qf, kf, vf, bf, s0, int(cfg.chunk))


def chunked_delta_rule_fwd(q, k, v, beta, state, config: LinearAttnConfig):
    """Explicit VJP forward: returns ((out, next_state), residual)."""
    if config.chunk < 1:
        raise KernelError(f"chunk must be >= 1, got {config.chunk}")
    qf, kf, vf, bf, s0 = _validate_delta(q, k, v, beta, state)
    with torch.no_grad():
        out, ns = _chunked_delta_torch(qf, kf, vf, bf, s0, int(config.chunk))
    return (out, ns), _DeltaResidual(q=qf, k=kf, v=vf, beta=bf, state0=s0, chunk=int(config.chunk))


def chunked_delta_rule_bwd(residual: _DeltaResidual, grads):
    """Explicit VJP backward: grads for (q, k, v, beta, state). The chunk interiors are
    recomputed from the residual inputs (no per-token state is ever stored)."""
    go, gs = grads
    leaves = [t.detach().clone().requires_grad_(True)
              for t in (residual.q, residual.k, residual.v, residual.beta, residual.state0)]
    with torch.enable_grad():
        out, ns = _chunked_delta_torch(*leaves, residual.chunk)
        go = torch.zeros_like(out) if go is None else _f32(go)
        gs = torch.zeros_like(ns) if gs is None else _f32(gs)
        gr = torch.autograd.grad([out, ns], leaves, [go, gs], allow_unused=True)
    return tuple(torch.zeros_like(l) if g is None else g for g, l in zip(gr, leaves))


# ---------------------------------------------------------------------------
# FP8 (E4M3FN) block-scaled quantisation
# ---------------------------------------------------------------------------
def _pad_last(x: Tensor, block: int):
    k = x.shape[-1]
    pad = (-k) % block
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
    return x, k


def fp8_quantize(x, *, block: int = DEFAULT_FP8_BLOCK) -> Fp8Meta:
    """Quantise along the last (contracting) axis in blocks of ``block``:
    scale = amax / 448 per block (1.0 for an all-zero block), q = e4m3(x / scale)."""
    if block < 1:
        raise KernelError(f"block must be >= 1, got {block}")
    x = _f32(x)
    if x.ndim < 1:
        raise KernelError("fp8_quantize needs at least one axis")
    xp, k = _pad_last(x, block)
    nb = xp.shape[-1] // block
    xb = xp.reshape(*xp.shape[:-1], nb, block)
    amax = xb.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / FP8_E4M3_MAX, torch.ones_like(amax))
    q = (xb / scale[..., None]).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(xp.shape)[..., :k].contiguous()
    return Fp8Meta(q=q.view(torch.int8), scale=scale, block=int(block), dtype=DType.FP8,
                   shape=tuple(x.shape))


def fp8_quantize_2d(w, *, block: int = DEFAULT_FP8_BLOCK) -> Fp8Meta:
    """Weight quantisation with one scale per ``block x block`` tile of a 2-D matrix."""
    w = _f32(w)
    if w.ndim != 2:
        raise KernelError("fp8_quantize_2d expects a 2-D matrix")
    r, c = w.shape
    pr, pc = (-r) % block, (-c) % block
    wp = torch.nn.functional.pad(w, (0, pc, 0, pr))
    tiles = wp.reshape((r + pr) // block, block, (c + pc) // block, block)
    amax = tiles.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / FP8_E4M3_MAX, torch.ones_like(amax))
    q = (tiles / scale[:, None, :, None]).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    q = q.to(torch.float8_e4m3fn).reshape(r + pr, c + pc)[:r, :c].contiguous()
    return Fp8Meta(q=q.view(torch.int8), scale=scale, block=int(block), dtype=DType.FP8,
                   block2d=True, shape=(r, c))


def fp8_dequantize(meta: Fp8Meta) -> Tensor:
    q = meta.q.view(torch.float8_e4m3fn).float()
    block = int(meta.block)
    if meta.block2d:
        r, c = q.shape
        s = meta.scale.repeat_interleave(block, 0)[:r].repeat_interleave(block, 1)[:, :c]
        return q * s
    s = meta.scale.repeat_interleave(block, dim=-1)[..., : q.shape[-1]]
    return q * s


class _Fp8LinearFn(torch.autograd.Function):
    """y = deq(q(x)) @ deq(q(w))^T with a straight-through backward on the dequantised
    tensors: gx = g @ w_hat, gw = g^T @ x_hat."""

    @staticmethod
    def forward(ctx, x, weight, block, weight_2d):
        xh = fp8_dequantize(fp8_quantize(x, block=block))
        wh = fp8_dequantize(fp8_quantize_2d(weight, block=block) if weight_2d
                            else fp8_quantize(weight, block=block))
        ctx.save_for_backward(xh, wh)
        return xh @ wh.transpose(-1, -2)

    @staticmethod
    def backward(ctx, g):
        xh, wh = ctx.saved_tensors
        g = _f32(g)
        gx = g @ wh
        gw = g.reshape(-1, g.shape[-1]).T @ xh.reshape(-1, xh.shape[-1])
        return gx, gw, None, None


def fp8_linear(x, weight, block: int = DEFAULT_FP8_BLOCK, *, weight_2d: bool = False) -> Tensor:
    """FP8 block-scaled linear: x (..., K), weight (N, K) -> (..., N), fp32 accumulate."""
    x, weight = _f32(x), _f32(weight)
    if weight.ndim != 2 or x.ndim < 1 or x.shape[-1] != weight.shape[-1]:
        raise KernelError(f"fp8_linear shapes {tuple(x.shape)} x {tuple(weight.shape)}")
    return _Fp8LinearFn.apply(x, weight, int(block), bool(weight_2d))


def fp8_linear_fwd(x, weight, block: int):
    x, weight = _f32(x), _f32(weight)
    xh = fp8_dequantize(fp8_quantize(x, block=block))
    wh = fp8_dequantize(fp8_quantize(weight, block=block))
    return xh @ wh.transpose(-1, -2), (xh, wh)


def fp8_linear_bwd(residual, g):
    xh, wh = residual
    g = _f32(g)
    return g @ wh, g.reshape(-1, g.shape[-1]).T @ xh.reshape(-1, xh.shape[-1])


# ---------------------------------------------------------------------------
# expert-parallel dispatch / combine (single-address-space form; the multi-GPU
# all-to-all version lives in prometheus_b200.parallel.ep)
# ---------------------------------------------------------------------------
def _validate_dispatch(tokens: Tensor, meta: DispatchMeta):
    if tokens.ndim != 2:
        raise KernelError(f"tokens must be (n_tokens, d_model), got {tuple(tokens.shape)}")
    n_tokens = int(tokens.shape[0])
    ids, probs, racks = meta.expert_ids, meta.probs, meta.racks
    n_experts = int(meta.n_experts)
    if ids.ndim != 2 or int(ids.shape[0]) != n_tokens:
        raise KernelError("expert_ids must be (n_tokens, top_k)")
    if tuple(probs.shape) != tuple(ids.shape):
        raise KernelError(f"probs shape {tuple(probs.shape)} != expert_ids shape {tuple(ids.shape)}")
    if tuple(racks.shape) != (n_experts,):
        raise KernelError(f"racks length {tuple(racks.shape)} != n_experts={n_experts}")
    if ids.numel() and bool(((ids < 0) | (ids >= n_experts)).any()):
        raise KernelError(f"expert id out of range [0, {n_experts})")
    return ids.long(), probs, racks.long(), n_experts, int(meta.max_racks)


def _check_rack_span(expert_ids: Tensor, racks: Tensor, max_racks: int) -> None:
    """KernelError if any token's chosen experts span more than max_racks racks."""
    if expert_ids.numel() == 0:
        return
    chosen = racks.long()[expert_ids.long()]
    if chosen.ndim == 1:
        chosen = chosen[:, None]
    ordered, _ = torch.sort(chosen, dim=1)
    n_unique = 1 + (ordered[:, 1:] != ordered[:, :-1]).sum(dim=1)
    if bool((n_unique > max_racks).any()):
        raise KernelError(f"token experts span more than max_racks={max_racks} distinct racks")


def dispatch_tables(expert_ids: Tensor, n_experts: int):
    """(token_index, k_index, max_per): slot = rank of the assignment inside its expert,
    ordered by increasing token index then k."""
    n_tokens, top_k = expert_ids.shape
    dev = expert_ids.device
    n_assign = n_tokens * top_k
    if n_assign == 0:
        empty = torch.full((n_experts, 0), -1, dtype=torch.int32, device=dev)
        return empty, empty.clone(), 0
    flat_e = expert_ids.reshape(-1).long()
    flat_t = torch.arange(n_tokens, device=dev).repeat_interleave(top_k)
    flat_k = torch.arange(top_k, device=dev).repeat(n_tokens)
    counts = torch.bincount(flat_e, minlength=n_experts)
    max_per = int(counts.max().item()) if n_experts else 0
    order = torch.argsort(flat_e, stable=True)
    sorted_e = flat_e[order]
    offsets = torch.zeros(n_experts + 1, dtype=torch.long, device=dev)
    offsets[1:] = torch.cumsum(counts, 0)
    slots = torch.empty(n_assign, dtype=torch.long, device=dev)
    slots[order] = torch.arange(n_assign, device=dev) - offsets[sorted_e]
    token_index = torch.full((n_experts, max_per), -1, dtype=torch.int32, device=dev)
    k_index = torch.full((n_experts, max_per), -1, dtype=torch.int32, device=dev)
    token_index[flat_e, slots] = flat_t.int()
    k_index[flat_e, slots] = flat_k.int()
    return token_index, k_index, max_per


def _gather_rows(tokens: Tensor, token_index: Tensor) -> Tensor:
    valid = token_index >= 0
    idx = token_index.clamp(min=0).long()
    return tokens[idx] * valid[..., None].to(tokens.dtype)


def ep_dispatch(tokens, meta: DispatchMeta):
    """Tokens to experts: returns (dispatched (E, max_per, d) zero-padded, residual).
    Differentiable w.r.t. tokens (the backward is the scatter-add of cotangents)."""
    tokens = _f32(tokens)
    ids, _, racks, n_experts, max_racks = _validate_dispatch(tokens, meta)
    _check_rack_span(ids, racks, max_racks)
    token_index, k_index, max_per = dispatch_tables(ids, n_experts)
    residual = _DispatchResidual(token_index=token_index, k_index=k_index,
                                 max_per_expert=max_per, n_tokens=int(tokens.shape[0]))
    return _gather_rows(tokens, token_index), residual


def ep_combine(expert_out, meta: DispatchMeta, residual: _DispatchResidual) -> Tensor:
    """Gate-weighted sum of expert outputs back to token order: (n_tokens, d_model)."""
    expert_out = _f32(expert_out)
    ti, ki = residual.token_index, residual.k_index
    if expert_out.ndim != 3 or tuple(expert_out.shape[:2]) != tuple(ti.shape):
        raise KernelError(f"expert_out shape {tuple(expert_out.shape)} does not match the tables")
    n_tokens = residual.n_tokens if residual.n_tokens is not None else int(meta.probs.shape[0])
    valid = ti >= 0
    t = ti.clamp(min=0).long()
    k = ki.clamp(min=0).long()
    w = _f32(meta.probs)[t, k] * valid.to(torch.float32)
    out = torch.zeros((n_tokens, expert_out.shape[-1]), dtype=torch.float32,
                      device=expert_out.device)
    return out.index_add(0, t.reshape(-1), (expert_out * w[..., None]).reshape(-1, expert_out.shape[-1]))


def ep_dispatch_fwd(tokens, meta: DispatchMeta):
    with torch.no_grad():
        return ep_dispatch(tokens, meta)


def ep_dispatch_bwd(residual: _DispatchResidual, g) -> Tensor:
    """Scatter of cotangents (E, max_per, d) back onto tokens (n_tokens, d)."""
    g = _f32(g)
    ti = residual.token_index
    n_tokens = residual.n_tokens
    if n_tokens is None:
        n_tokens = int(ti.max().item()) + 1 if ti.numel() else 0
    valid = (ti >= 0).to(torch.float32)
    out = torch.zeros((n_tokens, g.shape[-1]), dtype=torch.float32, device=g.device)
    return out.index_add(0, ti.clamp(min=0).long().reshape(-1),
                         (g * valid[..., None]).reshape(-1, g.shape[-1]))


def ep_combine_fwd(expert_out, meta: DispatchMeta, residual: _DispatchResidual):
    with torch.no_grad():
        return ep_combine(expert_out, meta, residual), (meta, residual)


def ep_combine_bwd(residual, g) -> Tensor:
    """Weighted scatter of token cotangents onto expert slots: (E, max_per, d)."""
    meta, res = residual
    g = _f32(g)
    valid = res.token_index >= 0
    t = res.token_index.clamp(min=0).long()
    k = res.k_index.clamp(min=0).long()
    w = _f32(meta.probs)[t, k] * valid.to(torch.float32)
    return g[t] * w[..., None]
