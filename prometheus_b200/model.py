"""Hybrid model: delta-rule linear attention + softmax attention (MLA or GQA),
dense SwiGLU or top-k MoE FFN, core-block recurrence, MTP heads, latent adapter.

This module is the parameter-tree (pytree of ``torch.Tensor``) definition of
the model and its plain-PyTorch forward. It runs on any device and dtype, is
differentiable by autograd, and is the numerical oracle for the fused sm_100a
engine in ``prometheus_b200.engine`` (which packs the same tree into flat
device buffers and runs hand-written kernels).

API parity with the reference ``model/__init__.py``: ``ModelConfig`` (:58-80),
``flagship_config``/``tiny_config`` (:110-159), ``validate_config`` (:242-281),
``attention_kind``/``ffn_kind`` (:284-302), ``rms_norm`` (:305), ``rope``/
``rope_2d`` (:361-381), ``linear_attention`` (:393), ``mla_attention`` (:435),
``moe`` (:552), ``latent_adapter`` (:607), ``init_params`` (:627),
``param_count`` (:699), ``forward`` (:803) with the truncated-recurrence
gradient cut. ``ModelConfig`` is a superset: explicit head geometry, GQA
softmax layers with RoPE, sigmoid-beta gated delta rule, dense FFN width and
router bias are optional fields whose defaults reproduce the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from enum import Enum
from typing import Any

import numpy as np
import torch

Tensor = torch.Tensor

INIT_SCALE = 0.02
ROPE_BASE = 10000.0
TRUNCATED_RECURRENCE = 4
LINEAR_TO_MLA = 3


class AttentionKind(str, Enum):
    LINEAR = "linear"
    MLA = "mla"
    GQA = "gqa"

    def __str__(self) -> str:  # StrEnum behaviour
        return self.value


class FfnKind(str, Enum):
    DENSE = "dense"
    MOE = "moe"

    def __str__(self) -> str:
        return self.value


class AttentionKindError(ValueError):
    """Layer index is outside the hybrid pattern."""


class ConfigError(ValueError):
    """Config violates an invariant (counts, ratios, required fields)."""


@dataclass(frozen=True)
class ModelConfig:
    """Discrete architecture. The first block of fields is the reference's;
    the second block (all optional) extends it for the B200 training configs."""

    d_model: int
    n_layers: int
    n_dense: int
    n_moe: int
    n_linear_attn: int
    n_mla: int
    n_routed_experts: int
    n_shared_experts: int
    top_k: int
    expert_hidden: int
    mtp_heads: int
    core_block_layers: int
    recurrence_train_mean: float
    recurrence_max: int
    vocab_size: int
    max_context: int
    max_racks: int = 4
    prelude_layers: int | None = None
    coda_layers: int | None = None
    adapter_hidden: int | None = None
    # ---- extensions (defaults reproduce the reference model) ----
    n_heads: int | None = None          # None: derived from d_model like the reference
    d_head: int | None = None
    n_kv_heads: int | None = None       # GQA key/value heads
    softmax_kind: str = "mla"           # "mla" (reference) or "gqa" (RoPE + grouped KV)
    softmax_every: int = 4              # every n-th layer is softmax; 0 = all layers linear
    delta_beta: str = "one"             # "one" (reference) or "sigmoid" (learned write gate)
    chunk: int = 64                     # delta-rule chunk length of the fused kernel
    dense_hidden: int | None = None     # dense FFN width; None: expert_hidden
    router_bias: bool = False           # aux-loss-free balancing bias on the routing scores
    rope_base: float = ROPE_BASE
    init_scale: float = INIT_SCALE
    mup_base_width: int | None = None   # muP: hidden-matrix init std scaled by sqrt(base/d_model)


# Reference flagship numbers (model/__init__.py:83-104).
FLAGSHIP_D_MODEL = 12288
FLAGSHIP_N_LAYERS = 96
FLAGSHIP_N_DENSE = 3
FLAGSHIP_N_MOE = 93
FLAGSHIP_N_LINEAR_ATTN = 72
FLAGSHIP_N_MLA = 24
FLAGSHIP_N_ROUTED_EXPERTS = 512
FLAGSHIP_N_SHARED_EXPERTS = 2
FLAGSHIP_TOP_K = 20
FLAGSHIP_EXPERT_HIDDEN = 4096
FLAGSHIP_MTP_HEADS = 2
FLAGSHIP_CORE_BLOCK_LAYERS = 8
FLAGSHIP_RECURRENCE_TRAIN_MEAN = 3.0
FLAGSHIP_RECURRENCE_MAX = 16
FLAGSHIP_VOCAB_SIZE = 256_000
FLAGSHIP_MAX_CONTEXT = 16_384
FLAGSHIP_MAX_RACKS = 4
FLAGSHIP_TOTAL_PARAMS = 7_400_000_000_000
FLAGSHIP_UNIQUE_ACTIVE_PARAMS = 400_000_000_000
FLAGSHIP_COMPUTE_ACTIVE_PARAMS = 450_000_000_000


def flagship_config() -> ModelConfig:
    return ModelConfig(
        d_model=FLAGSHIP_D_MODEL, n_layers=FLAGSHIP_N_LAYERS, n_dense=FLAGSHIP_N_DENSE,
        n_moe=FLAGSHIP_N_MOE, n_linear_attn=FLAGSHIP_N_LINEAR_ATTN, n_mla=FLAGSHIP_N_MLA,
        n_routed_experts=FLAGSHIP_N_ROUTED_EXPERTS, n_shared_experts=FLAGSHIP_N_SHARED_EXPERTS,
        top_k=FLAGSHIP_TOP_K, expert_hidden=FLAGSHIP_EXPERT_HIDDEN, mtp_heads=FLAGSHIP_MTP_HEADS,
        core_block_layers=FLAGSHIP_CORE_BLOCK_LAYERS,
        recurrence_train_mean=FLAGSHIP_RECURRENCE_TRAIN_MEAN,
        recurrence_max=FLAGSHIP_RECURRENCE_MAX, vocab_size=FLAGSHIP_VOCAB_SIZE,
        max_context=FLAGSHIP_MAX_CONTEXT, max_racks=FLAGSHIP_MAX_RACKS,
    )


def tiny_config() -> ModelConfig:
    """CPU stand-in (~10M): 8 layers, 3:1 linear/MLA, 1 dense + 7 MoE, 8 routed + 2 shared
    experts, top-2, 2 MTP heads, core block 2, vocab 256, context 128."""
    return ModelConfig(
        d_model=128, n_layers=8, n_dense=1, n_moe=7, n_linear_attn=6, n_mla=2,
        n_routed_experts=8, n_shared_experts=2, top_k=2, expert_hidden=256, mtp_heads=2,
        core_block_layers=2, recurrence_train_mean=FLAGSHIP_RECURRENCE_TRAIN_MEAN,
        recurrence_max=FLAGSHIP_RECURRENCE_MAX, vocab_size=256, max_context=128,
        max_racks=FLAGSHIP_MAX_RACKS, prelude_layers=3, coda_layers=3, adapter_hidden=128,
    )


# ---------------------------------------------------------------------------
# The five B200 training configurations
# ---------------------------------------------------------------------------
def config_tiny_fp32() -> ModelConfig:
    """4 layers, d=256, delta-rule attention 4 heads x 64 (chunk 64) on every layer, MoE FFN
    with 8 experts top-2 hidden 512, vocab 32768, muP-scaled N(0, 0.02) init."""
    return ModelConfig(
        d_model=256, n_layers=4, n_dense=0, n_moe=4, n_linear_attn=4, n_mla=0,
        n_routed_experts=8, n_shared_experts=0, top_k=2, expert_hidden=512, mtp_heads=0,
        core_block_layers=4, recurrence_train_mean=1.0, recurrence_max=1, vocab_size=32768,
        max_context=512, prelude_layers=0, coda_layers=0, adapter_hidden=256,
        n_heads=4, d_head=64, softmax_every=0, delta_beta="sigmoid", chunk=64,
        mup_base_width=256,
    )


def config_dense_1p3b(max_context: int = 4096) -> ModelConfig:
    """24 layers, d=2048; delta rule 16 heads x 128 (sigmoid beta, L2-normed q/k); every 4th
    layer softmax GQA 16 query / 4 KV heads + RoPE; SwiGLU 5632; vocab 131072."""
    return ModelConfig(
        d_model=2048, n_layers=24, n_dense=24, n_moe=0, n_linear_attn=18, n_mla=6,
        n_routed_experts=1, n_shared_experts=0, top_k=1, expert_hidden=5632, mtp_heads=0,
        core_block_layers=24, recurrence_train_mean=1.0, recurrence_max=1, vocab_size=131072,
        max_context=max_context, prelude_layers=0, coda_layers=0, adapter_hidden=2048,
        n_heads=16, d_head=128, n_kv_heads=4, softmax_kind="gqa", softmax_every=4,
        delta_beta="sigmoid", chunk=64, dense_hidden=5632, mup_base_width=2048,
    )


def config_moe_16b() -> ModelConfig:
    """28 layers, d=2048; 64 routed experts hidden 1408 top-6 + 2 shared, sigmoid router;
    attention as in the dense config; block-scaled FP8 linears are a TrainConfig choice."""
    return ModelConfig(
        d_model=2048, n_layers=28, n_dense=1, n_moe=27, n_linear_attn=21, n_mla=7,
        n_routed_experts=64, n_shared_experts=2, top_k=6, expert_hidden=1408, mtp_heads=0,
        core_block_layers=28, recurrence_train_mean=1.0, recurrence_max=1, vocab_size=131072,
        max_context=4096, max_racks=8, prelude_layers=0, coda_layers=0, adapter_hidden=2048,
        n_heads=16, d_head=128, n_kv_heads=4, softmax_kind="gqa", softmax_every=4,
        delta_beta="sigmoid", chunk=64, dense_hidden=5632, router_bias=True,
        mup_base_width=2048,
    )


def config_long_context() -> ModelConfig:
    """The 1.3B hybrid at sequence length 131072 (context-parallel over 8 ranks)."""
    return config_dense_1p3b(max_context=131072)


def config_latent() -> ModelConfig:
    """The 1.3B hybrid for latent-reasoning continued training (1024 + 8 + 512 tokens)."""
    return config_dense_1p3b(max_context=2048)


BASELINE_CONFIGS = {
    "tiny_fp32": config_tiny_fp32,
    "dense_1p3b": config_dense_1p3b,
    "moe_16b": config_moe_16b,
    "long_context": config_long_context,
    "latent": config_latent,
}


@dataclass(frozen=True)
class ForwardOutput:
    """Next-token logits plus MTP heads and the router aux used in the loss."""

    logits: Tensor
    mtp_logits: tuple
    z_loss: Tensor
    router_probs: Tensor
    expert_ids: Tensor
    hidden: Tensor
    r_used: int


# ---------------------------------------------------------------------------
# small numerics
# ---------------------------------------------------------------------------
def _f32(x: Any, like: Tensor | None = None) -> Tensor:
    if isinstance(x, Tensor):
        return x if x.dtype == torch.float32 else x.float()
    dev = like.device if like is not None else None
    return torch.as_tensor(np.asarray(x), dtype=torch.float32, device=dev)


def _silu(x: Tensor) -> Tensor:
    x = _f32(x)
    return x * (1.0 / (1.0 + torch.exp(-torch.clamp(x, -80.0, 80.0))))


def _sigmoid(x: Tensor) -> Tensor:
    x = _f32(x)
    return 1.0 / (1.0 + torch.exp(-torch.clamp(x, -80.0, 80.0)))


def _softmax(x: Tensor, dim: int = -1) -> Tensor:
    x = _f32(x)
    x = x - x.amax(dim=dim, keepdim=True)
    e = torch.exp(x)
    return e / torch.clamp(e.sum(dim=dim, keepdim=True), min=1e-12)


def _l2_normalize(x: Tensor, eps: float = 1e-6) -> Tensor:
    n = torch.linalg.vector_norm(x, dim=-1, keepdim=True)
    return x / torch.clamp(n, min=eps)


def _attn_geometry(d_model: int) -> tuple[int, int, int, int]:
    """(n_heads, d_head, d_nope, d_rope) derived from d_model (reference rule)."""
    d_head = 1
    for cand in (64, 32, 16, 8, 4, 2, 1):
        if d_model % cand == 0:
            d_head = cand
            break
    n_heads = d_model // d_head
    d_nope = d_head
    d_rope = (d_head // 2) // 2 * 2
    if d_rope < 2:
        d_rope = 2 if d_head >= 2 else d_head
    return n_heads, d_head, d_nope, d_rope


def head_geometry(config: ModelConfig) -> tuple[int, int, int]:
    """(n_heads, d_head, n_kv_heads) honouring explicit fields when present."""
    if config.n_heads is not None and config.d_head is not None:
        nh, dh = int(config.n_heads), int(config.d_head)
    else:
        nh, dh, _, _ = _attn_geometry(config.d_model)
    nkv = int(config.n_kv_heads) if config.n_kv_heads is not None else nh
    return nh, dh, nkv


def _recurrent_split(config: ModelConfig) -> tuple[int, int, int]:
    """Prelude / core / coda unique-layer counts. Sum equals n_layers."""
    core = int(config.core_block_layers)
    if core < 1 or core > config.n_layers:
        raise ConfigError("core_block_layers out of range")
    if config.prelude_layers is not None and config.coda_layers is not None:
        prelude, coda = int(config.prelude_layers), int(config.coda_layers)
        if prelude + core + coda != config.n_layers:
            raise ConfigError("prelude + core + coda must equal n_layers")
        if prelude < 0 or coda < 0:
            raise ConfigError("prelude_layers and coda_layers must be >= 0")
        return prelude, core, coda
    rest = config.n_layers - core
    prelude = rest // 2
    return prelude, core, rest - prelude


def validate_config(config: ModelConfig) -> None:
    """Raise ConfigError if counts or the hybrid ratio do not hold."""
    if config.n_layers < 1:
        raise ConfigError("n_layers must be >= 1")
    if config.n_dense + config.n_moe != config.n_layers:
        raise ConfigError("n_dense + n_moe must equal n_layers")
    if config.n_linear_attn + config.n_mla != config.n_layers:
        raise ConfigError("n_linear_attn + n_mla must equal n_layers")
    period = int(config.softmax_every)
    if period < 0:
        raise ConfigError("softmax_every must be >= 0")
    if period == 0:
        if config.n_mla != 0:
            raise ConfigError("softmax_every=0 requires n_mla == 0")
    else:
        if config.n_layers % period != 0:
            raise ConfigError("n_layers must be a multiple of the 3:1 hybrid period")
        if config.n_mla * (period - 1) != config.n_linear_attn:
            raise ConfigError("hybrid attention must be 3 linear : 1 MLA")
    if config.n_dense < 0 or config.n_moe < 0:
        raise ConfigError("n_dense and n_moe must be >= 0")
    for name in ("d_model", "vocab_size", "max_context", "n_routed_experts", "top_k",
                 "expert_hidden", "core_block_layers", "max_racks"):
        if getattr(config, name) < 1:
            raise ConfigError(f"{name} must be >= 1")
    if config.n_shared_experts < 0:
        raise ConfigError("n_shared_experts must be >= 0")
    if config.top_k > config.n_routed_experts:
        raise ConfigError("top_k cannot exceed n_routed_experts")
    if config.mtp_heads < 0:
        raise ConfigError("mtp_heads must be >= 0")
    if config.recurrence_max < 1:
        raise ConfigError("recurrence_max must be >= 1")
    if config.recurrence_train_mean <= 0:
        raise ConfigError("recurrence_train_mean must be > 0")
    if config.adapter_hidden is not None and config.adapter_hidden < 1:
        raise ConfigError("adapter_hidden must be >= 1")
    if config.softmax_kind not in ("mla", "gqa"):
        raise ConfigError("softmax_kind must be 'mla' or 'gqa'")
    if config.delta_beta not in ("one", "sigmoid"):
        raise ConfigError("delta_beta must be 'one' or 'sigmoid'")
    if (config.n_heads is None) != (config.d_head is None):
        raise ConfigError("n_heads and d_head must be given together")
    nh, dh, nkv = head_geometry(config)
    if nkv < 1 or nh % nkv != 0:
        raise ConfigError("n_heads must be a multiple of n_kv_heads")
    if config.softmax_kind == "gqa" and dh % 2 != 0:
        raise ConfigError("GQA with RoPE needs an even d_head")
    _recurrent_split(config)


def attention_kind(layer_index: int, config: ModelConfig) -> AttentionKind:
    """Linear vs softmax layer, starting at linear. Raises AttentionKindError if OOB."""
    if layer_index < 0 or layer_index >= config.n_layers:
        raise AttentionKindError(f"layer_index {layer_index} outside [0, {config.n_layers})")
    period = int(config.softmax_every)
    if period > 0 and layer_index % period == period - 1:
        return AttentionKind.GQA if config.softmax_kind == "gqa" else AttentionKind.MLA
    return AttentionKind.LINEAR


def ffn_kind(layer_index: int, config: ModelConfig) -> FfnKind:
    """First n_dense layers are dense; the rest are MoE."""
    if layer_index < 0 or layer_index >= config.n_layers:
        raise ConfigError(f"layer_index {layer_index} outside [0, {config.n_layers})")
    return FfnKind.DENSE if layer_index < config.n_dense else FfnKind.MOE


def rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    x = _f32(x)
    weight = _f32(weight, x)
    ms = torch.mean(torch.square(x), dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ms + eps)) * weight


# ---------------------------------------------------------------------------
# RoPE (interleaved even/odd pairs)
# ---------------------------------------------------------------------------
def _rope_angles(positions: Tensor, n_rot: int, rot_dim: int, x: Tensor, base: float) -> Tensor:
    inv_freq = torch.tensor(float(base), dtype=torch.float32, device=x.device) ** (
        -2.0 * torch.arange(n_rot, dtype=torch.float32, device=x.device) / float(rot_dim))
    pos = _f32(positions, x).to(x.device)
    if pos.ndim == 1:
        angle = pos[:, None] * inv_freq
        if x.ndim == 2:
            return angle
        if x.ndim == 3:
            return angle[None, :, :]
        if x.ndim == 4:
            return angle[None, :, None, :]
        raise ValueError(f"unsupported rank {x.ndim} for rope")
    if pos.ndim == 2:
        angle = pos[:, :, None] * inv_freq
        if x.ndim == 3:
            return angle
        if x.ndim == 4:
            return angle[:, :, None, :]
        raise ValueError(f"unsupported rank {x.ndim} for 2-D positions")
    raise ValueError("positions must be (seq,) or (batch, seq)")


def _apply_rope(x: Tensor, positions: Tensor, *, partial: bool, base: float = ROPE_BASE) -> Tensor:
    x = _f32(x)
    d = int(x.shape[-1])
    n_pairs = d // 2
    if n_pairs == 0:
        return x
    n_rot = n_pairs if not partial else max(1, n_pairs // 2)
    rot_dim = n_rot * 2
    rotated, passthrough = x[..., :rot_dim], x[..., rot_dim:]
    even, odd = rotated[..., 0::2], rotated[..., 1::2]
    angle = _rope_angles(positions, n_rot, rot_dim, x, base)
    cos, sin = torch.cos(angle), torch.sin(angle)
    out_rot = torch.stack([even * cos - odd * sin, even * sin + odd * cos], dim=-1)
    out_rot = out_rot.reshape(rotated.shape)
    if passthrough.shape[-1] == 0:
        return out_rot
    return torch.cat([out_rot, passthrough], dim=-1)


def rope(q: Tensor, k: Tensor, positions: Tensor, *, partial: bool = True,
         base: float = ROPE_BASE) -> tuple[Tensor, Tensor]:
    """RoPE on q and k. ``partial`` rotates only the first half of the pairs."""
    return (_apply_rope(q, positions, partial=partial, base=base),
            _apply_rope(k, positions, partial=partial, base=base))


def rope_2d(q: Tensor, k: Tensor, row: Tensor, col: Tensor) -> tuple[Tensor, Tensor]:
    """2-D RoPE on grid spans: first half of the head dim by row, second half by column."""
    q, k = _f32(q), _f32(k)
    d = int(q.shape[-1])
    if d % 2 != 0:
        raise ValueError("rope_2d requires an even last dimension")
    half = d // 2
    q1, k1 = rope(q[..., :half], k[..., :half], row, partial=False)
    q2, k2 = rope(q[..., half:], k[..., half:], col, partial=False)
    return torch.cat([q1, q2], dim=-1), torch.cat([k1, k2], dim=-1)


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def _ensure_heads(x: Tensor) -> tuple[Tensor, bool]:
    x = _f32(x)
    if x.ndim == 3:
        return x[:, :, None, :], True
    if x.ndim == 4:
        return x, False
    raise ValueError(f"expected 3-D or 4-D tensor, got shape {tuple(x.shape)}")


def linear_attention(q: Tensor, k: Tensor, v: Tensor, state: Tensor | None = None,
                     beta: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """Delta-rule linear attention with L2-normalised q, k. Returns (output, next_state).

    Per token ``S = (I - b k k^T) S + b k v^T``, ``o = q S`` (post-update read).
    ``beta`` None is the reference's b = 1; otherwise ``(batch, seq, heads)`` gates.
    The scan itself is ``kernels.chunked_delta_rule`` (chunked WY form).
    """
    from . import kernels

    q, squeeze = _ensure_heads(q)
    k, _ = _ensure_heads(k)
    v, _ = _ensure_heads(v)
    if q.shape != k.shape or q.shape[:3] != v.shape[:3] or q.shape[-1] != v.shape[-1]:
        raise ValueError("q, k, v must share batch/seq/heads and key/value dim")
    batch, seq, heads, dim = q.shape
    qn, kn = _l2_normalize(q), _l2_normalize(k)
    if state is None:
        s0 = None
    else:
        s0 = _f32(state)
        if s0.ndim == 3:
            s0 = s0[:, None, :, :]
        if tuple(s0.shape) != (batch, heads, dim, dim):
            raise ValueError(f"state shape {tuple(s0.shape)} != {(batch, heads, dim, dim)}")
    if beta is None:
        b = torch.ones((batch, seq, heads), dtype=torch.float32, device=q.device)
    else:
        b = _f32(beta)
        if b.ndim == 2:
            b = b[:, :, None]
    out, s = kernels.chunked_delta_rule(qn, kn, v, b, initial_state=s0)
    if squeeze:
        return out[:, :, 0, :], s[:, 0, :, :]
    return out, s


def mla_attention(q: Tensor, compressed_kv: Tensor, rope_k: Tensor, *,
                  qk_norm: bool = True) -> Tensor:
    """MLA-style softmax attention (keys = [compressed ‖ rope], values = compressed)."""
    q, ckv, rk = _f32(q), _f32(compressed_kv), _f32(rope_k)
    if q.ndim != 4:
        raise ValueError(f"q must be 4-D, got {tuple(q.shape)}")
    if ckv.ndim == 3:
        ckv = ckv[:, :, None, :]
    if rk.ndim == 3:
        rk = rk[:, :, None, :]
    if ckv.ndim != 4 or rk.ndim != 4:
        raise ValueError("compressed_kv and rope_k must be 3-D or 4-D")
    batch, seq_q, n_heads, d_q = q.shape
    seq_k, d_nope, d_rope = ckv.shape[1], ckv.shape[-1], rk.shape[-1]
    if d_q != d_nope + d_rope:
        raise ValueError(f"q last dim {d_q} must equal d_nope ({d_nope}) + d_rope ({d_rope})")

    def _bcast(x: Tensor) -> Tensor:
        if x.shape[2] == n_heads:
            return x
        if x.shape[2] == 1:
            return x.expand(x.shape[0], x.shape[1], n_heads, x.shape[3])
        raise ValueError(f"cannot broadcast heads {x.shape[2]} to {n_heads}")

    ckv_h, rk_h = _bcast(ckv), _bcast(rk)
    k = torch.cat([ckv_h, rk_h], dim=-1)
    v = ckv_h
    if qk_norm:
        ones = torch.ones((d_q,), dtype=torch.float32, device=q.device)
        q, k = rms_norm(q, ones), rms_norm(k, ones)
    scale = 1.0 / math.sqrt(float(d_q))
    scores = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    q_idx = torch.arange(seq_q, device=q.device)[:, None]
    k_idx = torch.arange(seq_k, device=q.device)[None, :]
    causal = k_idx > (q_idx + (seq_k - seq_q))
    scores = torch.where(causal[None, None], torch.full_like(scores, -1e9), scores)
    attn = _softmax(scores, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", attn, v)


def gqa_attention(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """Causal softmax attention with grouped KV heads. q: (B,S,Hq,D); k, v: (B,S,Hkv,D).
    Scale 1/sqrt(D), mask sentinel -1e9 and softmax floor 1e-12 as in ``mla_attention``."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    if hq % hkv != 0:
        raise ValueError("query heads must be a multiple of KV heads")
    g = hq // hkv
    kk = k.repeat_interleave(g, dim=2)
    vv = v.repeat_interleave(g, dim=2)
    scores = torch.einsum("bqhd,bkhd->bhqk", q, kk) * (1.0 / math.sqrt(float(d)))
    q_idx = torch.arange(sq, device=q.device)[:, None]
    k_idx = torch.arange(sk, device=q.device)[None, :]
    causal = k_idx > (q_idx + (sk - sq))
    scores = torch.where(causal[None, None], torch.full_like(scores, -1e9), scores)
    return torch.einsum("bhqk,bkhd->bqhd", _softmax(scores, dim=-1), vv)


# ---------------------------------------------------------------------------
# MoE
# ---------------------------------------------------------------------------
def _expert_to_rack(n_experts: int, max_racks: int, device=None) -> Tensor:
    n_racks = max(min(int(max_racks), int(n_experts)), 1)
    e = torch.arange(n_experts, dtype=torch.int64, device=device)
    return torch.clamp(e * n_racks // n_experts, max=n_racks - 1)


def _node_limited_topk(scores: Tensor, top_k: int, max_racks: int) -> Tensor:
    """Top-k experts per token touching at most ``max_racks`` racks, then fill any
    remaining slots by score. Ties break toward the lower expert index (stable sort).
    When the rack limit cannot bind (racks <= max_racks) this is a plain stable top-k."""
    n_tok, n_exp = scores.shape
    n_racks = max(min(int(max_racks), n_exp), 1)
    order = torch.argsort(-scores, dim=-1, stable=True)
    if n_racks <= int(max_racks):
        return order[:, :top_k].to(torch.int32)
    racks = _expert_to_rack(n_exp, max_racks, scores.device)
    order_c, racks_c = order.cpu().numpy(), racks.cpu().numpy()
    out = np.full((n_tok, top_k), -1, dtype=np.int32)
    for t in range(n_tok):
        used: set[int] = set()
        chosen: list[int] = []
        for e in order_c[t]:
            r = int(racks_c[e])
            if len(chosen) < top_k and (r in used or len(used) < max_racks):
                chosen.append(int(e))
                used.add(r)
        for e in order_c[t]:
            if len(chosen) >= top_k:
                break
            if int(e) not in chosen:
                chosen.append(int(e))
        out[t] = chosen[:top_k]
    return torch.as_tensor(out, device=scores.device)


def _swiglu(x: Tensor, w_gate: Tensor, w_up: Tensor, w_down: Tensor) -> Tensor:
    return (_silu(x @ w_gate) * (x @ w_up)) @ w_down


def moe(x: Tensor, *, router_weight: Tensor, routed_weights, shared_weights, top_k: int,
        max_racks: int = FLAGSHIP_MAX_RACKS, router_bias: Tensor | None = None):
    """Sigmoid gates, top-k routed + shared experts, node-limited routing.

    Returns (output, router_probs, expert_ids). Tokens are grouped per expert
    (sort + segment matmul) instead of gathering a weight copy per token, so it
    scales to 64 experts; the result equals the per-token formulation. ``router_bias``
    (aux-loss-free balancing) shifts the selection scores only, never the gates.
    """
    x = _f32(x)
    orig = x.shape
    d_model = orig[-1]
    flat = x.reshape(-1, d_model)
    probs = _sigmoid(flat @ _f32(router_weight, x))
    select = probs if router_bias is None else probs + _f32(router_bias, x)
    expert_ids = _node_limited_topk(select.detach(), int(top_k), int(max_racks)).long()
    top_scores = torch.gather(probs, 1, expert_ids)
    gates = top_scores / torch.clamp(top_scores.sum(dim=-1, keepdim=True), min=1e-9)
    w_gate, w_up, w_down = (_f32(t, x) for t in routed_weights)
    n_tok = flat.shape[0]
    flat_ids = expert_ids.reshape(-1)
    order = torch.argsort(flat_ids, stable=True)
    tok_of = (order // int(top_k))
    counts = torch.bincount(flat_ids, minlength=w_gate.shape[0]).tolist()
    xs = flat[tok_of]
    gs = gates.reshape(-1)[order]
    outs = []
    start = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        seg = xs[start:start + c]
        outs.append(_swiglu(seg, w_gate[e], w_up[e], w_down[e]))
        start += c
    routed = torch.cat(outs, dim=0) * gs[:, None] if outs else xs * 0.0
    out = torch.zeros_like(flat).index_add(0, tok_of, routed)
    s_gate, s_up, s_down = (_f32(t, x) for t in shared_weights)
    for j in range(int(s_gate.shape[0])):
        out = out + _swiglu(flat, s_gate[j], s_up[j], s_down[j])
    router_probs = probs.reshape(*orig[:-1], probs.shape[-1])
    ids = expert_ids.reshape(*orig[:-1], int(top_k)).to(torch.int32)
    del n_tok
    return out.reshape(orig), router_probs, ids


def _apply_latent_adapter(x: Tensor, w1: Tensor, w2: Tensor, norm_weight: Tensor) -> Tensor:
    x = _f32(x)
    h = _silu(x @ _f32(w1, x)) @ _f32(w2, x)
    return rms_norm(h, norm_weight)


def latent_adapter(x: Tensor, *, hidden: int) -> Tensor:
    """2-layer MLP + norm with identity-like weights (maps a thought into the residual stream)."""
    x = _f32(x)
    d = int(x.shape[-1])
    inv = 1.0 / math.sqrt(max(int(hidden), 1))
    w1 = torch.eye(d, int(hidden), dtype=torch.float32, device=x.device) * inv
    w2 = torch.eye(int(hidden), d, dtype=torch.float32, device=x.device) * inv
    return _apply_latent_adapter(x, w1, w2, torch.ones((d,), dtype=torch.float32, device=x.device))


# ---------------------------------------------------------------------------
# parameters
# ---------------------------------------------------------------------------
def _generator(rng: Any) -> torch.Generator:
    if isinstance(rng, torch.Generator):
        return rng
    g = torch.Generator(device="cpu")
    if rng is None:
        g.manual_seed(0)
    elif isinstance(rng, (int, np.integer)):
        g.manual_seed(int(rng))
    elif isinstance(rng, np.random.Generator):
        g.manual_seed(int(rng.integers(0, 2**31 - 1)))
    else:
        raise TypeError("rng must be None, an int, a numpy Generator or a torch Generator")
    return g


def init_params(config: ModelConfig, rng: Any, *, device=None, dtype=torch.float32,
                shapes_only: bool = False) -> dict:
    """Parameter tree with the reference's names. Matrices ~ N(0, init_scale^2) (hidden
    matrices scaled by sqrt(mup_base_width / d_model) when muP is on), norms = 1.
    ``shapes_only`` returns the same tree of meta tensors (no memory, no random numbers): the
    layout a trainer plans from before it initialises its own shards with ``init_leaf``."""
    validate_config(config)
    gen = None if shapes_only else _generator(rng)
    d = config.d_model
    n_heads, d_head, n_kv = head_geometry(config)
    _, _, d_nope, d_rope = _attn_geometry(d)
    if config.n_heads is not None:
        d_nope = d_head
        d_rope = max(2, (d_head // 2) // 2 * 2)
    kv_rank = d_head
    hidden = config.expert_hidden
    dense_hidden = config.dense_hidden if config.dense_hidden is not None else hidden
    adapter_h = config.adapter_hidden if config.adapter_hidden is not None else d
    std = float(config.init_scale)
    hid_std = std
    if config.mup_base_width is not None:
        hid_std = std * math.sqrt(float(config.mup_base_width) / float(d))

    def w(shape, s=None) -> Tensor:
        if shapes_only:
            return torch.empty(shape, dtype=dtype, device="meta")
        t = torch.randn(shape, generator=gen, dtype=torch.float32) * (hid_std if s is None else s)
        return t.to(device=device, dtype=dtype)

    def ones(n) -> Tensor:
        if shapes_only:
            return torch.empty((n,), dtype=dtype, device="meta")
        return torch.ones((n,), dtype=dtype, device=device)

    layers = []
    for i in range(config.n_layers):
        layer = {"pre_attn_norm": ones(d), "pre_ffn_norm": ones(d)}
        kind = attention_kind(i, config)
        if kind is AttentionKind.LINEAR:
            layer["W_q"] = w((d, n_heads, d_head))
            layer["W_k"] = w((d, n_heads, d_head))
            layer["W_v"] = w((d, n_heads, d_head))
            layer["W_o"] = w((n_heads, d_head, d))
            if config.delta_beta == "sigmoid":
                layer["W_beta"] = w((d, n_heads))
        elif kind is AttentionKind.GQA:
            layer["W_q"] = w((d, n_heads, d_head))
            layer["W_k"] = w((d, n_kv, d_head))
            layer["W_v"] = w((d, n_kv, d_head))
            layer["W_o"] = w((n_heads, d_head, d))
        else:
            layer["W_q"] = w((d, n_heads, d_nope + d_rope))
            layer["W_kv_compress"] = w((d, kv_rank))
            layer["W_kv_up"] = w((kv_rank, n_heads, d_nope))
            layer["W_rope_k"] = w((d, d_rope))
            layer["W_o"] = w((n_heads, d_nope, d))
        if ffn_kind(i, config) is FfnKind.DENSE:
            layer["ffn_gate"] = w((d, dense_hidden))
            layer["ffn_up"] = w((d, dense_hidden))
            layer["ffn_down"] = w((dense_hidden, d))
        else:
            n_r, n_s = config.n_routed_experts, config.n_shared_experts
            layer["router"] = w((d, n_r))
            if config.router_bias:
                layer["router_bias"] = torch.zeros((n_r,), dtype=dtype, device="meta" if shapes_only else device)
            layer["routed_gate"] = w((n_r, d, hidden))
            layer["routed_up"] = w((n_r, d, hidden))
            layer["routed_down"] = w((n_r, hidden, d))
            layer["shared_gate"] = w((n_s, d, hidden))
            layer["shared_up"] = w((n_s, d, hidden))
            layer["shared_down"] = w((n_s, hidden, d))
        layers.append(layer)
    mtp = []
    for _ in range(config.mtp_heads):
        mtp.append({"norm": ones(d), "proj": w((d, d)), "unembed": w((config.vocab_size, d), std)})
    return {
        "embed": w((config.vocab_size, d), std),
        "unembed": w((config.vocab_size, d), std),
        "final_norm": ones(d),
        "layers": layers,
        "mtp": mtp,
        "adapter_w1": w((d, adapter_h)),
        "adapter_w2": w((adapter_h, d)),
        "adapter_norm": ones(d),
    }


def init_leaf(config: ModelConfig, name: str, shape, seed: int, device) -> Tensor:
    """One leaf of the parameter tree, initialised on ``device`` from a generator keyed by
    ``(seed, name)``: norms are ones, ``router_bias`` zeros, embeddings N(0, init_scale^2), every
    other matrix N(0, (init_scale * sqrt(mup_base_width / d_model))^2). Same distribution as
    ``init_params`` (not the same numbers: that one draws every leaf from a single CPU stream);
    used for models too large to initialise on the host and for expert-parallel ranks, which only
    create the experts they own."""
    import zlib

    leaf = name.rsplit(".", 1)[-1]
    if leaf.endswith("norm"):
        return torch.ones(tuple(shape), dtype=torch.float32, device=device)
    if leaf == "router_bias":
        return torch.zeros(tuple(shape), dtype=torch.float32, device=device)
    std = float(config.init_scale)
    if leaf not in ("embed", "unembed") and config.mup_base_width is not None:
        std *= math.sqrt(float(config.mup_base_width) / float(config.d_model))
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
    return torch.randn(tuple(shape), generator=gen, dtype=torch.float32, device=device) * std


def param_count(params: Any) -> int:
    n = 0
    if isinstance(params, dict):
        for v in params.values():
            n += param_count(v)
    elif isinstance(params, (list, tuple)):
        for v in params:
            n += param_count(v)
    elif hasattr(params, "numel"):
        n += int(params.numel())
    elif hasattr(params, "size"):
        n += int(params.size)
    return n


def flatten_params(params: Any, prefix: str = "") -> dict[str, Tensor]:
    """Dotted-name view of the tree (``layers.3.W_q``), the naming used by checkpoints."""
    out: dict[str, Tensor] = {}
    if isinstance(params, dict):
        for k, v in params.items():
            out.update(flatten_params(v, f"{prefix}.{k}" if prefix else str(k)))
    elif isinstance(params, (list, tuple)):
        for i, v in enumerate(params):
            out.update(flatten_params(v, f"{prefix}.{i}" if prefix else str(i)))
    else:
        out[prefix] = params
    return out


def unflatten_params(flat: dict[str, Tensor]) -> dict:
    """Inverse of ``flatten_params`` (integer path components become list indices)."""
    root: dict = {}
    for name, val in flat.items():
        parts = name.split(".")
        node = root
        for i, p in enumerate(parts[:-1]):
            node = node.setdefault(p, {})
        node[parts[-1]] = val

    def fix(node):
        if isinstance(node, dict):
            node = {k: fix(v) for k, v in node.items()}
            if node and all(k.isdigit() for k in node):
                return [node[str(i)] for i in range(len(node))]
        return node

    return fix(root)


# ---------------------------------------------------------------------------
# blocks and forward
# ---------------------------------------------------------------------------
def _dense_ffn(x: Tensor, layer: dict) -> Tensor:
    return _swiglu(x, _f32(layer["ffn_gate"]), _f32(layer["ffn_up"]), _f32(layer["ffn_down"]))


def _linear_attn(x: Tensor, layer: dict, state: Tensor | None) -> tuple[Tensor, Tensor]:
    q = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_q"]))
    k = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_k"]))
    v = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_v"]))
    beta = None
    if "W_beta" in layer:
        beta = _sigmoid(torch.einsum("bsd,dh->bsh", x, _f32(layer["W_beta"])))
    y, state = linear_attention(q, k, v, state, beta=beta)
    return torch.einsum("bshe,hed->bsd", y, _f32(layer["W_o"])), state


def _mla_attn(x: Tensor, layer: dict, positions: Tensor, base: float) -> Tensor:
    q = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_q"]))
    ckv = torch.einsum("bsd,dc->bsc", x, _f32(layer["W_kv_compress"]))
    k_nope = torch.einsum("bsc,che->bshe", ckv, _f32(layer["W_kv_up"]))
    rope_k = torch.einsum("bsd,dr->bsr", x, _f32(layer["W_rope_k"]))
    d_nope = k_nope.shape[-1]
    q_nope, q_rope = q[..., :d_nope], q[..., d_nope:]
    rk = rope_k[:, :, None, :].expand(q_rope.shape)
    q_rope, rk = rope(q_rope, rk, positions, partial=False, base=base)
    q = torch.cat([q_nope, q_rope], dim=-1)
    y = mla_attention(q, k_nope, rk, qk_norm=True)
    return torch.einsum("bshe,hed->bsd", y, _f32(layer["W_o"]))


def _gqa_attn(x: Tensor, layer: dict, positions: Tensor, base: float) -> Tensor:
    q = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_q"]))
    k = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_k"]))
    v = torch.einsum("bsd,dhe->bshe", x, _f32(layer["W_v"]))
    q, k = rope(q, k, positions, partial=False, base=base)
    y = gqa_attention(q, k, v)
    return torch.einsum("bshe,hed->bsd", y, _f32(layer["W_o"]))


def _block(h: Tensor, layer: dict, config: ModelConfig, layer_index: int, positions: Tensor,
           lin_state: Tensor | None):
    """One pre-norm block. Returns h, lin_state, router_logits, probs, ids."""
    n = rms_norm(h, layer["pre_attn_norm"])
    kind = attention_kind(layer_index, config)
    if kind is AttentionKind.LINEAR:
        attn, lin_state = _linear_attn(n, layer, lin_state)
    elif kind is AttentionKind.GQA:
        attn, lin_state = _gqa_attn(n, layer, positions, config.rope_base), None
    else:
        attn, lin_state = _mla_attn(n, layer, positions, config.rope_base), None
    h = h + attn
    n = rms_norm(h, layer["pre_ffn_norm"])
    router_logits = router_probs = expert_ids = None
    if ffn_kind(layer_index, config) is FfnKind.DENSE:
        h = h + _dense_ffn(n, layer)
    else:
        routed = (layer["routed_gate"], layer["routed_up"], layer["routed_down"])
        shared = (layer["shared_gate"], layer["shared_up"], layer["shared_down"])
        y, router_probs, expert_ids = moe(
            n, router_weight=layer["router"], routed_weights=routed, shared_weights=shared,
            top_k=config.top_k, max_racks=config.max_racks,
            router_bias=layer.get("router_bias"))
        router_logits = n.reshape(-1, n.shape[-1]) @ _f32(layer["router"])
        h = h + y
    return h, lin_state, router_logits, router_probs, expert_ids


def _sample_r(config: ModelConfig, tokens: Tensor) -> int:
    seed = int(tokens.sum().item()) % (2**31)
    rng = np.random.default_rng(seed)
    mean = float(config.recurrence_train_mean)
    max_r = int(config.recurrence_max)
    p = min(max(1.0 / mean, 1e-6), 0.999)
    for _ in range(64):
        u = float(rng.random())
        k = int(np.floor(np.log(max(1.0 - u, 1e-12)) / np.log(1.0 - p))) + 1
        if 1 <= k <= max_r:
            return k
    return min(max_r, max(1, int(round(mean))))


def embed_tokens(tokens: Tensor, params: dict, config: ModelConfig,
                 thoughts: Tensor | None = None, inputs_embeds: Tensor | None = None):
    """Input embeddings (+ adapter-mapped thoughts prepended). Returns (h, n_thoughts)."""
    h = _f32(params["embed"])[tokens.long()] if inputs_embeds is None else _f32(inputs_embeds)
    n_thoughts = 0
    if thoughts is not None:
        th = _f32(thoughts)
        if th.ndim != 3 or th.shape[0] != tokens.shape[0]:
            raise ValueError("thoughts must be (batch, n_thoughts, d_model)")
        if th.shape[-1] != config.d_model:
            raise ValueError("thoughts last dim must equal d_model")
        n_thoughts = int(th.shape[1])
        if n_thoughts:
            adapted = _apply_latent_adapter(th, params["adapter_w1"], params["adapter_w2"],
                                            params["adapter_norm"])
            h = torch.cat([adapted, h], dim=1)
    return h, n_thoughts


def forward(tokens: Tensor, params: dict, config: ModelConfig, *, r: int | None = None,
            thoughts: Tensor | None = None, truncated_recurrence: int = TRUNCATED_RECURRENCE,
            inputs_embeds: Tensor | None = None) -> ForwardOutput:
    """FP32 forward of the whole model.

    ``r`` is the core-block iteration count (None: sampled from the heavy-tailed training
    distribution). Iteration 0 runs the core block on the prelude output; each later
    iteration adds that prelude output back (input injection) first. Backward flows only
    through the last ``min(truncated_recurrence, r)`` core iterations: the carry entering
    that window is detached, the injected prelude output is not. ``thoughts``
    ``(batch, n, d_model)`` are adapter-mapped and prepended; outputs drop those positions.
    ``inputs_embeds`` replaces the embedding lookup (used by the latent Jacobi solve).
    """
    validate_config(config)
    if type(truncated_recurrence) is not int or truncated_recurrence < 1:
        raise ConfigError("truncated_recurrence must be an int >= 1")
    tokens = torch.as_tensor(tokens)
    if tokens.ndim != 2:
        raise ValueError("tokens must be (batch, seq)")
    batch, seq = int(tokens.shape[0]), int(tokens.shape[1])
    if seq > config.max_context:
        raise ConfigError("sequence longer than max_context")
    if tokens.numel() and bool(((tokens < 0) | (tokens >= config.vocab_size)).any()):
        raise ConfigError("token id out of vocab")
    dev = params["embed"].device
    tokens = tokens.to(dev)
    h, n_thoughts = embed_tokens(tokens, params, config, thoughts, inputs_embeds)
    full_seq = int(h.shape[1])
    positions = torch.arange(full_seq, dtype=torch.float32, device=dev)
    r_used = int(r) if r is not None else _sample_r(config, tokens)
    if r_used < 1:
        raise ConfigError("r must be >= 1")
    prelude, core, coda = _recurrent_split(config)
    z_sum = torch.zeros((), dtype=torch.float32, device=dev)
    z_n = 0
    last_probs = torch.zeros((batch, full_seq, config.n_routed_experts), dtype=torch.float32,
                             device=dev)
    last_ids = torch.zeros((batch, full_seq, config.top_k), dtype=torch.int32, device=dev)

    def apply_range(carry, start: int, n: int):
        h_in, zs, zn, pr, ids = carry
        for j in range(n):
            h_in, _, logits, probs, eids = _block(h_in, params["layers"][start + j], config,
                                                  start + j, positions, None)
            if logits is not None:
                lse = torch.logsumexp(logits, dim=-1)
                zs = zs + torch.mean(torch.square(lse))
                zn = zn + 1
                pr, ids = probs, eids
        return h_in, zs, zn, pr, ids

    carry = apply_range((h, z_sum, z_n, last_probs, last_ids), 0, prelude)
    injected = carry[0]
    carry = apply_range(carry, prelude, core)

    def core_iter(c):
        return apply_range((c[0] + injected, *c[1:]), prelude, core)

    effective = min(truncated_recurrence, r_used)
    cut = r_used - effective
    if cut == 0:
        for _ in range(r_used - 1):
            carry = core_iter(carry)
    else:
        for _ in range(cut - 1):
            carry = core_iter(carry)
        carry = (carry[0].detach(), carry[1].detach(), carry[2], carry[3].detach(), carry[4])
        for _ in range(r_used - cut):
            carry = core_iter(carry)
    carry = apply_range(carry, prelude + core, coda)
    h, z_sum, z_n, last_probs, last_ids = carry

    h = rms_norm(h, params["final_norm"])
    hidden = h[:, n_thoughts:, :]
    logits = hidden @ _f32(params["unembed"]).T
    mtp_logits = []
    for head in params["mtp"]:
        mh = rms_norm(hidden, head["norm"])
        mh = mh @ _f32(head["proj"]) + hidden
        mtp_logits.append(mh @ _f32(head["unembed"]).T)
    z_loss = z_sum / float(z_n) if z_n > 0 else torch.zeros((), dtype=torch.float32, device=dev)
    return ForwardOutput(
        logits=logits, hidden=hidden, mtp_logits=tuple(mtp_logits),
        router_probs=last_probs[:, n_thoughts:, :], expert_ids=last_ids[:, n_thoughts:, :],
        z_loss=z_loss, r_used=r_used,
    )


def with_overrides(config: ModelConfig, **kw) -> ModelConfig:
    """Copy of a (frozen) config with some fields replaced."""
    return replace(config, **kw)
