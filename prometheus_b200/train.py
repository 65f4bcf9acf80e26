"""Training step on the parameter tree: losses, Muon / AdamW, WSD schedule, QK-clip.

This is the device-agnostic (plain PyTorch, fp32 masters) statement of one
optimizer step; ``prometheus_b200.engine.Trainer`` is the fused sm_100a
implementation of the same step for multi-GPU bf16/FP8 training and is tested
against this module.

API parity with the reference ``train/__init__.py``: ``TrainConfig`` (:112-133),
``flagship_train_config``/``tiny_train_config`` (:136-182), ``Batch``/
``LossBreakdown``/``StepOutput`` (:186-232), ``classify_param`` (:262),
``precision_for`` (:272), ``newton_schulz`` (:314), ``muon_update`` (:346),
``muon_rms_scale`` (:382), ``muon_transfer_step`` (:401), ``transferred_muon_lr``
(:461), ``qk_clip`` (:478), ``adamw_update`` (:503), ``wsd_lr`` (:542),
``soft_cap`` (:561), ``cross_entropy`` (:575), ``mtp_loss`` (:607), ``z_loss``
(:633), ``total_loss`` (:645), ``init_opt_state`` (:675), ``apply_precision``
(:691), ``train_step`` (:835).

Extensions (off by default so reference call sites behave the same):
``muon_all_matrices`` applies Muon to every matrix including head stacks
``(d, H, dh)`` and per-expert stacks ``(E, d, h)`` (the reference only updates
2-D leaves with Muon); ``r`` selects the core-block recurrence count;
``z_on_logits`` takes the router z-loss from the router logits returned by the
forward instead of from the sigmoid probabilities.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from enum import Enum
from typing import Any

import numpy as np
import torch

from . import model
from .model import ModelConfig

Tensor = torch.Tensor


class ParamKind(str, Enum):
    """Which optimizer a parameter takes. 2D hidden weights are Muon."""

    MUON_2D = "muon_2d"
    ADAMW = "adamw"

    def __str__(self) -> str:
        return self.value


class PrecisionKind(str, Enum):
    """Cast used in the forward, not the master-weight dtype."""

    FP8_LINEAR = "fp8_linear"
    BF16_STABLE = "bf16_stable"
    FP32_MASTER = "fp32_master"

    def __str__(self) -> str:
        return self.value


class TrainConfigError(ValueError):
    """TrainConfig violates an invariant."""


FLAGSHIP_PEAK_LR = 2.0e-4
FLAGSHIP_MUON_LR = 2.0e-2
FLAGSHIP_ADAMW_LR = 2.0e-4
FLAGSHIP_ADAMW_BETA1 = 0.9
FLAGSHIP_ADAMW_BETA2 = 0.95
FLAGSHIP_ADAMW_EPS = 1.0e-8
FLAGSHIP_ADAMW_WD = 0.1
FLAGSHIP_MUON_MOMENTUM = 0.95
FLAGSHIP_MUON_NS_STEPS = 5
FLAGSHIP_WARMUP_STEPS = 2_000
FLAGSHIP_STABLE_STEPS = 500_000
FLAGSHIP_DECAY_STEPS = 100_000
FLAGSHIP_Z_LOSS_WEIGHT = 1.0e-3
FLAGSHIP_SOFTCAP = 30.0
FLAGSHIP_QK_CLIP = 100.0
FLAGSHIP_FP8_BLOCK = 128
FLAGSHIP_GRAD_CLIP = 1.0
FLAGSHIP_BF16_TAIL_LAYERS = 2
MOONLIGHT_UPDATE_RMS = 0.2

_NS_A, _NS_B, _NS_C = 3.4445, -4.7750, 2.0315
_NS_EPS = 1e-7
_ADAMW_NAME_TOKS = ("embed", "norm", "bias", "sigma")
_BF16_NAME_TOKS = ("router", "norm", "embed", "adapter", "softmax", "sigma")


@dataclass(frozen=True)
class TrainConfig:
    peak_lr: float
    muon_lr: float
    adamw_lr: float
    adamw_beta1: float
    adamw_beta2: float
    adamw_eps: float
    adamw_wd: float
    muon_momentum: float
    muon_ns_steps: int
    warmup_steps: int
    stable_steps: int
    decay_steps: int
    z_loss_weight: float
    softcap: float
    qk_clip: float
    fp8_block: int
    grad_clip: float
    bf16_tail_layers: int
    n_layers: int


def flagship_train_config() -> TrainConfig:
    return TrainConfig(
        peak_lr=FLAGSHIP_PEAK_LR, muon_lr=FLAGSHIP_MUON_LR, adamw_lr=FLAGSHIP_ADAMW_LR,
        adamw_beta1=FLAGSHIP_ADAMW_BETA1, adamw_beta2=FLAGSHIP_ADAMW_BETA2,
        adamw_eps=FLAGSHIP_ADAMW_EPS, adamw_wd=FLAGSHIP_ADAMW_WD,
        muon_momentum=FLAGSHIP_MUON_MOMENTUM, muon_ns_steps=FLAGSHIP_MUON_NS_STEPS,
        warmup_steps=FLAGSHIP_WARMUP_STEPS, stable_steps=FLAGSHIP_STABLE_STEPS,
        decay_steps=FLAGSHIP_DECAY_STEPS, z_loss_weight=FLAGSHIP_Z_LOSS_WEIGHT,
        softcap=FLAGSHIP_SOFTCAP, qk_clip=FLAGSHIP_QK_CLIP, fp8_block=FLAGSHIP_FP8_BLOCK,
        grad_clip=FLAGSHIP_GRAD_CLIP, bf16_tail_layers=FLAGSHIP_BF16_TAIL_LAYERS, n_layers=96,
    )


def tiny_train_config() -> TrainConfig:
    """CPU stand-in: same discrete choices, short WSD, block 16, 8 layers."""
    base = flagship_train_config()
    return TrainConfig(**{**base.__dict__, "warmup_steps": 2, "stable_steps": 8,
                          "decay_steps": 4, "fp8_block": 16, "n_layers": 8})


def train_config_for(model_config: ModelConfig, **overrides) -> TrainConfig:
    """Flagship optimizer choices sized to ``model_config`` (layer count), with overrides."""
    base = flagship_train_config()
    fields = {**base.__dict__, "n_layers": int(model_config.n_layers),
              "bf16_tail_layers": min(FLAGSHIP_BF16_TAIL_LAYERS, int(model_config.n_layers))}
    fields.update(overrides)
    return TrainConfig(**fields)


@dataclass(frozen=True)
class Batch:
    """One packed training batch. Tokens are int; loss_mask is 0/1 float."""

    tokens: Tensor
    loss_mask: Tensor
    positions: Tensor


@dataclass(frozen=True)
class LossBreakdown:
    ce: Tensor
    mtp: Tensor
    z: Tensor
    total: Tensor


@dataclass(frozen=True)
class StepOutput:
    params: dict
    opt_state: dict
    loss: LossBreakdown
    lr: float
    grad_norm: Tensor
    step: int


def validate_train_config(config: TrainConfig) -> None:
    if min(float(config.peak_lr), float(config.muon_lr), float(config.adamw_lr)) <= 0:
        raise TrainConfigError("peak_lr, muon_lr, and adamw_lr must be > 0")
    total = int(config.warmup_steps) + int(config.stable_steps) + int(config.decay_steps)
    if total <= 0:
        raise TrainConfigError("warmup + stable + decay must be > 0")
    if int(config.bf16_tail_layers) > int(config.n_layers):
        raise TrainConfigError("bf16_tail_layers must be <= n_layers")


def _ndim(value: Any) -> int:
    return int(value.ndim) if hasattr(value, "ndim") else int(np.asarray(value).ndim)


def classify_param(name: str, value: Any) -> ParamKind:
    """2D hidden weights are Muon; embeddings, norms, biases, sigma are AdamW."""
    low = name.lower()
    if any(tok in low for tok in _ADAMW_NAME_TOKS):
        return ParamKind.ADAMW
    return ParamKind.MUON_2D if _ndim(value) == 2 else ParamKind.ADAMW


# How a stacked leaf splits into independent matrices for Muon: name suffix ->
# (number of leading batch axes, number of axes folded into the row dimension).
_STACK_RULES = {
    "W_q": (0, 1), "W_k": (0, 1), "W_v": (0, 1), "W_kv_up": (0, 1),   # (d, H, dh) -> d x (H dh)
    "W_o": (0, 2),                                                      # (H, dh, d) -> (H dh) x d
    "routed_gate": (1, 1), "routed_up": (1, 1), "routed_down": (1, 1),  # per expert
    "shared_gate": (1, 1), "shared_up": (1, 1), "shared_down": (1, 1),
}


def muon_matrix_view(name: str, shape) -> tuple[int, int, int] | None:
    """(batch, rows, cols) of the independent matrices inside a leaf, or None when the leaf
    is not a Muon parameter under the all-matrices rule (AdamW names, vectors, and
    matrices with a side below 32, e.g. the per-head beta projection)."""
    low = name.lower()
    if any(tok in low for tok in _ADAMW_NAME_TOKS):
        return None
    shape = tuple(int(s) for s in shape)
    leaf = name.split(".")[-1]
    if len(shape) == 2:
        b, r, c = 1, shape[0], shape[1]
    elif len(shape) == 3 and leaf in _STACK_RULES:
        nb, nrow = _STACK_RULES[leaf]
        if nb == 1:
            b, r, c = shape
        elif nrow == 1:
            b, r, c = 1, shape[0], shape[1] * shape[2]
        else:
            b, r, c = 1, shape[0] * shape[1], shape[2]
    else:
        return None
    if min(r, c) < 32:
        return None
    return b, r, c


def precision_for(name: str, config: TrainConfig) -> PrecisionKind:
    """FP8 on hidden linears; BF16 on router/norm/embed/softmax/tail/adapter."""
    low = name.lower()
    match = re.match(r"layers\.(\d+)\.", low)
    if match is not None and int(match.group(1)) >= int(config.n_layers) - int(config.bf16_tail_layers):
        return PrecisionKind.BF16_STABLE
    if any(tok in low for tok in _BF16_NAME_TOKS):
        return PrecisionKind.BF16_STABLE
    return PrecisionKind.FP8_LINEAR


def _f32(x: Any) -> Tensor:
    t = x if isinstance(x, Tensor) else torch.as_tensor(np.asarray(x))
    return t if t.dtype == torch.float32 else t.float()


def _positive_int(name: str, value: object) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, np.integer)) or int(value) < 1:
        raise ValueError(f"{name} must be an integer >= 1")
    return int(value)


def _finite_real(name: str, value: object) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float, np.integer, np.floating)):
        raise ValueError(name)
    f = float(value)
    if not math.isfinite(f):
        raise ValueError(name)
    return f


# ---------------------------------------------------------------------------
# Muon
# ---------------------------------------------------------------------------
def newton_schulz(matrix: Any, steps: int) -> Tensor:
    """Quintic Newton-Schulz orthogonalisation of a 2-D (or batched 3-D) matrix.
    ``X <- aX + (bG + cG^2) X`` with ``G = X X^T``; the input is transposed when it has
    more rows than columns and normalised by its Frobenius norm (zeros below 1e-7)."""
    if int(steps) < 1 or int(steps) % 2 == 0:
        raise ValueError("newton_schulz steps must be odd and >= 1")
    g = _f32(matrix)
    if g.ndim not in (2, 3):
        raise ValueError(f"newton_schulz expects a 2D matrix, got shape {tuple(g.shape)}")
    transposed = g.shape[-2] > g.shape[-1]
    x = g.transpose(-1, -2) if transposed else g
    fro = torch.linalg.matrix_norm(x, keepdim=True)
    x = torch.where(fro > _NS_EPS, x / torch.clamp(fro, min=_NS_EPS), torch.zeros_like(x))
    for _ in range(int(steps)):
        gram = x @ x.transpose(-1, -2)
        x = _NS_A * x + (_NS_B * gram + _NS_C * (gram @ gram)) @ x
    return x.transpose(-1, -2) if transposed else x


def muon_update(grad, momentum, *, lr: float, momentum_coeff: float, ns_steps: int):
    """Nesterov momentum then Newton-Schulz (Jordan scale). Returns (delta, new_momentum)."""
    g, m = _f32(grad), _f32(momentum)
    if g.shape != m.shape:
        raise ValueError(f"grad shape {tuple(g.shape)} != momentum shape {tuple(m.shape)}")
    if g.ndim != 2:
        raise ValueError(f"muon_update expects a 2D grad, got shape {tuple(g.shape)}")
    new_m = momentum_coeff * m + g
    orth = newton_schulz(g + momentum_coeff * new_m, int(ns_steps))
    rows, cols = int(orth.shape[0]), int(orth.shape[1])
    return float(lr) * math.sqrt(max(1.0, rows / max(cols, 1))) * orth, new_m


def muon_rms_scale(rows: int, cols: int) -> float:
    """0.2 * sqrt(max(rows, cols)): makes the Muon update RMS match AdamW's for any shape."""
    return MOONLIGHT_UPDATE_RMS * math.sqrt(max(_positive_int("rows", rows),
                                                _positive_int("cols", cols)))


def muon_transfer_step(param, grad, momentum, *, lr: float, momentum_coeff: float,
                       ns_steps: int, weight_decay: float):
    """One Muon step with the Moonlight RMS match and decoupled weight decay:
    ``new = p - lr * (muon_rms_scale(A, B) * O + wd * p)``. Returns (new_param, new_momentum)."""
    lr_f = _finite_real("lr", lr)
    wd_f = _finite_real("weight_decay", weight_decay)
    if wd_f < 0.0:
        raise ValueError("weight_decay must be >= 0")
    if isinstance(ns_steps, bool) or not isinstance(ns_steps, int) or ns_steps < 1 or ns_steps % 2 == 0:
        raise ValueError("ns_steps must be a positive odd integer")
    p, g, m = _f32(param), _f32(grad), _f32(momentum)
    if not (p.ndim == 2 and p.shape == g.shape == m.shape):
        raise ValueError(f"muon_transfer_step expects matching 2D matrices, got "
                         f"{tuple(p.shape)}, {tuple(g.shape)}, {tuple(m.shape)}")
    rows, cols = int(p.shape[0]), int(p.shape[1])
    if rows < 1 or cols < 1:
        raise ValueError("muon_transfer_step expects a non-empty matrix")
    new_m = momentum_coeff * m + g
    orth = newton_schulz(g + momentum_coeff * new_m, ns_steps)
    return p - lr_f * (muon_rms_scale(rows, cols) * orth + wd_f * p), new_m


def transferred_muon_lr(base_lr: float, *, width: int, base_width: int) -> float:
    """Under the Moonlight RMS match the update RMS is width-independent, so the tuned
    learning rate transfers unchanged."""
    lr = _finite_real("base_lr", base_lr)
    if lr < 0.0:
        raise ValueError("base_lr must be finite and >= 0")
    _positive_int("width", width)
    _positive_int("base_width", base_width)
    return lr


def qk_clip(q, k, max_logit: float):
    """Scale q and k by sqrt(tau / max|q k^T|) when the largest logit exceeds tau."""
    if max_logit <= 0:
        raise ValueError("qk_clip max_logit must be > 0")
    q32, k32 = _f32(q), _f32(k)
    if q32.shape[-1] != k32.shape[-1]:
        raise ValueError("q and k last dim (head dim) must match")
    mu = (q32 @ k32.transpose(-1, -2)).abs().max()
    tau = float(max_logit)
    scale = torch.where((mu > tau) & (mu != 0), torch.sqrt(tau / torch.clamp(mu, min=_NS_EPS)),
                        torch.ones_like(mu))
    return q32 * scale, k32 * scale


def adamw_update(param, grad, m, v, *, lr: float, beta1: float, beta2: float, eps: float,
                 wd: float, step: int):
    """Decoupled AdamW, 1-based bias correction. Returns (p, m, v)."""
    if int(step) < 1:
        raise ValueError("adamw_update step must be 1-based (>= 1)")
    p, g, m32, v32 = _f32(param), _f32(grad), _f32(m), _f32(v)
    m_t = beta1 * m32 + (1.0 - beta1) * g
    v_t = beta2 * v32 + (1.0 - beta2) * (g * g)
    t = int(step)
    m_hat = m_t / (1.0 - beta1**t)
    v_hat = v_t / (1.0 - beta2**t)
    return p * (1.0 - lr * wd) - lr * (m_hat / (torch.sqrt(v_hat) + eps)), m_t, v_t


def wsd_lr(step: int, config: TrainConfig) -> float:
    """Warmup (linear), stable (peak), decay (linear to 0). ``step`` is 1-based."""
    if int(step) < 1:
        raise ValueError("wsd_lr step must be 1-based (>= 1)")
    peak = float(config.peak_lr)
    warmup, stable, decay = int(config.warmup_steps), int(config.stable_steps), int(config.decay_steps)
    t = int(step)
    if warmup > 0 and t <= warmup:
        return peak * (t / warmup)
    if t <= warmup + stable:
        return peak
    if decay <= 0 or t >= warmup + stable + decay:
        return 0.0
    return peak * (1.0 - (t - warmup - stable) / decay)


# ---------------------------------------------------------------------------
# losses
# ---------------------------------------------------------------------------
def soft_cap(logits, cap: float) -> Tensor:
    if cap <= 0:
        raise ValueError("soft_cap cap must be > 0")
    return float(cap) * torch.tanh(_f32(logits) / float(cap))


def cross_entropy(logits, targets, loss_mask) -> Tensor:
    """Masked mean CE over already soft-capped logits; 0 for an empty mask."""
    logits_f, mask = _f32(logits), _f32(loss_mask)
    targets = torch.as_tensor(targets).to(logits_f.device)
    if tuple(logits_f.shape[:-1]) != tuple(targets.shape) or tuple(targets.shape) != tuple(mask.shape):
        raise ValueError(f"shape mismatch: logits {tuple(logits_f.shape)}, targets "
                         f"{tuple(targets.shape)}, mask {tuple(mask.shape)}")
    vocab = int(logits_f.shape[-1])
    flat = logits_f.reshape(-1, vocab)
    tgt = targets.reshape(-1).long()
    m = mask.reshape(-1)
    shifted = flat - flat.amax(dim=-1, keepdim=True)
    log_z = torch.log(torch.clamp(torch.exp(shifted).sum(dim=-1), min=1e-12))
    nll = -(shifted.gather(1, tgt[:, None])[:, 0] - log_z)
    denom = m.sum()
    return torch.where(denom > 0, (nll * m).sum() / torch.clamp(denom, min=1e-12),
                       torch.zeros_like(denom))


def mtp_loss(mtp_logits, tokens, loss_mask, cap: float | None = None) -> Tensor:
    """Mean over heads of the CE of head i on the token i + 1 steps ahead."""
    tokens_i = torch.as_tensor(tokens)
    mask = _f32(loss_mask)
    seq = int(tokens_i.shape[-1])
    losses = []
    for i, logits in enumerate(mtp_logits):
        offset = i + 1
        if offset >= seq:
            continue
        src = _f32(logits)[..., : seq - offset, :]
        if cap is not None:
            src = soft_cap(src, cap)
        m = mask[..., offset:] * mask[..., : seq - offset]
        losses.append(cross_entropy(src, tokens_i[..., offset:], m))
    if not losses:
        return torch.zeros((), dtype=torch.float32)
    return torch.stack(losses).mean()


def z_loss(router_probs) -> Tensor:
    """Mean squared log-sum-exp over the last axis (per token, then mean)."""
    p = _f32(router_probs)
    if p.numel() == 0:
        return torch.zeros((), dtype=torch.float32)
    return torch.mean(torch.logsumexp(p, dim=-1) ** 2)


def total_loss(ce, mtp, z, config: TrainConfig) -> Tensor:
    return _f32(ce) + _f32(mtp) + float(config.z_loss_weight) * _f32(z)


# ---------------------------------------------------------------------------
# tree helpers / optimizer state
# ---------------------------------------------------------------------------
def _map_tree(obj: Any, fn, prefix: str = "") -> Any:
    if isinstance(obj, dict):
        return {k: _map_tree(v, fn, f"{prefix}.{k}" if prefix else str(k)) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_map_tree(v, fn, f"{prefix}.{i}" if prefix else str(i)) for i, v in enumerate(obj)]
    if isinstance(obj, tuple):
        return tuple(_map_tree(v, fn, f"{prefix}.{i}" if prefix else str(i))
                     for i, v in enumerate(obj))
    return fn(prefix, obj)


def _is_muon(name: str, p: Any, all_matrices: bool) -> bool:
    if all_matrices:
        return muon_matrix_view(name, tuple(p.shape)) is not None
    return classify_param(name, p) is ParamKind.MUON_2D


def init_opt_state(params: dict, config: TrainConfig, *, muon_all_matrices: bool = False) -> dict:
    """FP32 optimizer state: ``{"momentum"}`` for Muon leaves, ``{"m", "v"}`` for AdamW."""
    del config

    def leaf(name: str, p: Any):
        z = lambda: torch.zeros_like(_f32(p))  # noqa: E731
        if _is_muon(name, p, muon_all_matrices):
            return {"momentum": z()}
        return {"m": z(), "v": z()}

    return _map_tree(params, leaf)


def apply_precision(params: dict, config: TrainConfig, *, materialize: bool = False) -> dict:
    """Copy of the master tree cast for the forward. With ``materialize`` the leaves are
    really rounded: FP8_LINEAR leaves through e4m3 with 128x128 (matrices) block scales,
    BF16_STABLE leaves through bf16; otherwise an fp32 copy (the reference behaviour)."""
    from . import kernels

    def leaf(name: str, p: Any):
        kind = precision_for(name, config)
        if kind is PrecisionKind.FP32_MASTER:
            raise TrainConfigError("precision_for must not return FP32_MASTER")
        t = _f32(p).clone()
        if not materialize:
            return t
        if kind is PrecisionKind.BF16_STABLE or t.ndim < 2:
            return t.bfloat16().float()
        flat = t.reshape(-1, t.shape[-1])
        return kernels.fp8_dequantize(
            kernels.fp8_quantize_2d(flat, block=int(config.fp8_block))).reshape(t.shape)

    return _map_tree(params, leaf)


def _leaves(obj: Any):
    if isinstance(obj, dict):
        for v in obj.values():
            yield from _leaves(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _leaves(v)
    else:
        yield obj


def _map_opt(p: Any, g: Any, s: Any, fn, prefix: str = ""):
    if isinstance(p, dict):
        out_p, out_s = {}, {}
        for k in p:
            name = f"{prefix}.{k}" if prefix else str(k)
            out_p[k], out_s[k] = _map_opt(p[k], g[k], s[k], fn, name)
        return out_p, out_s
    if isinstance(p, (list, tuple)):
        ps, ss = [], []
        for i, (pi, gi, si) in enumerate(zip(p, g, s, strict=True)):
            ni, nsi = _map_opt(pi, gi, si, fn, f"{prefix}.{i}" if prefix else str(i))
            ps.append(ni)
            ss.append(nsi)
        ctor = list if isinstance(p, list) else tuple
        return ctor(ps), ctor(ss)
    return fn(prefix, p, g, s)


def _clip_qk_weights(params: Any, max_logit: float) -> Any:
    if isinstance(params, dict):
        out = {k: _clip_qk_weights(v, max_logit) for k, v in params.items()}
        if "W_q" in out and "W_k" in out:
            q, k = out["W_q"], out["W_k"]
            if tuple(q.shape) == tuple(k.shape) and q.ndim >= 2:
                qc, kc = qk_clip(_f32(q).reshape(-1, q.shape[-1]), _f32(k).reshape(-1, k.shape[-1]),
                                 max_logit)
                out["W_q"], out["W_k"] = qc.reshape(q.shape), kc.reshape(k.shape)
        return out
    if isinstance(params, list):
        return [_clip_qk_weights(v, max_logit) for v in params]
    if isinstance(params, tuple):
        return tuple(_clip_qk_weights(v, max_logit) for v in params)
    return params


def _update_router_bias(params: Any, expert_ids: Tensor, n_experts: int, u: float = 1e-3,
                        router_probs: Tensor | None = None, rule: str = "probs") -> Any:
    """Aux-loss-free balancing: ``b <- b - u * sign(load - mean)`` on every ``router_bias``
    leaf. ``rule="probs"`` (the reference's, train/__init__.py:810-816): load = mean router
    probability per expert over the tokens of the last MoE layer. ``rule="count"``: load =
    fraction of the top-k assignments per expert in that layer, i.e. what the experts actually
    received (the fused trainer's default; the two can differ in sign for an expert that is often
    probable but rarely in the top k)."""
    if rule not in ("probs", "count"):
        raise ValueError("router_bias_rule must be 'probs' or 'count'")
    if rule == "probs" and router_probs is not None and router_probs.numel() > 0:
        load = _f32(router_probs).reshape(-1, router_probs.shape[-1]).mean(dim=0)
    elif expert_ids is None or expert_ids.numel() == 0:
        return params
    else:
        load = torch.bincount(expert_ids.reshape(-1).long(), minlength=n_experts).float()
        load = load / load.sum().clamp(min=1.0)
    delta = torch.sign(load - load.mean()) * float(u)

    def walk(obj):
        if isinstance(obj, dict):
            out = {k: walk(v) for k, v in obj.items()}
            if "router_bias" in out:
                b = _f32(out["router_bias"])
                n = min(int(b.shape[-1]), int(delta.shape[0]))
                b = b.clone()
                b[..., :n] -= delta[:n].to(b.device)
                out["router_bias"] = b
            return out
        if isinstance(obj, list):
            return [walk(v) for v in obj]
        if isinstance(obj, tuple):
            return tuple(walk(v) for v in obj)
        return obj

    return walk(params)


def compute_loss(params: dict, batch: Batch, model_config: ModelConfig,
                 train_config: TrainConfig, *, r: int = 1, z_on_logits: bool = False):
    """Forward + packed loss. Returns (total, (ce, mtp, z, forward_output))."""
    tokens = torch.as_tensor(batch.tokens)
    mask = _f32(batch.loss_mask)
    cap = float(train_config.softcap)
    out = model.forward(tokens, params, model_config, r=r)
    dev = out.logits.device
    tokens, mask = tokens.to(dev), mask.to(dev)
    ce = cross_entropy(soft_cap(out.logits[:, :-1, :], cap), tokens[:, 1:], mask[:, 1:])
    mtp = mtp_loss(out.mtp_logits, tokens, mask, cap).to(dev)
    z = out.z_loss if z_on_logits else z_loss(out.router_probs).to(dev)
    total = ce + mtp + float(train_config.z_loss_weight) * z
    return total, (ce, mtp, z, out)


def train_step(params: dict, opt_state: dict, batch: Batch, model_config: ModelConfig,
               train_config: TrainConfig, *, step: int, muon_transfer: bool = False,
               muon_weight_decay: float = 0.0, muon_all_matrices: bool = False, r: int = 1,
               z_on_logits: bool = False, router_bias_rule: str = "probs") -> StepOutput:
    """One FP32-master step: forward, loss, global-norm clip, Muon / AdamW, QK-clip,
    router-bias nudge (``router_bias_rule``: "probs" = the reference's mean router probability,
    "count" = share of the top-k assignments). ``step`` is 1-based."""
    validate_train_config(train_config)
    t = int(step)
    if t < 1:
        raise ValueError("train_step step must be 1-based (>= 1)")
    if not isinstance(muon_transfer, bool):
        raise ValueError("muon_transfer")
    muon_wd = 0.0
    if muon_transfer:
        try:
            muon_wd = _finite_real("muon_weight_decay", muon_weight_decay)
        except ValueError:
            raise ValueError("muon_weight_decay") from None
        if muon_wd < 0.0:
            raise ValueError("muon_weight_decay")
    sched = float(wsd_lr(t, train_config))
    peak = float(train_config.peak_lr)
    mult = sched / peak if peak > 0 else 0.0
    muon_lr_t = float(train_config.muon_lr) * mult
    adamw_lr_t = float(train_config.adamw_lr) * mult

    live = _map_tree(params, lambda _n, p: _f32(p).detach().clone().requires_grad_(True))
    total, (ce, mtp, z, out) = compute_loss(live, batch, model_config, train_config, r=r,
                                            z_on_logits=z_on_logits)
    leaves = list(_leaves(live))
    grads_flat = torch.autograd.grad(total, leaves, allow_unused=True)
    grads_flat = [torch.zeros_like(l) if g is None else g for g, l in zip(grads_flat, leaves)]
    it = iter(grads_flat)
    grads = _map_tree(live, lambda _n, _p: next(it))

    gnorm = torch.sqrt(torch.clamp(sum((g * g).sum() for g in grads_flat), min=0.0))
    clip = float(train_config.grad_clip)
    scale = torch.where(gnorm > clip, clip / (gnorm + 1e-6), torch.ones_like(gnorm)) if clip > 0 \
        else torch.ones_like(gnorm)

    beta = float(train_config.muon_momentum)
    ns = int(train_config.muon_ns_steps)

    def muon_leaf(name, p, g, s):
        view = muon_matrix_view(name, tuple(p.shape)) if muon_all_matrices else (1, *p.shape)
        b, rows, cols = view
        p2, g2, m2 = (x.reshape(b, rows, cols) for x in (p, g, s["momentum"]))
        new_m = beta * m2 + g2
        orth = newton_schulz(g2 + beta * new_m, ns)
        if muon_transfer:
            new_p = p2 - muon_lr_t * (muon_rms_scale(rows, cols) * orth + muon_wd * p2)
        else:
            new_p = p2 - muon_lr_t * math.sqrt(max(1.0, rows / max(cols, 1))) * orth
        return new_p.reshape(p.shape), {"momentum": new_m.reshape(p.shape)}

    def apply_one(name: str, p, g, s):
        p = p.detach()
        g = g * scale
        if _is_muon(name, p, muon_all_matrices):
            return muon_leaf(name, p, g, s)
        new_p, new_m, new_v = adamw_update(
            p, g, s["m"], s["v"], lr=adamw_lr_t, beta1=float(train_config.adamw_beta1),
            beta2=float(train_config.adamw_beta2), eps=float(train_config.adamw_eps),
            wd=float(train_config.adamw_wd), step=t)
        return new_p, {"m": new_m, "v": new_v}

    with torch.no_grad():
        new_params, new_opt = _map_opt(live, grads, opt_state, apply_one)
        if float(train_config.qk_clip) > 0:
            new_params = _clip_qk_weights(new_params, float(train_config.qk_clip))
        new_params = _update_router_bias(new_params, out.expert_ids,
                                         int(model_config.n_routed_experts),
                                         router_probs=out.router_probs, rule=router_bias_rule)
    return StepOutput(
        params=new_params, opt_state=new_opt,
        loss=LossBreakdown(ce=ce.detach(), mtp=mtp.detach(), z=z.detach(), total=total.detach()),
        lr=sched, grad_norm=gnorm.detach(), step=t,
    )
