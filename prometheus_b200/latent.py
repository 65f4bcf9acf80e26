"""Latent reasoning: PonderNet halting, the Stage-B loss, Jacobi-parallel thought updates,
the noisy latent policy, think-span layout, segment decoding, CODI alignment, and the
in-sequence latent-slot forward used for latent continued training.

API parity with the reference ``model/latent.py``: ``LatentConfig`` (:86-100),
``HaltOutput``/``StageBLoss``/``NoisyLatent``/``ThinkSpan``/``SegmentDecoder``/
``StageBObjective`` (:103-230), ``validate_latent_config`` (:313), ``ponder_distribution``
(:367), ``geometric_prior`` (:383), ``halt_from_logits`` (:410), ``halt_loss`` (:428),
``halt_kl`` (:451), ``thought_decode_ce`` (:473), ``answer_ce_at_depths`` (:523),
``stage_b_loss`` (:546), ``jacobi_sweeps`` (:619), ``clamp_sigma`` (:680),
``noisy_latent`` (:706), ``plan_think_layout`` (:743), ``insert_discrete_tool`` (:797),
``decode_thought_segment`` (:872), ``codi_alignment`` (:989), ``stage_b_objective`` (:1027).

``latent_slot_forward`` is new: the reference prepends thoughts to the sequence; the B200
latent-training configuration places K latent slots *between* a prefix and an answer and
solves them with a Jacobi fixed-point iteration whose every sweep is a full forward.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import Any, Callable, Sequence

import numpy as np
import torch

Tensor = torch.Tensor


class LatentError(ValueError):
    """A latent-reasoning argument or config is invalid."""


CHUNK_MIN_THOUGHTS = 4
CHUNK_MAX_THOUGHTS = 64
COMPRESSION_TOKENS_PER_THOUGHT = 8
DEFAULT_JACOBI_SWEEPS = 4
TRUNCATED_SWEEPS = 2
TRUNCATED_RECURRENCE = 4
DEFAULT_MAX_THOUGHTS = 16
DEFAULT_ALPHA_TRAJ = 1.0
DEFAULT_GAMMA_HALT = 1.0
DEFAULT_BETA_KL = 0.01
DEFAULT_LAMBDA_PRIOR = 0.2
HALT_EPS = 1e-6
SIGMA_MIN = 1e-4
SIGMA_MAX = 0.1


@dataclass(frozen=True)
class LatentConfig:
    max_thoughts: int = DEFAULT_MAX_THOUGHTS
    chunk_min: int = CHUNK_MIN_THOUGHTS
    chunk_max: int = CHUNK_MAX_THOUGHTS
    alpha_traj: float = DEFAULT_ALPHA_TRAJ
    gamma_halt: float = DEFAULT_GAMMA_HALT
    beta_kl: float = DEFAULT_BETA_KL
    lambda_prior: float = DEFAULT_LAMBDA_PRIOR
    jacobi_sweeps: int = DEFAULT_JACOBI_SWEEPS
    truncated_sweeps: int = TRUNCATED_SWEEPS
    sigma_min: float = SIGMA_MIN
    sigma_max: float = SIGMA_MAX


@dataclass(frozen=True)
class HaltOutput:
    """Halting over depths 0..K (K+1 slots); the last lambda is pinned to 1 so p sums to 1."""

    lambdas: Tensor
    p: Tensor
    expected_depth: Tensor


@dataclass(frozen=True)
class StageBLoss:
    l_task: Tensor
    l_traj: Tensor
    l_halt: Tensor
    l_kl: Tensor
    expected_depth: Tensor
    total: Tensor


@dataclass(frozen=True)
class NoisyLatent:
    mu: Tensor
    sigma: Tensor
    eps: Tensor
    z: Tensor
    log_density: Tensor


class SpanKind(str, Enum):
    LATENT = "latent"
    ANCHOR = "anchor"
    TOOL = "tool"

    def __str__(self) -> str:
        return self.value


@dataclass(frozen=True)
class ThinkSpan:
    kind: SpanKind
    n_thoughts: int
    token_ids: tuple


@dataclass(frozen=True)
class SegmentDecoder:
    w_in: Tensor
    w_h: Tensor
    bias: Tensor


@dataclass(frozen=True)
class StageBObjective:
    stage_b: StageBLoss
    l_align: Tensor
    total: Tensor


def _t(x: Any) -> Tensor:
    t = x if isinstance(x, Tensor) else torch.as_tensor(np.asarray(x))
    return t if t.dtype in (torch.float32, torch.float64) else t.float()


def _vec(x: Any, name: str) -> Tensor:
    t = _t(x)
    if t.ndim != 1 or t.shape[0] < 1:
        raise LatentError(f"{name} must be 1-D and non-empty")
    if not bool(torch.isfinite(t.detach()).all()):
        raise LatentError(f"{name} must be finite")
    return t


def validate_latent_config(config: LatentConfig) -> None:
    """Order of checks: max_thoughts, chunk bounds, weights, lambda_prior, sweeps, sigma."""
    if int(config.max_thoughts) < 0:
        raise LatentError("max_thoughts must be >= 0")
    lo, hi = int(config.chunk_min), int(config.chunk_max)
    if lo < CHUNK_MIN_THOUGHTS or hi > CHUNK_MAX_THOUGHTS or lo > hi:
        raise LatentError("chunk bounds invalid")
    for name in ("alpha_traj", "gamma_halt", "beta_kl"):
        v = float(getattr(config, name))
        if not math.isfinite(v) or v < 0.0:
            raise LatentError(f"{name} must be finite and non-negative")
    if not (0.0 < float(config.lambda_prior) < 1.0):
        raise LatentError("lambda_prior must be in (0, 1)")
    if int(config.jacobi_sweeps) < 1:
        raise LatentError("jacobi_sweeps must be >= 1")
    if not (1 <= int(config.truncated_sweeps) <= int(config.jacobi_sweeps)):
        raise LatentError("truncated_sweeps must sit in 1..=jacobi_sweeps")
    smin, smax = float(config.sigma_min), float(config.sigma_max)
    if not (math.isfinite(smin) and math.isfinite(smax)) or smin <= 0.0 or smax < smin:
        raise LatentError("sigma clamp bounds invalid")


# ---------------------------------------------------------------------------
# halting
# ---------------------------------------------------------------------------
def _pin_and_distribute(lam: Tensor) -> tuple[Tensor, Tensor]:
    n = lam.shape[0]
    clipped = torch.clamp(lam, HALT_EPS, 1.0 - HALT_EPS)
    last = torch.arange(n, device=lam.device) == n - 1
    clipped = torch.where(last, torch.ones_like(clipped), clipped)
    survive = torch.cat([torch.ones(1, dtype=lam.dtype, device=lam.device),
                         torch.cumprod(1.0 - clipped[:-1], dim=0)])
    return clipped, clipped * survive


def ponder_distribution(lambdas) -> Tensor:
    """p_m = lambda_m prod_{j<m} (1 - lambda_j), lambdas clipped, last pinned to 1."""
    return _pin_and_distribute(_vec(lambdas, "lambdas"))[1]


def geometric_prior(n: int, lambda_prior: float) -> np.ndarray:
    """Truncated geometric prior over n slots, renormalised (float64 NumPy, host side)."""
    n, lam = int(n), float(lambda_prior)
    if n < 1:
        raise LatentError("n must be >= 1")
    if not (0.0 < lam < 1.0):
        raise LatentError("lambda_prior must be in (0, 1)")
    g = lam * (1.0 - lam) ** np.arange(n, dtype=np.float64)
    total = g.sum()
    if total <= 0.0:
        raise LatentError("geometric prior mass vanished")
    return g / total


def halt_from_logits(halt_logits) -> HaltOutput:
    x = _vec(halt_logits, "halt_logits")
    lam, p = _pin_and_distribute(torch.sigmoid(torch.clamp(x, -80.0, 80.0)))
    depth = torch.arange(p.shape[0], dtype=p.dtype, device=p.device)
    return HaltOutput(lambdas=lam, p=p, expected_depth=(p * depth).sum())


def halt_loss(p, teacher_steps: int) -> Tensor:
    """-log(p[k] + eps) at the teacher's step count (clamped into range)."""
    p = _vec(p, "p")
    k = min(max(int(teacher_steps), 0), p.shape[0] - 1)
    return -torch.log(p[k] + HALT_EPS)


def halt_kl(p, lambda_prior: float) -> Tensor:
    p = _vec(p, "p")
    g = torch.as_tensor(geometric_prior(p.shape[0], float(lambda_prior)), dtype=p.dtype,
                        device=p.device)
    return (p * (torch.log(p + HALT_EPS) - torch.log(g + HALT_EPS))).sum()


# ---------------------------------------------------------------------------
# Stage-B loss
# ---------------------------------------------------------------------------
def thought_decode_ce(logits, teacher_ids, mask) -> Tensor:
    """Masked mean CE of decoding each thought to its teacher token (0 for an empty mask)."""
    lg = _t(logits)
    if lg.ndim != 2:
        raise LatentError("logits must be (n, vocab)")
    n, vocab = lg.shape
    if n < 1:
        raise LatentError("empty logits")
    ids = torch.as_tensor(np.asarray(teacher_ids) if not isinstance(teacher_ids, Tensor)
                          else teacher_ids).long().to(lg.device)
    m = _t(mask).to(lg.device)
    if ids.ndim != 1 or m.ndim != 1:
        raise LatentError("teacher_ids and mask must be 1-D")
    if ids.shape[0] != n or m.shape[0] != n:
        raise LatentError("length mismatch")
    if bool(((ids < 0) | (ids >= vocab)).any()):
        raise LatentError("teacher id outside [0, vocab)")
    ce = -torch.log_softmax(lg, dim=-1).gather(1, ids[:, None])[:, 0]
    kept = (m != 0).to(lg.dtype)
    denom = kept.sum()
    return torch.where(denom > 0, (ce * kept).sum() / torch.clamp(denom, min=1e-12),
                       torch.zeros_like(denom))


def answer_ce_at_depths(logits, answer_id: int) -> Tensor:
    lg = _t(logits)
    if lg.ndim != 2:
        raise LatentError("logits must be (K+1, vocab)")
    if lg.shape[0] < 1:
        raise LatentError("empty logits")
    aid = int(answer_id)
    if aid < 0 or aid >= lg.shape[1]:
        raise LatentError("answer_id outside [0, vocab)")
    return -torch.log_softmax(lg, dim=-1)[:, aid]


def stage_b_loss(halt_logits, answer_logits, thought_logits, teacher_ids, thought_mask,
                 answer_id: int, teacher_steps: int, config: LatentConfig) -> StageBLoss:
    """total = l_task + alpha l_traj + gamma l_halt + beta l_kl."""
    validate_latent_config(config)
    halt = _t(halt_logits)
    if halt.ndim != 1 or halt.shape[0] < 1:
        raise LatentError("halt_logits must be 1-D with length K+1")
    k = halt.shape[0] - 1
    answer = _t(answer_logits)
    if answer.ndim != 2 or answer.shape[0] != k + 1:
        raise LatentError("answer_logits must have length K+1")
    if k == 0:
        l_traj = torch.zeros((), dtype=halt.dtype, device=halt.device)
    else:
        thought = _t(thought_logits)
        if thought.ndim != 2 or thought.shape[0] != k:
            raise LatentError("thought_logits must have K rows")
        l_traj = thought_decode_ce(thought, teacher_ids, thought_mask)
    ho = halt_from_logits(halt)
    l_task = (ho.p * answer_ce_at_depths(answer, answer_id)).sum()
    l_halt = halt_loss(ho.p, teacher_steps)
    l_kl = halt_kl(ho.p, float(config.lambda_prior))
    total = l_task + config.alpha_traj * l_traj + config.gamma_halt * l_halt + config.beta_kl * l_kl
    return StageBLoss(l_task=l_task, l_traj=l_traj, l_halt=l_halt, l_kl=l_kl,
                      expected_depth=ho.expected_depth, total=total)


# ---------------------------------------------------------------------------
# Jacobi sweeps
# ---------------------------------------------------------------------------
def jacobi_sweeps(thoughts, update: Callable[[Tensor], Tensor], n_sweeps: int,
                  truncated_sweeps: int) -> Tensor:
    """All thoughts are updated at once per sweep (``current = update(current)``); gradient
    flows only through the last ``truncated_sweeps`` sweeps (the value entering that window
    is detached; ``truncated_sweeps == n_sweeps`` is the full unroll)."""
    cur = _t(thoughts)
    if cur.ndim != 2:
        raise LatentError("thoughts rank != 2")
    if cur.shape[0] < 1 or cur.shape[1] < 1:
        raise LatentError("thoughts n>=1 and d>=1")
    sweeps, trunc = int(n_sweeps), int(truncated_sweeps)
    if sweeps < 1:
        raise LatentError("n_sweeps must be >= 1")
    if trunc < 1 or trunc > sweeps:
        raise LatentError("truncated_sweeps not in 1..=n_sweeps")
    shape = tuple(cur.shape)
    cut = sweeps - trunc
    for i in range(sweeps):
        if cut > 0 and i == cut:
            cur = cur.detach()
        nxt = torch.as_tensor(update(cur))
        if tuple(nxt.shape) != shape:
            raise LatentError("update changed shape")
        cur = nxt
    return cur


# ---------------------------------------------------------------------------
# noisy latent policy
# ---------------------------------------------------------------------------
def clamp_sigma(sigma, config: LatentConfig) -> Tensor:
    s = _t(sigma)
    if s.numel() < 1:
        raise LatentError("sigma empty")
    if not bool(torch.isfinite(s.detach()).all()):
        raise LatentError("sigma non-finite")
    validate_latent_config(config)
    return torch.clamp(s, float(config.sigma_min), float(config.sigma_max))


def noisy_latent(mu, sigma, eps, config: LatentConfig) -> NoisyLatent:
    """z = mu + clamp(sigma) * eps with the diagonal-Gaussian log-density of z."""
    mu_a, sg, ep = _vec(mu, "mu"), _vec(sigma, "sigma"), _vec(eps, "eps")
    if not (mu_a.shape[0] == sg.shape[0] == ep.shape[0]):
        raise LatentError("length mismatch")
    s = clamp_sigma(sg, config)
    z = mu_a + s * ep
    c = (z - mu_a) / s
    logd = -0.5 * (c * c + 2.0 * torch.log(s) + math.log(2.0 * math.pi)).sum()
    return NoisyLatent(mu=mu_a, sigma=s, eps=ep, z=z, log_density=logd)


def gaussian_log_density(z, mu, sigma) -> Tensor:
    z, mu, sigma = _t(z), _t(mu), _t(sigma)
    c = (z - mu) / sigma
    return -0.5 * (c * c + 2.0 * torch.log(sigma) + math.log(2.0 * math.pi)).sum(dim=-1)


# ---------------------------------------------------------------------------
# think layout (host side)
# ---------------------------------------------------------------------------
def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def plan_think_layout(chunk_lengths: Sequence[int], anchor_token_ids: Sequence[int],
                      config: LatentConfig) -> tuple:
    """Latent chunks separated by one discrete anchor span each."""
    lengths = list(chunk_lengths)
    if not lengths:
        raise LatentError("chunk_lengths empty")
    for n in lengths:
        if not _is_int(n) or n < config.chunk_min or n > config.chunk_max:
            raise LatentError("chunk length out of range")
    anchors = list(anchor_token_ids)
    if not anchors:
        raise LatentError("anchor empty")
    if any(not _is_int(t) or t < 0 for t in anchors):
        raise LatentError("anchor token id")
    spans = []
    for i, n in enumerate(lengths):
        if i:
            spans.append(ThinkSpan(SpanKind.ANCHOR, 0, tuple(anchors)))
        spans.append(ThinkSpan(SpanKind.LATENT, n, ()))
    return tuple(spans)


def insert_discrete_tool(layout: Sequence[ThinkSpan], after_chunk: int,
                         tool_token_ids: Sequence[int]) -> tuple:
    """Insert a TOOL span right before the latent chunk that follows chunk ``after_chunk``
    (or at the end after the last chunk). The layout must be latent chunks with exactly one
    anchor between consecutive chunks, tools only after their anchor."""
    if isinstance(layout, (str, bytes)) or not isinstance(layout, Sequence):
        raise LatentError("layout")
    spans = tuple(layout)
    if not spans or not isinstance(spans[0], ThinkSpan) or spans[0].kind is not SpanKind.LATENT:
        raise LatentError("layout")
    if any(not isinstance(s, ThinkSpan) for s in spans):
        raise LatentError("layout")
    lat = [i for i, s in enumerate(spans) if s.kind is SpanKind.LATENT]
    for a, b in zip(lat, lat[1:]):
        between = [spans[j].kind for j in range(a + 1, b)]
        if sum(k is SpanKind.ANCHOR for k in between) != 1:
            raise LatentError("layout")
        if SpanKind.TOOL in between and between.index(SpanKind.ANCHOR) > between.index(SpanKind.TOOL):
            raise LatentError("layout")
    if any(s.kind is not SpanKind.TOOL for s in spans[lat[-1] + 1:]):
        raise LatentError("layout")
    if not _is_int(after_chunk) or after_chunk < 0 or after_chunk >= len(lat):
        raise LatentError("after_chunk")
    ids = list(tool_token_ids)
    if not ids:
        raise LatentError("tool empty")
    if any(not _is_int(t) or t < 0 for t in ids):
        raise LatentError("tool token id")
    at = len(spans) if after_chunk == len(lat) - 1 else lat[after_chunk + 1]
    return spans[:at] + (ThinkSpan(SpanKind.TOOL, 0, tuple(ids)),) + spans[at:]


# ---------------------------------------------------------------------------
# segment decoding / alignment
# ---------------------------------------------------------------------------
def decode_thought_segment(hidden, teacher_len: int, unembed, decoder: SegmentDecoder | None = None,
                           final_norm=None) -> Tensor:
    """Logits for the teacher tokens a thought stands for: the tied head for a one-token
    step, a small tanh recurrent decoder (state_0 = 0) for longer segments."""
    if not _is_int(teacher_len) or teacher_len < 1:
        raise LatentError("teacher_len")
    h = _t(hidden)
    if h.ndim != 1 or h.shape[0] < 1 or not bool(torch.isfinite(h.detach()).all()):
        raise LatentError("hidden")
    d = h.shape[0]
    u = _t(unembed)
    if u.ndim != 2 or u.shape[0] < 1 or u.shape[1] != d or not bool(torch.isfinite(u.detach()).all()):
        raise LatentError("unembed")
    w = None
    if final_norm is not None:
        w = _t(final_norm)
        if tuple(w.shape) != (d,) or not bool(torch.isfinite(w.detach()).all()):
            raise LatentError("final_norm")

    def tied(x: Tensor) -> Tensor:
        if w is not None:
            x = x * torch.rsqrt((x * x).mean() + 1e-6) * w
        return x @ u.T

    if teacher_len == 1:
        return tied(h)
    if not isinstance(decoder, SegmentDecoder):
        raise LatentError("decoder")
    w_in, w_h, bias = _t(decoder.w_in), _t(decoder.w_h), _t(decoder.bias)
    ok = tuple(w_in.shape) == (d, d) and tuple(w_h.shape) == (d, d) and tuple(bias.shape) == (d,)
    if not ok or not all(bool(torch.isfinite(t.detach()).all()) for t in (w_in, w_h, bias)):
        raise LatentError("decoder")
    state = torch.zeros_like(h)
    rows = []
    for _ in range(teacher_len):
        state = torch.tanh(h @ w_in + state @ w_h + bias)
        rows.append(tied(state))
    return torch.stack(rows, dim=0)


def codi_alignment(student_h, teacher_h) -> Tensor:
    """Mean squared distance to the (detached) teacher hidden states."""
    s, t = _t(student_h), _t(teacher_h)
    for name, a in (("student_h", s), ("teacher_h", t)):
        if a.ndim != 2 or a.shape[0] < 1 or a.shape[1] < 1 or not bool(torch.isfinite(a.detach()).all()):
            raise LatentError(name)
    if s.shape != t.shape:
        raise LatentError("shape")
    return ((s - t.detach()) ** 2).mean()


def stage_b_objective(halt_logits, answer_logits, thought_logits, teacher_ids, thought_mask,
                      answer_id: int, teacher_depth: int, config: LatentConfig, student_h,
                      teacher_h, *, align_weight: float = 1.0) -> StageBObjective:
    if isinstance(align_weight, bool) or not isinstance(align_weight, (int, float)) \
            or not math.isfinite(align_weight) or align_weight < 0:
        raise LatentError("align_weight")
    base = stage_b_loss(halt_logits, answer_logits, thought_logits, teacher_ids, thought_mask,
                        answer_id, teacher_depth, config)
    l_align = codi_alignment(student_h, teacher_h)
    return StageBObjective(stage_b=base, l_align=l_align, total=base.total + align_weight * l_align)


# ---------------------------------------------------------------------------
# in-sequence latent slots (prefix | K latent slots | answer), Jacobi-parallel
# ---------------------------------------------------------------------------
def latent_slot_embeddings(hidden: Tensor, embeds: Tensor, slot_start: int, k: int,
                           adapter: Callable[[Tensor], Tensor]) -> Tensor:
    """One Jacobi update of the input embeddings: slot j receives ``adapter(hidden at the
    position just before it)`` from the previous sweep; every other position keeps its
    token embedding. hidden, embeds: (B, S, d)."""
    if slot_start < 1 or slot_start + k > embeds.shape[1]:
        raise LatentError("latent slots outside the sequence")
    src = hidden[:, slot_start - 1:slot_start - 1 + k, :]
    new = embeds.clone()
    new[:, slot_start:slot_start + k, :] = adapter(src).to(embeds.dtype)
    return new


def latent_slot_forward(embeds: Tensor, forward_hidden: Callable[[Tensor], Tensor],
                        adapter: Callable[[Tensor], Tensor], slot_start: int, k: int, *,
                        n_sweeps: int = DEFAULT_JACOBI_SWEEPS, truncated_sweeps: int | None = None):
    """Final hidden states with the K latent slots solved by ``n_sweeps`` Jacobi sweeps.

    Sequentially, latent step j would feed the final hidden state of position
    ``slot_start + j - 1`` back as the input embedding of position ``slot_start + j``. The
    Jacobi form updates all K slots at once from the previous sweep's hidden states, so a
    sweep is one ordinary full-sequence forward (``n_sweeps`` forwards in total); with K + 1
    sweeps it equals the sequential solve exactly, and fewer sweeps is the fixed-point approximation. Gradient flows
    through the last ``truncated_sweeps`` sweeps (None = all: gradient through the whole
    recurrence). Returns (hidden of the last sweep, embeddings fed to it)."""
    sweeps = int(n_sweeps)
    trunc = sweeps if truncated_sweeps is None else int(truncated_sweeps)
    if sweeps < 1:
        raise LatentError("n_sweeps must be >= 1")
    if trunc < 1 or trunc > sweeps:
        raise LatentError("truncated_sweeps not in 1..=n_sweeps")
    cut = sweeps - trunc
    cur = embeds
    hidden = None
    for i in range(sweeps):
        if cut > 0 and i == cut:
            cur = cur.detach()
        hidden = forward_hidden(cur)
        if i + 1 < sweeps:
            cur = latent_slot_embeddings(hidden, embeds, slot_start, k, adapter)
    return hidden, cur
