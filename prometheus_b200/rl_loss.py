"""RL objective: GSPO sequence-level ratio with DAPO clip-higher, Dr.GRPO mean-centred
advantages, dynamic sampling, truncated importance sampling for stale rollouts, overlong
penalty, a separately clipped ratio for latent thoughts, and the routing-replay table.

API parity with the reference ``rl/loss/__init__.py`` (:94-530): ``LossConfig`` via
``make_config``, ``Sample``/``Group``/``RoutingTrace``/``LossBreakdown``, ``mean_center``,
``all_equal_reward``, ``drop_zero_advantage_groups``, ``sequence_ratio``, ``clip_higher``,
``staleness``, ``truncated_is``, ``overlong_soft_penalty``, ``gaussian_log_density``,
``latent_ratio``, ``routing_table``, ``gspo_dapo_loss``.

Log-probabilities may be Python floats (host bookkeeping) or torch tensors (the result is
then differentiable). Two options go beyond the reference, both off by default:
``length_normalize`` uses the GSPO ratio ``exp(mean(dlogp))`` instead of
``exp(sum(dlogp))``, and ``pessimistic`` takes ``min(r A, clip(r) A)`` (PPO style)
instead of ``clip(r) A``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import torch

GROUP_SIZE = 16
MAX_STALENESS = 4
DEFAULT_CLIP_EPS_LOW = 0.2
DEFAULT_CLIP_EPS_HIGH = 0.28


class LossError(ValueError):
    """An RL-loss argument is invalid."""


@dataclass(frozen=True)
class RoutingTrace:
    token_index: int
    layer_index: int
    expert_ids: tuple


@dataclass(frozen=True)
class Sample:
    token_logp_trainer: tuple
    token_logp_rollout: tuple
    latent_logp_trainer: tuple
    latent_logp_rollout: tuple
    reward: float
    n_tokens: int
    policy_version: int
    routing: tuple = ()


@dataclass(frozen=True)
class Group:
    prompt_id: str
    samples: tuple


@dataclass(frozen=True)
class LossConfig:
    clip_eps_low: float = DEFAULT_CLIP_EPS_LOW
    clip_eps_high: float = DEFAULT_CLIP_EPS_HIGH
    latent_clip_eps_low: float = DEFAULT_CLIP_EPS_LOW
    latent_clip_eps_high: float = DEFAULT_CLIP_EPS_HIGH
    loss_normalizer: float = 1.0
    overlong_cache: int = 0
    overlong_penalty: float = 0.0
    max_staleness: int = MAX_STALENESS
    tis_clip: float = 1.0
    kl_coeff: float = 0.0
    length_normalize: bool = False
    pessimistic: bool = False


@dataclass(frozen=True)
class LossBreakdown:
    pg: float
    tis: float
    overlong: float
    latent: float
    n_kept: int
    total: float


def make_config(clip_eps_low: float = DEFAULT_CLIP_EPS_LOW,
                clip_eps_high: float = DEFAULT_CLIP_EPS_HIGH,
                latent_clip_eps_low: float = DEFAULT_CLIP_EPS_LOW,
                latent_clip_eps_high: float = DEFAULT_CLIP_EPS_HIGH, loss_normalizer: float = 1.0,
                overlong_cache: int = 0, overlong_penalty: float = 0.0,
                max_staleness: int = MAX_STALENESS, tis_clip: float = 1.0, kl_coeff: float = 0.0,
                length_normalize: bool = False, pessimistic: bool = False) -> LossConfig:
    if min(clip_eps_low, clip_eps_high, latent_clip_eps_low, latent_clip_eps_high) < 0.0:
        raise LossError("epsilon must not be negative")
    if not math.isfinite(loss_normalizer) or loss_normalizer <= 0.0:
        raise LossError("loss_normalizer must be finite and positive")
    if overlong_cache < 0:
        raise LossError("overlong_cache must not be negative")
    if overlong_penalty < 0.0:
        raise LossError("overlong_penalty must not be negative")
    if max_staleness < 1 or max_staleness > MAX_STALENESS:
        raise LossError("max_staleness must be in 1 through MAX_STALENESS")
    if not math.isfinite(tis_clip) or tis_clip < 1.0:
        raise LossError("tis_clip must be finite and >= 1")
    if kl_coeff != 0.0:
        raise LossError("kl_coeff must be 0.0")
    return LossConfig(clip_eps_low, clip_eps_high, latent_clip_eps_low, latent_clip_eps_high,
                      loss_normalizer, overlong_cache, overlong_penalty, max_staleness, tis_clip,
                      kl_coeff, bool(length_normalize), bool(pessimistic))


def _is_t(x) -> bool:
    return isinstance(x, torch.Tensor)


def mean_center(rewards):
    """Dr.GRPO advantages: reward minus the group mean (no std division)."""
    if _is_t(rewards):
        if rewards.numel() == 0:
            raise LossError("empty rewards")
        return rewards - rewards.mean()
    if len(rewards) == 0:
        raise LossError("empty rewards")
    if any(not math.isfinite(r) for r in rewards):
        raise LossError("non-finite reward")
    mean = sum(rewards) / len(rewards)
    return tuple(r - mean for r in rewards)


def all_equal_reward(rewards: Sequence[float]) -> bool:
    if len(rewards) == 0:
        raise LossError("empty rewards")
    return all(r == rewards[0] for r in rewards)


def drop_zero_advantage_groups(groups: Sequence[Group]) -> tuple:
    """Dynamic sampling: groups whose rewards are all equal carry no gradient."""
    kept = []
    for g in groups:
        if len(g.samples) == 0:
            raise LossError("group with no samples")
        if not all_equal_reward(tuple(s.reward for s in g.samples)):
            kept.append(g)
    return tuple(kept)


def sequence_ratio(logp_new, logp_old, *, length_normalize: bool = False):
    """exp(sum(new - old)) over the sequence (or exp(mean) when length-normalised)."""
    if len(logp_new) == 0 or len(logp_old) == 0:
        raise LossError("empty log-probs")
    if len(logp_new) != len(logp_old):
        raise LossError("length mismatch")
    if _is_t(logp_new) or _is_t(logp_old):
        d = torch.as_tensor(logp_new) - torch.as_tensor(logp_old)
        return torch.exp(d.mean() if length_normalize else d.sum())
    if any(not math.isfinite(v) for v in (*logp_new, *logp_old)):
        raise LossError("non-finite log-prob")
    total = sum(n - o for n, o in zip(logp_new, logp_old))
    return math.exp(total / len(logp_new) if length_normalize else total)


def clip_higher(ratio, eps_low: float, eps_high: float):
    """Clip into [1 - eps_low, 1 + eps_high] (asymmetric: more room upward)."""
    if eps_low < 0.0 or eps_high < 0.0:
        raise LossError("epsilon must not be negative")
    if _is_t(ratio):
        return torch.clamp(ratio, 1.0 - eps_low, 1.0 + eps_high)
    if not math.isfinite(ratio):
        raise LossError("non-finite ratio")
    return min(max(ratio, 1.0 - eps_low), 1.0 + eps_high)


def staleness(trainer_version: int, policy_version: int) -> int:
    gap = trainer_version - policy_version
    if gap < 0:
        raise LossError("negative staleness")
    return gap


def truncated_is(logp_trainer, logp_rollout, k: int, tis_clip: float):
    """Importance weight of a rollout that is k versions stale: 1 for k = 0, else
    min(sequence ratio, tis_clip)."""
    if k < 0:
        raise LossError("negative staleness k")
    if tis_clip < 1.0:
        raise LossError("tis_clip must be >= 1")
    if k == 0:
        return torch.ones(()) if (_is_t(logp_trainer) or _is_t(logp_rollout)) else 1.0
    r = sequence_ratio(logp_trainer, logp_rollout)
    return torch.clamp(r, max=tis_clip) if _is_t(r) else min(r, tis_clip)


def overlong_soft_penalty(n_tokens: int, cache: int, penalty: float) -> float:
    if n_tokens < 0 or cache < 0 or penalty < 0.0:
        raise LossError("negative overlong argument")
    return 0.0 if n_tokens <= cache else penalty * (n_tokens - cache)


def gaussian_log_density(z, mu, sigma):
    """Sum of independent 1-D Gaussian log-densities."""
    if len(z) == 0 or len(mu) == 0 or len(sigma) == 0:
        raise LossError("empty gaussian inputs")
    if len(z) != len(mu) or len(z) != len(sigma):
        raise LossError("length mismatch")
    if _is_t(z) or _is_t(mu) or _is_t(sigma):
        z, mu, sigma = (torch.as_tensor(t, dtype=torch.float32) for t in (z, mu, sigma))
        return -0.5 * (((z - mu) / sigma) ** 2 + 2.0 * torch.log(sigma) + math.log(2 * math.pi)).sum()
    total = 0.0
    for zi, mi, si in zip(z, mu, sigma):
        if not (math.isfinite(zi) and math.isfinite(mi) and math.isfinite(si)):
            raise LossError("non-finite gaussian input")
        if si <= 0.0:
            raise LossError("sigma must be positive")
        total += ((zi - mi) / si) ** 2 + 2.0 * math.log(si) + math.log(2.0 * math.pi)
    return -0.5 * total


def latent_ratio(logp_new, logp_old):
    """Ratio over the latent thoughts of a sample; 1 when the sample has none."""
    if len(logp_new) == 0 and len(logp_old) == 0:
        return 1.0
    if len(logp_new) == 0 or len(logp_old) == 0:
        raise LossError("one latent side empty")
    return sequence_ratio(logp_new, logp_old)


def routing_table(traces: Sequence[RoutingTrace], n_tokens: int, n_layers: int, top_k: int) -> tuple:
    """Dense (token, layer) -> expert ids table for routing replay; every cell exactly once."""
    if n_tokens <= 0 or n_layers <= 0 or top_k <= 0:
        raise LossError("n_tokens, n_layers, and top_k must be positive")
    cells = {}
    for t in traces:
        key = (t.token_index, t.layer_index)
        if key in cells:
            raise LossError("duplicate (token, layer)")
        if not (0 <= t.token_index < n_tokens):
            raise LossError("token_index out of range")
        if not (0 <= t.layer_index < n_layers):
            raise LossError("layer_index out of range")
        if len(t.expert_ids) != top_k:
            raise LossError("expert_ids length must equal top_k")
        if any(e < 0 for e in t.expert_ids):
            raise LossError("expert id must be non-negative")
        cells[key] = tuple(t.expert_ids)
    if len(cells) != n_tokens * n_layers:
        raise LossError("missing (token, layer)")
    return tuple(tuple(cells[(i, j)] for j in range(n_layers)) for i in range(n_tokens))


def gspo_dapo_loss(group: Group, config: LossConfig, trainer_version: int) -> LossBreakdown:
    """Group objective: sum over samples of tis * clip(ratio) * advantage (discrete and
    latent parts clipped separately) plus the overlong penalty, divided by the constant
    ``loss_normalizer``. A group with identical rewards contributes nothing."""
    if len(group.samples) == 0:
        raise LossError("empty group")
    if group.prompt_id == "":
        raise LossError("empty prompt_id")
    gaps = []
    for s in group.samples:
        if len(s.token_logp_trainer) == 0 or len(s.token_logp_rollout) == 0:
            raise LossError("empty token log-probs")
        if len(s.token_logp_trainer) != len(s.token_logp_rollout):
            raise LossError("mismatched trainer/rollout lengths")
        if len(s.latent_logp_trainer) != len(s.latent_logp_rollout):
            raise LossError("mismatched trainer/rollout lengths")
        gap = staleness(trainer_version, s.policy_version)
        if gap > config.max_staleness:
            raise LossError("staleness exceeds max_staleness")
        gaps.append(gap)
    rewards = tuple(float(s.reward) for s in group.samples)
    if all_equal_reward(rewards):
        return LossBreakdown(pg=0.0, tis=0.0, overlong=0.0, latent=0.0, n_kept=0, total=0.0)
    adv = mean_center(rewards)

    def surrogate(r, a, lo, hi):
        c = clip_higher(r, lo, hi)
        if not config.pessimistic:
            return c * a
        return torch.minimum(r * a, c * a) if _is_t(r) else min(r * a, c * a)

    pg = lat = ol = tis = 0.0
    for s, a, gap in zip(group.samples, adv, gaps):
        r = sequence_ratio(s.token_logp_trainer, s.token_logp_rollout,
                           length_normalize=config.length_normalize)
        w = truncated_is(s.token_logp_trainer, s.token_logp_rollout, gap, config.tis_clip)
        if _is_t(w):
            w = w.detach()
        pg = pg + surrogate(r, a, config.clip_eps_low, config.clip_eps_high) * w
        if len(s.latent_logp_trainer) or len(s.latent_logp_rollout):
            rl = latent_ratio(s.latent_logp_trainer, s.latent_logp_rollout)
            lat = lat + surrogate(rl, a, config.latent_clip_eps_low, config.latent_clip_eps_high) * w
        ol = ol + overlong_soft_penalty(s.n_tokens, config.overlong_cache, config.overlong_penalty)
        tis = tis + w
    z = config.loss_normalizer
    n = len(group.samples)
    return LossBreakdown(pg=pg / z, tis=tis / n, overlong=ol / z, latent=lat / z, n_kept=n,
                         total=(pg + lat + ol) / z)
