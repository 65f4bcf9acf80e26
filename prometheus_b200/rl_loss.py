"""RL objective as one batched tensor loss.

Rollout groups are packed into padded tensors (``pack_groups``): per-token log-probabilities of
the trainer and of the rollout policy ``(N, T)`` with a mask, the same for the latent thoughts
``(N, L)``, and per-sample reward, group index, length and staleness. ``batched_loss`` then
evaluates the whole batch with a handful of masked reductions, on whatever device the tensors
live on (this is the form a GPU RL trainer calls once per step, with ``logp_trainer`` carrying
the graph):

* GSPO sequence ratio ``exp(sum(dlogp))`` per sample (``length_normalize``: ``exp(mean)``);
* DAPO clip-higher ``[1 - eps_low, 1 + eps_high]``, optionally the pessimistic PPO minimum;
* Dr.GRPO advantages: reward minus the group mean, no division by the deviation;
* dynamic sampling: a group whose rewards are all equal contributes nothing;
* truncated importance weights for stale rollouts: 1 when fresh, else ``min(ratio, tis_clip)``,
  never differentiated;
* the latent thoughts' own ratio, clipped with its own epsilons;
* the soft overlong penalty ``penalty * max(0, n_tokens - cache)``;
* everything divided by the constant ``loss_normalizer``.

The names of the reference's ``rl/loss/__init__.py`` (:94-530) are kept on top of it:
``LossConfig`` via ``make_config``, ``Sample`` / ``Group`` / ``RoutingTrace`` / ``LossBreakdown``,
the scalar helpers (``mean_center``, ``sequence_ratio``, ``clip_higher``, ``truncated_is``,
``overlong_soft_penalty``, ``gaussian_log_density``, ``latent_ratio``, ``staleness``,
``all_equal_reward``, ``drop_zero_advantage_groups``, ``routing_table``) and
``gspo_dapo_loss(group, config, trainer_version)``, which packs its one group and calls the
batched loss. Float inputs give float results, tensor inputs differentiable tensors.
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
    """A validated ``LossConfig``. The KL term is fixed at zero (the objective has none)."""
    problems = {
        "clip epsilons must be >= 0": min(clip_eps_low, clip_eps_high, latent_clip_eps_low,
                                          latent_clip_eps_high) < 0.0,
        "loss_normalizer must be a finite positive number": not (math.isfinite(loss_normalizer)
                                                                 and loss_normalizer > 0.0),
        "overlong_cache and overlong_penalty must be >= 0": overlong_cache < 0 or overlong_penalty < 0.0,
        f"max_staleness must lie in 1..{MAX_STALENESS}": not (1 <= max_staleness <= MAX_STALENESS),
        "tis_clip must be a finite number >= 1": not (math.isfinite(tis_clip) and tis_clip >= 1.0),
        "kl_coeff is not supported (must be 0)": kl_coeff != 0.0,
    }
    for message, bad in problems.items():
        if bad:
            raise LossError(message)
    return LossConfig(clip_eps_low, clip_eps_high, latent_clip_eps_low, latent_clip_eps_high,
                      loss_normalizer, overlong_cache, overlong_penalty, max_staleness, tis_clip,
                      kl_coeff, bool(length_normalize), bool(pessimistic))


def _is_t(x) -> bool:
    return isinstance(x, torch.Tensor)


def _finite(values, what: str) -> None:
    if any(not math.isfinite(float(v)) for v in values):
        raise LossError(f"{what} must be finite")


# ---------------------------------------------------------------------------
# packed batch + the batched loss
# ---------------------------------------------------------------------------
@dataclass
class PackedRollouts:
    """N samples of G groups, padded: ``logp_*`` ``(N, T)`` with ``mask`` (1 = real token),
    ``lat_*`` ``(N, L)`` with ``lat_mask``, ``reward`` / ``group`` / ``n_tokens`` / ``gap`` ``(N,)``."""

    logp_trainer: torch.Tensor
    logp_rollout: torch.Tensor
    mask: torch.Tensor
    lat_trainer: torch.Tensor
    lat_rollout: torch.Tensor
    lat_mask: torch.Tensor
    reward: torch.Tensor
    group: torch.Tensor
    n_tokens: torch.Tensor
    gap: torch.Tensor
    n_groups: int


def _pad_rows(rows, width: int, device, dtype=torch.float32):
    """Stack 1-D sequences (tuples of floats or tensors) into (N, width) + mask, keeping the
    autograd graph of tensor rows."""
    out, mask = [], torch.zeros((len(rows), max(width, 1)), dtype=dtype, device=device)
    for i, r in enumerate(rows):
        t = r.to(device=device, dtype=dtype) if _is_t(r) else torch.tensor(list(r), dtype=dtype, device=device)
        n = int(t.numel())
        mask[i, :n] = 1.0
        out.append(torch.nn.functional.pad(t.reshape(-1), (0, max(width, 1) - n)))
    return torch.stack(out), mask


def pack_groups(groups: Sequence[Group], trainer_version: int, config: LossConfig,
                device="cpu") -> PackedRollouts:
    """Validate and pack groups of samples for :func:`batched_loss`."""
    if len(groups) == 0:
        raise LossError("no groups to pack")
    samples, gidx, gaps = [], [], []
    for g, grp in enumerate(groups):
        if not grp.prompt_id:
            raise LossError("a group needs a prompt_id")
        if len(grp.samples) == 0:
            raise LossError(f"group {grp.prompt_id!r} has no samples")
        for s in grp.samples:
            nt, nr = len(s.token_logp_trainer), len(s.token_logp_rollout)
            if nt == 0 or nt != nr:
                raise LossError("trainer and rollout token log-probs must be non-empty and equally long")
            if len(s.latent_logp_trainer) != len(s.latent_logp_rollout):
                raise LossError("trainer and rollout latent log-probs must be equally long")
            if not _is_t(s.reward) and not math.isfinite(s.reward):
                raise LossError("a reward is not finite")
            gap = staleness(trainer_version, s.policy_version)
            if gap > config.max_staleness:
                raise LossError(f"rollout is {gap} versions stale (limit {config.max_staleness})")
            samples.append(s)
            gidx.append(g)
            gaps.append(gap)
    width = max(len(s.token_logp_trainer) for s in samples)
    lwidth = max(len(s.latent_logp_trainer) for s in samples)
    lt, mask = _pad_rows([s.token_logp_trainer for s in samples], width, device)
    lr, _ = _pad_rows([s.token_logp_rollout for s in samples], width, device)
    zt, lmask = _pad_rows([s.latent_logp_trainer for s in samples], lwidth, device)
    zr, _ = _pad_rows([s.latent_logp_rollout for s in samples], lwidth, device)
    f = lambda vals, dt=torch.float32: torch.tensor(vals, dtype=dt, device=device)      # noqa: E731
    return PackedRollouts(lt, lr, mask, zt, zr, lmask, f([float(s.reward) for s in samples]),
                          f(gidx, torch.int64), f([float(s.n_tokens) for s in samples]),
                          f(gaps, torch.int64), len(groups))


def batched_loss(p: PackedRollouts, config: LossConfig) -> dict:
    """The objective over a packed batch. Returns tensors: ``total`` (scalar, differentiable in
    ``p.logp_trainer`` / ``p.lat_trainer``), the parts ``pg`` / ``latent`` / ``overlong``, the
    mean importance weight ``tis``, per-group totals ``per_group`` ``(G,)``, the kept-sample
    mask ``kept`` ``(N,)`` and the advantages ``advantage`` ``(N,)``."""
    G = p.n_groups
    ones = torch.ones_like(p.reward)
    count = torch.zeros(G, device=p.reward.device).index_add(0, p.group, ones)
    mean = torch.zeros(G, device=p.reward.device).index_add(0, p.group, p.reward) / count.clamp(min=1.0)
    adv = p.reward - mean[p.group]
    # dynamic sampling: a group whose rewards are all equal has no signal
    hi = torch.full((G,), -math.inf, device=p.reward.device).scatter_reduce(0, p.group, p.reward, "amax")
    lo = torch.full((G,), math.inf, device=p.reward.device).scatter_reduce(0, p.group, p.reward, "amin")
    kept = (hi > lo)[p.group].to(p.reward.dtype)

    def ratio(new, old, mask, normalise):
        d = ((new - old) * mask).sum(dim=1)
        if normalise:
            d = d / mask.sum(dim=1).clamp(min=1.0)
        return torch.exp(d)

    def surrogate(r, eps_lo, eps_hi):
        c = torch.clamp(r, 1.0 - eps_lo, 1.0 + eps_hi)
        return torch.minimum(r * adv, c * adv) if config.pessimistic else c * adv

    r_tok = ratio(p.logp_trainer, p.logp_rollout, p.mask, config.length_normalize)
    # importance weight of stale rollouts: the plain (never length-normalised) sequence ratio,
    # truncated, and treated as a constant
    r_plain = ratio(p.logp_trainer, p.logp_rollout, p.mask, False)
    w = torch.where(p.gap == 0, torch.ones_like(r_plain), torch.clamp(r_plain, max=config.tis_clip)).detach()
    pg_i = surrogate(r_tok, config.clip_eps_low, config.clip_eps_high) * w
    has_lat = (p.lat_mask.sum(dim=1) > 0).to(p.reward.dtype)
    r_lat = ratio(p.lat_trainer, p.lat_rollout, p.lat_mask, False)
    lat_i = surrogate(r_lat, config.latent_clip_eps_low, config.latent_clip_eps_high) * w * has_lat
    ol_i = config.overlong_penalty * (p.n_tokens - float(config.overlong_cache)).clamp(min=0.0)
    z = float(config.loss_normalizer)
    pg, lat, ol = (pg_i * kept).sum() / z, (lat_i * kept).sum() / z, (ol_i * kept).sum() / z
    per_group = torch.zeros(G, device=p.reward.device).index_add(0, p.group, (pg_i + lat_i + ol_i) * kept) / z
    n_kept = kept.sum()
    return {"total": pg + lat + ol, "pg": pg, "latent": lat, "overlong": ol,
            "tis": (w * kept).sum() / n_kept.clamp(min=1.0), "per_group": per_group, "kept": kept,
            "advantage": adv, "n_kept": n_kept}


# ---------------------------------------------------------------------------
# the reference's per-piece helpers (floats or tensors)
# ---------------------------------------------------------------------------
def mean_center(rewards):
    """Dr.GRPO advantages: reward minus the group mean (no division by the deviation)."""
    if _is_t(rewards):
        if rewards.numel() == 0:
            raise LossError("rewards are empty")
        return rewards - rewards.mean()
    if len(rewards) == 0:
        raise LossError("rewards are empty")
    _finite(rewards, "rewards")
    mean = math.fsum(rewards) / len(rewards)
    return tuple(r - mean for r in rewards)


def all_equal_reward(rewards: Sequence[float]) -> bool:
    if len(rewards) == 0:
        raise LossError("rewards are empty")
    return max(rewards) == min(rewards)


def drop_zero_advantage_groups(groups: Sequence[Group]) -> tuple:
    """Dynamic sampling on the host: groups whose rewards are all equal carry no gradient."""
    for g in groups:
        if len(g.samples) == 0:
            raise LossError(f"group {g.prompt_id!r} has no samples")
    return tuple(g for g in groups if not all_equal_reward([s.reward for s in g.samples]))


def sequence_ratio(logp_new, logp_old, *, length_normalize: bool = False):
    """``exp(sum(new - old))`` over a sequence (``exp(mean)`` when length-normalised)."""
    n_new, n_old = len(logp_new), len(logp_old)
    if n_new == 0 or n_new != n_old:
        raise LossError("log-prob sequences must be non-empty and equally long")
    if _is_t(logp_new) or _is_t(logp_old):
        d = torch.as_tensor(logp_new) - torch.as_tensor(logp_old)
        return torch.exp(d.mean() if length_normalize else d.sum())
    _finite((*logp_new, *logp_old), "log-probs")
    total = math.fsum(a - b for a, b in zip(logp_new, logp_old))
    return math.exp(total / n_new if length_normalize else total)


def clip_higher(ratio, eps_low: float, eps_high: float):
    """Clip into ``[1 - eps_low, 1 + eps_high]``: more room upward than downward."""
    if min(eps_low, eps_high) < 0.0:
        raise LossError("clip epsilons must be >= 0")
    if _is_t(ratio):
        return torch.clamp(ratio, 1.0 - eps_low, 1.0 + eps_high)
    _finite((ratio,), "ratio")
    return min(max(ratio, 1.0 - eps_low), 1.0 + eps_high)


def staleness(trainer_version: int, policy_version: int) -> int:
    if policy_version > trainer_version:
        raise LossError("a rollout cannot come from a newer policy than the trainer's")
    return trainer_version - policy_version


def truncated_is(logp_trainer, logp_rollout, k: int, tis_clip: float):
    """Importance weight of a rollout ``k`` versions stale: 1 when fresh, else
    ``min(sequence ratio, tis_clip)``."""
    if k < 0 or tis_clip < 1.0:
        raise LossError("staleness must be >= 0 and tis_clip >= 1")
    tensor = _is_t(logp_trainer) or _is_t(logp_rollout)
    if k == 0:
        return torch.ones(()) if tensor else 1.0
    r = sequence_ratio(logp_trainer, logp_rollout)
    return torch.clamp(r, max=tis_clip) if tensor else min(r, tis_clip)


def overlong_soft_penalty(n_tokens: int, cache: int, penalty: float) -> float:
    if min(n_tokens, cache) < 0 or penalty < 0.0:
        raise LossError("overlong arguments must be >= 0")
    return penalty * max(0, n_tokens - cache)


def gaussian_log_density(z, mu, sigma):
    """Sum of independent 1-D Gaussian log-densities."""
    if len(z) == 0 or not (len(z) == len(mu) == len(sigma)):
        raise LossError("z, mu and sigma must be non-empty and equally long")
    if _is_t(z) or _is_t(mu) or _is_t(sigma):
        z, mu, sigma = (torch.as_tensor(t, dtype=torch.float32) for t in (z, mu, sigma))
        return -0.5 * (((z - mu) / sigma) ** 2 + 2.0 * torch.log(sigma) + math.log(2 * math.pi)).sum()
    _finite((*z, *mu, *sigma), "gaussian inputs")
    if min(sigma) <= 0.0:
        raise LossError("sigma must be positive")
    return -0.5 * math.fsum(((a - b) / s) ** 2 + 2.0 * math.log(s) + math.log(2.0 * math.pi)
                            for a, b, s in zip(z, mu, sigma))


def latent_ratio(logp_new, logp_old):
    """Ratio over the latent thoughts of a sample; 1 when the sample has none."""
    if len(logp_new) == 0 and len(logp_old) == 0:
        return 1.0
    if len(logp_new) == 0 or len(logp_old) == 0:
        raise LossError("only one side has latent log-probs")
    return sequence_ratio(logp_new, logp_old)


def routing_table(traces: Sequence[RoutingTrace], n_tokens: int, n_layers: int, top_k: int) -> tuple:
    """Dense ``(token, layer) -> expert ids`` table for routing replay; every cell exactly once."""
    if min(n_tokens, n_layers, top_k) <= 0:
        raise LossError("n_tokens, n_layers and top_k must be positive")
    grid = [[None] * n_layers for _ in range(n_tokens)]
    for t in traces:
        if not (0 <= t.token_index < n_tokens and 0 <= t.layer_index < n_layers):
            raise LossError("a routing trace lies outside the (token, layer) grid")
        if len(t.expert_ids) != top_k or min(t.expert_ids) < 0:
            raise LossError("a routing trace needs top_k non-negative expert ids")
        if grid[t.token_index][t.layer_index] is not None:
            raise LossError("two routing traces for one (token, layer)")
        grid[t.token_index][t.layer_index] = tuple(t.expert_ids)
    if any(cell is None for row in grid for cell in row):
        raise LossError("a (token, layer) cell has no routing trace")
    return tuple(tuple(row) for row in grid)


def gspo_dapo_loss(group: Group, config: LossConfig, trainer_version: int) -> LossBreakdown:
    """One group's objective (the batched loss on a batch of one group): the sum over samples
    of ``tis * clip(ratio) * advantage`` for the tokens and, separately clipped, for the latent
    thoughts, plus the overlong penalty, over ``loss_normalizer``. Equal rewards: all zero."""
    packed = pack_groups((group,), trainer_version, config)
    out = batched_loss(packed, config)
    n_kept = int(out["n_kept"])
    tensor_in = any(_is_t(x) for s in group.samples
                    for x in (s.token_logp_trainer, s.token_logp_rollout, s.latent_logp_trainer,
                              s.latent_logp_rollout))
    if n_kept == 0 and not tensor_in:
        return LossBreakdown(pg=0.0, tis=0.0, overlong=0.0, latent=0.0, n_kept=0, total=0.0)
    pick = (lambda t: t) if tensor_in else (lambda t: float(t))
    return LossBreakdown(pg=pick(out["pg"]), tis=pick(out["tis"]), overlong=pick(out["overlong"]),
                         latent=pick(out["latent"]), n_kept=n_kept, total=pick(out["total"]))
