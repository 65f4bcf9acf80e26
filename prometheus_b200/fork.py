"""Serving-engine deltas: recurrence bucketing, latent chunk validation, decode mode, KV
tier order, routing capture for replay, prefix groups for sub-agents, test-time-training
hooks. API parity with the reference ``sglang-fork/sglang_fork/fork.py:37-212``.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class ForkError(ValueError):
    """A serving-side argument is invalid."""


class DecodeMode(str, Enum):
    VERBAL = "verbal"
    LATENT = "latent"

    def __str__(self) -> str:
        return self.value


class KvTier(str, Enum):
    HBM = "hbm"
    GRACE = "grace"
    NVME = "nvme"
    DISTRIBUTED = "distributed"

    def __str__(self) -> str:
        return self.value


RECURRENCE_BUCKETS = (1, 2, 4, 8, 16)
RECURRENCE_MAX = 16
LATENT_CHUNK_MIN = 4
LATENT_CHUNK_MAX = 64
SUBAGENT_DEPTH_MAX = 3
KV_TIER_ORDER = (KvTier.HBM, KvTier.GRACE, KvTier.NVME, KvTier.DISTRIBUTED)


@dataclass(frozen=True)
class RecurrencePlan:
    r: int
    budget: int
    kv_shared: bool = True


@dataclass(frozen=True)
class LatentChunk:
    n_thoughts: int
    mode: DecodeMode = DecodeMode.LATENT


@dataclass(frozen=True)
class RoutingRecord:
    token_index: int
    layer_index: int
    expert_ids: tuple


@dataclass(frozen=True)
class PrefixGroup:
    parent_session: str
    child_sessions: tuple
    depth: int


@dataclass(frozen=True)
class TttHook:
    task_id: str
    lora_id: str


def bucket_recurrence(r: int, budget: int) -> RecurrencePlan:
    """Round the requested core-block iteration count up to the next bucket (so batches
    stay regular), then cap it by the budget and by RECURRENCE_MAX."""
    if r <= 0 or budget <= 0:
        raise ForkError("r and budget must be positive")
    up = next((b for b in RECURRENCE_BUCKETS if b >= r), RECURRENCE_MAX)
    return RecurrencePlan(r=min(up, budget, RECURRENCE_MAX), budget=budget, kv_shared=True)


def validate_latent_chunk(n_thoughts: int) -> LatentChunk:
    if not (LATENT_CHUNK_MIN <= n_thoughts <= LATENT_CHUNK_MAX):
        raise ForkError(f"n_thoughts {n_thoughts} outside [{LATENT_CHUNK_MIN}, {LATENT_CHUNK_MAX}]")
    return LatentChunk(n_thoughts=n_thoughts)


def decode_mode(in_think: bool, halt: bool) -> DecodeMode:
    """Latent decoding only inside a think span that has not halted."""
    return DecodeMode.LATENT if (in_think and not halt) else DecodeMode.VERBAL


def next_kv_tier(tier: KvTier):
    """The next colder tier, None after the last."""
    try:
        i = KV_TIER_ORDER.index(KvTier(tier))
    except ValueError as exc:
        raise ForkError(f"unknown kv tier {tier!r}") from exc
    return KV_TIER_ORDER[i + 1] if i + 1 < len(KV_TIER_ORDER) else None


def swap_waiting_session(decoding: bool) -> KvTier:
    """A session that is decoding stays in HBM; one waiting on a tool moves to host memory."""
    return KvTier.HBM if decoding else KvTier.GRACE


def capture_routing(token_index: int, layer_index: int, expert_ids, top_k: int) -> RoutingRecord:
    ids = tuple(expert_ids)
    if top_k <= 0:
        raise ForkError("top_k must be positive")
    if len(ids) != top_k:
        raise ForkError(f"expert_ids length {len(ids)} != top_k {top_k}")
    if any(e < 0 for e in ids):
        raise ForkError(f"negative expert id {min(ids)}")
    if len(set(ids)) != len(ids):
        raise ForkError("duplicate expert id")
    return RoutingRecord(token_index, layer_index, ids)


def schedule_prefix_group(parent_session: str, child_sessions, depth: int) -> PrefixGroup:
    kids = tuple(child_sessions)
    if not parent_session:
        raise ForkError("parent_session must be non-empty")
    if not kids:
        raise ForkError("child_sessions must be non-empty")
    if parent_session in kids:
        raise ForkError("parent_session must not appear in child_sessions")
    if not (1 <= depth <= SUBAGENT_DEPTH_MAX):
        raise ForkError(f"depth {depth} outside [1, {SUBAGENT_DEPTH_MAX}]")
    return PrefixGroup(parent_session, kids, depth)


def register_ttt(task_id: str, lora_id: str) -> TttHook:
    if not task_id or not lora_id:
        raise ForkError("task_id and lora_id must be non-empty")
    return TttHook(task_id, lora_id)
