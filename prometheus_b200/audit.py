"""Discrete-vs-latent audit: force a checkpoint into discrete chain-of-thought, compare the
answers of the two modes problem by problem, read latent thoughts back as token windows, and
check that planted latent bugs are visible.

API parity with the reference ``audit/__init__.py`` (:33-251). Tensors are torch (CPU or GPU;
numpy arrays are accepted and converted), so the thought logits of a trained model can be
audited where they live.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum

import torch

TOKENS_PER_THOUGHT = 8      # compression target of the latent curriculum


class AuditError(ValueError):
    """A checkpoint id, answer pair or tensor is not auditable."""


class Mode(str, Enum):
    DISCRETE = "discrete"
    LATENT = "latent"


class BugKind(str, Enum):
    ANSWER_SWAP = "answer_swap"
    DECODE_FLIP = "decode_flip"
    HALT_UNPINNED = "halt_unpinned"


@dataclass(frozen=True)
class CheckpointMode:
    checkpoint_id: str
    mode: Mode


@dataclass(frozen=True)
class AnswerPair:
    problem_id: str
    discrete_answer: str
    latent_answer: str
    gold: str | None = None


@dataclass(frozen=True)
class Divergence:
    problem_id: str
    discrete_answer: str
    latent_answer: str
    gold: str | None
    discrete_correct: bool | None
    latent_correct: bool | None
    diverge: bool


@dataclass(frozen=True)
class ThoughtStep:
    index: int
    token_ids: tuple


@dataclass(frozen=True)
class PlantedBug:
    kind: BugKind
    found: bool
    evidence: str


def force_discrete(checkpoint_id: str) -> CheckpointMode:
    if not isinstance(checkpoint_id, str) or not checkpoint_id.strip():
        raise AuditError("empty or whitespace-only checkpoint_id")
    return CheckpointMode(checkpoint_id, Mode.DISCRETE)


def compare_answers(pair: AnswerPair) -> Divergence:
    if not isinstance(pair.problem_id, str) or pair.problem_id == "":
        raise AuditError("empty problem_id")
    known = pair.gold is not None
    return Divergence(pair.problem_id, pair.discrete_answer, pair.latent_answer, pair.gold,
                      pair.discrete_answer == pair.gold if known else None,
                      pair.latent_answer == pair.gold if known else None,
                      pair.discrete_answer != pair.latent_answer)


def compare_suite(pairs: tuple) -> tuple:
    if not isinstance(pairs, tuple) or not pairs:
        raise AuditError("empty pairs")
    return tuple(compare_answers(p) for p in pairs)


def divergence_rate(pairs: tuple) -> float:
    """Share of problems on which the two modes disagree."""
    rows = compare_suite(pairs)
    return sum(r.diverge for r in rows) / len(rows)


def _tensor(x, what: str) -> torch.Tensor:
    if x is None:
        raise AuditError(f"{what} required")
    try:
        return torch.as_tensor(x)
    except Exception as e:      # noqa: BLE001 - any failure to view the input as a tensor
        raise AuditError(f"{what} must be an array") from e


def decode_thoughts(logits) -> tuple:
    """Greedy read-out of ``(n_thoughts, 8, vocab)`` logits: one ``ThoughtStep`` per thought,
    the smallest id on ties."""
    t = _tensor(logits, "logits")
    if t.ndim != 3:
        raise AuditError(f"logits rank must be 3, got {t.ndim}")
    n, window, vocab = t.shape
    if n < 1:
        raise AuditError("n_thoughts must be >= 1")
    if window != TOKENS_PER_THOUGHT:
        raise AuditError(f"thought window must be {TOKENS_PER_THOUGHT}, got {window}")
    if vocab < 1:
        raise AuditError("vocab must be >= 1")
    t = t.float()
    if not bool(torch.isfinite(t).all()):
        raise AuditError("logits must be finite")
    # first index of the maximum: compare against the row maximum, take the first hit
    first = (t == t.amax(-1, keepdim=True)).to(torch.int8).argmax(-1)
    return tuple(ThoughtStep(i, tuple(int(x) for x in first[i].tolist())) for i in range(n))


def find_planted_bug(kind: BugKind, pair: AnswerPair | None, logits, halt_lambdas) -> PlantedBug:
    kind = BugKind(kind)
    if kind is BugKind.ANSWER_SWAP:
        if pair is None:
            raise AuditError("pair required for ANSWER_SWAP")
        d = compare_answers(pair)
        text = f"answers diverge on {d.problem_id}" if d.diverge else f"no answer_swap on {d.problem_id}"
        return PlantedBug(kind, d.diverge, text)
    if kind is BugKind.DECODE_FLIP:
        t = _tensor(logits, "logits")
        a, b = decode_thoughts(t), decode_thoughts(-t.float())
        found = any(x.token_ids != y.token_ids for x, y in zip(a, b))
        rel = "disagrees with" if found else "matches"
        return PlantedBug(kind, found, f"greedy decode of logits {rel} greedy decode of -logits")
    lam = _tensor(halt_lambdas, "halt_lambdas")
    if lam.ndim != 1:
        raise AuditError("halt_lambdas must be 1-D")
    if lam.numel() < 1:
        raise AuditError("halt_lambdas empty")
    last = float(lam[-1])
    found = not math.isfinite(last) or last != 1.0
    text = f"last halt lambda is {last!r}, not pinned to 1.0" if found else "last halt lambda is pinned to 1.0"
    return PlantedBug(kind, found, text)
