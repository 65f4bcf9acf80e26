"""Evaluation harness: suite registry, ``prometheus.eval_result`` payloads, a fail-closed
decontamination index and a runner.

API parity with the reference ``evals/__init__.py`` (``PUBLIC_SUITES`` :25-48, metric names
:50-61, ``result_envelope`` :170-214, ``DecontamIndex`` :217-279, ``Runner`` :311-374). Two
deliberate differences: the runner takes its items from a provider the caller passes (the
reference fabricates fixture items when asked to run a public suite; the fixture provider is
still here, by name, for tests), and ``Runner.run_model`` scores a causal language model by
exact-match of its greedy continuation, so a trained ``engine.Trainer`` or the fp32 model can
be evaluated without writing a ``predict`` function.
"""
from __future__ import annotations

import hashlib
import re
from dataclasses import dataclass, field
from datetime import datetime, timezone
from enum import Enum
from typing import Callable, Iterable, Sequence

SCHEMA_ID = "prometheus.eval_result"
SCHEMA_VERSION = 1

PUBLIC_SUITES: tuple[str, ...] = (
    "re_bench", "mle_bench", "paperbench", "speedrun", "metr_time_horizon", "swe_bench_verified",
    "swe_bench_pro", "terminal_bench", "competitive_programming", "aime", "hmmt", "frontiermath",
    "minif2f", "putnambench", "arc_agi_1", "arc_agi_2", "arc_agi_3", "hle", "gpqa",
    "long_context_128k", "long_context_1m", "forecasting",
)
FORECASTING_METRICS: tuple[str, ...] = ("brier", "log_score", "paper_pnl", "leak_probe")
EFFICIENCY_METRICS: tuple[str, ...] = ("tokens_to_solve", "latent_steps", "recurrence_iterations")
SPLITS = ("train", "val", "test", "held_out")
NGRAM_N = 8
_WORD = re.compile(r"[0-9A-Za-z_]+")


class Split(str, Enum):
    TRAIN = "train"
    VAL = "val"
    TEST = "test"
    HELD_OUT = "held_out"


class DecontamStatus(str, Enum):
    PENDING = "pending"
    CLEAN = "clean"
    FLAGGED = "flagged"
    NOT_APPLICABLE = "not_applicable"


class UnknownSuiteError(KeyError):
    """The slug is not one of ``PUBLIC_SUITES``."""


class HarnessVersionError(ValueError):
    """A report without a harness version."""


class DecontamError(ValueError):
    """The index is empty (fail closed) or has no method hash."""


@dataclass(frozen=True)
class EvalItem:
    item_id: str
    suite: str
    split: str
    prompt: str
    answer: str | None = None
    metadata: dict = field(default_factory=dict)


@dataclass(frozen=True)
class EvalConfig:
    suite: str
    split: str
    checkpoint_id: str
    harness_version: str
    n_items: int | None = None
    seed: int = 0


@dataclass(frozen=True)
class Decontamination:
    status: DecontamStatus
    against: tuple = ()
    method_hash: str | None = None


def require_suite(slug: str) -> str:
    if slug not in PUBLIC_SUITES:
        raise UnknownSuiteError(slug)
    return slug


def _version(v) -> str:
    if not isinstance(v, str) or not v.strip():
        raise HarnessVersionError("missing harness_version")
    return v


def _split(s) -> str:
    s = s.value if isinstance(s, Split) else s
    if s not in SPLITS:
        raise ValueError(f"split must be one of {sorted(SPLITS)}")
    return s


def _words(text: str) -> list[str]:
    return [w.lower() for w in _WORD.findall(text)]


def _grams(words: Sequence[str]) -> set:
    if not words:
        return set()
    n = min(NGRAM_N, len(words))
    return {tuple(words[i:i + n]) for i in range(len(words) - n + 1)}


def _text_of(prompt: str, answer: str | None) -> str:
    return f"{prompt}\n{answer}" if answer else prompt


def result_envelope(*, result_id: str, suite: str, split: str, checkpoint_id: str, metrics: dict,
                    n_items: int, harness_version: str, decontamination: Decontamination | None = None,
                    per_item_hash: str | None = None, config_hash: str | None = None,
                    job_id: str | None = None, created_at: str | None = None) -> dict:
    """A ``prometheus.eval_result`` v1 payload (``contracts.validate`` accepts it)."""
    _version(harness_version)
    require_suite(suite)
    split = _split(split)
    if isinstance(n_items, bool) or not isinstance(n_items, int) or n_items < 0:
        raise ValueError("n_items must be a non-negative int")
    out = {"schema_id": SCHEMA_ID, "schema_version": SCHEMA_VERSION, "result_id": result_id, "suite": suite,
           "split": split, "checkpoint_id": checkpoint_id, "metrics": dict(metrics), "n_items": n_items,
           "created_at": created_at or datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")}
    if decontamination is not None:
        st = decontamination.status
        d = {"status": st.value if isinstance(st, DecontamStatus) else str(st), "against": list(decontamination.against)}
        if decontamination.method_hash is not None:
            d["method_hash"] = decontamination.method_hash
        out["decontamination"] = d
    for key, val in (("per_item_hash", per_item_hash), ("config_hash", config_hash), ("job_id", job_id)):
        if val is not None:
            out[key] = val
    return out


class DecontamIndex:
    """Eval items as 8-gram sets plus whole normalised texts, per suite. ``is_clean`` is False
    for a text that shares an n-gram (or is equal after normalisation) and raises when there is
    nothing to compare against: a missing index never reads as clean."""

    def __init__(self) -> None:
        self._by_suite: dict[str, tuple[set, set]] = {}
        self._hash: str | None = None

    def add(self, item: EvalItem) -> None:
        words = _words(_text_of(item.prompt, item.answer))
        grams, texts = self._by_suite.setdefault(item.suite, (set(), set()))
        grams |= _grams(words)
        texts.add(" ".join(words))
        h = hashlib.sha256()
        all_grams = sorted(set().union(*(g for g, _ in self._by_suite.values())))
        all_texts = sorted(set().union(*(t for _, t in self._by_suite.values())))
        for g in all_grams:
            h.update((" ".join(g) + "\n").encode())
        for t in all_texts:
            h.update((t + "\n").encode())
        self._hash = h.hexdigest()

    def _view(self, against):
        suites = self._by_suite if against is None else {s: self._by_suite[s] for s in against if s in self._by_suite}
        grams = set().union(*(g for g, _ in suites.values())) if suites else set()
        texts = set().union(*(t for _, t in suites.values())) if suites else set()
        return grams, texts

    def is_clean(self, text: str, *, against: tuple | None = None) -> bool:
        grams, texts = self._view(against)
        if self._hash is None or (not grams and not texts):
            raise DecontamError("decontamination index is empty or method hash is unset")
        words = _words(text)
        return " ".join(words) not in texts and _grams(words).isdisjoint(grams)

    def method_hash(self) -> str:
        if self._hash is None:
            raise DecontamError("method hash is unset")
        return self._hash


def fixture_items(suite: str, split: str, n: int) -> list[EvalItem]:
    """In-memory stand-in items (tests and dry runs only)."""
    return [EvalItem(f"{suite}-{split}-{i}", suite, split, f"{suite} {split} in-memory fixture item {i}", str(i),
                     {"fixture": True, "index": i}) for i in range(n)]


def _items_hash(items: Iterable[EvalItem]) -> str:
    h = hashlib.sha256()
    for it in items:
        h.update("\0".join((it.item_id, it.suite, it.split, it.prompt, it.answer or "")).encode() + b"\n")
    return h.hexdigest()


class Runner:
    """One suite, one checkpoint. ``items`` is a list or a callable ``(suite, split, n) -> items``;
    without it the fixture provider is used."""

    def __init__(self, config: EvalConfig, index: DecontamIndex | None = None,
                 items: Sequence[EvalItem] | Callable | None = None) -> None:
        _version(config.harness_version)
        require_suite(config.suite)
        _split(config.split)
        self.config, self.index, self._items = config, index, items

    def load_items(self) -> list[EvalItem]:
        n = 2 if self.config.n_items is None else self.config.n_items
        if isinstance(n, bool) or n < 0:
            raise ValueError("n_items must be a non-negative int")
        if self._items is None:
            return fixture_items(self.config.suite, _split(self.config.split), n)
        got = self._items(self.config.suite, _split(self.config.split), n) if callable(self._items) else list(self._items)
        return list(got)[:n] if self.config.n_items is not None else list(got)

    def run(self, predict: Callable[[EvalItem], str], extra_metrics: dict | None = None) -> dict:
        cfg = self.config
        items = self.load_items()
        correct, flagged = 0, False
        for it in items:
            if it.answer is not None and predict(it) == it.answer:
                correct += 1
            if self.index is not None and not self.index.is_clean(_text_of(it.prompt, it.answer), against=(it.suite,)):
                flagged = True
        if self.index is None:
            dec = Decontamination(DecontamStatus.PENDING)
        else:
            dec = Decontamination(DecontamStatus.FLAGGED if flagged else DecontamStatus.CLEAN, (cfg.suite,),
                                  self.index.method_hash())
        metrics = {"pass_at_1": correct / len(items) if items else 0.0}
        metrics.update(extra_metrics or {})
        cfg_blob = f"{cfg.suite}\n{cfg.split}\n{cfg.checkpoint_id}\n{cfg.harness_version}\n{cfg.n_items}\n{cfg.seed}\n"
        return result_envelope(result_id=f"eval-{cfg.suite}-{cfg.checkpoint_id}", suite=cfg.suite, split=_split(cfg.split),
                               checkpoint_id=cfg.checkpoint_id, metrics=metrics, n_items=len(items),
                               harness_version=cfg.harness_version, decontamination=dec,
                               per_item_hash=_items_hash(items), config_hash=hashlib.sha256(cfg_blob.encode()).hexdigest())

    def run_model(self, logits_fn: Callable, encode: Callable[[str], list], decode: Callable[[list], str],
                  max_new_tokens: int = 16) -> dict:
        """Greedy decoding with ``logits_fn(token_ids (1, S)) -> logits (1, S, V)``; an item passes
        when the decoded continuation, stripped, equals its answer. ``tokens_to_solve`` is the
        mean number of generated tokens."""
        import torch

        spent = []

        def predict(item: EvalItem) -> str:
            ids = list(encode(item.prompt))
            start = len(ids)
            want = len(encode(item.answer)) if item.answer else max_new_tokens
            for _ in range(min(max_new_tokens, max(1, want))):
                with torch.no_grad():
                    nxt = int(logits_fn(torch.tensor([ids]))[0, -1].argmax())
                ids.append(nxt)
            spent.append(len(ids) - start)
            return decode(ids[start:]).strip()

        result = self.run(predict)
        if spent:
            result["metrics"]["tokens_to_solve"] = sum(spent) / len(spent)
        return result
