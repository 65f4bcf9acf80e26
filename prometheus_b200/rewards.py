"""Learned-reward plumbing: rubric panels, contrastive-pair filters and the tampering detector.

The arithmetic and the validation live in C++ (``native.rewards``: weighted rubric scores,
the disagreement down-weighting, hack classification of a trajectory view, pair filters). This
module is the object layer a training job talks to, with the reward-API request / response
records of the contracts package on either side (reference rl/rewards/src/lib.rs:45-554):

* ``RubricPanel``: several graders score one output against a weighted rubric; the panel's value
  is the mean of the graders' weighted scores times ``1 - spread`` (spread = max - min), so
  disagreement lowers the reward and never drops a sample. ``passed`` is ``value > 0.5``.
* ``TamperPairFilter`` / ``RescoreFilter``: keep a contrastive pair only when its negative is a
  confirmed hack and its positive is clean, resp. when the positive re-scores strictly higher.
* ``TamperingDetector``: score 0 with the ``tampering`` flag for a confirmed hack, 1 otherwise.
* ``HeldOutHacks``: planted hacks for measuring the detector's recall; a training pair that
  names one of them is refused (``HeldOutLeak``).

Nothing here reads a clock: ``scored_at`` is the caller's string.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Iterable, Sequence

from .native import NativeError
from .native import rewards as _rw

DISAGREE_EPS = _rw.DISAGREE_EPS
Criterion, TrajectoryView = _rw.Criterion, _rw.TrajectoryView
refuse_exact = _rw.refuse_exact
HACK_KINDS = ("test_write", "special_case", "visible_pass_hidden_fail")

REQUEST_SCHEMA, RESPONSE_SCHEMA, SCHEMA_VERSION = "prometheus.reward_request", "prometheus.reward_response", 1


def _error(kind: str, message: str) -> NativeError:
    e = NativeError(message)
    e.kind = kind
    return e


def reward_request(request_id: str, task_id: str, rollout_id: str, trajectory_hash: str, verifier_id: str,
                   env_snapshot_id: str) -> dict:
    return {"schema_id": REQUEST_SCHEMA, "schema_version": SCHEMA_VERSION, "request_id": request_id,
            "task_id": task_id, "rollout_id": rollout_id, "trajectory_hash": trajectory_hash,
            "verifier_id": verifier_id, "env_snapshot_id": env_snapshot_id}


def _check_request(req: dict) -> None:
    if req.get("schema_id") != REQUEST_SCHEMA or req.get("schema_version") != SCHEMA_VERSION:
        raise _error("Schema", f"schema mismatch: expected {REQUEST_SCHEMA} v{SCHEMA_VERSION}, got "
                               f"{req.get('schema_id')} v{req.get('schema_version')}")


def _response(req: dict, scorer_id: str, scored_at: str, score: float, passed: bool, flags: Sequence[str] = (),
              evidence: dict | None = None) -> dict:
    out = {"schema_id": RESPONSE_SCHEMA, "schema_version": SCHEMA_VERSION, "request_id": req["request_id"],
           "task_id": req.get("task_id", ""), "score": float(score), "passed": bool(passed), "flags": list(flags),
           "scorer_id": scorer_id, "scored_at": scored_at}
    if evidence is not None:
        out["evidence"] = evidence
    return out


@dataclass
class Rubric:
    id: str
    criteria: list = field(default_factory=list)          # [(id, prompt, weight)] in scoring order

    def add(self, cid: str, prompt: str, weight: float = 1.0) -> "Rubric":
        self.criteria.append((cid, prompt, float(weight)))
        return self

    def total_weight(self) -> float:
        return float(sum(w for _c, _p, w in self.criteria))

    def native(self) -> list:
        return [Criterion(c, p, w) for c, p, w in self.criteria]


class ScriptedJudge:
    """A judge that answers from a table of exact prompts; anything else is unverifiable."""

    def __init__(self):
        self.replies: dict[str, str] = {}

    def insert(self, prompt: str, reply: str) -> None:
        self.replies[prompt] = reply

    def __call__(self, prompt: str) -> str:
        if prompt not in self.replies:
            raise _error("Unverifiable", f"unverifiable: no scripted reply for prompt: {prompt}")
        return self.replies[prompt]


def grader_prompt(grader_id: str, criterion_id: str, criterion_prompt: str, output: str) -> str:
    return f"grader:{grader_id}\ncriterion:{criterion_id}\n{criterion_prompt}\n\n{output}"


@dataclass
class RubricScore:
    grader_id: str
    scores: list          # [(criterion id, value)] in rubric order
    weighted: float


class RubricPanel:
    def __init__(self, panel_id: str, rubric: Rubric, grader_ids: Sequence[str], judge: Callable[[str], str]):
        self.id, self.rubric, self.grader_ids, self.judge = panel_id, rubric, list(grader_ids), judge

    def score(self, output: str) -> list[RubricScore]:
        replies: list[str] = []

        def recording(prompt: str) -> str:
            reply = self.judge(prompt)
            replies.append(reply)
            return reply

        weighted = _rw.rubric_score(self.rubric.native(), self.grader_ids, recording, output)
        n = len(self.rubric.criteria)
        out = []
        for g, (gid, w) in enumerate(weighted):
            vals = [float(r.strip()) for r in replies[g * n:(g + 1) * n]]
            out.append(RubricScore(gid, [(c[0], v) for c, v in zip(self.rubric.criteria, vals)], w))
        return out

    @staticmethod
    def combine(scores: Iterable[RubricScore]) -> float:
        return _rw.rubric_combine([s.weighted for s in scores])

    def verify(self, req: dict, output: str, scored_at: str) -> dict:
        _check_request(req)
        value = self.combine(self.score(output))
        evidence = {"kind": "rubric", "hash": hashlib.sha256(output.encode("utf-8")).hexdigest()}
        return _response(req, self.id, scored_at, value, value > 0.5, evidence=evidence)


@dataclass(frozen=True)
class ContrastivePair:
    """One RLCD pair; the assumed label is "prefer positive"."""
    input: str
    positive_prompt: str
    negative_prompt: str
    positive: str
    negative: str


class HeldOutHacks:
    def __init__(self):
        self._views: dict[str, TrajectoryView] = {}

    def insert(self, hack_id: str, view: TrajectoryView) -> None:
        self._views[hack_id] = view                      # same id again replaces, it does not add

    def contains(self, hack_id: str) -> bool:
        return hack_id in self._views

    def get(self, hack_id: str):
        return self._views.get(hack_id)

    def __len__(self) -> int:
        return len(self._views)

    def eval(self, detector: "TamperingDetector") -> "DetectReport":
        views = [self._views[k] for k in sorted(self._views)]
        flagged = sum(1 for v in views if detector.is_hack(v))
        assert not views or abs(_rw.held_out_recall(views) - flagged / len(views)) < 1e-12
        return DetectReport(len(views), flagged)


@dataclass(frozen=True)
class DetectReport:
    n: int
    flagged: int

    def recall(self) -> float:
        return 0.0 if self.n == 0 else self.flagged / self.n


class TamperPairFilter:
    """Keeps a pair only when the negative is a confirmed hack and the positive is clean. The
    pair's text is never looked at; the two trajectory views decide. ``trajectory_ids`` (with
    ``held_out``) guards the rule that planted evaluation hacks never become training pairs."""

    def keep(self, pair: ContrastivePair, positive: TrajectoryView, negative: TrajectoryView,
             held_out: HeldOutHacks | None = None, trajectory_ids: Sequence[str] = ()) -> None:
        if held_out is not None:
            for tid in trajectory_ids:
                if held_out.contains(tid):
                    raise _error("HeldOutLeak", "held-out hack used as training pair")
        _rw.tamper_pair_keep(positive, negative)


class RescoreFilter:
    def keep(self, positive: float, negative: float) -> None:
        _rw.rescore_keep(float(positive), float(negative))


class TamperingDetector:
    def __init__(self, detector_id: str):
        self.id = detector_id

    @staticmethod
    def kinds(view: TrajectoryView) -> list:
        return list(view.kinds())

    @staticmethod
    def is_hack(view: TrajectoryView) -> bool:
        return bool(view.is_confirmed_hack())

    def verify(self, req: dict, view: TrajectoryView, scored_at: str) -> dict:
        _check_request(req)
        score, passed, flags = _rw.tamper_verify(view)
        return _response(req, self.id, scored_at, score, passed, flags)
