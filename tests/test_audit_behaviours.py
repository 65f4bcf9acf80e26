"""Behaviour list of the latent-reasoning audit (``prometheus_b200.audit``; reference
tests/test_audit.py and audit/__init__.py): forcing discrete mode, answer comparison with and
without gold, greedy decode of thought logits (first maximum wins), and the three planted-bug
probes, each of which looks only at its own argument."""
import dataclasses
import math

import numpy as np
import pytest
import torch

from prometheus_b200 import audit as A

B = A.BugKind


def pair(pid, d, l, gold=None):
    return A.AnswerPair(pid, d, l, gold)


# ------------------------------------------------------------------------------ constants / types
def test_constants_and_enums():
    assert A.TOKENS_PER_THOUGHT == 8
    assert [m.value for m in A.Mode] == ["discrete", "latent"]
    assert [k.value for k in A.BugKind] == ["answer_swap", "decode_flip", "halt_unpinned"]
    assert issubclass(A.AuditError, ValueError)
    assert pair("p", "a", "b").gold is None
    for obj in (A.CheckpointMode("c", A.Mode.DISCRETE), pair("p", "a", "b"), A.compare_answers(pair("p", "a", "b")),
                A.ThoughtStep(0, (1,) * 8), A.PlantedBug(B.ANSWER_SWAP, False, "")):
        with pytest.raises(dataclasses.FrozenInstanceError):
            setattr(obj, dataclasses.fields(obj)[0].name, None)


# ------------------------------------------------------------------------------ discrete mode
def test_force_discrete():
    assert A.force_discrete("ckpt-7") == A.CheckpointMode("ckpt-7", A.Mode.DISCRETE)
    assert A.force_discrete("  padded id  ").checkpoint_id == "  padded id  "          # stored as given
    assert A.force_discrete("latent-run-3").mode is A.Mode.DISCRETE                     # the name decides nothing
    for bad in ("", " ", "\t\n", None, 7):
        with pytest.raises(A.AuditError):
            A.force_discrete(bad)


# ------------------------------------------------------------------------------ answers
@pytest.mark.parametrize("d, l, gold, want", [
    ("a", "b", None, (None, None, True)), ("a", "a", None, (None, None, False)),
    ("right", "wrong", "right", (True, False, True)), ("wrong", "right", "right", (False, True, True)),
    ("right", "right", "right", (True, True, False)), ("wrong", "wrong", "right", (False, False, False)),
    ("w1", "w2", "right", (False, False, True)), ("", "", None, (None, None, False)), ("", "x", "", (True, False, True)),
    ("Yes", "yes", "yes", (False, True, True)),
])
def test_compare_answers(d, l, gold, want):
    got = A.compare_answers(pair("p1", d, l, gold))
    assert (got.discrete_correct, got.latent_correct, got.diverge) == want
    assert (got.problem_id, got.discrete_answer, got.latent_answer, got.gold) == ("p1", d, l, gold)


def test_problem_ids():
    assert A.compare_answers(pair(" ", "a", "a")).problem_id == " "                     # whitespace is an id; empty is not
    for bad in ("", None):
        with pytest.raises(A.AuditError):
            A.compare_answers(pair(bad, "a", "b"))


def test_suites_keep_order_and_propagate_errors():
    pairs = (pair("p1", "4", "4", "4"), pair("p2", "4", "5", "4"), pair("p3", "", "x"), pair("p4", "z", "z"))
    rows = A.compare_suite(pairs)
    assert [r.problem_id for r in rows] == ["p1", "p2", "p3", "p4"] and [r.diverge for r in rows] == [False, True, True, False]
    assert A.divergence_rate(pairs) == 0.5 and A.divergence_rate(pairs[:1]) == 0.0
    assert len(A.compare_suite(pairs[:1])) == 1
    for bad in ((), [], list(pairs), (pairs[0], pair("", "a", "b"))):
        with pytest.raises(A.AuditError):
            A.compare_suite(bad)


# ------------------------------------------------------------------------------ decoding thoughts
def test_decode_takes_the_first_maximum():
    logits = np.zeros((2, 8, 4), dtype=np.float32)
    logits[0, :, 2] = 1.0
    logits[0, 3, 1] = 5.0
    steps = A.decode_thoughts(logits)
    assert steps == (A.ThoughtStep(0, (2, 2, 2, 1, 2, 2, 2, 2)), A.ThoughtStep(1, (0,) * 8))   # all-zero row: id 0
    tie = np.zeros((1, 8, 5))
    tie[0, :, 1] = tie[0, :, 3] = 2.0
    assert A.decode_thoughts(tie)[0].token_ids == (1,) * 8
    assert A.decode_thoughts(np.full((3, 8, 1), -4.0)) == tuple(A.ThoughtStep(i, (0,) * 8) for i in range(3))
    assert A.decode_thoughts(torch.tensor(logits)) == steps == A.decode_thoughts(logits.tolist())
    rng = np.random.default_rng(0)
    for n, v in ((1, 2), (3, 7), (5, 33)):
        x = rng.integers(-3, 4, size=(n, 8, v)).astype(np.float32)                      # many exact ties
        want = tuple(A.ThoughtStep(i, tuple(int(np.argmax(x[i, w])) for w in range(8))) for i in range(n))
        assert A.decode_thoughts(x) == want


@pytest.mark.parametrize("bad", [np.zeros((8, 4)), np.zeros((1, 1, 8, 4)), np.zeros((0, 8, 4)), np.zeros((2, 7, 4)),
                                 np.zeros((2, 9, 4)), np.zeros((2, 8, 0)), np.full((1, 8, 2), np.nan), np.full((1, 8, 2), np.inf),
                                 np.full((1, 8, 2), -np.inf), None, "logits", object()])
def test_decode_rejects(bad):
    with pytest.raises(A.AuditError):
        A.decode_thoughts(bad)


# ------------------------------------------------------------------------------ planted bugs
NAN_LOGITS, BAD_HALT = np.array([np.nan], dtype=np.float32), np.array([[1.0]])


def test_answer_swap_probe_looks_at_the_pair_only():
    cases = [(pair("bug", "right", "wrong", "right"), True), (pair("bug", "a", "b"), True), (pair("bug", "a", "a"), False),
             (pair("bug", "wrong", "wrong", "right"), False), (pair("bug", "wrong", "right", "right"), True)]
    for p, found in cases:
        got = A.find_planted_bug(B.ANSWER_SWAP, p, NAN_LOGITS, BAD_HALT)                # bad other arguments are ignored
        assert got.kind is B.ANSWER_SWAP and got.found is found and "bug" in got.evidence
    for p in (None, pair("", "a", "b")):
        with pytest.raises(A.AuditError):
            A.find_planted_bug(B.ANSWER_SWAP, p, None, None)
    assert A.find_planted_bug("answer_swap", cases[0][0], None, None).found


def test_decode_flip_probe():
    x = np.zeros((1, 8, 3), dtype=np.float32)
    x[0, :, 2] = 1.0                                                                     # argmax 2, argmax of -x is 0
    assert A.find_planted_bug(B.DECODE_FLIP, None, x, None).found
    assert not A.find_planted_bug(B.DECODE_FLIP, None, np.zeros((2, 8, 3)), None).found
    assert not A.find_planted_bug(B.DECODE_FLIP, None, np.full((2, 8, 3), 4.5), None).found   # all equal: both pick id 0
    y = np.zeros((1, 8, 3), dtype=np.float32)
    y[0, :, 0] = y[0, :, 1] = 1.0                                                        # tied maxima at 0 and 1: flip picks 2
    assert A.find_planted_bug(B.DECODE_FLIP, None, y, None).found
    assert A.find_planted_bug(B.DECODE_FLIP, pair("", "a", "b"), x, BAD_HALT).found      # pair and halts are ignored
    for bad in (None, NAN_LOGITS.reshape(1, 1, 1), np.zeros((8, 3)), np.full((1, 8, 3), np.inf)):
        with pytest.raises(A.AuditError):
            A.find_planted_bug(B.DECODE_FLIP, None, bad, None)


@pytest.mark.parametrize("lam, found", [([0.2, 0.9], True), ([0.2, 1.0], False), ([1.0], False), ([0.5], True),
                                        ([0.1, math.nextafter(1.0, 0.0)], True), ([0.1, math.nan], True), ([0.1, math.inf], True),
                                        ([0.1, -math.inf], True), ([math.nan, 1.0], False), ([math.inf, 0.3, 1.0], False)])
def test_halt_probe_checks_only_the_last_slot(lam, found):
    got = A.find_planted_bug(B.HALT_UNPINNED, pair("", "a", "b"), NAN_LOGITS, np.array(lam, dtype=np.float64))
    assert got.kind is B.HALT_UNPINNED and got.found is found


def test_halt_probe_argument_errors():
    for bad in (None, np.array(1.0), np.zeros((2, 2)), np.zeros((0,))):
        with pytest.raises(A.AuditError):
            A.find_planted_bug(B.HALT_UNPINNED, None, None, bad)
    with pytest.raises(ValueError):
        A.find_planted_bug("no_such_bug", None, None, None)


def test_random_halt_vectors_and_decodes_follow_the_rules():
    rng = np.random.default_rng(1)
    for _ in range(50):
        lam = rng.random(rng.integers(1, 6))
        if rng.random() < 0.5:
            lam[-1] = 1.0
        assert A.find_planted_bug(B.HALT_UNPINNED, None, None, lam).found == (lam[-1] != 1.0)
        x = rng.integers(-2, 3, size=(rng.integers(1, 4), 8, rng.integers(1, 6))).astype(np.float32)
        flip = any(np.argmax(x[i, w]) != np.argmax(-x[i, w]) for i in range(x.shape[0]) for w in range(8))
        assert A.find_planted_bug(B.DECODE_FLIP, None, x, None).found == flip
