"""evals, arc and audit modules (API parity with the reference's Python packages)."""
import numpy as np
import pytest
import torch

from prometheus_b200 import arc, audit, contracts, evals


def test_eval_envelope_runner_and_decontam():
    assert len(evals.PUBLIC_SUITES) == 22 and evals.require_suite("aime") == "aime"
    with pytest.raises(evals.UnknownSuiteError):
        evals.require_suite("mmlu")
    cfg = evals.EvalConfig("aime", "test", "ckpt-1", "h-1.0", n_items=3)
    out = evals.Runner(cfg).run(lambda it: it.answer if it.metadata["index"] != 1 else "wrong")
    contracts.validate(out)
    assert out["metrics"]["pass_at_1"] == pytest.approx(2 / 3) and out["n_items"] == 3
    assert out["decontamination"] == {"status": "pending", "against": []}
    assert out == {**evals.Runner(cfg).run(lambda it: it.answer if it.metadata["index"] != 1 else "wrong"),
                   "created_at": out["created_at"]}
    for bad in (dict(harness_version=" "), dict(suite="nope"), dict(split="dev")):
        kw = dict(suite="aime", split="test", checkpoint_id="c", harness_version="1")
        kw.update(bad)
        with pytest.raises((evals.HarnessVersionError, evals.UnknownSuiteError, ValueError)):
            evals.Runner(evals.EvalConfig(**kw))
    ix = evals.DecontamIndex()
    with pytest.raises(evals.DecontamError):
        ix.is_clean("anything")
    with pytest.raises(evals.DecontamError):
        ix.method_hash()
    ix.add(evals.EvalItem("q1", "gpqa", "test", "What is the boiling point of water at sea level in kelvin", "373"))
    assert ix.is_clean("an unrelated sentence about growing tomatoes in a cold northern climate indeed")
    assert not ix.is_clean("leak: what is the BOILING point of water at sea level in kelvin, asked someone")
    assert not ix.is_clean("What is the boiling point of water at sea level in kelvin 373")
    with pytest.raises(evals.DecontamError):
        ix.is_clean("x", against=("aime",))                      # nothing indexed for that suite: fail closed
    h1 = ix.method_hash()
    ix.add(evals.EvalItem("q2", "aime", "test", "short", "1"))
    assert ix.method_hash() != h1 and not ix.is_clean("Short 1", against=("aime",))
    # own items, flagged when the suite's items are in the index
    items = [evals.EvalItem("a", "gpqa", "test", "What is the boiling point of water at sea level in kelvin", "373")]
    res = evals.Runner(evals.EvalConfig("gpqa", "test", "c", "h"), ix, items).run(lambda it: "373")
    assert res["decontamination"]["status"] == "flagged" and res["metrics"]["pass_at_1"] == 1.0
    contracts.validate(res)
    # a "model": next token = (last token + 1) % 10 over single-character tokens
    def logits_fn(ids):
        out = torch.zeros(1, ids.shape[1], 10)
        out[0, torch.arange(ids.shape[1]), (ids[0] + 1) % 10] = 1.0
        return out
    seq = [evals.EvalItem("s", "hmmt", "test", "123", "456"), evals.EvalItem("t", "hmmt", "test", "78", "99")]
    r = evals.Runner(evals.EvalConfig("hmmt", "test", "c", "h"), None, seq).run_model(
        logits_fn, lambda s: [int(c) for c in s], lambda ids: "".join(str(i) for i in ids))
    assert r["metrics"]["pass_at_1"] == 0.5 and r["metrics"]["tokens_to_solve"] == 2.5


def test_arc_dsl_synthesis_and_ensemble():
    g = arc.make_grid([[1, 2, 3], [4, 5, 6]])
    want = {1: np.rot90(np.array(g.cells), -1), 3: np.rot90(np.array(g.cells), 1), 6: np.array(g.cells).T}
    for k, w in want.items():
        assert arc.apply_dihedral(g, k).cells == tuple(map(tuple, w.tolist()))
    for k in range(8):
        assert arc.apply_dihedral(arc.apply_dihedral(g, k), arc.inverse_dihedral(k)) == g
    for bad in ([], [[1, 2], [3]], [[10]], [[True]], [[0] * 31]):
        with pytest.raises(arc.ArcError):
            arc.make_grid(bad)
    with pytest.raises(arc.ArcError):
        arc.apply_dihedral(g, 8)
    with pytest.raises(arc.ArcError):
        arc.apply_color_perm(g, (0,) * 10)
    assert arc.apply_color_perm(g, (9, 8, 7, 6, 5, 4, 3, 2, 1, 0)).cells == ((8, 7, 6), (5, 4, 3))
    prog = arc.Program((arc.Op(arc.OpKind.ROT90), arc.Op(arc.OpKind.RECOLOR, 1, 7)))
    out = arc.execute(prog, g)
    assert out.cells == ((4, 7), (5, 2), (6, 3)) and arc.execute(arc.Program(()), g) == g
    with pytest.raises(arc.ArcError):
        arc.execute(arc.Program((arc.Op(arc.OpKind.RECOLOR, 1),)), g)
    train = (arc.Pair(g, out), arc.Pair(arc.make_grid([[1, 0]]), arc.execute(prog, arc.make_grid([[1, 0]]))))
    assert arc.consistent(prog, train) and not arc.consistent(arc.Program(()), train)
    cat = arc.default_catalog(2)
    assert len(cat) == 1 + 97 + 97 * 97 and cat[0] == arc.Program(())
    found = arc.synthesize(train, cat)
    assert found is not None and arc.consistent(found, train) and len(found.ops) == 2
    assert arc.synthesize(train, cat[:50]) is None
    for call in (lambda: arc.synthesize((), cat), lambda: arc.synthesize(train, ()), lambda: arc.consistent(prog, ())):
        with pytest.raises(arc.ArcError):
            call()
    a, b = arc.make_grid([[1]]), arc.make_grid([[2]])
    assert arc.vote((a, b, b)) == b and arc.vote((a, b)) == a
    with pytest.raises(arc.ArcError):
        arc.vote(())
    # recolouring commutes with every dihedral, so the ensemble agrees with the direct answer
    rec = arc.Program((arc.Op(arc.OpKind.RECOLOR, 2, 9),))
    assert arc.ensemble_predict(rec, g, tuple(range(8))) == arc.execute(rec, g)
    with pytest.raises(arc.ArcError):
        arc.ensemble_predict(rec, g, ())
    assert arc.sidecar_hook("t", "l") == arc.SidecarHook("t", "l")
    with pytest.raises(arc.ArcError):
        arc.sidecar_hook("", "l")


def test_audit_compare_decode_and_planted_bugs():
    assert audit.force_discrete("c1") == audit.CheckpointMode("c1", audit.Mode.DISCRETE)
    with pytest.raises(audit.AuditError):
        audit.force_discrete("  ")
    pairs = (audit.AnswerPair("p1", "4", "4", "4"), audit.AnswerPair("p2", "4", "5", "4"), audit.AnswerPair("p3", "", "x"))
    rows = audit.compare_suite(pairs)
    assert [(r.diverge, r.discrete_correct, r.latent_correct) for r in rows] == [
        (False, True, True), (True, True, False), (True, None, None)]
    assert audit.divergence_rate(pairs) == pytest.approx(2 / 3)
    with pytest.raises(audit.AuditError):
        audit.compare_suite(())
    with pytest.raises(audit.AuditError):
        audit.compare_answers(audit.AnswerPair("", "a", "b"))
    logits = torch.zeros(2, 8, 5)
    logits[0, :, 3] = 1.0
    logits[1, 2, 4] = 2.0
    steps = audit.decode_thoughts(logits)
    assert steps[0].token_ids == (3,) * 8 and steps[1].token_ids == (0, 0, 4, 0, 0, 0, 0, 0)    # ties -> smallest id
    assert audit.decode_thoughts(logits.numpy()) == steps
    for bad in (torch.zeros(2, 8), torch.zeros(0, 8, 5), torch.zeros(2, 7, 5), torch.full((1, 8, 2), float("nan"))):
        with pytest.raises(audit.AuditError):
            audit.decode_thoughts(bad)
    B = audit.BugKind
    assert audit.find_planted_bug(B.ANSWER_SWAP, pairs[1], None, None).found
    assert not audit.find_planted_bug(B.ANSWER_SWAP, pairs[0], None, None).found
    assert audit.find_planted_bug(B.DECODE_FLIP, None, logits, None).found
    assert not audit.find_planted_bug(B.DECODE_FLIP, None, torch.zeros(1, 8, 3), None).found
    assert audit.find_planted_bug("halt_unpinned", None, None, np.array([0.2, 0.9])).found
    assert not audit.find_planted_bug(B.HALT_UNPINNED, None, None, torch.tensor([0.2, 1.0])).found
    for args in ((B.ANSWER_SWAP, None, None, None), (B.DECODE_FLIP, None, None, None), (B.HALT_UNPINNED, None, None, None),
                 (B.HALT_UNPINNED, None, None, torch.zeros(2, 2))):
        with pytest.raises(audit.AuditError):
            audit.find_planted_bug(*args)
