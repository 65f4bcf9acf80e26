"""The Python / NumPy restatement of synthetic-data generation (``synth_twin``) against the C++
module on generated inputs: text rules (claims, fact check, answers), every grid family, the
seeded task generator and corpus statistics must agree exactly."""
import random

import numpy as np
import pytest

from prometheus_b200 import native
from prometheus_b200 import synth_twin as T

S = native.synth
A = S.arc

WORDS = ["the", "reactor", "produced", "not", "no", "1200", "3.5", "megawatts", "that", "output", "Answer:", "answer",
         "Paris", "is", "capital", "France.", "It", "was", "built", "in", "1999.", "never", "works!", "why?", "x", "\t", "  ",
         "naïve", "café", "ÉCOLE", "Not", "over", "their", "data.", "42", "7.", ".5", "1.2.3"]


def _text(rng, n):
    return " ".join(rng.choice(WORDS) for _ in range(n))


def test_text_rules_agree_with_the_native_module_on_generated_text():
    rng = random.Random(0)
    verdicts = set()
    for _ in range(400):
        src, claim = _text(rng, rng.randrange(1, 25)), _text(rng, rng.randrange(0, 8))
        assert T.extract_claims(src) == S.extract_claims(src)
        v = T.check_claim(src, claim)
        assert v == S.check_claim(src, claim), (src, claim)
        verdicts.add(v)
        fc = S.fact_check(src, claim)
        assert T.fact_check(src, claim) == [(c.text, c.verdict) for c in fc.claims]
    assert verdicts == {"supported", "not_in_source", "contradicted"}
    for style in T.STYLES:
        assert T.rewrite_prompt("doc", style) == S.generate_prompt("doc", style)
    assert tuple(S.STYLES) == T.STYLES and tuple(S.DOMAINS) == T.DOMAINS
    ex = [("The dam is 40 m tall.", "The dam is 40 m tall.", "supported"),
          ("The dam is 40 m tall.", "The dam is tall.", "not_in_source"),
          ("The dam is not tall.", "The dam is tall.", "contradicted")]
    assert T.precision(ex) == S.precision(ex)
    with pytest.raises(T.SynthError) as e:
        T.check_claim("", "x")
    assert e.value.kind == "EmptySource"


def test_answer_extraction_agrees_on_generated_completions():
    rng = random.Random(1)
    parts = ["reasoning line", "Answer: 42", "ANSWER :  x + 1  ", "answer:", "answer 7", "```python\nprint(1)\n```", "```\nbody\n```",
             "text ``` inline", "", "   ", "final\r", "```unterminated\ncode"]
    for _ in range(400):
        raw = "\n".join(rng.choice(parts) for _ in range(rng.randrange(0, 7))) + rng.choice(["", "\n", " \n\t"])
        assert T.extract_answer(raw) == S.extract_answer(raw), repr(raw)
    p = T.Problem("p1", "math", "2 + 2")
    assert T.solve_prompt(p) == S.generate_solve_prompt(S.Problem("p1", "math", "2 + 2", ""))


def test_rejection_sampler_and_orchestrator_follow_the_same_batching():
    calls = []

    def gen(prompts, max_tokens, temperature):
        calls.append(len(prompts))
        return [f"work\nAnswer: {len(p) % 3}" for p in prompts]

    verify = lambda prob, ans: ans == "1"                       # noqa: E731
    mine = T.RejectionSampler(gen, verify, n_samples=3, max_batch=4)
    probs = [T.Problem(f"p{i}", "math", "q" * (i + 1)) for i in range(3)]
    res = mine.sample_many(probs)
    assert calls == [4, 4, 1]
    theirs = S.RejectionSampler(gen, lambda prob, ans: ans == "1", 3, 512, 0.7, 4)
    ref = theirs.sample_many([S.Problem(p.problem_id, p.domain, p.prompt, "") for p in probs])
    assert [(r.problem_id, r.n_generated, r.n_accepted) for r in res] == \
        [(r.problem_id, r.n_generated, r.n_accepted) for r in ref]
    assert [[s.answer for s in r.samples] for r in res] == [[s.answer for s in r.samples] for r in ref]
    assert T.verified_correct_rate(res) == S.verified_correct_rate(ref)
    for bad, kind in ((lambda: mine.sample_many([]), "EmptyBatch"), (lambda: mine.sample_many(probs, 0), "ZeroSamples")):
        with pytest.raises(T.SynthError) as e:
            bad()
        assert e.value.kind == kind
    orch = T.Orchestrator(lambda ps, mt, t: ["The dam is 40 m tall. It is old."] * len(ps), max_batch=5,
                          styles=("news", "textbook"))
    out = orch.rephrase_many([("d1", "The dam is 40 m tall."), ("d2", "The dam is 41 m tall.")])
    assert [(r.source_id, r.style, r.accepted) for r in out] == [("d1", "news", True), ("d1", "textbook", True),
                                                                 ("d2", "news", False), ("d2", "textbook", False)]
    with pytest.raises(T.SynthError) as e:
        T.Orchestrator(lambda ps, mt, t: [], max_batch=1).rephrase("d", "doc", "news")
    assert e.value.kind == "LengthMismatch"


def _spec_pairs():
    return [(T.FamilySpec.make(s.kind, dict(s.params)), s) for s in A.parameter_grid()]


def test_every_family_of_the_parameter_grid_agrees_on_random_grids():
    rng = np.random.default_rng(3)
    pairs = _spec_pairs()
    assert [m.family_id() for m, _ in pairs] == [n.family_id() for _, n in pairs] and len(pairs) == 676
    for mine, theirs in pairs[::3]:
        mh, mw = (min(v, 8) for v in mine.max_input_hw())
        for _ in range(3):
            g = rng.integers(0, 10, size=(rng.integers(1, mh + 1), rng.integers(1, mw + 1)))
            if rng.random() < 0.3:
                g[:] = g.flat[0]                              # uniform grid: crop of pure background etc.
            assert mine.apply(g).tolist() == theirs.apply(g.tolist()), (mine.family_id(), g.tolist())
    g = [[1, 2, 3], [4, 5, 6]]
    for k, name in enumerate(T.DIHEDRALS):
        assert T.dihedral(g, k).tolist() == A.apply_dihedral(g, k) == T.dihedral(g, name).tolist()
    perm = [3, 1, 4, 0, 5, 9, 2, 6, 8, 7]
    assert T.color_perm(g, perm).tolist() == A.apply_color_perm(g, perm)
    for cells, kind in (([], "EmptyGrid"), ([[1, 2], [3]], "JaggedGrid"), ([[10]], "BadColor"), ([[0] * 31], "GridSize")):
        with pytest.raises(T.SynthError) as e:
            T.as_grid(cells)
        assert e.value.kind == kind
    for kind, params in (("recolor", {"src": 1, "dst": 1}), ("scale", {"factor": 4}), ("crop", {}), ("crop", {"bg": 0, "x": 1})):
        with pytest.raises(T.SynthError) as e:
            T.FamilySpec.make(kind, params).validate()
        assert e.value.kind == "UnknownFamily"


def test_seeded_generation_sampling_augmentation_and_statistics_agree():
    assert [s.family_id() for s in T.sample_family_specs(25, 7)] == [s.family_id() for s in A.sample_family_specs(25, 7)]
    mine_specs, their_specs = T.sample_family_specs(12, 99), A.sample_family_specs(12, 99)
    mine = T.corpus_sample(mine_specs, 1000, 3, 30)
    theirs = A.corpus_sample(their_specs, 1000, 3, 30)
    for a, b in zip(mine, theirs):
        assert (a.family_id, a.seed) == (b.family_id, b.seed)
        assert [(p.input.tolist(), p.output.tolist()) for p in a.train] == [(p.input, p.output) for p in b.train]
        assert a.test.input.tolist() == b.test.input and a.test.output.tolist() == b.test.output
    d, e = T.diversity_stats(mine), A.diversity_stats(theirs)
    assert (d["n_tasks"], d["n_families"], d["unique_test_inputs"], d["unique_test_outputs"], d["unique_tasks"],
            d["unique_shapes"], d["collision_rate"]) == (e.n_tasks, e.n_families, e.unique_test_inputs,
                                                         e.unique_test_outputs, e.unique_tasks, e.unique_shapes,
                                                         e.collision_rate)
    assert d["color_histogram"] == list(e.color_histogram)
    assert T.diversity_stats([mine[0], mine[0]])["collision_rate"] == 0.5 and T.diversity_stats([])["n_tasks"] == 0
    perm = [1, 2, 3, 4, 5, 6, 7, 8, 9, 0]
    for k in range(8):
        a, b = T.augment_task(mine[3], k, perm), A.augment_task(theirs[3], k, perm)
        assert a.test.output.tolist() == b.test.output and a.train[0].input.tolist() == b.train[0].input
    rng = T.SplitMix64(0)
    assert rng.next() == 0xE220A8397B1DCDAF                    # first SplitMix64 output for seed 0
