"""Synthetic-data generation (C++): rewrites with fact check, rejection sampling, procedural
ARC grids, agentic trajectories, against the contracts of the reference's synth crate."""
import numpy as np
import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

S = native.synth
A = S.arc
G = S.agentic


def _kind(e):
    return e.value.kind


# ------------------------------------------------------------------------------ rewrites
def test_prompt_claims_and_fact_check():
    assert S.STYLES == ["encyclopedia", "textbook", "conversational", "news", "technical", "simplified"]
    assert S.generate_prompt("Cats purr.", "news") == (
        "Rephrase the document in news style. Preserve every fact. Do not add facts.\n\nDocument:\nCats purr.")
    with pytest.raises(NativeError) as e:
        S.generate_prompt("", "news")
    assert _kind(e) == "EmptySource"
    with pytest.raises(NativeError):
        S.generate_prompt("x", "haiku")
    assert S.extract_claims("One thing. Another thing!  A third?\nNo stop here") == [
        "One thing.", "Another thing!", "A third?", "No stop here"]
    assert S.extract_claims("version 3.5 is out. ok") == ["version 3.5 is out.", "ok"] and S.extract_claims("  \n ") == []
    src = "The bridge opened in 1932 and spans 503 meters. It is not painted yearly."
    assert S.check_claim(src, "The bridge opened in 1932") == "supported"
    assert S.check_claim(src, "The bridge opened in 1932.") == "not_in_source"         # tokens keep their punctuation
    assert S.check_claim(src, "The bridge opened in 1933") == "contradicted"           # number not in source
    assert S.check_claim(src, "It is painted often") == "contradicted"                  # source negates "painted"
    assert S.check_claim(src, "The tunnel closed") == "not_in_source"
    assert S.check_claim(src, "   ") == "not_in_source" and S.check_claim(src, "it is") == "supported"
    with pytest.raises(NativeError) as e:
        S.check_claim("", "x")
    assert _kind(e) == "EmptySource"
    fc = S.fact_check(src, "The bridge spans 503 meters. The bridge opened in 1950. Birds nest there")
    assert [c.verdict for c in fc.claims] == ["supported", "contradicted", "not_in_source"]
    assert (fc.n_supported, fc.n_contradicted, fc.n_not_in_source) == (1, 1, 1) and not S.accept(fc)
    assert S.accept(S.fact_check(src, "")) and S.fact_check(src, "").claims == []
    assert S.token_count("a b  c") == 3 and S.token_count("") == 0 and S.token_count("abc", lambda t: 7) == 7
    ex = [(src, "The bridge opened in 1932", "supported"), (src, "It spans 503 meters.", "contradicted"),
          (src, "The tunnel closed", "supported")]
    assert S.precision(ex) == 0.5 and S.precision([]) == 0.0


def test_rewrite_orchestrator_batches_and_orders():
    calls = []

    def gen(prompts, max_tokens, temperature):
        calls.append((len(prompts), max_tokens, round(temperature, 3)))
        return [("Cats purr." if "Cats" in p else "Dogs bark in 1999.") + " style=" + p.split(" style")[0].split()[-1]
                for p in prompts]

    o = S.Orchestrator(gen, max_tokens=64, temperature=0.5, max_batch=4, styles=["news", "textbook", "technical"])
    docs = [("d1", "Cats purr."), ("d2", "Dogs bark in 2001.")]
    out = o.rephrase_many(docs)
    assert calls == [(4, 64, 0.5), (2, 64, 0.5)]
    assert [(r.source_id, r.style) for r in out] == [("d1", "news"), ("d1", "textbook"), ("d1", "technical"),
                                                     ("d2", "news"), ("d2", "textbook"), ("d2", "technical")]
    assert all(r.accepted for r in out[:3]) and not any(r.accepted for r in out[3:])      # 1999 is not in d2
    assert out[0].text == "Cats purr. style=news" and out[0].token_count == 3
    one = o.rephrase("d1", "Cats purr.", "simplified")
    assert one.style == "simplified" and one.accepted
    assert [r.style for r in o.rephrase_many(docs[:1], ["news"])] == ["news"]
    with pytest.raises(NativeError) as e:
        o.rephrase_many([])
    assert _kind(e) == "EmptyBatch"
    bad = S.Orchestrator(lambda p, m, t: [], styles=["news"])
    with pytest.raises(NativeError) as e:
        bad.rephrase_many(docs)
    assert _kind(e) == "LengthMismatch"
    # the batch generation engine plugs in directly
    eng = native.serve.LocalEngine("m", 1, 8, 30000)
    real = S.Orchestrator(lambda p, m, t: [c[1] for c in eng.generate(p, m, t)], max_tokens=4)
    assert len(real.rephrase_many(docs)) == 12


# -------------------------------------------------------------------- rejection sampling
def test_extract_answer_rules():
    assert S.extract_answer("thinking...\nAnswer: 42  \n") == "42"
    assert S.extract_answer("ANSWER : first\nanswer:second\nmore text") == "second"
    assert S.extract_answer("answer:\nthe last line") == "the last line"          # empty capture does not count
    assert S.extract_answer("text\n```python\nprint(1)\n```\nthen\n```\nx = 2\n```\n") == "x = 2\n"
    assert S.extract_answer("inline ```not a fence```\nlast") == "last"
    assert S.extract_answer("```\nunclosed") == "unclosed"
    assert S.extract_answer("a\n\nb\n  \n") == "b" and S.extract_answer("  \n ") == ""


def test_rejection_sampler():
    p1 = S.Problem("p1", "math", "2+2?", "symbolic-math")
    p2 = S.Problem("p2", "code", "print 1", "sandboxed-tests")
    with pytest.raises(NativeError):
        S.Problem("p", "poetry", "x", "v")
    assert S.generate_solve_prompt(p1) == (
        "Solve the following math problem. Put the final answer after the reasoning.\n\nProblem:\n2+2?")
    with pytest.raises(NativeError) as e:
        S.generate_solve_prompt(S.Problem("p", "math", "", "v"))
    assert _kind(e) == "EmptyPrompt"
    sizes = []
    counter = iter(range(1000))

    def gen(prompts, mt, temp):
        sizes.append(len(prompts))
        return [f"work\nAnswer: {4 if next(counter) % 2 == 0 else 5}" for _ in prompts]

    seen = []

    def verify(problem, answer):
        seen.append((problem.problem_id, answer))
        return answer == "4"

    s = S.RejectionSampler(gen, verify, n_samples=4, max_batch=3)
    res = s.sample_many([p1, p2])
    assert sizes == [3, 3, 2] and [r.problem_id for r in res] == ["p1", "p2"]
    assert [(r.n_generated, r.n_accepted) for r in res] == [(4, 2), (4, 2)] and res[0].verified_correct_rate() == 0.5
    assert [x.passed for x in res[0].samples] == [True, False, True, False] and res[0].samples[0].answer == "4"
    assert res[0].samples[0].token_count == 3 and seen[0] == ("p1", "4") and seen[4][0] == "p2"
    assert S.verified_correct_rate(res) == 0.5 and S.verified_correct_rate([]) == 0.0
    one = s.sample(p1, 2)
    assert one.n_generated == 2
    for call, kind in ((lambda: s.sample(p1, 0), "ZeroSamples"), (lambda: s.sample_many([], 2), "EmptyBatch")):
        with pytest.raises(NativeError) as e:
            call()
        assert _kind(e) == kind


# ---------------------------------------------------------------------------- ARC grids
def test_dihedral_group_and_color_perm_match_numpy():
    g = [[1, 2, 3], [4, 5, 6]]
    a = np.array(g)
    want = {"identity": a, "rot90": np.rot90(a, -1), "rot180": np.rot90(a, 2), "rot270": np.rot90(a, 1),
            "flip_h": a[:, ::-1], "flip_v": a[::-1, :], "transpose": a.T, "anti_transpose": np.rot90(a, 2).T}
    assert A.DIHEDRALS == list(want)
    for i, (name, w) in enumerate(want.items()):
        assert A.apply_dihedral(g, name) == w.tolist() == A.apply_dihedral(g, i) and A.dihedral_index(name) == i
    with pytest.raises(NativeError) as e:
        A.apply_dihedral(g, 8)
    assert _kind(e) == "BadDihedral"
    perm = [9, 8, 7, 6, 5, 4, 3, 2, 1, 0]
    assert A.apply_color_perm(g, perm) == [[8, 7, 6], [5, 4, 3]]
    for bad in ([0] * 10, list(range(9)), list(range(1, 11))):
        with pytest.raises(NativeError) as e:
            A.apply_color_perm(g, bad)
        assert _kind(e) == "BadPermutation"
    for cells, kind in (([], "EmptyGrid"), ([[]], "EmptyGrid"), ([[1, 2], [3]], "JaggedGrid"), ([[10]], "BadColor"),
                        ([[0] * 31], "GridSize")):
        with pytest.raises(NativeError) as e:
            A.validate_grid(cells)
        assert _kind(e) == kind
    assert A.flatten(g) == bytes([1, 2, 3, 4, 5, 6])
    assert A.tokenize_grid(lambda b: [x + 100 for x in b], g) == [101, 102, 103, 104, 105, 106]


def test_family_transforms():
    F = A.FamilySpec
    g = [[0, 1, 0], [0, 0, 2], [0, 0, 0]]
    assert F("translate", {"dx": 1, "dy": -1, "bg": 0}).apply(g) == [[2, 0, 0], [0, 0, 0], [0, 0, 1]]
    assert F("recolor", {"src": 1, "dst": 7}).apply(g) == [[0, 7, 0], [0, 0, 2], [0, 0, 0]]
    assert F("crop", {"bg": 0}).apply(g) == [[1, 0], [0, 2]] and F("crop", {"bg": 0}).apply([[0, 0]]) == [[0]]
    assert F("tile", {"nx": 2, "ny": 1}).apply([[1, 2]]) == [[1, 2, 1, 2]]
    assert F("tile", {"nx": 1, "ny": 2}).apply([[1, 2]]) == [[1, 2], [1, 2]]
    assert F("gravity", {"dir": 0, "bg": 0}).apply(g) == [[0, 0, 0], [0, 0, 0], [0, 1, 2]]
    assert F("gravity", {"dir": 1, "bg": 0}).apply(g) == [[0, 1, 2], [0, 0, 0], [0, 0, 0]]
    assert F("gravity", {"dir": 2, "bg": 0}).apply(g) == [[1, 0, 0], [2, 0, 0], [0, 0, 0]]
    assert F("gravity", {"dir": 3, "bg": 0}).apply(g) == [[0, 0, 1], [0, 0, 2], [0, 0, 0]]
    assert F("mirror", {"dihedral": 4}).apply([[1, 2]]) == [[2, 1]]
    assert F("scale", {"factor": 2}).apply([[1, 2]]) == [[1, 1, 2, 2], [1, 1, 2, 2]]
    assert F("border", {"color": 5, "width": 1}).apply([[1]]) == [[5, 5, 5], [5, 1, 5], [5, 5, 5]]
    assert F("translate", {"dx": 1, "dy": -1, "bg": 0}).family_id() == "translate:bg=0,dx=1,dy=-1"
    for kind, params in (("recolor", {"src": 1, "dst": 1}), ("scale", {"factor": 4}), ("border", {"color": 1, "width": 3}),
                         ("gravity", {"dir": 4, "bg": 0}), ("crop", {"bg": 10}), ("crop", {}), ("tile", {"nx": 0, "ny": 1}),
                         ("mirror", {"dihedral": 8}), ("crop", {"bg": 0, "extra": 1})):
        with pytest.raises(NativeError) as e:
            F(kind, params).validate()
        assert _kind(e) == "UnknownFamily"
    with pytest.raises(NativeError):
        F("spiral", {})


def test_task_generation_corpus_and_diversity():
    grid = A.parameter_grid()
    assert len(grid) == 490 + 90 + 10 + 16 + 40 + 8 + 2 + 20 and len({s.family_id() for s in grid}) == len(grid)
    specs = A.sample_family_specs(20, 7)
    assert [s.family_id() for s in specs] == [s.family_id() for s in A.sample_family_specs(20, 7)]
    assert [s.family_id() for s in specs] != [s.family_id() for s in A.sample_family_specs(20, 8)]
    assert len({s.family_id() for s in specs}) == 20 and A.sample_family_specs(0, 1) == []
    with pytest.raises(NativeError):
        A.sample_family_specs(10000, 1)
    spec = A.FamilySpec("scale", {"factor": 3})
    t = spec.generate(11)
    t2 = spec.generate(11)
    assert t.family_id == "scale:factor=3" and t.seed == 11 and len(t.train) == 3
    assert [(p.input, p.output) for p in t.train] == [(p.input, p.output) for p in t2.train] and t.test.input == t2.test.input
    for p in t.train + [t.test]:
        assert spec.apply(p.input) == p.output and len(p.input) <= 8 and len(p.output) <= 30
    assert len({str(p.input) for p in t.train + [t.test]}) == 4
    with pytest.raises(NativeError) as e:
        spec.generate(1, 0)
    assert _kind(e) == "EmptyTrain"
    tasks = A.corpus_sample(specs, 100, 3, 40)
    assert [x.seed for x in tasks[:3]] == [100, 101, 102] and tasks[20].family_id == tasks[0].family_id
    d = A.diversity_stats(tasks)
    assert d.n_tasks == 40 and d.n_families == 20 and d.unique_tasks == 40 and d.collision_rate == 0.0
    assert sum(d.color_histogram) > 0 and d.unique_shapes > 3 and d.unique_test_inputs > 30
    dup = A.diversity_stats([tasks[0], tasks[0]])
    assert dup.unique_tasks == 1 and dup.collision_rate == 0.5
    z = A.diversity_stats([])
    assert z.n_tasks == 0 and z.collision_rate == 0.0
    for call, kind in ((lambda: A.corpus_sample(specs, 1, 3, 0), "EmptyTasks"), (lambda: A.corpus_sample([], 1, 3, 2), "UnknownFamily"),
                       (lambda: A.corpus_sample(specs, 1, 0, 2), "EmptyTrain")):
        with pytest.raises(NativeError) as e:
            call()
        assert _kind(e) == kind
    perm = [1, 2, 3, 4, 5, 6, 7, 8, 9, 0]
    aug = A.augment_task(t, 1, perm)
    assert aug.family_id == t.family_id and aug.seed == t.seed
    assert aug.test.output == A.apply_color_perm(A.apply_dihedral(t.test.output, "rot90"), perm)
    ap = A.augment_pair(t.train[0], 6, perm)
    assert ap.input == A.apply_color_perm(A.apply_dihedral(t.train[0].input, 6), perm)


# ------------------------------------------------------------------------------ agentic
def test_agentic_trajectories():
    prompts = []

    def scripted(replies):
        it = iter(replies)

        def gen(ps, mt, temp):
            prompts.append(ps[0])
            return [next(it)]
        return gen

    def sandbox(tool, args):
        return "verified" if (tool, args) == ("submit", "final answer") else f"ran {tool}({args})"

    ok = G.generate_one(scripted(["  ls  -la  /tmp ", "submit   final answer"]), sandbox, "t1", "do it", 1, 5)[0]
    assert ok.outcome == "verified" and [(s.tool, s.args) for s in ok.steps] == [("ls", "-la  /tmp"), ("submit", "final answer")]
    assert prompts == ["do it", "do it\nls\n-la  /tmp\nran ls(-la  /tmp)"]
    bad = G.generate_one(scripted(["submit wrong"]), sandbox, "t1", "do it", 1, 5)[0]
    assert bad.outcome == "failed" and len(bad.steps) == 1
    empty = G.generate_one(scripted(["noop", "   "]), sandbox, "t1", "do it", 1, 5)[0]
    assert empty.outcome == "failed" and len(empty.steps) == 1
    trunc = G.generate_one(scripted(["a", "b", "c"]), sandbox, "t1", "do it", 1, 3)[0]
    assert trunc.outcome == "truncated" and len(trunc.steps) == 3
    assert G.outcome_verified_rate([ok, bad, empty, trunc]) == 0.25 and G.outcome_verified_rate([]) == 0.0
    assert [t.outcome for t in G.keep_verified([ok, bad, trunc])] == ["verified"]
    batch = G.generate_batch(scripted(["submit final answer"] * 4), sandbox, [("a", "p"), ("b", "q")], 2, 3)
    assert [[t.task_id for t in ts] for ts in batch] == [["a", "a"], ["b", "b"]]
    for call, kind in ((lambda: G.generate_one(scripted([]), sandbox, "t", "p", 0, 3), "ZeroSamples"),
                       (lambda: G.generate_one(scripted([]), sandbox, "t", "", 1, 3), "EmptyPrompt"),
                       (lambda: G.generate_batch(scripted([]), sandbox, [], 1, 3), "EmptyBatch"),
                       (lambda: G.generate_batch(scripted([]), sandbox, [("a", "")], 1, 3), "EmptyPrompt")):
        with pytest.raises(NativeError) as e:
            call()
        assert _kind(e) == kind
    with pytest.raises(NativeError) as e:
        G.generate_one(lambda ps, mt, t: ["a", "b"], sandbox, "t", "p", 1, 3)
    assert _kind(e) == "LengthMismatch"
