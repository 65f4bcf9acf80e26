"""Behaviour list of rejection sampling against verifiers (C++ ``native.synth`` through
``prometheus_b200.synth``; reference tests/test_synth_reject.py, synth/__init__.py): prompt
template, answer extraction rules, validation before any generation and its order, batching
across problems, what the verifier and the tokenizer see, and the aggregate rate; the C++ is
also compared with the plain-Python restatement on a grid of settings."""
import itertools

import pytest

from prometheus_b200 import synth as S
from prometheus_b200 import synth_twin as T
from prometheus_b200.native import NativeError


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def problem(pid="p1", domain="math", prompt="2+2?", verifier="symbolic-math"):
    return S.Problem(pid, domain, prompt, verifier)


class Gen:
    """Answers cycle through ``answers``; records every batch it is asked for."""

    def __init__(self, answers=("4", "5")):
        self.answers, self.batches, self.n = answers, [], 0

    def __call__(self, prompts, max_tokens, temperature):
        self.batches.append((list(prompts), max_tokens, temperature))
        out = []
        for _ in prompts:
            out.append(f"some work here\nAnswer: {self.answers[self.n % len(self.answers)]}")
            self.n += 1
        return out


def is_four(problem, answer):
    return answer == "4"


# ------------------------------------------------------------------------------ prompts / answers
def test_defaults_and_prompt_template():
    assert (S.DEFAULT_N_SAMPLES, S.DEFAULT_MAX_TOKENS, S.DEFAULT_MAX_BATCH) == (8, 512, 8) and abs(S.DEFAULT_TEMPERATURE - 0.7) < 1e-6
    for d in S.DOMAINS:
        text = S.generate_solve_prompt(problem(domain=d, prompt="ünïcode ☃ problem"))
        assert text == f"Solve the following {d} problem. Put the final answer after the reasoning.\n\nProblem:\nünïcode ☃ problem"
    assert err(lambda: S.generate_solve_prompt(problem(prompt=""))).kind == "EmptyPrompt"
    assert err(lambda: problem(domain="poetry")).kind in ("BadDomain", "Message", "Other", "Config")


@pytest.mark.parametrize("text, want", [
    ("work\nAnswer: 42", "42"), ("ANSWER:   spaced  ", "spaced"), ("answer: a\nAnswer: b", "b"), ("Answer:\nfallback line", "fallback line"),
    ("x\n```python\nprint(1)\n```", "print(1)\n"), ("```\nfirst\n```\n```js\nsecond\n```", "second\n"), ("```\nnever closed", "never closed"),
    ("line one\n\nline two\n   \n", "line two"), ("", ""), ("   \n\t\n", ""), ("only", "only"), ("Answer: 7   \n\n", "7"),
    ("Final answer: 9", "Final answer: 9"),
])
def test_answer_extraction(text, want):
    assert S.extract_answer(text) == want == T.extract_answer(text)


# ------------------------------------------------------------------------------ validation
def test_validation_happens_before_any_generation_and_in_order():
    gen = Gen()
    s = S.RejectionSampler(gen, is_four, n_samples=4, max_batch=3)
    assert err(lambda: s.sample(problem(), 0)).kind == "ZeroSamples"
    assert err(lambda: s.sample(problem(prompt=""), 2)).kind == "EmptyPrompt"
    assert err(lambda: s.sample(problem(prompt=""), 0)).kind == "ZeroSamples"              # the count is checked first
    assert err(lambda: s.sample_many([], 2)).kind == "EmptyBatch"
    assert err(lambda: s.sample_many([], 0)).kind == "EmptyBatch"                           # the empty batch wins over the count
    assert err(lambda: s.sample_many([problem()], 0)).kind == "ZeroSamples"
    assert err(lambda: s.sample_many([problem(), problem("p2", prompt="")], 2)).kind == "EmptyPrompt"
    assert gen.batches == []
    zero = S.RejectionSampler(gen, is_four, n_samples=0)
    assert err(lambda: zero.sample(problem())).kind == "ZeroSamples"                        # the configured default counts too
    short = S.RejectionSampler(lambda p, m, t: ["Answer: 4"] * (len(p) - 1), is_four, n_samples=2)
    assert err(lambda: short.sample(problem())).kind in ("LengthMismatch", "Message", "Other")


# ------------------------------------------------------------------------------ sampling
def test_one_problem_is_generated_in_chunks_and_keeps_rejected_traces():
    gen = Gen()
    s = S.RejectionSampler(gen, is_four, n_samples=5, max_tokens=64, temperature=0.25, max_batch=2)
    res = s.sample(problem())
    assert [len(b[0]) for b in gen.batches] == [2, 2, 1] and all(b[1] == 64 and abs(b[2] - 0.25) < 1e-6 for b in gen.batches)
    assert all(p == S.generate_solve_prompt(problem()) for b in gen.batches for p in b[0])
    assert (res.problem_id, res.n_generated, res.n_accepted) == ("p1", 5, 3) and res.verified_correct_rate() == pytest.approx(0.6)
    assert [x.passed for x in res.samples] == [True, False, True, False, True] and [x.answer for x in res.samples] == ["4", "5", "4", "5", "4"]
    assert all(x.text.startswith("some work here") for x in res.samples)                  # rejected traces are kept too
    assert s.sample(problem(), 2).n_generated == 2 and s.sample(problem(), None).n_generated == 5


def test_many_problems_share_batches_and_keep_their_order():
    gen = Gen(("4",))
    s = S.RejectionSampler(gen, lambda p, a: p.problem_id != "b", n_samples=3, max_batch=4)
    probs = [problem("a", prompt="A?"), problem("b", "code", "B?", "sandboxed-tests"), problem("c", prompt="C?")]
    res = s.sample_many(probs)
    assert [len(b[0]) for b in gen.batches] == [4, 4, 1]                                   # 9 prompts, packed across problems
    flat = [p for b in gen.batches for p in b[0]]
    assert flat == [S.generate_solve_prompt(p) for p in probs for _ in range(3)]
    assert [(r.problem_id, r.n_generated, r.n_accepted) for r in res] == [("a", 3, 3), ("b", 3, 0), ("c", 3, 3)]
    assert S.verified_correct_rate(res) == pytest.approx(6 / 9) and S.verified_correct_rate([]) == 0.0
    assert s.sample_many(probs[:1], 2)[0].n_generated == 2


def test_what_the_verifier_and_the_tokenizer_see():
    seen = []

    def verifier(p, answer):
        seen.append((p.problem_id, p.domain, p.verifier_id, answer))
        return True

    class Tok:
        def __init__(self):
            self.calls = []

        def encode(self, text):
            self.calls.append(text)
            return list(range(len(text)))

    tok = Tok()
    texts = iter(["three word text\nAnswer: x", "", "```\ncode\n```"])
    s = S.RejectionSampler(lambda p, m, t: [next(texts) for _ in p], verifier, n_samples=3, tokenizer=lambda text: len(tok.encode(text)))
    res = s.sample(problem())
    assert seen == [("p1", "math", "symbolic-math", "x"), ("p1", "math", "symbolic-math", ""), ("p1", "math", "symbolic-math", "code\n")]
    assert tok.calls == ["three word text\nAnswer: x", "```\ncode\n```"]                   # the raw text; an empty one is not encoded
    assert [x.token_count for x in res.samples] == [len("three word text\nAnswer: x"), 0, len("```\ncode\n```")]
    plain = S.RejectionSampler(lambda p, m, t: ["one two  three\nAnswer: 4"] * len(p), is_four, n_samples=1).sample(problem())
    assert plain.samples[0].token_count == 5                                               # whitespace-separated words without a tokenizer

    def broken(p, answer):
        raise RuntimeError("verifier fell over")

    with pytest.raises(Exception, match="fell over"):
        S.RejectionSampler(Gen(), broken, n_samples=1).sample(problem())


@pytest.mark.parametrize("n, max_batch, n_problems", list(itertools.product([1, 3, 5], [1, 2, 8], [1, 3])))
def test_grid_of_settings_matches_the_python_restatement(n, max_batch, n_problems):
    probs = [problem(f"p{i}", prompt=f"question {i}?") for i in range(n_problems)]
    tprobs = [T.Problem(f"p{i}", "math", f"question {i}?", "symbolic-math") for i in range(n_problems)]
    g1, g2 = Gen(("4", "5", "6")), Gen(("4", "5", "6"))
    mine = S.RejectionSampler(g1, is_four, n_samples=n, max_batch=max_batch).sample_many(probs)
    theirs = T.RejectionSampler(g2, lambda p, a: a == "4", n_samples=n, max_batch=max_batch).sample_many(tprobs)
    assert [len(b[0]) for b in g1.batches] == [len(b[0]) for b in g2.batches]
    assert [(r.problem_id, r.n_generated, r.n_accepted) for r in mine] == [(r.problem_id, r.n_generated, r.n_accepted) for r in theirs]
    assert [[(x.answer, x.passed, x.token_count) for x in r.samples] for r in mine] == \
        [[(x.answer, x.passed, x.token_count) for x in r.samples] for r in theirs]
