"""Synthetic-data generation restated in plain Python and NumPy.

The production implementation is C++ (``native.synth``); this module states the same contracts
a second time with different means -- regular expressions for the text rules, whole-array NumPy
operations for the grids -- so that each can be checked against the other on generated inputs
(``tests/test_synth_twin.py``). It is the counterpart of the reference's Python twin
(``synth/__init__.py:161-1331``: E1 rewrite prompts and the word-overlap fact check, E2 the
rejection sampler, E3 procedural ARC families with D4 x colour-permutation augmentation on a
SplitMix64 stream). Errors are ``SynthError`` with the same ``kind`` strings as the C++ module.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Callable, Sequence

import numpy as np

_WS = " \t\n\x0b\x0c\r"                      # the C locale's isspace set: what the C++ splits on
_WORD = re.compile(f"[^{re.escape(_WS)}]+")
_NUMBER = re.compile(r"[0-9]+(?:\.[0-9]+)?")
_SENTENCE_END = re.compile(f"(?<=[.!?])[{re.escape(_WS)}]+")
_ANSWER = re.compile(f"^[aA][nN][sS][wW][eE][rR][{re.escape(_WS)}]*:[{re.escape(_WS)}]*(?=[^{re.escape(_WS)}])(.*)$", re.S)
_ASCII_LOWER = {c: c + 32 for c in range(ord("A"), ord("Z") + 1)}

STYLES = ("encyclopedia", "textbook", "conversational", "news", "technical", "simplified")
DOMAINS = ("math", "code", "lean", "grid", "market")
STOP_WORDS = frozenset("that this with from they them have been were will would could should into over under "
                       "than then when what which their".split())


class SynthError(ValueError):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def _words(s: str) -> list[str]:
    return _WORD.findall(s)


def _lower(s: str) -> str:
    return s.translate(_ASCII_LOWER)          # ASCII letters only, like tolower in the C locale


# ------------------------------------------------------------------ E1: rewrites + fact check
def rewrite_prompt(text: str, style: str) -> str:
    if style not in STYLES:
        raise SynthError("Message", f"unknown style {style}")
    if not text:
        raise SynthError("EmptySource", "empty source")
    return f"Rephrase the document in {style} style. Preserve every fact. Do not add facts.\n\nDocument:\n{text}"


def numbers_in(text: str) -> list[str]:
    return _NUMBER.findall(text)


def extract_claims(text: str) -> list[str]:
    """Sentences: cut after '.', '!' or '?' when white space follows."""
    return [t for t in (p.strip(_WS) for p in _SENTENCE_END.split(text)) if t]


def check_claim(source: str, claim: str) -> str:
    """"supported" / "not_in_source" / "contradicted": a number absent from a source that has
    numbers contradicts; so does a content word the source negates ("not x" / "no x"); otherwise
    every content word (>= 4 characters, not a stop word) must occur in the source."""
    if not source:
        raise SynthError("EmptySource", "empty source")
    if not _words(claim):
        return "not_in_source"
    have = set(numbers_in(source))
    if have and any(n not in have for n in numbers_in(claim)):
        return "contradicted"
    src, cl = _words(_lower(source)), _words(_lower(claim))
    content = [w for w in cl if len(w) >= 4 and w not in STOP_WORDS]
    negated = {b for a, b in zip(src, src[1:]) if a in ("not", "no")}
    if negated & set(content):
        return "contradicted"
    if content:
        return "supported" if set(content) <= set(src) else "not_in_source"
    return "supported" if " ".join(cl) in " ".join(src) else "not_in_source"


def fact_check(source: str, rewrite: str) -> list[tuple[str, str]]:
    if not source:
        raise SynthError("EmptySource", "empty source")
    return [(c, check_claim(source, c)) for c in extract_claims(rewrite)]


def accept(checked: Sequence[tuple[str, str]]) -> bool:
    return all(v != "contradicted" for _c, v in checked)


def precision(examples: Sequence[tuple[str, str, str]]) -> float:
    """Of the claims the checker calls supported, the share whose gold label is supported."""
    called = [gold for source, claim, gold in examples if check_claim(source, claim) == "supported"]
    return sum(g == "supported" for g in called) / len(called) if called else 0.0


def token_count(text: str, counter: Callable[[str], int] | None = None) -> int:
    if not text:
        return 0
    return int(counter(text)) if counter else len(_words(text))


def _generate_chunked(gen, prompts, max_tokens, temperature, max_batch):
    out: list[str] = []
    for i in range(0, len(prompts), max_batch):
        chunk = list(prompts[i:i + max_batch])
        got = list(gen(chunk, max_tokens, temperature))
        if len(got) != len(chunk):
            raise SynthError("LengthMismatch", f"generator returned {len(got)} completions for {len(chunk)} prompts")
        out += got
    return out


@dataclass
class Rewrite:
    source_id: str
    style: str
    text: str
    token_count: int
    fact_check: list
    accepted: bool


class Orchestrator:
    """Batches rewrite prompts (documents major, styles minor), fact-checks every completion."""

    def __init__(self, generate, max_tokens=512, temperature=0.7, max_batch=8, styles=STYLES, counter=None):
        for s in styles:
            if s not in STYLES:
                raise SynthError("Message", f"unknown style {s}")
        if max_batch <= 0:
            raise SynthError("Message", "max_batch must be > 0")
        self.generate, self.max_tokens, self.temperature = generate, max_tokens, temperature
        self.max_batch, self.styles, self.counter = max_batch, tuple(styles), counter

    def _finish(self, source_id, source, style, completion) -> Rewrite:
        fc = fact_check(source, completion)
        return Rewrite(source_id, style, completion, token_count(completion, self.counter), fc, accept(fc))

    def rephrase(self, source_id: str, text: str, style: str) -> Rewrite:
        out = _generate_chunked(self.generate, [rewrite_prompt(text, style)], self.max_tokens, self.temperature, 1)
        return self._finish(source_id, text, style, out[0])

    def rephrase_many(self, docs: Sequence[tuple[str, str]], styles=None) -> list[Rewrite]:
        if not docs:
            raise SynthError("EmptyBatch", "empty batch")
        use = tuple(styles) if styles is not None else self.styles
        jobs = [(sid, text, s) for sid, text in docs for s in use]
        outs = _generate_chunked(self.generate, [rewrite_prompt(t, s) for _i, t, s in jobs], self.max_tokens,
                                 self.temperature, self.max_batch)
        return [self._finish(sid, text, s, o) for (sid, text, s), o in zip(jobs, outs)]


# ------------------------------------------------------------------ E2: rejection sampling
@dataclass
class Problem:
    problem_id: str
    domain: str
    prompt: str
    verifier_id: str = ""


def solve_prompt(p: Problem) -> str:
    if not p.prompt:
        raise SynthError("EmptyPrompt", "empty prompt")
    return f"Solve the following {p.domain} problem. Put the final answer after the reasoning.\n\nProblem:\n{p.prompt}"


def _last_fence(text: str) -> str | None:
    """Body of the last ``` block whose opening fence starts a line and has a line break after it."""
    last, i = None, 0
    while True:
        start = text.find("```", i)
        if start < 0:
            return last
        if start and text[start - 1] != "\n":
            i = start + 3
            continue
        nl = text.find("\n", start + 3)
        end = text.find("```", nl + 1) if nl >= 0 else -1
        if nl < 0 or end < 0:
            return last
        last, i = text[nl + 1:end], end + 3


def extract_answer(raw: str) -> str:
    """The last ``answer: ...`` line, else the body of the last fenced block, else the last
    non-blank line."""
    text = raw.rstrip(_WS)
    if not text:
        return ""
    lines = [l[:-1] if l.endswith("\r") else l for l in text.split("\n")]
    tagged = [m.group(1).strip(_WS) for m in map(_ANSWER.match, lines) if m]
    if tagged:
        return tagged[-1]
    fenced = _last_fence(text)
    if fenced is not None:
        return fenced
    return next((l for l in reversed(lines) if l.strip(_WS)), "")


@dataclass
class Sample:
    problem_id: str
    text: str
    answer: str
    passed: bool
    token_count: int


@dataclass
class RejectionResult:
    problem_id: str
    n_generated: int
    n_accepted: int
    samples: list = field(default_factory=list)

    @property
    def rate(self) -> float:
        return self.n_accepted / self.n_generated if self.n_generated else 0.0


def verified_correct_rate(results: Sequence[RejectionResult]) -> float:
    gen = sum(r.n_generated for r in results)
    return sum(r.n_accepted for r in results) / gen if gen else 0.0


class RejectionSampler:
    def __init__(self, generate, verify, n_samples=8, max_tokens=512, temperature=0.7, max_batch=8, counter=None):
        if max_batch <= 0:
            raise SynthError("Message", "max_batch must be > 0")
        self.generate, self.verify, self.n_samples = generate, verify, n_samples
        self.max_tokens, self.temperature, self.max_batch, self.counter = max_tokens, temperature, max_batch, counter

    def sample(self, problem: Problem, n: int | None = None) -> RejectionResult:
        return self.sample_many([problem], n)[0]

    def sample_many(self, problems: Sequence[Problem], n: int | None = None) -> list[RejectionResult]:
        n = self.n_samples if n is None else n
        if not problems:
            raise SynthError("EmptyBatch", "empty batch")
        if n == 0:
            raise SynthError("ZeroSamples", "n_samples must be > 0")
        prompts = [solve_prompt(p) for p in problems for _ in range(n)]
        outs = iter(_generate_chunked(self.generate, prompts, self.max_tokens, self.temperature, self.max_batch))
        results = []
        for p in problems:
            samples = []
            for _ in range(n):
                text = next(outs)
                ans = extract_answer(text)
                samples.append(Sample(p.problem_id, text, ans, bool(self.verify(p, ans)), token_count(text, self.counter)))
            results.append(RejectionResult(p.problem_id, n, sum(s.passed for s in samples), samples))
        return results


# ------------------------------------------------------------------ E3: procedural ARC grids
N_COLORS, MAX_GRID, MAX_SAMPLE_DIM, MAX_PAIR_ATTEMPTS = 10, 30, 8, 10000
DIHEDRALS = ("identity", "rot90", "rot180", "rot270", "flip_h", "flip_v", "transpose", "anti_transpose")
FAMILIES = ("translate", "recolor", "crop", "tile", "gravity", "mirror", "scale", "border")
_FAMILY_KEYS = {"translate": {"dx", "dy", "bg"}, "recolor": {"src", "dst"}, "crop": {"bg"}, "tile": {"nx", "ny"},
                "gravity": {"dir", "bg"}, "mirror": {"dihedral"}, "scale": {"factor"}, "border": {"color", "width"}}
_M64 = (1 << 64) - 1


def as_grid(cells) -> np.ndarray:
    """Validated ``(rows, cols)`` uint8 array of ARC colours."""
    rows = list(cells)
    if not rows or len(rows[0]) == 0:
        raise SynthError("EmptyGrid", "empty grid")
    if any(len(r) != len(rows[0]) for r in rows):
        raise SynthError("JaggedGrid", "jagged grid")
    if len(rows) > MAX_GRID or len(rows[0]) > MAX_GRID:
        raise SynthError("GridSize", f"grid size {len(rows)}x{len(rows[0])} out of range")
    g = np.asarray(rows, dtype=np.int64)
    if g.min() < 0 or g.max() >= N_COLORS:
        raise SynthError("BadColor", "ARC color out of range")
    return g.astype(np.uint8)


def dihedral(cells, k) -> np.ndarray:
    """The eight symmetries of the square, by name or index (rot90 is clockwise)."""
    if isinstance(k, str):
        if k not in DIHEDRALS:
            raise SynthError("Message", f"unknown dihedral {k}")
        k = DIHEDRALS.index(k)
    if not 0 <= k < 8:
        raise SynthError("BadDihedral", f"dihedral index {k} out of range")
    g = as_grid(cells)
    ops = (lambda a: a, lambda a: np.rot90(a, -1), lambda a: np.rot90(a, 2), lambda a: np.rot90(a, 1),
           lambda a: a[:, ::-1], lambda a: a[::-1, :], lambda a: a.T, lambda a: np.rot90(a, 2).T)
    return np.ascontiguousarray(ops[k](g))


def color_perm(cells, perm) -> np.ndarray:
    p = list(perm)
    if sorted(p) != list(range(N_COLORS)):
        raise SynthError("BadPermutation", "color permutation is not a permutation of 0..10")
    return np.asarray(p, dtype=np.uint8)[as_grid(cells)]


@dataclass(frozen=True)
class FamilySpec:
    kind: str
    params: tuple                     # sorted (name, value) pairs

    @staticmethod
    def make(kind: str, params: dict) -> "FamilySpec":
        if kind not in FAMILIES:
            raise SynthError("Message", f"unknown family {kind}")
        return FamilySpec(kind, tuple(sorted((str(k), int(v)) for k, v in params.items())))

    def family_id(self) -> str:
        return self.kind + (":" + ",".join(f"{k}={v}" for k, v in self.params) if self.params else "")

    def validate(self) -> dict:
        p = dict(self.params)
        color = lambda v: 0 <= v < N_COLORS          # noqa: E731
        ok = set(p) == _FAMILY_KEYS[self.kind] and {
            "translate": lambda: color(p["bg"]),
            "recolor": lambda: color(p["src"]) and color(p["dst"]) and p["src"] != p["dst"],
            "crop": lambda: color(p["bg"]),
            "tile": lambda: 1 <= p["nx"] <= MAX_GRID and 1 <= p["ny"] <= MAX_GRID,
            "gravity": lambda: 0 <= p["dir"] <= 3 and color(p["bg"]),
            "mirror": lambda: 0 <= p["dihedral"] < 8,
            "scale": lambda: p["factor"] in (2, 3),
            "border": lambda: color(p["color"]) and p["width"] in (1, 2),
        }[self.kind]()
        if not ok:
            raise SynthError("UnknownFamily", "unknown family")
        return p

    def apply(self, cells) -> np.ndarray:
        p = self.validate()
        g = np.asarray(cells, dtype=np.uint8)
        kind = self.kind
        if kind == "translate":                      # objects wrap round, later cells win
            out = np.full_like(g, p["bg"])
            r, c = np.nonzero(g != p["bg"])
            out[(r + p["dy"]) % g.shape[0], (c + p["dx"]) % g.shape[1]] = g[r, c]
        elif kind == "recolor":
            out = np.where(g == p["src"], np.uint8(p["dst"]), g)
        elif kind == "crop":                         # bounding box of everything that is not background
            r, c = np.nonzero(g != p["bg"])
            out = g[r.min():r.max() + 1, c.min():c.max() + 1] if r.size else np.full((1, 1), p["bg"], np.uint8)
        elif kind == "tile":
            out = np.tile(g, (p["ny"], p["nx"]))
        elif kind == "gravity":                      # 0 down, 1 up, 2 left, 3 right; order of the objects kept
            lines = g.T if p["dir"] <= 1 else g      # fall along each line, towards its start or its end
            to_end = p["dir"] in (0, 3)
            out = np.full_like(lines, p["bg"])
            for i, line in enumerate(lines):
                objs = line[line != p["bg"]]
                if to_end:
                    out[i, line.size - objs.size:] = objs
                else:
                    out[i, :objs.size] = objs
            out = out.T if p["dir"] <= 1 else out
        elif kind == "mirror":
            out = dihedral(g, p["dihedral"])
        elif kind == "scale":
            out = np.kron(g, np.ones((p["factor"], p["factor"]), dtype=np.uint8))
        else:                                        # border
            out = np.pad(g, p["width"], constant_values=p["color"])
        return as_grid(np.ascontiguousarray(out).tolist())

    def max_input_hw(self) -> tuple[int, int]:
        p = dict(self.params)
        if self.kind == "tile":
            return MAX_GRID // p["ny"], MAX_GRID // p["nx"]
        if self.kind == "scale":
            return MAX_GRID // p["factor"], MAX_GRID // p["factor"]
        if self.kind == "border":
            return MAX_GRID - 2 * p["width"], MAX_GRID - 2 * p["width"]
        return MAX_GRID, MAX_GRID


class SplitMix64:
    """The 64-bit SplitMix stream the generators draw from (``below(n)`` = next() mod n)."""

    def __init__(self, seed: int):
        self.state = seed & _M64

    def next(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        return z ^ (z >> 31)

    def below(self, n: int) -> int:
        return self.next() % n


@dataclass
class Pair:
    input: np.ndarray
    output: np.ndarray


@dataclass
class Task:
    family_id: str
    seed: int
    train: list
    test: Pair


def generate_task(spec: FamilySpec, seed: int, n_train: int = 3) -> Task:
    """``n_train + 1`` distinct (input, output) pairs of one family; the last drawn is the test
    pair. Inputs are uniform colours on a uniform shape of at most 8 x 8 (less where the output
    would outgrow 30 x 30)."""
    spec.validate()
    if n_train == 0:
        raise SynthError("EmptyTrain", "empty train")
    rng = SplitMix64(seed)
    mh, mw = (min(v, MAX_SAMPLE_DIM) for v in spec.max_input_hw())
    pairs, seen, attempts = [], set(), 0
    while len(pairs) < n_train + 1:
        attempts += 1
        if attempts > MAX_PAIR_ATTEMPTS:
            raise SynthError("Message", "could not sample distinct pairs")
        h = 1 + rng.below(mh)
        w = 1 + rng.below(mw)
        grid = np.array([rng.below(N_COLORS) for _ in range(h * w)], dtype=np.uint8).reshape(h, w)
        out = spec.apply(grid)
        key = (grid.shape, grid.tobytes(), out.shape, out.tobytes())
        if key in seen:
            continue
        seen.add(key)
        pairs.append(Pair(grid, out))
    return Task(spec.family_id(), seed, pairs[:-1], pairs[-1])


def parameter_grid() -> list[FamilySpec]:
    mk = FamilySpec.make
    colors = range(N_COLORS)
    grid = [mk("translate", {"dx": dx, "dy": dy, "bg": bg}) for bg in colors for dx in range(-3, 4) for dy in range(-3, 4)]
    grid += [mk("recolor", {"src": a, "dst": b}) for a in colors for b in colors if a != b]
    grid += [mk("crop", {"bg": bg}) for bg in colors]
    grid += [mk("tile", {"nx": nx, "ny": ny}) for nx in range(1, 5) for ny in range(1, 5)]
    grid += [mk("gravity", {"dir": d, "bg": bg}) for bg in colors for d in range(4)]
    grid += [mk("mirror", {"dihedral": d}) for d in range(8)]
    grid += [mk("scale", {"factor": f}) for f in (2, 3)]
    grid += [mk("border", {"color": c, "width": w}) for c in colors for w in (1, 2)]
    return grid


def sample_family_specs(n: int, seed: int) -> list[FamilySpec]:
    """The first ``n`` of a Fisher-Yates shuffle (front to back) of the parameter grid."""
    if n == 0:
        return []
    specs = parameter_grid()
    if n > len(specs):
        raise SynthError("Message", "requested more family specs than the parameter grid")
    rng = SplitMix64(seed)
    for i in range(len(specs)):
        j = i + rng.below(len(specs) - i)
        specs[i], specs[j] = specs[j], specs[i]
    return specs[:n]


def augment_pair(p: Pair, k, perm) -> Pair:
    return Pair(color_perm(dihedral(p.input, k), perm), color_perm(dihedral(p.output, k), perm))


def augment_task(t: Task, k, perm) -> Task:
    return Task(t.family_id, t.seed, [augment_pair(p, k, perm) for p in t.train], augment_pair(t.test, k, perm))


def corpus_sample(specs: Sequence[FamilySpec], seed: int, n_train: int, n: int) -> list[Task]:
    if n == 0:
        raise SynthError("EmptyTasks", "empty tasks")
    if not specs:
        raise SynthError("UnknownFamily", "unknown family")
    if n_train == 0:
        raise SynthError("EmptyTrain", "empty train")
    return [generate_task(specs[i % len(specs)], seed + i, n_train) for i in range(n)]


def diversity_stats(tasks: Sequence[Task]) -> dict:
    """Counts a corpus is judged by: families, distinct test inputs / outputs, distinct whole
    tasks, distinct grid shapes, the colour histogram over every grid, and the share of tasks
    that repeat an earlier one."""
    key = lambda g: (g.shape, g.tobytes())          # noqa: E731
    grids = [g for t in tasks for p in (*t.train, t.test) for g in (p.input, p.output)]
    whole = {(tuple((key(p.input), key(p.output)) for p in t.train), key(t.test.input), key(t.test.output))
             for t in tasks}
    hist = np.bincount(np.concatenate([g.ravel() for g in grids]), minlength=N_COLORS) if grids else np.zeros(N_COLORS, int)
    return {"n_tasks": len(tasks), "n_families": len({t.family_id for t in tasks}),
            "unique_test_inputs": len({key(t.test.input) for t in tasks}),
            "unique_test_outputs": len({key(t.test.output) for t in tasks}),
            "unique_tasks": len(whole), "unique_shapes": len({g.shape for g in grids}),
            "color_histogram": [int(v) for v in hist[:N_COLORS]],
            "collision_rate": 1.0 - len(whole) / len(tasks) if tasks else 0.0}
