"""Behaviour list of the data-mixture arithmetic (C++ ``native.mixture``; reference
data/mixture/tests/{validate,mix_hash,sample,decay,drop,ablations,catalog,tokens_seen,
properties}.rs): validation rules, the canonical JSON and its hash, inverse-CDF sampling in
source-table order, the decay re-weighting, drop-one ablations and the flagship catalog."""
import hashlib
import json
import math
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

MX = native.mixture
SRC = list(MX.SOURCES)


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def mix(weights, mix_id="m1", bucket="bucket", phase="pretrain"):
    return MX.Mix(mix_id, bucket, phase, weights)


def uniform8():
    return mix({s: 0.125 for s in SRC}, "uniform8")


def ordered(weights):
    return [(s, weights[s]) for s in SRC if s in weights]


# ------------------------------------------------------------------------------ validation
def test_source_table_and_constants():
    assert SRC == ["web", "code", "math_science_arxiv", "books_papers", "synthetic_rewrites", "synthetic_reasoning",
                   "procedural_arc", "agentic_trajectories"]
    assert MX.DECAY_SOURCES == ["code", "math_science_arxiv", "synthetic_reasoning"] and MX.WEIGHT_SUM_TOL == 1e-9


def test_valid_mixes():
    for m in (uniform8(), mix({"web": 0.5, "code": 0.5}), mix({"web": 1.0}), mix({"web": 1 / 3, "code": 1 / 3, "books_papers": 1 / 3}),
              mix({"web": 0.5 + 4e-10, "code": 0.5})):
        MX.validate_mix(m)


@pytest.mark.parametrize("build", [
    lambda: mix({"web": 1.0}, mix_id=""), lambda: mix({"web": 1.0}, bucket=""), lambda: mix({}),
    lambda: mix({"web": 0.0, "code": 1.0}), lambda: mix({"web": -0.5, "code": 1.5}), lambda: mix({"web": math.nan, "code": 0.5}),
    lambda: mix({"web": math.inf}), lambda: mix({"web": 0.5, "code": 0.4}), lambda: mix({"web": 0.5 + 1e-6, "code": 0.5}),
])
def test_invalid_mixes_are_config_errors(build):
    assert err(lambda: MX.validate_mix(build())).kind == "Config"


def test_unknown_sources_are_refused_when_the_mix_is_built():
    assert err(lambda: mix({"weeb": 1.0})).kind == "UnknownSource"
    assert err(lambda: mix({"web": 0.5, "Web": 0.5})).kind == "UnknownSource"


# ------------------------------------------------------------------------------ canonical form / hash
def test_canonical_json_is_compact_in_table_order_and_hash_is_its_sha256():
    m = mix({"agentic_trajectories": 0.25, "web": 0.5, "code": 0.25})                 # given out of order
    text = MX.canonical_json(m)
    assert text == '{"mix_id":"m1","mix_bucket":"bucket","phase":"pretrain","weights":{"web":0.5,"code":0.25,"agentic_trajectories":0.25}}'
    assert " " not in text and "\n" not in text and json.loads(text)["weights"] == {"web": 0.5, "code": 0.25, "agentic_trajectories": 0.25}
    h = MX.mix_hash(m)
    assert h == hashlib.sha256(text.encode()).hexdigest() == MX.mix_hash(m) and h == h.lower()
    same = mix({"code": 0.25, "web": 0.5, "agentic_trajectories": 0.25})
    assert MX.mix_hash(same) == h                                                     # insertion order is irrelevant
    others = [mix({"web": 0.5, "code": 0.25, "agentic_trajectories": 0.25}, mix_id="m2"),
              mix({"web": 0.5, "code": 0.25, "agentic_trajectories": 0.25}, phase="decay"),
              mix({"web": 0.5, "code": 0.25, "agentic_trajectories": 0.25}, bucket="b2"),
              mix({"web": 0.25, "code": 0.5, "agentic_trajectories": 0.25})]
    assert len({h} | {MX.mix_hash(o) for o in others}) == 5
    assert err(lambda: MX.canonical_json(mix({"web": math.nan}))).kind == "Config"
    u = json.loads(MX.canonical_json(uniform8()))
    assert list(u["weights"]) == SRC and list(u) == ["mix_id", "mix_bucket", "phase", "weights"]


# ------------------------------------------------------------------------------ sampling
def test_sampling_is_the_inverse_cdf_in_table_order():
    m = mix({"code": 0.25, "web": 0.5, "procedural_arc": 0.25})
    assert MX.sample_source(m, 0.0) == "web" and MX.sample_source(m, 0.4999) == "web"
    assert MX.sample_source(m, 0.5) == "code" and MX.sample_source(m, 0.7499) == "code"
    assert MX.sample_source(m, 0.75) == "procedural_arc" and MX.sample_source(m, math.nextafter(1.0, 0.0)) == "procedural_arc"
    u8 = uniform8()
    for k, s in enumerate(SRC):
        assert MX.sample_source(u8, k / 8) == s and MX.sample_source(u8, (k + 0.999) / 8) == s
    for bad in (1.0, 1.5, -0.001, math.nan, math.inf, -math.inf):
        assert err(lambda: MX.sample_source(m, bad)).kind == "Config"
    assert err(lambda: MX.sample_source(mix({"web": 0.5, "code": 0.4}), 0.1)).kind == "Config"
    rng = random.Random(1)
    last = -1
    for u in sorted(rng.random() for _ in range(200)):                                 # monotone in table order
        idx = SRC.index(MX.sample_source(u8, u))
        assert idx >= last
        last = idx
    counts = {s: 0 for s in m.weights}
    for i in range(4000):
        counts[MX.sample_source(m, (i + 0.5) / 4000)] += 1
    assert counts == {"web": 2000, "code": 1000, "procedural_arc": 1000}


# ------------------------------------------------------------------------------ decay
def m_decay(weights, factor):
    raw = {s: w * (factor if s in MX.DECAY_SOURCES else 1.0) for s, w in weights.items()}
    total = sum(raw.values())
    return {s: w / total for s, w in raw.items()}


@pytest.mark.parametrize("factor", [2.0, 1.5, 10.0])
def test_decay_boosts_the_decay_sources_and_renormalises(factor):
    for base in (uniform8(), mix({"web": 0.6, "code": 0.3, "books_papers": 0.1}), mix({"web": 0.5, "books_papers": 0.5})):
        d = MX.decay_reweight(base, factor)
        want = m_decay(dict(base.weights), factor)
        assert d.phase == "decay" and d.mix_id == base.mix_id and set(d.weights) == set(base.weights)
        assert sum(d.weights.values()) == pytest.approx(1.0, abs=1e-12)
        for s, w in want.items():
            assert d.weights[s] == pytest.approx(w, rel=1e-12)
            if any(x in base.weights for x in MX.DECAY_SOURCES) and len(set(base.weights) - set(MX.DECAY_SOURCES)):
                assert (d.weights[s] > base.weights[s]) == (s in MX.DECAY_SOURCES)
        MX.validate_mix(d)
    again = MX.decay_reweight(MX.decay_reweight(uniform8(), 2.0), 2.0)                 # an already decayed mix still re-weights
    assert again.weights["code"] > MX.decay_reweight(uniform8(), 2.0).weights["code"]


def test_decay_argument_errors():
    for bad in (1.0, 0.5, 0.0, -2.0, math.nan, math.inf):
        assert err(lambda: MX.decay_reweight(uniform8(), bad)).kind == "Config"
    assert err(lambda: MX.decay_reweight(mix({"web": 0.5, "code": 0.4}), 2.0)).kind == "Config"


# ------------------------------------------------------------------------------ drop / ablations
def test_drop_renormalises_and_keeps_ratios():
    base = mix({"web": 0.5, "code": 0.3, "books_papers": 0.2})
    d = MX.drop_source(base, "web")
    assert ordered(d.weights) == [("code", pytest.approx(0.6)), ("books_papers", pytest.approx(0.4))]
    assert d.weights["code"] / d.weights["books_papers"] == pytest.approx(0.3 / 0.2) and d.phase == base.phase
    assert d.mix_id == base.mix_id and d.mix_bucket == base.mix_bucket                 # the id is the caller's to change
    for s in SRC:
        got = MX.drop_source(uniform8(), s)
        assert s not in got.weights and len(got.weights) == 7 and all(w == pytest.approx(1 / 7) for w in got.weights.values())
        MX.validate_mix(got)
    assert err(lambda: MX.drop_source(base, "procedural_arc")).kind == "UnknownSource"    # not part of this mix
    assert err(lambda: MX.drop_source(mix({"web": 1.0}), "web")).kind == "Config"         # the last one cannot go
    assert err(lambda: MX.drop_source(mix({"web": 1.0}), "code")).kind == "UnknownSource"  # absent beats "last one"


def test_rung_two_ablations_drop_each_source_once_in_table_order():
    ab = MX.rung2_ablations(uniform8())
    assert len(ab) == 8 and [next(s for s in SRC if s not in a.weights) for a in ab] == SRC
    assert [a.weights for a in ab] == [MX.drop_source(uniform8(), s).weights for s in SRC]
    assert len({MX.mix_hash(a) for a in ab}) == 8                                      # told apart by their weights
    two = MX.rung2_ablations(mix({"code": 0.25, "web": 0.75}))
    assert [dict(a.weights) for a in two] == [{"code": 1.0}, {"web": 1.0}]
    assert err(lambda: MX.rung2_ablations(mix({"web": 1.0}))).kind == "Config"
    assert err(lambda: MX.rung2_ablations(mix({"web": 0.5, "code": 0.4}))).kind == "Config"


# ------------------------------------------------------------------------------ catalog / tokens
def test_flagship_catalog_rows():
    cat = MX.flagship_catalog()
    assert [row[0] for row in cat] == SRC
    by = {row[0]: row for row in cat}
    assert by["books_papers"][1] is None                                               # no unique-token figure published
    for name, unique, lo, hi in cat:
        assert 0 < lo <= hi and (unique is None or unique > 0)


def test_tokens_seen_is_unique_tokens_times_epochs():
    assert MX.tokens_seen(None, 5) is None and MX.tokens_seen(10, 0) == 0 and MX.tokens_seen(7, 3) == 21
    cat = {row[0]: row for row in MX.flagship_catalog()}
    assert MX.tokens_seen(cat["web"][1], 3) == cat["web"][1] * 3 and MX.tokens_seen(cat["books_papers"][1], 3) is None


@pytest.mark.parametrize("seed", range(5))
def test_generated_mixes_follow_the_model(seed):
    rng = random.Random(seed)
    names = rng.sample(SRC, rng.randint(2, 8))
    raw = [rng.random() + 0.05 for _ in names]
    weights = {s: w / sum(raw) for s, w in zip(names, raw)}
    m = mix(weights)
    MX.validate_mix(m)
    want = json.dumps({"mix_id": "m1", "mix_bucket": "bucket", "phase": "pretrain", "weights": dict(ordered(weights))}, separators=(",", ":"))
    assert json.loads(MX.canonical_json(m)) == json.loads(want) and list(json.loads(MX.canonical_json(m))["weights"]) == [s for s, _ in ordered(weights)]
    cum, edges = 0.0, []
    for s, w in ordered(weights):
        cum += w
        edges.append((cum, s))
    for _ in range(200):
        u = rng.random()
        assert MX.sample_source(m, u) == next((s for c, s in edges if u < c), edges[-1][1])
    victim = rng.choice(names)
    dropped = MX.drop_source(m, victim)
    rest = 1.0 - weights[victim]
    for s, w in dropped.weights.items():
        assert w == pytest.approx(weights[s] / rest, rel=1e-12)
    assert MX.mix_hash(MX.decay_reweight(m, 2.0)) == hashlib.sha256(MX.canonical_json(MX.decay_reweight(m, 2.0)).encode()).hexdigest()
