"""Behaviour list of the provider layer (C++ ``native.providers``; reference
harness/providers/tests/{aimd,broker,failover,fault,properties,validate}.rs): which response
bodies are faults and in what precedence, the additive-increase / multiplicative-decrease
window, ordered failover with capped backoff, and the token broker. Validation, the window
and failover are each compared with a Python model on random inputs."""
import hashlib
import json
import math
import random

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

P, R = native.providers, native.raft


def err(call, *a):
    with pytest.raises(NativeError) as e:
        call(*a)
    return e.value


# ------------------------------------------------------------------------------ validation
def model_validate(body):
    """Returns a fault kind or None."""
    if body.lower() == b"rate_limit":
        return "RateLimitText"
    try:
        obj = json.loads(body.decode("utf-8"))
    except (UnicodeDecodeError, ValueError):
        return "MalformedJson"
    if not isinstance(obj, dict):
        return "MalformedJson"
    if isinstance(obj.get("error"), str) and obj["error"].lower() == "rate_limit":
        return "RateLimitText"
    choices = obj.get("choices")
    if not isinstance(choices, list) or not choices:
        return "EmptyCompletion"

    def truncated_call(call):
        fn = call.get("function") if isinstance(call, dict) else None
        if not isinstance(fn, dict):
            return True
        args = fn.get("arguments")
        if isinstance(args, str):
            try:
                json.loads(args)
                return False
            except ValueError:
                return True
        return not isinstance(args, (dict, list))

    for c in choices:
        if not isinstance(c, dict) or c.get("finish_reason") != "length":
            continue
        if "tool_calls" in c:
            calls = c["tool_calls"]
        elif isinstance(c.get("message"), dict) and "tool_calls" in c["message"]:
            calls = c["message"]["tool_calls"]
        else:
            continue                                                                           # absent; a present null is not a list and counts as cut off
        if not isinstance(calls, list):
            return "TruncatedToolCall"
        if any(truncated_call(x) for x in calls):
            return "TruncatedToolCall"
    return None


def choice(finish="stop", calls="absent", on_message=False):
    c = {"finish_reason": finish, "message": {"content": "hi"}}
    if calls != "absent":
        (c["message"] if on_message else c)["tool_calls"] = calls
    return c


def call(arguments="absent"):
    fn = {"name": "f"}
    if arguments != "absent":
        fn["arguments"] = arguments
    return {"function": fn}


CORPUS = [
    b"rate_limit", b"RATE_LIMIT", b"Rate_Limit", b" rate_limit", b"rate_limit\n", b"rate limit", b'"rate_limit"',
    b'{"error": "rate_limit"}', b'{"error": "RATE_limit", "choices": [], "x": 1}', b'{"error": {"type": "rate_limit"}}', b'{"error": "rate_limit "}',
    b"", b"not json", b"[1]", b"3", b"null", b'"text"', b'{"choices": [', b'{"choices": []} trailing', b"\xff\xfe{}", b"{} ",
    b"{}", b'{"choices": []}', b'{"choices": null}', b'{"choices": {"0": 1}}', b'{"choices": "x"}',
] + [json.dumps({"choices": cs}).encode() for cs in (
    [choice()], [choice("length")], [choice("length", [])], [choice("length", [call('{"a": 1}')])], [choice("length", [call('{"a": 1')])],
    [choice("length", [call("")])], [choice("length", [call(None)])], [choice("length", [call()])], [choice("length", [call({"a": 1})])],
    [choice("length", [call([1])])], [choice("length", [call(5)])], [choice("length", "oops")], [choice("length", {"a": 1})],
    [choice("length", [{"function": "f"}])], [choice("length", [{}])], [choice("length", [call('{"a": 1')], on_message=True)],
    [choice("stop", [call('{"a": 1')])], [choice("tool_calls", [call('{"a"')])], [choice(), choice(), choice("length", [call("{")])],
    [choice("length", [call("{}"), call("[1, 2")])], [5, "x", None],
)]


@pytest.mark.parametrize("body", CORPUS, ids=lambda b: b[:40].decode("latin-1"))
def test_validation_corpus_agrees_with_the_model(body):
    want = model_validate(body)
    if want is None:
        assert json.loads(P.validate_response(body)) == json.loads(body)                       # a success hands back the parsed object
    else:
        assert err(P.validate_response, body).kind == want


def test_precedence_of_faults():
    assert err(P.validate_response, b'{"error": "rate_limit", "choices": []}').kind == "RateLimitText"   # a rate limit beats an empty completion
    assert err(P.validate_response, b"rate_limit").kind == "RateLimitText"                     # and is not "malformed JSON"
    assert err(P.validate_response, json.dumps({"choices": [choice("length", [call("{")])], "error": "other"}).encode()).kind == "TruncatedToolCall"
    assert err(P.validate_response, b'{"choices": [], "x": [').kind == "MalformedJson"


def test_random_bodies_agree_with_the_model():
    rng = random.Random(0)
    args = ['{"a": 1}', '{"a": 1', "", None, {"k": 1}, [1], 7, "absent", "[]", "nul"]
    for _ in range(400):
        cs = []
        for _ in range(rng.randint(0, 3)):
            calls = rng.choice(["absent", [], "text", None, [call(rng.choice(args)) for _ in range(rng.randint(1, 3))], [{"function": 3}]])
            cs.append(choice(rng.choice(["stop", "length", "length", None]), calls, on_message=rng.random() < 0.5))
        obj = {"choices": cs}
        if rng.random() < 0.15:
            obj["error"] = rng.choice(["rate_limit", "Rate_Limit", "other", 5])
        body = json.dumps(obj).encode()
        if rng.random() < 0.1:
            body = body[: rng.randint(0, len(body))]
        want = model_validate(body)
        if want is None:
            P.validate_response(body)
        else:
            assert err(P.validate_response, body).kind == want, body


# ------------------------------------------------------------------------------ AIMD
def model_shrink(window, cfg):
    scaled = window * cfg["decrease"]
    floored = int(min(max(math.floor(scaled), 0), 2 ** 32 - 1)) if math.isfinite(scaled) else 0
    return max(max(window - 1, 0) if floored >= window else floored, cfg["min_window"])


def test_window_steps():
    a = P.Aimd(P.AimdConfig())
    assert a.window == 1
    a.on_success(0)
    assert a.window == 2
    b = P.Aimd(P.AimdConfig(min_window=2, max_window=7, increase=2))
    assert b.window == 2
    for want in (4, 6, 7, 7):                                                                  # grows by the increase, clamps at the maximum
        b.on_success(10)
        assert b.window == want
    b.on_429()
    assert b.window == 3                                                                       # floor(7 / 2)
    b.on_outage()
    assert b.window == 2                                                                       # floor(3 / 2) = 1, clamped at the minimum
    b.on_429()
    assert b.window == 2
    b.on_success(30_000)
    assert b.window == 4                                                                       # exactly at the latency limit is still a success
    b.on_success(30_001)
    assert b.window == 2                                                                       # over it counts as congestion
    for decrease in (1.0, 1.5, 100.0):
        c = P.Aimd(P.AimdConfig(max_window=9, decrease=decrease))
        for _ in range(4):
            c.on_success(1)
        c.on_429()
        assert c.window == 4                                                                   # a factor that would not shrink still gives up one
    assert P.Aimd(P.AimdConfig(min_window=0)).window == 1                                      # never starts at zero


@pytest.mark.parametrize("seed", range(6))
def test_random_sequences_agree_with_the_model(seed):
    rng = random.Random(seed)
    cfg = dict(min_window=rng.randint(0, 4), max_window=rng.randint(4, 40), increase=rng.randint(1, 5), decrease=rng.choice([0.5, 0.75, 0.1, 0.99, 1.0, 2.0, 0.0]),
               latency_limit_ms=rng.choice([0, 10, 30_000]))
    a = P.Aimd(P.AimdConfig(**cfg))
    w = max(cfg["min_window"], 1)
    for _ in range(300):
        op = rng.choice(["ok", "ok", "ok", "429", "outage"])
        if op == "ok":
            lat = rng.choice([0, cfg["latency_limit_ms"], cfg["latency_limit_ms"] + 1, 10 ** 9])
            a.on_success(lat)
            w = model_shrink(w, cfg) if lat > cfg["latency_limit_ms"] else min(w + cfg["increase"], cfg["max_window"])
        else:
            (a.on_429 if op == "429" else a.on_outage)()
            w = model_shrink(w, cfg)
        assert a.window == w, (op, cfg)


# ------------------------------------------------------------------------------ failover
def test_failover_keeps_the_given_order():
    f = P.Failover(["a", "b", "c"])
    assert f.current() == "a" and f.providers == ["a", "b", "c"] and f.down == [] and f.wait_backoff_ms() == 100
    f.mark_down("b")
    assert f.current() == "a"
    f.mark_down("a")
    f.mark_down("a")                                                                           # marking twice changes nothing
    assert f.current() == "c" and sorted(f.down) == ["a", "b"] and f.wait_backoff_ms() == 400
    f.mark_down("c")
    assert err(f.current).kind == "NoProvider" and f.wait_backoff_ms() == 800                  # everything down: a wait, never an exit
    for _ in range(50):
        assert err(f.current).kind == "NoProvider" and f.wait_backoff_ms() == 800
    f.mark_up("b")
    f.mark_up("b")
    assert f.current() == "b"
    f.mark_up("a")
    assert f.current() == "a"                                                                  # the first slot is preferred again
    assert err(f.mark_down, "zz").kind == "NotFound" and err(f.mark_up, "zz").kind == "NotFound"
    empty = P.Failover([])
    assert err(empty.current).kind == "NoProvider" and empty.wait_backoff_ms() == 100
    many = P.Failover([f"p{i}" for i in range(12)])
    waits = []
    for i in range(12):
        many.mark_down(f"p{i}")
        waits.append(many.wait_backoff_ms())
    assert waits == [min(100 * 2 ** (i + 1), 100 * 2 ** 8) for i in range(12)]                 # doubles per provider down, capped at eight doublings


@pytest.mark.parametrize("seed", range(4))
def test_random_failover_operations_agree_with_the_model(seed):
    rng = random.Random(seed)
    names = [f"p{i}" for i in range(rng.randint(1, 6))]
    f, down = P.Failover(names), set()
    for _ in range(200):
        who = rng.choice(names + ["ghost"])
        op = rng.choice(["down", "up"])
        if who == "ghost":
            assert err(f.mark_down if op == "down" else f.mark_up, who).kind == "NotFound"
        elif op == "down":
            f.mark_down(who)
            down.add(who)
        else:
            f.mark_up(who)
            down.discard(who)
        up = [n for n in names if n not in down]
        if up:
            assert f.current() == up[0]
        else:
            assert err(f.current).kind == "NoProvider"
        assert f.wait_backoff_ms() == 100 * 2 ** min(len(down), 8) and sorted(f.down) == sorted(down)


# ------------------------------------------------------------------------------ token broker
def test_only_the_leader_brokers_and_it_commits_the_blob_first(tmp_path):
    g = R.LocalGroup.start(3, str(tmp_path / "g"))
    assert err(P.broker_refresh, g.get(1), "xai", 1_000, b"blob", 5).kind == "NotBroker"       # before any leader exists
    g.tick(0)
    for i in (1, 2):
        assert err(P.broker_refresh, g.get(i), "xai", 1_000, b"blob", 5).kind == "NotBroker" and g.get(i).state()["token"] is None
    (gen, blob), tok = P.broker_refresh(g.get(0), "xai", 60_000, b"secret blob", 7)
    assert (gen, blob) == (1, b"secret blob") and tok.expires_at == 60_007                     # the caller's clock, not the wall clock
    assert tok.token == hashlib.sha256(b"secret blob").hexdigest() and b"secret" not in tok.token.encode()   # a digest, never the blob
    assert all(tuple(g.get(i).state()["token"]) == (1, b"secret blob") for i in range(3))
    (gen2, _), tok2 = P.broker_refresh(g.get(0), "xai", 10, b"next", 8)
    assert gen2 == 2 and tok2.token == hashlib.sha256(b"next").hexdigest() and tok2.expires_at == 18
    assert g.get(0).state()["token_broker"] is None                                            # brokering does not need the role lease
    solo = R.Cluster.bootstrap(str(tmp_path / "solo"), R.NodeInfo("a", ""))
    assert P.broker_refresh(solo, "openai", 1, b"b", 0)[0][0] == 1
