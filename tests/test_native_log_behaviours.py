"""Behaviour list of the hash-chained event log (C++ ``native.log``; reference
harness/log/tests/{append,create_open,crash,fault,hashes,properties,schema}.rs): hashes
against published golden values and a Python restatement, sequence and chain rules, a child
process that dies right after an append, torn and mutated lines, schema checks on replay."""
import hashlib
import json
import os
import subprocess
import sys

import pytest

from prometheus_b200 import contracts, native
from prometheus_b200.native import NativeError

LOG = native.log
ZERO = "0" * 64
F1_TS, F1_TYPE = "2026-09-16T12:00:00Z", "session.start"


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


def canonical(obj):
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode()


def p_hash(obj):
    return hashlib.sha256(canonical(obj)).hexdigest()


def e_hash(seq, prev, ph, ts, kind):
    return hashlib.sha256(f"{seq}|{prev}|{ph}|{ts}|{kind}".encode()).hexdigest()


def replay(path):
    """Independent reader: returns the list of records of a valid chain, else raises."""
    out, prev = [], ZERO
    for n, line in enumerate(open(path, encoding="utf-8").read().splitlines()):
        rec = json.loads(line)
        assert rec["seq"] == n and rec["prev_hash"] == prev and rec["payload_hash"] == p_hash(rec["payload"])
        assert rec["hash"] == e_hash(n, prev, rec["payload_hash"], rec["timestamp"], rec["event_type"])
        prev = rec["hash"]
        out.append(rec)
    return out


# ------------------------------------------------------------------------------ hashes
def test_published_hash_values():
    assert LOG.GENESIS_PREV_HASH == ZERO
    assert LOG.payload_hash("{}") == "44136fa355b3678a1146ad16f7e8649e94fb4fc21fe77e8310c060f61caaff8a"
    assert LOG.payload_hash('{"cycle": 1}') == "9ea9926526cd16b40c70cd8988bfa74bb6c857dbb64faf55ea20a1c42d5ab122"
    assert LOG.payload_hash('{"msg": "hello", "n": 1, "ok": true}') == "2fa4793603fe17e52b611317579148d3b47e527b3f6f8163240c0d734ca6273c"
    assert LOG.payload_hash('{"note": "ΔRCI café"}') == "e8d13b8f2f569be2e3ef0a2803761f39ed4d93cf167636d3e3c7a6d3c7562e00"
    ph = LOG.payload_hash('{"cycle":1}')
    assert LOG.event_hash(0, ZERO, ph, F1_TS, F1_TYPE) == "c975ddd2d64d8781552891f9b1b5241208b703554c6f323a47336d2b5de5d74c"


@pytest.mark.parametrize("payload", [{}, {"b": 1, "a": {"z": [3, {"y": 1, "x": 2}], "k": None}}, {"n": 10, "f": 1.5, "neg": -3, "big": 2 ** 53},
                                     {"s": "quote \" slash \\ tab \t newline \n", "u": "日本語 ☃", "e": ""}, {"t": True, "f": False, "l": []}])
def test_payload_hash_is_the_sha256_of_sorted_compact_json(payload):
    assert LOG.payload_hash(json.dumps(payload)) == p_hash(payload)
    shuffled = json.dumps(dict(reversed(list(payload.items()))), indent=2)                 # key order and spacing do not matter
    assert LOG.payload_hash(shuffled) == p_hash(payload)


def test_event_hash_is_the_sha256_of_the_bar_joined_fields():
    ph = p_hash({"x": 1})
    for seq in (0, 1, 10, 123456789):
        assert LOG.event_hash(seq, ZERO, ph, "t", "e") == e_hash(seq, ZERO, ph, "t", "e")  # decimal, no leading zeros
    assert LOG.event_hash(10, ZERO, ph, "t", "e") != LOG.event_hash(1, ZERO, ph, "t", "e")
    assert LOG.payload_hash('{"n": 1}') != LOG.payload_hash('{"n": 1.5}')                   # an integer is not written as a float
    assert LOG.payload_hash('{"n": 1}') == p_hash({"n": 1})


# ------------------------------------------------------------------------------ create / open
def test_create_and_open_rules(tmp_path):
    d = tmp_path / "log"
    log = LOG.EventLog.create(str(d))
    assert len(log) == 0 and log.events() == [] and log.get(0) is None and log.dir == str(d)
    assert (d / "events.jsonl").read_bytes() == b""
    log.verify()
    err(lambda: LOG.EventLog.create(str(d)))
    (tmp_path / "file").write_text("x")
    err(lambda: LOG.EventLog.create(str(tmp_path / "file")))
    err(lambda: LOG.EventLog.open(str(tmp_path / "file")))
    err(lambda: LOG.EventLog.create(str(tmp_path / "no" / "parent")))
    err(lambda: LOG.EventLog.open(str(tmp_path / "missing")))
    assert len(LOG.EventLog.open(str(d))) == 0
    (d / "events.jsonl").unlink()
    err(lambda: LOG.EventLog.open(str(d)))                                                 # a directory without its file is not a log


def test_appends_number_and_chain_the_records(tmp_path):
    log = LOG.EventLog.create(str(tmp_path / "log"))
    first = log.append(F1_TYPE, '{"cycle": 1}', F1_TS)
    assert (first.seq, first.prev_hash) == (0, ZERO)
    assert first.payload_hash == "9ea9926526cd16b40c70cd8988bfa74bb6c857dbb64faf55ea20a1c42d5ab122"
    assert first.hash == "c975ddd2d64d8781552891f9b1b5241208b703554c6f323a47336d2b5de5d74c"
    assert (first.task_id, first.attempt, first.node_id) == (None, None, None)
    made = [first] + [log.append("tick", json.dumps({"z": i, "a": [i]}), f"2026-09-16T12:00:0{i}Z", task_id=f"t{i}", attempt=i, node_id="n") for i in range(1, 6)]
    assert [e.seq for e in made] == list(range(6)) and all(b.prev_hash == a.hash for a, b in zip(made, made[1:]))
    assert [e.hash for e in log.events()] == [e.hash for e in made] and log.get(5).hash == made[5].hash and log.get(6) is None and len(log) == 6
    assert err(lambda: log.append("", "{}", "9")).kind == "Schema" and len(log) == 6       # a refused append leaves nothing behind
    err(lambda: log.append("tick", "not json", "9"))
    assert len(log) == 6
    lines = (tmp_path / "log" / "events.jsonl").read_text().splitlines()
    assert len(lines) == 6 and [json.loads(x)["seq"] for x in lines] == list(range(6))     # one object per line
    assert [r["hash"] for r in replay(tmp_path / "log" / "events.jsonl")] == [e.hash for e in made]
    assert lines[3] == made[3].line() and json.loads(lines[3])["payload"] == {"a": [3], "z": 3}
    for rec in map(json.loads, lines):
        contracts.validate(rec)
    assert json.loads(lines[0])["task_id"] is None and json.loads(lines[2])["attempt"] == 2 and json.loads(lines[2])["node_id"] == "n"


@pytest.mark.parametrize("n", [0, 1, 7, 40])
def test_reopen_gives_the_identical_chain_and_appends_continue_it(tmp_path, n):
    d = str(tmp_path / "log")
    log = LOG.EventLog.create(d)
    for i in range(n):
        log.append("e", json.dumps({"i": i, "u": "é☃"}), f"ts{i}")
    want = [e.line() for e in log.events()]
    del log
    again = LOG.EventLog.open(d)
    assert [e.line() for e in again.events()] == want and len(again) == n
    nxt = again.append("after", "{}", "later")
    assert nxt.seq == n and nxt.prev_hash == (json.loads(want[-1])["hash"] if n else ZERO)
    assert json.loads(again.get(n - 1).payload_json if n else "{}").get("u", "é☃") == "é☃"
    assert len(replay(tmp_path / "log" / "events.jsonl")) == n + 1


# ------------------------------------------------------------------------------ crashes
CHILD = """
import os, sys
from prometheus_b200 import native
log = native.log.EventLog.create(sys.argv[1])
for i in range(int(sys.argv[2])):
    log.append("tick", '{"i": %d}' % i, str(i))
if sys.argv[3] == "abort":
    os.abort()
os._exit(0)
"""


@pytest.mark.parametrize("n, how", [(1, "exit"), (2, "exit"), (1, "abort")])
def test_a_process_that_dies_right_after_an_append_loses_nothing(tmp_path, n, how):
    d = str(tmp_path / "log")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join(sys.path))
    subprocess.run([sys.executable, "-c", CHILD, d, str(n), how], env=env, timeout=120, stderr=subprocess.DEVNULL)
    log = LOG.EventLog.open(d)
    assert len(log) == n and [json.loads(e.payload_json)["i"] for e in log.events()] == list(range(n))
    assert log.append("next", "{}", "x").seq == n
    assert len(replay(tmp_path / "log" / "events.jsonl")) == n + 1


def test_torn_lines_never_become_records(tmp_path):
    d = tmp_path / "log"
    log = LOG.EventLog.create(str(d))
    for i in range(3):
        log.append("tick", json.dumps({"i": i}), str(i))
    whole = (d / "events.jsonl").read_bytes()
    fourth = LOG.EventLog.open(str(d)).append("tick", '{"i": 3}', "3").line().encode()
    for cut in (1, len(fourth) // 2, len(fourth) - 1):
        (d / "events.jsonl").write_bytes(whole + fourth[:cut])
        got = LOG.EventLog.open(str(d))
        assert len(got) == 3 and got.append("tick", '{"i": 3}', "3").seq == 3              # the sequence number is not skipped
        assert len(replay(d / "events.jsonl")) == 4
    first = whole.split(b"\n")[0]
    (d / "events.jsonl").write_bytes(first[: len(first) // 2])                             # even the very first line
    empty = LOG.EventLog.open(str(d))
    assert len(empty) == 0 and empty.append("tick", "{}", "0").prev_hash == ZERO


# ------------------------------------------------------------------------------ mutation
def _three(tmp_path):
    d = tmp_path / "log"
    log = LOG.EventLog.create(str(d))
    for i in range(3):
        log.append("tick", json.dumps({"i": i}), str(i), task_id="t")
    return d, [json.loads(x) for x in (d / "events.jsonl").read_text().splitlines()]


def flip(h):
    return ("e" if h[0] == "f" else "f") + h[1:]


def _write(d, recs):
    (d / "events.jsonl").write_text("".join(json.dumps(r, separators=(",", ":")) + "\n" for r in recs))


@pytest.mark.parametrize("mutate", [
    lambda r: r[1].__setitem__("hash", flip(r[1]["hash"])),
    lambda r: r[1].__setitem__("payload_hash", flip(r[1]["payload_hash"])),
    lambda r: r[1].__setitem__("payload", {"i": 99}),
    lambda r: r[2].__setitem__("prev_hash", ZERO),
    lambda r: r[1].__setitem__("seq", 5),
    lambda r: r.pop(1),
    lambda r: r[0].__setitem__("timestamp", "other"),
    lambda r: r[0].__setitem__("event_type", "tock"),
    lambda r: r.insert(1, dict(r[0])),
    lambda r: r.reverse(),
], ids=["hash", "payload_hash", "payload", "prev_hash", "seq", "gap", "timestamp", "type", "duplicate", "order"])
def test_a_changed_complete_line_fails_the_open(tmp_path, mutate):
    d, recs = _three(tmp_path)
    _write(d, recs)
    assert len(LOG.EventLog.open(str(d))) == 3                                             # rewriting unchanged is fine
    mutate(recs)
    _write(d, recs)
    assert err(lambda: LOG.EventLog.open(str(d))).kind in ("Corrupt", "BrokenChain")
    with pytest.raises(Exception):
        replay(d / "events.jsonl")                                                         # the independent reader agrees


@pytest.mark.parametrize("field, value", [("schema_version", 2), ("schema_version", None), ("schema_id", "prometheus.other"), ("schema_id", None)])
def test_foreign_schema_is_rejected_on_replay(tmp_path, field, value):
    d, recs = _three(tmp_path)
    if value is None:
        del recs[0][field]
    else:
        recs[0][field] = value
    _write(d, recs)
    err(lambda: LOG.EventLog.open(str(d)))


def test_a_log_written_by_the_python_restatement_opens(tmp_path):
    d = tmp_path / "log"
    LOG.EventLog.create(str(d))
    recs, prev = [], ZERO
    for i, (payload, task, attempt, node) in enumerate([({"cycle": 1}, None, None, None), ({"k": "ü", "n": [1, 2]}, "t1", 3, "node-a")]):
        ph = p_hash(payload)
        h = e_hash(i, prev, ph, F1_TS, F1_TYPE)
        recs.append({"schema_id": "prometheus.event_log", "schema_version": 1, "seq": i, "prev_hash": prev, "hash": h, "timestamp": F1_TS,
                     "event_type": F1_TYPE, "task_id": task, "attempt": attempt, "node_id": node, "payload": payload, "payload_hash": ph})
        prev = h
    (d / "events.jsonl").write_text("".join(json.dumps(r, ensure_ascii=False) + "\n" for r in recs), encoding="utf-8")
    log = LOG.EventLog.open(str(d))
    assert len(log) == 2 and log.get(0).hash == "c975ddd2d64d8781552891f9b1b5241208b703554c6f323a47336d2b5de5d74c"
    e = log.get(1)
    assert (e.task_id, e.attempt, e.node_id, json.loads(e.payload_json)) == ("t1", 3, "node-a", {"k": "ü", "n": [1, 2]})
    assert log.append("more", "{}", "t").prev_hash == prev
