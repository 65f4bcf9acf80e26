"""Event log (hash chain, torn-line recovery, fail-closed), mixture, tokenizer."""
import hashlib
import json

import pytest

from prometheus_b200 import contracts, native

LOG = native.log
MX = native.mixture
TK = native.tokenizer


def test_event_log_chain_and_line_format(tmp_path):
    d = str(tmp_path / "log")
    log = LOG.EventLog.create(d)
    with pytest.raises(native.NativeError):
        LOG.EventLog.create(d)
    e0 = log.append("task.enqueued", json.dumps({"b": 2, "a": 1}), "2026-01-01T00:00:10Z", task_id="t1")
    e1 = log.append("task.claimed", "{}", "11", task_id="t1", attempt=1, node_id="n0")
    assert e0.seq == 0 and e0.prev_hash == "0" * 64 and e1.prev_hash == e0.hash
    ph = hashlib.sha256(b'{"a":1,"b":2}').hexdigest()
    assert e0.payload_hash == ph
    assert e0.hash == hashlib.sha256(f"0|{'0' * 64}|{ph}|2026-01-01T00:00:10Z|task.enqueued".encode()).hexdigest()
    lines = (tmp_path / "log" / "events.jsonl").read_text().splitlines()
    first = json.loads(lines[0])
    assert list(first) == ["schema_id", "schema_version", "seq", "prev_hash", "hash", "timestamp",
                           "event_type", "task_id", "attempt", "node_id", "payload", "payload_hash"]
    contracts.validate(first)
    with pytest.raises(native.NativeError) as e:
        log.append("", "{}", "12")
    assert e.value.kind == "Schema"
    del log
    again = LOG.EventLog.open(d)
    assert len(again) == 2 and again.get(1).node_id == "n0"
    again.verify()


def test_event_log_torn_tail_is_truncated_and_broken_chain_fails_closed(tmp_path):
    d = tmp_path / "log"
    log = LOG.EventLog.create(str(d))
    for i in range(3):
        log.append("tick", json.dumps({"i": i}), str(i))
    del log
    path = d / "events.jsonl"
    good = path.read_bytes()
    path.write_bytes(good + b'{"schema_id":"prometheus.event_log","seq":3,"pre')   # torn append
    reopened = LOG.EventLog.open(str(d))
    assert len(reopened) == 3 and path.read_bytes() == good
    reopened.append("tick", "{}", "3")
    del reopened
    lines = path.read_bytes().split(b"\n")
    lines[1] = lines[1].replace(b'"i":1', b'"i":7')
    path.write_bytes(b"\n".join(lines))
    with pytest.raises(native.NativeError) as e:
        LOG.EventLog.open(str(d))
    assert e.value.kind == "Corrupt"
    with pytest.raises(native.NativeError):
        LOG.EventLog.open(str(tmp_path / "missing"))


def _mix(**w):
    return MX.Mix("m1", "bucket", "pretrain", w)


def test_mixture_hash_decay_ablation_sampling():
    m = _mix(web=0.5, code=0.25, synthetic_reasoning=0.25)
    MX.validate_mix(m)
    text = MX.canonical_json(m)
    assert text == ('{"mix_id":"m1","mix_bucket":"bucket","phase":"pretrain",'
                    '"weights":{"web":0.5,"code":0.25,"synthetic_reasoning":0.25}}')
    assert MX.mix_hash(m) == hashlib.sha256(text.encode()).hexdigest()
    d = MX.decay_reweight(m, 2.0)
    assert d.phase == "decay" and d.weights["web"] == pytest.approx(1 / 3)
    assert sum(d.weights.values()) == pytest.approx(1.0)
    ab = MX.rung2_ablations(m)
    assert [sorted(a.weights) for a in ab] == [["code", "synthetic_reasoning"],
                                               ["synthetic_reasoning", "web"], ["code", "web"]]
    assert MX.sample_source(m, 0.0) == "web" and MX.sample_source(m, 0.6) == "code"
    assert MX.sample_source(m, 0.99) == "synthetic_reasoning"
    with pytest.raises(native.NativeError):
        MX.validate_mix(_mix(web=0.5, code=0.4))
    with pytest.raises(native.NativeError) as e:
        _mix(weeb=1.0)
    assert e.value.kind == "UnknownSource"
    with pytest.raises(native.NativeError):
        MX.sample_source(m, 1.0)
    assert MX.tokens_seen(10, 3) == 30 and MX.tokens_seen(None, 3) is None
    assert len(MX.flagship_catalog()) == 8 and MX.SOURCES[0] == "web"


def test_tokenizer_train_encode_roundtrip_and_artifacts(tmp_path):
    docs = ["the cat sat on the mat", "the dog sat on the log", "héllo wörld"]
    t = TK.Tokenizer.train(docs, "tok-test", 290)
    assert t.merges[0] == (4 + ord("t"), 4 + ord("h")) or len(t.merges) == 20
    # most frequent pair first, ties to the smallest (left, right)
    counts = {}
    for doc in docs:
        b = [4 + c for c in doc.encode()]
        for p in zip(b, b[1:]):
            counts[p] = counts.get(p, 0) + 1
    best = max(counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))[0]
    assert t.merges[0] == best
    for doc in docs + ["unseen ☃ text"]:
        ids = t.encode(doc)
        assert t.decode(ids) == doc
    assert len(t.encode(docs[0])) < len(docs[0].encode())
    assert t.encode_grid([0, 9, 3]) == [260, 269, 263]
    with pytest.raises(native.NativeError) as e:
        t.encode_grid([10])
    assert e.value.kind == "BadColor"
    with pytest.raises(native.NativeError) as e:
        t.decode([100000])
    assert e.value.kind == "UnknownId"
    with pytest.raises(native.NativeError) as e:
        TK.Tokenizer.train(docs, "x", 270)
    assert e.value.kind == "VocabTooSmall"
    t.freeze("2026-01-01T00:00:00Z")
    t.freeze("2026-01-01T00:00:00Z")
    with pytest.raises(native.NativeError):
        t.freeze("2027-01-01T00:00:00Z")
    pointer = json.loads(t.save(str(tmp_path / "tok")))
    blob = (tmp_path / "tok" / "vocab.jsonl").read_bytes()
    assert pointer["artifact"]["content_hash"] == hashlib.sha256(blob).hexdigest() == t.vocab_hash()
    lines = blob.decode().splitlines()
    assert json.loads(lines[0]) == {"id": 0, "kind": "special", "name": "bos"}
    assert json.loads(lines[4]) == {"byte": 0, "id": 4, "kind": "byte"}
    assert json.loads(lines[-1])["kind"] == "header" and len(lines) == 4 + 256 + 10 + len(t.merges) + 1
    contract = json.loads((tmp_path / "tok" / "tokenizer.json").read_text())
    contracts.validate(contract)
    contracts.validate(pointer)
    back = TK.Tokenizer.load(str(tmp_path / "tok"))
    assert back.merges == t.merges and back.frozen and back.encode(docs[1]) == t.encode(docs[1])
    assert TK.baseline_byte_tokens_per_word("ab cd") == 2.5 and t.tokens_per_word("the cat") <= 3.5
