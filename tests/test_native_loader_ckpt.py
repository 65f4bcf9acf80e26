"""C++ loader and checkpoint store: byte-level compatibility with the reference formats
(data/loader/src/lib.rs, ckpt/src/lib.rs) and behaviour under host-injected faults."""
import json
import threading
import time
from pathlib import Path

import pytest

from prometheus_b200 import native

L = native.loader
C = native.ckpt
GOLD = Path(__file__).resolve().parent.parent / "prometheus_b200" / "contracts" / "goldens" / "v1"

M64 = (1 << 64) - 1


def _splitmix_order(n, seed, epoch):
    state = seed ^ ((0x9E3779B97F4A7C15 * (epoch + 1)) & M64)
    order = list(range(n))

    def nxt():
        nonlocal state
        state = (state + 0x9E3779B97F4A7C15) & M64
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    for i in range(n - 1, 0, -1):
        j = nxt() % (i + 1)
        order[i], order[j] = order[j], order[i]
    return order


@pytest.mark.parametrize("n,seed,epoch", [(1, 3, 0), (2, 0, 0), (17, 7, 0), (17, 7, 5), (100, M64, 2**32 - 1)])
def test_shuffle_matches_splitmix_fisher_yates(n, seed, epoch):
    assert L.shuffle_order(n, seed, epoch) == _splitmix_order(n, seed, epoch)
    assert sorted(L.shuffle_order(n, seed, epoch)) == list(range(n))


PACK_GOLDENS = [
    (1, [[10, 11, 12], [20, 21]], ("concat_eos", 4, True), [([10, 11, 12, 1], [1, 1, 1, 1], None), ([20, 21, 0, 0], [1, 1, 0, 0], None)]),
    (1, [[10, 11, 12], [20, 21]], ("concat_eos", 4, False), [([10, 11, 12, 20], [1, 1, 1, 1], None), ([21, 0, 0, 0], [1, 0, 0, 0], None)]),
    (9, [[1, 2, 3, 4, 5, 6, 7]], ("concat_eos", 3, True), [([1, 2, 3], [1, 1, 1], None), ([4, 5, 6], [1, 1, 1], None), ([7, 0, 0], [1, 0, 0], None)]),
    (9, [[10, 11], [20]], ("document_mask", 4, True), [([10, 11, 9, 20], [1, 1, 1, 1], [0, 0, 0, 1])]),
    # the last partial sequence of a document-mask packing is padded (mask 0, document id 0)
    (9, [[10], [20, 21]], ("document_mask", 5, True), [([10, 9, 20, 21, 0], [1, 1, 1, 1, 0], [0, 0, 1, 1, 0])]),
]


@pytest.mark.parametrize("eos,docs,cfg,expected", PACK_GOLDENS)
def test_pack_goldens(eos, docs, cfg, expected):
    p = L.Packing("g", cfg[1], cfg[0], cfg[2], 0)
    got = L.pack(docs, p, eos)
    assert [(s.tokens, s.mask, s.document_ids) for s in got] == expected


def test_pack_single_document_golden():
    """One document per sequence: truncated to the length, documents shorter than
    ``drop_short_below`` dropped, the rest padded; no document ids (single_document.json of the
    reference's loader goldens)."""
    p = L.Packing("golden-single-document", 4, "single_document", False, 0, drop_short_below=2)
    got = L.pack([[1, 2], [3], [4, 5, 6, 7, 8]], p, 1)
    assert [(s.tokens, s.mask, s.document_ids) for s in got] == \
        [([1, 2, 0, 0], [1, 1, 0, 0], None), ([4, 5, 6, 7], [1, 1, 1, 1], None)]


def test_pack_single_and_errors():
    p = L.Packing("s", 4, "single_document", True, 7, drop_short_below=2)
    got = L.pack([[1], [1, 2, 3, 4, 5], [8, 9]], p, 0)
    assert [(s.tokens, s.mask) for s in got] == [([1, 2, 3, 4], [1, 1, 1, 1]), ([8, 9, 7, 7], [1, 1, 0, 0])]
    with pytest.raises(native.NativeError) as e:
        L.pack([[1]], p, 0)
    assert e.value.kind == "DroppedShort"
    with pytest.raises(native.NativeError) as e:
        L.pack([], p, 0)
    assert e.value.kind == "Empty"
    with pytest.raises(native.NativeError) as e:
        L.Packing("x", 4, "zigzag")
    assert e.value.kind == "UnknownStrategy"
    with pytest.raises(native.NativeError) as e:
        L.pack([[1]], L.Packing("x", 0), 0)
    assert e.value.kind == "BadSequenceLength"


def test_packing_and_state_json_are_sorted_and_compact():
    p = L.Packing("p", 8, "document_mask", False, 3)
    text = p.to_json()
    assert text == json.dumps(json.loads(text), sort_keys=True, separators=(",", ":"))
    assert "drop_short_below" not in text and json.loads(text)["schema_id"] == "prometheus.packing"
    assert L.Packing.from_json(text).strategy == "document_mask"
    st = L.LoaderState()
    st.shuffle_seed = 2**64 - 1
    st.data_mix_hash = "ab"
    t = st.to_json()
    assert t == json.dumps(json.loads(t), sort_keys=True, separators=(",", ":"))
    assert json.loads(t)["packing_remainder_hash"] == \
        "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert L.LoaderState.from_json(t) == st
    gold = json.loads((GOLD / "loader_state.default.json").read_text())
    assert L.LoaderState.from_json(json.dumps(gold)).shard_offset == gold["shard_offset"]


def _seqs(n, length=3):
    return [L.PackedSequence([i] * length, [1] * length) for i in range(n)]


def test_loader_cursor_accounting_and_resume():
    n, seed = 7, 11
    p = L.Packing("p", 3)
    ld = L.Loader(_seqs(n), p, seed, "mix")
    seen = []
    for step in range(5):
        b = ld.next_batch(3)
        seen += [t[0] for t in b.tokens]
        assert b.state.step == step + 1 and b.state.consumed_token_count == 9 * (step + 1)
    order = _splitmix_order(n, seed, 0) + _splitmix_order(n, seed, 1) + _splitmix_order(n, seed, 2)
    assert seen == order[:15]
    st = ld.state()
    assert (st.epoch, st.shard_offset, st.shard_index) == (2, 1, 0)
    # resume from a saved cursor reproduces the same next batch
    ld2 = L.Loader(_seqs(n), p, seed, "mix")
    ld2.next_batch(3)
    saved = L.LoaderState.from_json(ld2.state().to_json())
    a = ld2.next_batch(4)
    b = L.reconstruct(_seqs(n), p, saved, 4)
    assert a.tokens == b.tokens and a.state == b.state
    toks, mask = L.Loader.from_state(_seqs(n), p, saved).next_batch_arrays(4)
    assert toks.tolist() == a.tokens and mask.shape == (4, 3)
    with pytest.raises(native.NativeError) as e:
        L.Loader([], p, 0, "").next_batch(1)
    assert e.value.kind == "Exhausted"


# ------------------------------------------------------------------ checkpoints
def test_sha256_nist_vectors():
    assert C.sha256_hex(b"") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert C.sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    assert C.sha256_hex(b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq") == \
        "248d6a61d20638b8e5c026930c3e6039a33ce45964ff2167f6ecedd419db06c1"
    assert C.sha256_hex(b"a" * 1_000_000) == "cdc76e5c9914fb9281a1c7e284d73e67f1809a48a497200e046d39ccc7112cd0"


def _ckpt(cid="c1", payload=b"\x01\x02\x03\x04", parent=None):
    m = C.Manifest()
    m.checkpoint_id = cid
    m.parent_checkpoint_id = parent
    m.step = 10
    m.rung = 0
    m.model_config_hash = "a" * 64
    m.data_mix_hash = "b" * 64
    m.tokenizer_id = "tok"
    m.created_at = "2026-01-01T00:00:00Z"
    m.weights = [C.WeightMeta("embed", 0, [2, 2], "fp32")]
    m.optimizer = [C.OptimizerMeta("embed.m", 0, "adamw")]
    m.rng = [C.RngState("dropout", 0, "c" * 64)]
    m.loader_state_json = json.dumps({"epoch": 1})
    return C.Checkpoint(m, [C.ShardBlob("embed", 0, payload)], [C.ShardBlob("embed.m", 0, payload + b"x")])


def test_manifest_json_layout_and_golden_roundtrip():
    text = _ckpt().manifest.to_json()
    d = json.loads(text)
    assert text == json.dumps(d, sort_keys=True, separators=(",", ":"))
    assert d["parent_checkpoint_id"] is None and "precision" not in d and "git_commit" not in d
    assert "mesh_axes" not in d["weights"][0] and d["schema_version"] == 1
    gold = (GOLD / "checkpoint.default.json").read_text()
    m = C.Manifest.from_json(gold)
    assert json.loads(m.to_json()) == json.loads(gold)
    with pytest.raises(native.NativeError) as e:
        C.Manifest.from_json(gold.replace("prometheus.checkpoint", "other"))
    assert e.value.kind == "Schema"


def test_dir_store_layout_and_restore(tmp_path):
    cp = C.Checkpointer(C.DirStore(str(tmp_path / "s")))
    assert cp.save_persistent(_ckpt()) == "c1"
    names = sorted(p.name for p in (tmp_path / "s").iterdir())
    assert names == sorted(["c1", C.sha256_hex(b"\x01\x02\x03\x04"), C.sha256_hex(b"\x01\x02\x03\x04x")])
    back = cp.restore("c1")
    assert back.weights[0].bytes == b"\x01\x02\x03\x04"
    assert back.manifest.weights[0].content_hash == C.sha256_hex(b"\x01\x02\x03\x04")
    with pytest.raises(native.NativeError) as e:
        cp.restore("nope")
    assert e.value.kind == "NotFound"
    with pytest.raises(native.NativeError):
        C.DirStore(str(tmp_path / "s")).put("../escape", b"x")
    # a flipped byte on disk is caught by the per-shard hash
    shard = tmp_path / "s" / C.sha256_hex(b"\x01\x02\x03\x04")
    shard.write_bytes(b"\xfe\x02\x03\x04")
    with pytest.raises(native.NativeError) as e:
        cp.restore("c1")
    assert e.value.kind == "HashMismatch"


def test_prepare_rejects_wrong_hash_and_missing_shard():
    cp = C.Checkpointer(C.MemoryStore())
    c = _ckpt()
    m = c.manifest
    w = m.weights
    w[0].content_hash = "0" * 64
    m.weights = w
    c.manifest = m
    with pytest.raises(native.NativeError) as e:
        cp.save_in_memory(c)
    assert e.value.kind == "HashMismatch"
    c2 = _ckpt()
    c2.weights = []
    with pytest.raises(native.NativeError) as e:
        cp.save_persistent(c2)
    assert e.value.kind == "MissingShard"


def test_in_memory_replicas():
    cp = C.Checkpointer(C.MemoryStore())
    with pytest.raises(native.NativeError):
        cp.restore_latest_memory()
    cp.save_in_memory(_ckpt())
    assert cp.replica_len(0) == cp.replica_len(1) == 9
    assert cp.restore_latest_memory().manifest.checkpoint_id == "c1"
    cp.drop_replica(1)
    with pytest.raises(native.NativeError) as e:
        cp.replica_len(1)
    assert e.value.kind == "ReplicaLost"


def test_async_save_returns_before_store_finishes_and_reports_errors():
    inner = C.MemoryStore()
    slow = C.FaultyStore(inner)
    slow.block()
    cp = C.Checkpointer(slow)
    t0 = time.time()
    pending = cp.save_persistent_async(_ckpt())
    assert time.time() - t0 < 1.0 and not pending.is_finished()
    with pytest.raises(native.NativeError) as e:
        cp.save_persistent_async(_ckpt("c2"))
    assert e.value.kind == "SaveInFlight"
    threading.Timer(0.1, slow.release).start()
    pending.wait()
    assert pending.is_finished() and cp.restore("c1").optimizer[0].bytes == b"\x01\x02\x03\x04x"
    # an injected store failure surfaces from wait(), and does not wedge later saves
    bad = C.FaultyStore(C.MemoryStore())
    bad.fail_on_put(2)
    cp2 = C.Checkpointer(bad)
    p2 = cp2.save_persistent_async(_ckpt())
    with pytest.raises(native.NativeError):
        p2.wait()
    del p2
    p3 = cp2.save_persistent_async(_ckpt("c3"))
    p3.wait()
    assert cp2.restore("c3").manifest.checkpoint_id == "c3"


def test_cross_rack_placement_and_faults():
    racks = ["r0", "r1", "r2", "r3"]
    assert C.plan_cross_rack(racks, "r3") == ("r0", "r1")
    with pytest.raises(native.NativeError):
        C.plan_cross_rack(["a", "b"], "a")
    cp = C.Checkpointer(C.MemoryStore())
    assert cp.save_cross_rack(_ckpt(), "r1", racks) == ("r2", "r3")
    assert cp.cross_rack_destinations("r1") == ("r2", "r3")
    cp.lose_rack("r2")
    assert cp.restore_from_rack("r3").manifest.checkpoint_id == "c1"
    cp.corrupt_rack("r3")
    with pytest.raises(native.NativeError) as e:
        cp.restore_from_rack("r3")
    assert e.value.kind == "HashMismatch"
    with pytest.raises(native.NativeError):
        cp.save_cross_rack(_ckpt(), "r0", racks[:3] + ["r3"]) if False else cp.lose_rack("r9")


def test_host_ram_offload():
    h = C.HostRamOffload()
    h.put("layers.0.m", b"123")
    assert h.get("layers.0.m") == b"123" and len(h) == 1
    h.remove("layers.0.m")
    with pytest.raises(native.NativeError):
        h.get("layers.0.m")
