"""Checkpoint store behaviour list (names follow the reference's ckpt/tests/{persistent,dir_store,
memory_store,in_memory,async_save,offload,cross_rack,fault,properties}.rs), against the C++ module.
Every fault is a flipped byte or a blocked put on the host."""
import json
import random
import threading

import pytest

from prometheus_b200 import native

C = native.ckpt


def kind_of(fn, *a, **k):
    with pytest.raises(native.NativeError) as e:
        fn(*a, **k)
    return e.value.kind


def ckpt(cid="c1", shards=(("embed", 0, b"\x01\x02\x03\x04", [2, 2], "fp32"),), opt=(("embed.m", 0, b"mm"),),
         parent=None, created="2026-01-01T00:00:00Z"):
    m = C.Manifest()
    m.checkpoint_id, m.parent_checkpoint_id, m.step, m.rung = cid, parent, 3, 1
    m.model_config_hash, m.data_mix_hash, m.tokenizer_id, m.created_at = "a" * 64, "b" * 64, "tok", created
    m.weights = [C.WeightMeta(n, r, shape, dt) for n, r, _b, shape, dt in shards]
    m.optimizer = [C.OptimizerMeta(n, r, "adamw") for n, r, _b in opt]
    m.rng = [C.RngState("dropout", 0, "c" * 64), C.RngState("data", 1, "d" * 64)]
    m.loader_state_json = json.dumps({"epoch": 2})
    return C.Checkpoint(m, [C.ShardBlob(n, r, b) for n, r, b, _s, _d in shards],
                        [C.ShardBlob(n, r, b) for n, r, b in opt])


def same(a, b):
    return ([(w.name, w.shard_rank, bytes(w.bytes)) for w in a.weights] ==
            [(w.name, w.shard_rank, bytes(w.bytes)) for w in b.weights] and
            [(w.name, w.shard_rank, bytes(w.bytes)) for w in a.optimizer] ==
            [(w.name, w.shard_rank, bytes(w.bytes)) for w in b.optimizer])


# ----------------------------------------------------------------- persistent
def test_memory_replicas_is_two_and_cross_rack_copies_is_two():
    assert C.MEMORY_REPLICAS == 2 and C.CROSS_RACK_COPIES == 2


def test_save_persistent_restore_bitwise_equal_with_hashes_and_created_at():
    cp = C.Checkpointer(C.MemoryStore())
    src = ckpt()
    cp.save_persistent(src)
    back = cp.restore("c1")
    assert same(src, back)
    assert back.manifest.weights[0].content_hash == C.sha256_hex(b"\x01\x02\x03\x04")
    assert back.manifest.optimizer[0].content_hash == C.sha256_hex(b"mm")
    assert back.manifest.created_at == "2026-01-01T00:00:00Z"            # not replaced by the wall clock
    assert kind_of(cp.restore, "other") == "NotFound"


def test_two_persistent_ids_restore_independently_and_parent_rng_kept():
    cp = C.Checkpointer(C.MemoryStore())
    cp.save_persistent(ckpt("a"))
    cp.save_persistent(ckpt("b", shards=(("embed", 0, b"\x09\x09\x09\x09", [4], "int8"),), parent="a"))
    a, b = cp.restore("a"), cp.restore("b")
    assert bytes(a.weights[0].bytes) == b"\x01\x02\x03\x04" and bytes(b.weights[0].bytes) == b"\x09" * 4
    assert b.manifest.parent_checkpoint_id == "a" and a.manifest.parent_checkpoint_id is None
    assert [(r.scope, r.rank, r.state_hash) for r in b.manifest.rng] == [("dropout", 0, "c" * 64), ("data", 1, "d" * 64)]


@pytest.mark.parametrize("dtype,shape,nbytes", [("fp32", [2, 3], 24), ("bf16", [5], 10), ("fp8", [7, 1], 7), ("fp16", [3], 6), ("nvfp4", [8], 4),
                                                ("int32", [], 4), ("int8", [0], 0)])
def test_shape_and_dtype_preserved_for_every_dtype(dtype, shape, nbytes):
    cp = C.Checkpointer(C.MemoryStore())
    cp.save_persistent(ckpt(shards=(("w", 0, bytes(range(nbytes)), shape, dtype),)))
    w = cp.restore("c1").manifest.weights[0]
    assert (w.dtype, list(w.shape)) == (dtype, shape)


def test_multiple_shards_roundtrip_by_name_and_rank():
    shards = tuple((n, r, f"{n}{r}".encode() * 3, [3], "int8") for n in ("q", "k") for r in (0, 1, 2))
    cp = C.Checkpointer(C.MemoryStore())
    src = ckpt(shards=shards, opt=tuple((f"{n}.m", r, b"o" + bytes([r])) for n, r, *_ in shards))
    cp.save_persistent(src)
    assert same(src, cp.restore("c1"))


def test_empty_shard_bytes_hash_is_nist_empty():
    cp = C.Checkpointer(C.MemoryStore())
    cp.save_persistent(ckpt(shards=(("w", 0, b"", [0], "int8"),)))
    assert cp.restore("c1").manifest.weights[0].content_hash == \
        "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"


# ------------------------------------------------------------------ dir store
def test_dirstore_put_get_reopen_overwrite_and_missing(tmp_path):
    root = tmp_path / "deep" / "store"
    s = C.DirStore(str(root))                              # creates the missing directory
    assert root.is_dir() and not s.contains("k")
    s.put("k", b"one")
    s.put("k", b"two")
    s.put("empty", b"")
    again = C.DirStore(str(root))
    assert again.get("k") == b"two" and again.get("empty") == b"" and again.contains("k")
    assert kind_of(again.get, "missing") == "NotFound"


def test_dirstore_save_drop_reopen_restore(tmp_path):
    src = ckpt()
    C.Checkpointer(C.DirStore(str(tmp_path))).save_persistent(src)
    assert same(src, C.Checkpointer(C.DirStore(str(tmp_path))).restore("c1"))


# --------------------------------------------------------------- memory store
def test_memory_store_put_get_contains_vs_dict_random_keys():
    rng = random.Random(1)
    s, ref = C.MemoryStore(), {}
    for _ in range(200):
        k = f"k{rng.randrange(20)}"
        if rng.random() < 0.6:
            v = rng.randbytes(rng.randrange(0, 9))
            s.put(k, v)
            ref[k] = v
        elif k in ref:
            assert s.get(k) == ref[k]
        else:
            assert not s.contains(k) and kind_of(s.get, k) == "NotFound"


# ------------------------------------------------------------------ in memory
def test_in_memory_latest_two_equal_copies_and_index_errors():
    cp = C.Checkpointer(C.MemoryStore())
    assert kind_of(cp.restore_latest_memory) == "NotFound"
    cp.save_in_memory(ckpt("first"))
    second = ckpt("second", shards=(("embed", 0, b"\x05\x06\x07\x08\x09", [5], "int8"),))
    cp.save_in_memory(second)
    assert cp.restore_latest_memory().manifest.checkpoint_id == "second"
    assert cp.replica_len(0) == cp.replica_len(1) == second.payload_len() > 0
    with pytest.raises(native.NativeError):
        cp.replica_len(2)
    assert same(second, cp.restore_latest_memory())


def test_rejected_checkpoint_writes_nothing_anywhere():
    store = C.FaultyStore(C.MemoryStore())
    cp = C.Checkpointer(store)
    bad = ckpt()
    bad.weights = []
    assert kind_of(cp.save_in_memory, bad) == "MissingShard"
    assert kind_of(cp.save_persistent, bad) == "MissingShard"
    assert kind_of(cp.save_cross_rack, bad, "r0", ["r0", "r1", "r2"]) == "MissingShard"
    assert kind_of(cp.save_persistent_async, bad) == "MissingShard"       # and starts no write
    assert store.puts() == 0 and kind_of(cp.restore_latest_memory) == "NotFound"
    assert kind_of(cp.cross_rack_destinations, "r0") == "NotFound"
    no_opt = ckpt()
    no_opt.optimizer = []
    assert kind_of(cp.save_persistent, no_opt) == "MissingShard"


# ---------------------------------------------------------------------- async
def test_async_save_blocked_put_in_flight_wait_and_dropped_handle():
    store = C.FaultyStore(C.MemoryStore())
    store.block()
    cp = C.Checkpointer(store)
    pending = cp.save_persistent_async(ckpt())
    assert not pending.is_finished() and pending.checkpoint_id == "c1"
    puts = store.puts()
    assert kind_of(cp.save_persistent_async, ckpt("c2")) == "SaveInFlight" and store.puts() == puts
    threading.Timer(0.05, store.release).start()
    pending.wait()
    assert pending.is_finished() and same(ckpt(), cp.restore("c1"))
    # dropping the handle does not cancel the write
    store.block()
    p = cp.save_persistent_async(ckpt("c3"))
    del p
    store.release()
    for _ in range(200):
        try:
            cp.restore("c3")
            break
        except native.NativeError:
            threading.Event().wait(0.01)
    assert same(ckpt(), cp.restore("c3"))


# -------------------------------------------------------------------- offload
def test_host_ram_offload_vs_dict_random_names():
    rng = random.Random(2)
    h, ref = C.HostRamOffload(), {}
    assert kind_of(h.remove, "nope") == "NotFound"
    for _ in range(200):
        k = f"layers.{rng.randrange(10)}.m"
        op = rng.random()
        if op < 0.5:
            v = rng.randbytes(rng.randrange(0, 6))
            h.put(k, v)
            ref[k] = v
        elif op < 0.8:
            if k in ref:
                assert h.get(k) == ref[k]
            else:
                assert kind_of(h.get, k) == "NotFound"
        elif k in ref:
            h.remove(k)
            del ref[k]
    assert len(h) == len(ref)


# ----------------------------------------------------------------- cross rack
def test_plan_cross_rack_walk_order_and_rejections():
    racks = ["a", "b", "c", "d", "e"]
    assert C.plan_cross_rack(racks, "a") == ("b", "c")
    assert C.plan_cross_rack(racks, "d") == ("e", "a")                    # walks on from the source, wrapping
    assert C.plan_cross_rack(racks, "e") == ("a", "b")
    for fleet, src in (([], "a"), (["a", "b", "c"], "z"), (["a", "b"], "a"), (["a", "a", "b"], "a")):
        with pytest.raises(native.NativeError):
            C.plan_cross_rack(fleet, src)


def test_plan_cross_rack_on_generated_fleets():
    rng = random.Random(4)
    for _ in range(50):
        n = rng.randrange(3, 12)
        racks = [f"r{i}" for i in range(n)]
        i = rng.randrange(n)
        assert C.plan_cross_rack(racks, racks[i]) == (racks[(i + 1) % n], racks[(i + 2) % n])


def test_save_cross_rack_touches_neither_store_nor_memory_replicas():
    store = C.FaultyStore(C.MemoryStore())
    cp = C.Checkpointer(store)
    assert cp.save_cross_rack(ckpt(), "a", ["a", "b", "c", "d"]) == ("b", "c")
    assert store.puts() == 0 and kind_of(cp.restore_latest_memory) == "NotFound"
    assert same(ckpt(), cp.restore_from_rack("b")) and same(ckpt(), cp.restore_from_rack("c"))


def test_lose_and_corrupt_rack_affect_one_copy_only():
    cp = C.Checkpointer(C.MemoryStore())
    racks = ["a", "b", "c", "d"]
    cp.save_cross_rack(ckpt(), "a", racks)
    cp.corrupt_rack("b")
    assert kind_of(cp.restore_from_rack, "b") == "HashMismatch" and same(ckpt(), cp.restore_from_rack("c"))
    cp.lose_rack("b")
    assert kind_of(cp.restore_from_rack, "b") in ("NotFound", "RackLost")
    assert cp.cross_rack_destinations("a") == ("b", "c")                  # the plan survives the loss


def test_two_sources_occupied_destination_and_resave():
    cp = C.Checkpointer(C.MemoryStore())
    racks = ["a", "b", "c", "d", "e", "f"]
    cp.save_cross_rack(ckpt("from-a"), "a", racks)                         # -> b, c
    cp.save_cross_rack(ckpt("from-d"), "d", racks)                         # -> e, f
    assert cp.restore_from_rack("b").manifest.checkpoint_id == "from-a"
    assert cp.restore_from_rack("f").manifest.checkpoint_id == "from-d"
    # b holds a's copy: a save from f (-> a, b) finds b occupied and changes nothing
    assert kind_of(cp.save_cross_rack, ckpt("from-f"), "f", racks) in ("RackOccupied", "Rack", "Other")
    assert cp.restore_from_rack("b").manifest.checkpoint_id == "from-a"
    # saving a again replaces its own copies
    cp.save_cross_rack(ckpt("from-a-2"), "a", racks)
    assert cp.restore_from_rack("c").manifest.checkpoint_id == "from-a-2"
    assert cp.restore_from_rack("e").manifest.checkpoint_id == "from-d"


# ---------------------------------------------------------------------- faults
def test_flipped_weight_or_optimizer_blob_is_hash_mismatch():
    for which in ("w", "o"):
        store = C.MemoryStore()
        cp = C.Checkpointer(store)
        cp.save_persistent(ckpt())
        store.corrupt(C.sha256_hex(b"\x01\x02\x03\x04" if which == "w" else b"mm"))
        assert kind_of(cp.restore, "c1") == "HashMismatch"


def test_manifest_blob_removed_from_store_is_missing_shard_or_not_found(tmp_path):
    cp = C.Checkpointer(C.DirStore(str(tmp_path)))
    cp.save_persistent(ckpt())
    (tmp_path / C.sha256_hex(b"mm")).unlink()
    assert kind_of(cp.restore, "c1") in ("MissingShard", "NotFound")


def test_save_restore_vs_python_model_random_checkpoints():
    rng = random.Random(9)
    cp = C.Checkpointer(C.MemoryStore())
    for i in range(20):
        shards = tuple((f"w{j}", r, rng.randbytes(rng.randrange(0, 40)), [1], "int8")
                       for j in range(rng.randrange(1, 4)) for r in range(rng.randrange(1, 3)))
        src = ckpt(f"id{i}", shards=shards, opt=tuple((f"{n}.v", r, rng.randbytes(3)) for n, r, *_ in shards))
        (cp.save_persistent if i % 2 else cp.save_in_memory)(src)
        back = cp.restore(f"id{i}") if i % 2 else cp.restore_latest_memory()
        assert same(src, back)
        assert [w.content_hash for w in back.manifest.weights] == [C.sha256_hex(s[2]) for s in shards]
