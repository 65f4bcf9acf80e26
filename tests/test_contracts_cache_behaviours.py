"""Behaviour lists of the contract registry (``prometheus_b200.contracts``; reference
tests/test_contracts.py, contracts/__init__.py) and of the content-addressed compile cache
(``prometheus_b200.compile_cache``; reference tests/test_compile_cache.py,
kernels/compile_cache.py): every schema with its golden, the ways a payload is refused,
versions and migration; cache keys, the on-disk record, torn and foreign files as misses."""
import copy
import hashlib
import json
import struct

import pytest

from prometheus_b200 import compile_cache as CC
from prometheus_b200 import contracts as C

SCHEMAS = [s.value for s in C.SchemaId]


# ------------------------------------------------------------------------------ contracts
def test_sixteen_schemas():
    assert len(SCHEMAS) == 16 and all(s.startswith("prometheus.") for s in SCHEMAS) and len(set(SCHEMAS)) == 16


@pytest.mark.parametrize("sid", SCHEMAS)
def test_schema_and_golden_round_trip(sid):
    path = C.schema_path(sid, 1)
    assert path.is_file() and json.loads(path.read_text()) == C.load_schema(sid, 1)
    g = C.load_golden(sid, 1)
    assert g["schema_id"] == sid and g["schema_version"] == 1
    C.validate(g)
    C.validate(json.loads(json.dumps(g)))                                               # survives a JSON round trip
    assert C.current_version(sid) == 1 and tuple(C.supported_versions(sid)) == (1,)
    same = C.migrate(g, 1)
    assert same == g and same is not g                                                   # version 1 -> 1: equal, but a copy
    same["schema_id"] = "changed"
    assert g["schema_id"] == sid
    with pytest.raises(C.MigrationError):
        C.migrate(g, 99)


@pytest.mark.parametrize("sid", SCHEMAS)
def test_payloads_are_refused_for_the_usual_reasons(sid):
    g = C.load_golden(sid, 1)
    schema = C.load_schema(sid, 1)
    wrong_id = dict(g, schema_id="prometheus.not_a_schema")
    with pytest.raises((C.ValidationError, C.UnknownSchemaError)):
        C.validate(wrong_id)
    other = next(s for s in SCHEMAS if s != sid)
    with pytest.raises(C.ValidationError):
        C.validate(dict(g, schema_id=other))                                             # another schema's id: its required fields are missing or extra
    for field in schema["required"]:
        if field in ("schema_id", "schema_version"):
            continue
        with pytest.raises(C.ValidationError):
            C.validate({k: v for k, v in g.items() if k != field})
    with pytest.raises(C.ValidationError):
        C.validate(dict(g, surprise_field=1))
    for field in schema["required"]:
        if isinstance(g.get(field), str) and field != "schema_id" and schema["properties"][field].get("minLength"):
            with pytest.raises(C.ValidationError):
                C.validate(dict(g, **{field: ""}))
    with pytest.raises((C.ValidationError, C.UnknownSchemaError)):
        C.validate(dict(g, schema_version=2))


def test_formats_unknown_ids_and_versions():
    g = C.load_golden("prometheus.checkpoint", 1)
    sha_fields = [k for k, v in g.items() if isinstance(v, str) and len(v) == 64 and set(v) <= set("0123456789abcdef")]
    for k in sha_fields:
        for bad in (g[k].upper(), g[k][:-1], g[k] + "0", "g" * 64):
            with pytest.raises(C.ValidationError):
                C.validate(dict(g, **{k: bad}))
    for bad in ("yesterday", "2026-13-01T00:00:00Z", "2026-01-01T25:00:00Z", ""):
        with pytest.raises(C.ValidationError):
            C.validate(dict(g, created_at=bad))
    for payload in ({"schema_id": "prometheus.nope", "schema_version": 1}, {"schema_version": 1}, {}, {"schema_id": 7, "schema_version": 1}):
        with pytest.raises((C.UnknownSchemaError, C.ValidationError)):
            C.validate(payload)
    with pytest.raises(C.UnknownSchemaError):
        C.current_version("prometheus.nope")
    with pytest.raises((C.UnknownSchemaError, FileNotFoundError, ValueError)):
        C.schema_path("prometheus.checkpoint", 7)
    C.validate_named("prometheus.checkpoint", g)
    with pytest.raises(C.ValidationError):
        C.validate_named("prometheus.rollout", g)                                        # the named schema must be the payload's


def test_event_log_golden_chains_from_the_genesis_hash():
    g = C.load_golden("prometheus.event_log", 1)
    assert g["prev_hash"] == "0" * 64 or len(g["prev_hash"]) == 64
    m = copy.deepcopy(g)
    m["prev_hash"] = "0" * 63
    with pytest.raises(C.ValidationError):
        C.validate(m)


# ------------------------------------------------------------------------------ compile cache
def test_program_hash():
    assert CC.program_hash(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    for blob in (b"\x00", b"kernel source\n" * 100, bytes(range(256))):
        assert CC.program_hash(blob) == hashlib.sha256(blob).hexdigest()
    for bad in (b"", "text", None, 3, bytearray(b"x"), memoryview(b"x")):
        with pytest.raises(CC.CacheError):
            CC.program_hash(bad)
    assert issubclass(CC.CacheError, ValueError)


def test_store_lookup_and_the_record_on_disk(tmp_path):
    cache = CC.CompileCache(tmp_path / "cc")
    prog, art = b"__global__ void k() {}", bytes(range(200)) * 3
    assert cache.lookup(prog) is None
    key = cache.store(prog, art)
    assert key == hashlib.sha256(prog).hexdigest() != hashlib.sha256(art).hexdigest()    # keyed by the program, not the artifact
    assert cache.lookup(prog) == art
    blob = (tmp_path / "cc" / key).read_bytes()
    assert blob == b"CC01" + struct.pack(">Q", len(art)) + art + hashlib.sha256(art).digest()
    assert cache.store(prog, art) == key and [p.name for p in (tmp_path / "cc").iterdir()] == [key]     # idempotent: one file
    with pytest.raises(CC.CacheError):
        cache.store(prog, art + b"!")
    assert cache.lookup(prog) == art                                                     # the first artifact stays
    second = CC.CompileCache(tmp_path / "cc")                                            # another handle on the same directory
    assert second.lookup(prog) == art
    second.store(b"other program", b"other artifact")
    assert cache.lookup(b"other program") == b"other artifact"


def test_empty_inputs_write_nothing(tmp_path):
    cache = CC.CompileCache(tmp_path)
    for prog, art in ((b"p", b""), (b"", b"a"), (b"p", "text"), ("p", b"a")):
        with pytest.raises(CC.CacheError):
            cache.store(prog, art)
    with pytest.raises(CC.CacheError):
        cache.lookup(b"")
    assert list(tmp_path.iterdir()) == []


def test_foreign_partial_and_torn_files_are_misses(tmp_path):
    cache = CC.CompileCache(tmp_path)
    prog, art = b"program", b"artifact bytes " * 10
    key = CC.program_hash(prog)
    (tmp_path / "README").write_text("not a record")
    (tmp_path / f".{key}.deadbeef.partial").write_bytes(b"CC01 half written")
    assert cache.lookup(prog) is None
    full = b"CC01" + struct.pack(">Q", len(art)) + art + hashlib.sha256(art).digest()
    for torn in (full[:10], full[:-1], full[:-32], full + b"x", b"XX01" + full[4:], full[:12] + b"\x00" + full[13:]):
        (tmp_path / key).write_bytes(torn)
        assert cache.lookup(prog) is None                                                # never a short or corrupt hit
    (tmp_path / key).unlink()
    cache.store(prog, art)
    assert cache.lookup(prog) == art                                                     # partial siblings do not get in the way
    assert (tmp_path / f".{key}.deadbeef.partial").exists()


def test_get_or_compile(tmp_path):
    cache = CC.CompileCache(tmp_path)
    calls = []

    def compiler(program):
        calls.append(program)
        return b"built:" + program

    assert cache.get_or_compile(b"src", compiler) == (b"built:src", False)
    assert cache.get_or_compile(b"src", compiler) == (b"built:src", True) and calls == [b"src"]
    cache.store(b"pre", b"stored")
    assert cache.get_or_compile(b"pre", compiler) == (b"stored", True) and calls == [b"src"]

    def broken(program):
        raise RuntimeError("nvcc fell over")

    with pytest.raises(RuntimeError, match="fell over"):
        cache.get_or_compile(b"bad", broken)
    for empty in (lambda p: b"", lambda p: None, lambda p: "text"):
        with pytest.raises(CC.CacheError):
            cache.get_or_compile(b"bad", empty)
    assert cache.lookup(b"bad") is None


def test_cache_root(tmp_path):
    (tmp_path / "file").write_text("x")
    with pytest.raises(CC.CacheError):
        CC.CompileCache(tmp_path / "file")
    made = CC.CompileCache(tmp_path / "a" / "b" / "c")
    assert (tmp_path / "a" / "b" / "c").is_dir() and made.lookup(b"p") is None
