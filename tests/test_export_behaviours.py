"""Behaviour list of the weight export for the serving engine (``prometheus_b200.export``;
reference tests/test_sglang_export.py and sglang-fork/sglang_fork/export.py): flattening a
parameter tree, the three storage types (float32 pass-through, per-tensor 8-bit code, packed
4-bit e2m1 with one scale per 16 values), content hashes of little-endian bytes, the files
written, read-back parity and the contract record."""
import hashlib
import json

import numpy as np
import pytest
import torch

from prometheus_b200 import contracts, export as E

CREATED = "2026-09-16T12:00:00Z"
SHA = "2c9a93d84ad4df28371eab9ca3e915b257ae530b5d77e66a548628892464c228"
FP8_ONES_CONTENT = "af9613760f72635fbdb44a5a0a63c39f12af30f950a6ee5c971be188e89c4051"
FP8_ONES_SCALE = "4abeb7e04407af6d4256f29b91c71479bd701e60ee7468c778f55b1df0247dc7"
BF16_ONES_CONTENT = "b638277a8690e175a9137feff1e43c067f9faf4e2f600caf468fb05b0403b717"


def sha_le(a):
    return hashlib.sha256(np.ascontiguousarray(a).astype(a.dtype.newbyteorder("<")).tobytes()).hexdigest()


def tree(seed=0, cols=8):
    rng = np.random.default_rng(seed)
    return {"w": rng.standard_normal((4, cols)).astype(np.float32),
            "blocks": [{"a": rng.standard_normal((3,)).astype(np.float32)}, {"a": rng.standard_normal((2, 2)).astype(np.float32)}]}


def export(params, dtype, out, **kw):
    base = dict(export_id="exp-1", source_checkpoint_id="ckpt-1", tokenizer_id="tok-1", dtype=dtype, created_at=CREATED, out_dir=str(out))
    base.update(kw)
    return E.export_weights(params, **base)


# ------------------------------------------------------------------------------ constants / flatten
def test_constants():
    assert (E.SCHEMA_ID, E.SCHEMA_VERSION, E.TARGET) == ("prometheus.weight_export", 1, "sglang")
    assert E.DTYPES == ("bf16", "fp8", "nvfp4") and issubclass(E.ExportError, ValueError)


def test_flatten_uses_dotted_names_indices_and_sorted_order():
    flat = E.flatten_params({"z": np.zeros(1), "a": {"c": np.ones(2), "b": [np.zeros(3), (np.ones(1),)]}})
    assert list(flat) == ["a.b.0", "a.b.1.0", "a.c", "z"]
    assert list(E.flatten_params({"k": (np.zeros(1), np.ones(1))})) == list(E.flatten_params({"k": [np.zeros(1), np.ones(1)]}))
    assert list(E.flatten_params({"a": {"b": {"c": np.zeros(1)}}, "A": np.zeros(1)})) == ["A", "a.b.c"]
    assert E.flatten_params({}) == {}
    t = E.flatten_params({"t": torch.ones(2, 2, dtype=torch.bfloat16)})["t"]
    assert isinstance(t, np.ndarray) and t.dtype == np.float32 and t.tolist() == [[1.0, 1.0], [1.0, 1.0]]
    for bad in ({"a": 1.0}, {"a": "text"}, {"a": {"b": None}}, [np.zeros(1)], {"a": [np.zeros(1), 3]}):
        with pytest.raises(E.ExportError):
            E.flatten_params(bad)


# ------------------------------------------------------------------------------ storage types
def test_bf16_storage_is_a_float32_copy():
    x = tree()["w"]
    q, s = E.quantize(x, "bf16")
    assert s is None and q.dtype == np.float32 and np.array_equal(q, x) and q is not x
    assert np.array_equal(E.dequantize(q, None, "bf16"), x)
    assert sha_le(E.quantize(np.ones((4, 8), np.float32), "bf16")[0]) == BF16_ONES_CONTENT
    with pytest.raises(E.ExportError):
        E.dequantize(q, np.float32(1.0), "bf16")


def test_fp8_storage_is_one_scale_per_tensor_and_byte_codes():
    x = tree(4)["w"]
    q, s = E.quantize(x, "fp8")
    assert q.dtype == np.uint8 and q.shape == x.shape and s.shape == () and s.dtype == np.float32
    assert float(s) == pytest.approx(float(np.max(np.abs(x))) / 448.0, rel=1e-6)
    back = E.dequantize(q, s, "fp8")
    assert np.max(np.abs(back - x)) <= float(s) * (448.0 / 127.0) / 2 + 1e-6           # half a code step
    ones, so = E.quantize(np.ones((4, 8), np.float32), "fp8")
    assert sha_le(ones) == FP8_ONES_CONTENT and sha_le(so) == FP8_ONES_SCALE
    np.testing.assert_allclose(E.dequantize(ones, so, "fp8"), 1.0, rtol=1e-6)
    assert np.array_equal(E.dequantize(q, 2 * s, "fp8"), 2 * back)                      # linear in the scale
    neg, sn = E.quantize(-x, "fp8")
    np.testing.assert_allclose(E.dequantize(neg, sn, "fp8"), -back, atol=float(s) * 448.0 / 127.0)
    with pytest.raises(E.ExportError):
        E.dequantize(q, None, "fp8")


def test_nvfp4_storage_packs_two_values_per_byte_with_block_scales():
    x = tree(5)["w"]                                                                     # (4, 8): padded to one block of 16
    q, s = E.quantize(x, "nvfp4")
    assert q.dtype == np.uint8 and q.shape == (4, 8) and s.shape == (4, 1)
    np.testing.assert_allclose(s, np.max(np.abs(x), axis=-1, keepdims=True) / 6.0, rtol=1e-6)
    back = E.dequantize(q, s, "nvfp4")
    assert back.shape == (4, 16) and np.all(back[:, 8:] == 0)
    levels = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float32)
    want = np.sign(x) * levels[np.argmin(np.abs(np.abs(x / s)[..., None] - levels), -1)] * s
    np.testing.assert_allclose(back[:, :8], want, rtol=1e-6, atol=1e-7)
    wide = np.random.default_rng(1).standard_normal((2, 40)).astype(np.float32)        # three blocks, last one ragged
    qw, sw = E.quantize(wide, "nvfp4")
    assert qw.shape == (2, 24) and sw.shape == (2, 3) and E.dequantize(qw, sw, "nvfp4").shape == (2, 48)
    for bad_q, bad_s in ((qw[:, :23], sw), (qw, sw[:, :2])):
        with pytest.raises(E.ExportError):
            E.dequantize(bad_q, bad_s, "nvfp4")


@pytest.mark.parametrize("dtype", E.DTYPES)
def test_zeros_round_trip_and_argument_errors(dtype):
    x = np.zeros((4, 8), np.float32)
    q, s = E.quantize(x, dtype)
    assert np.all(E.dequantize(q, s, dtype)[..., :8] == 0)
    for bad in (np.array([1.0, np.nan]), np.array([np.inf]), np.array([-np.inf, 0.0])):
        with pytest.raises(E.ExportError):
            E.quantize(bad, dtype)
    with pytest.raises(E.ExportError):
        E.quantize(x, "int3")
    with pytest.raises(E.ExportError):
        E.dequantize(q, s, "int3")


# ------------------------------------------------------------------------------ export / parity
@pytest.mark.parametrize("dtype", E.DTYPES)
def test_export_writes_files_and_hashes_their_bytes(tmp_path, dtype):
    params = tree(7)
    out = export(params, dtype, tmp_path)
    flat = E.flatten_params(params)
    assert (out.target, out.dtype, out.shard_count, out.created_at) == ("sglang", dtype, 3, CREATED)
    assert [s.name for s in out.shards] == list(flat) == ["blocks.0.a", "blocks.1.a", "w"]
    for s in out.shards:
        q = np.load(tmp_path / s.path, allow_pickle=False)
        want_q, want_s = E.quantize(flat[s.name], dtype)
        assert np.array_equal(q, want_q) and s.content_hash == sha_le(q) and s.dtype == dtype
        assert (s.scale_hash is None) == (dtype == "bf16")
        if s.scale_hash is not None:
            sc = np.load(tmp_path / f"{s.name}.scale.npy", allow_pickle=False)
            assert s.scale_hash == sha_le(sc) and np.array_equal(sc, want_s)
    side = json.loads((tmp_path / E.SIDECAR_NAME).read_text())
    assert side["format"] == E.SIDECAR_FORMAT and [e["name"] for e in side["shards"]] == list(flat) and side["dtype"] == dtype
    err = E.parity_max_abs_err(params, out, str(tmp_path))
    if dtype == "bf16":
        assert err == 0.0
    else:
        assert 0.0 < err < (0.05 if dtype == "fp8" else 0.8)                             # shapes are cropped back, not padded


def test_export_argument_errors(tmp_path):
    params = tree()
    for kw in (dict(dtype="fp16"), dict(export_id=""), dict(source_checkpoint_id=""), dict(tokenizer_id=""),
               dict(routing_table_hash="abc"), dict(routing_table_hash=SHA.upper()), dict(routing_table_hash=SHA + "0")):
        with pytest.raises(E.ExportError):
            export(params, kw.pop("dtype", "bf16"), tmp_path, **kw)
    with pytest.raises(E.ExportError):
        export({}, "bf16", tmp_path)
    ok = export(params, "bf16", tmp_path / "r", routing_table_hash=SHA)
    assert ok.routing_table_hash == SHA
    with pytest.raises(E.ExportError):
        E.parity_max_abs_err({"other": np.zeros(1, np.float32)}, ok, str(tmp_path / "r"))


# ------------------------------------------------------------------------------ contract
def test_contract_record(tmp_path):
    out = export(tree(), "fp8", tmp_path, routing_table_hash=SHA)
    rec = E.to_contract(out)
    contracts.validate_named(E.SCHEMA_ID, rec)
    assert rec["target"] == "sglang" and rec["routing_table_hash"] == SHA and rec["created_at"] == CREATED
    assert [s["name"] for s in rec["shards"]] == [s.name for s in out.shards] and all("scale_hash" in s for s in rec["shards"])
    plain = E.to_contract(export(tree(), "bf16", tmp_path / "b"))
    assert "routing_table_hash" not in plain and all("scale_hash" not in s for s in plain["shards"])    # absent, not null
    empty = E.WeightExport("e", "c", "t", "sglang", "bf16", 0, (), None, CREATED)
    with pytest.raises(E.ExportError):
        E.to_contract(empty)
