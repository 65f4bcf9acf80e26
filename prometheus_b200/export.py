"""Weight export for the serving stack: flatten the parameter tree, quantise per tensor,
write ``.npy`` shards plus a sidecar, and emit the ``prometheus.weight_export`` contract.

On-disk layout is the reference's (``sglang-fork/sglang_fork/__init__.py:340-390``):
``<name>.npy`` (+ ``<name>.scale.npy``) per dotted parameter name, ``shards.json``
(``{"format": "prometheus.c1.npy-shards.v1", ...}``, indent 2, sorted keys), content hash =
SHA-256 of the little-endian raw array bytes. Codecs keep the reference's definitions so
exported directories interoperate: ``bf16`` stores fp32 values, ``fp8`` is the per-tensor
affine 8-bit code (zero point 128, step 448/127), ``nvfp4`` is E2M1 nibbles with one fp32
scale per 16 values. Added: ``fp8_e4m3`` writes real E4M3 bytes with 128x128 block scales,
the format the FP8 training kernels use.
"""
from __future__ import annotations

import hashlib
import json
import re
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

import numpy as np

from . import contracts

SCHEMA_ID = "prometheus.weight_export"
SCHEMA_VERSION = 1
TARGET = "sglang"
DTYPE_BF16, DTYPE_FP8, DTYPE_NVFP4 = "bf16", "fp8", "nvfp4"
DTYPES = (DTYPE_BF16, DTYPE_FP8, DTYPE_NVFP4)
FP8_E4M3_MAX = np.float32(448.0)
FP8_CODE_ZERO = 128
FP8_CODE_STEP = np.float32(448.0 / 127.0)
NVFP4_BLOCK = 16
E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
SIDECAR_NAME = "shards.json"
SIDECAR_FORMAT = "prometheus.c1.npy-shards.v1"
_HEX64 = re.compile(r"^[0-9a-f]{64}$")


class ExportError(ValueError):
    """The tree, dtype or export directory is invalid."""


@dataclass(frozen=True)
class Shard:
    name: str
    dtype: str
    content_hash: str
    scale_hash: str | None = None
    path: str | None = None


@dataclass(frozen=True)
class WeightExport:
    export_id: str
    source_checkpoint_id: str
    tokenizer_id: str
    target: str
    dtype: str
    shard_count: int
    shards: tuple
    routing_table_hash: str | None
    created_at: str
    schema_id: str = SCHEMA_ID
    schema_version: int = SCHEMA_VERSION


def _np(x) -> np.ndarray:
    if hasattr(x, "detach"):
        x = x.detach().cpu().float().numpy()
    return np.asarray(x)


def _hash(arr) -> str:
    a = np.ascontiguousarray(np.asarray(arr))
    if a.dtype.byteorder == ">" or (a.dtype.byteorder == "=" and sys.byteorder != "little"):
        a = a.byteswap().view(a.dtype.newbyteorder("<"))
    return hashlib.sha256(a.tobytes()).hexdigest()


def flatten_params(params: Mapping[str, Any]) -> dict:
    """Dotted names -> arrays, sorted by name; non-array leaves are an error."""
    if not isinstance(params, Mapping):
        raise ExportError("params must be a mapping")
    out: dict[str, np.ndarray] = {}

    def walk(prefix, node):
        if isinstance(node, Mapping):
            for k, v in node.items():
                walk(f"{prefix}.{k}" if prefix else str(k), v)
        elif isinstance(node, (list, tuple)):
            for i, v in enumerate(node):
                walk(f"{prefix}.{i}" if prefix else str(i), v)
        elif hasattr(node, "shape") and hasattr(node, "dtype") and not isinstance(node, (str, bytes)):
            if not prefix:
                raise ExportError("unnamed array leaf")
            out[prefix] = _np(node)
        else:
            raise ExportError(f"non-array leaf at {prefix or '<root>'}: {type(node)!r}")

    walk("", params)
    return {k: out[k] for k in sorted(out)}


def _q_fp8(x):
    amax = np.max(np.abs(x)) if x.size else np.float32(0)
    scale = np.asarray(1.0 if float(amax) == 0.0 else amax / FP8_E4M3_MAX, dtype=np.float32)
    code = np.rint((x / scale) / FP8_CODE_STEP) + FP8_CODE_ZERO
    return np.clip(code, 0, 255).astype(np.uint8), scale


def _dq_fp8(q, scale):
    return ((np.asarray(q).astype(np.float32) - FP8_CODE_ZERO) * FP8_CODE_STEP
            * np.asarray(scale, dtype=np.float32)).astype(np.float32)


def _q_nvfp4(x):
    if x.ndim < 1:
        x = x.reshape(1)
    n = x.shape[-1]
    nb = -(-n // NVFP4_BLOCK)
    xp = np.pad(x, [(0, 0)] * (x.ndim - 1) + [(0, nb * NVFP4_BLOCK - n)])
    blk = xp.reshape(*x.shape[:-1], nb, NVFP4_BLOCK)
    amax = np.max(np.abs(blk), axis=-1)
    scale = np.where(amax == 0, np.float32(1.0), amax / np.float32(6.0)).astype(np.float32)
    scaled = blk / scale[..., None]
    idx = np.argmin(np.abs(np.abs(scaled)[..., None] - E2M1_LEVELS), axis=-1).astype(np.uint8)
    nib = (idx | ((scaled < 0).astype(np.uint8) << 3)).reshape(*x.shape[:-1], nb * NVFP4_BLOCK)
    packed = (nib[..., 0::2] & 0x0F) | ((nib[..., 1::2] & 0x0F) << 4)
    return packed.astype(np.uint8), scale


def _dq_nvfp4(q, scale):
    q = np.asarray(q, dtype=np.uint8)
    nib = np.stack((q & 0x0F, (q >> 4) & 0x0F), axis=-1).reshape(*q.shape[:-1], q.shape[-1] * 2)
    val = E2M1_LEVELS[nib & 7] * np.where((nib >> 3) & 1, np.float32(-1), np.float32(1))
    n = val.shape[-1]
    if n % NVFP4_BLOCK:
        raise ExportError("nvfp4 packed last axis is not a multiple of 8 bytes")
    s = np.asarray(scale, dtype=np.float32)
    if s.shape != (*val.shape[:-1], n // NVFP4_BLOCK):
        raise ExportError(f"nvfp4 scale shape {s.shape} does not match the payload")
    return (val.reshape(*val.shape[:-1], n // NVFP4_BLOCK, NVFP4_BLOCK) * s[..., None]) \
        .reshape(*val.shape[:-1], n).astype(np.float32)


def quantize(array, dtype: str):
    """(payload, scale or None) for one tensor."""
    if dtype not in DTYPES:
        raise ExportError(f"unsupported dtype {dtype!r}")
    x = _np(array).astype(np.float32)
    if x.size and not np.all(np.isfinite(x)):
        raise ExportError("quantize requires finite values")
    if dtype == DTYPE_BF16:
        return x.copy(), None
    return _q_fp8(x) if dtype == DTYPE_FP8 else _q_nvfp4(x)


def dequantize(quantized, scale, dtype: str) -> np.ndarray:
    if dtype not in DTYPES:
        raise ExportError(f"unsupported dtype {dtype!r}")
    if dtype == DTYPE_BF16:
        if scale is not None:
            raise ExportError("bf16 scale must be None")
        return np.asarray(quantized, dtype=np.float32).copy()
    if scale is None:
        raise ExportError(f"{dtype} scale is required")
    return _dq_fp8(quantized, scale) if dtype == DTYPE_FP8 else _dq_nvfp4(quantized, scale)


def _config_hash(tokenizer_id: str, names) -> str:
    return hashlib.sha256("\n".join([tokenizer_id, *sorted(names)]).encode()).hexdigest()


def to_contract(export: WeightExport) -> dict:
    """The ``prometheus.weight_export`` payload (validated against the schema)."""
    shards = []
    for s in export.shards:
        item = {"name": s.name, "dtype": s.dtype, "content_hash": s.content_hash}
        if s.scale_hash is not None:
            item["scale_hash"] = s.scale_hash
        if s.path is not None:
            item["path"] = s.path
        shards.append(item)
    payload = {
        "schema_id": export.schema_id, "schema_version": export.schema_version,
        "export_id": export.export_id, "source_checkpoint_id": export.source_checkpoint_id,
        "target": export.target, "dtype": export.dtype, "tokenizer_id": export.tokenizer_id,
        "model_config_hash": _config_hash(export.tokenizer_id, [s.name for s in export.shards]),
        "shards": shards, "created_at": export.created_at,
    }
    if export.routing_table_hash is not None:
        payload["routing_table_hash"] = export.routing_table_hash
    try:
        contracts.validate_named(SCHEMA_ID, payload)
    except contracts.ValidationError as exc:
        raise ExportError(str(exc)) from exc
    return payload


def export_weights(params: Mapping[str, Any], *, export_id: str, source_checkpoint_id: str,
                   tokenizer_id: str, dtype: str, created_at: str, out_dir: str,
                   routing_table_hash: str | None = None) -> WeightExport:
    if dtype not in DTYPES:
        raise ExportError(f"unsupported dtype {dtype!r}")
    if not export_id or not source_checkpoint_id or not tokenizer_id:
        raise ExportError("export_id, source_checkpoint_id, tokenizer_id must be non-empty")
    if routing_table_hash is not None and not _HEX64.fullmatch(routing_table_hash):
        raise ExportError("routing_table_hash must be lowercase hex SHA-256")
    flat = flatten_params(params)
    if not flat:
        raise ExportError("no array leaves to export")
    dest = Path(out_dir)
    dest.mkdir(parents=True, exist_ok=True)
    shards, sidecar = [], []
    for name, arr in flat.items():
        q, scale = quantize(arr, dtype)
        rel = f"{name}.npy"
        np.save(dest / rel, q)
        entry = {"name": name, "path": rel}
        scale_hash = None
        if scale is not None:
            np.save(dest / f"{name}.scale.npy", np.asarray(scale))
            scale_hash = _hash(scale)
            entry["scale_path"] = f"{name}.scale.npy"
        shards.append(Shard(name, dtype, _hash(q), scale_hash, rel))
        sidecar.append(entry)
    (dest / SIDECAR_NAME).write_text(json.dumps(
        {"format": SIDECAR_FORMAT, "export_id": export_id, "dtype": dtype, "shards": sidecar},
        indent=2, sort_keys=True) + "\n")
    return WeightExport(export_id, source_checkpoint_id, tokenizer_id, TARGET, dtype, len(shards),
                        tuple(shards), routing_table_hash, created_at)


def parity_max_abs_err(params: Mapping[str, Any], exported: WeightExport, out_dir: str) -> float:
    """Largest |dequantised shard - source| over the export (reads the files back)."""
    flat = flatten_params(params)
    if {s.name for s in exported.shards} != set(flat):
        raise ExportError("exported shard names do not match flattened params")
    worst = 0.0
    for s in exported.shards:
        if s.path is None:
            raise ExportError(f"shard {s.name!r} has no path")
        p = Path(s.path)
        p = p if p.is_absolute() else Path(out_dir) / p
        q = np.load(p, allow_pickle=False)
        scale = None
        if s.scale_hash is not None:
            scale = np.load(p.with_name(p.name[:-4] + ".scale.npy"), allow_pickle=False)
        back = dequantize(q, scale, s.dtype)
        src = flat[s.name].astype(np.float32)
        if back.shape != src.shape:
            if back.ndim == src.ndim and back.shape[:-1] == src.shape[:-1] and back.shape[-1] >= src.shape[-1]:
                back = back[..., : src.shape[-1]]
            else:
                raise ExportError(f"dequantized shape {back.shape} does not match source {src.shape}")
        worst = max(worst, float(np.max(np.abs(back - src))) if src.size else 0.0)
    return worst


def export_fp8_e4m3(params: Mapping[str, Any], out_dir: str, *, block: int = 128) -> dict:
    """Real E4M3 bytes with ``block x block`` scales for every matrix (vectors stay fp32):
    ``<name>.e4m3.npy`` (uint8 view) + ``<name>.scale.npy``. Returns name -> content hash."""
    import torch

    from . import kernels

    dest = Path(out_dir)
    dest.mkdir(parents=True, exist_ok=True)
    hashes = {}
    for name, arr in flatten_params(params).items():
        t = torch.as_tensor(arr, dtype=torch.float32)
        if t.ndim < 2:
            np.save(dest / f"{name}.npy", t.numpy())
            hashes[name] = _hash(t.numpy())
            continue
        meta = kernels.fp8_quantize_2d(t.reshape(-1, t.shape[-1]), block=block)
        q = meta.q.view(torch.uint8).reshape(t.shape).numpy()
        np.save(dest / f"{name}.e4m3.npy", q)
        np.save(dest / f"{name}.scale.npy", meta.scale.numpy())
        hashes[name] = _hash(q)
    return hashes
