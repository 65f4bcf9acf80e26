"""Versioned JSON contracts for every cross-module format (checkpoint manifest, loader
state, packing, event log, weight export, tokenizer, rollout, ...).

The 16 schemas and their golden payloads under ``schemas/v1`` and ``goldens/v1`` are data
shared with the reference (``contracts/schemas/v1/*.schema.json``); this module is the
registry and validator: ``validate``, ``validate_named``, ``migrate``, ``load_schema``,
``load_golden``, ``current_version``, ``supported_versions``, ``schema_path``, ``SchemaId``
(reference ``contracts/__init__.py:48-273``). Validation is JSON Schema draft 2020-12 with
``$ref`` resolved against the other files of the same version directory.
"""
from __future__ import annotations

import copy
import json
from datetime import datetime
from enum import Enum
from functools import lru_cache
from pathlib import Path
from typing import Any, Mapping

from jsonschema import Draft202012Validator, FormatChecker
from referencing import Registry, Resource

CONTRACTS_ROOT = Path(__file__).resolve().parent
SCHEMA_DIR = CONTRACTS_ROOT / "schemas"
GOLDEN_DIR = CONTRACTS_ROOT / "goldens"
_PREFIX = "prometheus."


class ValidationError(ValueError):
    """Payload does not match its schema."""


class UnknownSchemaError(KeyError):
    """No schema file for that id / version."""


class MigrationError(ValueError):
    """No migration path between the two versions."""


def _discover() -> dict[str, str]:
    names = set()
    for vdir in SCHEMA_DIR.glob("v*"):
        for f in vdir.glob("*.schema.json"):
            if not f.name.startswith("_"):
                names.add(f.name[: -len(".schema.json")])
    return {n.upper(): _PREFIX + n for n in sorted(names)}


SchemaId = Enum("SchemaId", _discover(), type=str)
SchemaId.__str__ = lambda self: self.value  # type: ignore[assignment]


def _sid(schema_id) -> "SchemaId":
    try:
        return SchemaId(schema_id.value if isinstance(schema_id, SchemaId) else schema_id)
    except ValueError as exc:
        raise UnknownSchemaError(str(schema_id)) from exc


def _short(sid) -> str:
    return str(_sid(sid).value)[len(_PREFIX):]


def _ver(version) -> int:
    if isinstance(version, bool) or not isinstance(version, int) or version < 1:
        raise UnknownSchemaError(f"version {version!r}")
    return version


def schema_path(schema_id, version: int) -> Path:
    path = SCHEMA_DIR / f"v{_ver(version)}" / f"{_short(schema_id)}.schema.json"
    if not path.is_file():
        raise UnknownSchemaError(f"{_sid(schema_id).value}@v{version}")
    return path


def load_schema(schema_id, version: int) -> dict:
    return json.loads(schema_path(schema_id, version).read_text(encoding="utf-8"))


def supported_versions(schema_id) -> list[int]:
    short = _short(schema_id)
    found = sorted(int(d.name[1:]) for d in SCHEMA_DIR.iterdir()
                   if d.is_dir() and d.name[:1] == "v" and d.name[1:].isdigit()
                   and (d / f"{short}.schema.json").is_file())
    if not found:
        raise UnknownSchemaError(str(schema_id))
    return found


def current_version(schema_id) -> int:
    return supported_versions(schema_id)[-1]


def load_golden(schema_id, version: int, name: str = "default") -> dict:
    path = GOLDEN_DIR / f"v{_ver(version)}" / f"{_short(schema_id)}.{name}.json"
    if not path.is_file():
        raise UnknownSchemaError(f"{_sid(schema_id).value}@v{version}/{name}")
    return json.loads(path.read_text(encoding="utf-8"))


def _is_datetime(value) -> bool:
    if not isinstance(value, str):
        return True
    try:
        datetime.fromisoformat(value[:-1] + "+00:00" if value.endswith("Z") else value)
    except ValueError:
        return False
    return True


@lru_cache(maxsize=1)
def _formats() -> FormatChecker:
    fc = FormatChecker()
    fc.checkers = dict(Draft202012Validator.FORMAT_CHECKER.checkers)
    fc.checkers.setdefault("date-time", (_is_datetime, ()))
    return fc


@lru_cache(maxsize=8)
def _registry(version: int) -> Registry:
    pairs = []
    for path in sorted((SCHEMA_DIR / f"v{version}").glob("*.json")):
        doc = json.loads(path.read_text(encoding="utf-8"))
        if isinstance(doc.get("$id"), str):
            pairs.append((doc["$id"], Resource.from_contents(doc)))
    return Registry().with_resources(pairs)


def _select(payload: Mapping[str, Any]):
    if not isinstance(payload, Mapping):
        raise ValidationError("payload must be an object")
    if "schema_id" not in payload:
        raise ValidationError("missing schema_id")
    if not isinstance(payload["schema_id"], str):
        raise ValidationError("schema_id must be a string")
    sid = _sid(payload["schema_id"])
    if "schema_version" not in payload:
        raise ValidationError("missing schema_version")
    v = payload["schema_version"]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ValidationError("schema_version must be an integer")
    if v not in supported_versions(sid):
        raise UnknownSchemaError(f"{sid.value}@v{v}")
    return sid, v


def validate(payload: Mapping[str, Any]) -> None:
    """Raise ``ValidationError`` unless ``payload`` matches the schema it names."""
    sid, version = _select(payload)
    validator = Draft202012Validator(load_schema(sid, version), registry=_registry(version),
                                     format_checker=_formats())
    errors = sorted(validator.iter_errors(payload), key=lambda e: list(e.absolute_path))
    if errors:
        raise ValidationError("; ".join(e.message for e in errors))


def validate_named(schema_id, payload: Mapping[str, Any]) -> None:
    """``validate`` plus a check that the payload names the expected schema."""
    if isinstance(payload, Mapping) and payload.get("schema_id") != _sid(schema_id).value:
        raise ValidationError(f"expected schema_id {_sid(schema_id).value}")
    validate(payload)


def migrate(payload: Mapping[str, Any], to_version: int) -> dict:
    """Copy of ``payload`` at ``to_version``; v1 is the only version, so only the identity."""
    if not isinstance(payload, Mapping):
        raise ValidationError("payload must be an object")
    v = payload.get("schema_version")
    if isinstance(v, bool) or not isinstance(v, int):
        raise ValidationError("schema_version must be an integer")
    if v == to_version:
        return copy.deepcopy(dict(payload))
    raise MigrationError(f"no migration from v{v} to v{to_version}")


def generate_python(out_dir) -> None:
    """Write pydantic models for every schema under ``out_dir`` (``types.py`` + ``__init__.py``);
    reference ``contracts/__init__.py:250-257``."""
    from .codegen import write_python

    write_python(Path(out_dir))


def generate_cpp(out_dir) -> None:
    """Write ``contracts_types.hpp`` (structs with ``from_json`` / ``to_json`` over the native JSON
    value) under ``out_dir``. The reference emits serde types for its Rust crates at this point
    (``contracts/__init__.py:260-265``); the native layer here is C++."""
    from .codegen import write_cpp

    write_cpp(Path(out_dir))


generate_native = generate_cpp


def generate_all() -> None:
    """Python types under ``contracts/generated``, the C++ header under ``csrc/native/generated``."""
    generate_python(CONTRACTS_ROOT / "generated")
    generate_cpp(CONTRACTS_ROOT.parent.parent / "csrc" / "native" / "generated")
