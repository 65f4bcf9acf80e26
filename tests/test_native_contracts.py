"""C++ schema validator against the 16 contract schemas and the Python validator."""
import copy
import json
from pathlib import Path

import pytest

from prometheus_b200 import contracts, native
from prometheus_b200.native import NativeError

C = native.contracts
ROOT = str(Path(contracts.__file__).parent / "schemas")
GOLDENS = sorted((Path(contracts.__file__).parent / "goldens" / "v1").glob("*.default.json"))


def _kind(e):
    return e.value.kind


def _agree(payload):
    """Both validators accept, or both reject."""
    try:
        contracts.validate(payload)
        py_ok = True
    except (contracts.ValidationError, contracts.UnknownSchemaError):
        py_ok = False
    try:
        C.validate(json.dumps(payload), ROOT)
        cc_ok = True
    except NativeError:
        cc_ok = False
    assert py_ok == cc_ok, (py_ok, cc_ok, payload)
    return cc_ok


def test_every_golden_validates_and_mutations_agree_with_python():
    assert len(GOLDENS) == 16
    n_rejected = 0
    for path in GOLDENS:
        g = json.loads(path.read_text())
        C.validate(json.dumps(g), ROOT)
        assert C.current_version(g["schema_id"], ROOT) == 1
        for key in list(g):
            if key in ("schema_id", "schema_version"):
                continue
            dropped = {k: v for k, v in g.items() if k != key}
            n_rejected += not _agree(dropped)
            for bad in (None, -1, "", [], {}, "x" * 3, 1.5, True):
                m = copy.deepcopy(g)
                m[key] = bad
                n_rejected += not _agree(m)
        extra = dict(g, not_a_field=1)
        assert not _agree(extra)
    assert n_rejected > 200


def test_envelope_errors_migrate_and_formats():
    g = json.loads(GOLDENS[0].read_text())
    for payload, kind in (([1], "Validation"), ({"schema_version": 1}, "Validation"), ({"schema_id": 3, "schema_version": 1}, "Validation"),
                          ({"schema_id": "prometheus.checkpoint"}, "Validation"),
                          ({"schema_id": "prometheus.checkpoint", "schema_version": "1"}, "Validation"),
                          ({"schema_id": "prometheus.checkpoint", "schema_version": 1.5}, "Validation"),
                          ({"schema_id": "prometheus.checkpoint", "schema_version": 2}, "UnknownSchema"),
                          ({"schema_id": "prometheus.nope", "schema_version": 1}, "UnknownSchema"),
                          ({"schema_id": "other.checkpoint", "schema_version": 1}, "UnknownSchema"),
                          ({"schema_id": "prometheus.../x", "schema_version": 1}, "UnknownSchema")):
        with pytest.raises(NativeError) as e:
            C.validate(json.dumps(payload), ROOT)
        assert _kind(e) == kind, payload
    with pytest.raises(NativeError) as e:
        C.validate("{not json", ROOT)
    assert _kind(e) == "Validation"
    assert json.loads(C.migrate(json.dumps(g), 1)) == g
    with pytest.raises(NativeError) as e:
        C.migrate(json.dumps(g), 2)
    assert _kind(e) == "Migration" and "v1 to v2" in str(e.value)
    with pytest.raises(NativeError) as e:
        C.current_version("prometheus.nope", ROOT)
    assert _kind(e) == "UnknownSchema"
    for s, ok in (("2026-01-02T03:04:05Z", True), ("2026-01-02T03:04:05.123+02:00", True), ("2026-02-30T00:00:00Z", False),
                  ("2026-01-02 03:04:05Z", False), ("2026-01-02T03:04:05", False), ("2024-02-29T23:59:60Z", True),
                  ("2026-13-01T00:00:00Z", False), ("nonsense", False)):
        assert C.valid_datetime(s) == ok, s
