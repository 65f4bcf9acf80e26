"""Generated contract types: the pydantic models parse every golden payload and reject the broken
fixtures; the C++ header compiles against the native JSON value and round-trips every golden.
(reference strategy: tests/test_contracts.py:220-234 -- generated Python parses each golden, the
generated native source names a type for every schema.)"""
import importlib.util
import json
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

from prometheus_b200 import contracts
from prometheus_b200.contracts import codegen

ROOT = Path(__file__).resolve().parents[1]


def _no_nulls(x):
    """Optional members that are null and members that are absent are the same value to the structs."""
    if isinstance(x, dict):
        return {k: _no_nulls(v) for k, v in x.items() if v is not None}
    return [_no_nulls(v) for v in x] if isinstance(x, list) else x

IDS = list(contracts.SchemaId)


def _load_generated(tmp_path):
    contracts.generate_python(tmp_path / "gen")
    spec = importlib.util.spec_from_file_location("pb_generated_types", tmp_path / "gen" / "types.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["pb_generated_types"] = mod
    spec.loader.exec_module(mod)
    for name in dir(mod):
        obj = getattr(mod, name)
        if isinstance(obj, type) and hasattr(obj, "model_rebuild") and obj.__module__ == mod.__name__:
            obj.model_rebuild(_types_namespace=vars(mod))
    return mod


def test_lowering_names_one_struct_per_schema_and_shared_definition():
    structs = {s.name: s for s in codegen.lower()}
    for sid in IDS:
        short = sid.value.split(".", 1)[1]
        st = structs[codegen.camel(short)]
        assert st.schema_id == sid.value
        assert any(m.name == "schema_id" and m.shape.has_const for m in st.members)
    for shared in ("Mesh", "Artifact", "Provenance", "Decontamination"):
        assert shared in structs
    order = list(structs)
    assert order.index("Mesh") < order.index("Checkpoint")          # children are emitted first


def test_pydantic_models_parse_every_golden_and_round_trip(tmp_path):
    mod = _load_generated(tmp_path)
    for sid in IDS:
        payload = contracts.load_golden(sid, 1)
        model = getattr(mod, codegen.camel(sid.value.split(".", 1)[1]))
        assert model.SCHEMA_ID == sid.value
        obj = model.model_validate(payload)
        again = obj.model_dump(by_alias=True, exclude_none=True)
        contracts.validate(again)
        assert _no_nulls(again) == _no_nulls(payload)


def test_pydantic_models_reject_what_the_schemas_reject(tmp_path):
    import pydantic

    mod = _load_generated(tmp_path)
    good = contracts.load_golden(contracts.SchemaId.TOKENIZER, 1)
    cases = {
        "extra": {**good, "surprise": 1},
        "missing": {k: v for k, v in good.items() if k != "vocab_size"},
        "wrong_id": {**good, "schema_id": "prometheus.vocab"},
        "wrong_version": {**good, "schema_version": 2},
        "bad_type": {**good, "vocab_size": "many"},
        "bool_as_int": {**good, "vocab_size": True},
    }
    for name, payload in cases.items():
        with pytest.raises(pydantic.ValidationError):
            mod.Tokenizer.model_validate(payload)
        with pytest.raises((contracts.ValidationError, contracts.UnknownSchemaError)):
            contracts.validate(payload)


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_cpp_header_compiles_and_round_trips_every_golden(tmp_path):
    contracts.generate_cpp(tmp_path)
    text = (tmp_path / "contracts_types.hpp").read_text()
    for sid in IDS:
        assert f"struct {codegen.camel(sid.value.split('.', 1)[1])} " in text
    cases = []
    for sid in IDS:
        name = codegen.camel(sid.value.split(".", 1)[1])
        cases.append(f'  if (which == "{sid.value}") {{ std::cout << {name}::from_json(j).to_json().dump(); return 0; }}')
    main = tmp_path / "main.cpp"
    main.write_text(
        '#include <fstream>\n#include <iostream>\n#include <sstream>\n#include "contracts_types.hpp"\n'
        "using namespace pbn::contracts_gen;\n"
        "int main(int argc, char** argv) {\n"
        "  std::ifstream f(argv[1]); std::stringstream ss; ss << f.rdbuf();\n"
        "  try {\n"
        "  pbn::Json j = pbn::Json::parse(ss.str());\n"
        '  std::string which = j.at("schema_id").as_string();\n' + "\n".join(cases) + "\n"
        '  } catch (const pbn::Error& e) { std::cerr << e.what(); return 3; }\n'
        "  return 2;\n}\n")
    exe = tmp_path / "roundtrip"
    subprocess.run(["g++", "-std=c++17", "-O0", "-I", str(ROOT / "csrc" / "native"), "-I", str(tmp_path), str(main),
                    "-o", str(exe)], check=True)
    for sid in IDS:
        payload = contracts.load_golden(sid, 1)
        p = tmp_path / "in.json"
        p.write_text(json.dumps(payload))
        res = subprocess.run([str(exe), str(p)], capture_output=True, text=True)
        assert res.returncode == 0, (sid, res.stderr)
        assert _no_nulls(json.loads(res.stdout)) == _no_nulls(payload), sid
    bad = dict(contracts.load_golden(contracts.SchemaId.TOKENIZER, 1), surprise=1)
    p.write_text(json.dumps(bad))
    res = subprocess.run([str(exe), str(p)], capture_output=True, text=True)
    assert res.returncode == 3 and "unknown field surprise" in res.stderr
