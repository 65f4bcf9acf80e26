"""Typed bindings generated from the contract schemas: pydantic models for Python, plain structs
with ``from_json`` / ``to_json`` over the native ``pbn::Json`` value for C++.

    python -m prometheus_b200.contracts.codegen --python OUT_DIR --cpp OUT_DIR

Same job as the reference's ``contracts/_generate.py`` (pydantic + serde types, one model per
schema plus one per shared object definition); the native side of this framework is C++, so the
second emitter writes a header instead of Rust. The pipeline is schema -> ``Shape`` tree -> text:

* a ``Shape`` is one of ``str / int / num / bool / any / list[Shape] / map[Shape] / struct`` with
  the constraints pydantic can carry (``const``, ``enum``, ``ge`` / ``le``, ``min_length``,
  ``pattern``) and a nullable flag;
* an object schema with ``properties`` becomes a struct (named after its path: ``Rollout``,
  ``RolloutLatents``); shared ``$defs`` objects become one struct each, shared scalar ``$defs``
  are inlined;
* ``additionalProperties: false`` becomes ``extra="forbid"`` in pydantic and an unknown-key
  check in the C++ ``from_json``.

The generated C++ keeps free-form values (``any``, objects without ``properties``) as
``pbn::Json``, so a round trip through the structs is lossless.
"""
from __future__ import annotations

import argparse
import json
import keyword
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from . import SCHEMA_DIR, supported_versions, SchemaId

CPP_RESERVED = {"class", "default", "delete", "new", "operator", "private", "public", "template", "namespace",
                "union", "int", "long", "double", "float", "bool", "char", "auto", "register", "switch", "case"}


@dataclass
class Shape:
    kind: str                                  # str int num bool any list map struct
    item: "Shape | None" = None                # list / map element
    struct: str | None = None                  # struct name
    nullable: bool = False
    const: Any = None
    has_const: bool = False
    enum: tuple = ()
    limits: dict = field(default_factory=dict)  # ge le min_length pattern min_items


@dataclass
class Member:
    name: str
    shape: Shape
    required: bool


@dataclass
class Struct:
    name: str
    members: list
    closed: bool                               # additionalProperties: false
    schema_id: str | None = None               # set for the 16 top-level payloads


def camel(text: str) -> str:
    return "".join(p[:1].upper() + p[1:] for p in re.split(r"[^0-9A-Za-z]+", text) if p)


class Lowering:
    """Schema documents of one version directory -> ordered list of ``Struct``."""

    def __init__(self, version: int):
        self.dir = SCHEMA_DIR / f"v{version}"
        self.docs = {p.name: json.loads(p.read_text(encoding="utf-8")) for p in sorted(self.dir.glob("*.json"))}
        self.structs: dict[str, Struct] = {}

    def resolve(self, ref: str, here: str) -> tuple[dict, str, str]:
        """``$ref`` -> (schema, file it lives in, a name hint)."""
        file, _, frag = ref.partition("#")
        file = file or here
        node: Any = self.docs[file]
        hint = file.split(".")[0]
        for part in [p for p in frag.split("/") if p]:
            node = node[part]
            hint = part
        return node, file, hint

    def shape(self, sch: dict, here: str, hint: str) -> Shape:
        if "$ref" in sch:
            target, file, name = self.resolve(sch["$ref"], here)
            if target.get("type") == "object" and "properties" in target:
                return Shape("struct", struct=self.struct(camel(name), target, file))
            return self.shape(target, file, name)
        if "const" in sch:
            v = sch["const"]
            kind = "bool" if isinstance(v, bool) else "int" if isinstance(v, int) else "num" if isinstance(v, float) else "str"
            return Shape(kind, const=v, has_const=True)
        types = sch.get("type")
        nullable = False
        if isinstance(types, list):
            nullable = "null" in types
            rest = [t for t in types if t != "null"]
            types = rest[0] if len(rest) == 1 else None
        out: Shape
        if "enum" in sch and all(isinstance(v, str) for v in sch["enum"]):
            out = Shape("str", enum=tuple(sch["enum"]))
        elif types == "string":
            out = Shape("str", limits={k: sch[s] for k, s in (("min_length", "minLength"), ("pattern", "pattern")) if s in sch})
        elif types in ("integer", "number"):
            out = Shape("int" if types == "integer" else "num",
                        limits={k: sch[s] for k, s in (("ge", "minimum"), ("le", "maximum")) if s in sch})
        elif types == "boolean":
            out = Shape("bool")
        elif types == "array":
            out = Shape("list", item=self.shape(sch.get("items", {}), here, hint + "_item"),
                        limits={"min_items": sch["minItems"]} if "minItems" in sch else {})
        elif types == "object" and "properties" in sch:
            out = Shape("struct", struct=self.struct(camel(hint), sch, here))
        elif types == "object":
            extra = sch.get("additionalProperties")
            out = Shape("map", item=self.shape(extra, here, hint + "_value") if isinstance(extra, dict) else Shape("any"),
                        limits={"min_items": sch["minProperties"]} if "minProperties" in sch else {})
        else:
            out = Shape("any")
        out.nullable = nullable
        return out

    def struct(self, name: str, sch: dict, here: str, schema_id: str | None = None) -> str:
        if name in self.structs:
            return name
        st = Struct(name, [], sch.get("additionalProperties") is False, schema_id)
        self.structs[name] = st                     # registered before the members: cycles terminate
        need = set(sch.get("required", ()))
        members = [Member(key, self.shape(sub, here, f"{name}_{key}"), key in need)
                   for key, sub in sch.get("properties", {}).items()]
        st.members = members
        # children first, so that the emitted text needs no forward declarations
        self.structs[name] = self.structs.pop(name)
        return name

    def run(self) -> list:
        for file, doc in self.docs.items():
            if file.startswith("_"):
                continue
            short = file[: -len(".schema.json")]
            self.struct(camel(short), doc, file, schema_id=f"prometheus.{short}")
        return list(self.structs.values())


def lower(version: int | None = None) -> list:
    version = version or max(supported_versions(next(iter(SchemaId))))
    return Lowering(version).run()


# ------------------------------------------------------------------------------------ pydantic

def _py_type(s: Shape) -> str:
    if s.has_const:
        t = f"Literal[{s.const!r}]"
    elif s.enum:
        t = "Literal[" + ", ".join(repr(v) for v in s.enum) + "]"
    elif s.kind == "struct":
        t = s.struct
    elif s.kind == "list":
        t = f"list[{_py_type(s.item)}]"
    elif s.kind == "map":
        t = f"dict[str, {_py_type(s.item)}]"
    else:
        t = {"str": "str", "int": "StrictInt", "num": "float", "bool": "StrictBool", "any": "Any"}[s.kind]
    return f"{t} | None" if s.nullable else t


def _py_member(m: Member) -> str:
    args = []
    attr = m.name
    if keyword.iskeyword(attr) or attr.startswith("_") or attr in ("model_config", "schema", "copy", "json", "dict"):
        attr = attr.strip("_") + "_"
        args.append(f"alias={m.name!r}")
    lim = m.shape.limits
    if not m.shape.has_const and not m.shape.enum:
        for key in ("ge", "le", "min_length", "pattern"):
            if key in lim:
                args.append(f"{key}={lim[key]!r}")
        if "min_items" in lim:
            args.append(f"min_length={lim['min_items']!r}")
    t = _py_type(m.shape)
    if m.required:
        default = "..."
    else:
        default = "None"
        if not m.shape.nullable:
            t += " | None"
    head = f"    {attr}: {t}"
    if not args and m.required:
        return head
    return f"{head} = Field({', '.join([default] + args)})"


def pydantic_source(structs: list) -> str:
    out = ['"""Contract types generated from the JSON schemas. Regenerate; do not edit."""',
           "from __future__ import annotations", "", "from typing import Any, Literal", "",
           "from pydantic import BaseModel, ConfigDict, Field, StrictBool, StrictInt", "", ""]
    for st in structs:
        out.append(f"class {st.name}(BaseModel):")
        out.append(f'    model_config = ConfigDict(extra="{"forbid" if st.closed else "allow"}", populate_by_name=True, protected_namespaces=())')
        if st.schema_id:
            out.append(f"    SCHEMA_ID: ClassVar[str] = {st.schema_id!r}")
        out += [_py_member(m) for m in st.members] or ["    pass"]
        out += ["", ""]
    text = "\n".join(out).rstrip() + "\n"
    return text.replace("from typing import Any, Literal", "from typing import Any, ClassVar, Literal")


# ------------------------------------------------------------------------------------------ C++

def _cpp_ident(name: str) -> str:
    ident = re.sub(r"[^0-9A-Za-z_]", "_", name)
    return ident + "_" if ident in CPP_RESERVED or ident[:1].isdigit() else ident


def _cpp_type(s: Shape) -> str:
    if s.kind == "struct":
        return s.struct
    if s.kind == "list":
        return f"std::vector<{_cpp_type(s.item)}>"
    if s.kind == "map":
        return f"std::map<std::string, {_cpp_type(s.item)}>"
    return {"str": "std::string", "int": "int64_t", "num": "double", "bool": "bool", "any": "pbn::Json"}[s.kind]


def _cpp_read(s: Shape, expr: str, depth: int = 0) -> str:
    """C++ expression that converts the ``pbn::Json`` ``expr`` to the shape's type."""
    if s.kind == "struct":
        return f"{s.struct}::from_json({expr})"
    if s.kind == "list":
        v = f"e{depth}"
        return (f"[&]{{ {_cpp_type(s)} out; for (const auto& {v} : ({expr}).arr()) out.push_back({_cpp_read(s.item, v, depth + 1)}); "
                f"return out; }}()")
    if s.kind == "map":
        v = f"kv{depth}"
        return (f"[&]{{ {_cpp_type(s)} out; for (const auto& {v} : ({expr}).obj()) out.emplace({v}.first, "
                f"{_cpp_read(s.item, v + '.second', depth + 1)}); return out; }}()")
    return {"str": f"({expr}).as_string()", "int": f"({expr}).as_i64()", "num": f"({expr}).as_double()",
            "bool": f"({expr}).as_bool()", "any": f"({expr})"}[s.kind]


def _cpp_write(s: Shape, expr: str, depth: int = 0) -> str:
    if s.kind == "struct":
        return f"({expr}).to_json()"
    if s.kind == "list":
        v = f"e{depth}"
        return (f"[&]{{ pbn::JsonArray out; for (const auto& {v} : {expr}) out.push_back({_cpp_write(s.item, v, depth + 1)}); "
                f"return pbn::Json(std::move(out)); }}()")
    if s.kind == "map":
        v = f"kv{depth}"
        return (f"[&]{{ pbn::JsonObject out; for (const auto& {v} : {expr}) out.emplace({v}.first, "
                f"{_cpp_write(s.item, v + '.second', depth + 1)}); return pbn::Json(std::move(out)); }}()")
    if s.kind == "int":
        return f"pbn::Json(static_cast<int64_t>({expr}))"
    return f"pbn::Json({expr})"


def _cpp_literal(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return repr(v)
    return json.dumps(v)


def cpp_source(structs: list) -> str:
    out = ["// Contract types generated from the JSON schemas. Regenerate; do not edit.", "#pragma once",
           "#include <cstdint>", "#include <map>", "#include <optional>", "#include <string>", "#include <vector>", "",
           '#include "common.hpp"', "", "namespace pbn::contracts_gen {", ""]
    for st in structs:
        out.append(f"struct {st.name} {{")
        if st.schema_id:
            out.append(f"  static constexpr const char* kSchemaId = {json.dumps(st.schema_id)};")
        for m in st.members:
            t = _cpp_type(m.shape)
            opt = (not m.required) or m.shape.nullable
            init = f" = {_cpp_literal(m.shape.const)}" if m.shape.has_const and not opt else ""
            out.append(f"  {'std::optional<' + t + '>' if opt else t} {_cpp_ident(m.name)}{init};")
        out.append("")
        out.append(f"  static {st.name} from_json(const pbn::Json& j) {{")
        out.append(f"    {st.name} v;")
        out.append("    const auto& o = j.obj();")
        if st.closed:
            names = ", ".join(json.dumps(m.name) for m in st.members)
            out.append(f"    static const char* const known[] = {{{names}}};")
            out.append("    for (const auto& kv : o) {")
            out.append("      bool ok = false;")
            out.append("      for (const char* k : known) ok = ok || kv.first == k;")
            out.append(f'      if (!ok) throw pbn::Error("Schema", "{st.name}: unknown field " + kv.first);')
            out.append("    }")
        for m in st.members:
            key, ident = json.dumps(m.name), _cpp_ident(m.name)
            read = _cpp_read(m.shape, "*p")
            out.append(f"    if (const pbn::Json* p = j.find({key}); p != nullptr" +
                       (" && !p->is_null()" if m.shape.nullable or not m.required else "") + ") {")
            out.append(f"      v.{ident} = {read};")
            if m.shape.has_const:
                cmp = f"*v.{ident}" if (not m.required or m.shape.nullable) else f"v.{ident}"
                out.append(f'      if (!({cmp} == {_cpp_literal(m.shape.const)})) throw pbn::Error("Schema", "{st.name}.{m.name}: unexpected value");')
            if m.shape.enum:
                cmp = f"*v.{ident}" if (not m.required or m.shape.nullable) else f"v.{ident}"
                tests = " && ".join(f"{cmp} != {json.dumps(e)}" for e in m.shape.enum)
                out.append(f'      if ({tests}) throw pbn::Error("Schema", "{st.name}.{m.name}: not one of the allowed values");')
            out.append("    }" + (f' else if (p == nullptr) {{ throw pbn::Error("Schema", "{st.name}: missing field {m.name}"); }}'
                                  if m.required else ""))
        out.append("    (void)o;")
        out.append("    return v;")
        out.append("  }")
        out.append("")
        out.append("  pbn::Json to_json() const {")
        out.append("    pbn::JsonObject o;")
        for m in st.members:
            key, ident = json.dumps(m.name), _cpp_ident(m.name)
            if (not m.required) or m.shape.nullable:
                out.append(f"    if ({ident}) o.emplace({key}, {_cpp_write(m.shape, '*' + ident)});")
                if m.required:
                    out.append(f"    else o.emplace({key}, pbn::Json(nullptr));")
            else:
                out.append(f"    o.emplace({key}, {_cpp_write(m.shape, ident)});")
        out.append("    return pbn::Json(std::move(o));")
        out.append("  }")
        out.append("};")
        out.append("")
    out.append("}  // namespace pbn::contracts_gen")
    return "\n".join(out) + "\n"


def write_python(out_dir) -> Path:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "__init__.py").write_text('"""Generated contract types."""\nfrom .types import *  # noqa: F401,F403\n',
                                         encoding="utf-8")
    path = out_dir / "types.py"
    path.write_text(pydantic_source(lower()), encoding="utf-8")
    return path


def write_cpp(out_dir) -> Path:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / "contracts_types.hpp"
    path.write_text(cpp_source(lower()), encoding="utf-8")
    return path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m prometheus_b200.contracts.codegen")
    ap.add_argument("--python", metavar="DIR")
    ap.add_argument("--cpp", metavar="DIR")
    a = ap.parse_args(argv)
    if not a.python and not a.cpp:
        ap.error("nothing to do: give --python and / or --cpp")
    if a.python:
        print(write_python(a.python))
    if a.cpp:
        print(write_cpp(a.cpp))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
