"""Repository invariants a CI job enforces besides the test suite.

    python -m prometheus_b200.utils.ci_checks tree            # from the repository root
    python -m prometheus_b200.utils.ci_checks skips junit.xml

tree   production code does not import ``tests``; every ``.cu`` / ``.cpp`` under ``csrc`` is
       picked up by the build (a source left out is never compiled or tested); every native
       ``bind_*`` function is registered in ``bindings.cpp``.
skips  the only acceptable pytest skip on a CPU runner is a missing GPU.
(reference: ``.github/ci/checks.py``, same two sub-commands for its Python + Cargo tree)
"""
from __future__ import annotations

import re
import sys
import xml.etree.ElementTree as ET
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
_TEST_IMPORT = re.compile(r"^\s*(from|import)\s+tests(\.|\s|$)", re.M)
_GPU_SKIP = re.compile(r"\b(GPU|GPUs|CUDA)\b", re.I)


def check_test_imports(root: Path = ROOT) -> list:
    errors = []
    for path in list((root / "prometheus_b200").rglob("*.py")) + [root / "bench.py", root / "__graft_entry__.py"]:
        if path.exists() and _TEST_IMPORT.search(path.read_text(encoding="utf-8")):
            errors.append(f"production code imports tests/: {path.relative_to(root)}")
    return errors


def check_sources_are_built(root: Path = ROOT) -> list:
    from .. import _build

    errors = []
    built = {p.resolve() for p in _build.kernel_sources()}
    for cu in (root / "csrc").rglob("*.cu"):
        if cu.resolve() not in built:
            errors.append(f"{cu.relative_to(root)} is not compiled by the kernel build")
    bindings = (root / "csrc" / "native" / "bindings.cpp").read_text(encoding="utf-8")
    for cpp in (root / "csrc" / "native").glob("*.cpp"):
        for name in re.findall(r"^void (bind_\w+)\(", cpp.read_text(encoding="utf-8"), re.M):
            if bindings.count(name) < 2:      # a declaration and a call
                errors.append(f"{name} ({cpp.name}) is not registered in bindings.cpp")
    return errors


def check_skips(junit_xml: Path) -> list:
    errors = []
    for case in ET.parse(junit_xml).getroot().iter("testcase"):
        for sk in case.findall("skipped"):
            msg = (sk.get("message") or "") + (sk.text or "")
            if not _GPU_SKIP.search(msg):
                errors.append(f"{case.get('classname')}::{case.get('name')} skipped for a reason other than a GPU: {msg.strip()[:120]}")
    return errors


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["tree"]:
        errors = check_test_imports() + check_sources_are_built()
    elif argv[:1] == ["skips"] and len(argv) == 2:
        errors = check_skips(Path(argv[1]))
    else:
        print(__doc__)
        return 2
    for e in errors:
        print(e)
    return 1 if errors else 0


if __name__ == "__main__":
    raise SystemExit(main())
