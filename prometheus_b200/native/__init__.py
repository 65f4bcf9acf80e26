"""C++ systems components (pybind11 module built in-tree under ``_lib``).

``prometheus_b200.native.loader`` / ``.ckpt`` / ... are the sub-modules of the
compiled ``_pb200_native`` extension; ``NativeError`` is the exception every
component raises, with a ``kind`` attribute naming the failure class.
"""
from __future__ import annotations

import importlib.util
import sys

from .. import _build


def _load():
    name = "_pb200_native"
    if name in sys.modules:
        return sys.modules[name]
    path = _build.native_lib_path()        # honours PB200_NATIVE_SANITIZE
    if not path.exists():
        import os

        _build.build_native(sanitize=os.environ.get(_build.SANITIZE_ENV, ""))
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_ext = _load()
NativeError = _ext.NativeError


def __getattr__(attr):
    return getattr(_ext, attr)
