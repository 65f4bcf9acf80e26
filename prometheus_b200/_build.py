"""In-tree build of the native libraries.

Two shared objects are produced next to the package (never installed into
site-packages, so a process that loads them shows the in-tree path):

* ``prometheus_b200/_lib/libpb200_kernels.so`` — every ``csrc/kernels/*.cu`` and
  ``csrc/comm/*.cu`` compiled by ``nvcc`` for ``sm_100a`` only. The kernels
  export a plain C ABI (raw device pointers + a stream handle) and are bound
  with ``ctypes``; nothing in them depends on the PyTorch headers, so a file
  compiles in seconds.
* ``prometheus_b200/_lib/_pb200_native*.so`` — the C++17 systems code under
  ``csrc/native`` (checkpoint store, data loader, controller, observability,
  harness) bound with pybind11.

``python -m prometheus_b200._build`` builds both; ``build_all()`` is what
``__graft_entry__.build()`` calls. Objects are rebuilt only when their source
(or a shared header) is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "_lib"
OBJ_DIR = ROOT / "build" / "obj"

KERNEL_LIB = LIB_DIR / "libpb200_kernels.so"
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]


SANITIZE_ENV = "PB200_NATIVE_SANITIZE"     # "", "address,undefined" or "thread": which build to load


def _san_tag(sanitize: str | None) -> str:
    return "" if not sanitize else "_" + sanitize.replace(",", "_")


def native_lib_path(sanitize: str | None = None) -> Path:
    """The pybind11 module; with ``sanitize`` (default: the ``PB200_NATIVE_SANITIZE``
    environment variable) the instrumented build that lives beside it in ``_lib/san_*``."""
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    sanitize = os.environ.get(SANITIZE_ENV, "") if sanitize is None else sanitize
    if sanitize:
        return LIB_DIR / ("san" + _san_tag(sanitize)) / f"_pb200_native{suffix}"
    return LIB_DIR / f"_pb200_native{suffix}"


def sanitizer_runtime(sanitize: str) -> str:
    """Path of the sanitizer runtime to ``LD_PRELOAD`` when an instrumented module is loaded
    into an uninstrumented interpreter."""
    lib = "libtsan.so" if "thread" in sanitize else "libasan.so"
    # libstdc++ rides along: the interpreter is not linked against it, and the runtime resolves
    # its __cxa_throw interceptor when it starts
    paths = [subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
             for name in (lib, "libstdc++.so")]
    return " ".join(paths)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src_list, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_list)


def _run(cmd, verbose=False):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def kernel_sources() -> list[Path]:
    return sorted(list((CSRC / "kernels").glob("*.cu")) + list((CSRC / "comm").glob("*.cu")))


def build_kernels(verbose: bool = False, force: bool = False, debug_bounds: bool = False) -> Path:
    """Compile every .cu for sm_100a and link libpb200_kernels.so. ``debug_bounds`` builds
    ``libpb200_kernels_dbg.so`` with ``-DPB_DEBUG_BOUNDS`` instead: indices that come from data
    are checked in the kernels and a violation is recorded and skipped rather than executed
    (``PB200_DEBUG_BOUNDS=1`` makes the package load that library)."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    tag = "dbg_" if debug_bounds else ""
    extra = ["-DPB_DEBUG_BOUNDS"] if debug_bounds else []
    target = LIB_DIR / "libpb200_kernels_dbg.so" if debug_bounds else KERNEL_LIB
    headers = list((CSRC / "kernels").glob("*.cuh")) + list((CSRC / "comm").glob("*.cuh"))
    srcs = kernel_sources()
    objs, jobs = [], []
    for src in srcs:
        obj = OBJ_DIR / (tag + src.parent.name + "_" + src.stem + ".o")
        objs.append(obj)
        if force or _newer([src, *headers], obj):
            jobs.append([nvcc, *NVCC_ARCH, *NVCC_FLAGS, *extra, "-rdc=false", "-I", CSRC / "kernels", "-I",
                         CSRC / "comm", "-c", src, "-o", obj])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(objs, target):
        # link beside the target and rename: a process (or a snapshot of the tree) never sees a
        # half-written library
        tmp = target.with_name(target.name + ".tmp")
        _run([nvcc, *NVCC_ARCH, "-shared", "-o", tmp, *objs], verbose)
        os.replace(tmp, target)
    return target


def build_native(verbose: bool = False, force: bool = False, sanitize: str = "") -> Path | None:
    """Compile csrc/native/*.cpp into the pybind11 module (host only, no CUDA).

    ``sanitize`` = ``"address,undefined"`` or ``"thread"`` builds an instrumented copy
    (``-fsanitize=...``, ``-O1 -g``, frame pointers kept) under ``_lib/san_*`` for the host-side
    race / memory checks of the systems code (the asynchronous checkpoint writer, the loader):
    load it with ``PB200_NATIVE_SANITIZE=<same string>`` and the matching runtime preloaded
    (``sanitizer_runtime``)."""
    srcs = sorted((CSRC / "native").glob("*.cpp"))
    if not srcs:
        return None
    import pybind11

    if sanitize not in ("", "address,undefined", "thread"):
        raise ValueError("sanitize must be '', 'address,undefined' or 'thread'")
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    headers = [h for pat in ("*.hpp", "*.h", "*.inc") for h in (CSRC / "native").glob(pat)]
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", CSRC / "native"]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function"]
    link_extra = []
    if sanitize:
        flags = ["-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={sanitize}", "-std=c++17", "-fPIC",
                 "-fvisibility=hidden", "-Wall", "-Wno-unused-function"]
        link_extra = [f"-fsanitize={sanitize}"]
    objs, jobs = [], []
    for src in srcs:
        obj = OBJ_DIR / ("native" + _san_tag(sanitize) + "_" + src.stem + ".o")
        objs.append(obj)
        if force or _newer([src, *headers], obj):
            jobs.append(["g++", *flags, *inc, "-c", src, "-o", obj])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    out = native_lib_path(sanitize)
    out.parent.mkdir(parents=True, exist_ok=True)
    if force or jobs or _newer(objs, out):
        tmp = out.with_name(out.name + ".tmp")
        _run(["g++", "-shared", "-o", tmp, *objs, *link_extra, "-lpthread", "-lz"], verbose)
        os.replace(tmp, out)
    return out


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_kernels(verbose, force)
    build_kernels(verbose, force, debug_bounds=True)     # the self-checking variant rides along
    build_native(verbose, force)


if __name__ == "__main__":
    san = [a.split("=", 1)[1] for a in sys.argv if a.startswith("--sanitize=")]
    if "--debug-bounds" in sys.argv:
        print("built:", build_kernels(verbose="-v" in sys.argv, force="--force" in sys.argv, debug_bounds=True))
    elif san:
        print("built:", build_native(verbose="-v" in sys.argv, force="--force" in sys.argv, sanitize=san[0]))
    else:
        build_all(verbose="-v" in sys.argv, force="--force" in sys.argv)
        print("built:", KERNEL_LIB, native_lib_path(""))
