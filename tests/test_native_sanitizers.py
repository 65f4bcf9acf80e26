"""Host-side memory and race checks of the C++ systems code: the loader, the checkpoint store
(its asynchronous writer thread above all) and the controller run their own test files under
AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer, in a child interpreter
with the instrumented build of the module (``python -m prometheus_b200._build --sanitize=...``)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from prometheus_b200 import _build

ROOT = Path(__file__).resolve().parent.parent


def _run_under(sanitize: str, files, extra_env):
    _build.build_native(sanitize=sanitize)
    env = dict(os.environ, **extra_env)
    env[_build.SANITIZE_ENV] = sanitize
    env["LD_PRELOAD"] = _build.sanitizer_runtime(sanitize)
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", *[str(ROOT / "tests" / f) for f in files]]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)


@pytest.mark.skipif(not Path(_build.sanitizer_runtime("address,undefined").split()[0]).exists(),
                    reason="no sanitizer runtime in this toolchain")
def test_loader_ckpt_control_clean_under_asan_ubsan():
    res = _run_under("address,undefined", ["test_native_loader_ckpt.py", "test_native_control_obs.py"],
                     {"ASAN_OPTIONS": "detect_leaks=0", "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1"})
    out = res.stdout + res.stderr
    assert res.returncode == 0 and " passed" in out, out[-3000:]
    assert "AddressSanitizer" not in out and "runtime error:" not in out, out[-3000:]


@pytest.mark.skipif(not Path(_build.sanitizer_runtime("thread").split()[0]).exists(),
                    reason="no sanitizer runtime in this toolchain")
def test_async_checkpoint_writer_clean_under_tsan():
    res = _run_under("thread", ["test_native_loader_ckpt.py"],
                     {"TSAN_OPTIONS": "exitcode=66:halt_on_error=0:report_signal_unsafe=0"})
    out = res.stdout + res.stderr
    assert res.returncode == 0 and " passed" in out, out[-3000:]
    assert "ThreadSanitizer" not in out, out[-3000:]
