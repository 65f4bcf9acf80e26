"""Content-addressed cache of compiled kernel artifacts.

In this framework the "program" is the text handed to ``nvcc`` (kernel source +
flags) and the artifact is the cubin / shared object it produced; the cache is a
flat directory on shared storage so a cold start compiles each kernel once per
cluster, not once per rank.

On-disk record (same as the reference ``kernels/compile_cache.py:21-60``):
``b"CC01" | u64 big-endian payload length | payload | sha256(payload)``, stored in
a file named ``sha256(program)``. Files are published with a same-directory
rename after ``fsync`` so a reader sees a complete record or nothing; anything
that does not parse as a complete record (short file, wrong magic, bad
checksum) is a miss.
"""
from __future__ import annotations

import hashlib
import os
import struct
import uuid
from pathlib import Path
from typing import Callable

_TAG = b"CC01"
_HEAD = struct.Struct(">4sQ")
_DIGEST_LEN = hashlib.sha256().digest_size


class CacheError(ValueError):
    """Program bytes, artifact, or cache root broke the compile-cache contract."""


def program_hash(program: bytes) -> str:
    """Lower-case hex SHA-256 of the program bytes (the cache key)."""
    if not isinstance(program, bytes):
        raise CacheError(f"program must be bytes, got {type(program).__name__}")
    if not program:
        raise CacheError("empty program")
    return hashlib.sha256(program).hexdigest()


def _pack(payload: bytes) -> bytes:
    return b"".join((_HEAD.pack(_TAG, len(payload)), payload, hashlib.sha256(payload).digest()))


def _unpack(blob: bytes) -> bytes | None:
    if len(blob) < _HEAD.size + _DIGEST_LEN:
        return None
    tag, n = _HEAD.unpack_from(blob)
    if tag != _TAG or n == 0 or len(blob) != _HEAD.size + n + _DIGEST_LEN:
        return None
    body = blob[_HEAD.size:_HEAD.size + n]
    if hashlib.sha256(body).digest() != blob[_HEAD.size + n:]:
        return None
    return body


def _publish(path: Path, data: bytes) -> None:
    tmp = path.with_name(f".{path.name}.{uuid.uuid4().hex}.partial")
    try:
        with open(tmp, "wb") as fh:
            fh.write(data)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, path)
    finally:
        try:
            tmp.unlink()
        except FileNotFoundError:
            pass


class CompileCache:
    """Directory of artifacts keyed by ``program_hash``. The root is created if missing."""

    def __init__(self, root) -> None:
        root = Path(root)
        if root.exists() and not root.is_dir():
            raise CacheError(f"cache root is not a directory: {root}")
        root.mkdir(parents=True, exist_ok=True)
        self.root = root

    def _read(self, key: str) -> bytes | None:
        p = self.root / key
        try:
            return _unpack(p.read_bytes()) if p.is_file() else None
        except OSError:
            return None

    def lookup(self, program: bytes) -> bytes | None:
        """Artifact stored for ``program`` or None. Never compiles."""
        return self._read(program_hash(program))

    def store(self, program: bytes, compiled: bytes) -> str:
        """Publish ``compiled`` for ``program``; idempotent for identical bytes, an error
        when a different artifact is already stored under the same program."""
        key = program_hash(program)
        if not isinstance(compiled, bytes):
            raise CacheError(f"compiled must be bytes, got {type(compiled).__name__}")
        if not compiled:
            raise CacheError("empty compiled artifact")
        have = self._read(key)
        if have is not None:
            if have == compiled:
                return key
            raise CacheError("program already stored with a different artifact")
        _publish(self.root / key, _pack(compiled))
        return key

    def get_or_compile(self, program: bytes, compile: Callable[[bytes], bytes]):
        """``(artifact, hit)``; ``compile`` runs once, only on a miss, and its result is
        stored. An exception from ``compile`` propagates and stores nothing."""
        hit = self.lookup(program)
        if hit is not None:
            return hit, True
        made = compile(program)
        if not isinstance(made, bytes) or not made:
            raise CacheError("compile returned an empty artifact")
        self.store(program, made)
        return made, False
