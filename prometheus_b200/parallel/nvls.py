"""NVLS multicast buffers: the in-switch (``multimem``) variant of the broadcast and reduce
paths, selected at run time next to the peer-to-peer one.

``NvlsBuffer.create(nbytes, group)`` returns a buffer every rank of the group holds a copy of,
with two addresses: ``local`` (this GPU's copy) and ``mc`` (the multicast address: a
``multimem.st`` there lands in every rank's copy, a ``multimem.ld_reduce`` returns the sum over
the copies, both done by the NVSwitch). It returns ``None`` on every rank when any rank cannot
set it up (no multicast support on the device, a driver that refuses, no permission on the
fabric): callers then keep the peer-to-peer kernels. Nothing here raises for that case.

Set-up (csrc/comm/nvls.cu for the driver calls): rank 0 creates the multicast object and
exports a POSIX file descriptor, which travels to the other ranks over a Unix-domain socket
(``SCM_RIGHTS``); every rank adds its device, then allocates and binds its physical memory,
then maps the multicast address. The phases are separated by barriers of the process group and
an agreement (all-reduce MIN) on success, so no rank binds memory to an object another rank
has already abandoned.

A rank must not exit while its memory is bound: ``close()`` is collective and callers release
the buffer before they leave (the trainer does so in ``Trainer.close``).

Reference: the reference only plans in-switch collectives (spec/05-training-system.md:11-16).
"""
from __future__ import annotations

import ctypes
import os
import socket
import uuid

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import ptr, stream_ptr

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
PI = ctypes.POINTER(ctypes.c_int)
PP = ctypes.POINTER(ctypes.c_void_p)
_lib.register("pb_nvls_supported", [PI])
_lib.register("pb_nvls_rounded_size", [L, I])
_lib.register("pb_nvls_create", [L, I, PI, PP])
_lib.register("pb_nvls_import", [I, L, I, PP])
_lib.register("pb_nvls_close_fd", [I])
_lib.register("pb_nvls_add_device", [P])
_lib.register("pb_nvls_bind_map", [P, PP, PP])
_lib.register("pb_nvls_free", [P])
_lib.register("pb_mm_muon_apply", [P, P, P, L, F, F, F, P])
_lib.register("pb_mm_adamw", [P, P, P, P, P, L, F, F, F, F, F, I, P, F, F, P])
_lib.register("pb_mm_allreduce_f32", [P, L, L, P])


def _fn(name):
    lib = _lib.load()
    fn = getattr(lib, name)
    return fn


def supported() -> bool:
    """This device and driver offer multicast objects (says nothing about the peers)."""
    if os.environ.get("PB200_NVLS", "1") == "0" or not torch.cuda.is_available():
        return False
    out = ctypes.c_int(0)
    _fn("pb_nvls_supported")(ctypes.byref(out))
    return bool(out.value)


def _all_ok(ok: bool, group, device) -> bool:
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(int(t.item()))


def _send_fd_to_ranks(fd: int | None, group, rank: int, world: int) -> int | None:
    """Rank 0's file descriptor to every other rank of the group (one box): Unix-domain
    sockets named by a token rank 0 broadcasts. Returns the received descriptor (rank 0: its
    own), or None on failure."""
    token = [uuid.uuid4().hex if rank == 0 else None]
    src = dist.get_global_rank(group, 0) if group is not None else 0
    dist.broadcast_object_list(token, src=src, group=group)
    path = lambda r: f"/tmp/pb200_nvls_{token[0]}_{r}"     # noqa: E731
    got: int | None = fd
    listener = None
    try:
        if rank != 0:
            listener = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            listener.bind(path(rank))
            listener.listen(1)
            listener.settimeout(30.0)
        dist.barrier(group)                      # every listener is up
        if rank == 0:
            for r in range(1, world):
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
                    s.settimeout(30.0)
                    s.connect(path(r))
                    socket.send_fds(s, [b"m"], [fd])
        else:
            conn, _ = listener.accept()
            with conn:
                conn.settimeout(30.0)
                _, fds, _, _ = socket.recv_fds(conn, 1, 1)
                got = fds[0] if fds else None
    except OSError:
        got = None
    finally:
        if listener is not None:
            listener.close()
            try:
                os.unlink(path(rank))
            except OSError:
                pass
    return got


class NvlsBuffer:
    """A multicast-backed buffer. Use :meth:`create`; ``None`` means "not available here"."""

    def __init__(self, handle, local_ptr: int, mc_ptr: int, nbytes: int, group, device):
        self._handle = handle
        self.local_ptr, self.mc_ptr, self.nbytes = local_ptr, mc_ptr, nbytes
        self.group, self.device = group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        from .symm import _RawCuda

        self._raw = _RawCuda(local_ptr, nbytes)
        self.bytes = torch.as_tensor(self._raw, device=device)

    @classmethod
    def create(cls, nbytes: int, group=None) -> "NvlsBuffer | None":
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        device = torch.device("cuda", torch.cuda.current_device())
        if world < 2 or not _all_ok(supported(), group, device):
            return None
        size = int(_fn("pb_nvls_rounded_size")(int(nbytes), world))
        if not _all_ok(size > 0, group, device):
            return None
        handle, fd = ctypes.c_void_p(), ctypes.c_int(-1)
        ok = True
        if rank == 0:
            ok = _fn("pb_nvls_create")(size, world, ctypes.byref(fd), ctypes.byref(handle)) == 0
        if not _all_ok(ok, group, device):
            cls._abandon(handle, fd.value)
            return None
        got = _send_fd_to_ranks(fd.value if rank == 0 else None, group, rank, world)
        ok = got is not None
        if ok and rank != 0:
            ok = _fn("pb_nvls_import")(int(got), size, world, ctypes.byref(handle)) == 0
        if got is not None:
            _fn("pb_nvls_close_fd")(int(got))       # the handle holds its own reference
        if not _all_ok(ok, group, device):
            cls._abandon(handle, -1)
            return None
        ok = _fn("pb_nvls_add_device")(handle) == 0
        if not _all_ok(ok, group, device):          # also: every device is added before any bind
            cls._abandon(handle, -1)
            return None
        local, mc = ctypes.c_void_p(), ctypes.c_void_p()
        ok = _fn("pb_nvls_bind_map")(handle, ctypes.byref(local), ctypes.byref(mc)) == 0
        torch.cuda.synchronize()
        if not _all_ok(ok, group, device):          # also: every rank is bound before any use
            torch.cuda.synchronize()
            dist.barrier(group)
            cls._abandon(handle, -1)
            return None
        return cls(handle, int(local.value), int(mc.value), size, group, device)

    @staticmethod
    def _abandon(handle, fd: int) -> None:
        if fd is not None and fd >= 0:
            _fn("pb_nvls_close_fd")(int(fd))
        if handle is not None and handle.value:
            _fn("pb_nvls_free")(handle)

    def view(self, dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        nb = numel * torch.empty((), dtype=dtype).element_size()
        return self.bytes[byte_offset:byte_offset + nb].view(dtype)

    def mc_at(self, byte_offset: int) -> int:
        return self.mc_ptr + byte_offset

    def close(self) -> None:
        """Collective: every rank calls it, with nothing of any rank still using the buffer."""
        if self._handle is None:
            return
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.bytes = None
        _fn("pb_nvls_free")(self._handle)
        self._handle = None
        dist.barrier(self.group)


def allreduce_f32(buf: NvlsBuffer, numel: int, sym) -> None:
    """In-switch all-reduce (sum) of the first ``numel`` fp32 elements of ``buf`` on the current
    stream: afterwards every rank's copy holds the sum. ``sym``: a ``SymmetricGroup`` whose
    bounded device barriers (slots 1 and 2) order the phases. ``numel`` a multiple of
    4 x world."""
    from .fsdp import split_bounds
    from ..ops._lib import call

    lo, hi = split_bounds(numel // 4, buf.world, buf.rank)
    sym.barrier(1)                       # every rank's inputs are written
    call("pb_mm_allreduce_f32", buf.mc_ptr, lo * 4, (hi - lo) * 4, stream_ptr())
    sym.barrier(2)                       # every slice is reduced and written back
