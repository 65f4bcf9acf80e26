"""Symmetric memory across the ranks of one box (CUDA IPC) and the kernels that use it.

Each rank allocates a device buffer of the same size, exports its IPC handle, and opens
every peer's handle, so a kernel on any rank can load from / store to any peer's buffer at
the same offset over NVLink. Handles travel once through ``torch.distributed``
(``all_gather_object``); nothing else uses the host after set-up.

``SymmetricBuffer``  one allocation + peers' base pointers (``.ptrs`` as a ctypes array)
``SymmetricGroup``   the rank set: flag words for the bounded device barrier, a scalar slot
                     array, and wrappers of the fused kernels in ``csrc/comm/symm.cu``
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import call, ptr, stream_ptr

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
PP = ctypes.POINTER(ctypes.c_void_p)
_lib.register("pb_symm_alloc", [L, PP])
_lib.register("pb_symm_free", [P])
_lib.register("pb_ipc_get_handle", [P, P])
_lib.register("pb_ipc_open_handle", [P, PP])
_lib.register("pb_ipc_close_handle", [P])
_lib.register("pb_barrier_all", [PP, I, I, I, I, L, P, P])
_lib.register("pb_reduce_nparts", [L])
_lib.register("pb_reduce_to_owner", [PP, I, L, L, P, P, P, I, P])
_lib.register("pb_publish_scalar", [PP, I, I, P, P])
_lib.register("pb_sum_slots", [P, I, P, P])
_lib.register("pb_adamw_bcast", [P, P, P, P, PP, I, L, L, F, F, F, F, F, I, P, F, F, P])
_lib.register("pb_muon_apply_bcast", [P, P, PP, I, L, L, F, F, F, P])
# ZeRO-3 parameter sharding (csrc/comm/fsdp.cu)
_lib.register("pb_shard_gather", [PP, L, L, P, I, I, I, P])
_lib.register("pb_muon_apply_table", [P, P, L, I, F, F, F, P, PP, I, I, P])
_lib.register("pb_adamw_table", [P, P, P, P, L, F, F, F, F, F, I, P, F, F, L, L, L, PP, I, I, P])

MAX_RANKS = 8
_DT = {torch.float32: "<f4", torch.bfloat16: None, torch.uint8: "|u1", torch.int32: "<i4"}


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view a raw allocation."""

    def __init__(self, addr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (addr, False),
                                         "version": 3, "strides": None}


GUARD_BYTES = 256          # canary zone on each side of every symmetric allocation
GUARD_BYTE = 0xA5


class SymmetricBuffer:
    """One allocation per rank, mapped by every peer. The usable range is fenced by two
    256-byte canary zones filled with a fixed pattern: peers write into this memory with raw
    pointers, so an off-by-one of a peer kernel lands in a canary instead of in a neighbouring
    allocation, and ``canaries_intact()`` (checked by the trainer after each collective phase
    when ``debug_canaries`` is on, and by the tests) sees it."""

    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks share symmetric memory")
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        local = ctypes.c_void_p()
        call("pb_symm_alloc", self.nbytes + 2 * GUARD_BYTES, ctypes.byref(local))
        self._base_ptr = local.value
        self.local_ptr = local.value + GUARD_BYTES
        handle = ctypes.create_string_buffer(64)
        call("pb_ipc_get_handle", self._base_ptr, ctypes.cast(handle, P))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self._opened = []
        addrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                addrs.append(self.local_ptr)
                continue
            out = ctypes.c_void_p()
            buf = ctypes.create_string_buffer(h, 64)
            call("pb_ipc_open_handle", ctypes.cast(buf, P), ctypes.byref(out))
            self._opened.append(out.value)
            addrs.append(out.value + GUARD_BYTES)
        self.addrs = addrs
        self.ptrs = (ctypes.c_void_p * MAX_RANKS)(*(addrs + [None] * (MAX_RANKS - self.world)))
        dev = torch.device("cuda", torch.cuda.current_device())
        self._raw_all = _RawCuda(self._base_ptr, self.nbytes + 2 * GUARD_BYTES)
        whole = torch.as_tensor(self._raw_all, device=dev)
        self._guards = (whole[:GUARD_BYTES], whole[GUARD_BYTES + self.nbytes:])
        for g in self._guards:
            g.fill_(GUARD_BYTE)
        self.bytes = whole[GUARD_BYTES:GUARD_BYTES + self.nbytes]

    def canaries_intact(self) -> bool:
        """True while nothing has written outside the usable range of this rank's allocation
        (synchronises: it reads the guard zones back)."""
        return all(bool((g == GUARD_BYTE).all()) for g in self._guards)

    def view(self, dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        """Typed view of the local allocation."""
        nb = numel * torch.empty((), dtype=dtype).element_size()
        return self.bytes[byte_offset:byte_offset + nb].view(dtype)

    def peer_ptrs(self, byte_offset: int = 0):
        """ctypes array of every rank's base pointer plus ``byte_offset``."""
        vals = [a + byte_offset for a in self.addrs] + [None] * (MAX_RANKS - self.world)
        return (ctypes.c_void_p * MAX_RANKS)(*vals)

    def close_peers(self):
        """Unmap the peers' allocations (first phase of a collective release)."""
        for a in self._opened:
            call("pb_ipc_close_handle", a)
        self._opened = []

    def free_local(self):
        """Free this rank's allocation. Only after every peer has unmapped it: freeing an
        exported allocation that an importer still has open is undefined."""
        self.bytes = None
        self._guards = ()
        if self.local_ptr:
            call("pb_symm_free", self._base_ptr)
            self.local_ptr = None

    def close(self):
        """Collective release: unmap peers, meet, free."""
        self.close_peers()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.free_local()


class SymmetricGroup:
    """Flags + scalar slots shared by the ranks, and the collective kernels over them."""

    N_SLOTS = 8

    def __init__(self, group=None, wait_budget_s: float = 20.0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ctrl = SymmetricBuffer(4096, group)
        self.flag_ptrs = self.ctrl.peer_ptrs(0)                 # uint32 [N_SLOTS][8]
        self.slot_ptrs = self.ctrl.peer_ptrs(1024)              # float [8]
        self.slots_local = self.ctrl.view(torch.float32, MAX_RANKS, 1024)
        self.epoch = [0] * self.N_SLOTS
        self.budget_ns = int(wait_budget_s * 1e9)
        dev = self.ctrl.bytes.device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.scalar = torch.zeros(1, dtype=torch.float32, device=dev)
        dist.barrier(group)

    def barrier(self, slot: int = 0) -> None:
        """Device-side barrier on the current stream (bounded; see ``check``)."""
        self.epoch[slot] += 1
        call("pb_barrier_all", self.flag_ptrs, self.rank, self.world, slot, self.epoch[slot],
             self.budget_ns, ptr(self.status), stream_ptr())

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"peer wait timed out on rank {self.rank} (code {code})")

    def reduce_to_owner(self, grad: "SymmetricBuffer", byte_offset: int, lo: int, n: int,
                        out: torch.Tensor, scratch: torch.Tensor, sumsq: torch.Tensor,
                        accumulate: bool) -> None:
        """out[lo:lo+n] = rank-ordered fp32 sum of every rank's grad[lo:lo+n]."""
        call("pb_reduce_to_owner", grad.peer_ptrs(byte_offset), self.world, lo, n, ptr(out),
             ptr(scratch), ptr(sumsq), int(accumulate), stream_ptr())

    def allreduce_scalar(self, value: torch.Tensor, out: torch.Tensor) -> None:
        """out = sum over ranks (rank order) of one fp32 per rank. Uses barrier slot 1."""
        call("pb_publish_scalar", self.slot_ptrs, self.rank, self.world, ptr(value), stream_ptr())
        self.barrier(1)
        call("pb_sum_slots", ptr(self.slots_local), self.world, ptr(out), stream_ptr())
        self.barrier(2)   # nobody overwrites a slot before everyone has read it
