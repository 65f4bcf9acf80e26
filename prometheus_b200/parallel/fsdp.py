"""FSDP / ZeRO-3 shard arithmetic (host definition) and ownership planning.

``fsdp_shard`` / ``fsdp_all_gather`` / ``fsdp_reduce_scatter`` / ``zero3_views`` take all
ranks' tensors in one call and define the semantics the device kernels implement
(reference ``parallel/fsdp.py:118-222``): ``numpy.array_split`` bounds (the first
``dim % n`` ranks get one extra), gather = concatenation, reduce-scatter = **left fold in
fp32 in rank order**, then shard, then cast back. ``pb_reduce_to_owner`` (csrc/comm/symm.cu)
folds peers' gradient slices in exactly that order, so a multi-GPU step is bitwise
reproducible and equal to this function.

``plan_ownership`` is the matrix-ownership partition the trainer uses: Muon needs whole
matrices, so each matrix is owned by one rank (optimizer state, Newton-Schulz and the
update happen there) instead of every matrix being cut into 1/n slices.
"""
from __future__ import annotations

from typing import Sequence

import torch

Tensor = torch.Tensor


def _err(msg: str):
    from . import MeshError

    raise MeshError(msg)


def _check_n_rank(n, rank):
    if isinstance(n, bool) or not isinstance(n, int) or n < 1:
        _err(f"n must be an int >= 1, got {n!r}")
    if isinstance(rank, bool) or not isinstance(rank, int) or rank < 0 or rank >= n:
        _err(f"rank {rank!r} out of range for n={n}")
    return n, rank


def _axis(axis, ndim):
    if isinstance(axis, bool) or not isinstance(axis, int):
        _err("axis must be an int")
    a = axis + ndim if axis < 0 else axis
    if a < 0 or a >= ndim:
        _err(f"axis {axis} out of range for ndim={ndim}")
    return a


def split_bounds(dim: int, n: int, rank: int) -> tuple[int, int]:
    """``numpy.array_split`` bounds of ``rank`` among ``n`` over ``dim`` elements."""
    base, rem = divmod(dim, n)
    if rank < rem:
        lo = rank * (base + 1)
        return lo, lo + base + 1
    lo = rem * (base + 1) + (rank - rem) * base
    return lo, lo + base


def fsdp_shard(param, n: int, axis: int, rank: int) -> Tensor:
    n, rank = _check_n_rank(n, rank)
    t = torch.as_tensor(param)
    a = _axis(axis, t.ndim)
    dim = t.shape[a]
    if dim < n:
        _err(f"axis {axis} length {dim} < n={n}; zero-size shard is invalid")
    lo, hi = split_bounds(dim, n, rank)
    return t.narrow(a, lo, hi - lo)


def _check_same(arrays: Sequence[Tensor], skip_axis):
    ref = arrays[0]
    for t in arrays[1:]:
        if t.dtype != ref.dtype:
            _err(f"mixed dtypes {ref.dtype} vs {t.dtype}")
        if t.ndim != ref.ndim:
            _err(f"mismatched ranks {ref.ndim} vs {t.ndim}")
        for i in range(ref.ndim):
            if i != skip_axis and t.shape[i] != ref.shape[i]:
                _err(f"mismatched shapes {tuple(ref.shape)} vs {tuple(t.shape)}")


def _seq(values, what):
    try:
        vals = [torch.as_tensor(v) for v in values]
    except TypeError:
        _err(f"{what} must be a non-empty sequence")
    if not vals:
        _err(f"{what} must be a non-empty sequence")
    return vals


def fsdp_all_gather(shards, axis: int) -> Tensor:
    arrays = _seq(shards, "shards")
    a = _axis(axis, arrays[0].ndim)
    _check_same(arrays, a)
    return arrays[0] if len(arrays) == 1 else torch.cat(arrays, dim=a)


def _acc_dtype(dtype):
    if dtype == torch.bool or dtype.is_complex:
        _err(f"reduce-scatter does not support dtype {dtype}")
    if dtype.is_floating_point:
        return torch.float64 if dtype == torch.float64 else torch.float32
    return torch.int64


def fsdp_reduce_scatter(partials, axis: int, rank: int) -> Tensor:
    """Sum (left fold in the accumulation dtype, rank order), shard, cast back."""
    arrays = _seq(partials, "partials")
    _check_same(arrays, None)
    n, rank = _check_n_rank(len(arrays), rank)
    out_dtype = arrays[0].dtype
    acc_dtype = _acc_dtype(out_dtype)
    acc = arrays[0].to(acc_dtype)
    for p in arrays[1:]:
        acc = acc + p.to(acc_dtype)
    return fsdp_shard(acc, n, axis, rank).to(out_dtype)


def zero3_views(param, kind, n: int, axis: int, rank: int):
    """(bf16 device view, fp32 master view) of one parameter: shard first, then cast.
    Routed experts are not FSDP-sharded (both views are the whole tensor)."""
    from . import ParamKind

    if not isinstance(kind, ParamKind):
        _err(f"kind must be a parallel.ParamKind, got {type(kind).__name__}")
    t = torch.as_tensor(param)
    if not t.dtype.is_floating_point:
        _err(f"non-floating param dtype {t.dtype}")
    sel = t if kind is ParamKind.ROUTED_EXPERT else fsdp_shard(t, n, axis, rank)
    return sel.to(torch.bfloat16), sel.to(torch.float32)


def plan_ownership(counts: Sequence[int], world: int) -> list[list[tuple[int, int]]]:
    """Split each shape class of ``counts[c]`` equal matrices into ``world`` contiguous
    index ranges: ``plan[rank][c] = (first, last_exclusive)`` (array_split bounds, so the
    load differs by at most one matrix per class)."""
    if world < 1:
        _err("world must be >= 1")
    return [[split_bounds(int(c), world, r) for c in counts] for r in range(world)]


# ---------------------------------------------------------------------------
# fused all-gather + GEMM over peer memory
# ---------------------------------------------------------------------------
class AgWeight:
    """A weight ``(N, K)`` bf16 sharded by rows over the ranks of a group, held in symmetric
    memory so that the consuming GEMM gathers it itself.

    Every rank allocates the full ``N x K`` buffer; rows ``[rank R, (rank + 1) R)`` with
    ``R = N / world`` are the rank's authoritative shard, the other rows are landing space.
    ``linear(x)`` launches one kernel (``pb_gemm_bf16_ag``): copier warps pull the peers' rows
    over NVLink panel by panel while the tensor-core tiles of the panels already present run,
    starting with the rank's own panel. Forward only (the trainer keeps replicated bf16
    weights refreshed by the update kernels; this is the FSDP-style alternative for weights
    that should stay sharded)."""

    def __init__(self, n: int, k: int, group=None, wait_budget_s: float = 20.0):
        from .symm import SymmetricBuffer, SymmetricGroup

        self.sym = SymmetricGroup(group, wait_budget_s)
        self.world, self.rank = self.sym.world, self.sym.rank
        if n % self.world or (n // self.world) % 8 or n <= 128 or k % 8:
            _err("AgWeight needs N divisible by world with shards of a multiple of 8 rows, N > 128, K % 8 == 0")
        self.n, self.k = int(n), int(k)
        self.rows = n // self.world
        self.buf = SymmetricBuffer(n * k * 2, group)
        self.full = self.buf.view(torch.bfloat16, n * k).view(n, k)
        self.ptrs = self.buf.peer_ptrs(0)
        self.ready = torch.zeros((n + 255) // 256, dtype=torch.int32, device=self.full.device)
        self.epoch = 0
        self.budget_ns = int(wait_budget_s * 1e9)

    @property
    def shard(self) -> Tensor:
        """This rank's rows (a view into the symmetric buffer; write the weights here)."""
        return self.full[self.rank * self.rows:(self.rank + 1) * self.rows]

    def linear(self, x: Tensor) -> Tensor:
        """``x @ W^T`` for ``x`` of shape ``(M, K)`` bf16 -> ``(M, N)`` bf16."""
        from ..ops._lib import call, ptr, stream_ptr
        from ..ops.functional import status_word

        x = x.contiguous()
        m = x.shape[0]
        out = torch.empty((m, self.n), dtype=torch.bfloat16, device=x.device)
        self.sym.barrier(3)            # every rank's shard is final and nobody still reads old rows
        self.epoch += 1
        call("pb_gemm_bf16_ag", ptr(x), self.ptrs, ptr(out), m, self.n, self.k, self.k, self.k, self.n,
             self.rank, self.world, ptr(self.ready), self.epoch, self.budget_ns,
             ptr(status_word(x.device)), stream_ptr())
        return out

    def close(self) -> None:
        self.buf.close()
