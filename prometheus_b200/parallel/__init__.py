"""Parallelism: mesh arithmetic, FSDP / EP / CP / PP building blocks, symmetric memory.

API parity with the reference ``parallel/__init__.py`` (:27-215): ``Axis``, ``ParamKind``,
``MeshError``, ``MeshSpec``, ``PartitionSpec``, ``StageRange``, ``flagship_mesh``,
``tiny_mesh``, ``validate_mesh``, ``device_ids``, ``coord_of``, ``fsdp_partition``,
``pipeline_stage_layers``, ``context_parallel_on``, ``fsdp_shard``, ``fsdp_all_gather``,
``fsdp_reduce_scatter``, ``zero3_views``, ``circular_pipeline``,
``pipeline_forward_schedule``, ``spmd_circular_pipeline``, ``cp_split_seq``,
``cp_ring_schedule``, ``ring_attention_rank``, ``ring_attention``, ``ep_dispatch``,
``ep_combine``.

The list-of-ranks functions (all ranks' shards in one call) are the host-side
definitions used by the tests; the multi-process versions run over
``torch.distributed`` (NCCL on GPUs, gloo on CPU) and over peer memory
(``prometheus_b200.parallel.symm``).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any

from .. import kernels as _kernels


class Axis(str, Enum):
    """Named mesh axes. FSDP shares the EP axis."""

    DP = "dp"
    FSDP = "fsdp"
    EP = "ep"
    PP = "pp"
    CP = "cp"

    def __str__(self) -> str:
        return self.value


class ParamKind(str, Enum):
    """Which FSDP vs EP rule applies to a parameter."""

    ATTENTION = "attention"
    DENSE = "dense"
    SHARED_EXPERT = "shared_expert"
    ROUTED_EXPERT = "routed_expert"
    OTHER = "other"

    def __str__(self) -> str:
        return self.value


class MeshError(ValueError):
    """Mesh, partition, or pipeline layout is invalid."""


FLAGSHIP_EP = 72
FLAGSHIP_FSDP = 72
FLAGSHIP_PP = 12
FLAGSHIP_DP = 115
FLAGSHIP_CP_PRETRAIN = 1
FLAGSHIP_GPUS_PER_REPLICA = FLAGSHIP_EP * FLAGSHIP_PP


@dataclass(frozen=True)
class MeshSpec:
    """Integer device mesh; ``n_devices = dp * pp * ep * cp`` and ``fsdp == ep``."""

    dp: int
    fsdp: int
    ep: int
    pp: int
    cp: int

    @property
    def n_devices(self) -> int:
        return self.dp * self.pp * self.ep * self.cp


@dataclass(frozen=True)
class PartitionSpec:
    """Axis names per tensor dimension. None means replicated on that dim."""

    axes: tuple


@dataclass(frozen=True)
class StageRange:
    """Half-open unique-layer range assigned to one PP stage."""

    start: int
    end: int


def flagship_mesh() -> MeshSpec:
    return MeshSpec(dp=FLAGSHIP_DP, fsdp=FLAGSHIP_FSDP, ep=FLAGSHIP_EP, pp=FLAGSHIP_PP,
                    cp=FLAGSHIP_CP_PRETRAIN)


def tiny_mesh() -> MeshSpec:
    """8 devices: EP=2, FSDP=2, PP=2, DP=2, CP=1."""
    return MeshSpec(dp=2, fsdp=2, ep=2, pp=2, cp=1)


def box_mesh(n_gpus: int = 8, *, cp: int = 1) -> MeshSpec:
    """One B200 box: FSDP = EP = n_gpus / cp ranks, no pipeline, no outer DP."""
    if n_gpus < 1 or cp < 1 or n_gpus % cp != 0:
        raise MeshError("n_gpus must be a positive multiple of cp")
    return MeshSpec(dp=1, fsdp=n_gpus // cp, ep=n_gpus // cp, pp=1, cp=cp)


def validate_mesh(spec: MeshSpec) -> None:
    for name in ("dp", "fsdp", "ep", "pp", "cp"):
        if getattr(spec, name) < 1:
            raise MeshError(f"{name} must be positive")
    if spec.fsdp != spec.ep:
        raise MeshError("fsdp must equal ep")


def device_ids(spec: MeshSpec) -> tuple:
    validate_mesh(spec)
    return tuple(range(spec.n_devices))


def coord_of(device: int, spec: MeshSpec) -> tuple:
    """(dp, pp, ep, cp) coordinate of ``device``; cp is innermost, dp outermost."""
    validate_mesh(spec)
    if device < 0 or device >= spec.n_devices:
        raise MeshError("device id out of range")
    cp_i = device % spec.cp
    rest = device // spec.cp
    ep_i = rest % spec.ep
    rest //= spec.ep
    return (rest // spec.pp, rest % spec.pp, ep_i, cp_i)


def fsdp_partition(kind: ParamKind) -> PartitionSpec:
    """Attention/dense/shared shard on FSDP; routed experts are not FSDP-sharded."""
    return PartitionSpec((None,)) if kind == ParamKind.ROUTED_EXPERT else PartitionSpec(("fsdp",))


def pipeline_stage_layers(n_layers: int, n_pp: int, core_block_layers: int,
                          recurrence: int) -> tuple:
    """FLOP-balanced contiguous layer ranges per PP stage; the last ``core_block_layers``
    layers cost ``recurrence`` each. Greedy: each boundary is the one whose prefix cost is
    closest to its ideal share, leaving at least one layer per remaining stage."""
    if n_layers < 1 or n_pp < 1:
        raise MeshError("n_layers and n_pp must be positive")
    if n_pp > n_layers:
        raise MeshError("n_pp cannot exceed n_layers")
    if core_block_layers < 0 or core_block_layers > n_layers:
        raise MeshError("core_block_layers out of range")
    if recurrence < 1:
        raise MeshError("recurrence must be positive")
    cum = [0]
    for i in range(n_layers):
        cum.append(cum[-1] + (recurrence if i >= n_layers - core_block_layers else 1))
    total = cum[-1]
    out, start = [], 0
    for s in range(n_pp - 1):
        hi = n_layers - (n_pp - 1 - s)
        end = min(range(start + 1, hi + 1), key=lambda e: (abs(n_pp * cum[e] - total * (s + 1)), e))
        out.append(StageRange(start, end))
        start = end
    out.append(StageRange(start, n_layers))
    return tuple(out)


def context_parallel_on(seq_len: int, max_context_pretrain: int) -> bool:
    return seq_len > max_context_pretrain


def ep_dispatch(tokens: Any, meta: Any):
    """Tokens to experts (single address space): wraps ``kernels.ep_dispatch``."""
    return _kernels.ep_dispatch(tokens, meta)


def ep_combine(expert_out: Any, meta: Any, residual: Any):
    return _kernels.ep_combine(expert_out, meta, residual)


from .fsdp import fsdp_all_gather, fsdp_reduce_scatter, fsdp_shard, zero3_views  # noqa: E402
from .schedule import circular_pipeline, pipeline_forward_schedule  # noqa: E402
from .pp import spmd_circular_pipeline, spmd_pipeline_train  # noqa: E402
from .cp import (cp_ring_schedule, cp_split_seq, ring_attention, ring_attention_rank,  # noqa: E402
                 delta_state_handoff, compose_affine)
