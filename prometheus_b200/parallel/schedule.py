"""Pipeline tick schedule and the in-process pipeline runner.

Reference ``parallel/schedule.py:20-103``: at tick ``t`` stage ``s`` runs microbatch
``t - s`` when that index is valid; ``n_microbatches + n_stages - 1`` ticks in total.
"""
from __future__ import annotations

from typing import Callable, Sequence


def pipeline_forward_schedule(n_microbatches: int, n_stages: int) -> tuple:
    from . import MeshError

    if n_microbatches < 1 or n_stages < 1:
        raise MeshError("n_microbatches and n_stages must be >= 1, got "
                        f"n_microbatches={n_microbatches}, n_stages={n_stages}")
    return tuple(
        tuple((t - s) if 0 <= t - s < n_microbatches else None for s in range(n_stages))
        for t in range(n_microbatches + n_stages - 1))


def circular_pipeline(microbatches: Sequence, stage_fns: Sequence[Callable]) -> tuple:
    """Run every stage on every microbatch in schedule order (one process, sequential
    within a tick by increasing stage). ``result[m] = f_last(... f_0(mb[m]))``."""
    from . import MeshError

    acts = list(microbatches)
    fns = tuple(stage_fns)
    if not acts or not fns:
        raise MeshError(f"microbatches and stage_fns must be non-empty, got {len(acts)} "
                        f"microbatches and {len(fns)} stages")
    for tick in pipeline_forward_schedule(len(acts), len(fns)):
        for stage, mb in enumerate(tick):
            if mb is not None:
                acts[mb] = fns[stage](acts[mb])
    return tuple(acts)
