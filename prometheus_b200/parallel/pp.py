"""Pipeline parallelism over ``torch.distributed`` point-to-point (NCCL on GPUs, gloo on CPU).

``spmd_circular_pipeline`` is the multi-process counterpart of the reference's
``parallel/placement.py:86-226`` (``shard_map`` over a ``"pp"`` mesh axis, a scan over
ticks, ``ppermute(i -> i+1)``, ``psum`` to replicate the outputs): every rank of the
group is one stage, runs the same tick loop, receives its input activation from the
previous stage and posts its output to the next with non-blocking ``isend`` / ``irecv``: the
receive of the next microbatch is posted before the current one is computed, so the transfer
of tick ``t + 1`` overlaps the compute of tick ``t``. The last stage's outputs are replicated
with a single broadcast of the stacked outputs; their shape travels once per call (it is the
same for every microbatch), not once per microbatch. With no process group (or a group of
one) it degenerates to the in-process runner.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

from .schedule import circular_pipeline, pipeline_forward_schedule


def spmd_circular_pipeline(microbatches: Sequence[torch.Tensor], n_stages: int,
                           stage_fn: Callable, *, group=None, replicate: bool = True):
    """Run ``stage_fn(stage_index, x)`` as an ``n_stages``-deep pipeline.

    Every rank passes the same ``microbatches`` (only stage 0 reads them). Activations must
    keep the microbatch's shape and dtype between stages (a stage that changes them must
    be the last). Returns the tuple of last-stage outputs in microbatch order on every rank
    when ``replicate`` (else only on the last stage; other ranks get ``None`` entries).
    Raises ``MeshError`` if the group has fewer ranks than stages.
    """
    from . import MeshError

    mbs = list(microbatches)
    if n_stages < 1 or not mbs:
        raise MeshError("n_stages must be >= 1 and microbatches non-empty")
    if not dist.is_available() or not dist.is_initialized() or n_stages == 1:
        if n_stages > 1:
            raise MeshError(f"{n_stages} stages need {n_stages} ranks; no process group")
        return circular_pipeline(mbs, [lambda x: stage_fn(0, x)])
    world = dist.get_world_size(group)
    if world < n_stages:
        raise MeshError(f"{n_stages} stages need {n_stages} ranks, group has {world}")
    rank = dist.get_rank(group)
    stage = rank
    if stage >= n_stages:          # spare ranks only take part in the final broadcast
        outs = [None] * len(mbs)
    else:
        outs = [None] * len(mbs)
        pending = []
        nxt = dist.get_global_rank(group, stage + 1) if group is not None else stage + 1
        prv = dist.get_global_rank(group, stage - 1) if group is not None and stage > 0 else stage - 1
        mine = [tick[stage] for tick in pipeline_forward_schedule(len(mbs), n_stages) if tick[stage] is not None]

        def post_recv(mb):
            buf = torch.empty_like(mbs[mb])
            return dist.irecv(buf, src=prv, group=group), buf

        inflight = post_recv(mine[0]) if stage > 0 and mine else None
        for j, mb in enumerate(mine):
            if stage == 0:
                x = mbs[mb]
            else:
                req, x = inflight
                # the next microbatch's receive is in flight while this one is computed
                inflight = post_recv(mine[j + 1]) if j + 1 < len(mine) else None
                req.wait()
            y = stage_fn(stage, x)
            if stage + 1 < n_stages:
                pending.append((dist.isend(y.contiguous(), dst=nxt, group=group), y))
            else:
                outs[mb] = y
        for req, _keep in pending:
            req.wait()
    if not replicate:
        return tuple(outs)
    last = dist.get_global_rank(group, n_stages - 1) if group is not None else n_stages - 1
    # one shape message and one broadcast for all microbatches (they share shape and dtype)
    meta = [None]
    if rank == n_stages - 1:
        meta = [(tuple(outs[0].shape), outs[0].dtype)]
    dist.broadcast_object_list(meta, src=last, group=group)
    shape, dtype = meta[0]
    if rank == n_stages - 1:
        stacked = torch.stack([o.contiguous() for o in outs])
    else:
        stacked = torch.empty((len(mbs), *shape), dtype=dtype, device=mbs[0].device)
    dist.broadcast(stacked, src=last, group=group)
    return tuple(stacked[m] for m in range(len(mbs)))
