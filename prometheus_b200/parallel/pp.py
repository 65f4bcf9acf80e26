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

``spmd_pipeline_train`` adds what the reference's pipeline does not have: the backward. All
microbatches go forward (activations kept per stage), then come back in reverse order: the
last stage differentiates the loss, every other stage receives the gradient of its output
from the next stage, back-propagates through its own saved graph (parameter gradients
accumulate locally in ``.grad``) and sends the gradient of its input to the previous stage,
again with the next receive posted before the current backward runs.
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


def spmd_pipeline_train(microbatches: Sequence[torch.Tensor], n_stages: int, stage_fn: Callable,
                        loss_fn: Callable, *, group=None):
    """Forward and backward of an ``n_stages``-deep pipeline over ``microbatches`` (all forwards,
    then all backwards in reverse microbatch order).

    ``stage_fn(stage, x)`` is this rank's stage (its parameters' ``.grad`` accumulate);
    ``loss_fn(y, m)`` maps the last stage's output of microbatch ``m`` to a scalar. Returns the
    sum of the microbatch losses on the last stage (``None`` on the others). Activations keep the
    microbatch's shape and dtype between stages. Gradients equal those of the unsplit model:
    ``d(sum_m loss_m) / d(parameters of every stage)``."""
    from . import MeshError

    mbs = list(microbatches)
    if n_stages < 1 or not mbs:
        raise MeshError("n_stages must be >= 1 and microbatches non-empty")
    if n_stages == 1 or not (dist.is_available() and dist.is_initialized()):
        if n_stages > 1:
            raise MeshError(f"{n_stages} stages need {n_stages} ranks; no process group")
        total = None
        for m, x in enumerate(mbs):
            loss = loss_fn(stage_fn(0, x), m)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        return total
    world = dist.get_world_size(group)
    if world < n_stages:
        raise MeshError(f"{n_stages} stages need {n_stages} ranks, group has {world}")
    stage = dist.get_rank(group)
    if stage >= n_stages:
        return None
    g = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    first, last = stage == 0, stage == n_stages - 1
    n = len(mbs)

    def irecv_like(src):
        buf = torch.empty_like(mbs[0])
        return dist.irecv(buf, src=src, group=group), buf

    # ---- forward: keep (input leaf, output) of every microbatch
    saved, sends = [], []
    inflight = None if first else irecv_like(g(stage - 1))
    for m in range(n):
        if first:
            x = mbs[m]
        else:
            req, x = inflight
            inflight = irecv_like(g(stage - 1)) if m + 1 < n else None
            req.wait()
            x.requires_grad_(True)
        y = stage_fn(stage, x)
        saved.append((x, y))
        if not last:
            sends.append((dist.isend(y.detach().contiguous(), dst=g(stage + 1), group=group), y))
    for req, _keep in sends:
        req.wait()
    # ---- backward, last microbatch first
    total, sends = None, []
    inflight = None if last else irecv_like(g(stage + 1))
    for m in reversed(range(n)):
        x, y = saved[m]
        if last:
            loss = loss_fn(y, m)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        else:
            req, gy = inflight
            inflight = irecv_like(g(stage + 1)) if m > 0 else None
            req.wait()
            y.backward(gy)
        if not first:
            sends.append((dist.isend(x.grad.contiguous(), dst=g(stage - 1), group=group), x))
        saved[m] = None
    for req, _keep in sends:
        req.wait()
    return total
