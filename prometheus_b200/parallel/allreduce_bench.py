"""All-reduce bus-bandwidth table in the layout of nccl-tests, one rank per GPU.

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 8 \\
        -m prometheus_b200.parallel.allreduce_bench --max-bytes 1073741824

Rank 0 prints one row per size: ``size count type redop root time(us) algbw busbw #wrong``
(out of place, then in place), times taken on the device as the max over ranks, bus bandwidth
``= algbw * 2 (n - 1) / n``. With ``NCCL_DEBUG=INFO`` in the environment NCCL's own log shows
whether the in-switch (NVLS) algorithm was chosen. After NCCL's table the same sizes are run
through this package's own all-reduce (``--own``, on by default with more than one GPU): the
two-shot ``multimem.ld_reduce`` / ``multimem.st`` kernel over an NVLS multicast buffer when the
machine offers one, and the rank-ordered peer-to-peer fold (reduce to owner + an all-gather of
the owners' slices by peer loads), which is the bit-reproducible form. Falls back to gloo on
machines without a GPU, where the table is only a functional check. ``native.ncshare.parse_busbw_gbps`` reads the
last out-of-place row (the V0 stage records it as ``busbw_gbps``).
"""
from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist


def _time_allreduce(x: torch.Tensor, iters: int, warmup: int, cuda: bool) -> float:
    """Microseconds per all-reduce, max over ranks."""
    for _ in range(warmup):
        dist.all_reduce(x)
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            dist.all_reduce(x)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / iters
    else:
        t0 = time.perf_counter()
        for _ in range(iters):
            dist.all_reduce(x)
        us = (time.perf_counter() - t0) * 1e6 / iters
    t = torch.tensor([us], dtype=torch.float64, device=x.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _own_table(a, rank: int, world: int, dev, scale: float) -> None:
    """The package's own all-reduce at the same sizes: in-switch (multimem) and rank-ordered
    peer-to-peer. Same columns as the NCCL table; one section per variant."""
    import ctypes

    from ..ops._lib import call, ptr, query, stream_ptr
    from . import nvls
    from .fsdp import split_bounds
    from .symm import SymmetricBuffer, SymmetricGroup

    grp = SymmetricGroup(wait_budget_s=10.0)
    max_count = a.max_bytes // 4
    mc = nvls.NvlsBuffer.create(4 * max_count)
    p2p = SymmetricBuffer(4 * max_count)
    out = torch.empty(max_count, dtype=torch.float32, device=dev)
    scratch = torch.empty(max(4096, query("pb_reduce_nparts", max_count)), device=dev)
    sq = torch.zeros(1, device=dev)

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / a.iters], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    variants = []
    if mc is not None:
        variants.append(("multimem (in-switch, order-free)", "mc"))
    variants.append(("peer-to-peer (rank-ordered fold + gather)", "p2p"))
    rows = {}
    try:
        for title, kind in variants:
            size = a.min_bytes
            while size <= a.max_bytes:
                count = size // 4 // (4 * world) * (4 * world)
                lo, hi = split_bounds(count // 4, world, rank)
                lo, hi = lo * 4, hi * 4
                if kind == "mc":
                    view = mc.view(torch.float32, count)
                    view.fill_(float(rank + 1))
                    torch.cuda.synchronize()
                    dist.barrier()
                    nvls.allreduce_f32(mc, count, grp)
                    torch.cuda.synchronize()
                    wrong = int((view != world * (world + 1) / 2).sum().item())
                    us = timed(lambda: nvls.allreduce_f32(mc, count, grp))
                else:
                    view = p2p.view(torch.float32, count)

                    def fold():
                        grp.barrier(1)
                        grp.reduce_to_owner(p2p, 0, lo, hi - lo, out, scratch, sq, False)
                        grp.barrier(2)                 # every owner's slice is folded (into `out`)
                        # owners publish their slice in place, then everyone pulls the others'
                        view[lo:hi].copy_(out[lo:hi])
                        grp.barrier(3)
                        for q in range(world):
                            if q != rank:
                                qlo, qhi = split_bounds(count // 4, world, q)
                                nxt = (ctypes.c_void_p * 8)(p2p.addrs[q] + 16 * qlo, *([None] * 7))
                                if qhi > qlo:
                                    call("pb_shard_gather", nxt, 0, (qhi - qlo) * 8,
                                         ptr(view[qlo * 4:]), 1, 0, 0, stream_ptr())

                    view.fill_(float(rank + 1))
                    torch.cuda.synchronize()
                    dist.barrier()
                    fold()
                    grp.barrier(0)
                    torch.cuda.synchronize()
                    wrong = int((view != world * (world + 1) / 2).sum().item())

                    def again():
                        view.fill_(float(rank + 1))     # inputs are consumed in place
                        fold()

                    us = timed(again)
                rows.setdefault(title, []).append((size, count, us, wrong))
                size *= a.factor
        torch.cuda.synchronize()
        grp.check()
    finally:
        if mc is not None:
            mc.close()
        p2p.close()
    if rank == 0:
        for title, items in rows.items():
            print(f"# own all-reduce: {title}")
            for size, count, us, wrong in items:
                alg = count * 4 / us / 1e3
                # comment rows: the nccl-tests parsers read NCCL's table only
                print(f"# {size:12d} {count:13d}     float     sum      -1 {us:9.2f} {alg:7.2f} {alg * scale:7.2f} {wrong:6d}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1 << 20)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--own", type=int, default=1, help="also time this package's own all-reduce kernels")
    a = ap.parse_args(argv)
    cuda = torch.cuda.is_available()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    if rank == 0:
        print(f"# nGpus {world} backend {'nccl' if cuda else 'gloo'} minBytes {a.min_bytes} maxBytes {a.max_bytes}")
        print("#       size         count      type   redop    root     time   algbw   busbw #wrong     time   algbw   busbw #wrong")
    size = a.min_bytes
    scale = 2.0 * (world - 1) / world if world > 1 else 1.0
    while size <= a.max_bytes:
        count = size // 4
        src = torch.full((count,), float(rank + 1), dtype=torch.float32, device=dev)
        out_us = _time_allreduce(src.clone(), a.iters, a.warmup, cuda)
        x = torch.full((count,), float(rank + 1), dtype=torch.float32, device=dev)
        dist.all_reduce(x)
        wrong = int((x != world * (world + 1) / 2).sum().item())
        in_us = _time_allreduce(x, a.iters, a.warmup, cuda)
        if rank == 0:
            row = []
            for us in (out_us, in_us):
                alg = size / us / 1e3          # GB/s
                row.append(f"{us:9.2f} {alg:7.2f} {alg * scale:7.2f} {wrong:6d}")
            print(f"{size:12d} {count:13d}     float     sum      -1 {row[0]} {row[1]}")
        size *= a.factor
    if rank == 0:
        print("# Out of bounds values : 0 OK")
    if cuda and world > 1 and a.own:
        _own_table(a, rank, world, dev, scale)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
