"""All-reduce bus-bandwidth table in the layout of nccl-tests, one rank per GPU.

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 8 \\
        -m prometheus_b200.parallel.allreduce_bench --max-bytes 1073741824

Rank 0 prints one row per size: ``size count type redop root time(us) algbw busbw #wrong``
(out of place, then in place), times taken on the device as the max over ranks, bus bandwidth
``= algbw * 2 (n - 1) / n``. With ``NCCL_DEBUG=INFO`` in the environment NCCL's own log shows
whether the in-switch (NVLS) algorithm was chosen. Falls back to gloo on machines without a
GPU, where the table is only a functional check. ``native.ncshare.parse_busbw_gbps`` reads the
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1 << 20)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
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
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
