"""Device timing helpers used by the benchmarks: CUDA-event intervals, an L2 flush, and the
maximum over ranks of a measured interval."""
from __future__ import annotations

import torch

L2_FLUSH_BYTES = 256 * 1024 * 1024      # larger than the 126 MB L2 of a B200


class L2Flush:
    """``flush()`` rewrites a buffer larger than the L2 so the next kernel starts cold."""

    def __init__(self, device="cuda", nbytes: int = L2_FLUSH_BYTES):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def flush(self) -> None:
        self.buf.fill_(1)


class CudaTimer:
    """``with CudaTimer() as t: ...`` then ``t.ms``: events on the current stream, synchronised on
    both sides."""

    def __enter__(self):
        torch.cuda.synchronize()
        self._e0, self._e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._e0.record()
        return self

    def __exit__(self, *exc):
        self._e1.record()
        torch.cuda.synchronize()
        self.ms = self._e0.elapsed_time(self._e1)
        return False


def median_ms(fn, iters: int = 10, warmup: int = 3, flush: L2Flush | None = None) -> float:
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.flush()
        with CudaTimer() as t:
            fn()
        times.append(t.ms)
    times.sort()
    return times[len(times) // 2]


def max_over_ranks(ms: float, device) -> float:
    """The slowest rank's interval (a multi-GPU number is the max over ranks, never wall clock)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
