"""Multi-GPU micro-benchmarks of the fused compute + collective paths (run under torchrun).

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node N \\
        -m prometheus_b200.parallel.microbench [--only reduce|bcast|ag_gemm|ep|cp]

Every number is device-timed with CUDA events after warm-up, the max over ranks, and is set
against the roofline of its path: the slower of (FLOPs / measured GEMM rate) and (bytes that
cross NVLink per GPU / link bandwidth). Link bandwidth: the measured 770 GB/s per direction per
GPU (900 nominal); GEMM rate: ``MEASURED_PEAKS.json`` when present. Rank 0 prints one JSON line
per path.

    reduce   gradient reduce-to-owner (rank-ordered fp32 fold of every peer's slice, sum of
             squares on the fly)                                              [F2, first half]
    bcast    Muon update + bf16 refresh stored into every peer               [F2, second half]
    ag_gemm  all-gather fused into the consuming GEMM                         [F1]
    ep       expert-parallel MoE FFN: route, dispatch (peer stores), grouped GEMMs, combine (peer
             loads), forward + backward                                      [F3]
    cp       delta-rule state hand-off (push + bounded wait + compose)        [F4]
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NOMINAL_LINK_GBS = 900.0  # NVLink 5 per direction per GPU
_link_gbs: float | None = None


def link_gbs(dev=None) -> float:
    """Peer bandwidth per direction per GPU, measured once per process: every rank pulls 256 MiB
    from its next rank's symmetric buffer with 16-byte loads (the gather kernel of the ZeRO-3
    path), CUDA events, minimum over the ranks. It is the denominator of every link-bound
    roofline below; the nominal figure is only the fallback when the measurement cannot run."""
    global _link_gbs
    if _link_gbs is not None:
        return _link_gbs
    try:
        import ctypes

        from ..ops import _lib
        from ..ops._lib import call, ptr, stream_ptr
        from .symm import SymmetricBuffer

        _lib.register("pb_shard_gather", [ctypes.POINTER(ctypes.c_void_p), ctypes.c_long, ctypes.c_long,
                                          ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_void_p])
        world, rank = dist.get_world_size(), dist.get_rank()
        n = 128 * 1024 * 1024                                   # bf16 elements = 256 MiB
        buf = SymmetricBuffer(2 * n)
        dst = torch.empty(n, dtype=torch.bfloat16, device=buf.bytes.device)
        nxt = (ctypes.c_void_p * 8)(buf.addrs[(rank + 1) % world], *([None] * 7))
        run = lambda: call("pb_shard_gather", nxt, 0, n, ptr(dst), 1, 0, 0, stream_ptr())  # noqa: E731
        ms = timed(run, buf.bytes.device, iters=5, warmup=2)
        _link_gbs = 2.0 * n / (ms * 1e-3) / 1e9
        buf.close()
    except Exception:       # no peer mapping on this machine
        _link_gbs = NOMINAL_LINK_GBS
    return _link_gbs


def _peaks() -> dict:
    from ..ops.microbench import peaks

    return peaks()


def timed(fn, dev, iters: int = 10, warmup: int = 3) -> float:
    """Milliseconds per call, max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def roofline(ms: float, flops: float, link_bytes: float) -> dict:
    t_compute = flops / (_peaks()["bf16_tflops"] * 1e12) * 1e3
    t_link = link_bytes / (link_gbs() * 1e9) * 1e3
    bound = max(t_compute, t_link)
    return {"ms": ms, "roofline_ms": bound, "bound_by": "compute" if t_compute >= t_link else "link",
            "fraction_of_roofline": bound / ms if ms > 0 else 0.0}


def bench_reduce(dev, rank, world, a):
    from ..ops._lib import query
    from .symm import SymmetricBuffer, SymmetricGroup

    n = a.elements // world * world
    grp = SymmetricGroup(wait_budget_s=10.0)
    buf = SymmetricBuffer(4 * n)
    buf.view(torch.float32, n).normal_()
    lo, cnt = rank * (n // world), n // world
    out = torch.zeros(n, device=dev)
    scratch = torch.empty(max(4096, query("pb_reduce_nparts", cnt)), device=dev)
    sq = torch.zeros(1, device=dev)

    def step():
        grp.barrier(0)
        grp.reduce_to_owner(buf, 0, lo, cnt, out, scratch, sq, False)

    ms = timed(step, dev, a.iters)
    grp.check()
    link = 4.0 * cnt * (world - 1)                 # bytes this GPU pulls from its peers
    res = {"path": "reduce_to_owner", "world": world, "elements": n, "link_bytes_per_gpu": link,
           "achieved_link_gbs": link / ms / 1e6, **roofline(ms, 0.0, link)}
    buf.close()
    return res


def bench_bcast(dev, rank, world, a):
    from ..ops._lib import call, ptr, stream_ptr
    from .symm import SymmetricBuffer, SymmetricGroup

    n = a.elements // world * world
    grp = SymmetricGroup(wait_budget_s=10.0)
    lp = SymmetricBuffer(2 * n)
    cnt = n // world
    master = torch.randn(n, device=dev)
    upd = torch.randn(cnt, device=dev).to(torch.bfloat16)
    ptrs = lp.peer_ptrs(0)

    def step():
        grp.barrier(0)
        call("pb_muon_apply_bcast", ptr(master), ptr(upd), ptrs, world, rank * cnt, cnt, 1e-3, 0.2, 0.0,
             stream_ptr())

    ms = timed(step, dev, a.iters)
    grp.check()
    link = 2.0 * cnt * (world - 1)                 # bf16 stores this GPU sends to its peers
    res = {"path": "muon_apply_bcast", "world": world, "elements": n, "link_bytes_per_gpu": link,
           "achieved_link_gbs": link / ms / 1e6, **roofline(ms, 0.0, link)}
    lp.close()
    return res


def bench_ag_gemm(dev, rank, world, a):
    from ..ops import functional as ops
    from .fsdp import AgWeight

    M, N, K = a.m, a.n, a.k
    agw = AgWeight(N, K, wait_budget_s=10.0)
    agw.shard.normal_(0, 0.02)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    ms = timed(lambda: agw.linear(x), dev, a.iters)
    ms_plain = timed(lambda: ops.gemm(x, agw.full), dev, a.iters)
    gathered = [torch.empty_like(agw.shard) for _ in range(world)]
    ms_nccl = timed(lambda: (dist.all_gather(gathered, agw.shard), ops.gemm(x, agw.full)), dev, a.iters)
    agw.sym.check()
    link = 2.0 * N * K * (world - 1) / world
    res = {"path": "all_gather_gemm", "world": world, "m": M, "n": N, "k": K, "plain_gemm_ms": ms_plain,
           "nccl_all_gather_plus_gemm_ms": ms_nccl, "link_bytes_per_gpu": link,
           "tflops": 2.0 * M * N * K / ms / 1e9, **roofline(ms, 2.0 * M * N * K, link)}
    agw.close()
    return res


def bench_ep(dev, rank, world, a):
    from .ep import EpContext, ep_moe_ffn
    from .symm import SymmetricGroup

    T, d, E, h, k = a.tokens, 2048, 8 * world, 1408, 6
    El = E // world
    g = torch.Generator(device=dev).manual_seed(0)
    r = lambda *s, sc: (torch.randn(*s, device=dev, generator=g) * sc).to(torch.bfloat16)
    rw = r(E, d, sc=0.02).requires_grad_(True)
    wgu = r(El, 2 * h, d, sc=0.02).requires_grad_(True)
    wd = r(El, d, h, sc=0.02).requires_grad_(True)
    x = torch.randn(T, d, device=dev, generator=torch.Generator(device=dev).manual_seed(1 + rank)).to(torch.bfloat16)
    x.requires_grad_(True)
    go = torch.randn(T, d, device=dev).to(torch.bfloat16)
    grp = SymmetricGroup(wait_budget_s=10.0)
    ep = EpContext(grp, d, E, max_rows=int(2.0 * T * k) + El * 128)

    res = {"path": "ep_moe_ffn", "world": world, "tokens_per_rank": T, "experts": E, "top_k": k}
    flops = 2.0 * T * k * 3 * d * h                # per rank (balanced routing)
    remote = (world - 1) / world
    for fp8 in (False, True):
        def fwd():
            with torch.no_grad():
                ep_moe_ffn(x, rw, None, wgu, wd, k, ep, fp8=fp8)

        def both():
            for t_ in (x, rw, wgu, wd):
                t_.grad = None
            out, _, _ = ep_moe_ffn(x, rw, None, wgu, wd, k, ep, fp8=fp8)
            out.backward(go)

        ms_f, ms_b = timed(fwd, dev, a.iters), timed(both, dev, a.iters)
        grp.check()
        if a.profile and rank == 0:
            # kernel shares of one forward + backward (diagnosis only: timings taken under the
            # profiler are not reported as results)
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                both()
                torch.cuda.synchronize()
            print(("fp8_wire" if fp8 else "bf16_wire") + " kernel shares\n"
                  + prof.key_averages().table(sort_by="cuda_time_total", row_limit=24, max_name_column_width=60),
                  flush=True)
        if a.profile and rank != 0:
            both()          # the other ranks run the same collective layer while rank 0 is profiled
            torch.cuda.synchronize()
        # bytes crossing NVLink per rank: dispatch out (bf16, or e4m3 + one fp32 scale per 128)
        # + combine back (bf16); the backward moves bf16 both ways
        out_b = T * k * d * ((1.0 + 4.0 / 128) if fp8 else 2.0) * remote
        back_b = T * k * d * 2.0 * remote
        tag = "fp8_wire" if fp8 else "bf16_wire"
        res[tag] = {"fwd": {"tflops": flops / ms_f / 1e9, **roofline(ms_f, flops, out_b + back_b)},
                    "fwd_bwd": {"tflops": 3 * flops / ms_b / 1e9,
                                **roofline(ms_b, 3 * flops, out_b + 3 * back_b)}}
    return res


def bench_cp(dev, rank, world, a):
    from .cp import DeltaCpContext

    bh = a.states
    cp = DeltaCpContext(bh, wait_budget_s=10.0)
    p = torch.randn(bh, 128, 128, device=dev) * 0.05
    r = torch.randn(bh, 128, 128, device=dev)
    ms = timed(lambda: cp.handoff(p, r), dev, a.iters)
    cp.check()
    link = 2.0 * bh * 128 * 128 * 4 * (world - 1)   # the last rank receives every earlier rank's (P, R)
    res = {"path": "cp_state_handoff", "world": world, "states": bh, "link_bytes_worst_gpu": link,
           "exposed_us": ms * 1e3, **roofline(ms, 2.0 * bh * (world - 1) * 2 * 128 ** 3 / 60.0, link)}
    cp.close()
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--elements", type=int, default=256 * 1024 * 1024, help="fp32 gradient elements (reduce / bcast)")
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--states", type=int, default=16)
    ap.add_argument("--profile", action="store_true", help="print kernel shares of the EP layer (rank 0)")
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from datetime import timedelta

    dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=120))
    table = {"reduce": bench_reduce, "bcast": bench_bcast, "ag_gemm": bench_ag_gemm, "ep": bench_ep, "cp": bench_cp}
    for name, fn in table.items():
        if a.only and a.only != name:
            continue
        res = fn(dev, rank, world, a)
        if rank == 0:
            print(json.dumps(res), flush=True)
        dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
