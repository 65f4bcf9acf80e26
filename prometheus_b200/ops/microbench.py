"""Per-kernel micro-benchmarks (CUDA-event timed, L2 flushed between iterations).

    python -m prometheus_b200.ops.microbench gemm --m 16384 --n 2048 --k 2048
    python -m prometheus_b200.ops.microbench delta --seqs 32 --seq-len 4096
    python -m prometheus_b200.ops.microbench rmsnorm --rows 131072 --d 2048
    python -m prometheus_b200.ops.microbench ce --rows 4096 --vocab 131072
    python -m prometheus_b200.ops.microbench attn --batch 8 --seq-len 4096
    python -m prometheus_b200.ops.microbench elementwise --rows 32768 [--only rope]

Each prints one JSON line with the achieved rate and its fraction of the measured peak
(``MEASURED_PEAKS.json`` at the repository root when present, else the stated fallback).
Used for the roofline lines in ``profiles/`` and as the small case for ``ncu`` captures.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

BF16 = torch.bfloat16


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


def timeit(fn, iters=10, warmup=3, flush=True) -> float:
    """Median milliseconds per call; a 256 MB write between calls evicts the 126 MB L2."""
    junk = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if junk is not None:
            junk.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(a):
    from . import functional as ops

    if a.debug:
        from ._lib import call

        call("pb_gemm_set_variant", a.debug)
    x = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device="cuda").to(BF16)
    w = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device="cuda").to(BF16)
    ms = timeit(lambda: ops.gemm(x, w, a_mn=a.a_mn, b_mn=a.b_mn), a.iters)
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    out = {"kernel": "gemm_bf16", "m": a.m, "n": a.n, "k": a.k, "a_mn": a.a_mn, "b_mn": a.b_mn,
           "ms": ms, "tflops": tf, "frac_of_peak": tf / peaks()["bf16_tflops"]}
    if a.compare:
        xr = x.t() if a.a_mn else x
        wr = w if a.b_mn else w.t()
        ms_l = timeit(lambda: xr @ wr, a.iters)
        out["library_ms"] = ms_l
        out["library_tflops"] = 2.0 * a.m * a.n * a.k / ms_l / 1e9
    if a.sustain > 0:
        # steady state under the power cap: each variant runs back to back for `sustain` seconds
        # while NVML is polled for the SM clock and the board power (read-only queries)
        import threading
        import time

        import pynvml

        from ._lib import call

        pynvml.nvmlInit()
        hdl = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        xr = x.t() if a.a_mn else x
        wr = w if a.b_mn else w.t()
        runs = [("library", None)] + [(f"variant={v}", int(v)) for v in (a.variants or "0").split(",")]
        out["sustained"] = {}
        for name, flag in runs:
            if flag is not None:
                call("pb_gemm_set_variant", flag)
            fn = (lambda: xr @ wr) if flag is None else (lambda: ops.gemm(x, w, a_mn=a.a_mn, b_mn=a.b_mn))
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            samples, stop = [], threading.Event()

            def poll():
                while not stop.is_set():
                    samples.append((pynvml.nvmlDeviceGetClockInfo(hdl, pynvml.NVML_CLOCK_SM),
                                    pynvml.nvmlDeviceGetPowerUsage(hdl) / 1000.0))
                    time.sleep(0.02)

            th = threading.Thread(target=poll)
            th.start()
            n, t0 = 0, time.perf_counter()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            while time.perf_counter() - t0 < a.sustain:
                for _ in range(50):
                    fn()
                n += 50
                torch.cuda.synchronize()
            e1.record()
            torch.cuda.synchronize()
            stop.set()
            th.join()
            ms_s = e0.elapsed_time(e1) / n
            clk = sorted(c for c, _ in samples[len(samples) // 4:])
            pw = sorted(w_ for _, w_ in samples[len(samples) // 4:])
            out["sustained"][name] = {"tflops": round(2.0 * a.m * a.n * a.k / ms_s / 1e9, 1),
                                      "sm_mhz_median": clk[len(clk) // 2] if clk else None,
                                      "watts_median": round(pw[len(pw) // 2], 1) if pw else None}
        call("pb_gemm_set_variant", a.debug)
        return out
    if a.variants:
        # the same product under several pb_gemm_set_variant values, timed in this process one after
        # the other (same GPU, same clocks): 0 = default dispatch, 8 = single-CTA kernel only
        from ._lib import call

        out["variants_tflops"] = {}
        for rep in range(2):
            for flag in [int(v) for v in a.variants.split(",")]:
                call("pb_gemm_set_variant", flag)
                ms_v = timeit(lambda: ops.gemm(x, w, a_mn=a.a_mn, b_mn=a.b_mn), a.iters)
                out["variants_tflops"].setdefault(str(flag), []).append(round(2.0 * a.m * a.n * a.k / ms_v / 1e9, 1))
        call("pb_gemm_set_variant", a.debug)
    return out


def bench_fp8(a):
    from . import fp8

    x = torch.randn((a.m, a.k), device="cuda").to(BF16)
    w = (torch.randn((a.n, a.k), device="cuda") * 0.05).to(BF16)
    xq, sx = fp8.quantize_rows(x)
    wq, sw = fp8.quantize_blocks(w)
    ms = timeit(lambda: fp8.gemm_fp8(xq, sx, wq, sw), a.iters)
    ms_q = timeit(lambda: fp8.quantize_rows(x), a.iters)
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    out = {"kernel": "gemm_fp8_blockscaled", "m": a.m, "n": a.n, "k": a.k, "ms": ms, "tflops": tf,
           "vs_bf16_peak": tf / peaks()["bf16_tflops"], "quant_rows_ms": ms_q,
           "quant_rows_gbs": (a.m * a.k * 3 + a.m * a.k // 32) / ms_q / 1e6}
    if a.probes:
        # Parts of the kernel timed alone (debug build of the library: PB200_DEBUG_BOUNDS=1).
        # Their outputs are not products; only the times mean something.
        from ._lib import call, ptr, stream_ptr
        from .functional import status_word

        c = torch.empty((a.m, a.n), dtype=BF16, device="cuda")
        names = {1: "no_promotion", 2: "accumulate_in_place", 3: "fma_only", 4: "tmem_loads_only"}
        for probe, name in names.items():
            t = timeit(lambda: call("pb_gemm_fp8_probe", ptr(xq), ptr(sx), ptr(wq), ptr(sw), ptr(c), a.m, a.n, a.k, a.n,
                                    probe, ptr(status_word(x.device)), stream_ptr()), a.iters)
            out[f"probe_{name}_ms"] = t
            out[f"probe_{name}_tflops"] = 2.0 * a.m * a.n * a.k / t / 1e9
    return out


def bench_moe(a):
    """One MoE FFN layer (router, placement, grouped GEMMs, combine), forward + backward."""
    from . import moe

    T, d, E, h, k = a.tokens, a.d, a.experts, a.hidden, a.top_k
    x = torch.randn(T, d, device="cuda").to(BF16).requires_grad_(True)
    rw = (torch.randn(E, d, device="cuda") * 0.02).to(BF16).requires_grad_(True)
    wgu = (torch.randn(E, 2 * h, d, device="cuda") * 0.02).to(BF16).requires_grad_(True)
    wd = (torch.randn(E, d, h, device="cuda") * 0.02).to(BF16).requires_grad_(True)
    go = torch.randn(T, d, device="cuda").to(BF16)

    def fwd():
        return moe.moe_ffn(x, rw, None, wgu, wd, k)[0]

    def both():
        for t in (x, rw, wgu, wd):
            t.grad = None
        fwd().backward(go)

    ms_f = timeit(fwd, a.iters)
    ms_b = timeit(both, a.iters)
    flops = 2.0 * T * k * 3 * d * h
    return {"kernel": "moe_ffn", "tokens": T, "experts": E, "top_k": k, "d": d, "hidden": h,
            "fwd_ms": ms_f, "fwd_bwd_ms": ms_b, "fwd_tflops": flops / ms_f / 1e9,
            "fwd_bwd_tflops": 3 * flops / ms_b / 1e9, "peaks": peaks()}


def bench_delta(a):
    from .. import kernels

    B, S, H, D = a.seqs, a.seq_len, 16, 128
    q = torch.nn.functional.normalize(torch.randn(B, S, H, D, device="cuda"), dim=-1).to(BF16)
    k = torch.nn.functional.normalize(torch.randn(B, S, H, D, device="cuda"), dim=-1).to(BF16)
    v = torch.randn(B, S, H, D, device="cuda").to(BF16)
    beta = torch.rand(B, S, H, device="cuda").to(BF16)
    leaves = [t.requires_grad_(True) for t in (q, k, v, beta)]
    go = torch.randn(B, S, H, D, device="cuda").to(BF16)

    from .delta import delta_rule_fused, scan_segments

    seg = a.segments if a.segments else scan_segments(B * H, S // 64)

    def fwd():
        with torch.no_grad():
            delta_rule_fused(q, k, v, beta, None, n_seg=seg)

    def fwdbwd():
        o, _ = delta_rule_fused(*leaves, None, n_seg=seg)
        o.backward(go)

    if a.once:                       # one call of each, for a profiler capture of a small case
        fwdbwd()
        torch.cuda.synchronize()
        return {"kernel": "delta_rule", "seqs": B, "seq_len": S, "segments": seg, "once": True}
    ms_f, ms_fb = timeit(fwd, a.iters), timeit(fwdbwd, a.iters)
    chunks = B * H * S // 64
    flops_scan = chunks * 2.0 * (3 * 64 * 128 * 128 + 64 * 64 * 128)
    return {"kernel": "delta_rule", "seqs": B, "seq_len": S, "heads": H, "segments": seg, "fwd_ms": ms_f,
            "fwd_bwd_ms": ms_fb, "scan_fwd_tflops_if_all_scan": flops_scan / ms_f / 1e9}


def bench_rmsnorm(a):
    from . import functional as ops

    x = torch.randn(a.rows, a.d, device="cuda").to(BF16)
    r = torch.randn(a.rows, a.d, device="cuda").to(BF16)
    w = torch.ones(a.d, device="cuda")
    ms = timeit(lambda: ops.add_rmsnorm(x, r, w), a.iters)
    gbs = 4 * a.rows * a.d * 2 / ms / 1e6
    return {"kernel": "add_rmsnorm_fwd", "rows": a.rows, "d": a.d, "ms": ms, "gbs": gbs,
            "frac_of_peak": gbs / peaks()["hbm_gbs"]}


def bench_ce(a):
    from ._lib import call, ptr, stream_ptr

    logits = torch.randn(a.rows, a.vocab, device="cuda").to(BF16)
    tgt = torch.randint(0, a.vocab, (a.rows,), device="cuda", dtype=torch.int32)
    wt = torch.full((a.rows,), 1.0 / a.rows, device="cuda")
    loss = torch.empty(a.rows, device="cuda")
    ms = timeit(lambda: call("pb_softcap_ce", ptr(logits), ptr(tgt), ptr(wt), ptr(loss), None,
                             a.rows, a.vocab, 30.0, 1, stream_ptr()), a.iters)
    gbs = 2 * a.rows * a.vocab * 2 / ms / 1e6
    return {"kernel": "softcap_ce", "rows": a.rows, "vocab": a.vocab, "ms": ms, "gbs": gbs,
            "frac_of_peak": gbs / peaks()["hbm_gbs"]}


def bench_elementwise(a):
    """Every HBM-bound kernel of the training step on the 1.3B shapes: achieved bytes / time
    against the measured copy bandwidth. Bytes are the algorithmic minimum (each input read once,
    each output written once)."""
    from . import fp8, moe
    from . import functional as ops
    from . import latent as LK
    from ._lib import call, ptr, stream_ptr

    rows, d, hid = a.rows, 2048, 5632
    peak = peaks()["hbm_gbs"]
    out = {"kernel": "elementwise_suite", "rows": rows, "results": {}}

    def add(name, nbytes, fn, only=None):
        if a.only and a.only != name:
            return
        ms = timeit(fn, a.iters)
        gbs = nbytes / ms / 1e6
        out["results"][name] = {"ms": ms, "gbs": gbs, "frac_of_measured_copy": gbs / peak}

    x = torch.randn(rows, d, device="cuda").to(BF16)
    r = torch.randn(rows, d, device="cuda").to(BF16)
    w = torch.ones(d, device="cuda")
    add("add_rmsnorm_fwd", 4 * rows * d * 2, lambda: ops.add_rmsnorm(x, r, w))
    xg = x.clone().requires_grad_(True)
    y = ops.rmsnorm(xg, w)
    gy = torch.randn_like(y)
    add("rmsnorm_bwd", 3 * rows * d * 2, lambda: torch.autograd.grad(y, xg, gy, retain_graph=True))
    gu = torch.randn(rows, 2 * hid, device="cuda").to(BF16)
    add("swiglu_fwd", 3 * rows * hid * 2, lambda: ops.swiglu(gu))
    gug = gu.clone().requires_grad_(True)
    sy = ops.swiglu(gug)
    gs = torch.randn_like(sy)
    add("swiglu_bwd", 5 * rows * hid * 2, lambda: torch.autograd.grad(sy, gug, gs, retain_graph=True))
    S = 4096
    q = torch.randn(rows // S, S, 16, 128, device="cuda").to(BF16)
    # the forms the trainer calls: written over the projection output, no copy
    q2 = q.reshape(rows, d)
    with torch.no_grad():
        add("rope", 2 * rows * d * 2, lambda: ops.rope2d_(q2, 16, seq_len=S))
        add("l2norm_fwd", 2 * rows * d * 2 + rows * 16 * 4, lambda: ops.l2norm_(q2, 128))
        xn = torch.nn.functional.normalize(torch.randn(rows, d, device="cuda").view(rows, 16, 128), dim=-1)
        xn = xn.reshape(rows, d).to(BF16)
        inv = torch.ones(rows * 16, device="cuda")
        gq = torch.randn(rows, d, device="cuda").to(BF16)
        add("l2norm_bwd", 3 * rows * d * 2 + rows * 16 * 4,
            lambda: call("pb_l2norm_bwd", ptr(gq), ptr(xn), ptr(inv), rows * 16, 128, stream_ptr()))
    add("fp8_quant_rows", rows * d * 3 + rows * d // 32, lambda: fp8.quantize_rows(x))
    wq = torch.randn(hid, d, device="cuda").to(BF16)
    add("fp8_quant_blocks", hid * d * 3, lambda: fp8.quantize_blocks(wq))
    E, k = 64, 6
    rw = (torch.randn(E, d, device="cuda") * 0.02).to(BF16)
    logits = ops.gemm(x, rw).float()
    add("moe_route", 2 * rows * E * 4 + rows * k * 8, lambda: moe.route(logits, None, k))
    vocab, ce_rows = 131072, min(rows, 4096)
    lg = torch.randn(ce_rows, vocab, device="cuda").to(BF16)
    tgt = torch.randint(0, vocab, (ce_rows,), device="cuda", dtype=torch.int32)
    wt = torch.full((ce_rows,), 1.0 / ce_rows, device="cuda")
    loss = torch.empty(ce_rows, device="cuda")
    add("softcap_ce_fwd_bwd", 2 * ce_rows * vocab * 2,
        lambda: call("pb_softcap_ce", ptr(lg), ptr(tgt), ptr(wt), ptr(loss), None, ce_rows, vocab, 30.0, 1,
                     stream_ptr()))
    B, Sl, K = 64, 1544, 8
    hidden = torch.randn(B, Sl, d, device="cuda").to(BF16)
    emb = torch.randn(B, Sl, d, device="cuda").to(BF16)
    w1 = (torch.randn(d, d, device="cuda") * 0.02).to(BF16)
    w2 = (torch.randn(d, d, device="cuda") * 0.02).to(BF16)
    with torch.no_grad():
        add("latent_jacobi_step", 2 * B * Sl * d * 2, lambda: LK.jacobi_step(hidden, emb, w1, w2, w, 1024, K))
    return out


def bench_attn(a):
    """Causal GQA attention, forward and forward+backward, against the library kernel PyTorch
    dispatches to for the same call."""
    import torch.nn.functional as F

    from . import attention

    q = torch.randn(a.batch, a.seq_len, a.heads, 128, device="cuda").to(BF16).requires_grad_()
    k = torch.randn(a.batch, a.seq_len, a.kv_heads, 128, device="cuda").to(BF16).requires_grad_()
    v = torch.randn(a.batch, a.seq_len, a.kv_heads, 128, device="cuda").to(BF16).requires_grad_()
    go = torch.randn_like(q)

    def ours(bwd):
        o = attention.causal_gqa(q, k, v)
        if bwd:
            torch.autograd.grad(o, (q, k, v), go)

    def lib(bwd):
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=True, enable_gqa=True)
        if bwd:
            torch.autograd.grad(o, (q, k, v), go.transpose(1, 2))

    if a.once:      # one forward + backward of our kernels and nothing else: the ncu small case
        ours(True)
        torch.cuda.synchronize()
        return {"kernel": "attn_causal_gqa", "once": True}
    flops_fwd = 2 * 2 * a.batch * a.heads * a.seq_len * a.seq_len * 128 / 2   # causal half
    out = {"kernel": "attn_causal_gqa", "batch": a.batch, "seq_len": a.seq_len, "heads": a.heads,
           "kv_heads": a.kv_heads}
    for name, fn in (("ours", ours), ("sdpa", lib)):
        f = timeit(lambda: fn(False), a.iters)
        fb = timeit(lambda: fn(True), a.iters)
        out[name] = {"fwd_ms": f, "fwd_tflops": flops_fwd / f / 1e9, "fwd_bwd_ms": fb,
                     "fwd_bwd_tflops": 3.5 * flops_fwd / fb / 1e9}
    out["frac_of_peak_fwd"] = out["ours"]["fwd_tflops"] / peaks()["bf16_tflops"]
    return out


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="which", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192)
    g.add_argument("--a-mn", action="store_true")
    g.add_argument("--b-mn", action="store_true")
    g.add_argument("--compare", action="store_true")
    g.add_argument("--debug", type=int, default=0, help="kernel variant bits, see pb_gemm_set_variant")
    g.add_argument("--sustain", type=float, default=0.0,
                   help="seconds per variant of back-to-back launches with NVML clock / power polling")
    g.add_argument("--variants", default="", help="comma-separated pb_gemm_set_variant values to time side by side")
    d = sub.add_parser("delta")
    f = sub.add_parser("fp8")
    f.add_argument("--m", type=int, default=8192)
    f.add_argument("--n", type=int, default=8192)
    f.add_argument("--k", type=int, default=8192)
    f.add_argument("--probes", action="store_true",
                   help="also time the kernel's parts alone (needs PB200_DEBUG_BOUNDS=1: the debug build)")
    mo = sub.add_parser("moe")
    mo.add_argument("--tokens", type=int, default=32768)
    mo.add_argument("--experts", type=int, default=8)
    mo.add_argument("--top-k", type=int, default=6)
    mo.add_argument("--d", type=int, default=2048)
    mo.add_argument("--hidden", type=int, default=1408)
    d.add_argument("--seqs", type=int, default=4)
    d.add_argument("--seq-len", type=int, default=4096)
    d.add_argument("--segments", type=int, default=0, help="segments per sequence of the state walk (0: automatic)")
    d.add_argument("--once", action="store_true")
    r = sub.add_parser("rmsnorm")
    r.add_argument("--rows", type=int, default=131072)
    r.add_argument("--d", type=int, default=2048)
    c = sub.add_parser("ce")
    c.add_argument("--rows", type=int, default=4096)
    c.add_argument("--vocab", type=int, default=131072)
    el = sub.add_parser("elementwise")
    el.add_argument("--rows", type=int, default=32768)
    el.add_argument("--only", default="")
    at = sub.add_parser("attn")
    at.add_argument("--batch", type=int, default=8)
    at.add_argument("--seq-len", type=int, default=4096)
    at.add_argument("--heads", type=int, default=16)
    at.add_argument("--kv-heads", type=int, default=4)
    at.add_argument("--once", action="store_true")
    for s in (g, d, r, c, f, mo, at, el):
        s.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    out = {"gemm": bench_gemm, "delta": bench_delta, "rmsnorm": bench_rmsnorm, "ce": bench_ce,
           "fp8": bench_fp8, "moe": bench_moe, "attn": bench_attn,
           "elementwise": bench_elementwise}[a.which](a)
    out["peaks"] = peaks()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
