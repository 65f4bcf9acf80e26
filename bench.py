#!/usr/bin/env python
"""Headline benchmark: training throughput of the ~1.3B dense hybrid in bf16.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W      (N > 1)

Metric: train tokens/s over the whole job, device-timed with CUDA events, max over
ranks. Model: 24 layers, d_model 2048, delta-rule attention 16 x 128 (sigmoid beta,
L2-normed q/k), every 4th layer softmax GQA 16q/4kv + RoPE, SwiGLU 5632, vocab
131072, sequence 4096, Muon on matrices + AdamW on embeddings/norms. Weak scaling:
32 sequences per GPU per step (global batch 256 at 8 GPUs). Seeded synthetic
tokens, random-init weights. Every timed step is a full forward, backward,
gradient synchronisation and optimizer step.

Rank 0 prints one JSON line: the dense model's tokens/s as ``value`` with ``mfu`` (model FLOPs
against the measured cuBLAS bf16 rate) and ``exposed_comm_ms`` (step time minus the same steps
without peer traffic), and under ``secondary.moe16b`` the 16B FP8 expert-parallel
mixture-of-experts configuration measured in the same run where it fits in memory.
``--impl reference`` reports whether the unmodified
reference (JAX) can run the same metric on this machine.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "train tokens/sec/box (device-timed, max over ranks)"
MODEL_NAME = "hybrid-1.3B-dense (24L d2048 delta16x128+GQA16/4 SwiGLU5632 vocab131072)"
SEQ_LEN = 4096
SEQS_PER_GPU = 32


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (invalid as a result)")
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "p2p", "nccl"],
                    help="gradient path at N > 1: peer-memory reduce-to-owner + update-broadcast kernels "
                         "(auto / p2p, the product) or NCCL collectives only (the baseline)")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "dp", "fsdp"],
                    help="N > 1: fsdp (auto) = bf16 weights as 1/N shards gathered layer by layer, optimizer "
                         "state for owned matrices only; dp = replicated weights, ownership-sharded optimizer")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the 16B mixture-of-experts measurement that follows the dense one")
    ap.add_argument("--secondary-layers", type=int, default=0,
                    help="debug only: run the secondary measurement on a model cut to this many layers")
    ap.add_argument("--no-exposed", action="store_true",
                    help="skip the extra timed steps without peer traffic (exposed_comm_ms reads 0)")
    ap.add_argument("--config", default="dense", choices=["dense", "latent", "moe16b", "longctx"],
                    help="dense: the headline 1.3B hybrid (default). latent: the same model with 1024-token "
                         "prefix + 8 latent slots + 512-token answer, 4 Jacobi sweeps, 8 sequences per GPU. "
                         "moe16b: 28-layer 64-expert top-6 MoE with FP8 linears, expert parallel over the ranks.")
    return ap.parse_args()


def reference_arm(args) -> int:
    """The reference is JAX on a single device in fp32; it needs `jax`, which is not
    installed and cannot be installed offline."""
    ref = ROOT / "baseline" / "_ref"
    why = None
    if not ref.exists():
        why = "baseline/_ref not installed"
    else:
        sys.path.insert(0, str(ref))
        try:
            import jax  # noqa: F401
        except Exception as e:  # pragma: no cover - depends on the machine
            why = f"reference imports jax, which is not installed offline ({type(e).__name__}); " \
                  "its model also has no GQA/sigmoid-beta config at this shape"
    if why is None:
        why = ("reference model cannot instantiate this config (MLA only, beta=1, derived head "
               "geometry, fp32 single device)")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


def estimate_rank_bytes(cfg, world: int, expert_parallel: bool, tokens_per_micro: int) -> int:
    """Rough device bytes one rank needs to train ``cfg``: bf16 weight + fp32 gradient, master
    and one moment per parameter it holds, plus the saved activations of one micro-batch."""
    from prometheus_b200 import model

    shapes = model.init_params(cfg, 0, shapes_only=True)
    flat = model.flatten_params(shapes)
    held = 0
    for name, t in flat.items():
        n = int(t.numel())
        held += n // world if (expert_parallel and ".routed_" in name) else n
    # saved activations per layer, in units of one (tokens x d_model) bf16 tensor: about 20 for
    # a dense layer, 12 + 3 per routed slot for a mixture-of-experts layer
    act = tokens_per_micro * cfg.d_model * 2 * cfg.n_layers * ((12 + 3 * cfg.top_k) if cfg.n_moe else 20)
    return held * 14 + act


def measure(args, config: str, world: int, rank: int, local_rank: int, dev, steps: int, warmup: int,
            with_clocks: bool, with_exposed: bool) -> dict:
    """Build the trainer of one configuration and time it: ``steps`` device-timed steps, the
    same through the public host API, and (optionally) the steps again without peer traffic."""
    import torch
    import torch.distributed as dist

    from prometheus_b200 import engine, model, train
    from prometheus_b200.ops import _lib
    from prometheus_b200.utils import flops

    seq_len, seqs, micro = args.seq_len, args.seqs_per_gpu, args.micro_batch
    model_name = MODEL_NAME
    trainer_kw = {}
    sweeps = 1
    fsdp = world > 1 and args.parallelism in ("auto", "fsdp") and args.grad_sync != "nccl"
    if config == "latent":
        seq_len = 1024 + 8 + 512
        seqs = 8 if seqs == SEQS_PER_GPU else seqs
        sweeps = 4
        model_name += " + latent slots (prefix 1024 | K=8 | answer 512, 4 Jacobi sweeps)"
    if config == "longctx":
        # one sequence split over the ranks (context parallel), 16384 tokens per rank:
        # 8 ranks hold the 131072-token sequence of the long-context configuration
        seq_len, seqs, micro = 16384 * world, 1, 1
        trainer_kw = dict(context_parallel=world > 1)
        fsdp = False
        model_name += f" at sequence length {seq_len} (context parallel over {world} rank(s))"
    cfg = model.config_dense_1p3b(max_context=seq_len)
    if config == "moe16b":
        cfg = model.with_overrides(model.config_moe_16b(), max_context=seq_len)
        seqs = 8 if seqs == SEQS_PER_GPU else seqs
        # top-6 routing keeps six expert-side copies of every token's activations per MoE
        # layer: 16384 tokens per micro-batch keep the 27 MoE layers' saved activations near 55 GB
        micro = 4 if micro == 8 else micro
        # receive buffers sized for 1.5 x the balanced load (a layer that needs more latches an
        # overflow code, which the step reports)
        trainer_kw = dict(fp8=True, expert_parallel=world > 1, ep_capacity_factor=1.5)
        fsdp = fsdp and args.parallelism == "fsdp"
        model_name = "moe-16B (28L d2048, 64 routed top-6 + 2 shared experts h1408, FP8 e4m3 block-scaled linears)"
    cut = args.layers or (args.secondary_layers if config != args.config else 0)
    if cut:
        n_dense = 1 if config == "moe16b" else cut
        cfg = model.with_overrides(cfg, n_layers=cut, n_dense=n_dense, n_moe=cut - n_dense,
                                   n_linear_attn=cut * 3 // 4, n_mla=cut // 4, core_block_layers=cut)
    need = estimate_rank_bytes(cfg, world, config == "moe16b" and world > 1, micro * seq_len)
    free_b, total_b = torch.cuda.mem_get_info(dev)
    if need > 0.92 * total_b:
        return {"skipped": f"needs about {need / 2**30:.0f} GiB per rank at {world} GPU(s), "
                           f"the device has {total_b / 2**30:.0f} GiB", "bytes_needed_per_rank": int(need)}
    tcfg = train.train_config_for(cfg, warmup_steps=100, stable_steps=10_000, decay_steps=1000)
    torch.manual_seed(1234)
    tr = engine.Trainer(cfg, tcfg, seed=0, device=dev, micro_batch=micro, grad_sync=args.grad_sync,
                        fsdp=fsdp, **trainer_kw)
    step_kw = {}
    if config == "latent":
        tr.set_latent_slots(1024, 8, 4)
        mask = torch.ones(seqs, seq_len, device=dev)
        mask[:, 1024:1032] = 0
        step_kw = dict(loss_mask=mask)

    B, S = seqs, seq_len
    cp = config == "longctx"
    gen = torch.Generator().manual_seed(1000 + (0 if cp else rank))     # CP ranks slice the same sequence
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, S), generator=gen, dtype=torch.int64)
                   for _ in range(min(steps + warmup, 4))]
    host_masks = None
    if cp and world > 1:
        sliced = [tr.cp_slice(t, torch.ones(B, S)) for t in host_tokens]
        host_tokens = [a.contiguous() for a, _ in sliced]
        host_masks = [m.contiguous().pin_memory() for _, m in sliced]
    host_tokens = [t.pin_memory() for t in host_tokens]
    dev_tokens = [t.to(dev) for t in host_tokens]
    dev_masks = [m.to(dev) for m in host_masks] if host_masks else None

    def kw_for(i, host=False):
        if dev_masks is None:
            return step_kw
        return dict(loss_mask=(host_masks if host else dev_masks)[i % len(dev_masks)])

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n, fn):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = None
        for i in range(n):
            out = fn(i)
        e1.record()
        sync_all()
        return e0.elapsed_time(e1), out

    for i in range(warmup):
        tr.step(dev_tokens[i % len(dev_tokens)], **kw_for(i))
    sync_all()

    sampler = ClockSampler(local_rank)
    if rank == 0 and with_clocks:
        sampler.start()
    launches0 = _lib.launch_count
    ms, out = timed(steps, lambda i: tr.step(dev_tokens[i % len(dev_tokens)], **kw_for(i)))
    launches = _lib.launch_count - launches0
    last_loss = float(out["loss"].item())
    tr.raise_on_status(int(out["status"].item()))

    # end to end through the public API: pinned host tokens in, loss value out, every step
    def host_step(i):
        hkw = kw_for(i, host=True)
        extra = []
        if hkw:
            m = hkw["loss_mask"]
            extra = [m if m.device.type == "cpu" else m.cpu().pin_memory()]
        return tr.step_from_host(host_tokens[i % len(host_tokens)], *extra)

    ms_e2e, res = timed(steps, host_step)
    e2e_loss = res["loss"]
    clocks = sampler.stop() if (rank == 0 and with_clocks) else {}
    ms_noop = None
    if with_exposed and world > 1 and tr.sym is not None:
        # the same steps with the peer traffic of the gradient fold, the weight refresh and the
        # parameter gathers left out (the kernels' arithmetic and local memory traffic stay)
        tr.comm_noop = True
        tr.step(dev_tokens[0], **kw_for(0))
        ms_noop, _ = timed(steps, lambda i: tr.step(dev_tokens[i % len(dev_tokens)], **kw_for(i)))
        tr.comm_noop = False

    t = torch.tensor([ms, ms_e2e, ms_noop if ms_noop is not None else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_noop_max = float(t[0]), float(t[1]), float(t[2])
    tokens_per_step = B * S * (1 if cp else world)
    value = tokens_per_step * steps / (ms / 1e3)
    e2e_value = tokens_per_step * steps / (ms_e2e / 1e3)
    peaks = flops.measured_peaks()
    mem = tr.memory_report()
    par = "single"
    if world > 1:
        par = f"cp{world}" if cp else (f"fsdp{world}" if tr.fsdp else f"dp{world}")
        if config == "moe16b":
            par += f"+ep{world}"
    result = {
        "value": value, "ms_per_step": ms / steps,
        "mfu": flops.mfu(value, cfg, S, world, sweeps=sweeps),
        "mfu_of": f"{peaks['source']} cuBLAS bf16 burst {peaks['bf16_tflops']:.0f} TFLOP/s per GPU",
        "exposed_comm_ms": (max(0.0, (ms - ms_noop_max) / steps) if ms_noop is not None else 0.0),
        "config": {
            "model": model_name if not cut else f"DEBUG {cut} layers",
            "global_batch": B * (1 if cp else world), "seq_len": S, "parallelism": par,
            "micro_batch": micro, "grad_sync": args.grad_sync,
            "l2": f"per-step working set ({mem['weights_bf16_bytes'] / 2**30:.1f} GiB bf16 weights on "
                  f"this rank + activations) exceeds the 126 MB L2; no flush needed",
            "weights_plus_optimizer_bytes_per_rank": mem["weights_plus_state_bytes"],
        },
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                   "reasons": clocks.get("reasons", [])},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / steps,
                "h2d_bytes_per_step": int(host_tokens[0].numel() * 8 + (host_masks[0].numel() * 4 if host_masks else 0)),
                "d2h_bytes_per_step": 12},
        "gpu_launches": launches, "loss": last_loss, "e2e_loss": e2e_loss,
    }
    tr.close()
    del tr, dev_tokens, dev_masks
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return result


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"--gpus {args.gpus} needs torchrun with that many ranks", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    main_res = measure(args, args.config, world, rank, local_rank, dev, args.steps, args.warmup,
                       with_clocks=True, with_exposed=not args.no_exposed)
    if "skipped" in main_res:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": None, "n_gpus": world, "impl": "ours",
                              "unavailable": main_res["skipped"]}), flush=True)
        return 0
    secondary = {}
    if args.config == "dense" and not args.no_secondary and (not args.layers or args.secondary_layers):
        # the 16B FP8 mixture-of-experts configuration, expert parallel over the same ranks, in
        # the same run wherever it fits
        # a failure here (out of memory, a latched device status) must not cost the primary
        # measurement its line: it is reported under secondary.moe16b.error instead
        try:
            sec = measure(args, "moe16b", world, rank, local_rank, dev, max(2, min(args.steps, 3)), 3,
                          with_clocks=False, with_exposed=False)
        except Exception as e:          # noqa: BLE001
            sec = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        if "error" in sec:
            secondary["moe16b"] = {"value": None, "error": sec["error"]}
        elif "skipped" in sec:
            secondary["moe16b"] = {"value": None, "skipped": sec["skipped"],
                                   "bytes_needed_per_rank": sec["bytes_needed_per_rank"]}
        else:
            secondary["moe16b"] = {k: sec[k] for k in ("value", "ms_per_step", "mfu", "config",
                                                       "gpu_launches", "loss")}
            secondary["moe16b"]["unit"] = "tokens/s"
    if rank == 0:
        value = main_res["value"]
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": vs_baseline(value, world, args),
            "dtype": "bf16", "data": "synthetic (seeded uniform tokens, random-init weights)",
            "config": main_res["config"], "clocks": main_res["clocks"], "e2e": main_res["e2e"],
            "gpu_launches": main_res["gpu_launches"], "mfu": main_res["mfu"], "mfu_of": main_res["mfu_of"],
            "exposed_comm_ms": main_res["exposed_comm_ms"],
            "loss": main_res["loss"], "e2e_loss": main_res["e2e_loss"], "impl": "ours",
        }
        if secondary:
            line["secondary"] = secondary
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def vs_baseline(value: float, world: int, args):
    """value / the baseline number recorded for this GPU count. The reference publishes no
    throughput; the recorded baseline is this repository's own NCCL-only gradient path
    (``--grad-sync nccl``) on the same configuration, kept in ``baseline/nccl_only.json``."""
    if args.config != "dense" or args.layers:
        return None
    try:
        table = json.loads((ROOT / "baseline" / "nccl_only.json").read_text())
        base = table.get(str(world), {}).get("tokens_per_s")
        return value / base if base else None
    except Exception:
        return None


if __name__ == "__main__":
    sys.exit(main())
