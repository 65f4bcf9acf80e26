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

Rank 0 prints one JSON line. ``--impl reference`` reports whether the unmodified
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


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from prometheus_b200 import engine, model, train
    from prometheus_b200.ops import _lib

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

    model_name = MODEL_NAME
    trainer_kw = {}
    if args.config == "latent":
        args.seq_len = 1024 + 8 + 512
        if args.seqs_per_gpu == SEQS_PER_GPU:
            args.seqs_per_gpu = 8
        model_name += " + latent slots (prefix 1024 | K=8 | answer 512, 4 Jacobi sweeps)"
    if args.config == "longctx":
        # one sequence split over the ranks (context parallel), 16384 tokens per rank:
        # 8 ranks hold the 131072-token sequence of the long-context configuration
        args.seq_len = 16384 * world
        args.seqs_per_gpu = 1
        args.micro_batch = 1
        trainer_kw = dict(context_parallel=world > 1)
        model_name += f" at sequence length {args.seq_len} (context parallel over {world} rank(s))"
    cfg = model.config_dense_1p3b(max_context=args.seq_len)
    if args.config == "moe16b":
        cfg = model.with_overrides(model.config_moe_16b(), max_context=args.seq_len)
        if args.seqs_per_gpu == SEQS_PER_GPU:
            args.seqs_per_gpu = 8
        if args.micro_batch == 8:
            # top-6 routing keeps six expert-side copies of every token's activations per MoE
            # layer: 16384 tokens per micro-batch keep the 27 MoE layers' saved activations near 55 GB
            args.micro_batch = 4
        trainer_kw = dict(fp8=True, expert_parallel=world > 1)
        model_name = "moe-16B (28L d2048, 64 routed top-6 + 2 shared experts h1408, FP8 e4m3 block-scaled linears)"
    if args.layers:
        n_dense = 1 if args.config == "moe16b" else args.layers
        cfg = model.with_overrides(cfg, n_layers=args.layers, n_dense=n_dense, n_moe=args.layers - n_dense,
                                   n_linear_attn=args.layers * 3 // 4, n_mla=args.layers // 4,
                                   core_block_layers=args.layers)
    tcfg = train.train_config_for(cfg, warmup_steps=100, stable_steps=10_000, decay_steps=1000)
    torch.manual_seed(1234)
    tr = engine.Trainer(cfg, tcfg, seed=0, device=dev, micro_batch=args.micro_batch,
                        grad_sync=args.grad_sync, **trainer_kw)
    step_kw = {}
    if args.config == "latent":
        tr.set_latent_slots(1024, 8, 4)
        mask = torch.ones(args.seqs_per_gpu, args.seq_len, device=dev)
        mask[:, 1024:1032] = 0
        step_kw = dict(loss_mask=mask)

    B, S = args.seqs_per_gpu, args.seq_len
    cp = args.config == "longctx"
    gen = torch.Generator().manual_seed(1000 + (0 if cp else rank))     # CP ranks slice the same sequence
    n_batches = args.steps + args.warmup
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, S), generator=gen, dtype=torch.int64)
                   for _ in range(min(n_batches, 4))]
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

    for i in range(args.warmup):
        tr.step(dev_tokens[i % len(dev_tokens)], **kw_for(i))
    sync_all()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        out = tr.step(dev_tokens[i % len(dev_tokens)], **kw_for(i))
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    launches = _lib.launch_count - launches0
    last_loss = float(out["loss"].item())

    # end to end through the public API: pinned host tokens in, loss value out, every step
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    e2e_loss = 0.0
    for i in range(args.steps):
        hkw = kw_for(i, host=True)
        res = tr.step_from_host(host_tokens[i % len(host_tokens)],
                                *([hkw["loss_mask"] if hkw["loss_mask"].device.type == "cpu"
                                   else hkw["loss_mask"].cpu().pin_memory()] if hkw else []))
        e2e_loss = res["loss"]
    f1.record()
    sync_all()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else {}

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    tokens_per_step = B * S * (1 if cp else world)
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded uniform tokens, random-init weights)",
            "config": {
                "model": model_name if not args.layers else f"DEBUG {args.layers} layers",
                "global_batch": B * (1 if cp else world), "seq_len": S,
                "parallelism": (f"cp{world}" if cp else f"dp{world}" + ("+ep" + str(world) if args.config == "moe16b" else ""))
                if world > 1 else "single",
                "micro_batch": args.micro_batch, "grad_sync": args.grad_sync,
                "l2": "per-step working set (3.5 GB bf16 weights + activations) exceeds the 126 MB L2",
            },
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                       "reasons": clocks.get("reasons", [])},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(host_tokens[0].numel() * 8 + (host_masks[0].numel() * 4 if host_masks else 0)),
                    "d2h_bytes_per_step": 8},
            "gpu_launches": launches,
            "loss": last_loss, "e2e_loss": e2e_loss, "impl": "ours",
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
