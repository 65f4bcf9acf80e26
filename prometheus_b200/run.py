"""Training run loop and command line.

    python -m prometheus_b200.run --preset dense_1p3b --steps 100
    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 8 \\
        -m prometheus_b200.run --preset moe_16b --set fp8=true --set expert_parallel=true
    python -m prometheus_b200.run --preset tiny_fp32 --device cpu --steps 3

``--preset`` names one of the five shipped configurations, ``--set key=value`` overrides a field
of the model config, the train config or the run options (whichever has that name). The loop is
the wiring of the pieces that exist on their own elsewhere in the package:

* batches come from the native ``Loader`` (deterministic shuffle / pack / resume) as pinned host
  arrays, one step ahead of the device (the copy of step ``t + 1`` overlaps the compute of ``t``);
  the documents are seeded synthetic token streams of uneven length;
* steps run on ``engine.Trainer`` (GPU) or, for ``--device cpu``, on the fp32 ``train.train_step``;
* the loss goes to the native ``SpikeLog``: a spike rolls the trainer back to the last in-memory
  checkpoint and skips the offending batch, as the elastic controller prescribes;
* a ``supervisor.RunSupervisor`` holds the native ``Controller``, ``Tracer`` and ``MetricLog``:
  every phase of a step is a tracer span (and an NVTX range on a GPU); the step is bracketed as
  a collective for the watchdog; the device status word comes back with the loss, and a latched
  wait-timeout becomes a ``WatchdogTimeout`` health event before the loop stops; every
  ``sdc_every`` steps the replicated state is checksummed on the device and voted on;
  ``train.loss / grad_norm / lr / tokens_per_s / mfu``, ``comm.exposed_ms``, ``moe.load.*`` and
  ``fp8.amax.*`` go to the metric log (``--set metric_log=path`` for a JSONL file);
* checkpoints (in memory every ``ckpt_every`` steps, persistent at the end and every
  ``persist_every``) carry the loader cursor, so ``--resume`` continues bit-exactly.

(reference: there is no run loop in the reference beyond ``train.train_step``; the preset /
``--set`` layer is the thin CLI its config section asks for, ``control`` / ``obs`` are its crates.)
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys
import time

import numpy as np
import torch

from . import model, native, train

PRESETS = {
    "tiny_fp32": model.config_tiny_fp32,
    "dense_1p3b": model.config_dense_1p3b,
    "moe_16b": model.config_moe_16b,
    "long_context": model.config_long_context,
    "latent": model.config_latent,
}


@dataclasses.dataclass
class RunOptions:
    steps: int = 10
    batch: int = 8                    # sequences per rank per step
    seq_len: int = 0                  # 0: the preset's max_context (capped at 4096)
    micro_batch: int = 4
    seed: int = 0
    fp8: bool = False
    expert_parallel: bool = False
    context_parallel: bool = False
    ckpt_dir: str = ""
    ckpt_every: int = 50
    persist_every: int = 0
    spike_threshold: float = 0.5
    n_docs: int = 512                 # synthetic documents
    log_every: int = 1
    latent_slots: str = ""            # "start,k,sweeps[,truncated]"
    fsdp: bool = True                 # ZeRO-3 weights + owned-only optimizer state at world > 1
    allow_fallback: bool = False      # PyTorch / library forms for geometries without a kernel
    recurrence: int = 1               # core-block iterations per forward
    sdc_every: int = 0                # checksum vote over the replicated state every N steps
    metric_log: str = ""              # JSONL sink of the metric log
    straggler_ms: int = 600_000


def _coerce(value: str, current):
    if isinstance(current, bool):
        return value.lower() in ("1", "true", "yes", "on")
    if isinstance(current, int) and not isinstance(current, bool):
        return int(value)
    if isinstance(current, float):
        return float(value)
    if current is None:
        try:
            return json.loads(value)
        except ValueError:
            return value
    return type(current)(value)


def apply_overrides(pairs, cfg, tcfg, opts):
    """``key=value`` strings onto whichever of the three dataclasses has the key."""
    for pair in pairs:
        if "=" not in pair:
            raise ValueError(f"--set expects key=value, got {pair!r}")
        key, value = pair.split("=", 1)
        for holder in ("opts", "cfg", "tcfg"):
            obj = {"opts": opts, "cfg": cfg, "tcfg": tcfg}[holder]
            if hasattr(obj, key):
                new = dataclasses.replace(obj, **{key: _coerce(value, getattr(obj, key))})
                if holder == "opts":
                    opts = new
                elif holder == "cfg":
                    cfg = new
                else:
                    tcfg = new
                break
        else:
            raise ValueError(f"unknown setting {key!r}")
    return cfg, tcfg, opts


def synthetic_documents(vocab: int, n_docs: int, seq_len: int, seed: int):
    """Seeded uniform token documents of uneven length (packing has something to do)."""
    rng = np.random.default_rng(seed)
    return [rng.integers(4, vocab, size=int(rng.integers(seq_len // 4, seq_len * 2))).tolist() for _ in range(n_docs)]


def build_loader(docs, seq_len: int, seed: int, state_json: str | None = None):
    L = native.loader
    packing = L.Packing("run", seq_len)
    seqs = L.pack(docs, packing, 1)              # token 1 = eos between documents
    if state_json:
        return L.Loader.from_state(seqs, packing, L.LoaderState.from_json(state_json)), len(seqs)
    return L.Loader(seqs, packing, seed, "synthetic"), len(seqs)


class Prefetcher:
    """Pinned host batches one step ahead; ``next()`` returns device tensors whose copy was
    issued on a side stream while the previous step ran."""

    def __init__(self, loader, batch: int, device):
        self.loader, self.batch, self.device = loader, batch, torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.ready = None
        self._issue()

    def _issue(self):
        toks, mask = self.loader.next_batch_arrays(self.batch)
        state = self.loader.state().to_json()
        t, m = torch.from_numpy(np.ascontiguousarray(toks)), torch.from_numpy(np.ascontiguousarray(mask))
        if self.cuda:
            t, m = t.pin_memory(), m.pin_memory()
            with torch.cuda.stream(self.stream):
                dt, dm = t.to(self.device, non_blocking=True), m.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
            self.ready = (dt, dm, state, ev, (t, m))
        else:
            self.ready = (t, m, state, None, None)

    def next(self):
        dt, dm, state, ev, _keep = self.ready
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        self._issue()
        return dt, dm, state


def run(preset: str, sets=(), *, device: str | None = None, resume: str | None = None, out=sys.stdout) -> dict:
    if preset not in PRESETS:
        raise ValueError(f"unknown preset {preset!r}; choose from {sorted(PRESETS)}")
    cfg = PRESETS[preset]()
    tcfg = train.train_config_for(cfg)
    cfg, tcfg, opts = apply_overrides(sets, cfg, tcfg, RunOptions())
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    seq_len = opts.seq_len or min(cfg.max_context, 4096)
    import os

    import torch.distributed as dist

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if device == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
        else:
            dist.init_process_group("gloo")
    dev = torch.device(device, int(os.environ.get("LOCAL_RANK", "0"))) if device == "cuda" else torch.device("cpu")

    # data-parallel ranks read different documents; context-parallel ranks slice the same ones
    docs = synthetic_documents(cfg.vocab_size, opts.n_docs, seq_len,
                               opts.seed + (0 if opts.context_parallel else 1000 * rank))
    from . import supervisor
    from .utils import flops as flops_util

    sup = supervisor.RunSupervisor(world=world, rank=rank, tokens_per_step=opts.batch * seq_len * world,
                                   microbatch_tokens=max(1, min(opts.micro_batch, opts.batch)) * seq_len,
                                   sdc_period_steps=opts.sdc_every, straggler_timeout_ms=opts.straggler_ms,
                                   metric_sink=(opts.metric_log if rank == 0 and opts.metric_log else None))
    metrics, mlog = sup.metrics, sup.log
    spikes = native.obs.SpikeLog(10000, float(opts.spike_threshold), 8, 0)

    gpu = dev.type == "cuda"
    loader_state = None
    if gpu:
        from . import checkpoint, engine

        tr = engine.Trainer(cfg, tcfg, seed=opts.seed, device=dev, micro_batch=opts.micro_batch, fp8=opts.fp8,
                            expert_parallel=opts.expert_parallel, context_parallel=opts.context_parallel,
                            fsdp=opts.fsdp and not opts.context_parallel, allow_fallback=opts.allow_fallback,
                            recurrence=opts.recurrence)
        tr.time_phases = True
        tr.collect_amax = bool(opts.fp8)
        if opts.latent_slots:
            tr.set_latent_slots(*[int(x) for x in opts.latent_slots.split(",")])
        ck = checkpoint.TrainerCheckpointer(opts.ckpt_dir or None)
        if resume:
            info = ck.restore(tr, resume)
            loader_state = (info or {}).get("loader_state") if isinstance(info, dict) else None
    else:
        params = model.init_params(cfg, opts.seed)
        opt_state = train.init_opt_state(params, tcfg, muon_all_matrices=True)
        saved = None
    loader, n_seq = build_loader(docs, seq_len, opts.seed, json.dumps(loader_state) if loader_state else None)
    feed = Prefetcher(loader, opts.batch, dev)

    history, skipped, t_last = [], 0, time.perf_counter()
    step = tr.step_count if gpu else 0
    last_saved_step = step
    while step < opts.steps:
        t_step0 = time.perf_counter()
        with sup.phase("data"):
            tokens, mask, cursor = feed.next()
        status = 0
        with sup.phase("step"), sup.collective("train_step"):
            if gpu:
                if tr.cp:
                    tokens, mask = tr.cp_slice(tokens, mask)
                with sup.phase("launch"):
                    res = tr.step(tokens, mask)
                with sup.phase("readback"):
                    # loss, gradient norm and the device status word in one device-to-host copy
                    host = torch.stack([res["loss"].float().reshape(()), res["grad_norm"].float().reshape(()),
                                        res["status"].float().reshape(())]).cpu()
                loss, gnorm, lr, status = float(host[0]), float(host[1]), float(res["lr"]), int(host[2])
            else:
                b = train.Batch(tokens=tokens, loss_mask=mask, positions=torch.arange(tokens.shape[1]))
                o = train.train_step(params, opt_state, b, cfg, tcfg, step=step + 1, muon_transfer=True,
                                     muon_all_matrices=True)
                loss, gnorm, lr = float(o.loss.ce), float(o.grad_norm), float(o.lr)
        step += 1
        health = sup.after_step(step, (time.perf_counter() - t_step0) * 1e3, status)
        if status:
            # a bounded device wait ran out: the step ran on partial data. The controller has the
            # health event (the replica is drained there); this process stops instead of
            # checkpointing a corrupt state.
            metrics.inc("health.watchdog_timeouts", {"preset": preset}, 1)
            if gpu:
                tr.raise_on_status(status)
        if gpu and sup.sdc_due(step):
            with sup.phase("sdc_probe"):
                gone = sup.sdc_probe(step, supervisor.replicated_state(tr), group=tr.pg)
            if gone:
                raise RuntimeError(f"silent data corruption: replicas {gone} disagree with the majority "
                                   f"at step {step} ({sup.last_sdc_error})")
        actions = [str(a) for a in spikes.observe(step, loss, f"batch-{step}", preset)]
        rolled_back = any("Rollback" in a or "SkipShard" in a for a in actions) and step > 8
        if rolled_back:
            # a loss spike: undo this step and continue with the next batch
            skipped += 1
            if gpu and ck.last_id is not None:
                ck.restore(tr)
                step = tr.step_count
            elif not gpu and saved is not None:
                params, opt_state, step = saved
        elif not gpu:
            params, opt_state = o.params, o.opt_state
        now = time.perf_counter()
        tps = tokens.numel() * world / max(now - t_last, 1e-9)
        t_last = now
        labels = {"preset": preset}
        values = {"train.loss": loss, "train.grad_norm": gnorm, "train.lr": lr, "train.tokens_per_s": tps,
                  "train.grad_accumulation": float(health["grad_accumulation"])}
        if gpu:
            values["train.mfu"] = flops_util.mfu(tps, cfg, tokens.shape[1] * (world if tr.cp else 1), world,
                                                 recurrence=tr.recurrence,
                                                 sweeps=(tr.latent_slots[2] if tr.latent_slots else 1))
            if tr.phase_times:
                values["comm.exposed_ms"] = tr.phase_times["sync_ms"] if world > 1 else 0.0
                values["train.fwd_bwd_ms"] = tr.phase_times["fwd_bwd_ms"]
                values["train.opt_ms"] = tr.phase_times["opt_ms"]
            values.update(supervisor.moe_load_stats(tr.moe_load))
            for name, t in tr.amax.items():
                values[f"fp8.amax.{name}"] = float(t)
            tr.amax = {}
        sup.record(step, values, labels)
        metrics.set("loss", labels, loss)
        metrics.inc("steps", labels, 1)
        mlog.record("loss", labels, step, loss)
        history.append({"step": step, "loss": loss, "grad_norm": gnorm, "lr": lr, "tokens_per_s": tps,
                        "rolled_back": rolled_back, "mfu": values.get("train.mfu"),
                        "exposed_comm_ms": values.get("comm.exposed_ms")})
        if rank == 0 and opts.log_every and step % opts.log_every == 0:
            print(json.dumps(history[-1]), file=out, flush=True)
        if opts.ckpt_every and step % opts.ckpt_every == 0 and not rolled_back:
            if gpu:
                ck.save_memory(tr, loader_state=json.loads(cursor))
            else:
                saved = (params, opt_state, step)
            last_saved_step = step
        if gpu and opts.persist_every and step % opts.persist_every == 0:
            ck.save_persistent(tr, loader_state=json.loads(cursor))
    final_id = None
    if gpu and opts.ckpt_dir:
        final_id = ck.save_persistent(tr, wait=True, loader_state=json.loads(loader.state().to_json()))
    sup.close()
    summary = {"preset": preset, "steps": step, "final_loss": history[-1]["loss"] if history else None,
               "phase_ms": {k: round(v, 3) for k, v in sup.phase_ms.items()}, "live_replicas": sup.live(),
               "skipped_batches": skipped, "sequences_packed": n_seq, "checkpoint_id": final_id,
               "last_memory_checkpoint_step": last_saved_step, "world": world, "device": str(dev)}
    if rank == 0:
        print(json.dumps({"summary": summary}), file=out, flush=True)
    return {"summary": summary, "history": history}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m prometheus_b200.run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--preset", required=True, choices=sorted(PRESETS))
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    ap.add_argument("--steps", type=int)
    ap.add_argument("--device", choices=["cuda", "cpu"])
    ap.add_argument("--resume", help="checkpoint id to continue from (with --set ckpt_dir=...)")
    a = ap.parse_args(argv)
    sets = list(a.set) + ([f"steps={a.steps}"] if a.steps is not None else [])
    run(a.preset, sets, device=a.device, resume=a.resume)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
