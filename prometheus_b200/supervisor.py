"""Run supervision: the native controller, tracer and metrics wired round a training loop.

``RunSupervisor`` owns one ``native.control.Controller`` (elastic data parallelism, collective
watchdog, silent-data-corruption vote, loss-spike policy), one ``native.obs.Tracer`` (nested
host spans, mirrored as NVTX ranges on a GPU so a timeline tool shows the same phases), and the
``Metrics`` / ``MetricLog`` pair. The loop calls

* ``phase(name)``            a span round a phase of the step (data, forward-backward, sync, ...);
* ``collective(name)``       ``begin_collective`` / ``end_collective`` round a synchronisation, so
                             ``tick`` can see one that never ended;
* ``after_step(...)``        step time -> straggler detection; a latched device wait-timeout code
                             -> ``HealthKind.WatchdogTimeout`` -> the replica is drained and the
                             gradient accumulation of the survivors goes up;
* ``sdc_probe(...)``         every ``sdc_period`` steps: 64-bit checksums of state that must be
                             bit-identical on every replica (the fp32 vectors every rank updates,
                             the replicated bf16 weights), exchanged, voted on by the controller;
                             the odd one out is quarantined;
* ``record(...)``            ``train.loss``, ``train.grad_norm``, ``train.lr``, ``train.tokens_per_s``,
                             ``train.mfu``, ``comm.exposed_ms``, ``moe.load.max`` / ``moe.load.mean``,
                             ``fp8.amax.*`` into the metric log (JSONL sink optional).

Nothing here needs a GPU; the GPU-specific parts (NVTX, the checksum kernel) are used when a
CUDA tensor is handed in. Reference: control/src/lib.rs:208-226 (grad accumulation from live
replicas), :483-568 (shard-hash vote), :576-630 (collective watchdog), obs/src/lib.rs:160-215
(tracer) of the reference, none of which its train step calls.
"""
from __future__ import annotations

import contextlib
import time
import torch

from . import native


def _now_ms() -> int:
    return int(time.monotonic() * 1000)


def checksum64(t: torch.Tensor) -> int:
    """Position-weighted 64-bit checksum of a tensor's 32-bit words: equal bits, equal value.
    CUDA tensors use the device kernel (no copy of the data to the host); the CPU form is the
    same arithmetic in numpy, so a host copy of a shard hashes to the device's value."""
    flat = t.detach().contiguous().reshape(-1)
    nbytes = flat.numel() * flat.element_size()
    if nbytes % 4:
        raise ValueError("checksum64 needs a multiple of 4 bytes")
    if flat.is_cuda:
        from .ops._lib import call, ptr, stream_ptr

        out = torch.zeros(1, dtype=torch.int64, device=flat.device)
        call("pb_checksum_u32", ptr(flat), nbytes // 4, ptr(out), stream_ptr())
        return int(out.item()) & 0xFFFFFFFFFFFFFFFF
    import numpy as np

    words = flat.view(torch.uint8).numpy().view("<u4").astype(np.uint64)
    idx = np.arange(words.size, dtype=np.uint64)
    with np.errstate(over="ignore"):
        acc = ((words + np.uint64(0x9E3779B97F4A7C15)) * (idx * np.uint64(2) + np.uint64(1))).sum(dtype=np.uint64)
    return int(acc) & 0xFFFFFFFFFFFFFFFF


class RunSupervisor:
    def __init__(self, *, world: int, rank: int, tokens_per_step: int, microbatch_tokens: int,
                 sdc_period_steps: int = 0, straggler_timeout_ms: int = 60_000,
                 collective_watchdog_ms: int = 60_000, ranks_per_rack: int = 1,
                 metric_sink: str | None = None, nvtx: bool = True):
        C = native.control
        self.world, self.rank = int(world), int(rank)
        self.replicas = [f"r{r}" for r in range(self.world)]
        self.me = self.replicas[self.rank]
        cfg = C.ElasticConfig(int(tokens_per_step), int(microbatch_tokens), int(sdc_period_steps),
                              int(straggler_timeout_ms), int(collective_watchdog_ms))
        # the vote quarantines the offender's whole rack: inside one box every GPU is its own
        # failure domain (ranks_per_rack = 1); a multi-box job groups the ranks of a box
        specs = [C.ReplicaSpec(self.replicas[r], f"rack{r // max(1, ranks_per_rack)}")
                 for r in range(self.world)]
        self.controller = C.Controller(cfg, specs)
        self.sdc_period = int(sdc_period_steps)
        self.tracer = native.obs.Tracer()
        self.metrics = native.obs.Metrics()
        self.log = native.obs.MetricLog()
        if metric_sink:
            self.log.open_sink(metric_sink)
        self._nvtx = bool(nvtx) and torch.cuda.is_available()
        self.phase_ms: dict[str, float] = {}
        self.quarantined: list[str] = []
        self.last_sdc_error: str | None = None
        self.last_health_error: str | None = None

    # ------------------------------------------------------------------ spans
    @contextlib.contextmanager
    def phase(self, name: str):
        """A named span: host tracer + (on a GPU) an NVTX range of the same name."""
        span = self.tracer.start(name)
        if self._nvtx:
            torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            if self._nvtx:
                torch.cuda.nvtx.range_pop()
            self.phase_ms[name] = self.phase_ms.get(name, 0.0) + float(self.tracer.end(span))

    @contextlib.contextmanager
    def collective(self, name: str):
        """Watchdog bracket round a synchronisation of this replica."""
        self.controller.begin_collective(name, self.me, _now_ms())
        try:
            yield
        finally:
            self.controller.end_collective(name, self.me, _now_ms())

    # ----------------------------------------------------------------- health
    def live(self) -> list[str]:
        return list(self.controller.live_replicas())

    def grad_accumulation(self) -> int:
        return int(self.controller.grad_accumulation())

    def after_step(self, step: int, step_ms: float, status_code: int = 0,
                   replica: str | None = None) -> dict:
        """Feed one step's outcome to the controller. ``status_code`` is the device status word
        read back with the loss: non-zero means a bounded device wait ran out, which is
        reported as a watchdog timeout of that replica (it is drained; the survivors'
        gradient accumulation rises to keep the tokens per step)."""
        who = replica or self.me
        C = native.control
        now = _now_ms()
        if status_code:
            try:
                self.controller.report_health(C.HealthEvent(who, who, C.HealthKind.WatchdogTimeout, now,
                                                            f"device wait timed out (code {status_code})"))
            except native.NativeError as e:
                # the last live replica cannot be drained: the event is kept for the caller, who
                # stops the run instead
                self.last_health_error = str(e)
        else:
            self.controller.observe_step_time(who, int(step), int(step_ms))
        self.controller.tick(now)
        return {"live": self.live(), "grad_accumulation": self.grad_accumulation(),
                "state": str(self.controller.replica_state(who)).split(".")[-1]}

    def replica_left(self, replica: str) -> dict:
        """A replica announced (or was found) gone between steps."""
        self.controller.fail_replica(replica)
        return {"live": self.live(), "grad_accumulation": self.grad_accumulation()}

    # -------------------------------------------------------------------- SDC
    def sdc_due(self, step: int) -> bool:
        return self.sdc_period > 0 and step > 0 and step % self.sdc_period == 0

    def sdc_probe(self, step: int, shards: dict[str, torch.Tensor], group=None,
                  exchange=None) -> list[str]:
        """Checksum ``shards`` (name -> tensor that must be bit-identical on every replica),
        exchange the values over the ranks and let the controller vote. Returns the replicas
        newly quarantined. ``exchange(local: dict) -> list[dict]`` overrides the transport
        (default: ``torch.distributed.all_gather_object`` on ``group``)."""
        local = {name: f"{checksum64(t):016x}" for name, t in shards.items()}
        if exchange is not None:
            every = exchange(local)
        elif self.world > 1:
            import torch.distributed as dist

            every = [None] * dist.get_world_size(group)
            dist.all_gather_object(every, local, group=group)
        else:
            every = [local]
        live = set(self.live())
        for r, hashes in enumerate(every):
            rep = self.replicas[r] if len(every) == self.world else self.me
            if rep not in live or hashes is None:
                continue
            for name, h in hashes.items():
                self.controller.report_shard_hash(rep, name, h, int(step))
        before = set(self.live())
        try:
            self.controller.check_sdc(int(step))
        except Exception as e:          # the controller reports a mismatch after acting on it
            if "HashMismatch" not in f"{type(e).__name__} {e}" and "mismatch" not in str(e):
                raise
            self.last_sdc_error = str(e)
        gone = sorted(before - set(self.live()))
        self.quarantined += gone
        return gone

    # ---------------------------------------------------------------- metrics
    def record(self, step: int, values: dict[str, float], labels: dict | None = None) -> None:
        labels = dict(labels or {})
        for name, v in values.items():
            if v is None:
                continue
            self.metrics.set(name, labels, float(v))
            self.log.record(name, labels, int(step), float(v))

    def close(self) -> None:
        self.log.close_sink()


def replicated_state(trainer) -> dict[str, torch.Tensor]:
    """What must be bit-identical on every data-parallel rank of an ``engine.Trainer``: the fp32
    vectors (every rank applies the same update to them) and, when the bf16 weights are
    replicated, those too. Expert-parallel and sharded ranges are each rank's own and are left
    out."""
    out = {"vec.master": trainer.vec_master}
    if getattr(trainer, "sym", None) is not None and not getattr(trainer, "fsdp", False) \
            and not getattr(trainer, "ep", False):
        out["lp.muon"] = trainer.muon_lp.view(torch.int32)      # element counts are multiples of 8
        out["lp.adam"] = trainer.adam_lp.view(torch.int32)
    return out


def moe_load_stats(load: torch.Tensor | None) -> dict[str, float]:
    """``moe.load.max`` / ``moe.load.mean``: the largest and the mean per-expert share of the
    assignments (times the expert count, so 1.0 is perfect balance), over the MoE layers."""
    if load is None:
        return {}
    rel = load * load.shape[-1]
    return {"moe.load.max": float(rel.max()), "moe.load.mean": float(rel.mean())}
