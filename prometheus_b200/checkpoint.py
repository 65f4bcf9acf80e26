"""Checkpoint / resume for the GPU trainer on the native content-addressed store.

A checkpoint is the reference's on-disk object (ckpt/src/lib.rs:28-59 of the reference): a
``prometheus.checkpoint`` v1 manifest naming every weight shard and optimizer shard by
sha256, plus the shard blobs. ``capture`` turns a live :class:`~prometheus_b200.engine.Trainer`
into one (fp32 masters per engine weight; Muon momentum or AdamW moments per weight; the step
count; the data-loader envelope), ``apply`` puts one back, and :class:`TrainerCheckpointer`
drives the native ``Checkpointer`` (two in-memory replicas every step, persistent saves on a
background thread, cross-rack copies) the way the reference's train loop is specified to
(ckpt/src/lib.rs:427-526, 617-673).

With ownership sharding (world > 1) each rank only keeps its own matrices' masters and
optimizer state current. ``capture`` therefore first sums the owned ranges across ranks, so
every rank holds the full state and rank 0's checkpoint is complete; ``apply`` loads the
full state on every rank. Restoring is bit-exact: blobs are the raw little-endian buffers.
"""
from __future__ import annotations

import datetime as _dt
import hashlib
import json
import math
from typing import Any

import torch

from . import native

ZERO_HASH = "0" * 64


def _ck():
    return native.ckpt


def model_config_hash(cfg) -> str:
    """sha256 of the canonical (sorted-key, compact) JSON of the model configuration."""
    from dataclasses import asdict, is_dataclass

    d = asdict(cfg) if is_dataclass(cfg) else dict(cfg)
    d = {k: (v.name if hasattr(v, "name") and not isinstance(v, (str, int, float)) else v)
         for k, v in d.items()}
    return hashlib.sha256(json.dumps(d, sort_keys=True, separators=(",", ":"),
                                     default=str).encode()).hexdigest()


def _bytes(t: torch.Tensor) -> bytes:
    return t.detach().contiguous().cpu().numpy().tobytes()


def _full_state(tr) -> dict[str, torch.Tensor]:
    """All flat fp32 state buffers, complete on every rank."""
    if hasattr(tr, "full_state"):          # the trainer knows its own (possibly sharded) layout
        return tr.full_state()
    bufs = {"muon.master": tr.muon_master, "muon.mom": tr.muon_mom,
            "adam.master": tr.adam_master, "adam.m": tr.adam_m, "adam.v": tr.adam_v,
            "vec.master": tr.vec_master, "vec.m": tr.vec_m, "vec.v": tr.vec_v}
    if getattr(tr, "sym", None) is None:
        return bufs
    import torch.distributed as dist

    out = dict(bufs)
    ranges, local_ranges = [], []
    for key, units in tr.unit_classes.items():
        rows, cols = key[:2]
        lo_u, hi_u = tr.own_units[key]
        rng = (units[0].off + lo_u * rows * cols, units[0].off + hi_u * rows * cols)
        # expert-parallel weights are each rank's own: kept local here, saved as per-rank shards
        (local_ranges if len(key) > 2 else ranges).append(rng)
    for key in ("muon.master", "muon.mom"):
        full = torch.zeros_like(bufs[key])
        for lo, hi in ranges:
            full[lo:hi] = bufs[key][lo:hi]
        dist.all_reduce(full, group=tr.pg)
        for lo, hi in local_ranges:
            full[lo:hi] = bufs[key][lo:hi]
        out[key] = full
    a_lo, a_hi = tr.own_adam
    for key in ("adam.master", "adam.m", "adam.v"):
        full = torch.zeros_like(bufs[key])
        full[a_lo:a_hi] = bufs[key][a_lo:a_hi]
        dist.all_reduce(full, group=tr.pg)
        out[key] = full
    return out


def capture(tr, *, rung: int = 0, data_mix_hash: str = ZERO_HASH, tokenizer_id: str = "byte-fallback",
            loader_state: dict | None = None, parent: str | None = None,
            created_at: str | None = None, git_commit: str | None = None):
    """Snapshot a Trainer into a native ``Checkpoint`` (collective when world > 1)."""
    C = _ck()
    state = _full_state(tr)
    weights, opt, wmeta, ometa = [], [], [], []
    sharded = getattr(tr, "world", 1) > 1 and getattr(tr, "sym", None) is not None

    def per_rank(t: torch.Tensor, local: bool):
        """[(shard_rank, bytes)]: one shard, or one per rank for expert-parallel weights."""
        if not (local and sharded):
            return [(0, _bytes(t))]
        import torch.distributed as dist

        parts = [torch.empty_like(t) for _ in range(tr.world)]
        dist.all_gather(parts, t.contiguous(), group=tr.pg)
        return [(r, _bytes(p)) for r, p in enumerate(parts)]

    for w in tr.weights.values():
        n = int(math.prod(w.shape))
        sl = slice(w.off, w.off + n)
        g = w.group
        local = bool(getattr(w, "local", False))
        axes = ["ep"] if local and sharded else []
        for r, blob in per_rank(state[f"{g}.master"][sl], local):
            weights.append(C.ShardBlob(w.name, r, blob))
            wmeta.append(C.WeightMeta(w.name, r, list(w.shape), "fp32", C.sha256_hex(blob), axes))
        if g == "muon":
            parts = [("mom", "muon", state["muon.mom"][sl])]
        else:
            parts = [("m", "adamw", state[f"{g}.m"][sl]), ("v", "adamw", state[f"{g}.v"][sl])]
        for suffix, kind, t in parts:
            for r, ob in per_rank(t, local):
                opt.append(C.ShardBlob(f"{w.name}.{suffix}", r, ob))
                ometa.append(C.OptimizerMeta(f"{w.name}.{suffix}", r, kind, C.sha256_hex(ob)))
    # aux-loss-free balancing biases: state without an optimizer (same on every rank)
    for i, b in sorted(getattr(tr, "router_bias", {}).items()):
        blob = _bytes(b.float())
        name = f"layers.{i}.router_bias"
        weights.append(C.ShardBlob(name, 0, blob))
        wmeta.append(C.WeightMeta(name, 0, [int(b.numel())], "fp32", C.sha256_hex(blob), []))
    m = C.Manifest()
    m.step = int(tr.step_count)
    m.rung = int(rung)
    m.model_config_hash = model_config_hash(tr.cfg)
    m.data_mix_hash = data_mix_hash
    m.tokenizer_id = tokenizer_id
    m.precision = ("bf16", "none")
    m.dp = int(tr.world)
    m.ep = int(tr.world) if getattr(tr, "ep", False) else 1
    m.weights, m.optimizer = wmeta, ometa
    if loader_state is not None:
        m.loader_state_json = json.dumps(loader_state, sort_keys=True, separators=(",", ":"))
    rng = [("torch.cpu", torch.get_rng_state())]
    if torch.cuda.is_available() and getattr(tr.device, "type", "cpu") == "cuda":
        rng.append(("torch.cuda", torch.cuda.get_rng_state(tr.device)))
    m.rng = [C.RngState(scope, int(tr.rank), hashlib.sha256(_bytes(s)).hexdigest()) for scope, s in rng]
    # the generator state itself travels as a shard (``rng.<scope>.<rank>``) next to its hash in
    # the manifest, so a run with stochastic parts resumes bit for bit
    mine = [(scope, _bytes(st)) for scope, st in rng]
    every = [mine]
    if getattr(tr, "world", 1) > 1 and torch.distributed.is_available() and torch.distributed.is_initialized():
        every = [None] * tr.world          # every rank's generators, so all ranks build one manifest
        torch.distributed.all_gather_object(every, mine, group=getattr(tr, "pg", None))
    for r, states in enumerate(every):
        r = r if len(every) > 1 else int(tr.rank)
        for scope, blob in states:
            name = f"rng.{scope}.{r}"
            weights.append(C.ShardBlob(name, r, blob))
            wmeta.append(C.WeightMeta(name, r, [len(blob)], "int8", C.sha256_hex(blob), []))
    m.weights = wmeta
    m.created_at = created_at or _dt.datetime.now(_dt.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")
    m.parent_checkpoint_id = parent
    m.git_commit = git_commit
    ident = hashlib.sha256()
    for x in wmeta:
        ident.update(x.content_hash.encode())
    for x in ometa:
        ident.update(x.content_hash.encode())
    ident.update(str(m.step).encode())
    m.checkpoint_id = ident.hexdigest()
    return C.Checkpoint(m, weights, opt)


def apply(tr, ckpt, *, strict_config: bool = True) -> dict[str, Any] | None:
    """Load a checkpoint into a Trainer (same model configuration). Returns the data-loader
    envelope stored with it (or None)."""
    m = ckpt.manifest
    if strict_config and m.model_config_hash != model_config_hash(tr.cfg):
        raise ValueError("checkpoint was written for a different model configuration")
    me = int(getattr(tr, "rank", 0))

    def by_name(blobs):
        out = {}
        for b in blobs:     # a rank's own shard wins over shard 0
            if b.name not in out or b.shard_rank == me:
                out[b.name] = b.bytes
        return out

    wb, ob = by_name(ckpt.weights), by_name(ckpt.optimizer)
    dev = tr.device

    def put(dst: torch.Tensor, raw: bytes, what: str):
        if len(raw) != dst.numel() * 4:
            raise ValueError(f"{what}: {len(raw)} bytes for {dst.numel()} fp32 values")
        src = torch.frombuffer(bytearray(raw), dtype=torch.float32)
        dst.copy_(src.to(dev))

    def blob_f32(raw: bytes, numel: int, what: str):
        if len(raw) != numel * 4:
            raise ValueError(f"{what}: {len(raw)} bytes for {numel} fp32 values")
        return torch.frombuffer(bytearray(raw), dtype=torch.float32)

    if hasattr(tr, "_store_state"):
        # sharded-state trainer: every rank reads the full tensors and keeps what it stores
        with torch.no_grad():
            for w in tr.weights.values():
                n = int(math.prod(w.shape))
                parts = [("master", wb[w.name], w.name)]
                if w.group == "muon":
                    parts.append(("mom", ob[w.name + ".mom"], w.name + ".mom"))
                else:
                    parts += [("m", ob[w.name + ".m"], w.name + ".m"), ("v", ob[w.name + ".v"], w.name + ".v")]
                for which, raw, what in parts:
                    full = blob_f32(raw, n, what).to(dev).view(w.shape)
                    tr._store_state(w, which, full)
                    if which == "master":
                        tr._store_lp(w, full)
            for i, b in getattr(tr, "router_bias", {}).items():
                name = f"layers.{i}.router_bias"
                if name in wb:
                    put(b, wb[name], name)
        if getattr(tr, "fsdp", False):
            tr._fsdp_invalidate()
        tr.step_count = int(m.step)
        _restore_rng(tr, wb)
        if getattr(tr, "sym", None) is not None:
            torch.cuda.synchronize()
            torch.distributed.barrier(tr.pg)
        raw = getattr(m, "loader_state_json", "")
        return json.loads(raw) if raw and raw != "{}" else None

    with torch.no_grad():
        for w in tr.weights.values():
            n = int(math.prod(w.shape))
            sl = slice(w.off, w.off + n)
            g = w.group
            master = {"muon": tr.muon_master, "adam": tr.adam_master, "vec": tr.vec_master}[g]
            put(master[sl], wb[w.name], w.name)
            if g == "muon":
                put(tr.muon_mom[sl], ob[w.name + ".mom"], w.name + ".mom")
            else:
                mm, vv = (tr.adam_m, tr.adam_v) if g == "adam" else (tr.vec_m, tr.vec_v)
                put(mm[sl], ob[w.name + ".m"], w.name + ".m")
                put(vv[sl], ob[w.name + ".v"], w.name + ".v")
        tr.muon_lp.copy_(tr.muon_master)
        tr.adam_lp.copy_(tr.adam_master)
        for i, b in getattr(tr, "router_bias", {}).items():
            name = f"layers.{i}.router_bias"
            if name in wb:
                put(b, wb[name], name)
    tr.step_count = int(m.step)
    _restore_rng(tr, wb)
    if getattr(tr, "sym", None) is not None:
        torch.cuda.synchronize()
        torch.distributed.barrier(tr.pg)
    raw = getattr(m, "loader_state_json", "")
    return json.loads(raw) if raw and raw != "{}" else None


def _restore_rng(tr, blobs_by_name: dict) -> None:
    """Put back the generator states saved as ``rng.<scope>.<rank>`` shards (this rank's own)."""
    me = int(getattr(tr, "rank", 0))
    raw = blobs_by_name.get(f"rng.torch.cpu.{me}")
    if raw is not None:
        torch.set_rng_state(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
    raw = blobs_by_name.get(f"rng.torch.cuda.{me}")
    if raw is not None and torch.cuda.is_available() and getattr(tr.device, "type", "cpu") == "cuda":
        torch.cuda.set_rng_state(torch.frombuffer(bytearray(raw), dtype=torch.uint8), tr.device)


def broadcast_checkpoint(ckpt, error: str | None, tr):
    """Rank 0's checkpoint (or its error) to every rank of the trainer's group. Returns an
    object with the ``manifest`` / ``weights`` / ``optimizer`` fields :func:`apply` reads.
    Blobs travel as byte tensors through the group's backend (NCCL: via the GPU)."""
    import types

    import torch.distributed as dist

    group = getattr(tr, "pg", None)
    backend = dist.get_backend(group)
    dev = tr.device if backend == "nccl" else torch.device("cpu")
    # ranks inside `group` address rank 0 of the group
    src = dist.get_global_rank(group, 0) if group is not None else 0
    head = [None]
    if tr.rank == 0:
        if error is not None:
            head[0] = {"error": error}
        else:
            m = ckpt.manifest
            head[0] = {"error": None, "step": int(m.step), "model_config_hash": m.model_config_hash,
                       "loader_state_json": getattr(m, "loader_state_json", ""),
                       "weights": [(b.name, int(b.shard_rank), len(b.bytes)) for b in ckpt.weights],
                       "optimizer": [(b.name, int(b.shard_rank), len(b.bytes)) for b in ckpt.optimizer]}
    dist.broadcast_object_list(head, src=src, group=group)
    info = head[0]
    if info["error"] is not None:
        raise RuntimeError(f"checkpoint restore failed on rank 0: {info['error']}")
    if tr.rank == 0:
        blobs = {"weights": list(ckpt.weights), "optimizer": list(ckpt.optimizer)}
    out = {"weights": [], "optimizer": []}
    me = int(tr.rank)
    for kind in ("weights", "optimizer"):
        for j, (name, shard_rank, nbytes) in enumerate(info[kind]):
            if tr.rank == 0:
                t = torch.frombuffer(bytearray(blobs[kind][j].bytes), dtype=torch.uint8).to(dev)
            else:
                t = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            dist.broadcast(t, src=src, group=group)
            # a rank keeps shard 0 and its own shard of every name (what apply() looks at)
            if shard_rank in (0, me):
                out[kind].append(types.SimpleNamespace(name=name, shard_rank=shard_rank,
                                                       bytes=t.cpu().numpy().tobytes()))
    manifest = types.SimpleNamespace(step=info["step"], model_config_hash=info["model_config_hash"],
                                     loader_state_json=info["loader_state_json"])
    return types.SimpleNamespace(manifest=manifest, weights=out["weights"], optimizer=out["optimizer"])


class TrainerCheckpointer:
    """The save policy of the reference's train loop on the native ``Checkpointer``: an
    in-memory checkpoint (two replicas) whenever asked, a persistent one written by a
    background thread so the step loop never waits on the file system, and restore by id or
    from the newest in-memory replica."""

    def __init__(self, root: str | None = None, *, racks: list[str] | None = None):
        C = _ck()
        self.store = C.DirStore(root) if root is not None else C.MemoryStore()
        self.cp = C.Checkpointer(self.store)
        self.racks = racks
        self.pending = None
        self.last_id: str | None = None

    def save_memory(self, tr, **kw) -> str:
        ck = capture(tr, parent=self.last_id, **kw)
        if tr.rank == 0:
            self.last_id = self.cp.save_in_memory(ck)
        else:
            self.last_id = ck.manifest.checkpoint_id
        return self.last_id

    def save_persistent(self, tr, *, wait: bool = False, **kw) -> str:
        ck = capture(tr, parent=self.last_id, **kw)
        self.last_id = ck.manifest.checkpoint_id
        if tr.rank == 0:
            self.wait()
            self.pending = self.cp.save_persistent_async(ck)
            if wait:
                self.wait()
        return self.last_id

    def wait(self) -> None:
        if self.pending is not None:
            self.pending.wait()
            self.pending = None

    def restore(self, tr, checkpoint_id: str | None = None):
        """Load a checkpoint (by id, else the newest in-memory replica) into the trainer.
        Collective when the trainer spans several ranks: only rank 0 holds the replicas and
        reads the store, so it loads the checkpoint and broadcasts it; every rank then applies
        it. A failure on rank 0 (unknown id, hash mismatch) is raised on every rank."""
        self.wait()
        if getattr(tr, "world", 1) <= 1:
            ck = self.cp.restore(checkpoint_id) if checkpoint_id else self.cp.restore_latest_memory()
            return apply(tr, ck)
        ck, err = None, None
        if tr.rank == 0:
            try:
                ck = self.cp.restore(checkpoint_id) if checkpoint_id else self.cp.restore_latest_memory()
            except Exception as e:          # noqa: BLE001 - re-raised on every rank below
                err = f"{type(e).__name__}: {e}"
        return apply(tr, broadcast_checkpoint(ck, err, tr))
