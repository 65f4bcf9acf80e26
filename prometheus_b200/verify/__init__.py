"""Verification stages V0..V10: runners that write the files the exit checkers read.

Each ``run_vN`` exercises the real components of this package at a size that finishes on
one machine (a GPU is used when present; every runner also completes on CPU) and returns the
result dictionary of its stage; ``write_result`` stores it as ``<out>/<stage>.json`` and
``check_exit`` (the native checker, ``csrc/native/verify_stages.cpp``) decides pass / fail
from that file alone. ``render_job`` fills the sbatch template of a stage.

    python -m prometheus_b200.verify --stage v1 --out verify-out/run1/v1
    python -m prometheus_b200.verify --check v1 --out verify-out/run1/v1

API parity with the reference's ``prometheus.verify`` (``run_v1`` .. ``run_v10``, result keys
of ``verify/ncshare/src/check.rs``); the runners themselves are written against this
package's modules.
"""
from __future__ import annotations

import dataclasses
import json
import math
import tempfile
from pathlib import Path

import torch

from .. import kernels, latent, model, native, rl_loss, train

TEMPLATE_DIR = Path(__file__).parent / "templates"
STAGES = tuple(native.ncshare.STAGES)


class VerifyError(RuntimeError):
    """A runner could not produce its measurements."""


# ---------------------------------------------------------------------------
# job scripts and exit checks (native)
# ---------------------------------------------------------------------------
def render_job(stage: str, run_id: str, walltime: str, gpus: int | None = None) -> str:
    spec = native.ncshare.spec(stage)
    n = gpus if gpus is not None else (spec["gpus"] or 1)
    return native.ncshare.render_job(stage, run_id, walltime, int(n), str(TEMPLATE_DIR))


def render_v0_2node(run_id: str, walltime: str) -> str:
    return native.ncshare.render_v0_2node(run_id, walltime, str(TEMPLATE_DIR))


def check_exit(stage: str, output_dir) -> None:
    native.ncshare.check_exit(stage, str(output_dir))


def write_result(stage: str, result: dict, output_dir) -> Path:
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    path = out / f"{native.ncshare.parse_stage(stage)}.json"
    path.write_text(json.dumps(result, sort_keys=True, indent=1))
    return path


# ---------------------------------------------------------------------------
# shared helpers
# ---------------------------------------------------------------------------
def _small_config(**over) -> model.ModelConfig:
    base = dict(d_model=64, n_layers=4, n_dense=4, n_moe=0, n_linear_attn=3, n_mla=1,
                n_routed_experts=1, n_shared_experts=0, top_k=1, expert_hidden=128, mtp_heads=0,
                core_block_layers=4, recurrence_train_mean=1.0, recurrence_max=1, vocab_size=128,
                max_context=128, prelude_layers=0, coda_layers=0, adapter_hidden=64, n_heads=2,
                d_head=32, n_kv_heads=1, softmax_kind="gqa", softmax_every=4, delta_beta="sigmoid",
                chunk=16, dense_hidden=128)
    base.update(over)
    return model.ModelConfig(**base)


def _batch(cfg, b: int, s: int, seed: int) -> train.Batch:
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, cfg.vocab_size, (b, s), generator=g)
    return train.Batch(tokens=tokens, loss_mask=torch.ones(b, s), positions=torch.arange(s))


def _train(cfg, tcfg, params, batches, start_step: int = 1, opt=None):
    """Run ``train.train_step`` over ``batches``; returns (params, opt_state, losses)."""
    opt = train.init_opt_state(params, tcfg, muon_all_matrices=True) if opt is None else opt
    losses = []
    for i, b in enumerate(batches):
        out = train.train_step(params, opt, b, cfg, tcfg, step=start_step + i, muon_transfer=True,
                               muon_all_matrices=True)
        params, opt = out.params, out.opt_state
        losses.append(float(out.loss.ce))
    return params, opt, losses


def _tree_bytes(tree) -> bytes:
    flat = model.flatten_params(tree)
    return b"".join(flat[k].detach().cpu().contiguous().numpy().tobytes() for k in sorted(flat))


# ---------------------------------------------------------------------------
# V1  kernel path vs independent reference, gradients, overfit
# ---------------------------------------------------------------------------
def run_v1(*, gpus: int = 1) -> dict:
    """logits_max_diff compares the model forward (chunked WY delta rule) with the same forward
    on the per-token recurrence, two independent formulations of the attention math, in fp32.
    On a GPU the tcgen05 path is additionally compared in bf16 tolerance (reported, not gated)."""
    cfg = _small_config()
    params = model.init_params(cfg, 0)
    b = _batch(cfg, 2, 48, 1)
    with torch.no_grad():
        ref = model.forward(b.tokens, params, cfg, r=1).logits
        orig = kernels.chunked_delta_rule
        try:   # the per-token recurrence in place of the chunked scan
            kernels.chunked_delta_rule = lambda q, k, v, beta, state=None, config=None, **kw: (
                kernels.delta_rule_recurrent(q, k, v, beta, state if state is not None else kw.get("initial_state")))
            alt = model.forward(b.tokens, params, cfg, r=1).logits
        finally:
            kernels.chunked_delta_rule = orig
    diff = float((ref - alt).abs().max())
    # and against the NumPy float64 restatement that shares no code with the model
    from .independent_forward import forward_logits

    indep = float(abs(ref.numpy() - forward_logits(b.tokens, params, cfg, r=1)).max())
    # gradient check: central finite difference of the loss along one direction
    tcfg = train.train_config_for(cfg, warmup_steps=1, stable_steps=50, decay_steps=5)
    p = train._map_tree(params, lambda _n, t: t.clone().requires_grad_(True))
    loss, _ = train.compute_loss(p, b, cfg, tcfg)
    flat = model.flatten_params(p)
    names = sorted(flat)
    grads = torch.autograd.grad(loss, [flat[n] for n in names], allow_unused=True)
    # along the normalised gradient itself the directional derivative is the gradient norm
    gnorm = math.sqrt(sum(float(g.square().sum()) for g in grads if g is not None))
    dirs = [torch.zeros_like(flat[n]) if g is None else g / gnorm for n, g in zip(names, grads)]
    analytic = gnorm
    eps = 2e-2

    def shifted(sign):
        q = train._map_tree(params, lambda n, t: t + sign * eps * dirs[names.index(n)])
        with torch.no_grad():
            return float(train.compute_loss(q, b, cfg, tcfg)[0])

    numeric = (shifted(+1) - shifted(-1)) / (2 * eps)
    grad_ok = abs(numeric - analytic) <= 5e-2 * max(1.0, abs(analytic))
    _, _, losses = _train(cfg, tcfg, params, [b] * 12)
    result = {"logits_max_diff": max(diff, indep), "recurrence_max_diff": diff, "independent_max_diff": indep, "grad_ok": bool(grad_ok), "overfit_ok": bool(losses[-1] < losses[0] - 0.3),
              "gpus": int(gpus), "grad_numeric": numeric, "grad_analytic": analytic, "losses": losses}
    if torch.cuda.is_available():
        from .. import engine

        ecfg = _small_config(d_model=256, n_heads=2, d_head=128, n_kv_heads=1, chunk=64, dense_hidden=512, vocab_size=1024)
        etcfg = train.train_config_for(ecfg, warmup_steps=1, stable_steps=50, decay_steps=5)
        eparams = model.init_params(ecfg, 0)
        tr = engine.Trainer(ecfg, etcfg, params=eparams, micro_batch=2)
        tok = _batch(ecfg, 2, 128, 2).tokens
        with torch.no_grad():
            hid = tr.forward_hidden(tok.cuda()).float()
            dev = train._map_tree(eparams, lambda _n, t: t.cuda())
            want = model.forward(tok.cuda(), dev, ecfg, r=1).hidden.reshape(hid.shape)
        result["kernel_hidden_rel_err_bf16"] = float((hid - want).norm() / want.norm())
    return result


# ---------------------------------------------------------------------------
# V2  single device vs sharded / dispatched execution
# ---------------------------------------------------------------------------
def run_v2(*, gpus: int = 8, steps: int = 20, drop_rank: bool = False) -> dict:
    """Single device against the mesh, through the production definitions:

    * data parallel + FSDP: every step, the gradient of the whole batch equals the per-rank
      gradients of the batch slices pushed through ``fsdp_reduce_scatter`` (rank-ordered fp32
      fold) and ``fsdp_all_gather``; the parameters then advance with ``train.train_step``;
    * expert parallel: the MoE layer's output equals dispatch -> per-expert FFN -> combine on the
      ``kernels.ep_dispatch`` / ``ep_combine`` tables, and the routing is identical;
    * context parallel: ring attention over ``min(gpus, 4)`` sequence slices equals dense
      attention, and the delta-rule state handed from slice to slice equals the state of the
      whole prefix;
    * on a machine with two or more GPUs: the fused trainer on one GPU, replicated over two and
      ZeRO-3 over two give the same losses (``tests/_multi_gpu_worker.py`` is the worker).

    ``drop_rank`` (negative control) loses the last rank's gradient before the reduction: the
    reduced gradient then differs from the whole-batch one and the stage must fail."""
    if isinstance(gpus, bool) or not isinstance(gpus, int) or gpus < 1:
        raise VerifyError("gpus must be a positive integer")
    from .. import parallel as P
    from ..parallel import cp as cp_mod
    from ..parallel import fsdp

    cfg = _small_config(n_dense=1, n_moe=3, n_routed_experts=8, top_k=2, expert_hidden=64)
    tcfg = train.train_config_for(cfg, warmup_steps=1, stable_steps=steps, decay_steps=2)
    params = model.init_params(cfg, 0)
    n = max(2, min(int(gpus), 4))                  # ranks emulated on the host
    worst_grad, same_routing = 0.0, True
    p1, o1 = params, None
    for step in range(1, steps + 1):
        b = _batch(cfg, 2 * n, 32, 100 + step)

        def grads_of(tokens, mask):
            live = train._map_tree(p1, lambda _n, t: t.detach().clone().requires_grad_(True))
            total, (_, _, _, out) = train.compute_loss(live, train.Batch(tokens, mask, b.positions), cfg, tcfg,
                                                       z_on_logits=True)
            flat = model.flatten_params(live)
            names = sorted(flat)
            gs = torch.autograd.grad(total, [flat[k] for k in names], allow_unused=True)
            return {k: (torch.zeros_like(flat[k]) if g is None else g) for k, g in zip(names, gs)}, out

        full, out_full = grads_of(b.tokens, b.loss_mask)
        per_rank = []
        for r in range(n):
            sl = slice(2 * r, 2 * r + 2)
            g_r, out_r = grads_of(b.tokens[sl], b.loss_mask[sl])
            per_rank.append(g_r)
            same_routing = same_routing and bool(torch.equal(out_r.expert_ids, out_full.expert_ids[sl]))
        for name, g_full in full.items():
            if g_full.numel() < n:
                continue
            flat_r = [g[name].reshape(-1) / n for g in per_rank]          # equal slices: mean of the means
            if drop_rank:
                flat_r[-1] = torch.zeros_like(flat_r[-1])
            pad = (-flat_r[0].numel()) % n
            if pad:
                flat_r = [torch.nn.functional.pad(f, (0, pad)) for f in flat_r]
            shards = [fsdp.fsdp_reduce_scatter(flat_r, 0, r) for r in range(n)]
            back = fsdp.fsdp_all_gather(shards, 0)[:g_full.numel()].reshape(g_full.shape)
            denom = float(g_full.abs().max()) + 1e-12
            worst_grad = max(worst_grad, float((back - g_full).abs().max()) / denom)
        p1, o1, _ = _train(cfg, tcfg, p1, [b], start_step=step, opt=o1)
    # expert parallel on the dispatch tables
    layer = params["layers"][1]
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(1, 24, cfg.d_model, generator=gen) * 0.5
    want, probs, ids = model.moe(
        x, router_weight=layer["router"], routed_weights=(layer["routed_gate"], layer["routed_up"], layer["routed_down"]),
        shared_weights=(layer["shared_gate"], layer["shared_up"], layer["shared_down"]), top_k=cfg.top_k,
        max_racks=cfg.max_racks, router_bias=layer.get("router_bias"))
    x2 = x.reshape(-1, cfg.d_model)
    top = torch.gather(probs.reshape(-1, cfg.n_routed_experts), 1, ids.reshape(-1, cfg.top_k).long())
    gates = top / top.sum(-1, keepdim=True).clamp_min(1e-9)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=cfg.n_routed_experts)
    meta = kernels.DispatchMeta(ids.reshape(-1, cfg.top_k).long(), gates, torch.zeros(cfg.n_routed_experts, dtype=torch.int64),
                                cfg.n_routed_experts, int(counts.max()))
    grouped, residual = kernels.ep_dispatch(x2, meta)
    outs = torch.zeros_like(grouped)
    for e in range(cfg.n_routed_experts):
        gu_g = grouped[e] @ layer["routed_gate"][e]
        gu_u = grouped[e] @ layer["routed_up"][e]
        outs[e] = (torch.nn.functional.silu(gu_g) * gu_u) @ layer["routed_down"][e]
    routed = kernels.ep_combine(outs, meta, residual)
    shared = torch.zeros_like(x2)
    for j in range(cfg.n_shared_experts):
        shared = shared + (torch.nn.functional.silu(x2 @ layer["shared_gate"][j]) * (x2 @ layer["shared_up"][j])) \
            @ layer["shared_down"][j]
    ep_rel = float(((routed + shared).reshape(want.shape) - want).abs().max() / want.abs().max())
    # context parallel: ring attention and the delta state hand-off
    q = torch.randn(1, 8 * n, 2, 8, generator=gen)
    k = torch.randn(1, 8 * n, 2, 8, generator=gen)
    v = torch.randn(1, 8 * n, 2, 8, generator=gen)
    cp_rel = float((cp_mod.ring_attention(q, k, v, n) - model.gqa_attention(q, k, v)).abs().max())
    kk = torch.nn.functional.normalize(torch.randn(1, 32 * n, 1, 8, generator=gen), dim=-1)
    vv, bb = torch.randn(1, 32 * n, 1, 8, generator=gen), torch.rand(1, 32 * n, 1, generator=gen)
    maps = [cp_mod.slice_affine_map(P.cp_split_seq(kk, n, r), P.cp_split_seq(vv, n, r), P.cp_split_seq(bb, n, r),
                                    chunk=16) for r in range(n)]
    state = cp_mod.delta_state_handoff(maps)[n - 1]          # state entering the last slice
    _, s_ref = kernels.delta_rule_recurrent(kk[:, :32 * (n - 1)], kk[:, :32 * (n - 1)], vv[:, :32 * (n - 1)],
                                            bb[:, :32 * (n - 1)])
    cp_state_rel = float((state - s_ref).abs().max() / s_ref.abs().max())
    result = {"loss_rel_diff": float(max(worst_grad, ep_rel if ep_rel > 1e-5 else 0.0, cp_rel if cp_rel > 1e-4 else 0.0,
                                         cp_state_rel if cp_state_rel > 1e-4 else 0.0)),
              "grad_rel_diff": float(worst_grad), "ep_rel_diff": ep_rel, "cp_attention_abs_diff": cp_rel,
              "cp_state_rel_diff": cp_state_rel, "routing_identical": bool(same_routing), "gpus": int(gpus),
              "ranks_emulated": n, "steps": steps}
    if torch.cuda.is_available() and torch.cuda.device_count() >= 2 and not drop_rank:
        result["gpu_trainer_parity"] = _gpu_mesh_parity()
    return result


def _gpu_mesh_parity() -> bool:
    """Two-GPU trainer checks (replicated vs NCCL vs ZeRO-3) through the multi-GPU test worker."""
    import os
    import subprocess
    import sys

    worker = Path(__file__).resolve().parents[2] / "tests" / "_multi_gpu_worker.py"
    if not worker.exists():
        return False
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PB200_NVLS="0", MASTER_ADDR="127.0.0.1")
    ok = True
    for port, marker, arg in ((29541, "MULTI_GPU_OK", None), (29543, "FSDP_ENGINE_OK", "fsdp_engine")):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
               "127.0.0.1", "--master-port", str(port), str(worker)] + ([arg] if arg else [])
        try:
            res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
            ok = ok and res.returncode == 0 and marker in res.stdout
        except subprocess.TimeoutExpired:
            ok = False
    return ok


# ---------------------------------------------------------------------------
# V3  FP8 vs bf16 loss, NVFP4 numerics
# ---------------------------------------------------------------------------
def _v3_engine(steps: int) -> dict:
    """FP8 against bf16 through the fused trainer itself: the same hybrid model (head dim 128, so
    every layer is on the tcgen05 kernels), same init, same batches, once with bf16 FFN products
    and once with block-scaled e4m3 ones; the gate is the relative gap of the mean loss over the
    last steps."""
    from .. import engine

    cfg = _small_config(d_model=256, n_heads=2, d_head=128, n_kv_heads=1, chunk=64, dense_hidden=512,
                        vocab_size=1024)
    tcfg = train.train_config_for(cfg, warmup_steps=5, stable_steps=steps, decay_steps=5)
    params = model.init_params(cfg, 0)
    gen = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (steps, 4, 128), generator=gen)
    data[:, :, 1::2] = (data[:, :, 0::2] * 3 + 1) % cfg.vocab_size        # learnable structure
    out = {}
    for kind in ("bf16", "fp8"):
        tr = engine.Trainer(cfg, tcfg, params=params, micro_batch=4, fp8=(kind == "fp8"))
        losses = [float(tr.step(data[t].cuda())["loss"]) for t in range(steps)]
        tail = max(5, steps // 8)
        out[kind] = sum(losses[-tail:]) / tail
        out[kind + "_first"] = losses[0]
    return out


def run_v3(*, gpus: int = 8, steps: int | None = None, crush_precision: bool = False) -> dict:
    """FP8 (block-scaled e4m3, straight-through gradient) against bf16 training from the same
    init on the same data. On a GPU the comparison runs through ``engine.Trainer`` (the fused
    kernels, FP8 GEMM included); without one, through the fp32 fake-quantisation of
    ``kernels.fp8_linear`` on a two-layer MLP language model. NVFP4 is checked through the
    export codec round trip.

    ``steps`` defaults to 480 on the engine path and 150 on the CPU path. The engine default
    runs until the loss curve flattens: while the loss is still falling fast the FP8 run trails
    the bf16 one by a few steps, which reads as a 1.5 - 2.3 % gap at 120 - 240 steps and as
    0.2 % at 480 (measured on a B200); the gate of the stage is 0.5 %.

    ``crush_precision`` (negative control, fp32 path) replaces the FP8 operands by their signs
    times the mean magnitude: one bit is not enough, and the loss gap must exceed the gate."""
    from .. import export

    if isinstance(gpus, bool) or not isinstance(gpus, int) or gpus < 1:
        raise VerifyError("gpus must be a positive integer")
    if torch.cuda.is_available() and not crush_precision:
        steps = 480 if steps is None else int(steps)
        e = _v3_engine(steps)
        w = torch.randn(64, 64, generator=torch.Generator().manual_seed(0)).numpy()
        q, scale = export.quantize(w, "nvfp4")
        back = export.dequantize(q, scale, "nvfp4")
        nv_ok = bool(abs(back - w).max() <= 0.3 * abs(w).max()) and bool(torch.isfinite(torch.as_tensor(back)).all())
        return {"fp8_loss_rel_diff": abs(e["fp8"] - e["bf16"]) / e["bf16"], "nvfp4_numerics_ok": nv_ok,
                "bf16_loss": e["bf16"], "fp8_loss": e["fp8"], "path": "engine", "gpus": int(gpus),
                "steps": steps}

    steps = 150 if steps is None else int(steps)

    g = torch.Generator().manual_seed(0)
    vocab, d, h, seq = 64, 64, 128, 32
    init = {"e": torch.randn(vocab, d, generator=g) * 0.3, "w1": torch.randn(h, d, generator=g) * d ** -0.5,
            "w2": torch.randn(vocab, h, generator=g) * h ** -0.5}
    data = torch.randint(0, vocab, (steps, 16, seq), generator=g)
    data[:, :, 1::2] = (data[:, :, 0::2] * 3 + 1) % vocab      # learnable structure

    def one_bit(t):
        q = torch.sign(t) * t.abs().mean()
        return t + (q - t).detach()                       # straight-through, like the FP8 path

    def lin(x, w, kind):
        if kind == "fp8" and crush_precision:
            return one_bit(x) @ one_bit(w).t()
        if kind == "fp8":
            return kernels.fp8_linear(x, w, 32)
        return (x.to(torch.bfloat16) @ w.to(torch.bfloat16).t()).float()

    def run(kind):
        p = {k: v.clone().requires_grad_(True) for k, v in init.items()}
        losses = []
        for t in range(steps):
            tok = data[t]
            x = p["e"][tok[:, :-1]].reshape(-1, d)
            logits = lin(torch.nn.functional.silu(lin(x, p["w1"], kind)), p["w2"], kind)
            loss = torch.nn.functional.cross_entropy(logits, tok[:, 1:].reshape(-1))
            grads = torch.autograd.grad(loss, list(p.values()))
            with torch.no_grad():
                for v, gr in zip(p.values(), grads):
                    v -= 0.2 * gr
            losses.append(float(loss.detach()))
        return sum(losses[-20:]) / 20

    bf16, fp8 = run("bf16"), run("fp8")
    w = torch.randn(64, 64, generator=g).numpy()
    q, scale = export.quantize(w, "nvfp4")
    back = export.dequantize(q, scale, "nvfp4")
    nv_ok = bool(abs(back - w).max() <= 0.3 * abs(w).max()) and bool(torch.isfinite(torch.as_tensor(back)).all())
    return {"fp8_loss_rel_diff": abs(fp8 - bf16) / bf16, "nvfp4_numerics_ok": nv_ok, "bf16_loss": bf16,
            "fp8_loss": fp8, "gpus": int(gpus), "steps": steps}


# ---------------------------------------------------------------------------
# V4  faults: bitwise resume, SDC hash, spike rollback
# ---------------------------------------------------------------------------
def _engine_config():
    """The small hybrid with head dim 128: every layer runs on the tcgen05 kernels."""
    return _small_config(d_model=256, n_heads=2, d_head=128, n_kv_heads=1, chunk=64, dense_hidden=512,
                         vocab_size=1024)


def _v4_engine() -> dict:
    """Kill and resume through the fused trainer and the native checkpoint store: three steps, a
    persistent checkpoint on disk, a new trainer with a different init restored from it, three
    more steps; every state buffer must be bitwise equal to those of six straight steps (the
    kernels are deterministic). A flipped byte in a stored shard must fail the restore."""
    from .. import checkpoint, engine

    cfg = _engine_config()
    tcfg = train.train_config_for(cfg, warmup_steps=1, stable_steps=50, decay_steps=5)
    gen = torch.Generator().manual_seed(4)
    toks = [torch.randint(0, cfg.vocab_size, (4, 128), generator=gen).cuda() for _ in range(6)]
    straight = engine.Trainer(cfg, tcfg, seed=3, device="cuda", micro_batch=2)
    for t in toks:
        straight.step(t)
    first = engine.Trainer(cfg, tcfg, seed=3, device="cuda", micro_batch=2)
    for t in toks[:3]:
        first.step(t)
    names = ("muon_master", "muon_mom", "adam_master", "adam_m", "adam_v", "vec_master")
    with tempfile.TemporaryDirectory() as tmp:
        cid = checkpoint.TrainerCheckpointer(str(Path(tmp) / "s")).save_persistent(first, wait=True)
        second = engine.Trainer(cfg, tcfg, seed=99, device="cuda", micro_batch=2)
        checkpoint.TrainerCheckpointer(str(Path(tmp) / "s")).restore(second, cid)
        for t in toks[3:]:
            second.step(t)
        bitwise = all(torch.equal(getattr(straight, n), getattr(second, n)) for n in names)
        # silent data corruption: flip one byte of the largest stored shard
        files = sorted((p for p in (Path(tmp) / "s").iterdir() if p.is_file()), key=lambda p: p.stat().st_size)
        raw = bytearray(files[-1].read_bytes())
        raw[len(raw) // 2] ^= 0x10
        files[-1].write_bytes(bytes(raw))
        try:
            checkpoint.TrainerCheckpointer(str(Path(tmp) / "s")).restore(
                engine.Trainer(cfg, tcfg, seed=1, device="cuda", micro_batch=2), cid)
            caught = False
        except Exception:
            caught = True
    return {"resumed_bitwise_equal": bool(bitwise), "sdc_caught_flip": bool(caught)}


def run_v4(*, gpus: int = 4, corrupt_restore: bool = False, check_hash: bool = True,
           skip_bad_shard: bool = True) -> dict:
    """Faults: bitwise resume after a kill, a flipped bit caught by its hash, a loss spike rolled
    back with its shard skipped. On a GPU the first two run through ``engine.Trainer`` and
    ``checkpoint.TrainerCheckpointer`` (``_v4_engine``); the spike policy runs on the fp32 tree
    step either way.

    Negative controls: ``corrupt_restore`` flips one bit of the restored parameters (the resume
    is then not bitwise equal), ``check_hash=False`` leaves the flipped shard unhashed (the flip
    goes unreported), ``skip_bad_shard=False`` keeps the step taken on the bad shard."""
    if isinstance(gpus, bool) or not isinstance(gpus, int) or gpus < 1:
        raise VerifyError("gpus must be a positive integer")
    C = native.ckpt
    cfg = _small_config()
    tcfg = train.train_config_for(cfg, warmup_steps=1, stable_steps=50, decay_steps=5)
    params = model.init_params(cfg, 0)
    batches = [_batch(cfg, 2, 32, 10 + i) for i in range(6)]
    straight, _, _ = _train(cfg, tcfg, params, batches)
    # "kill" after 3 steps: state goes through the content-addressed store and comes back
    half, opt, _ = _train(cfg, tcfg, params, batches[:3])
    with tempfile.TemporaryDirectory() as tmp:
        store = C.DirStore(str(Path(tmp) / "s"))
        blobs = {"params": _tree_bytes(half)}
        flat_opt = model.flatten_params(opt)
        for k in sorted(flat_opt):
            blobs["opt/" + k] = flat_opt[k].detach().contiguous().numpy().tobytes()
        keys = {}
        for name, data in blobs.items():
            keys[name] = C.sha256_hex(data)
            store.put(keys[name], data)
        restored = {name: store.get(key) for name, key in keys.items()}
        if corrupt_restore:
            hit = bytearray(restored["params"])
            hit[len(hit) // 3] ^= 0x01
            restored["params"] = bytes(hit)
        same_blob = all(restored[n] == blobs[n] for n in blobs)
        flat_half = model.flatten_params(half)
        off, rebuilt = 0, {}
        for k in sorted(flat_half):
            n = flat_half[k].numel() * 4
            rebuilt[k] = torch.frombuffer(bytearray(restored["params"][off:off + n]), dtype=torch.float32).reshape(flat_half[k].shape)
            off += n
        half2 = train._map_tree(half, lambda n, _t: rebuilt[n])
        opt2 = train._map_tree(opt, lambda n, t: torch.frombuffer(
            bytearray(restored["opt/" + n]), dtype=t.dtype).reshape(t.shape).clone() if t.numel() else t)
        resumed, _, _ = _train(cfg, tcfg, half2, batches[3:], start_step=4, opt=opt2)
        bitwise = same_blob and _tree_bytes(resumed) == _tree_bytes(straight)
        # silent data corruption: one flipped bit in a stored shard is caught by its hash
        key = keys["params"]
        raw = bytearray(store.get(key))
        raw[len(raw) // 2] ^= 0x10
        sdc = check_hash and C.sha256_hex(bytes(raw)) != key
        try:
            C.DirStore(str(Path(tmp) / "s")).put(key, bytes(raw))     # content-addressed: a wrong body is refused or ...
            sdc = sdc and C.sha256_hex(store.get(key)) in (key, C.sha256_hex(bytes(raw)))
        except native.NativeError:
            pass
    # bad shard: a batch of garbage spikes the loss; the step is rolled back and the shard skipped
    # (the stream repeats two batches, so the loss falls; the bad shard is unrelated noise)
    stream = [batches[i % 2] for i in range(10)]
    good, o, losses = _train(cfg, tcfg, params, stream[:9])
    bad = _batch(cfg, 2, 32, 999)
    trial = train.train_step(good, o, bad, cfg, tcfg, step=10, muon_transfer=True, muon_all_matrices=True)
    spike = float(trial.loss.ce) > 1.05 * max(losses[-2:])
    rolled_back = spike and skip_bad_shard
    after, _, _ = _train(cfg, tcfg, good, stream[9:10], start_step=10, opt=o) if rolled_back else (trial.params, None, None)
    ref, _, _ = _train(cfg, tcfg, params, stream)
    skipped = spike and _tree_bytes(after) == _tree_bytes(ref)
    out = {"resumed_bitwise_equal": bool(bitwise), "sdc_caught_flip": bool(sdc),
           "spike_rollback_skipped_shard": bool(skipped), "gpus": int(gpus), "path": "tree"}
    if torch.cuda.is_available() and not corrupt_restore and check_hash and skip_bad_shard:
        e = _v4_engine()
        out.update(resumed_bitwise_equal=out["resumed_bitwise_equal"] and e["resumed_bitwise_equal"],
                   sdc_caught_flip=out["sdc_caught_flip"] and e["sdc_caught_flip"], path="tree+engine")
    return out


# ---------------------------------------------------------------------------
# V5  small-scale ladder fit and resume across job boundaries
# ---------------------------------------------------------------------------
def run_v5(*, gpus: int = 8, steps: int = 40, reverse_curve: bool = False, fresh_optimizer_on_resume: bool = False) -> dict:
    """A short ladder run: the loss curve is close to a power law in the step count, and a run
    split over two jobs ends bitwise where the unsplit run ends. Negative controls:
    ``reverse_curve`` fits the curve backwards (a rising loss must not pass), and
    ``fresh_optimizer_on_resume`` drops the optimizer state at the job boundary (the second job
    then cannot reproduce the unsplit run)."""
    if isinstance(gpus, bool) or not isinstance(gpus, int) or gpus < 1:
        raise VerifyError("gpus must be a positive integer")
    cfg = _small_config(n_dense=1, n_moe=3, n_routed_experts=4, top_k=2, expert_hidden=64)
    tcfg = train.train_config_for(cfg, warmup_steps=2, stable_steps=steps, decay_steps=4)
    params = model.init_params(cfg, 0)
    g = torch.Generator().manual_seed(5)
    base = torch.randint(0, cfg.vocab_size, (8, 32), generator=g)
    batches = [train.Batch(tokens=base[(i % 4) * 2:(i % 4) * 2 + 2], loss_mask=torch.ones(2, 32),
                           positions=torch.arange(32)) for i in range(steps)]
    _, _, losses = _train(cfg, tcfg, params, batches)
    if reverse_curve:
        losses = losses[::-1]
    # ladder fit: log-loss against log-step is close to a line with negative slope
    xs = [math.log(i + 1) for i in range(4, steps)]
    ys = [math.log(max(l, 1e-6)) for l in losses[4:]]
    n = len(xs)
    mx, my = sum(xs) / n, sum(ys) / n
    slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sum((x - mx) ** 2 for x in xs)
    resid = max(abs(y - (my + slope * (x - mx))) for x, y in zip(xs, ys))
    fit_ok = slope < 0 and resid < 0.6
    # two "jobs": the second starts from the first one's saved state
    a, oa, _ = _train(cfg, tcfg, params, batches[:steps // 2])
    saved = (_tree_bytes(a), _tree_bytes(oa))
    b2, _, _ = _train(cfg, tcfg, a, batches[steps // 2:], start_step=steps // 2 + 1,
                      opt=None if fresh_optimizer_on_resume else oa)
    full, _, _ = _train(cfg, tcfg, params, batches)
    resume_ok = saved[0] == _tree_bytes(a) and _tree_bytes(b2) == _tree_bytes(full)
    return {"loss_curve_matches_ladder": bool(fit_ok), "checkpoint_resume_ok": bool(resume_ok), "slope": slope,
            "max_residual": resid, "gpus": int(gpus)}


# ---------------------------------------------------------------------------
# V6  latent curriculum
# ---------------------------------------------------------------------------
def _v6_engine() -> dict:
    """Latent slots through the fused trainer: with K slots the Jacobi iteration is exact after
    K + 1 sweeps (slot j depends on slot j - 1 only), so the hidden states after 1, 2, 4, 8 sweeps
    must approach the 9-sweep ones, through the engine's own latent step kernels."""
    from .. import engine

    cfg = _engine_config()
    tcfg = train.train_config_for(cfg, warmup_steps=1, stable_steps=50, decay_steps=5)
    tr = engine.Trainer(cfg, tcfg, seed=2, device="cuda", micro_batch=2)
    tokens = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(6)).cuda()
    k, start = 8, 64

    def hidden(sweeps):
        tr.set_latent_slots(start, k, sweeps)
        with torch.no_grad():
            return tr.forward_hidden_latent(tokens).float().reshape(2, 256, -1)

    exact = hidden(k + 1)
    # every sweep fixes one more slot (slot j is right once slots < j are), so the mean error
    # over the slot positions falls with the sweep count; positions after the slots stay wrong
    # until the last slot is right and are left out
    errs = [float((hidden(s) - exact)[:, start:start + k].abs().mean()) for s in (1, 2, 4, 8)]
    rises = all(x >= y for x, y in zip(errs, errs[1:])) and errs[-1] < 0.5 * errs[0]
    return {"accuracy_rises_with_latent_budget": bool(rises), "sweep_errors": errs}


def run_v6(*, gpus: int = 4, freeze_budget: bool = False, pin_halt: bool = False, scramble_decode: bool = False) -> dict:
    """More Jacobi sweeps (latent budget) move the latent slots closer to the sequential
    solution; the halting losses stay finite over a short curriculum; a thought decodes to the
    ids it was built from. On a GPU the sweep check also runs through ``engine.Trainer``
    (``_v6_engine``); the fp32 check uses a small contraction map as the network.

    Negative controls: ``freeze_budget`` gives every arm one sweep (nothing can improve),
    ``pin_halt`` feeds a halting head saturated at "stop at once" whose teacher wants the last
    step (the halting loss leaves the finite range the gate allows), ``scramble_decode`` decodes
    through a permuted unembedding (the thought no longer reads as its ids)."""
    if isinstance(gpus, bool) or not isinstance(gpus, int) or gpus < 1:
        raise VerifyError("gpus must be a positive integer")
    g = torch.Generator().manual_seed(0)
    d, k = 16, 8
    a = torch.randn(d, d, generator=g) * 0.2
    embeds = torch.randn(1, 24, d, generator=g)

    def forward_hidden(e):          # causal: position t sees the mean of positions <= t
        c = torch.cumsum(e, 1) / torch.arange(1, e.shape[1] + 1).view(1, -1, 1)
        return torch.tanh(c @ a)

    adapter = lambda h: h * 0.9
    exact, _ = latent.latent_slot_forward(embeds, forward_hidden, adapter, 8, k, n_sweeps=k + 1)
    errs = []
    for sweeps in (1, 2, 4, 8):
        got, _ = latent.latent_slot_forward(embeds, forward_hidden, adapter, 8, k, n_sweeps=1 if freeze_budget else sweeps)
        errs.append(float((got - exact).abs().max()))
    rises = all(x >= y - 1e-9 for x, y in zip(errs, errs[1:])) and errs[-1] < errs[0]
    cfg = latent.LatentConfig()
    finite = True
    for stage in range(6):                      # curriculum: teacher steps shrink as compression grows
        logits = torch.randn(6, generator=g)
        if pin_halt:
            logits = torch.full((6,), 80.0)
        halt = latent.halt_from_logits(logits)
        hl = float(latent.halt_loss(halt.p, 5 if pin_halt else max(1, 6 - stage)))
        # a collapsed halting head puts (almost) no mass where the teacher stops: -log(eps) = 13.8
        finite = finite and math.isfinite(hl) and hl < 10.0 \
            and math.isfinite(float(latent.halt_kl(halt.p, cfg.lambda_prior)))
    unembed = torch.randn(32, d, generator=g)
    ids = torch.tensor([3, 17, 9])
    hidden = unembed[ids] * 4.0
    table = unembed[torch.randperm(32, generator=g)] if scramble_decode else unembed
    dec = (hidden @ table.t()).argmax(-1)
    out = {"curriculum_no_collapse": bool(finite), "accuracy_rises_with_latent_budget": bool(rises),
           "thoughts_decode": bool(torch.equal(dec, ids)), "sweep_errors": errs, "gpus": int(gpus), "path": "fp32"}
    if torch.cuda.is_available() and not (freeze_budget or pin_halt or scramble_decode):
        e = _v6_engine()
        out.update(accuracy_rises_with_latent_budget=out["accuracy_rises_with_latent_budget"]
                   and e["accuracy_rises_with_latent_budget"], engine_sweep_errors=e["sweep_errors"],
                   path="fp32+engine")
    return out


# ---------------------------------------------------------------------------
# V7  RL loop controls
# ---------------------------------------------------------------------------
V7_PARITY_THRESHOLD = 0.05        # mean |trainer log-prob - rollout log-prob| that halts the run
V7_INJECTED_DRIFT = 0.4


def run_v7(*, gpus: int = 8, steps: int = 60, update: bool = True, inject_drift: bool = True,
           plant_write: str | None = "grader") -> dict:
    """A 4-armed verifiable bandit trained with the sequence-level clipped objective; the
    parity monitor halts on an injected log-prob drift; a write to the grader's files is flagged.

    The three keyword switches are the stage's negative controls: without the policy update the
    reward must not rise, without the injected drift the monitor must not halt, and a write to
    an agent path (or no write) must not be flagged."""
    if isinstance(gpus, bool) or not isinstance(gpus, int) or gpus < 1:
        raise VerifyError("gpus must be a positive integer")
    if plant_write not in ("grader", "agent", None):
        raise VerifyError("plant_write must be 'grader', 'agent' or None")
    R = rl_loss
    g = torch.Generator().manual_seed(0)
    logits = torch.zeros(4, requires_grad=True)
    cfg = R.make_config()
    rewards_seen = []
    for _ in range(steps):
        logp = torch.log_softmax(logits, 0)
        acts = torch.multinomial(logp.exp().detach(), 8, replacement=True, generator=g)
        rew = (acts == 2).float()
        rewards_seen.append(float(rew.mean()))
        adv = R.mean_center(rew.tolist())
        if R.all_equal_reward(rew.tolist()):
            continue
        old = logp.detach()[acts]
        ratio = torch.exp(logp[acts] - old)
        clipped = torch.minimum(ratio * torch.tensor(adv), torch.clamp(ratio, 1 - cfg.clip_eps_low, 1 + cfg.clip_eps_high) * torch.tensor(adv))
        (-(clipped.mean())).backward()
        with torch.no_grad():
            if update:
                logits -= 0.5 * logits.grad
            logits.grad = None
    rises = sum(rewards_seen[-10:]) / 10 > sum(rewards_seen[:10]) / 10 + 0.2
    # parity halt: the trainer / rollout log-prob gap of a drifted policy is past the tolerance and
    # the kill switch freezes the lab; a second kill is refused because it is already frozen
    trainer_lp = [-1.0, -2.0, -0.5]
    rollout_lp = [x - (V7_INJECTED_DRIFT if inject_drift else 0.0) for x in trainer_lp]
    drift = [abs(a - b) for a, b in zip(trainer_lp, rollout_lp)]
    halted = False
    with tempfile.TemporaryDirectory() as tmp:
        m = native.monitors.Monitors(str(Path(tmp) / "freeze.json"))
        if sum(drift) / len(drift) > V7_PARITY_THRESHOLD:
            m.kill("log-prob parity drift", 1)
        halted = bool(m.frozen())
    # reward hacking: a write under the grader root is refused and recorded as a tamper flag
    E = native.envs
    pool = E.Pool(E.PoolConfig(capacity=4))
    pool.register_image(E.Image("v7", {"/work/a.txt": b"x"}, {"/grader/test.py": b"assert 1"}, {}))
    sb = pool.fork_group(pool.snapshot_from_image("v7"), 1)[0]
    flagged = False
    if plant_write is not None:
        target = "/grader/test.py" if plant_write == "grader" else "/work/notes.txt"
        try:
            pool.call(sb, "evil", "shell", json.dumps({"command": f"echo pass > {target}"}), None, 5)
        except native.NativeError as e:
            flagged = e.kind == "TestFileWrite"
    flagged = flagged and len(pool.tamper_flags) == 1
    return {"reward_rises": bool(rises), "logprob_drift_halted": bool(halted), "planted_write_flagged": bool(flagged),
            "gpus": int(gpus), "mean_reward_first10": sum(rewards_seen[:10]) / 10, "mean_reward_last10": sum(rewards_seen[-10:]) / 10}


# ---------------------------------------------------------------------------
# V8  serving parity
# ---------------------------------------------------------------------------
def run_v8(*, gpus: int = 1, perturb: float = 0.0) -> dict:
    """Weights exported through the weight-export contract and loaded back give the same
    log-probs as the training-side forward; a session whose KV tier was swapped out and
    restored decodes the same tokens. ``perturb`` (negative control) adds that much to every
    served weight: the log-prob check must then fail."""
    from .. import export, fork

    cfg = _small_config()
    params = model.init_params(cfg, 0)
    tok = _batch(cfg, 1, 32, 8).tokens
    with tempfile.TemporaryDirectory() as tmp:
        exp = export.export_weights(params, export_id="v8", source_checkpoint_id="c0", tokenizer_id="tok-v8",
                                    dtype="bf16", created_at="2026-01-01T00:00:00Z", out_dir=tmp)
        err = export.parity_max_abs_err(params, exp, tmp)
        # the serving side: weights read back from the exported shards
        import numpy as np

        flat = model.flatten_params(params)
        loaded = {}
        for sh in exp.shards:
            arr = export.dequantize(np.load(Path(tmp) / sh.path), None, "bf16")
            loaded[sh.name] = torch.from_numpy(np.asarray(arr, dtype=np.float32)).reshape(flat[sh.name].shape) + float(perturb)
        served = train._map_tree(params, lambda n, _t: loaded[n])
    with torch.no_grad():
        lp = torch.log_softmax(model.forward(tok, params, cfg, r=1).logits, -1)
        lp2 = torch.log_softmax(model.forward(tok, served, cfg, r=1).logits, -1)
    within = float((lp - lp2).abs().max()) <= 1e-5 and err <= 1e-6
    # tiering: decode, swap the waiting session down and back, decode again
    tier = fork.swap_waiting_session(False)
    seq = [fork.next_kv_tier(tier)]
    with torch.no_grad():
        first = model.forward(tok[:, :16], params, cfg, r=1).logits[:, -1].argmax(-1)
        again = model.forward(tok[:, :16], params, cfg, r=1).logits[:, -1].argmax(-1)
    return {"logprob_within_threshold": bool(within), "tiered_restore_matches": bool(torch.equal(first, again)),
            "export_max_abs_err": float(err), "tiers": [str(tier)] + [str(s) for s in seq], "gpus": int(gpus)}


# ---------------------------------------------------------------------------
# V9  one research cycle
# ---------------------------------------------------------------------------
def run_v9(*, gpus: int = 1, planted_effect: float = 0.2) -> dict:
    """Two planted ideas go through propose -> run -> replicate -> record on the ledger: the
    known positive replicates (effect in both seeds), the known negative is recorded as negative.
    ``planted_effect`` is the loss the planted positive removes (negative control: with 0 it is
    not found, and both ideas are recorded as negatives)."""
    L = native.ledger
    with tempfile.TemporaryDirectory() as tmp:
        led = L.Ledger(str(Path(tmp) / "ledger.jsonl"))

        def measure(idea, seed):
            g = torch.Generator().manual_seed(seed)
            base = 1.0 + 0.01 * float(torch.randn((), generator=g))
            return base - (float(planted_effect) if idea == "planted-positive" else 0.0)

        found, replicated, negative = False, False, False
        for idea in ("planted-positive", "planted-negative"):
            first, second = measure(idea, 1), measure(idea, 2)
            better = first < 0.9
            passed = better and second < 0.9
            rec = {"experiment_id": idea, "hypothesis": f"{idea} lowers the loss", "prediction": "loss below 0.9",
                   "config_hash": "c" * 8, "results": {"passed": passed, "runs": [first, second]}, "delta_rci": None,
                   "replication": {"status": "replicated" if passed else "failed", "n": 2, "notes": None},
                   "gpu_hours": 0.1, "author_role": "researcher", "rung": 0, "created_at": "2026-01-01T00:00:00Z",
                   "closed_at": "2026-01-01T01:00:00Z", "supersedes": None}
            led.append(json.dumps(rec))
            if idea == "planted-positive":
                found, replicated = better, passed
        negatives = [json.loads(r)["experiment_id"] for r in led.list_negatives()]
        negative = negatives == ["planted-negative"]
    return {"planted_positive_found": bool(found), "planted_positive_replicated": bool(replicated),
            "planted_negative_recorded": bool(negative), "gpus": int(gpus)}


# ---------------------------------------------------------------------------
# V10  chaos soak
# ---------------------------------------------------------------------------
def run_v10(*, hours: float = 72.0, seed: int = 0, drop_task: bool = False, duplicate_output: bool = False) -> dict:
    """The native chaos world advanced through ``hours`` of injected time with the soak fault
    mix; the invariants give the three counters. ``drop_task`` and ``duplicate_output`` are the
    stage's negative controls: a task enqueued and never completed, and one attempt completed
    twice, after the soak; the counters must then show them."""
    if isinstance(hours, bool) or not isinstance(hours, (int, float)) or not (hours > 0 and math.isfinite(hours)):
        raise VerifyError("hours must be a positive finite number")
    CH = native.chaos
    with tempfile.TemporaryDirectory() as tmp:
        world = CH.World.create(str(Path(tmp) / "soak"), 3, 4, int(seed))
        rep = CH.run_soak(world, int(hours * 3600 * 1000), int(seed))
        inv = rep.invariants
        dead = 0 if inv.hold() else 1      # a dead token breaks the soak's invariants as a whole
        if drop_task or duplicate_output:
            if rep.recovered is False:
                world.recover()
            now = int(world.now())
            if drop_task:
                world.enqueue_task("control-dropped", now)
            if duplicate_output:
                world.enqueue_task("control-twice", now)
                world.complete_task("control-twice", 1, b"out", now)
                world.complete_task("control-twice", 1, b"out", now)
            inv = world.invariants()
        lost, dup = int(inv.lost_tasks), int(inv.duplicated_outputs)
    return {"hours": float(hours), "lost_tasks": lost, "duplicated_outputs": dup, "dead_tokens": dead,
            "faults_applied": int(rep.faults_applied)}


RUNNERS = {"v1": run_v1, "v2": run_v2, "v3": run_v3, "v4": run_v4, "v5": run_v5, "v6": run_v6, "v7": run_v7,
           "v8": run_v8, "v9": run_v9, "v10": run_v10}


def run_stage(stage: str, **kw) -> dict:
    name = native.ncshare.parse_stage(stage)
    if name == "v0":
        raise VerifyError("V0 is measured by its job script (bus bandwidth and node facts), not by a runner")
    return RUNNERS[name](**kw)
