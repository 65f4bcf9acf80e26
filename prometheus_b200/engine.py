"""Fused sm_100a trainer: the model on flat device buffers driven by hand-written kernels.

``Trainer`` packs a parameter tree (``model.init_params`` layout) into

* fp32 master / gradient / optimizer-state flat buffers, one per optimizer group
  (Muon matrices laid out by shape class so Newton-Schulz runs as batched GEMMs;
  AdamW leaves in one slab updated by one launch), and
* a bf16 working copy in kernel layout (every projection stored ``(out, in)`` so the
  forward GEMM reads both operands K-major; gate and up projections adjacent so the
  FFN input is read once),

and runs forward / backward through ``prometheus_b200.ops`` (tcgen05 GEMM, fused
RMSNorm+residual, RoPE, SwiGLU, L2-norm, delta rule, fused soft-cap CE with the
unembedding) with weight gradients accumulated in fp32 straight into the flat
gradient buffer by the GEMM epilogue. The optimizer step is device-resident:
global-norm clip factor, momentum, Newton-Schulz and the parameter update never
synchronise with the host.

Numerics contract: same step as ``train.train_step(..., muon_transfer=True,
muon_all_matrices=True)`` with bf16 activations; tested against it.
Reference call stack being replaced: ``train/__init__.py:835-985`` ->
``model/__init__.py:803-995``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from . import model as M
from . import train as T
from .ops import _lib
from .ops import functional as ops
from .ops._lib import call, ptr, stream_ptr

Tensor = torch.Tensor
BF16 = torch.bfloat16


@dataclass
class Unit:
    """One independent Muon matrix inside a packed weight: rows [r0, r0+rows) of it."""

    weight: str
    r0: int
    rows: int
    cols: int
    off: int = 0          # element offset in the Muon flat buffers


@dataclass
class Weight:
    """A packed kernel-layout tensor and where it lives in the flat buffers."""

    name: str
    shape: tuple
    group: str            # "muon" | "adam"
    lp: bool              # has a bf16 working copy (matrices); norms are used in fp32
    off: int = 0
    units: list = field(default_factory=list)
    sources: list = field(default_factory=list)   # [(tree_name, row0, rows, to_engine, to_tree)]


def _t2(x: Tensor) -> Tensor:
    return x.reshape(x.shape[0], -1).t().contiguous()


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, w):
        ctx.save_for_backward(tokens)
        ctx.w_ref = w
        return w[tokens]

    @staticmethod
    def backward(ctx, dy):
        (tokens,) = ctx.saved_tensors
        mg = ctx.w_ref.main_grad
        mg.index_add_(0, tokens.reshape(-1), dy.reshape(-1, dy.shape[-1]).float())
        return None, None


class Trainer:
    """Single-process-per-GPU trainer for the dense hybrid configurations."""

    def __init__(self, model_config: M.ModelConfig, train_config: T.TrainConfig, *,
                 params: dict | None = None, seed: int = 0, device="cuda", micro_batch: int = 4,
                 muon_weight_decay: float = 0.0, process_group=None, ce_chunk_rows: int = 4096,
                 grad_sync: str = "auto"):
        M.validate_config(model_config)
        T.validate_train_config(train_config)
        if model_config.n_moe != 0:
            raise NotImplementedError("MoE layers run through prometheus_b200.parallel.ep")
        self.cfg, self.tcfg = model_config, train_config
        self.device = torch.device(device)
        self.micro_batch = int(micro_batch)
        self.muon_wd = float(muon_weight_decay)
        self.pg = process_group
        self.world = 1
        self.rank = 0
        if process_group is not None or (torch.distributed.is_available()
                                         and torch.distributed.is_initialized()):
            self.world = torch.distributed.get_world_size(process_group)
            self.rank = torch.distributed.get_rank(process_group)
        self.grad_sync = grad_sync
        self.ce_chunk_rows = int(ce_chunk_rows)
        self.step_count = 0
        self.launches = 0
        _lib.load()
        if params is None:
            params = M.init_params(model_config, seed)
        self._plan(params)
        self._allocate()
        self.load_tree(params)

    # ------------------------------------------------------------------ layout
    def _plan(self, params: dict) -> None:
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        d = cfg.d_model
        ws: list[Weight] = []

        def mat(name, shape, sources, unit_rows=None):
            w = Weight(name=name, shape=tuple(shape), group="muon", lp=True, sources=sources)
            rows, cols = shape
            if min(rows if unit_rows is None else min(unit_rows), cols) < 32:
                w.group = "adam"
            else:
                r0 = 0
                for r in (unit_rows or [rows]):
                    w.units.append(Unit(weight=name, r0=r0, rows=r, cols=cols))
                    r0 += r
            ws.append(w)

        def vec(name, n, tree_name):
            ws.append(Weight(name=name, shape=(n,), group="adam", lp=False,
                             sources=[(tree_name, 0, n, None, None)]))

        def src(tree_name, r0, rows):
            return (tree_name, r0, rows, "t2", None)

        ws.append(Weight("embed", (cfg.vocab_size, d), "adam", True,
                         sources=[("embed", 0, cfg.vocab_size, None, None)]))
        ws.append(Weight("unembed", (cfg.vocab_size, d), "adam", True,
                         sources=[("unembed", 0, cfg.vocab_size, None, None)]))
        vec("final_norm", d, "final_norm")
        self.layer_kinds = []
        for i in range(cfg.n_layers):
            p = f"layers.{i}."
            kind = M.attention_kind(i, cfg)
            self.layer_kinds.append(kind)
            vec(p + "pre_attn_norm", d, p + "pre_attn_norm")
            vec(p + "pre_ffn_norm", d, p + "pre_ffn_norm")
            if kind is M.AttentionKind.MLA:
                raise NotImplementedError("the fused engine runs linear and GQA layers")
            kvh = nh if kind is M.AttentionKind.LINEAR else nkv
            mat(p + "q", (nh * dh, d), [src(p + "W_q", 0, nh * dh)])
            mat(p + "k", (kvh * dh, d), [src(p + "W_k", 0, kvh * dh)])
            mat(p + "v", (kvh * dh, d), [src(p + "W_v", 0, kvh * dh)])
            if kind is M.AttentionKind.LINEAR and cfg.delta_beta == "sigmoid":
                mat(p + "beta", (nh, d), [src(p + "W_beta", 0, nh)])
            mat(p + "o", (d, nh * dh), [(p + "W_o", 0, d, "o", None)])
            hid = cfg.dense_hidden if cfg.dense_hidden is not None else cfg.expert_hidden
            mat(p + "gate_up", (2 * hid, d),
                [src(p + "ffn_gate", 0, hid), src(p + "ffn_up", hid, hid)], unit_rows=[hid, hid])
            mat(p + "down", (d, hid), [src(p + "ffn_down", 0, d)])
        self.weights = {w.name: w for w in ws}
        # Muon flat layout: units grouped by (rows, cols) so each class is one batched NS.
        classes: dict[tuple, list[Unit]] = {}
        for w in ws:
            for u in w.units:
                classes.setdefault((u.rows, u.cols), []).append(u)
        self.unit_classes = classes
        off = 0
        for key in sorted(classes):
            for u in classes[key]:
                u.off = off
                off += u.rows * u.cols
        self.n_muon = off
        # A packed Muon weight must be contiguous in the flat buffer: its units are adjacent
        # when they share a shape class and were appended consecutively (gate, up).
        for w in ws:
            if w.group == "muon":
                w.off = w.units[0].off
                for a, b in zip(w.units, w.units[1:]):
                    assert b.off == a.off + a.rows * a.cols
        off = 0
        for w in ws:
            if w.group == "adam":
                w.off = off
                off += int(math.prod(w.shape))
                off = (off + 7) // 8 * 8
        self.n_adam = off

    def _allocate(self) -> None:
        dev = self.device
        f32 = dict(dtype=torch.float32, device=dev)
        self.muon_master = torch.zeros(self.n_muon, **f32)
        self.muon_grad = torch.zeros(self.n_muon, **f32)
        self.muon_mom = torch.zeros(self.n_muon, **f32)
        self.muon_lp = torch.zeros(self.n_muon, dtype=BF16, device=dev)
        self.adam_master = torch.zeros(self.n_adam, **f32)
        self.adam_grad = torch.zeros(self.n_adam, **f32)
        self.adam_m = torch.zeros(self.n_adam, **f32)
        self.adam_v = torch.zeros(self.n_adam, **f32)
        self.adam_lp = torch.zeros(self.n_adam, dtype=BF16, device=dev)
        max_unit = max((r * c * len(us) for (r, c), us in self.unit_classes.items()),
                       default=1)
        self.ns_x = [torch.empty(max_unit, dtype=BF16, device=dev) for _ in range(2)]
        max_g = max((min(r, c) ** 2 * len(us) for (r, c), us in self.unit_classes.items()),
                    default=1)
        self.ns_g = [torch.empty(max_g, dtype=BF16, device=dev) for _ in range(2)]
        nparts = max(_lib.query("pb_sumsq_nparts", max(self.n_muon, self.n_adam, 1)), 1)
        self.opt_scratch = torch.empty(nparts + 8, **f32)
        self.gnorm_sq = torch.zeros(1, **f32)
        self.p: dict[str, Tensor] = {}
        for w in self.weights.values():
            n = int(math.prod(w.shape))
            master = self.muon_master if w.group == "muon" else self.adam_master
            grad = self.muon_grad if w.group == "muon" else self.adam_grad
            lpbuf = self.muon_lp if w.group == "muon" else self.adam_lp
            t = (lpbuf if w.lp else master)[w.off:w.off + n].view(w.shape)
            t.requires_grad_(True)
            t.main_grad = grad[w.off:w.off + n].view(w.shape)
            t.master = master[w.off:w.off + n].view(w.shape)
            self.p[w.name] = t

    # ------------------------------------------------------------ tree <-> flat
    @staticmethod
    def _to_engine(t: Tensor, how) -> Tensor:
        if how == "t2":
            return _t2(t)
        if how == "o":
            return t.reshape(-1, t.shape[-1]).t().contiguous()
        return t

    def load_tree(self, params: dict) -> None:
        """Copy a parameter tree (reference layout) into the flat buffers."""
        flat = M.flatten_params(params)
        with torch.no_grad():
            for w in self.weights.values():
                dst = self.p[w.name].master
                for tree_name, r0, rows, how, _ in w.sources:
                    src = self._to_engine(flat[tree_name].detach().float(), how)
                    dst[r0:r0 + rows].copy_(src.to(self.device))
            self.muon_lp.copy_(self.muon_master)
            self.adam_lp.copy_(self.adam_master)

    def export_tree(self) -> dict:
        """Parameter tree (reference layout, fp32, on CPU) from the master buffers."""
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        out: dict[str, Tensor] = {}
        for w in self.weights.values():
            src = self.p[w.name].master.detach().cpu()
            for tree_name, r0, rows, how, _ in w.sources:
                blk = src[r0:r0 + rows]
                if how == "t2":
                    t = blk.t().contiguous()
                    leaf = tree_name.split(".")[-1]
                    if leaf in ("W_q", "W_k", "W_v"):
                        t = t.reshape(t.shape[0], -1, dh)
                elif how == "o":
                    t = blk.t().contiguous().reshape(nh, dh, cfg.d_model)
                else:
                    t = blk.clone()
                out[tree_name] = t
        return M.unflatten_params(out)

    # ------------------------------------------------------------------ forward
    def _delta_layer(self, n: Tensor, i: int, B: int, S: int) -> Tensor:
        from . import kernels

        cfg = self.cfg
        nh, dh, _ = M.head_geometry(cfg)
        pre = f"layers.{i}."
        q = ops.linear(n, self.p[pre + "q"]).view(B, S, nh, dh)
        k = ops.linear(n, self.p[pre + "k"]).view(B, S, nh, dh)
        v = ops.linear(n, self.p[pre + "v"]).view(B, S, nh, dh)
        q, k = ops.l2norm(q), ops.l2norm(k)
        if cfg.delta_beta == "sigmoid":
            wb = self.p[pre + "beta"]
            beta = torch.sigmoid(_SmallLinear.apply(n, wb)).view(B, S, nh)
        else:
            beta = torch.ones((B, S, nh), dtype=BF16, device=n.device)
        o, _ = kernels.chunked_delta_rule(q, k, v, beta, None,
                                          kernels.LinearAttnConfig(chunk=cfg.chunk))
        return ops.linear(o.reshape(B * S, nh * dh), self.p[pre + "o"])

    def _gqa_layer(self, n: Tensor, i: int, B: int, S: int) -> Tensor:
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        pre = f"layers.{i}."
        q = ops.linear(n, self.p[pre + "q"]).view(B, S, nh, dh)
        k = ops.linear(n, self.p[pre + "k"]).view(B, S, nkv, dh)
        v = ops.linear(n, self.p[pre + "v"]).view(B, S, nkv, dh)
        q = ops.rope_(q, seq_len=S, base=cfg.rope_base)
        k = ops.rope_(k, seq_len=S, base=cfg.rope_base)
        from .ops import attention

        o = attention.causal_gqa(q, k, v)
        return ops.linear(o.reshape(B * S, nh * dh), self.p[pre + "o"])

    def forward_hidden(self, tokens: Tensor, inputs_embeds: Tensor | None = None) -> Tensor:
        """Final-norm hidden states (B*S, d) in bf16 for a (B, S) token batch."""
        cfg = self.cfg
        B, S = tokens.shape
        if inputs_embeds is None:
            h = _EmbedFn.apply(tokens, self.p["embed"]).reshape(B * S, cfg.d_model)
        else:
            h = inputs_embeds.reshape(B * S, cfg.d_model)
        n = ops.rmsnorm(h, self.p["layers.0.pre_attn_norm"])
        for i in range(cfg.n_layers):
            pre = f"layers.{i}."
            if self.layer_kinds[i] is M.AttentionKind.LINEAR:
                a = self._delta_layer(n, i, B, S)
            else:
                a = self._gqa_layer(n, i, B, S)
            n2, h = ops.add_rmsnorm(a, h, self.p[pre + "pre_ffn_norm"])
            gu = ops.linear(n2, self.p[pre + "gate_up"])
            f = ops.linear(ops.swiglu(gu), self.p[pre + "down"])
            nxt = f"layers.{i + 1}.pre_attn_norm" if i + 1 < cfg.n_layers else "final_norm"
            n, h = ops.add_rmsnorm(f, h, self.p[nxt])
        return n

    def loss(self, tokens: Tensor, loss_mask: Tensor, denom: Tensor | float) -> Tensor:
        """Masked mean next-token CE (soft-capped) of one micro-batch, scaled by 1/denom."""
        B, S = tokens.shape
        hid = self.forward_hidden(tokens)
        targets = torch.roll(tokens, -1, dims=1).reshape(-1).to(torch.int32)
        wt = loss_mask.float().clone()
        wt[:, 0] = 0.0                          # mask[:, 1:] aligned to the predicting position
        wt = torch.roll(wt, -1, dims=1).reshape(-1) / denom
        return ops.softcap_cross_entropy(hid, self.p["unembed"], targets, wt.contiguous(),
                                         float(self.tcfg.softcap), self.ce_chunk_rows)

    # ---------------------------------------------------------------- optimizer
    def _sync_grads(self) -> None:
        if self.world == 1:
            return
        import torch.distributed as dist

        for g in (self.muon_grad, self.adam_grad):
            dist.all_reduce(g, group=self.pg)

    def _newton_schulz_class(self, rows: int, cols: int, units: list[Unit], steps: int) -> Tensor:
        """Batched quintic Newton-Schulz over all units of one shape, in bf16 on the
        tcgen05 GEMM. Input: self.ns_x[0] holds the normalised Nesterov momenta."""
        nb = len(units)
        x = self.ns_x[0][: nb * rows * cols].view(nb, rows, cols)
        y = self.ns_x[1][: nb * rows * cols].view(nb, rows, cols)
        m = min(rows, cols)
        g = self.ns_g[0][: nb * m * m].view(nb, m, m)
        pm = self.ns_g[1][: nb * m * m].view(nb, m, m)
        a, b, c = T._NS_A, T._NS_B, T._NS_C
        wide = rows <= cols
        for _ in range(steps):
            if wide:
                ops.gemm(x, x, out=g)                                     # G = X X^T
            else:
                ops.gemm(x, x, a_mn=True, b_mn=True, out=g)               # G = X^T X
            ops.gemm(g, g, out=pm, d=g, alpha=c, beta=b)                  # P = b G + c G^2
            if wide:
                ops.gemm(pm, x, b_mn=True, out=y, d=x, alpha=1.0, beta=a)  # aX + P X
            else:
                ops.gemm(x, pm, out=y, d=x, alpha=1.0, beta=a)            # aX + X P
            x, y = y, x
            self.launches += 3
        return x

    def optimizer_step(self, lr_mult: float, gscale: float = 1.0) -> None:
        """Clip, AdamW slab, batched Muon; refreshes the bf16 working copies."""
        tc = self.tcfg
        st = stream_ptr()
        clip = float(tc.grad_clip)
        call("pb_sumsq_f32", ptr(self.muon_grad), self.n_muon, ptr(self.opt_scratch),
             ptr(self.gnorm_sq), 0, st)
        call("pb_sumsq_f32", ptr(self.adam_grad), self.n_adam, ptr(self.opt_scratch),
             ptr(self.gnorm_sq), 1, st)
        self.launches += 4
        step = self.step_count
        call("pb_adamw", ptr(self.adam_master), ptr(self.adam_grad), ptr(self.adam_m),
             ptr(self.adam_v), ptr(self.adam_lp), self.n_adam, float(tc.adamw_lr) * lr_mult,
             float(tc.adamw_beta1), float(tc.adamw_beta2), float(tc.adamw_eps),
             float(tc.adamw_wd), step, ptr(self.gnorm_sq), clip, gscale, st)
        self.launches += 1
        lr = float(tc.muon_lr) * lr_mult
        beta = float(tc.muon_momentum)
        for (rows, cols), units in sorted(self.unit_classes.items()):
            n = rows * cols
            base = units[0].off
            x0 = self.ns_x[0]
            for j, u in enumerate(units):
                assert u.off == base + j * n
                call("pb_muon_prepare", ptr(self.muon_grad[u.off:]), ptr(self.muon_mom[u.off:]),
                     ptr(x0[j * n:]), n, beta, ptr(self.gnorm_sq), clip, gscale,
                     ptr(self.opt_scratch), st)
                self.launches += 3
            xo = self._newton_schulz_class(rows, cols, units, int(tc.muon_ns_steps))
            call("pb_muon_apply", ptr(self.muon_master[base:]), ptr(xo),
                 ptr(self.muon_lp[base:]), n * len(units), lr, T.muon_rms_scale(rows, cols),
                 self.muon_wd, st)
            self.launches += 1

    def zero_grad(self) -> None:
        self.muon_grad.zero_()
        self.adam_grad.zero_()

    # --------------------------------------------------------------------- step
    def step(self, tokens: Tensor, loss_mask: Tensor | None = None) -> dict:
        """One optimizer step over a local batch (B_local, S) of token ids on the device.
        Returns device scalars: loss (mean CE over the global batch) and grad_norm."""
        self.step_count += 1
        t = self.step_count
        sched = T.wsd_lr(t, self.tcfg)
        lr_mult = sched / float(self.tcfg.peak_lr)
        if loss_mask is None:
            loss_mask = torch.ones_like(tokens, dtype=torch.float32)
        denom = loss_mask[:, 1:].sum().float()
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(denom, group=self.pg)
        denom = denom.clamp(min=1.0)
        total = torch.zeros((), dtype=torch.float32, device=tokens.device)
        mb = self.micro_batch
        for b0 in range(0, tokens.shape[0], mb):
            l = self.loss(tokens[b0:b0 + mb], loss_mask[b0:b0 + mb], denom)
            l.backward()
            total += l.detach()
        self._sync_grads()
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(total, group=self.pg)
        self.optimizer_step(lr_mult)
        gnorm = self.gnorm_sq.sqrt()
        self.zero_grad()
        return {"loss": total, "grad_norm": gnorm, "lr": sched, "step": t}


    def step_from_host(self, host_tokens: Tensor, host_mask: Tensor | None = None) -> dict:
        """Public end-to-end step: token ids (and optional mask) in pinned host memory are
        copied to the device, one optimizer step runs, and the loss and gradient norm are
        read back to the host as Python floats."""
        tok = host_tokens.to(self.device, non_blocking=True)
        mask = None if host_mask is None else host_mask.to(self.device, non_blocking=True)
        out = self.step(tok, mask)
        host = torch.stack([out["loss"], out["grad_norm"].reshape(())]).cpu()
        return {"loss": float(host[0]), "grad_norm": float(host[1]), "lr": out["lr"],
                "step": out["step"]}


class _SmallLinear(torch.autograd.Function):
    """Skinny projection (a handful of output features, e.g. the per-head write gate):
    library matmul, fp32 main-grad accumulation. Not a hot op (N = heads)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        ctx.w_ref = w
        return x @ w.t()

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        mg = getattr(ctx.w_ref, "main_grad", None)
        dw = None
        if mg is not None:
            mg.addmm_(dy.float().t(), x.float())
        else:
            dw = dy.t() @ x
        return dy @ w, dw
