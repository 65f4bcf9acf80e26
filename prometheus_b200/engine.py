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
LAZY_INIT_PARAMS = 3_000_000_000      # above this many parameters the host never holds the model


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
    local: bool = False   # expert-parallel: this rank's experts only (no gradient reduction,
                          # no broadcast of the update)


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


class _FsdpLayerHook(torch.autograd.Function):
    """Identity on a layer's output whose backward runs before any backward node of that layer:
    it makes the layer's gathered weights resident again and starts the previous layer's pull."""

    @staticmethod
    def forward(ctx, x, trainer, layer):
        ctx.trainer, ctx.layer = trainer, layer
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.trainer._fsdp_enter(ctx.layer, backward=True)
        return g, None, None


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (peer flag, barrier, mbarrier) ran out during a step: the
    gradients or weights of that step may be partial. Carries the latched code."""

    def __init__(self, code: int, rank: int, step: int):
        super().__init__(f"device-side wait timed out (code {code}) on rank {rank} at step {step}")
        self.code, self.rank, self.step = int(code), int(rank), int(step)


class Trainer:
    """Single-process-per-GPU trainer for the hybrid configurations: delta-rule and GQA
    attention layers, dense SwiGLU or mixture-of-experts (routed + shared) FFNs."""

    def __init__(self, model_config: M.ModelConfig, train_config: T.TrainConfig, *,
                 params: dict | None = None, seed: int = 0, device="cuda", micro_batch: int = 4,
                 muon_weight_decay: float = 0.0, process_group=None, ce_chunk_rows: int = 4096,
                 grad_sync: str = "auto", expert_parallel: bool = False,
                 ep_capacity_factor: float = 2.0, fp8: bool = False, context_parallel: bool = False,
                 cp_layout: str = "zigzag",
                 z_loss_mode: str = "layers_logits", router_bias_rule: str = "count",
                 allow_fallback: bool = False, fsdp: bool = False, nvls: bool | str = "auto",
                 recurrence: int = 1,
                 truncated_recurrence: int = M.TRUNCATED_RECURRENCE, check_status_every: int = 1):
        M.validate_config(model_config)
        T.validate_train_config(train_config)
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
        # ZeRO-3: bf16 working weights kept as 1/world shards in symmetric memory and gathered
        # layer by layer into two rotating landing buffers, one layer ahead of the compute;
        # fp32 masters and optimizer moments only for the matrices this rank owns
        self.fsdp = bool(fsdp) and self.world > 1
        self.comm_noop = False      # timing only: skip the peer traffic (see exposed-comm measurement)
        # replicated mode: broadcast the refreshed weights with one multimem.st through an NVLS
        # multicast object when the machine offers one ("auto": use it if it can be set up on
        # every rank, else the peer-to-peer stores; False: never)
        self.nvls_mode = nvls
        self.nvls_lp = None
        self.ep = bool(expert_parallel) and self.world > 1 and model_config.n_moe > 0
        self.ep_capacity_factor = float(ep_capacity_factor)
        # block-scaled FP8 forward for the FFN / expert products (1 x 128 activations,
        # 128 x 128 weights), straight-through bf16 backward
        self.fp8 = bool(fp8)
        # context parallelism: the ranks of the group hold consecutive slices of every sequence
        # (rank order = sequence order). Delta-rule layers hand their chunk state from rank to
        # rank over peer memory, softmax layers gather K / V and run the offset attention kernel;
        # weights and gradients are handled exactly as under data parallelism.
        self.cp = bool(context_parallel) and self.world > 1
        self.cp_ctx = None
        # "zigzag": rank r holds half-slices r and 2 world - 1 - r of every sequence, so causal
        # attention costs every rank the same and keys / values and their gradients move by this
        # package's own peer-memory kernels; "contiguous": rank order = sequence order, softmax
        # layers gather K / V through the collective library (the last rank does 1.9x the mean)
        if cp_layout not in ("zigzag", "contiguous"):
            raise ValueError("cp_layout must be 'zigzag' or 'contiguous'")
        self.cp_zigzag = self.cp and cp_layout == "zigzag"
        has_mla = any(M.attention_kind(i, model_config) is M.AttentionKind.MLA for i in range(model_config.n_layers))
        if self.cp and (model_config.mtp_heads or has_mla or expert_parallel):
            raise ValueError("context parallelism supports the delta-rule + GQA hybrids without MTP heads, "
                             "MLA layers or expert parallelism")
        # per-layer, per-head largest attention logit of the last forward (the statistic the
        # MuonClip-style QK-clip monitors); filled by the attention kernel when switched on
        self.track_max_logit = False
        self.latent_slots: tuple | None = None      # see set_latent_slots
        self.max_logits: dict[int, Tensor] = {}
        self.ep_ctx = None
        self.side_stream = None
        if self.ep and model_config.n_routed_experts % self.world:
            raise ValueError("expert parallelism needs n_routed_experts divisible by the world size")
        self.ce_chunk_rows = int(ce_chunk_rows)
        # router z-loss: "layers_logits" = mean over the MoE layer applications of
        # mean(logsumexp(router logits)^2), the model's own definition
        # (model/__init__.py:975-995 of the reference); "last_probs" = the reference train
        # step's form, the last MoE layer's sigmoid scores (train/__init__.py:785,909).
        if z_loss_mode not in ("layers_logits", "last_probs"):
            raise ValueError("z_loss_mode must be 'layers_logits' or 'last_probs'")
        self.z_loss_mode = z_loss_mode
        # aux-loss-free balancing statistic, per MoE layer: "count" = share of the top-k
        # assignments (what the dispatch really sends to an expert), "probs" = mean router
        # score per expert (the reference's rule, train/__init__.py:810).
        if router_bias_rule not in ("count", "probs"):
            raise ValueError("router_bias_rule must be 'count' or 'probs'")
        self.router_bias_rule = router_bias_rule
        # head dims the tcgen05 delta-rule / attention kernels do not cover raise unless the
        # caller opts into the PyTorch / library forms (test-sized models)
        self.allow_fallback = bool(allow_fallback)
        # depth recurrence: the core block runs `recurrence` times per forward with the prelude
        # output injected from the second iteration on; gradient flows through the last
        # `truncated_recurrence` iterations (model/__init__.py:932-970 of the reference)
        if int(recurrence) < 1 or int(truncated_recurrence) < 1:
            raise ValueError("recurrence and truncated_recurrence must be >= 1")
        self.recurrence = int(recurrence)
        self.truncated_recurrence = int(truncated_recurrence)
        # the kernels latch a status word when a bounded wait runs out; every
        # `check_status_every`-th step reads it back with the loss and raises (0: never)
        self.check_status_every = int(check_status_every)
        self.debug_canaries = False        # check the symmetric buffers' guard zones after every step
        self.time_phases = False           # record CUDA events round the phases of every step
        self.phase_times: dict[str, float] = {}
        self.collect_amax = False          # keep the largest |final hidden| of the step (FP8 range probe)
        self.amax: dict[str, Tensor] = {}
        self.router_records: list = []
        self._router_load: dict[int, Tensor] = {}
        self.moe_load: Tensor | None = None          # (MoE layers, experts) load shares, last step
        self.last_max_logits: Tensor | None = None   # (GQA layers, heads) largest logits, last step
        self.step_count = 0
        self.launches = 0
        self.router_bias: dict[int, Tensor] = {}
        self.router_bias_rate = 1e-3
        self.last_router = None
        _lib.load()
        self.seed = int(seed)
        if params is None:
            # Large models are never materialised on the host: the trainer plans from shapes and
            # draws each of its own weights on the device (an expert-parallel rank only its experts).
            shapes = M.init_params(model_config, seed, shapes_only=True)
            params = shapes if M.param_count(shapes) > LAZY_INIT_PARAMS else M.init_params(model_config, seed)
        self._plan(params)
        self._allocate()
        self.load_tree(params)

    # ------------------------------------------------------------------ layout
    def _plan(self, params: dict) -> None:
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        d = cfg.d_model
        ws: list[Weight] = []

        def mat(name, shape, sources, unit_rows=None, local=False):
            w = Weight(name=name, shape=tuple(shape), group="muon", lp=True, sources=sources,
                       local=local)
            rows, cols = shape
            if min(rows if unit_rows is None else min(unit_rows), cols) < 32 and not local:
                w.group = "adam"
            else:
                r0 = 0
                for r in (unit_rows or [rows]):
                    w.units.append(Unit(weight=name, r0=r0, rows=r, cols=cols))
                    r0 += r
            ws.append(w)

        def vec(name, n, tree_name):
            ws.append(Weight(name=name, shape=(n,), group="vec", lp=False,
                             sources=[(tree_name, 0, n, None, None)]))

        def src(tree_name, r0, rows):
            return (tree_name, r0, rows, "t2", None)

        ws.append(Weight("embed", (cfg.vocab_size, d), "adam", True,
                         sources=[("embed", 0, cfg.vocab_size, None, None)]))
        ws.append(Weight("unembed", (cfg.vocab_size, d), "adam", True,
                         sources=[("unembed", 0, cfg.vocab_size, None, None)]))
        vec("final_norm", d, "final_norm")
        for j in range(cfg.mtp_heads):
            vec(f"mtp.{j}.norm", d, f"mtp.{j}.norm")
            mat(f"mtp.{j}.proj", (d, d), [src(f"mtp.{j}.proj", 0, d)])
            ws.append(Weight(f"mtp.{j}.unembed", (cfg.vocab_size, d), "adam", True,
                             sources=[(f"mtp.{j}.unembed", 0, cfg.vocab_size, None, None)]))
        # latent adapter (thought vector -> residual stream): 2-layer SiLU MLP + RMSNorm
        ah = cfg.adapter_hidden if cfg.adapter_hidden is not None else d
        mat("adapter_w1", (ah, d), [src("adapter_w1", 0, ah)])
        mat("adapter_w2", (d, ah), [src("adapter_w2", 0, d)])
        vec("adapter_norm", d, "adapter_norm")
        self.layer_kinds = []
        self.moe_layers: list[int] = []
        for i in range(cfg.n_layers):
            p = f"layers.{i}."
            kind = M.attention_kind(i, cfg)
            self.layer_kinds.append(kind)
            vec(p + "pre_attn_norm", d, p + "pre_attn_norm")
            vec(p + "pre_ffn_norm", d, p + "pre_ffn_norm")
            if kind is M.AttentionKind.MLA:
                # keys = [up-projected compressed KV | shared rotary key], values = the
                # up-projected part (model/__init__.py:435-482, 737-750 of the reference)
                dn = dh
                dr = max(2, (dh // 2) // 2 * 2)
                self.mla_dims = (dn, dr, dh)
                mat(p + "q", (nh * (dn + dr), d), [src(p + "W_q", 0, nh * (dn + dr))])
                mat(p + "kv_c", (dh, d), [src(p + "W_kv_compress", 0, dh)])
                mat(p + "kv_up", (nh * dn, dh), [src(p + "W_kv_up", 0, nh * dn)])
                mat(p + "rope_k", (dr, d), [src(p + "W_rope_k", 0, dr)])
                mat(p + "o", (d, nh * dn), [(p + "W_o", 0, d, "o", None)])
            else:
                kvh = nh if kind is M.AttentionKind.LINEAR else nkv
                mat(p + "q", (nh * dh, d), [src(p + "W_q", 0, nh * dh)])
                mat(p + "k", (kvh * dh, d), [src(p + "W_k", 0, kvh * dh)])
                mat(p + "v", (kvh * dh, d), [src(p + "W_v", 0, kvh * dh)])
                if kind is M.AttentionKind.LINEAR and cfg.delta_beta == "sigmoid":
                    # rows padded to a multiple of 8 (16-byte rows for the GEMM's operands);
                    # the padding rows are zero, see no gradient and are not exported
                    mat(p + "beta", ((nh + 7) // 8 * 8, d), [src(p + "W_beta", 0, nh)])
                mat(p + "o", (d, nh * dh), [(p + "W_o", 0, d, "o", None)])
            if M.ffn_kind(i, cfg) is M.FfnKind.DENSE:
                hid = cfg.dense_hidden if cfg.dense_hidden is not None else cfg.expert_hidden
                mat(p + "gate_up", (2 * hid, d),
                    [src(p + "ffn_gate", 0, hid), src(p + "ffn_up", hid, hid)],
                    unit_rows=[hid, hid])
                mat(p + "down", (d, hid), [src(p + "ffn_down", 0, d)])
            else:
                # routed experts followed by the shared experts (always-on, gate 1), all the
                # same shape: one grouped product covers both
                n_r, n_s, hid = cfg.n_routed_experts, cfg.n_shared_experts, cfg.expert_hidden
                self.moe_layers.append(i)
                mat(p + "router", (n_r, d), [src(p + "router", 0, n_r)])
                gu_src, dn_src = [], []
                if self.ep:
                    # this rank's routed experts only; shared experts are replicated dense FFNs
                    el = n_r // self.world
                    for j in range(el):
                        e = self.rank * el + j
                        gu_src.append((p + "routed_gate", 2 * j * hid, hid, ("e", e), None))
                        gu_src.append((p + "routed_up", (2 * j + 1) * hid, hid, ("e", e), None))
                        dn_src.append((p + "routed_down", j * d, d, ("e", e), None))
                    mat(p + "moe_gu", (2 * hid * el, d), gu_src, unit_rows=[hid] * (2 * el), local=True)
                    mat(p + "moe_down", (d * el, hid), dn_src, unit_rows=[d] * el, local=True)
                    for j in range(n_s):
                        mat(p + f"shared{j}_gate_up", (2 * hid, d),
                            [(p + "shared_gate", 0, hid, ("e", j), None),
                             (p + "shared_up", hid, hid, ("e", j), None)], unit_rows=[hid, hid])
                        mat(p + f"shared{j}_down", (d, hid), [(p + "shared_down", 0, d, ("e", j), None)])
                    continue
                for e in range(n_r + n_s):
                    kind_, idx = ("routed", e) if e < n_r else ("shared", e - n_r)
                    gu_src.append((p + kind_ + "_gate", 2 * e * hid, hid, ("e", idx), None))
                    gu_src.append((p + kind_ + "_up", (2 * e + 1) * hid, hid, ("e", idx), None))
                    dn_src.append((p + kind_ + "_down", e * d, d, ("e", idx), None))
                mat(p + "moe_gu", (2 * hid * (n_r + n_s), d), gu_src,
                    unit_rows=[hid] * (2 * (n_r + n_s)))
                mat(p + "moe_down", (d * (n_r + n_s), hid), dn_src, unit_rows=[d] * (n_r + n_s))
        self.weights = {w.name: w for w in ws}
        # Muon flat layout: units grouped by (rows, cols) so each class is one batched NS.
        classes: dict[tuple, list[Unit]] = {}
        for w in ws:
            for u in w.units:
                key = (u.rows, u.cols, 1) if w.local else (u.rows, u.cols)
                classes.setdefault(key, []).append(u)
        self.unit_classes = classes
        self.unit_index = {(u.weight, u.r0): (key, j) for key, us in classes.items()
                           for j, u in enumerate(us)}
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
        for grp in ("adam", "vec"):
            off = 0
            for w in ws:
                if w.group == grp:
                    w.off = off
                    off += int(math.prod(w.shape))
                    off = (off + 7) // 8 * 8
            setattr(self, "n_" + grp, off)

    def _allocate(self) -> None:
        dev = self.device
        f32 = dict(dtype=torch.float32, device=dev)
        self.sym = None
        self.sym_lp = None
        n_m, n_a, n_v = self.n_muon, self.n_adam, self.n_vec
        if self.fsdp and self.grad_sync == "nccl":
            raise ValueError("fsdp=True needs the peer-memory gradient path (grad_sync auto / p2p)")
        if self.world > 1 and self.grad_sync in ("auto", "p2p"):
            # Gradients and bf16 working weights live in symmetric memory: peers read the
            # former (reduce to owner) and write the latter (update + broadcast / shard store).
            from .parallel.symm import SymmetricBuffer, SymmetricGroup

            ok, err = 1, None
            try:
                self.sym = SymmetricGroup(self.pg)
                self.sym_grad = SymmetricBuffer(4 * (n_m + n_a + n_v), self.pg)
                if self.fsdp:
                    self._plan_fsdp()
                    self.sym_lp = SymmetricBuffer(2 * self.n_sym_w, self.pg)
                else:
                    if self.nvls_mode in ("auto", True):
                        from .parallel.nvls import NvlsBuffer

                        self.nvls_lp = NvlsBuffer.create(2 * (n_m + n_a), self.pg)
                        if self.nvls_lp is None and self.nvls_mode is True:
                            raise RuntimeError("nvls=True but no multicast object could be set up")
                    if self.nvls_lp is None:
                        self.sym_lp = SymmetricBuffer(2 * (n_m + n_a), self.pg)
            except RuntimeError as e:      # peer mapping refused on this machine
                ok, err = 0, e
            flag = torch.tensor([ok], dtype=torch.int32, device=dev)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN, group=self.pg)
            if int(flag.item()) == 0:
                if self.grad_sync == "p2p" or self.fsdp:
                    raise RuntimeError(f"symmetric memory unavailable: {err}")
                self.sym = None
        if self.sym is None:
            self.fsdp = False
        if self.sym is not None:
            self.muon_grad = self.sym_grad.view(torch.float32, n_m, 0)
            self.adam_grad = self.sym_grad.view(torch.float32, n_a, 4 * n_m)
            self.vec_grad = self.sym_grad.view(torch.float32, n_v, 4 * (n_m + n_a))
            if not self.fsdp:
                lp_buf = self.nvls_lp if self.nvls_lp is not None else self.sym_lp
                self.muon_lp = lp_buf.view(BF16, n_m, 0)
                self.adam_lp = lp_buf.view(BF16, n_a, 2 * n_m)
        else:
            self.muon_grad = torch.zeros(n_m, **f32)
            self.adam_grad = torch.zeros(n_a, **f32)
            self.vec_grad = torch.zeros(n_v, **f32)
            self.muon_lp = torch.zeros(n_m, dtype=BF16, device=dev)
            self.adam_lp = torch.zeros(n_a, dtype=BF16, device=dev)
        # ownership: rank r updates units [lo, hi) of every Muon shape class and one
        # contiguous slice of the AdamW slab; fp32 vectors are updated by every rank.
        from .parallel.fsdp import split_bounds

        w_, r_ = (self.world, self.rank) if self.sym is not None else (1, 0)
        self.own_units = {key: ((0, len(us)) if len(key) > 2 else split_bounds(len(us), w_, r_))
                          for key, us in self.unit_classes.items()}
        a_lo, a_hi = split_bounds(n_a // 8, w_, r_)
        self.own_adam = (a_lo * 8, a_hi * 8)
        # State storage. Replicated mode keeps full-size master / moment buffers addressed by
        # the global flat offsets (only the owned ranges are ever current). ZeRO mode allocates
        # the owned ranges only: class_lbase[key] / adam_shift translate a global offset of an
        # owned element into the compact buffers.
        self.compact = self.fsdp
        self.class_range: dict[tuple, tuple] = {}
        self.class_lbase: dict[tuple, int] = {}
        lb = 0
        for key in sorted(self.unit_classes):
            units = self.unit_classes[key]
            n = key[0] * key[1]
            lo_u, hi_u = self.own_units[key]
            glo, ghi = units[0].off + lo_u * n, units[0].off + hi_u * n
            self.class_range[key] = (glo, ghi)
            self.class_lbase[key] = lb if self.compact else glo
            lb += ghi - glo
        self.adam_shift = self.own_adam[0] if self.compact else 0
        n_m_state = max(lb, 8) if self.compact else n_m
        n_a_state = max(self.own_adam[1] - self.own_adam[0], 8) if self.compact else n_a
        self.muon_master = torch.zeros(n_m_state, **f32)
        self.muon_mom = torch.zeros(n_m_state, **f32)
        self.adam_master = torch.zeros(n_a_state, **f32)
        self.adam_m = torch.zeros(n_a_state, **f32)
        self.adam_v = torch.zeros(n_a_state, **f32)
        self.vec_master = torch.zeros(n_v, **f32)
        self.vec_m = torch.zeros(n_v, **f32)
        self.vec_v = torch.zeros(n_v, **f32)
        max_unit = max((k_[0] * k_[1] * (self.own_units[k_][1] - self.own_units[k_][0])
                        for k_ in self.unit_classes), default=1)
        self.ns_x = [torch.empty(max(max_unit, 1), dtype=BF16, device=dev) for _ in range(2)]
        max_g = max((min(k_[0], k_[1]) ** 2 * (self.own_units[k_][1] - self.own_units[k_][0])
                     for k_ in self.unit_classes), default=1)
        self.ns_g = [torch.empty(max(max_g, 1), dtype=BF16, device=dev) for _ in range(2)]
        nparts = max(_lib.query("pb_sumsq_nparts", max(n_m, n_a, n_v, 1)), 1)
        if self.sym is not None:
            nparts = max(nparts, _lib.query("pb_reduce_nparts", max(n_m, n_a, n_v, 1)))
        for k_ in self.unit_classes:        # batched Muon prepare: (partials + 1) per owned matrix
            nb_ = self.own_units[k_][1] - self.own_units[k_][0]
            nparts = max(nparts, nb_ * (_lib.query("pb_sumsq_nparts", k_[0] * k_[1]) + 1))
        self.opt_scratch = torch.empty(nparts + 8, **f32)
        self.gnorm_sq = torch.zeros(1, **f32)
        self.local_sq = torch.zeros(1, **f32)
        self.vec_sq = torch.zeros(1, **f32)
        grads = {"muon": self.muon_grad, "adam": self.adam_grad, "vec": self.vec_grad}
        if self.fsdp:
            self._allocate_fsdp()
        self.p: dict[str, Tensor] = {}
        for w in self.weights.values():
            n = int(math.prod(w.shape))
            if not w.lp:
                t = self.vec_master[w.off:w.off + n].view(w.shape)
            elif self.fsdp:
                t = self._fsdp_view(w)
            else:
                lpbuf = self.muon_lp if w.group == "muon" else self.adam_lp
                t = lpbuf[w.off:w.off + n].view(w.shape)
            t.requires_grad_(True)
            t.main_grad = grads[w.group][w.off:w.off + n].view(w.shape)
            self.p[w.name] = t

    # ------------------------------------------------------------ ZeRO-3 layout
    def _plan_fsdp(self) -> None:
        """Group the bf16 working weights into blobs (one per layer, one per vocabulary-sized
        table), cut every blob into ``world`` equal chunks, and lay the symmetric weight buffer
        out as [this rank's chunk of every blob | replicated small weights | this rank's experts]."""
        W = self.world
        blobs: dict[tuple, dict] = {}
        rep = 0
        for w in self.weights.values():
            if not w.lp:
                continue
            n = (int(math.prod(w.shape)) + 7) // 8 * 8
            if w.local:
                w.mode, w.blob = "local", None
            elif w.name.startswith("layers."):
                w.mode, w.blob = "shard", ("layer", int(w.name.split(".")[1]))
            elif w.name in ("embed", "unembed") or w.name.endswith(".unembed"):
                w.mode, w.blob = "shard", (w.name,)
            else:
                w.mode, w.blob = "bcast", None          # adapter, MTP projections: small
            if w.mode == "shard":
                b = blobs.setdefault(w.blob, {"key": w.blob, "weights": [], "L": 0})
                w.pos = b["L"]
                b["weights"].append(w.name)
                b["L"] += n
            else:
                w.pos = rep
                rep += n
        off = 0
        for b in blobs.values():
            b["L"] = (b["L"] + 8 * W - 1) // (8 * W) * (8 * W)
            b["chunk"] = b["L"] // W
            b["shard_off"] = off
            b["slot"] = f"layer{b['key'][1] % 2}" if b["key"][0] == "layer" else "big"
            off += b["chunk"]
        self.blobs = blobs
        self.n_shard = off
        self.rep_off = off
        self.n_sym_w = off + rep

    def _allocate_fsdp(self) -> None:
        dev = self.device
        sizes = {"layer0": 8, "layer1": 8, "big": 8}
        for b in self.blobs.values():
            sizes[b["slot"]] = max(sizes[b["slot"]], b["L"])
        self.landing = {k: torch.empty(v, dtype=BF16, device=dev) for k, v in sizes.items()}
        self.slot_state = {k: {"blob": None, "ready": None, "waited": True} for k in sizes}
        self.fetch_stream = torch.cuda.Stream(dev)
        self.sym_w_local = self.sym_lp.view(BF16, self.n_sym_w, 0)
        # destination tables of the update kernels: per Muon unit (pos, chunk, base)
        self.dest_tables: dict[tuple, Tensor] = {}
        for key, units in self.unit_classes.items():
            rows = []
            for u in units:
                w = self.weights[u.weight]
                rows.append(self._dest_of(w, u.r0 * u.cols))
            self.dest_tables[key] = torch.tensor(rows, dtype=torch.int64, device=dev).reshape(-1, 3)
        # AdamW slab: the pieces of bf16-backed weights inside this rank's slab range
        a_lo, a_hi = self.own_adam
        self.adam_segments = []
        for w in self.weights.values():
            if w.group != "adam":
                continue
            n = int(math.prod(w.shape))
            lo, hi = max(w.off, a_lo), min(w.off + n, a_hi)
            if hi > lo:
                self.adam_segments.append((lo, hi - lo, self._dest_of(w, lo - w.off)))

    def _dest_of(self, w: "Weight", elem: int) -> tuple:
        """(pos, chunk, base) of element ``elem`` of a weight's bf16 copy (see csrc/comm/fsdp.cu)."""
        if w.mode == "shard":
            b = self.blobs[w.blob]
            return (w.pos + elem, b["chunk"], b["shard_off"])
        return (0, 0 if w.mode == "bcast" else -1, self.rep_off + w.pos + elem)

    def _fsdp_view(self, w: "Weight") -> Tensor:
        n = int(math.prod(w.shape))
        if w.mode == "shard":
            b = self.blobs[w.blob]
            return self.landing[b["slot"]][w.pos:w.pos + n].view(w.shape)
        o = self.rep_off + w.pos
        return self.sym_w_local[o:o + n].view(w.shape)

    def _fsdp_fetch(self, key: tuple) -> None:
        """Enqueue the all-gather of a blob into its landing slot on the fetch stream (no-op
        when the slot already holds it). The slot's previous occupant may still be in use by
        kernels already enqueued on the compute stream: the copy waits for them."""
        b = self.blobs[key]
        st = self.slot_state[b["slot"]]
        if st["blob"] == key:
            return
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        self.fetch_stream.wait_event(ev)
        with torch.cuda.stream(self.fetch_stream):
            if not self.comm_noop:
                call("pb_shard_gather", self.sym_lp.ptrs, b["shard_off"], b["chunk"],
                     ptr(self.landing[b["slot"]]), self.world, self.rank, 64, stream_ptr())
            ready = torch.cuda.Event()
            ready.record(self.fetch_stream)
        st.update(blob=key, ready=ready, waited=False)

    def _fsdp_ensure(self, key: tuple) -> None:
        """The compute stream may read the blob's landing slot after this call."""
        self._fsdp_fetch(key)
        st = self.slot_state[self.blobs[key]["slot"]]
        if not st["waited"]:
            torch.cuda.current_stream(self.device).wait_event(st["ready"])
            st["waited"] = True

    def _fsdp_enter(self, layer: int, backward: bool = False) -> None:
        """Layer ``layer`` is about to run (forward or backward): make its weights resident and
        start pulling the next layer's into the other slot."""
        self._fsdp_ensure(("layer", layer))
        nxt = layer - 1 if backward else layer + 1
        if 0 <= nxt < self.cfg.n_layers and ("layer", nxt) in self.blobs:
            self._fsdp_fetch(("layer", nxt))

    def _fsdp_invalidate(self) -> None:
        for st in self.slot_state.values():
            st.update(blob=None, ready=None, waited=True)

    def weight(self, name: str) -> Tensor:
        """The bf16 working tensor of a weight, resident (gathers its blob first under ZeRO-3)."""
        if self.fsdp:
            w = self.weights[name]
            if w.lp and w.mode == "shard":
                self._fsdp_ensure(w.blob)
        return self.p[name]

    def memory_report(self) -> dict:
        """Bytes this rank holds for weights and optimizer state (gradients and activations not
        counted): what ZeRO sharding is meant to shrink."""
        state = sum(t.numel() * 4 for t in (self.muon_master, self.muon_mom, self.adam_master,
                                            self.adam_m, self.adam_v, self.vec_master, self.vec_m,
                                            self.vec_v))
        if self.fsdp:
            lp = 2 * self.n_sym_w
            landing = sum(2 * t.numel() for t in self.landing.values())
        else:
            lp = 2 * (self.n_muon + self.n_adam)
            landing = 0
        return {"weights_bf16_bytes": lp, "landing_bytes": landing, "optimizer_state_bytes": state,
                "gradient_bytes": 4 * (self.n_muon + self.n_adam + self.n_vec),
                "weights_plus_state_bytes": lp + landing + state}

    def symmetric_buffers(self) -> list:
        """Every symmetric allocation this trainer's kernels let peers write into."""
        bufs = [b for b in (getattr(self, "sym_grad", None), self.sym_lp) if b is not None]
        for ctx in (self.ep_ctx, self.cp_ctx):
            for attr in ("counts", "xbuf", "ybuf", "dotbuf", "xqbuf", "xsbuf", "arrbuf", "buf"):
                b = getattr(ctx, attr, None) if ctx is not None else None
                if b is not None and hasattr(b, "canaries_intact"):
                    bufs.append(b)
        if self.cp_ctx is not None and hasattr(self.cp_ctx, "symmetric_buffers"):
            bufs += self.cp_ctx.symmetric_buffers()
        if self.sym is not None:
            bufs.append(self.sym.ctrl)
        return bufs

    def check_canaries(self) -> None:
        """Raise if a peer (or this rank) wrote outside the usable range of any symmetric
        buffer: the guard zones on both sides of each allocation must still hold their pattern.
        Synchronises; meant for debugging runs and tests (``debug_canaries`` runs it every step)."""
        for i, b in enumerate(self.symmetric_buffers()):
            if not b.canaries_intact():
                raise RuntimeError(f"rank {self.rank}: a canary zone of symmetric buffer {i} "
                                   f"({b.nbytes} bytes) was overwritten")

    def close(self) -> None:
        """Release the symmetric-memory mappings (collective: every rank calls it)."""
        if self.sym is None:
            return
        torch.cuda.synchronize(self.device)
        torch.distributed.barrier(self.pg)
        self.p = {}
        for name in ("muon_grad", "adam_grad", "vec_grad", "muon_lp", "adam_lp", "sym_w_local"):
            if hasattr(self, name):
                delattr(self, name)
        if self.nvls_lp is not None:
            self.nvls_lp.close()
            self.nvls_lp = None
        bufs = [self.sym_grad] + ([self.sym_lp] if getattr(self, "sym_lp", None) is not None else [])
        for ctx in (self.ep_ctx, self.cp_ctx):
            for attr in ("counts", "xbuf", "ybuf", "dotbuf", "xqbuf", "xsbuf", "arrbuf", "buf"):
                b = getattr(ctx, attr, None) if ctx is not None else None
                if b is not None and hasattr(b, "close"):
                    bufs.append(b)
        if self.cp_ctx is not None:
            if hasattr(self.cp_ctx, "symmetric_buffers"):
                bufs += self.cp_ctx.symmetric_buffers()
            else:
                bufs.append(self.cp_ctx.sym.ctrl)
        bufs.append(self.sym.ctrl)
        for b in bufs:
            b.close_peers()
        torch.cuda.synchronize(self.device)
        torch.distributed.barrier(self.pg)     # nobody maps a peer's memory any more
        for b in bufs:
            b.free_local()
        self.sym = self.ep_ctx = self.cp_ctx = None
        torch.distributed.barrier(self.pg)

    # ------------------------------------------------------------ tree <-> flat
    @staticmethod
    def _to_engine(t: Tensor, how) -> Tensor:
        if isinstance(how, tuple):          # ("e", index): one expert of a stacked tensor
            return _t2(t[how[1]])
        if how == "t2":
            return _t2(t)
        if how == "o":
            return t.reshape(-1, t.shape[-1]).t().contiguous()
        return t

    def _owned_pieces(self, group: str, g0: int, g1: int):
        """Intersections of the global flat range [g0, g1) of a state group with what this
        rank stores: ``[(global_start, global_end, local_start)]``."""
        out = []
        if not self.compact:            # full-size buffers addressed by the global offsets
            return [(g0, g1, g0)]
        if group == "muon":
            for key, (glo, ghi) in self.class_range.items():
                lo, hi = max(g0, glo), min(g1, ghi)
                if hi > lo:
                    out.append((lo, hi, self.class_lbase[key] + lo - glo))
        elif group == "adam":
            lo, hi = max(g0, self.own_adam[0]), min(g1, self.own_adam[1])
            if hi > lo:
                out.append((lo, hi, lo - self.adam_shift))
        else:
            out.append((g0, g1, g0))
        return out

    def _state_buffers(self, group: str) -> dict:
        if group == "muon":
            return {"master": self.muon_master, "mom": self.muon_mom}
        if group == "adam":
            return {"master": self.adam_master, "m": self.adam_m, "v": self.adam_v}
        return {"master": self.vec_master, "m": self.vec_m, "v": self.vec_v}

    def _store_state(self, w: Weight, which: str, full: Tensor) -> None:
        """Write one state tensor of a weight (fp32, the weight's shape) into what this rank
        stores of it; ``which`` in master / mom / m / v."""
        n = int(math.prod(w.shape))
        flat = full.reshape(-1)
        buf = self._state_buffers(w.group)[which]
        for lo, hi, l0 in self._owned_pieces(w.group, w.off, w.off + n):
            buf[l0:l0 + hi - lo].copy_(flat[lo - w.off:hi - w.off])

    def _store_lp(self, w: Weight, full: Tensor) -> None:
        """Refresh the bf16 working copy of a weight from its full fp32 value (this rank's part
        of it under ZeRO-3)."""
        if not w.lp:
            return
        n = int(math.prod(w.shape))
        flat = full.reshape(-1).to(BF16)
        if not self.fsdp or w.mode != "shard":
            self.p[w.name].detach().reshape(-1).copy_(flat)
            return
        b = self.blobs[w.blob]
        c0 = self.rank * b["chunk"]                # blob positions of my chunk: [c0, c0 + chunk)
        lo, hi = max(w.pos, c0), min(w.pos + n, c0 + b["chunk"])
        if hi > lo:
            dst0 = b["shard_off"] + lo - c0
            self.sym_w_local[dst0:dst0 + hi - lo].copy_(flat[lo - w.pos:hi - w.pos])

    def load_tree(self, params: dict) -> None:
        """Copy a parameter tree (reference layout) into the flat buffers."""
        flat = M.flatten_params(params)
        with torch.no_grad():
            for w in self.weights.values():
                full = torch.zeros(w.shape, dtype=torch.float32, device=self.device)
                for tree_name, r0, rows, how, _ in w.sources:
                    leaf = flat[tree_name]
                    if not leaf.is_meta:
                        src = self._to_engine(leaf.detach().float(), how)
                    elif isinstance(how, tuple):     # shapes-only tree: draw just this expert
                        src = _t2(M.init_leaf(self.cfg, f"{tree_name}.{how[1]}", leaf.shape[1:], self.seed,
                                              self.device))
                    else:
                        src = self._to_engine(M.init_leaf(self.cfg, tree_name, leaf.shape, self.seed,
                                                          self.device), how)
                    full[r0:r0 + rows].copy_(src.to(self.device))
                self._store_state(w, "master", full)
                self._store_lp(w, full)
                del full
            self.router_bias = {}
            for i in self.moe_layers:
                name = f"layers.{i}.router_bias"
                if self.cfg.router_bias:
                    b = flat.get(name)
                    self.router_bias[i] = (torch.zeros(self.cfg.n_routed_experts)
                                           if b is None or b.is_meta else b.detach().float().clone()).to(self.device)
        if self.fsdp:
            self._fsdp_invalidate()
        if self.sym is not None:
            torch.cuda.synchronize()
            torch.distributed.barrier(self.pg)

    def full_state(self) -> dict:
        """Every flat fp32 state buffer at its full (global) size, complete on every rank:
        ``muon.master / muon.mom / adam.master / adam.m / adam.v / vec.master / vec.m / vec.v``.
        With ownership sharding each rank contributes the ranges it owns and the rest comes from
        a sum over the ranks (collective); expert-parallel ranges stay this rank's own."""
        out = {"vec.master": self.vec_master, "vec.m": self.vec_m, "vec.v": self.vec_v}
        if self.sym is None:
            out.update({"muon.master": self.muon_master, "muon.mom": self.muon_mom,
                        "adam.master": self.adam_master, "adam.m": self.adam_m, "adam.v": self.adam_v})
            return out
        import torch.distributed as dist

        f32 = dict(dtype=torch.float32, device=self.device)
        for which, buf in (("master", self.muon_master), ("mom", self.muon_mom)):
            full = torch.zeros(self.n_muon, **f32)
            local = []
            for key, (glo, ghi) in self.class_range.items():
                if ghi <= glo:
                    continue
                l0 = self.class_lbase[key]
                if len(key) > 2:
                    local.append((glo, ghi, l0))      # this rank's experts: not summed
                else:
                    full[glo:ghi] = buf[l0:l0 + ghi - glo]
            dist.all_reduce(full, group=self.pg)
            for glo, ghi, l0 in local:
                full[glo:ghi] = buf[l0:l0 + ghi - glo]
            out["muon." + which] = full
        a_lo, a_hi = self.own_adam
        for which, buf in (("master", self.adam_master), ("m", self.adam_m), ("v", self.adam_v)):
            full = torch.zeros(self.n_adam, **f32)
            full[a_lo:a_hi] = buf[a_lo - self.adam_shift:a_hi - self.adam_shift]
            dist.all_reduce(full, group=self.pg)
            out["adam." + which] = full
        return out

    def load_full_state(self, state: dict) -> None:
        """Inverse of :meth:`full_state`: every rank is given the full buffers and keeps what it
        stores; the bf16 working copies are rebuilt from the masters."""
        with torch.no_grad():
            for w in self.weights.values():
                n = int(math.prod(w.shape))
                for which in self._state_buffers(w.group):
                    full = state[f"{w.group}.{which}"][w.off:w.off + n].to(self.device)
                    self._store_state(w, which, full)
                    if which == "master":
                        self._store_lp(w, full)
        if self.fsdp:
            self._fsdp_invalidate()
        if self.sym is not None:
            torch.cuda.synchronize()
            torch.distributed.barrier(self.pg)

    def gather_masters(self) -> dict:
        """Full fp32 master buffers per group on every rank (see :meth:`full_state`)."""
        st = self.full_state()
        return {"muon": st["muon.master"], "adam": st["adam.master"], "vec": st["vec.master"]}

    def export_tree(self) -> dict:
        """Parameter tree (reference layout, fp32, on CPU) from the master buffers."""
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        out: dict[str, Tensor] = {}
        full = self.gather_masters()
        stacked: dict[str, dict[int, Tensor]] = {}
        for w in self.weights.values():
            n = int(math.prod(w.shape))
            src = full[w.group][w.off:w.off + n].view(w.shape).cpu()
            for tree_name, r0, rows, how, _ in w.sources:
                blk = src[r0:r0 + rows]
                if isinstance(how, tuple):
                    stacked.setdefault(tree_name, {})[how[1]] = blk.t().contiguous()
                    continue
                if how == "t2":
                    t = blk.t().contiguous()
                    leaf = tree_name.split(".")[-1]
                    if leaf == "W_q" or leaf == "W_kv_up":
                        t = t.reshape(t.shape[0], nh, -1)
                    elif leaf in ("W_k", "W_v"):
                        t = t.reshape(t.shape[0], -1, dh)
                elif how == "o":
                    t = blk.t().contiguous().reshape(nh, dh, cfg.d_model)
                else:
                    t = blk.clone()
                out[tree_name] = t
        if self.ep:
            # every rank holds a slice of the routed experts: exchange them (host side)
            import torch.distributed as dist

            every = [None] * self.world
            dist.all_gather_object(every, {k: v for k, v in stacked.items() if "routed_" in k},
                                   group=self.pg)
            for part in every:
                for tree_name, blocks in part.items():
                    stacked.setdefault(tree_name, {}).update(blocks)
        for tree_name, parts in stacked.items():
            out[tree_name] = torch.stack([parts[j] for j in range(len(parts))])
        for i, b in self.router_bias.items():
            out[f"layers.{i}.router_bias"] = b.detach().cpu().clone()
        return M.unflatten_params(out)

    # ------------------------------------------------------------------ forward
    def _delta_layer(self, n: Tensor, i: int, B: int, S: int) -> Tensor:
        from . import kernels

        cfg = self.cfg
        nh, dh, _ = M.head_geometry(cfg)
        pre = f"layers.{i}."
        # q and k are normalised over their own projection outputs (no copy)
        if cfg.delta_beta == "sigmoid":
            # the per-head write gate rides along as a fourth (skinny) projection of the same
            # input on the same kernel; its input gradient folds into the shared dx epilogue
            q, k, v, bl = ops.linear_multi(n, (self.p[pre + "q"], self.p[pre + "k"], self.p[pre + "v"],
                                               self.p[pre + "beta"]))
            beta = torch.sigmoid(bl[:, :nh]).view(B, S, nh)
        else:
            q, k, v = ops.linear_multi(n, (self.p[pre + "q"], self.p[pre + "k"], self.p[pre + "v"]))
            beta = torch.ones((B, S, nh), dtype=BF16, device=n.device)
        q = ops.l2norm_(q, dh).view(B, S, nh, dh)
        k = ops.l2norm_(k, dh).view(B, S, nh, dh)
        v = v.view(B, S, nh, dh)
        if self.cp_zigzag:
            from .parallel.cp import delta_rule_zigzag

            o = delta_rule_zigzag(q, k, v, beta, self._zigzag_ctx(B * nh))
        elif self.cp:
            from .parallel.cp import DeltaCpContext, delta_rule_cp

            if self.cp_ctx is None or self.cp_ctx.bh != B * nh:
                self.cp_ctx = DeltaCpContext(B * nh, self.pg)
            o = delta_rule_cp(q, k, v, beta, self.cp_ctx)
        else:
            o, _ = kernels.chunked_delta_rule(q, k, v, beta, None,
                                              kernels.LinearAttnConfig(chunk=cfg.chunk),
                                              allow_fallback=self.allow_fallback)
        return ops.linear(o.reshape(B * S, nh * dh), self.p[pre + "o"])

    def _ffn_linear(self, x: Tensor, w: Tensor, xq=None) -> Tensor:
        """``xq``: the e4m3 rows + scales of ``x`` when the norm kernel that produced it wrote
        them too (one quantisation shared by every FP8 consumer of the normalised stream)."""
        if self.fp8 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
            from .ops import fp8

            return fp8.fp8_linear(x, w, xq)
        return ops.linear(x, w)

    def _mla_layer(self, n: Tensor, i: int, B: int, S: int) -> Tensor:
        """Latent-KV softmax attention. Projections run on the tcgen05 GEMM; the rotary
        split, the unit-weight QK RMSNorm and the softmax core are PyTorch (the reference's
        tiny / flagship geometries, not a benchmark path)."""
        cfg = self.cfg
        if not self.allow_fallback:
            raise ValueError("MLA layers run their softmax core on the library attention; "
                             "construct the Trainer with allow_fallback=True to use them")
        nh = M.head_geometry(cfg)[0]
        dn, dr, _ = self.mla_dims
        pre = f"layers.{i}."
        q = ops.linear(n, self.p[pre + "q"]).view(B, S, nh, dn + dr)
        ckv = ops.linear(n, self.p[pre + "kv_c"])
        k_nope = ops.linear(ckv, self.p[pre + "kv_up"]).view(B, S, nh, dn)
        rk = ops.linear(n, self.p[pre + "rope_k"]).view(B, S, 1, dr).expand(B, S, nh, dr)
        pos = torch.arange(S, dtype=torch.float32, device=n.device)
        q_rope, rk = M.rope(q[..., dn:].float(), rk.float(), pos, partial=False, base=cfg.rope_base)
        qf = torch.cat([q[..., :dn].float(), q_rope], dim=-1)
        kf = torch.cat([k_nope.float(), rk], dim=-1)
        qf = qf * torch.rsqrt(qf.square().mean(-1, keepdim=True) + 1e-6)
        kf = kf * torch.rsqrt(kf.square().mean(-1, keepdim=True) + 1e-6)
        o = F.scaled_dot_product_attention(qf.transpose(1, 2).to(BF16), kf.transpose(1, 2).to(BF16),
                                           k_nope.transpose(1, 2), is_causal=True,
                                           scale=1.0 / math.sqrt(dn + dr))
        o = o.transpose(1, 2).reshape(B * S, nh * dn)
        return ops.linear(o, self.p[pre + "o"])

    def _moe_layer(self, n2: Tensor, i: int, n2q=None) -> Tensor:
        from .ops import moe

        cfg = self.cfg
        pre = f"layers.{i}."
        hid = cfg.expert_hidden
        w_gu = self.p[pre + "moe_gu"]
        w_dn = self.p[pre + "moe_down"]
        if self.ep:
            from .parallel.ep import EpContext, ep_moe_ffn

            T_ = n2.shape[0]
            el = cfg.n_routed_experts // self.world
            if self.ep_ctx is None:
                rows = int(self.ep_capacity_factor * T_ * cfg.top_k) + 128 * el
                self.ep_ctx = EpContext(self.sym, cfg.d_model, cfg.n_routed_experts, rows)
            # the shared experts (dense, always on) run on a side stream, so their GEMMs fill
            # the SMs while the routed path is in its barriers, pushes and pulls
            shared = None
            main = torch.cuda.current_stream(self.device)
            if cfg.n_shared_experts:
                if self.side_stream is None:
                    self.side_stream = torch.cuda.Stream(self.device)
                side = self.side_stream
                side.wait_stream(main)
                n2.record_stream(side)
                for t_ in (n2q or ()):
                    t_.record_stream(side)
                with torch.cuda.stream(side):
                    for j in range(cfg.n_shared_experts):
                        gu = self._ffn_linear(n2, self.p[pre + f"shared{j}_gate_up"], n2q)
                        sj = self._ffn_linear(ops.swiglu(gu), self.p[pre + f"shared{j}_down"])
                        shared = sj if shared is None else shared + sj
            out, probs, ids, logits = ep_moe_ffn(
                n2, self.p[pre + "router"], self.router_bias.get(i), w_gu, w_dn, cfg.top_k, self.ep_ctx,
                shapes=((el, 2 * hid, cfg.d_model), (el, cfg.d_model, hid)), return_logits=True,
                fp8=self.fp8)
            if shared is not None:
                main.wait_stream(self.side_stream)
                shared.record_stream(main)
                out = out + shared
            self._record_router(i, probs, ids, logits)
            return out
        n_e = cfg.n_routed_experts + cfg.n_shared_experts
        out, probs, ids, logits = moe.moe_ffn(
            n2, self.p[pre + "router"], self.router_bias.get(i), w_gu, w_dn, cfg.top_k,
            n_shared=cfg.n_shared_experts,
            shapes=((n_e, 2 * hid, cfg.d_model), (n_e, cfg.d_model, hid)), fp8=self.fp8,
            return_logits=True)
        self._record_router(i, probs, ids, logits)
        return out

    def _record_router(self, layer: int, probs: Tensor, ids: Tensor, logits: Tensor) -> None:
        """One MoE layer application of the current micro-batch: the z-loss term (kept in the
        graph) and the per-layer balancing statistic (detached)."""
        self.last_router = (probs, ids)
        if self.tcfg.z_loss_weight and self.z_loss_mode == "layers_logits":
            z = torch.logsumexp(logits, dim=-1).square().mean()
        else:
            z = None
        self.router_records.append((layer, z, probs))
        if self.router_bias:
            with torch.no_grad():
                if self.router_bias_rule == "count":
                    stat = torch.bincount(ids.reshape(-1).long(),
                                          minlength=self.cfg.n_routed_experts).float()
                else:
                    stat = probs.detach().sum(dim=0)
            acc = self._router_load.get(layer)
            self._router_load[layer] = stat if acc is None else acc + stat

    def _zigzag_ctx(self, rows: int):
        """The zig-zag context of this trainer (``rows`` = micro-batch x heads; the delta-rule
        and the softmax layers of the hybrid share the head count)."""
        from .parallel.cp import ZigzagCpContext

        if self.cp_ctx is None or self.cp_ctx.rows != rows:
            self.cp_ctx = ZigzagCpContext(rows, self.pg)
        return self.cp_ctx

    def _gqa_layer(self, n: Tensor, i: int, B: int, S: int) -> Tensor:
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        pre = f"layers.{i}."
        q, k, v = ops.linear_multi(n, (self.p[pre + "q"], self.p[pre + "k"], self.p[pre + "v"]))
        pos = None
        if self.cp_zigzag:      # global positions of this rank's two half-slices
            half = S // 2
            ar = torch.arange(half, dtype=torch.int32, device=n.device)
            pos = torch.cat([ar + self.rank * half, ar + (2 * self.world - 1 - self.rank) * half]).repeat(B)
        elif self.cp:      # global positions of this rank's slice
            pos = (torch.arange(S, dtype=torch.int32, device=n.device) + self.rank * S).repeat(B)
        # rotary embedding over the projection outputs themselves (no copy)
        q = ops.rope2d_(q, nh, seq_len=S, pos=pos, base=cfg.rope_base).view(B, S, nh, dh)
        k = ops.rope2d_(k, nkv, seq_len=S, pos=pos, base=cfg.rope_base).view(B, S, nkv, dh)
        v = v.view(B, S, nkv, dh)
        from .ops import attention

        if self.cp_zigzag:
            from .parallel.cp import zigzag_attention

            o = zigzag_attention(q, k, v, self._zigzag_ctx(B * nh))
            return ops.linear(o.reshape(B * S, nh * dh), self.p[pre + "o"])
        if self.cp:
            from .parallel.cp import cp_attention

            o = cp_attention(q, k, v, self.pg)
            return ops.linear(o.reshape(B * S, nh * dh), self.p[pre + "o"])
        if self.track_max_logit:
            o, rowmax = attention.causal_gqa(q, k, v, return_max_logit=True,
                                             allow_fallback=self.allow_fallback)
            m = rowmax.amax(dim=(0, 2)).float()               # per head, for QK-clip
            prev = self.max_logits.get(i)
            self.max_logits[i] = m if prev is None else torch.maximum(prev, m)
        else:
            o = attention.causal_gqa(q, k, v, allow_fallback=self.allow_fallback)
        return ops.linear(o.reshape(B * S, nh * dh), self.p[pre + "o"])

    def _layers(self, x: Tensor, res: Tensor | None, start: int, count: int, B: int, S: int):
        """Layers ``start .. start + count`` on a residual stream held as a pending sum
        ``x + res`` (``res`` None: the stream is ``x``). The add is fused into the next
        normalisation, so the pair is also what comes back."""
        cfg = self.cfg
        for i in range(start, start + count):
            pre = f"layers.{i}."
            if self.fsdp:
                self._fsdp_enter(i)
            if res is None:
                n, h = ops.rmsnorm(x, self.p[pre + "pre_attn_norm"]), x
            else:
                n, h = ops.add_rmsnorm(x, res, self.p[pre + "pre_attn_norm"])
            if self.layer_kinds[i] is M.AttentionKind.LINEAR:
                a = self._delta_layer(n, i, B, S)
            elif self.layer_kinds[i] is M.AttentionKind.MLA:
                a = self._mla_layer(n, i, B, S)
            else:
                a = self._gqa_layer(n, i, B, S)
            # FP8 linears: the norm kernel also writes the e4m3 rows + scales its consumers read
            want_q = self.fp8 and (pre + "gate_up" in self.p or (self.ep and cfg.n_shared_experts > 0))
            if want_q:
                n2, h, n2q = ops.add_rmsnorm(a, h, self.p[pre + "pre_ffn_norm"], emit_fp8=True)
            else:
                (n2, h), n2q = ops.add_rmsnorm(a, h, self.p[pre + "pre_ffn_norm"]), None
            if pre + "gate_up" in self.p:
                gu = self._ffn_linear(n2, self.p[pre + "gate_up"], n2q)
                f = self._ffn_linear(ops.swiglu(gu), self.p[pre + "down"])
            else:
                f = self._moe_layer(n2, i, n2q)
            if self.fsdp and torch.is_grad_enabled():
                # the backward of this layer starts here: its weights must be resident again
                f = _FsdpLayerHook.apply(f, self, i)
            x, res = f, h
        return x, res

    def _adapt_thoughts(self, thoughts: Tensor) -> Tensor:
        """Thought vectors (B, n, d) -> residual-stream rows: SiLU MLP + RMSNorm, the products
        on the tcgen05 GEMM (model/__init__.py:601-614 of the reference)."""
        from .ops import latent as LK

        B, n, d = thoughts.shape
        t2 = thoughts.to(BF16).reshape(B * n, d).contiguous()
        a = ops.linear(LK._SiluFn.apply(ops.linear(t2, self.p["adapter_w1"])), self.p["adapter_w2"])
        return ops.rmsnorm(a, self.p["adapter_norm"]).view(B, n, d)

    def forward_hidden(self, tokens: Tensor, inputs_embeds: Tensor | None = None, *,
                       r: int | None = None, thoughts: Tensor | None = None) -> Tensor:
        """Final-norm hidden states (B*S, d) in bf16 for a (B, S) token batch.

        ``r`` core-block iterations (default: the trainer's ``recurrence``): iteration 0 runs the
        core block on the prelude output, every later one on ``carry + prelude output``; the
        carry entering the last ``truncated_recurrence`` iterations is detached, so the earlier
        iterations run without a graph. ``thoughts`` (B, n, d) are adapter-mapped and prepended;
        their positions are dropped from the result. Reference: model/__init__.py:866-881,
        928-971."""
        cfg = self.cfg
        B, S = tokens.shape
        if inputs_embeds is None:
            h = _EmbedFn.apply(tokens, self.weight("embed")).reshape(B, S, cfg.d_model)
        else:
            h = inputs_embeds.reshape(B, S, cfg.d_model)
        n_th = 0
        if thoughts is not None and thoughts.shape[1] > 0:
            n_th = int(thoughts.shape[1])
            h = torch.cat([self._adapt_thoughts(thoughts), h], dim=1)
            S = S + n_th
        h = h.reshape(B * S, cfg.d_model)
        r_used = self.recurrence if r is None else int(r)
        if r_used < 1:
            raise ValueError("r must be >= 1")
        prelude, core, coda = M._recurrent_split(cfg)
        x, res = self._layers(h, None, 0, prelude, B, S)
        if r_used == 1:
            x, res = self._layers(x, res, prelude, core, B, S)
        else:
            injected = x if res is None else x + res
            cut = r_used - min(self.truncated_recurrence, r_used)

            def iterate(carry, first):
                if first:
                    return self._layers(injected, None, prelude, core, B, S)
                xs, rs = carry
                return self._layers(xs + rs, injected, prelude, core, B, S)

            carry = None
            with torch.no_grad():          # iterations whose output is cut off from the graph
                for it in range(cut):
                    carry = iterate(carry, it == 0)
            for it in range(cut, r_used):
                carry = iterate(carry, it == 0)
            x, res = carry
        x, res = self._layers(x, res, prelude + core, coda, B, S)
        n = ops.rmsnorm(x, self.p["final_norm"]) if res is None else \
            ops.add_rmsnorm(x, res, self.p["final_norm"])[0]
        if n_th:
            n = n.view(B, S, cfg.d_model)[:, n_th:].reshape(B * (S - n_th), cfg.d_model)
        return n

    def set_latent_slots(self, slot_start: int, k: int, n_sweeps: int = 4,
                         truncated_sweeps: int | None = None) -> None:
        """Latent training layout (prefix | K latent slots | answer): positions
        ``slot_start .. slot_start + k`` of every sequence are latent slots whose input
        embeddings are solved by ``n_sweeps`` Jacobi sweeps (each a full forward); gradient
        flows through the last ``truncated_sweeps`` sweeps. ``k = 0`` switches it off. The
        caller's loss mask should exclude the slot positions."""
        if k == 0:
            self.latent_slots = None
            return
        if slot_start < 1 or k < 0 or n_sweeps < 1:
            raise ValueError("latent slots need slot_start >= 1, k >= 0, n_sweeps >= 1")
        trunc = n_sweeps if truncated_sweeps is None else int(truncated_sweeps)
        if trunc < 1 or trunc > n_sweeps:
            raise ValueError("truncated_sweeps not in 1..=n_sweeps")
        self.latent_slots = (int(slot_start), int(k), int(n_sweeps), trunc)

    def forward_hidden_latent(self, tokens: Tensor) -> Tensor:
        """``forward_hidden`` with the latent slots of ``set_latent_slots`` solved by Jacobi
        sweeps; the per-sweep embedding update is ``ops.latent.jacobi_step`` (gather, adapter
        MLP on the tcgen05 GEMM, fused normalise + scatter)."""
        from .ops import latent as LK

        start, k, sweeps, trunc = self.latent_slots
        B, S = tokens.shape
        d = self.cfg.d_model
        embeds = _EmbedFn.apply(tokens, self.weight("embed")).reshape(B, S, d)
        cur, hidden = embeds, None
        for i in range(sweeps):
            if sweeps - trunc > 0 and i == sweeps - trunc:
                cur = cur.detach()
            hidden = self.forward_hidden(tokens, inputs_embeds=cur)
            if i + 1 < sweeps:
                cur = LK.jacobi_step(hidden.reshape(B, S, d), embeds, self.p["adapter_w1"],
                                     self.p["adapter_w2"], self.p["adapter_norm"], start, k)
        return hidden

    def loss(self, tokens: Tensor, loss_mask: Tensor, denom: Tensor | float,
             mtp_denoms: list | None = None) -> Tensor:
        """Masked mean next-token CE (soft-capped) of one micro-batch, scaled by 1/denom, plus
        the multi-token-prediction heads (head j predicts j + 1 tokens ahead from
        ``rmsnorm(h) @ proj + h`` with its own unembedding; mean over heads) and the router
        z-loss."""
        self.router_records = []
        if self.cp:
            # tokens / mask carry one extra column: the first token of the next rank's slice
            # (anything with mask 0 on the last rank), so every local position has its target
            # (zig-zag: one such column after each of the two half-slices)
            parts = 2 if self.cp_zigzag else 1
            tk = tokens.reshape(tokens.shape[0], parts, -1)
            mk = loss_mask.float().reshape(tokens.shape[0], parts, -1)
            targets = tk[:, :, 1:].reshape(-1).to(torch.int32)
            wt = mk[:, :, 1:].reshape(-1) / denom
            tokens = tk[:, :, :-1].reshape(tokens.shape[0], -1).contiguous()
            loss_mask = mk[:, :, :-1].reshape(tokens.shape[0], -1).contiguous()
            B, S = tokens.shape
            hid = self.forward_hidden(tokens)
        else:
            B, S = tokens.shape
            hid = self.forward_hidden_latent(tokens) if self.latent_slots else self.forward_hidden(tokens)
            targets = torch.roll(tokens, -1, dims=1).reshape(-1).to(torch.int32)
            wt = loss_mask.float().clone()
            wt[:, 0] = 0.0                          # mask[:, 1:] aligned to the predicting position
            wt = torch.roll(wt, -1, dims=1).reshape(-1) / denom
        if self.collect_amax:
            with torch.no_grad():
                a = hid.detach().abs().amax().float()
                prev = self.amax.get("final_hidden")
                self.amax["final_hidden"] = a if prev is None else torch.maximum(prev, a)
        ce = ops.softcap_cross_entropy(hid, self.weight("unembed"), targets, wt.contiguous(),
                                       float(self.tcfg.softcap), self.ce_chunk_rows)
        n_mtp = self.cfg.mtp_heads
        for j in range(n_mtp):
            off = j + 1
            if off >= S:
                continue
            m = loss_mask.float()
            wj = torch.zeros_like(m)
            wj[:, : S - off] = m[:, off:] * m[:, : S - off]
            dj = mtp_denoms[j] if mtp_denoms is not None else wj.sum().clamp(min=1.0)
            tj = torch.roll(tokens, -off, dims=1).reshape(-1).to(torch.int32)
            mh = ops.linear(ops.rmsnorm(hid, self.p[f"mtp.{j}.norm"]), self.p[f"mtp.{j}.proj"]) + hid
            ce = ce + ops.softcap_cross_entropy(mh, self.weight(f"mtp.{j}.unembed"), tj,
                                                (wj.reshape(-1) / (dj * n_mtp)).contiguous(),
                                                float(self.tcfg.softcap), self.ce_chunk_rows)
        if self.moe_layers and self.tcfg.z_loss_weight and self.router_records:
            if self.z_loss_mode == "layers_logits":
                # mean over every MoE layer application of mean(logsumexp(logits)^2)
                zs = [z for _, z, _ in self.router_records if z is not None]
                z = torch.stack(zs).mean()
            else:
                # the reference train step's form: the last MoE layer's sigmoid scores
                z = torch.logsumexp(self.router_records[-1][2], dim=-1).square().mean()
            ce = ce + float(self.tcfg.z_loss_weight) * z * (self._micro_weight(loss_mask, denom))
        self.router_records = []
        return ce

    @staticmethod
    def _micro_weight(loss_mask: Tensor, denom) -> Tensor:
        """Share of the step's loss tokens in this micro-batch (auxiliary terms are weighted by
        it so that they sum to one step-level mean)."""
        m = loss_mask.float()[:, 1:].sum()
        return m / denom

    # ---------------------------------------------------------------- optimizer
    def _sync_grads(self) -> None:
        """Make the owned gradient slices (and all vector gradients) global sums and put the
        squared global gradient norm in ``self.gnorm_sq``."""
        st = stream_ptr()
        if self.world > 1 and self.sym is None:
            import torch.distributed as dist

            for g in (self.muon_grad, self.adam_grad, self.vec_grad):
                dist.all_reduce(g, group=self.pg)
        if self.sym is None:
            call("pb_sumsq_f32", ptr(self.muon_grad), self.n_muon, ptr(self.opt_scratch),
                 ptr(self.gnorm_sq), 0, st)
            call("pb_sumsq_f32", ptr(self.adam_grad), self.n_adam, ptr(self.opt_scratch),
                 ptr(self.gnorm_sq), 1, st)
            call("pb_sumsq_f32", ptr(self.vec_grad), self.n_vec, ptr(self.opt_scratch),
                 ptr(self.gnorm_sq), 1, st)
            return
        sym = self.sym
        noop = self.comm_noop               # timing only: same kernels minus the peer traffic
        if self.fsdp:                       # no pull of a working weight may still be in flight
            torch.cuda.current_stream(self.device).wait_stream(self.fetch_stream)
        if not noop:
            sym.barrier(0)                  # every rank's backward is complete
        first = True

        def fold(byte_off, lo, n, out):
            nonlocal first
            if noop:
                call("pb_sumsq_f32", ptr(out[lo:]), n, ptr(self.opt_scratch), ptr(self.local_sq),
                     0 if first else 1, st)
            else:
                sym.reduce_to_owner(self.sym_grad, byte_off, lo, n, out, self.opt_scratch,
                                    self.local_sq, not first)
            first = False

        for key, units in sorted(self.unit_classes.items()):
            rows, cols = key[:2]
            lo_u, hi_u = self.own_units[key]
            if hi_u > lo_u:
                lo = units[0].off + lo_u * rows * cols
                if len(key) > 2:       # this rank's experts: the local gradient is the gradient
                    call("pb_sumsq_f32", ptr(self.muon_grad[lo:]), (hi_u - lo_u) * rows * cols,
                         ptr(self.opt_scratch), ptr(self.local_sq), 0 if first else 1, st)
                    first = False
                else:
                    fold(0, lo, (hi_u - lo_u) * rows * cols, self.muon_grad)
        a_lo, a_hi = self.own_adam
        if a_hi > a_lo:
            fold(4 * self.n_muon, a_lo, a_hi - a_lo, self.adam_grad)
        if first:
            self.local_sq.zero_()
        # vectors: every rank folds all peers (same order, same bits) into a private copy
        if not hasattr(self, "vec_sum"):
            self.vec_sum = torch.zeros_like(self.vec_master)
        if noop:
            self.vec_sum.copy_(self.vec_grad)
            call("pb_sumsq_f32", ptr(self.vec_sum), self.n_vec, ptr(self.opt_scratch),
                 ptr(self.vec_sq), 0, st)
            self.gnorm_sq.copy_(self.local_sq)
        else:
            sym.reduce_to_owner(self.sym_grad, 4 * (self.n_muon + self.n_adam), 0, self.n_vec,
                                self.vec_sum, self.opt_scratch, self.vec_sq, False)
            sym.allreduce_scalar(self.local_sq, self.gnorm_sq)   # also: all reads of grads done
        self.gnorm_sq.add_(self.vec_sq)

    def _newton_schulz_class(self, rows: int, cols: int, nb: int, steps: int) -> Tensor:
        """Batched quintic Newton-Schulz over ``nb`` matrices of one shape, in bf16 on the
        tcgen05 GEMM. Input: self.ns_x[0] holds the normalised Nesterov momenta."""
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
        return x

    def optimizer_step(self, lr_mult: float, gscale: float = 1.0) -> None:
        """Clip, AdamW slabs, batched Muon on the owned matrices; refreshes the bf16 working
        copies: locally, into every peer's replica, or into the shard holders (ZeRO-3)."""
        tc = self.tcfg
        st = stream_ptr()
        clip = float(tc.grad_clip)
        step = self.step_count
        hp = (float(tc.adamw_lr) * lr_mult, float(tc.adamw_beta1), float(tc.adamw_beta2),
              float(tc.adamw_eps), float(tc.adamw_wd))
        vec_grad = self.vec_sum if self.sym is not None else self.vec_grad
        call("pb_adamw", ptr(self.vec_master), ptr(vec_grad), ptr(self.vec_m), ptr(self.vec_v),
             None, self.n_vec, *hp, step, ptr(self.gnorm_sq), clip, gscale, st)
        a_lo, a_hi = self.own_adam
        sh = self.adam_shift
        peers_on = self.sym is not None and not self.comm_noop
        if self.fsdp:
            for lo, n, (pos, chunk, base) in self.adam_segments:
                if not peers_on:       # timing only: same arithmetic, bf16 result to a scratch buffer
                    call("pb_adamw", ptr(self.adam_master[lo - sh:]), ptr(self.adam_grad[lo:]),
                         ptr(self.adam_m[lo - sh:]), ptr(self.adam_v[lo - sh:]),
                         ptr(self._noop_scratch(n)), n, *hp, step, ptr(self.gnorm_sq), clip, gscale, st)
                    continue
                call("pb_adamw_table", ptr(self.adam_master[lo - sh:]), ptr(self.adam_grad[lo:]),
                     ptr(self.adam_m[lo - sh:]), ptr(self.adam_v[lo - sh:]), n, *hp, step,
                     ptr(self.gnorm_sq), clip, gscale, pos, chunk, base, self.sym_lp.ptrs,
                     self.world, self.rank, st)
        elif self.sym is None:
            call("pb_adamw", ptr(self.adam_master), ptr(self.adam_grad), ptr(self.adam_m),
                 ptr(self.adam_v), ptr(self.adam_lp), self.n_adam, *hp, step, ptr(self.gnorm_sq),
                 clip, gscale, st)
        elif a_hi > a_lo:
            if peers_on and self.nvls_lp is not None:
                # one multimem.st per 16 bytes: the switch replicates it into every rank's copy
                call("pb_mm_adamw", ptr(self.adam_master[a_lo:]), ptr(self.adam_grad[a_lo:]),
                     ptr(self.adam_m[a_lo:]), ptr(self.adam_v[a_lo:]),
                     self.nvls_lp.mc_at(2 * (self.n_muon + a_lo)), a_hi - a_lo, *hp, step,
                     ptr(self.gnorm_sq), clip, gscale, st)
            elif peers_on:
                call("pb_adamw_bcast", ptr(self.adam_master), ptr(self.adam_grad), ptr(self.adam_m),
                     ptr(self.adam_v), self.sym_lp.peer_ptrs(2 * self.n_muon), self.world, a_lo,
                     a_hi - a_lo, *hp, step, ptr(self.gnorm_sq), clip, gscale, st)
            else:
                call("pb_adamw", ptr(self.adam_master[a_lo:]), ptr(self.adam_grad[a_lo:]),
                     ptr(self.adam_m[a_lo:]), ptr(self.adam_v[a_lo:]), ptr(self.adam_lp[a_lo:]),
                     a_hi - a_lo, *hp, step, ptr(self.gnorm_sq), clip, gscale, st)
        lr = float(tc.muon_lr) * lr_mult
        beta = float(tc.muon_momentum)
        for key, units in sorted(self.unit_classes.items()):
            rows, cols = key[:2]
            lo_u, hi_u = self.own_units[key]
            nb = hi_u - lo_u
            if nb == 0:
                continue
            n = rows * cols
            base = units[0].off + lo_u * n           # gradients: global flat offsets
            lb = self.class_lbase[key]               # masters / momenta: where this rank keeps them
            # momentum, Nesterov and Frobenius normalisation of the whole shape class: three
            # launches whatever the number of matrices
            call("pb_muon_prepare_batched", ptr(self.muon_grad[base:]), ptr(self.muon_mom[lb:]),
                 ptr(self.ns_x[0]), n, nb, beta, ptr(self.gnorm_sq), clip, gscale,
                 ptr(self.opt_scratch), st)
            xo = self._newton_schulz_class(rows, cols, nb, int(tc.muon_ns_steps))
            scale = T.muon_rms_scale(rows, cols)
            if self.fsdp and peers_on:
                call("pb_muon_apply_table", ptr(self.muon_master[lb:]), ptr(xo), n, nb, lr, scale,
                     self.muon_wd, ptr(self.dest_tables[key][lo_u:]), self.sym_lp.ptrs, self.world,
                     self.rank, st)
            elif self.fsdp:            # timing only: bf16 result to a scratch buffer
                call("pb_muon_apply", ptr(self.muon_master[lb:]), ptr(xo),
                     ptr(self._noop_scratch(n * nb)), n * nb, lr, scale, self.muon_wd, st)
            elif self.sym is None or len(key) > 2 or not peers_on:
                call("pb_muon_apply", ptr(self.muon_master[lb:]), ptr(xo),
                     ptr(self.muon_lp[base:]), n * nb, lr, scale, self.muon_wd, st)
            elif self.nvls_lp is not None:
                call("pb_mm_muon_apply", ptr(self.muon_master[lb:]), ptr(xo),
                     self.nvls_lp.mc_at(2 * base), n * nb, lr, scale, self.muon_wd, st)
            else:
                call("pb_muon_apply_bcast", ptr(self.muon_master), ptr(xo),
                     self.sym_lp.peer_ptrs(0), self.world, base, n * nb, lr, scale,
                     self.muon_wd, st)
        if self.fsdp:
            self._fsdp_invalidate()         # every landing slot is stale now
        if self.sym is not None and not self.comm_noop:
            self.sym.barrier(3)             # every peer's stores into my weights have landed

    def _noop_scratch(self, n: int) -> Tensor:
        """bf16 scratch the no-traffic timing mode writes refreshed weights to (so that the
        real shards keep valid contents)."""
        t = getattr(self, "_noop_lp", None)
        if t is None or t.numel() < n:
            t = torch.empty(n, dtype=BF16, device=self.device)
            self._noop_lp = t
        return t

    def zero_grad(self) -> None:
        self.muon_grad.zero_()
        self.adam_grad.zero_()
        self.vec_grad.zero_()

    # --------------------------------------------------------------------- step
    def step(self, tokens: Tensor, loss_mask: Tensor | None = None) -> dict:
        """One optimizer step over a local batch (B_local, S) of token ids on the device.
        Returns device scalars: loss (mean CE over the global batch) and grad_norm.
        Under context parallelism the batch is what ``cp_slice`` returns: this rank's slice plus
        one next-token column, ``(B, S_local + 1)``, or with the zig-zag split its two half-slices
        each followed by that column, ``(B, S_local + 2)``."""
        self.step_count += 1
        t = self.step_count
        sched = T.wsd_lr(t, self.tcfg)
        peak = float(self.tcfg.peak_lr)
        lr_mult = sched / peak if peak > 0 else 0.0
        self._router_load = {}
        clip_qk = float(self.tcfg.qk_clip) > 0 and not self.cp and any(
            k_ is M.AttentionKind.GQA for k_ in self.layer_kinds) and \
            M.head_geometry(self.cfg)[1] == 128
        self.track_max_logit = clip_qk
        self.max_logits = {}
        if loss_mask is None:
            loss_mask = torch.ones_like(tokens, dtype=torch.float32)
        if self.cp_zigzag:     # two half-slices, each followed by its next-token column
            denom = loss_mask.float().reshape(loss_mask.shape[0], 2, -1)[:, :, 1:].sum()
        else:
            denom = loss_mask[:, 1:].sum().float()
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(denom, group=self.pg)
        denom = denom.clamp(min=1.0)
        total = torch.zeros((), dtype=torch.float32, device=tokens.device)
        mtp_denoms = None
        if self.cfg.mtp_heads:
            S = tokens.shape[1]
            m = loss_mask.float()
            dj = torch.stack([(m[:, j + 1:] * m[:, : S - j - 1]).sum()
                              for j in range(self.cfg.mtp_heads)])
            if self.world > 1:
                import torch.distributed as dist

                dist.all_reduce(dj, group=self.pg)
            mtp_denoms = list(dj.clamp(min=1.0))
        mb = self.micro_batch
        ev = None
        if self.time_phases:
            self._harvest_phase_times()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
        for b0 in range(0, tokens.shape[0], mb):
            l = self.loss(tokens[b0:b0 + mb], loss_mask[b0:b0 + mb], denom, mtp_denoms)
            l.backward()
            total += l.detach()
        if ev is not None:
            ev[1].record()
        if self.router_bias and self._router_load:
            # aux-loss-free balancing, every MoE layer from its own load:
            # b_i <- b_i - u sign(load_i - mean(load_i))
            layers = sorted(self._router_load)
            load = torch.stack([self._router_load[i] for i in layers])
            if self.world > 1:
                import torch.distributed as dist

                dist.all_reduce(load, group=self.pg)
            load = load / load.sum(dim=1, keepdim=True).clamp(min=1.0)
            delta = torch.sign(load - load.mean(dim=1, keepdim=True)) * self.router_bias_rate
            for row, i in enumerate(layers):
                self.router_bias[i].sub_(delta[row])
            self.moe_load = load            # (MoE layers, experts) shares, for the metrics
        self._sync_grads()
        if ev is not None:
            ev[2].record()
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(total, group=self.pg)
        self.optimizer_step(lr_mult)
        if clip_qk and self.max_logits:
            self._qk_clip()
        if ev is not None:
            ev[3].record()
            self._phase_events = ev
        gnorm = self.gnorm_sq.sqrt()
        self.zero_grad()
        if self.debug_canaries and self.sym is not None:
            self.check_canaries()
        return {"loss": total, "grad_norm": gnorm, "lr": sched, "step": t,
                "status": self.status_tensor()}

    def _harvest_phase_times(self) -> None:
        """Device times of the previous step's phases (its events have completed by the time the
        next step starts, so reading them does not stall): forward + backward, the gradient
        synchronisation (barrier wait + fold: what the compute stream spent inside
        communication, i.e. an upper bound of the exposed communication), optimizer + weight
        refresh."""
        ev = getattr(self, "_phase_events", None)
        if ev is None or not ev[3].query():
            return
        self.phase_times = {"fwd_bwd_ms": ev[0].elapsed_time(ev[1]), "sync_ms": ev[1].elapsed_time(ev[2]),
                            "opt_ms": ev[2].elapsed_time(ev[3])}
        self._phase_events = None

    def _qk_clip(self) -> None:
        """QK-clip on the logits the attention kernel saw this step: heads whose largest scaled
        logit exceeded ``qk_clip`` have the rows of their query / key projections scaled so that
        the same inputs would give exactly ``qk_clip`` (``pb_qk_clip_rescale``). Every rank
        applies the same factors (the maxima are reduced over the ranks) to its bf16 copy and to
        the fp32 masters it holds. Reference: train/__init__.py:478-500, 791-807 (there on the
        weight rows themselves; here on observed logits)."""
        cfg = self.cfg
        nh, dh, nkv = M.head_geometry(cfg)
        layers = sorted(self.max_logits)
        m = torch.stack([self.max_logits[i] for i in layers]).contiguous()
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.pg)
        tau = float(self.tcfg.qk_clip)
        st = stream_ptr()
        for row, i in enumerate(layers):
            pre = f"layers.{i}."
            for name, is_k, heads in ((pre + "q", 0, nh), (pre + "k", 1, nkv)):
                w = self.weights[name]
                n = heads * dh * cfg.d_model
                args = (heads * dh, cfg.d_model, dh, nh // nkv, nh, is_k, 0, ptr(m[row]), tau, st)
                pieces = self._owned_pieces("muon", w.off, w.off + n)
                owned = bool(pieces) and pieces[0][1] - pieces[0][0] == n
                master = self.muon_master[pieces[0][2]:] if owned else None
                if self.sym is None:
                    call("pb_qk_clip_rescale", ptr(master), ptr(self.p[name]), *args)
                elif not self.fsdp:
                    # replicas must stay bit-identical: every rank rescales its bf16 copy from
                    # the copy itself; the fp32 master is rescaled where it lives
                    call("pb_qk_clip_rescale", ptr(master), None, *args)
                    call("pb_qk_clip_rescale", None, ptr(self.p[name]), *args)
                elif owned:
                    # the owner rescales the master and re-stores its bf16 value to the shard
                    # holders (the update kernel with a zero step)
                    key, idx = self.unit_index[(name, 0)]
                    call("pb_qk_clip_rescale", ptr(master), None, *args)
                    call("pb_muon_apply_table", ptr(master), ptr(self.ns_x[0]), n, 1, 0.0, 0.0, 0.0,
                         ptr(self.dest_tables[key][idx:]), self.sym_lp.ptrs, self.world, self.rank, st)
        if self.fsdp:
            self._fsdp_invalidate()
            self.sym.barrier(3)
        self.last_max_logits = m

    def status_tensor(self) -> Tensor:
        """Device int32: non-zero when a bounded device-side wait of this rank's kernels or of the
        peer-memory collectives ran out since the last check."""
        st = ops.status_word(self.device)
        if self.sym is not None:
            return torch.maximum(st, self.sym.status.to(st.device))
        return st

    def raise_on_status(self, code: int) -> None:
        """Turn a latched wait-timeout code into an exception and clear the words, so a step that
        ran on partial gradients or stale weights is never silently kept."""
        if code:
            ops.status_word(self.device).zero_()
            if self.sym is not None:
                self.sym.status.zero_()
            raise DeviceWaitTimeout(code, self.rank, self.step_count)


    def cp_slice(self, tokens: Tensor, loss_mask: Tensor | None = None):
        """This rank's slice of full sequences ``(B, S)`` for a context-parallel step:
        ``(tokens (B, S/world + 1), mask (B, S/world + 1))`` (zig-zag: two half-slices, each with
        its extra column, ``S/world + 2`` in all) with the extra column holding the next
        slice's first token (mask 0 after the end of the sequence)."""
        B, S = tokens.shape
        parts = 2 * self.world if self.cp_zigzag else self.world
        if S % parts:
            raise ValueError(f"sequence length must be divisible by {parts}")
        sl = S // parts
        mask = torch.ones_like(tokens, dtype=torch.float32) if loss_mask is None else loss_mask.float()
        tok_x = torch.cat([tokens, tokens[:, :1]], dim=1)
        m_x = torch.cat([mask, torch.zeros_like(mask[:, :1])], dim=1)
        # zig-zag: half-slices rank and 2 world - 1 - rank, each followed by its next token
        starts = [self.rank * sl, (parts - 1 - self.rank) * sl] if self.cp_zigzag else [self.rank * sl]
        tok = torch.cat([tok_x[:, lo:lo + sl + 1] for lo in starts], dim=1)
        m = torch.cat([m_x[:, lo:lo + sl + 1] for lo in starts], dim=1)
        return tok.contiguous(), m.contiguous()

    def step_from_host(self, host_tokens: Tensor, host_mask: Tensor | None = None) -> dict:
        """Public end-to-end step: token ids (and optional mask) in pinned host memory are
        copied to the device, one optimizer step runs, and the loss and gradient norm are
        read back to the host as Python floats."""
        tok = host_tokens.to(self.device, non_blocking=True)
        mask = None if host_mask is None else host_mask.to(self.device, non_blocking=True)
        out = self.step(tok, mask)
        # the status word rides in the same read-back as the loss: no extra synchronisation
        host = torch.stack([out["loss"], out["grad_norm"].reshape(()),
                            out["status"].reshape(()).float()]).cpu()
        if self.check_status_every and out["step"] % self.check_status_every == 0:
            self.raise_on_status(int(host[2]))
        return {"loss": float(host[0]), "grad_norm": float(host[1]), "lr": out["lr"],
                "step": out["step"], "status": int(host[2])}
