"""Expert parallelism: the MoE FFN with its experts spread over the ranks of one box.

Rank r owns routed experts ``[r * El, (r + 1) * El)``. Tokens reach their experts and come
back through symmetric memory (``csrc/comm/ep.cu``): the sender stores its rows straight into
the owner's receive buffer over NVLink (push), the owner runs the grouped tcgen05 GEMMs on
what arrived, and the sender reads its results back out of the owner's buffer (pull) while
applying the gates. With ``fp8=True`` the rows cross NVLink as e4m3 bytes plus 1 x 128 scales
(half the bytes), quantised by the sending kernel, and the grouped FP8 GEMM reads the receive
buffers as they are. The only synchronisation is three bounded device barriers per direction
(counts visible, rows landed, results ready); the GEMMs write their results straight into the
buffer the peers pull from. There is no host round trip and no library collective in the layer.

Reference behaviour: ``kernels/__init__.py`` ``ep_dispatch`` / ``ep_combine`` of the reference
(stable token order per expert, capacity overflow reported rather than silently reordered) and
``model/__init__.py:485-598`` for the routing math.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops import moe as M
from ..ops._lib import call, ptr, stream_ptr
from .symm import PP, SymmetricBuffer, SymmetricGroup

P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
_lib.register("pb_ep_layout", [PP, I, I, I, I, P, P, P, P, P, P, P, P])
_lib.register("pb_ep_dispatch", [P, L, P, P, P, P, P, I, I, I, I, I, PP, I, P, P, P])
_lib.register("pb_ep_dispatch_fp8", [P, L, P, P, P, P, I, I, I, I, I, PP, PP, PP, I, P, P, P])
_lib.register("pb_ep_zero_pad_fp8", [P, P, I, I, P, P, I, P])
_lib.register("pb_ep_combine", [PP, I, P, P, P, P, I, I, I, P, P])
_lib.register("pb_ep_rowdot", [P, P, P, I, I, P, P])
_lib.register("pb_ep_pull_scalar", [PP, I, P, P, P, I, P, P])

BF16 = torch.bfloat16
Tensor = torch.Tensor


class EpContext:
    """Symmetric buffers of one expert-parallel group (shared by all MoE layers).

    ``max_rows``: rows a rank can receive per layer (multiple of 128). A layer that needs more
    latches an overflow code in the status word (``SymmetricGroup.check``) and drops the excess
    pairs; size it as ``capacity_factor * tokens_per_rank * top_k`` plus 127 rows per local expert.
    """

    def __init__(self, sym: SymmetricGroup, d_model: int, n_experts: int, max_rows: int,
                 fuse_dispatch: bool = False):
        self.sym = sym
        # FP8 path only: True = no barrier between dispatch and the first grouped GEMM, the
        # GEMM's TMA producer takes each 128-row block when the senders' per-row counts say it
        # is complete; False = one bounded barrier, then the plain grouped GEMM. Measured on
        # two B200s at 32768 tokens per rank the barrier form is the faster one (the senders
        # push in token order, so blocks complete late, and the per-row system-scope counts
        # cost the senders more than the barrier costs the owners).
        self.fuse_dispatch = bool(fuse_dispatch)
        self.world, self.rank = sym.world, sym.rank
        if n_experts % self.world:
            raise ValueError("the expert count must be divisible by the expert-parallel size")
        self.E, self.El, self.d = n_experts, n_experts // self.world, d_model
        self.max_rows = (int(max_rows) + 127) // 128 * 128
        g = sym.group
        self.counts = SymmetricBuffer(4 * n_experts, g)
        self.fp8_ok = d_model % 128 == 0
        if self.fp8_ok:        # FP8 receive buffers: e4m3 rows and their [d / 128, max_rows] scales
            self.xqbuf = SymmetricBuffer(self.max_rows * d_model, g)
            self.xsbuf = SymmetricBuffer(4 * (d_model // 128) * self.max_rows, g)
            self.xq_local = self.xqbuf.view(torch.uint8, self.max_rows * d_model).view(self.max_rows, d_model)
            self.xs_local = self.xsbuf.view(torch.float32, (d_model // 128) * self.max_rows).view(
                d_model // 128, self.max_rows)
            # fused dispatch: rows landed per 128-row block of this rank's FP8 receive buffer
            # (peers add to it), and how many each block expects (from the layout)
            self.arrbuf = SymmetricBuffer(4 * (self.max_rows // 128), g)
            self.arrived_local = self.arrbuf.view(torch.int32, self.max_rows // 128)
            self.blk_expect = torch.zeros(self.max_rows // 128, dtype=torch.int32,
                                          device=self.arrived_local.device)
        self.xbuf = SymmetricBuffer(2 * self.max_rows * d_model, g)
        self.ybuf = SymmetricBuffer(2 * self.max_rows * d_model, g)
        self.dotbuf = SymmetricBuffer(4 * self.max_rows, g)
        self.counts_local = self.counts.view(torch.int32, n_experts)
        self.x_local = self.xbuf.view(BF16, self.max_rows * d_model).view(self.max_rows, d_model)
        self.y_local = self.ybuf.view(BF16, self.max_rows * d_model).view(self.max_rows, d_model)
        self.dot_local = self.dotbuf.view(torch.float32, self.max_rows)

    def layout(self):
        dev = self.x_local.device
        i32 = dict(dtype=torch.int32, device=dev)
        pl = M.Placement(row_of=None, expert_off=torch.empty(self.El + 1, **i32),
                         totals=torch.empty(self.El, **i32), k_len=torch.empty(self.El, **i32),
                         mblk_group=torch.empty(self.max_rows // 128, **i32), rows=self.max_rows,
                         n_experts=self.El, top_k=0)
        send_base = torch.empty(self.E, **i32)
        call("pb_ep_layout", self.counts.ptrs, self.rank, self.world, self.E, self.max_rows,
             ptr(pl.expert_off), ptr(pl.totals), ptr(pl.k_len), ptr(pl.mblk_group), ptr(send_base),
             ptr(self.blk_expect) if self.fp8_ok else None, ptr(self.sym.status), stream_ptr())
        return pl, send_base

    def dispatch(self, x: Tensor, ids: Tensor, local: M.Placement, send_base: Tensor,
                 scale: Tensor | None):
        T, k = ids.shape
        dev = x.device
        dest_rank = torch.empty(T * k, dtype=torch.int32, device=dev)
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        call("pb_ep_dispatch", ptr(x), x.stride(0), ptr(ids), ptr(local.row_of), ptr(local.expert_off),
             ptr(send_base), ptr(scale), T * k, k, self.d, self.El, self.max_rows, self.xbuf.ptrs,
             self.world, ptr(dest_rank), ptr(dest_row), stream_ptr())
        return dest_rank, dest_row

    def dispatch_fp8(self, x: Tensor, ids: Tensor, local: M.Placement, send_base: Tensor,
                     count_arrivals: bool = True):
        """Quantise and push: e4m3 rows + 1 x 128 scales into the owners' FP8 receive buffers,
        and (``count_arrivals``) one count per landed row into the owner's per-block arrival
        counters, which its grouped GEMM waits on block by block."""
        T, k = ids.shape
        dev = x.device
        dest_rank = torch.empty(T * k, dtype=torch.int32, device=dev)
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        call("pb_ep_dispatch_fp8", ptr(x), x.stride(0), ptr(ids), ptr(local.row_of), ptr(local.expert_off),
             ptr(send_base), T * k, k, self.d, self.El, self.max_rows, self.xqbuf.ptrs, self.xsbuf.ptrs,
             self.arrbuf.ptrs if count_arrivals else None, self.world, ptr(dest_rank), ptr(dest_row),
             stream_ptr())
        return dest_rank, dest_row

    def zero_pad_fp8(self, pl: M.Placement) -> None:
        call("pb_ep_zero_pad_fp8", ptr(self.xq_local), ptr(self.xs_local), self.d, self.max_rows,
             ptr(pl.expert_off), ptr(pl.totals), self.El, stream_ptr())

    def combine(self, dest_rank, dest_row, gates, T: int, k: int, add: Tensor | None = None) -> Tensor:
        out = torch.empty((T, self.d), dtype=BF16, device=dest_rank.device)
        call("pb_ep_combine", self.ybuf.ptrs, self.world, ptr(dest_rank), ptr(dest_row), ptr(gates),
             ptr(add), T, k, self.d, ptr(out), stream_ptr())
        return out

    def zero_pad(self, pl: M.Placement) -> None:
        call("pb_moe_zero_pad", ptr(self.x_local), self.d, ptr(pl.expert_off), ptr(pl.totals),
             self.El, stream_ptr())


def _copy_used(src: Tensor, used: Tensor) -> Tensor:
    """A copy of the rows of a worst-case-sized 2-D buffer that are in use (``used``: device int32
    count); the rest of the result is uninitialised and never read."""
    dst = torch.empty_like(src)
    call("pb_copy_rows_dyn", ptr(src), ptr(dst), src.shape[1] * src.element_size(), src.shape[0],
         ptr(used), stream_ptr())
    return dst


class _EpMoeFn(torch.autograd.Function):
    """Barrier slots: 4 = every rank's per-expert counts are written (forward only), 5 = every
    pushed row has landed, 6 = every owner's results are in its pull buffer. No barrier
    separates layers or directions: a rank overwrites a peer's receive buffer only after passing
    slot 6 of the previous layer, which the peer reached after its last read of that buffer, and
    its own pull buffers only after slot 4 (forward) or 5 (backward) of the layer, which every
    puller of the previous contents reached after its pulls."""

    @staticmethod
    def forward(ctx, x, router_w, router_bias, w_gu_p, w_down_p, top_k, ep, shapes, fp8=False):
        from ..ops import fp8 as F8
        from ..ops.functional import gemm

        w_gu = w_gu_p.view(shapes[0]) if shapes is not None else w_gu_p      # [El, 2h, d]
        w_down = w_down_p.view(shapes[1]) if shapes is not None else w_down_p
        T, d = x.shape
        h = w_gu.shape[1] // 2
        sym = ep.sym
        use_fp8 = bool(fp8) and ep.fp8_ok and h % 128 == 0
        logits = gemm(x, router_w, out_dtype=torch.float32)
        probs, ids, gates = M.route(logits, router_bias, top_k)
        local = M.place(ids, ep.E)
        ep.counts_local.copy_(local.totals)
        sym.barrier(4)
        pl, send_base = ep.layout()
        used = pl.expert_off[ep.El:]            # device int: rows of the receive buffer in use
        if use_fp8 and ep.fuse_dispatch:
            # Fused dispatch + first grouped GEMM: no barrier between them. The senders count
            # every landed row into the owner's per-block counters and the GEMM's TMA producer
            # takes a 128-row block as soon as that block is complete (bounded wait).
            ep.zero_pad_fp8(pl)                 # padding rows only: disjoint from what peers store
            wq, sw = F8.quantize_blocks(w_gu.contiguous())
            dest_rank, dest_row = ep.dispatch_fp8(x, ids, local, send_base)
            gu = F8.gemm_fp8(ep.xq_local, ep.xs_local, wq, sw, mblk_group=pl.mblk_group,
                             arrived=ep.arrived_local, expect=ep.blk_expect, budget_ns=sym.budget_ns)
            ep.arrived_local.zero_()            # before this rank's next slot-4 arrival
            saved_x = (_copy_used(ep.xq_local, used), ep.xs_local.clone())
        elif use_fp8:
            dest_rank, dest_row = ep.dispatch_fp8(x, ids, local, send_base, count_arrivals=False)
            sym.barrier(5)                      # every row has landed
            ep.zero_pad_fp8(pl)
            wq, sw = F8.quantize_blocks(w_gu.contiguous())
            gu = F8.gemm_fp8(ep.xq_local, ep.xs_local, wq, sw, mblk_group=pl.mblk_group)
            # what the backward differentiates against: the quantised rows (half the bytes of a
            # bf16 copy); the receive buffer itself is overwritten by the next layer's senders
            saved_x = (_copy_used(ep.xq_local, used), ep.xs_local.clone())
        else:
            dest_rank, dest_row = ep.dispatch(x, ids, local, send_base, None)
            sym.barrier(5)
            ep.zero_pad(pl)
            xp = _copy_used(ep.x_local, used)
            gu = M.grouped_gemm(xp, w_gu, pl)
            saved_x = (xp, xp.new_empty(0))
        if use_fp8:
            _none, hq, sh = F8.swiglu_quantize(gu, used, keep_bf16=False)   # SwiGLU -> e4m3 rows in one pass
            wq, sw = F8.quantize_blocks(w_down.contiguous())
            F8.gemm_fp8(hq, sh, wq, sw, mblk_group=pl.mblk_group, out=ep.y_local)
            saved_h = (hq, sh)         # the backward differentiates against the quantised rows
        else:
            hs = torch.empty((pl.rows, h), dtype=BF16, device=x.device)
            call("pb_swiglu_fwd_dyn", ptr(gu), ptr(hs), pl.rows, h, ptr(used), stream_ptr())
            M.grouped_gemm(hs, w_down, pl, out=ep.y_local)
            saved_h = (hs, hs.new_empty(0))
        y = _copy_used(ep.y_local, used)        # the gate gradient needs <y_row, dy_row> later
        sym.barrier(6)                          # results are ready to be pulled
        out = ep.combine(dest_rank, dest_row, gates, T, top_k)
        ctx.save_for_backward(x, router_w, w_gu, w_down, probs, ids, gates, saved_x[0], saved_x[1], gu,
                              saved_h[0], saved_h[1], y, dest_rank, dest_row, send_base)
        ctx.pl, ctx.local, ctx.ep, ctx.use_fp8 = pl, local, ep, use_fp8
        ctx.refs = (router_w, w_gu_p, w_down_p)
        ctx.mark_non_differentiable(ids)
        return out, probs, ids, logits

    @staticmethod
    def backward(ctx, d_out, d_probs, _di, d_logits=None):
        from ..ops import fp8 as F8
        from ..ops.functional import gemm

        (x, router_w, w_gu, w_down, probs, ids, gates, xs0, xs1, gu, hs0, hs1, y, dest_rank, dest_row,
         send_base) = ctx.saved_tensors
        router_ref, gu_ref, down_ref = ctx.refs
        pl, local, ep = ctx.pl, ctx.local, ctx.ep
        sym = ep.sym
        T, d = x.shape
        k = ids.shape[1]
        E = router_w.shape[0]
        h = w_gu.shape[1] // 2
        d_out = d_out.contiguous()
        gflat = gates.reshape(-1)
        ep.dispatch(d_out, ids, local, send_base, gflat)       # dY rows = gate * dOut[t], bf16
        sym.barrier(5)
        ep.zero_pad(pl)
        dyp = ep.x_local            # read in place: nobody overwrites it before slot 6 below
        used = pl.expert_off[ep.El:]
        call("pb_ep_rowdot", ptr(y), ptr(dyp), ptr(used), pl.rows, d, ptr(ep.dot_local), stream_ptr())
        # straight-through on what the FP8 products multiplied: quantised weights and rows
        wd_b = F8.fakequant_blocks(w_down.contiguous()) if ctx.use_fp8 else w_down
        dh = M.grouped_gemm(dyp, wd_b, pl, b_mn=True)
        hs = F8.dequantize_rows_bf16(hs0, hs1, used) if ctx.use_fp8 else hs0
        g_down = M._acc_grad(down_ref, w_down.shape, lambda o, acc: M.grouped_wgrad(dyp, hs, pl, o, acc))
        del hs, wd_b
        dgu = torch.empty_like(gu)
        call("pb_swiglu_bwd_dyn", ptr(dh), ptr(gu), ptr(dgu), pl.rows, h, ptr(used), stream_ptr())
        xp = F8.dequantize_rows_bf16(xs0, xs1, used) if ctx.use_fp8 else xs0
        g_gu = M._acc_grad(gu_ref, w_gu.shape, lambda o, acc: M.grouped_wgrad(dgu, xp, pl, o, acc))
        del xp
        wg_b = F8.fakequant_blocks(w_gu.contiguous()) if ctx.use_fp8 else w_gu
        M.grouped_gemm(dgu, wg_b, pl, b_mn=True, out=ep.y_local)
        del wg_b
        sym.barrier(6)
        dgates = torch.empty((T, k), dtype=torch.float32, device=x.device)
        call("pb_ep_pull_scalar", ep.dotbuf.ptrs, ep.world, ptr(dest_rank), ptr(dest_row), ptr(gflat),
             T * k, ptr(dgates), stream_ptr())
        dlogits = torch.empty((T, E), dtype=torch.float32, device=x.device)
        call("pb_moe_route_bwd", ptr(dgates), ptr(gates), ptr(probs), ptr(ids), T, E, k, ptr(dlogits),
             stream_ptr())
        if d_probs is not None:
            dlogits = dlogits + d_probs * probs * (1.0 - probs)
        if d_logits is not None:
            dlogits = dlogits + d_logits
        dl = dlogits.to(BF16)
        dx_r = gemm(dl, router_w, b_mn=True)
        dx = ep.combine(dest_rank, dest_row, None, T, k, add=dx_r)
        mg = getattr(router_ref, "main_grad", None)
        g_router = None
        if mg is not None:
            gemm(dl, x, a_mn=True, b_mn=True, out=mg.view(router_w.shape), d=mg.view(router_w.shape),
                 beta=1.0)
        else:
            g_router = gemm(dl, x, a_mn=True, b_mn=True)
        return dx, g_router, None, g_gu, g_down, None, None, None, None


def ep_moe_ffn(x: Tensor, router_w: Tensor, router_bias: Tensor | None, w_gu_local: Tensor,
               w_down_local: Tensor, top_k: int, ep: EpContext, shapes=None,
               return_logits: bool = False, fp8: bool = False):
    """Routed-expert FFN with the experts sharded over ``ep``'s ranks. x [T, d] are this rank's
    tokens; router_w [E, d] is replicated; w_gu_local [El, 2h, d] and w_down_local [El, d, h]
    are this rank's experts. Returns (out [T, d], probs [T, E], ids [T, k]). Collective: every
    rank of the group must call it (same layer order), forward and backward. ``return_logits``
    appends the router logits [T, E] fp32 (differentiable). ``fp8``: tokens cross NVLink as e4m3
    rows + 1 x 128 scales and both expert products run on the block-scaled FP8 GEMM
    (straight-through backward on the quantised rows and weights, as bf16 products)."""
    res = _EpMoeFn.apply(x, router_w, router_bias, w_gu_local, w_down_local, int(top_k), ep, shapes,
                         bool(fp8))
    return res if return_logits else res[:3]
