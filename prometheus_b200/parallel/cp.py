"""Context parallelism: sequence split, ring schedule, ring attention with an online-softmax
fold, and the delta-rule chunk-state hand-off.

Softmax layers follow the reference (``parallel/cp.py:45-324``): equal contiguous chunks,
ring step ``t`` sees KV owner ``(rank - t) mod n``, fold state ``(m, l, acc)`` starting at
``(-inf, 0, 0)``, causal mask by global index with the ``-1e9`` sentinel, softmax floor
``1e-12``.

Delta-rule layers (no counterpart in the reference): over one rank's slice the state map is
affine, ``S_out = P S_in + R`` with ``P = prod_chunks (I - K^T W)`` and ``R`` the state
reached from zero. Ranks build ``(P_r, R_r)`` locally in parallel, exchange those small
operands (heads x 128 x 128 fp32), prefix-compose them in rank order, and then run the
chunk walk once with the true incoming state. ``delta_state_handoff`` is that composition.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

Tensor = torch.Tensor
_MASK = -1e9
_FLOOR = 1e-12


def _err(msg):
    from . import MeshError

    raise MeshError(msg)


def _int(v, name):
    if isinstance(v, bool) or not isinstance(v, int):
        _err(f"{name} must be a Python int")
    return v


def cp_split_seq(x, n: int, rank: int, *, axis: int = 1) -> Tensor:
    n, rank, axis = _int(n, "n"), _int(rank, "rank"), _int(axis, "axis")
    if n < 1:
        _err(f"n must be >= 1, got {n}")
    if rank < 0 or rank >= n:
        _err(f"rank {rank} out of range for n={n}")
    t = torch.as_tensor(x)
    a = axis + t.ndim if axis < 0 else axis
    if a < 0 or a >= t.ndim:
        _err(f"axis {axis} out of range for ndim={t.ndim}")
    dim = t.shape[a]
    if dim < n:
        _err(f"dimension {dim} is smaller than n={n}")
    if dim % n != 0:
        _err(f"dimension {dim} is not divisible by n={n}")
    chunk = dim // n
    return t if n == 1 else t.narrow(a, rank * chunk, chunk)


def cp_ring_schedule(n: int, rank: int) -> tuple:
    n, rank = _int(n, "n"), _int(rank, "rank")
    if n < 1:
        _err(f"n must be >= 1, got {n}")
    if rank < 0 or rank >= n:
        _err(f"rank {rank} out of range for n={n}")
    return tuple((rank - t) % n for t in range(n))


def online_softmax_step(state, q, k, v, *, q_offset: int, k_offset: int, causal: bool,
                        scale: float):
    """Fold one KV block into ``(m, l, acc)``. q: (B,Cq,H,D); k, v: (B,Ck,Hkv,D)."""
    m, ell, acc = state
    g = q.shape[2] // k.shape[2]
    if g > 1:
        k, v = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        qi = q_offset + torch.arange(q.shape[1], device=q.device)
        ki = k_offset + torch.arange(k.shape[1], device=q.device)
        scores = torch.where(ki[None, :] > qi[:, None], torch.full_like(scores, _MASK), scores)
    m_new = torch.maximum(m, scores.amax(dim=-1, keepdim=True))
    alpha = torch.exp(m - m_new)
    p = torch.exp(scores - m_new)
    ell = alpha * ell + p.sum(dim=-1, keepdim=True)
    acc = alpha * acc + torch.einsum("bhqk,bkhd->bhqd", p, v.float())
    return m_new, ell, acc


def ring_attention_rank(q, ks: Sequence, vs: Sequence, rank: int, *, causal: bool = True,
                        scale: float | None = None) -> Tensor:
    """Attention output of ``rank``'s query block against every KV block, folded in ring
    order. ``ks[r]``/``vs[r]`` are rank r's blocks (equal lengths)."""
    n = len(ks)
    if n < 1 or len(vs) != n:
        _err("ks and vs must be non-empty and the same length")
    if rank < 0 or rank >= n:
        _err(f"rank {rank} out of range for n={n}")
    q = torch.as_tensor(q)
    b, c, h, d = q.shape
    for name, blocks in (("k", ks), ("v", vs)):
        for t in blocks:
            if t.ndim != 4 or t.shape[0] != b or t.shape[1] != c:
                _err(f"{name} block shape {tuple(t.shape)} incompatible with q {tuple(q.shape)}")
    sc = 1.0 / math.sqrt(d) if scale is None else float(scale)
    dv = vs[0].shape[-1]
    state = (torch.full((b, h, c, 1), -math.inf, dtype=torch.float32, device=q.device),
             torch.zeros((b, h, c, 1), dtype=torch.float32, device=q.device),
             torch.zeros((b, h, c, dv), dtype=torch.float32, device=q.device))
    for owner in cp_ring_schedule(n, rank):
        state = online_softmax_step(state, q, ks[owner], vs[owner], q_offset=rank * c,
                                    k_offset=owner * c, causal=causal, scale=sc)
    _, ell, acc = state
    return (acc / torch.clamp(ell, min=_FLOOR)).permute(0, 2, 1, 3)


def ring_attention(q, k, v, n: int, *, causal: bool = True, scale: float | None = None) -> Tensor:
    """All ranks in one call: split, run every rank's fold, concatenate along the sequence."""
    if _int(n, "n") < 1:
        _err(f"n must be >= 1, got {n}")
    qs = [cp_split_seq(q, n, r) for r in range(n)]
    ks = [cp_split_seq(k, n, r) for r in range(n)]
    vs = [cp_split_seq(v, n, r) for r in range(n)]
    return torch.cat([ring_attention_rank(qs[r], ks, vs, r, causal=causal, scale=scale)
                      for r in range(n)], dim=1)


def ring_attention_distributed(q, k, v, *, group=None, causal: bool = True,
                               scale: float | None = None) -> Tensor:
    """One rank's share over ``torch.distributed``: KV blocks travel to the next rank with
    non-blocking send/recv while the current block is folded."""
    import torch.distributed as dist

    n, rank = dist.get_world_size(group), dist.get_rank(group)
    b, c, h, d = q.shape
    sc = 1.0 / math.sqrt(d) if scale is None else float(scale)
    state = (torch.full((b, h, c, 1), -math.inf, dtype=torch.float32, device=q.device),
             torch.zeros((b, h, c, 1), dtype=torch.float32, device=q.device),
             torch.zeros((b, h, c, v.shape[-1]), dtype=torch.float32, device=q.device))
    cur_k, cur_v = k.contiguous(), v.contiguous()
    nxt = (rank + 1) % n
    prv = (rank - 1) % n
    if group is not None:
        nxt, prv = dist.get_global_rank(group, nxt), dist.get_global_rank(group, prv)
    for t, owner in enumerate(cp_ring_schedule(n, rank)):
        reqs = []
        if t + 1 < n:
            nk, nv = torch.empty_like(cur_k), torch.empty_like(cur_v)
            ops = [dist.P2POp(dist.isend, cur_k, nxt, group), dist.P2POp(dist.isend, cur_v, nxt, group),
                   dist.P2POp(dist.irecv, nk, prv, group), dist.P2POp(dist.irecv, nv, prv, group)]
            reqs = dist.batch_isend_irecv(ops)
        state = online_softmax_step(state, q, cur_k, cur_v, q_offset=rank * c,
                                    k_offset=owner * c, causal=causal, scale=sc)
        for r in reqs:
            r.wait()
        if t + 1 < n:
            cur_k, cur_v = nk, nv
    _, ell, acc = state
    return (acc / torch.clamp(ell, min=_FLOOR)).permute(0, 2, 1, 3)


# ---------------------------------------------------------------------------
# delta-rule state hand-off
# ---------------------------------------------------------------------------
def compose_affine(first, second):
    """Map applying ``first`` then ``second``: (P2 P1, P2 R1 + R2)."""
    p1, r1 = first
    p2, r2 = second
    return p2 @ p1, p2 @ r1 + r2


def slice_affine_map(k, v, beta, chunk: int = 64):
    """(P, R) of one rank's slice: state leaving the slice = P @ state entering + R.
    k: (B,S,H,Dk) L2-normalised keys, v: (B,S,H,Dv), beta: (B,S,H)."""
    from ..kernels import wy_chunk_operands
    from ..ops.delta import affine_inclusive_scan, chunk_affine_maps

    b, s, h, dk = k.shape
    if s % chunk != 0:
        _err(f"slice length {s} must be a multiple of the chunk {chunk}")
    n = s // chunk

    def chunks(x):
        return x.float().reshape(b, n, chunk, h, x.shape[-1]).permute(0, 3, 1, 2, 4)

    kc, vc = chunks(k), chunks(v)
    bc = beta.float().reshape(b, n, chunk, h).permute(0, 3, 1, 2)
    w, uhat = wy_chunk_operands(kc, vc, bc)
    p, r = chunk_affine_maps(kc, w, uhat)
    pacc, racc = affine_inclusive_scan(p, r)
    return pacc[:, :, -1], racc[:, :, -1]


def delta_state_handoff(maps: Sequence, s0: Tensor | None = None) -> list:
    """Incoming state of every rank from all ranks' slice maps (exclusive prefix composition
    in rank order). ``maps[r] = (P_r, R_r)`` with shapes (B,H,Dk,Dk) and (B,H,Dk,Dv)."""
    if not maps:
        _err("maps must be non-empty")
    p0, r0 = maps[0]
    state = torch.zeros_like(r0) if s0 is None else s0.float()
    out = []
    for p, r in maps:
        out.append(state)
        state = p @ state + r
    return out


def delta_state_handoff_distributed(local_map, *, group=None, s0: Tensor | None = None) -> Tensor:
    """One rank's incoming state: all-gather the (P, R) operands (a few MB) and compose the
    prefix locally; every rank does the same tiny computation, no serial rank-to-rank wait."""
    import torch.distributed as dist

    n, rank = dist.get_world_size(group), dist.get_rank(group)
    p, r = local_map
    ps = [torch.empty_like(p) for _ in range(n)]
    rs = [torch.empty_like(r) for _ in range(n)]
    dist.all_gather(ps, p.contiguous(), group=group)
    dist.all_gather(rs, r.contiguous(), group=group)
    return delta_state_handoff(list(zip(ps, rs)), s0)[rank]


# ---------------------------------------------------------------------------
# delta-rule layer over a context-parallel group, on peer memory
# ---------------------------------------------------------------------------
class DeltaCpContext:
    """Symmetric buffers and epochs of the device-side state hand-off (``csrc/comm/cp.cu``).

    One context serves every delta-rule layer of a model with ``batch * heads`` states of
    128 x 128; a device barrier before each push keeps a rank from overwriting slots a peer
    is still composing from."""

    def __init__(self, bh: int, group=None, wait_budget_s: float = 20.0):
        from ..ops._lib import query
        from .symm import SymmetricBuffer, SymmetricGroup

        self.group = group
        self.sym = SymmetricGroup(group, wait_budget_s)
        self.world, self.rank = self.sym.world, self.sym.rank
        self.bh = int(bh)
        self.buf = SymmetricBuffer(query("pb_cp_buffer_bytes", self.bh), group)
        self.ptrs = self.buf.peer_ptrs(0)
        self.epoch = [0, 0]
        self.budget_ns = int(wait_budget_s * 1e9)

    def handoff(self, p: Tensor, r: Tensor, s0: Tensor | None = None, reverse: bool = False) -> Tensor:
        """State entering this rank (forward) or state gradient leaving it (reverse), from
        every rank's ``(P, R)``; fp32 ``(bh, 128, 128)`` in and out."""
        from ..ops._lib import call, ptr, stream_ptr

        d = 1 if reverse else 0
        p = p.reshape(self.bh, 128, 128).float().contiguous()
        r = r.reshape(self.bh, 128, 128).float().contiguous()
        s0c = None if s0 is None else s0.reshape(self.bh, 128, 128).float().contiguous()
        out = torch.empty_like(r)
        self.sym.barrier(2 + d)                 # peers have finished reading the previous maps
        self.epoch[d] += 1
        call("pb_cp_push", ptr(p), ptr(r), self.ptrs, self.rank, self.world, self.bh, d,
             self.epoch[d], stream_ptr())
        call("pb_cp_compose", self.buf.local_ptr, ptr(s0c), ptr(out), self.rank, self.world, self.bh,
             d, self.epoch[d], self.budget_ns, ptr(self.sym.status), stream_ptr())
        return out

    def check(self) -> None:
        self.sym.check()

    def close(self) -> None:
        self.buf.close()


# ---------------------------------------------------------------------------
# zig-zag split: balanced causal attention, delta-rule chain over 2 x world half-slices
# ---------------------------------------------------------------------------
def zigzag_positions(world: int, rank: int) -> tuple[int, int]:
    """Chain positions (half-slice indices) of rank ``rank``: ``rank`` and ``2 world - 1 - rank``.
    Causal attention over half-slice ``p`` costs ``p + 1/2`` units, so every rank does
    ``2 world`` units: no rank waits for the one that holds the end of the sequence."""
    return rank, 2 * world - 1 - rank


def zigzag_slice(x: Tensor, world: int, rank: int, *, axis: int = 1) -> Tensor:
    """This rank's two half-slices of ``x`` along ``axis``, concatenated (near half first)."""
    n = x.shape[axis]
    if n % (2 * world):
        _err(f"length {n} is not divisible by 2 x {world}")
    half = n // (2 * world)
    a, b = zigzag_positions(world, rank)
    return torch.cat([x.narrow(axis, a * half, half), x.narrow(axis, b * half, half)], dim=axis)


class ZigzagCpContext:
    """Peer-memory state of one context-parallel group with the zig-zag split
    (``csrc/comm/cp.cu``, chain mode): the delta-rule state chain over ``2 world`` half-slices,
    the gather of keys / values and the return of their gradients. No collective-library call
    on the layer path: peers' memory is read and written by this package's own kernels with
    plain loads and stores, every wait is bounded and latches ``sym.status``.

    ``rows`` = batch x delta heads of the model's delta-rule layers; the key / value buffers are
    sized on first use. One sequence per micro-batch (``batch == 1``) for the attention part."""

    SLOT_CHAIN = (2, 3)       # device-barrier slots: before a chain push, per direction
    SLOT_KV, SLOT_DKV = 4, 5

    def __init__(self, rows: int, group=None, wait_budget_s: float = 20.0):
        from ..ops._lib import query
        from .symm import SymmetricBuffer, SymmetricGroup

        self.group = group
        self.sym = SymmetricGroup(group, wait_budget_s)
        self.world, self.rank = self.sym.world, self.sym.rank
        self.rows = int(rows)
        self.bh = 2 * self.rows                     # local maps: two half-slices per sequence
        self.chain = SymmetricBuffer(query("pb_cp_chain_bytes", self.rows, self.world), group)
        self.chain.bytes[:256].zero_()
        self.chain_ptrs = self.chain.peer_ptrs(0)
        self.epoch = [0, 0]
        self.budget_ns = int(wait_budget_s * 1e9)
        self._kv = None
        self._parity = [0, 0]
        torch.cuda.synchronize()
        import torch.distributed as dist

        dist.barrier(group)

    # ------------------------------------------------------------- delta-rule chain
    def _chain_view(self, direction: int, which: int) -> Tensor:
        per = self.rows * 2 * self.world * 128 * 128
        off = 256 + (direction * 2 + which) * per * 4
        return self.chain.view(torch.float32, per, off)

    def handoff(self, p: Tensor, r: Tensor, s0: Tensor | None = None, reverse: bool = False) -> Tensor:
        """``p``, ``r``: fp32 ``(batch * 2 * heads, 128, 128)``, the maps of this rank's two
        half-slices per sequence (local sequence index ``(b * 2 + half) * heads + h``). Returns,
        in the same layout, the state entering each of them (forward) or the state gradient
        leaving each of them (reverse)."""
        from ..ops._lib import call, ptr, stream_ptr

        d = 1 if reverse else 0
        n = p.shape[0]
        heads_batch = n // 2
        if n != self.bh:
            _err(f"context was built for {self.bh} local maps, got {n}")
        p = p.reshape(n, 128, 128).float().contiguous()
        r = r.reshape(n, 128, 128).float().contiguous()
        self.sym.barrier(self.SLOT_CHAIN[d])        # peers have folded the previous maps
        self.epoch[d] += 1
        # batch and heads only fix the (b, half, h) -> (row, position) map; rows = batch * heads
        call("pb_cp_push_chain", ptr(p), ptr(r), self.chain_ptrs, self.rank, self.world,
             self._batch, heads_batch // self._batch, d, self.epoch[d], stream_ptr())
        call("pb_cp_wait_chain", self.chain.local_ptr, self.world, d, self.epoch[d], self.budget_ns,
             ptr(self.sym.status), stream_ptr())
        w2 = 2 * self.world
        p_all, r_all = self._chain_view(d, 0), self._chain_view(d, 1)
        s_all = torch.empty((self.rows, w2, 128, 128), dtype=torch.float32, device=p.device)
        call("pb_delta_compose", ptr(p_all), ptr(r_all), None, ptr(s_all), None, None, self.rows, w2,
             d, stream_ptr())
        a, b = zigzag_positions(self.world, self.rank)
        heads = heads_batch // self._batch
        mine = s_all[:, [a, b]].reshape(self._batch, heads, 2, 128, 128).permute(0, 2, 1, 3, 4)
        return mine.reshape(n, 128, 128).contiguous()

    _batch = 1

    def set_batch(self, batch: int) -> None:
        if self.rows % batch:
            _err("rows must be batch x heads")
        self._batch = int(batch)

    # --------------------------------------------------------- keys / values
    def _kv_buffers(self, half_elems: int, device):
        from .symm import SymmetricBuffer

        if self._kv is None or self._kv["half_elems"] != half_elems:
            full = 2 * self.world * half_elems
            stage = [SymmetricBuffer(4 * half_elems * 2, self.group) for _ in range(2)]
            grads = [SymmetricBuffer(2 * full * 2, self.group) for _ in range(2)]
            self._kv = {"half_elems": half_elems, "full": full, "stage": stage, "grads": grads}
        return self._kv

    def gather_kv(self, k: Tensor, v: Tensor):
        """k, v: this rank's ``(1, 2 L, Hkv, D)`` bf16 (two half-slices). Returns natural-order
        ``(1, 2 world L, Hkv, D)`` keys and values of the whole sequence, pulled from the peers."""
        from ..ops._lib import call, ptr, stream_ptr

        b, s2, hkv, d = k.shape
        if b != 1:
            _err("zig-zag attention takes one sequence per micro-batch")
        half = s2 // 2
        half_elems = half * hkv * d
        kv = self._kv_buffers(half_elems, k.device)
        par = self._parity[0]
        self._parity[0] ^= 1
        st = kv["stage"][par]
        stage = st.view(torch.bfloat16, 4 * half_elems)
        stage[:2 * half_elems].copy_(k.reshape(-1))
        stage[2 * half_elems:].copy_(v.reshape(-1))
        # one barrier per layer: the two staging buffers alternate, and a peer reaches the next
        # barrier only after its pull of this buffer has finished on its stream
        self.sym.barrier(self.SLOT_KV)
        kf = torch.empty((1, 2 * self.world * half, hkv, d), dtype=k.dtype, device=k.device)
        vf = torch.empty_like(kf)
        call("pb_cp_kv_gather", st.peer_ptrs(0), ptr(kf), ptr(vf), self.world, half_elems * 2, stream_ptr())
        return kf, vf

    def grad_buffers(self, half_elems: int):
        """This rank's ``[dK | dV]`` buffer of the current backward layer, as two bf16 views of
        ``full`` elements each (written by the attention backward, read by the peers)."""
        kv = self._kv
        par = self._parity[1]
        self._parity[1] ^= 1
        g = kv["grads"][par]
        full = kv["full"]
        return g, g.view(torch.bfloat16, full), g.view(torch.bfloat16, full, full * 2)

    def reduce_dkv(self, gbuf, half_elems: int, like: Tensor):
        from ..ops._lib import call, ptr, stream_ptr

        self.sym.barrier(self.SLOT_DKV)             # every rank's dK / dV are complete
        dk = torch.empty_like(like)
        dv = torch.empty_like(like)
        call("pb_cp_kv_reduce", gbuf.peer_ptrs(0), ptr(dk), ptr(dv), self.rank, self.world, half_elems,
             self._kv["full"], stream_ptr())
        return dk, dv

    def check(self) -> None:
        self.sym.check()

    def symmetric_buffers(self):
        out = [self.chain, self.sym.ctrl]
        if self._kv is not None:
            out += self._kv["stage"] + self._kv["grads"]
        return out

    def close(self) -> None:
        for b in self.symmetric_buffers()[:-1]:
            b.close()


class _ZigzagAttnFn(torch.autograd.Function):
    """Causal GQA attention of a zig-zag split sequence. Forward: gather K / V (peer pulls), then
    the offset kernel once per half-slice (queries at chain position ``p`` against keys
    ``[0, (p + 1) L)``). Backward: the two backward calls leave dK / dV of the prefixes they saw
    in this rank's symmetric buffer; every owner sums its rows over the ranks in rank order."""

    @staticmethod
    def forward(ctx, q, k, v, zz):
        from ..ops._lib import call, ptr, stream_ptr
        from ..ops.functional import status_word

        b, s2, hq, d = q.shape
        hkv = k.shape[2]
        L = s2 // 2
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        kf, vf = zz.gather_kv(k, v)
        out = torch.empty_like(q)
        lse2 = torch.empty((2, b, hq, L), dtype=torch.float32, device=q.device)
        scale = 1.0 / math.sqrt(d)
        status = ptr(status_word(q.device))
        row_q, es = hq * d, q.element_size()
        for half, pos in enumerate(zigzag_positions(zz.world, zz.rank)):
            off = half * L * row_q * es
            call("pb_attn_fwd_cp", q.data_ptr() + off, ptr(kf), ptr(vf), out.data_ptr() + off,
                 ptr(lse2[half]), None, b, L, (pos + 1) * L, pos * L, hq, hkv, row_q, hkv * d, row_q,
                 float(scale), status, stream_ptr())
        ctx.save_for_backward(q, kf, vf, out, lse2)
        ctx.zz, ctx.kshape = zz, tuple(k.shape)
        return out

    @staticmethod
    def backward(ctx, d_out):
        from ..ops._lib import call, ptr, stream_ptr
        from ..ops.functional import status_word

        q, kf, vf, out, lse2 = ctx.saved_tensors
        zz = ctx.zz
        b, s2, hq, d = q.shape
        _, _, hkv, _ = ctx.kshape
        L = s2 // 2
        half_elems = L * hkv * d
        d_out = d_out.contiguous()
        dq = torch.empty_like(q)
        delta = torch.empty_like(lse2)
        scale = 1.0 / math.sqrt(d)
        status = ptr(status_word(q.device))
        row_q, es = hq * d, q.element_size()
        gbuf, dk_full, dv_full = zz.grad_buffers(half_elems)
        near, far = zigzag_positions(zz.world, zz.rank)
        # far half first: it sees the longer prefix and writes every row the near half will add to
        tmp_k = torch.empty((near + 1) * half_elems, dtype=q.dtype, device=q.device)
        tmp_v = torch.empty_like(tmp_k)
        for half, pos, dk, dv in ((1, far, dk_full, dv_full), (0, near, tmp_k, tmp_v)):
            off = half * L * row_q * es
            call("pb_attn_bwd_cp", q.data_ptr() + off, ptr(kf), ptr(vf), out.data_ptr() + off,
                 d_out.data_ptr() + off, ptr(lse2[half]), ptr(delta[half]), dq.data_ptr() + off, ptr(dk),
                 ptr(dv), b, L, (pos + 1) * L, pos * L, hq, hkv, row_q, hkv * d, row_q, float(scale),
                 status, stream_ptr())
        dk_full[:tmp_k.numel()] += tmp_k
        dv_full[:tmp_v.numel()] += tmp_v
        like = torch.empty(ctx.kshape, dtype=q.dtype, device=q.device)
        dk, dv = zz.reduce_dkv(gbuf, half_elems, like)
        return dq, dk, dv, None


def zigzag_attention(q: Tensor, k: Tensor, v: Tensor, zz: ZigzagCpContext) -> Tensor:
    """Causal GQA attention for sequences split zig-zag over ``zz``'s ranks. q ``(B, 2 L, Hq, 128)``,
    k / v ``(B, 2 L, Hkv, 128)`` bf16: this rank's two half-slices, near one first; ``L`` a
    multiple of 256."""
    if q.shape[1] % 512:
        _err("zig-zag attention needs half-slices that are multiples of 256 tokens")
    if q.shape[0] == 1:
        return _ZigzagAttnFn.apply(q, k, v, zz)
    # the peer buffers hold one sequence: a micro-batch of several goes through one at a time
    return torch.cat([_ZigzagAttnFn.apply(q[b:b + 1], k[b:b + 1], v[b:b + 1], zz)
                      for b in range(q.shape[0])], dim=0)


def delta_rule_zigzag(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, zz: ZigzagCpContext) -> Tensor:
    """Delta rule over a zig-zag split sequence: the two half-slices of every sequence are run
    as separate batch entries whose incoming states come from the fold over the ``2 world``
    chain positions. Shapes as ``delta_rule_cp`` (local length = two half-slices)."""
    from ..ops.delta import delta_rule_fused

    b, s2, h, d = q.shape
    zz.set_batch(b)
    halves = [t.reshape(b * 2, s2 // 2, *t.shape[2:]) for t in (q, k, v, beta)]
    out, _ = delta_rule_fused(*halves, None, cp=zz)
    return out.reshape(b, s2, h, d)


def delta_rule_cp(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, cp: DeltaCpContext) -> Tensor:
    """This rank's slice of the delta-rule output for a sequence split contiguously over the
    ranks of ``cp`` (rank order = sequence order). Shapes as ``ops.delta.delta_rule_fused``;
    head dim 128, slice length a multiple of 64."""
    if q.shape[0] * q.shape[2] != cp.bh:
        _err(f"context was built for batch*heads = {cp.bh}, got {q.shape[0] * q.shape[2]}")
    from ..ops.delta import delta_rule_fused

    # two local passes: the slice's affine map (summary walk, no outputs), the hand-off of
    # (P, R) between ranks, then the segmented walk from the true incoming state; backward the
    # same with P^T (ops.delta._DeltaFusedFn)
    out, _ = delta_rule_fused(q, k, v, beta, None, cp=cp)
    return out


# ---------------------------------------------------------------------------
# softmax attention over a context-parallel group: gathered K / V + offset kernel
# ---------------------------------------------------------------------------
class _CpAttentionFn(torch.autograd.Function):
    """Each rank holds one contiguous slice of the sequence. K and V of all ranks are
    all-gathered (a few hundred MB at 131072 tokens with 4 KV heads), the tcgen05 kernel runs
    the local queries against the gathered prefix with the rank's offset, and the key / value
    gradients go back to their owners with a reduce-scatter."""

    @staticmethod
    def forward(ctx, q, k, v, group):
        import torch.distributed as dist

        from ..ops.attention import _AttnCpFn

        world, rank = dist.get_world_size(group), dist.get_rank(group)
        b, s, hkv, d = k.shape
        kg = torch.empty((world, b, s, hkv, d), dtype=k.dtype, device=k.device)
        vg = torch.empty_like(kg)
        dist.all_gather_into_tensor(kg, k.contiguous(), group=group)
        dist.all_gather_into_tensor(vg, v.contiguous(), group=group)
        kf = kg.permute(1, 0, 2, 3, 4).reshape(b, world * s, hkv, d)
        vf = vg.permute(1, 0, 2, 3, 4).reshape(b, world * s, hkv, d)
        ctx.group, ctx.world, ctx.shape = group, world, (b, s, hkv, d)
        with torch.enable_grad():
            ql, kl, vl = q.detach().requires_grad_(), kf.detach().requires_grad_(), vf.detach().requires_grad_()
            out = _AttnCpFn.apply(ql, kl, vl, rank * s, 1.0 / math.sqrt(d))
        ctx.inner = (ql, kl, vl, out)
        return out.detach()

    @staticmethod
    def backward(ctx, d_out):
        import torch.distributed as dist

        ql, kl, vl, out = ctx.inner
        dq, dkf, dvf = torch.autograd.grad(out, (ql, kl, vl), d_out)
        b, s, hkv, d = ctx.shape
        w = ctx.world
        # [B, W*S, ...] -> [W, B, S, ...] so that chunk r of the scatter is rank r's slice
        dkg = dkf.reshape(b, w, s, hkv, d).permute(1, 0, 2, 3, 4).contiguous().float()
        dvg = dvf.reshape(b, w, s, hkv, d).permute(1, 0, 2, 3, 4).contiguous().float()
        dk = torch.empty((b, s, hkv, d), dtype=torch.float32, device=d_out.device)
        dv = torch.empty_like(dk)
        dist.reduce_scatter_tensor(dk, dkg, group=ctx.group)
        dist.reduce_scatter_tensor(dv, dvg, group=ctx.group)
        ctx.inner = None
        return dq, dk.to(d_out.dtype), dv.to(d_out.dtype), None


def cp_attention(q: Tensor, k: Tensor, v: Tensor, group=None) -> Tensor:
    """Causal GQA attention for a sequence split contiguously over ``group`` (rank order =
    sequence order). q ``(B, S_loc, Hq, 128)``, k / v ``(B, S_loc, Hkv, 128)`` bf16 on the GPU,
    ``S_loc`` a multiple of 256."""
    return _CpAttentionFn.apply(q, k, v, group)
