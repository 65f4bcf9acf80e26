"""Mixture-of-experts kernels and the grouped GEMMs against fp32 PyTorch (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _r(*shape, seed=0, scale=1.0, dtype=BF16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


def _close(got, ref, tol):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err:.4g} vs scale {scale:.4g}"


@pytest.mark.parametrize("T,E,k", [(7, 8, 2), (1000, 64, 6), (300, 40, 3)])
def test_route_and_placement(T, E, k):
    from prometheus_b200.ops import moe

    logits = _r(T, E, seed=1, dtype=torch.float32)
    logits[:, 3] = logits[:, 5]                      # ties break toward the lower index
    bias = _r(E, seed=2, scale=0.1, dtype=torch.float32)
    probs, ids, gates = moe.route(logits, bias, k)
    p_ref = torch.sigmoid(logits)
    ids_ref = torch.argsort(-(p_ref + bias), dim=-1, stable=True)[:, :k]
    assert torch.equal(ids.long(), ids_ref)
    top = torch.gather(p_ref, 1, ids_ref)
    torch.testing.assert_close(probs, p_ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(gates, top / top.sum(-1, keepdim=True), rtol=1e-5, atol=1e-6)
    pl = moe.place(ids, E)
    torch.cuda.synchronize()
    flat = ids.reshape(-1).long().cpu()
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(pl.totals.cpu().long(), counts)
    off = pl.expert_off.cpu().long()
    assert (off % 128 == 0).all() and off[0] == 0
    assert torch.equal(off[1:] - off[:-1], (counts + 127) // 128 * 128)
    rows = pl.row_of.cpu().long()
    assert rows.unique().numel() == rows.numel()
    for e in range(E):
        mine = rows[flat == e]
        assert torch.equal(mine, off[e] + torch.arange(mine.numel()))   # stable, dense
    mg = pl.mblk_group.cpu().long()
    used = int(off[-1]) // 128
    assert (mg[used:] == -1).all()
    for m in range(used):
        assert off[mg[m]] <= m * 128 < off[mg[m] + 1]


def test_grouped_gemms_match_per_expert_products():
    from prometheus_b200.ops import functional as ops
    from prometheus_b200.ops import moe

    T, E, k, K, N = 700, 6, 2, 256, 320
    ids = torch.randint(0, E, (T, k), device="cuda", dtype=torch.int32)
    ids[:, 1] = (ids[:, 0] + 1 + torch.randint(0, E - 1, (T,), device="cuda", dtype=torch.int32)) % E
    ids[ids == 4] = 2                                  # expert 4 gets nothing
    ids[:, 1] = torch.where(ids[:, 1] == ids[:, 0], (ids[:, 0] + 1) % E, ids[:, 1])
    ids[ids == 4] = 5
    pl = moe.place(ids.contiguous(), E)
    x = _r(T, K, seed=1)
    xp = moe.permute(x, pl)
    w = _r(E, N, K, seed=2, scale=0.1)
    y = moe.grouped_gemm(xp, w, pl)
    wt = w.transpose(1, 2).contiguous()
    y2 = moe.grouped_gemm(xp, wt, pl, b_mn=True)
    g = _r(pl.rows, N, seed=3)
    acc = torch.full((E, N, K), 0.5, dtype=torch.float32, device="cuda")
    off, tot = pl.expert_off.cpu().tolist(), pl.totals.cpu().tolist()
    for e in range(E):                                 # zero the padding rows of g
        g[off[e] + tot[e]:off[e + 1]] = 0
    moe.grouped_wgrad(g, xp, pl, acc, True)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    for e in range(E):
        seg = slice(off[e], off[e] + tot[e])
        ref = xp[seg].float() @ w[e].float().t()
        if tot[e]:
            _close(y[seg], ref, 2e-2)
            _close(y2[seg], ref, 2e-2)
        assert (xp[off[e] + tot[e]:off[e + 1]] == 0).all()
        _close(acc[e], 0.5 + g[seg].float().t() @ xp[seg].float(), 2e-2)
    assert tot[4] == 0


@pytest.mark.parametrize("n_shared", [0, 2])
def test_moe_ffn_matches_fp32_reference(n_shared):
    from prometheus_b200.ops import functional as ops
    from prometheus_b200.ops import moe

    T, d, E, h, k = 500, 256, 8, 192, 2
    x = _r(T, d, seed=1).requires_grad_(True)
    rw = _r(E, d, seed=2, scale=0.2).requires_grad_(True)
    bias = _r(E, seed=3, scale=0.05, dtype=torch.float32)
    wgu = _r(E + n_shared, 2 * h, d, seed=4, scale=0.08).requires_grad_(True)
    wd = _r(E + n_shared, d, h, seed=5, scale=0.08).requires_grad_(True)
    go = _r(T, d, seed=6)
    out, probs, ids = moe.moe_ffn(x, rw, bias, wgu, wd, k, n_shared=n_shared)
    zw = 0.3
    ((out.float() * go.float()).sum() + zw * torch.logsumexp(probs, -1).square().mean()).backward()
    torch.cuda.synchronize()
    ops.check_status("cuda")
    leaves = [t.detach().float().requires_grad_(True) for t in (x, rw, wgu, wd)]
    o_ref, p_ref, i_ref = moe.moe_ffn_ref(leaves[0], leaves[1], bias, leaves[2], leaves[3], k,
                                          n_shared=n_shared)
    ((o_ref * go.float()).sum() + zw * torch.logsumexp(p_ref, -1).square().mean()).backward()
    assert (ids == i_ref).float().mean().item() > 0.995   # bf16 logits may flip near-ties
    _close(out, o_ref, 3e-2)
    _close(probs, p_ref, 1e-2)
    for got, ref in zip((x, rw, wgu, wd), leaves):
        _close(got.grad, ref.grad, 6e-2)
