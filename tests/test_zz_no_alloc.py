"""The allocation-free RMSNorm backward (for hosts that cannot call cudaMalloc where they
need the kernel) must give the same dx and dw as the regular entry point. It is called
through its exported C symbol, twice in a row, because every call reuses one fixed
scratch array inside the library. Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from prometheus_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.lib_path()))
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.pb_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, P]
    lib.pb_rmsnorm_bwd_noalloc.restype = I
    lib.pb_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    lib.pb_rmsnorm_bwd.restype = I
    lib.pb_rmsnorm_bwd_nparts.argtypes = [I, I]
    lib.pb_rmsnorm_bwd_nparts.restype = I
    lib.pb_rmsnorm_bwd_noalloc_max_d.restype = I
    return lib


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, d) in enumerate([(3000, 2048), (517, 1024)]):
        g = torch.Generator(device="cuda").manual_seed(call)
        dy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
        h = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
        dres = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
        w = 1 + 0.1 * torch.randn(d, device="cuda", generator=g)
        rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6)
        dx_a, dx_b = torch.empty_like(h), torch.empty_like(h)
        dw_a, dw_b = torch.zeros(d, device="cuda"), torch.zeros(d, device="cuda")
        scratch = torch.empty(lib.pb_rmsnorm_bwd_nparts(rows, d) * d, device="cuda")
        rc = lib.pb_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                dres.data_ptr(), dx_a.data_ptr(), dw_a.data_ptr(),
                                scratch.data_ptr(), 0, rows, d, stream)
        assert rc == 0
        rc = lib.pb_rmsnorm_bwd_noalloc(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                        dres.data_ptr(), dx_b.data_ptr(), dw_b.data_ptr(), 0, rows,
                                        d, stream)
        assert rc == 0
        torch.cuda.synchronize()
        # same kernels, same reduction order: the tolerance of the other kernel tests is ample
        scale = dx_a.float().abs().max().item() + 1e-6
        assert (dx_a.float() - dx_b.float()).abs().max().item() <= 2e-2 * scale
        assert (dw_a - dw_b).abs().max().item() <= 2e-2 * (dw_a.abs().max().item() + 1e-6)
        # and against plain PyTorch fp32
        xh = h.float() * rstd[:, None]
        gw = dy.float() * w
        ref_dx = rstd[:, None] * (gw - xh * (gw * xh).mean(-1, keepdim=True)) + dres.float()
        assert (dx_b.float() - ref_dx).abs().max().item() <= 3e-2 * ref_dx.abs().max().item()
        ref_dw = (dy.float() * xh).sum(0)
        assert (dw_b - ref_dw).abs().max().item() <= 2e-2 * ref_dw.abs().max().item()
        cos = torch.nn.functional.cosine_similarity(dw_b, ref_dw, dim=0).item()
        assert cos > 0.9999, cos


def test_noalloc_rejects_widths_beyond_its_fixed_scratch():
    lib = _lib()
    too_wide = lib.pb_rmsnorm_bwd_noalloc_max_d() + 8
    x = torch.zeros(8, too_wide, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(too_wide, device="cuda")
    r = torch.ones(8, device="cuda")
    rc = lib.pb_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), r.data_ptr(), None,
                                    x.data_ptr(), w.data_ptr(), 0, 8, too_wide,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 3
