"""ctypes binding of ``libpb200_kernels.so`` (the hand-written sm_100a kernels).

Every exported function takes raw device pointers, sizes and a CUDA stream
handle and returns 0 on success (a CUDA error code or a small positive library
code otherwise). ``call(name, *args)`` raises on a non-zero return, so a
missing or failing kernel is never silently replaced by a PyTorch fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from pathlib import Path

import torch

import os

# PB200_DEBUG_BOUNDS=1 loads the -DPB_DEBUG_BOUNDS build (python -m prometheus_b200._build
# --debug-bounds): data-dependent indices are checked and a violation is recorded, not executed
_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / (
    "libpb200_kernels_dbg.so" if os.environ.get("PB200_DEBUG_BOUNDS", "0") == "1" else "libpb200_kernels.so")
_lib = None

P, I, L, F = c_void_p, c_int, c_long, c_float

_SIGS = {
    "pb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "pb_rmsnorm_fwd_fp8": [P, P, P, P, P, P, P, P, I, I, F, P],
    "pb_rmsnorm_bwd_nparts": [I, I],
    "pb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, P],
    "pb_rope": [P, P, L, I, I, I, I, F, I, P],
    "pb_swiglu_fwd": [P, P, L, I, P],
    "pb_swiglu_bwd": [P, P, P, L, I, P],
    "pb_l2norm_fwd": [P, P, L, I, F, P],
    "pb_l2norm_bwd": [P, P, P, L, I, P],
    "pb_softcap_ce": [P, P, P, P, P, L, I, F, I, P],
    "pb_sigmoid": [P, P, L, P],
    "pb_sumsq_nparts": [L],
    "pb_sumsq_f32": [P, L, P, P, I, P],
    "pb_sumsq_bf16": [P, L, P, P, I, P],
    "pb_adamw": [P, P, P, P, P, L, F, F, F, F, F, I, P, F, F, P],
    "pb_muon_prepare": [P, P, P, L, F, P, F, F, P, P],
    "pb_muon_prepare_batched": [P, P, P, L, I, F, P, F, F, P, P],
    "pb_muon_apply": [P, P, P, L, F, F, F, P],
    "pb_qk_clip_rescale": [P, P, I, I, I, I, I, I, L, P, F, P],
    "pb_checksum_u32": [P, L, P, P],
    "pb_cast_f32_bf16": [P, P, L, F, P],
    "pb_axpy_bf16_f32": [P, P, L, F, P],
    "pb_transpose_bf16": [P, P, I, I, I, P],
    "pb_wait_flag_probe": [P, I, L, P, P],
    "pb_set_flag": [P, I, P],
    "pb_delta_scan_fwd": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, P, P],
    "pb_delta_scan_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, I, P, P],
    "pb_delta_scan_fwd_seg": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P],
    "pb_delta_scan_bwd_seg": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P],
    "pb_delta_scan_summary_fwd": [P, P, P, P, P, I, I, I, I, I, P, P],
    "pb_delta_scan_summary_bwd": [P, P, P, P, P, P, I, I, I, I, I, P, P],
    "pb_delta_compose": [P, P, P, P, P, P, I, I, I, P],
    "pb_latent_gather": [P, P, I, I, I, I, I, P],
    "pb_latent_scatter": [P, P, I, I, I, I, I, P],
    "pb_latent_norm_scatter": [P, P, P, P, P, I, I, I, I, I, F, P],
    "pb_silu_fwd": [P, P, L, P],
    "pb_silu_bwd": [P, P, P, L, P],
    "pb_gemm_bf16_ag": [P, P, P, I, I, I, L, L, L, I, I, P, I, L, P, P],
    "pb_cp_buffer_bytes": [I],
    "pb_cp_push": [P, P, P, I, I, I, I, I, P],
    "pb_cp_compose": [P, P, P, I, I, I, I, I, L, P, P],
    "pb_cp_chain_bytes": [I, I],
    "pb_cp_push_chain": [P, P, P, I, I, I, I, I, I, P],
    "pb_cp_wait_chain": [P, I, I, I, L, P, P],
    "pb_cp_kv_gather": [P, P, P, I, L, P],
    "pb_cp_kv_reduce": [P, P, P, I, I, L, L, P],
    "pb_attn_fwd": [P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, P],
    "pb_attn_fwd_cp": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P, P],
    "pb_attn_bwd_cp": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P, P],
    "pb_attn_bwd": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, P],
    "pb_delta_prep_fwd": [P, P, P, P, I, P, P, P, P, P, I, I, I, I, P, I, P],
    "pb_delta_prep_bwd": [P, P, P, P, I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P, I, P],
    "pb_gemm_bf16_grouped": [P, P, P, I, I, I, I, L, L, L, L, I, P, P, I, P],
    "pb_gemm_bf16_grouped_wgrad": [P, P, P, P, I, I, I, I, L, L, L, L, I, I, F, P, P, P, I, P],
    "pb_moe_route": [P, P, I, I, I, P, P, P, P],
    "pb_moe_route_bwd": [P, P, P, P, I, I, I, P, P],
    "pb_moe_sort_nblocks": [I, I],
    "pb_moe_sort": [P, I, I, I, P, P, P, P, P, P, I, P],
    "pb_moe_permute": [P, P, P, I, I, I, L, P, P, P, I, P],
    "pb_moe_combine": [P, P, P, P, I, I, I, P, L, P],
    "pb_debug_bounds_enabled": [],
    "pb_moe_zero_pad": [P, I, P, P, I, P],
    "pb_moe_combine_bwd": [P, P, P, I, I, I, P, P],
    "pb_fp8_quant_rows": [P, L, I, I, P, P, P],
    "pb_fp8_quant_blocks": [P, L, I, I, P, P, P],
    "pb_fp8_fakequant_blocks": [P, L, I, I, P, P],
    "pb_fp8_dequant_rows": [P, P, L, I, I, P, P, P],
    "pb_fp8_quant_rows_dyn": [P, L, I, I, P, P, P, P],
    "pb_swiglu_quant": [P, P, I, I, P, P, P, P],
    "pb_swiglu_fwd_dyn": [P, P, L, I, P, P],
    "pb_swiglu_bwd_dyn": [P, P, P, L, I, P, P],
    "pb_copy_rows_dyn": [P, P, L, L, P, P],
    "pb_gemm_fp8_blockscaled": [P, P, P, P, P, I, I, I, I, L, P, P, I, P],
    "pb_gemm_fp8_grouped_arrive": [P, P, P, P, P, I, I, I, I, L, P, P, P, L, P, P],
    "pb_gemm_fp8_probe": [P, P, P, P, P, I, I, I, L, I, P, P],       # debug build only
    "pb_gemm_set_variant": [I],
    "pb_gemm_bf16": [P, P, P, P, I, I, I, I, L, L, L, L, L, L, L, L, I, I, I, I, F, F, P, I, P],
}


class KernelLibraryMissing(RuntimeError):
    """The compiled kernel library is absent: run ``python -m prometheus_b200._build``."""


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def register(name: str, argtypes: list) -> None:
    """Declare the signature of another exported symbol (used by sibling op modules)."""
    _SIGS[name] = argtypes
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def load():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelLibraryMissing(f"{_LIB_PATH} not built")
        _lib = ctypes.CDLL(str(_LIB_PATH))
        for name, argtypes in _SIGS.items():
            if hasattr(_lib, name):
                fn = getattr(_lib, name)
                fn.argtypes = argtypes
                fn.restype = c_int
    return _lib


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    """Device pointer of a tensor (None passes a null pointer)."""
    if t is None:
        return None
    return t.data_ptr()


# kernels launched by one call of each entry point (for launch accounting)
_LAUNCHES = {"pb_rmsnorm_bwd": 2, "pb_sumsq_f32": 2, "pb_sumsq_bf16": 2, "pb_muon_prepare": 3,
             "pb_muon_prepare_batched": 3}
launch_count = 0


def call(name: str, *args) -> None:
    global launch_count
    fn = getattr(load(), name)
    rc = fn(*args)
    launch_count += _LAUNCHES.get(name, 1)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


def debug_bounds_read() -> dict | None:
    """The first bounds violation recorded since the last call (debug-bounds build only):
    ``{"kernel", "hits", "index", "limit"}``, or None when there was none. Synchronises."""
    lib = load()
    if not lib.pb_debug_bounds_enabled():
        raise RuntimeError("the loaded kernel library was built without PB_DEBUG_BOUNDS")
    first = None
    for tu in ("elementwise", "moe", "ep"):            # one record per source file that checks
        fn = getattr(lib, f"pb_debug_bounds_read_{tu}")
        fn.argtypes, fn.restype = [c_void_p], c_int
        buf = (ctypes.c_longlong * 4)()
        rc = fn(ctypes.cast(buf, c_void_p))
        if rc != 0:
            raise RuntimeError(f"pb_debug_bounds_read_{tu} failed with code {rc}")
        if buf[1] and first is None:
            first = {"file": tu, "kernel": int(buf[0]), "hits": int(buf[1]), "index": int(buf[2]),
                     "limit": int(buf[3])}
    return first


def query(name: str, *args) -> int:
    """Call a host-only helper that returns a value instead of a status."""
    return getattr(load(), name)(*args)
