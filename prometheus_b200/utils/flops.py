"""Model FLOPs of one training step, for the MFU figure the benchmarks and the run loop report.

Counted per token, multiply-add = 2 FLOPs, backward = 2 x forward for every product:

* every weight matrix a token passes through: ``6 * in * out`` (the unembedding included, the
  embedding lookup not); a MoE layer counts its router, ``top_k`` routed and the shared experts;
* delta-rule layer, per head of dimension D with chunk C (the chunked WY form the kernels run):
  state read ``q S``, state correction ``w S`` and state update ``k^T u``, ``2 D^2`` each, plus the
  chunk-local products (``K K^T``, ``Q K^T``, ``T K``, ``T V``, ``M U``) of ``2 C D`` each per token,
  averaged over the causal triangle where they are triangular: ``6 D^2 + 8 C D`` forward;
* causal softmax layer with H query heads: ``Q K^T`` and ``P V`` over half the square,
  ``2 S D H`` forward per token, and 2.5 x that backward (five products against two);
* Newton-Schulz per Muon matrix (m <= n): ``steps * (4 m^2 n + 2 m^3)``, once per step.

MFU = model FLOPs per second / the measured dense bf16 throughput of the GPU (the cuBLAS burst
figure of ``MEASURED_PEAKS.json`` when that file is present, else 1.59 PFLOP/s).
Reference: the metric is named (tokens/s, MFU, exposed communication) but never computed there.
"""
from __future__ import annotations

import json
from pathlib import Path

from .. import model as M

FALLBACK_BF16_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0


def measured_peaks() -> dict:
    """``{"bf16_tflops", "bf16_tflops_sustained", "hbm_gbs", "source"}`` from the measurement file
    at the repository root, or the fallback figures."""
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        d = json.loads(path.read_text())
        return {"bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0,
                "hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


def matmul_params_per_token(cfg: M.ModelConfig) -> int:
    """Weight-matrix elements one token multiplies against in a forward pass (active parameters
    without the embedding table)."""
    nh, dh, nkv = M.head_geometry(cfg)
    d = cfg.d_model
    total = cfg.vocab_size * d * (1 + cfg.mtp_heads) + cfg.mtp_heads * d * d
    for i in range(cfg.n_layers):
        kind = M.attention_kind(i, cfg)
        if kind is M.AttentionKind.LINEAR:
            total += 3 * nh * dh * d + nh * dh * d + (nh * d if cfg.delta_beta == "sigmoid" else 0)
        elif kind is M.AttentionKind.GQA:
            total += nh * dh * d + 2 * nkv * dh * d + nh * dh * d
        else:
            dr = max(2, (dh // 2) // 2 * 2)
            total += nh * (dh + dr) * d + dh * d + nh * dh * dh + dr * d + nh * dh * d
        if M.ffn_kind(i, cfg) is M.FfnKind.DENSE:
            hid = cfg.dense_hidden if cfg.dense_hidden is not None else cfg.expert_hidden
            total += 3 * d * hid
        else:
            total += cfg.n_routed_experts * d
            total += 3 * d * cfg.expert_hidden * (cfg.top_k + cfg.n_shared_experts)
    return int(total)


def flops_per_token(cfg: M.ModelConfig, seq_len: int, recurrence: int = 1) -> float:
    """Forward + backward model FLOPs per token at sequence length ``seq_len`` (optimizer work
    is separate: :func:`newton_schulz_flops`). ``recurrence`` > 1 repeats the core block."""
    nh, dh, _ = M.head_geometry(cfg)
    prelude, core, coda = M._recurrent_split(cfg)
    repeat = [1] * cfg.n_layers
    for i in range(prelude, prelude + core):
        repeat[i] = int(recurrence)
    total = 6.0 * cfg.vocab_size * cfg.d_model * (1 + cfg.mtp_heads)
    d = cfg.d_model
    nkv = M.head_geometry(cfg)[2]
    for i in range(cfg.n_layers):
        kind = M.attention_kind(i, cfg)
        mat = 0
        extra = 0.0
        if kind is M.AttentionKind.LINEAR:
            mat += 4 * nh * dh * d + (nh * d if cfg.delta_beta == "sigmoid" else 0)
            extra = 3.0 * nh * (6.0 * dh * dh + 8.0 * cfg.chunk * dh)
        elif kind is M.AttentionKind.GQA:
            mat += 2 * nh * dh * d + 2 * nkv * dh * d
            extra = 3.5 * 2.0 * seq_len * dh * nh
        else:
            dr = max(2, (dh // 2) // 2 * 2)
            mat += nh * (dh + dr) * d + dh * d + nh * dh * dh + dr * d + nh * dh * d
            extra = 3.5 * 2.0 * seq_len * (dh + dr / 2.0) * nh
        if M.ffn_kind(i, cfg) is M.FfnKind.DENSE:
            hid = cfg.dense_hidden if cfg.dense_hidden is not None else cfg.expert_hidden
            mat += 3 * d * hid
        else:
            mat += cfg.n_routed_experts * d + 3 * d * cfg.expert_hidden * (cfg.top_k + cfg.n_shared_experts)
        total += repeat[i] * (6.0 * mat + extra)
    return float(total)


def newton_schulz_flops(unit_shapes, steps: int) -> float:
    """FLOPs of the quintic iteration over ``[(rows, cols), ...]`` Muon matrices."""
    total = 0.0
    for rows, cols in unit_shapes:
        m, n = (rows, cols) if rows <= cols else (cols, rows)
        total += steps * (4.0 * m * m * n + 2.0 * m * m * m)
    return total


def mfu(tokens_per_s: float, cfg: M.ModelConfig, seq_len: int, n_gpus: int, *, recurrence: int = 1,
        sweeps: int = 1, peak_tflops: float | None = None) -> float:
    """Fraction of ``n_gpus`` x the bf16 peak that the model FLOPs of this token rate amount to
    (``sweeps``: forward passes per token of the latent Jacobi solve, all with a backward)."""
    peak = (peak_tflops if peak_tflops is not None else measured_peaks()["bf16_tflops"]) * 1e12
    return tokens_per_s * flops_per_token(cfg, seq_len, recurrence) * sweeps / (peak * max(n_gpus, 1))
