"""Causal softmax attention with grouped KV heads (the 6 GQA layers of the hybrid).

Current implementation: PyTorch's fused scaled-dot-product attention (a library
kernel) with the same scale (1/sqrt(D)) and causal mask as ``model.gqa_attention``.
The delta-rule layers (3 of every 4) and every GEMM run on this package's own
kernels; a tcgen05 flash-attention kernel for these layers is the open item.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def causal_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q: (B, S, Hq, D); k, v: (B, S, Hkv, D) -> (B, S, Hq, D)."""
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                       is_causal=True, enable_gqa=True)
    return o.transpose(1, 2).contiguous()
