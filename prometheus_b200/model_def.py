"""Standalone layer table for the serving engine (no tensors): which attention and FFN
kind every layer uses and whether it belongs to the recurrent core block, with count
validation. API parity with the reference ``sglang-fork/sglang_fork/model_def.py:84-268``
(3 linear : 1 softmax pattern, first ``n_dense`` layers dense, core block = last
``core_block_layers`` layers, exactly two MTP heads); ``from_model_config`` builds it from
a ``model.ModelConfig``.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from enum import Enum


class AttentionKind(str, Enum):
    LINEAR = "linear"
    MLA = "mla"

    def __str__(self) -> str:
        return self.value


class FfnKind(str, Enum):
    DENSE = "dense"
    MOE = "moe"

    def __str__(self) -> str:
        return self.value


class ModelDefError(ValueError):
    """Counts or the layer table are inconsistent."""


LINEAR_TO_MLA = 3
_PERIOD = LINEAR_TO_MLA + 1
_MTP_HEADS = 2


@dataclass(frozen=True)
class SglangLayer:
    index: int
    attention: AttentionKind
    ffn: FfnKind
    in_core_block: bool


@dataclass(frozen=True)
class SglangModelDef:
    d_model: int
    n_layers: int
    n_dense: int
    n_moe: int
    n_linear_attn: int
    n_mla: int
    n_routed_experts: int
    n_shared_experts: int
    top_k: int
    expert_hidden: int
    mtp_heads: int
    core_block_layers: int
    recurrence_train_mean: float
    recurrence_max: int
    vocab_size: int
    max_context: int
    max_racks: int = 4
    layers: tuple = ()


def _need(ok: bool, msg: str) -> None:
    if not ok:
        raise ModelDefError(msg)


def _check_index(i: int, n: int) -> None:
    _need(0 <= i < n, f"layer_index {i} outside [0, {n})")


def attention_kind(layer_index: int, n_layers: int) -> AttentionKind:
    _check_index(layer_index, n_layers)
    return AttentionKind.MLA if layer_index % _PERIOD == LINEAR_TO_MLA else AttentionKind.LINEAR


def ffn_kind(layer_index: int, n_dense: int, n_layers: int) -> FfnKind:
    _check_index(layer_index, n_layers)
    return FfnKind.DENSE if layer_index < n_dense else FfnKind.MOE


def in_core_block(layer_index: int, n_layers: int, core_block_layers: int) -> bool:
    _check_index(layer_index, n_layers)
    return layer_index >= n_layers - core_block_layers


def _row(i: int, n_layers: int, n_dense: int, core: int) -> SglangLayer:
    return SglangLayer(i, attention_kind(i, n_layers), ffn_kind(i, n_dense, n_layers),
                       in_core_block(i, n_layers, core))


def from_counts(d_model: int, n_layers: int, n_dense: int, n_moe: int, n_linear_attn: int,
                n_mla: int, n_routed_experts: int, n_shared_experts: int, top_k: int,
                expert_hidden: int, mtp_heads: int, core_block_layers: int,
                recurrence_train_mean: float, recurrence_max: int, vocab_size: int,
                max_context: int, max_racks: int = 4) -> SglangModelDef:
    _need(n_layers >= 1, f"n_layers must be >= 1, got {n_layers}")
    _need(n_dense >= 0 and n_moe >= 0, "n_dense and n_moe must be >= 0")
    _need(n_dense + n_moe == n_layers, f"n_dense + n_moe ({n_dense} + {n_moe}) != n_layers ({n_layers})")
    _need(n_linear_attn >= 0 and n_mla >= 0, "n_linear_attn and n_mla must be >= 0")
    _need(n_linear_attn + n_mla == n_layers,
          f"n_linear_attn + n_mla ({n_linear_attn} + {n_mla}) != n_layers ({n_layers})")
    _need(n_linear_attn == LINEAR_TO_MLA * n_mla,
          f"attention is not {LINEAR_TO_MLA}:1 (n_linear_attn={n_linear_attn}, n_mla={n_mla})")
    _need(mtp_heads == _MTP_HEADS, f"mtp_heads must be {_MTP_HEADS}, got {mtp_heads}")
    _need(1 <= core_block_layers <= n_layers, f"core_block_layers {core_block_layers} outside [1, {n_layers}]")
    for name, v, lo in (("d_model", d_model, 1), ("n_routed_experts", n_routed_experts, 1),
                        ("n_shared_experts", n_shared_experts, 0), ("top_k", top_k, 1),
                        ("expert_hidden", expert_hidden, 1), ("recurrence_max", recurrence_max, 1),
                        ("vocab_size", vocab_size, 1), ("max_context", max_context, 1),
                        ("max_racks", max_racks, 1)):
        _need(v >= lo, f"{name} must be >= {lo}, got {v}")
    _need(top_k <= n_routed_experts, f"top_k {top_k} > n_routed_experts {n_routed_experts}")
    _need(recurrence_train_mean > 0, f"recurrence_train_mean must be > 0, got {recurrence_train_mean}")
    rows = tuple(_row(i, n_layers, n_dense, core_block_layers) for i in range(n_layers))
    tally = {
        "linear": sum(r.attention is AttentionKind.LINEAR for r in rows),
        "mla": sum(r.attention is AttentionKind.MLA for r in rows),
        "dense": sum(r.ffn is FfnKind.DENSE for r in rows),
        "moe": sum(r.ffn is FfnKind.MOE for r in rows),
        "core": sum(r.in_core_block for r in rows),
    }
    for key, want in (("linear", n_linear_attn), ("mla", n_mla), ("dense", n_dense), ("moe", n_moe),
                      ("core", core_block_layers)):
        _need(tally[key] == want, f"filled {key} {tally[key]} != {want}")
    return SglangModelDef(d_model, n_layers, n_dense, n_moe, n_linear_attn, n_mla, n_routed_experts,
                          n_shared_experts, top_k, expert_hidden, mtp_heads, core_block_layers,
                          recurrence_train_mean, recurrence_max, vocab_size, max_context, max_racks,
                          rows)


def from_model_config(config) -> SglangModelDef:
    """Layer table of a ``model.ModelConfig`` (reference fields only)."""
    names = [f.name for f in fields(SglangModelDef) if f.name != "layers"]
    return from_counts(**{n: getattr(config, n) for n in names})


def mtp_head_count(defn: SglangModelDef) -> int:
    _need(defn.mtp_heads == _MTP_HEADS, f"mtp_heads must be {_MTP_HEADS}, got {defn.mtp_heads}")
    return defn.mtp_heads


def layer_table(defn: SglangModelDef) -> tuple:
    """The rows, re-checked against the rules (a hand-built definition may be wrong)."""
    _need(len(defn.layers) == defn.n_layers, f"len(layers) {len(defn.layers)} != n_layers {defn.n_layers}")
    for i, row in enumerate(defn.layers):
        want = _row(i, defn.n_layers, defn.n_dense, defn.core_block_layers)
        _need(row.index == i, f"layers[{i}].index is {row.index}")
        _need(row.attention == want.attention, f"layers[{i}].attention {row.attention} != {want.attention}")
        _need(row.ffn == want.ffn, f"layers[{i}].ffn {row.ffn} != {want.ffn}")
        _need(row.in_core_block == want.in_core_block,
              f"layers[{i}].in_core_block {row.in_core_block} != {want.in_core_block}")
    return defn.layers
