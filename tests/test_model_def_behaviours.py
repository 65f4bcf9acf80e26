"""Behaviour list of the serving layer table (``prometheus_b200.model_def``; reference
tests/test_sglang_model_def.py and sglang-fork/sglang_fork/model_def.py:84-268): the 3 : 1
attention pattern, dense-then-MoE feed-forward layers, the core block at the end of the stack,
count validation and re-validation of hand-built tables."""
import dataclasses

import pytest

from prometheus_b200 import model, model_def as M

A, Fk = M.AttentionKind, M.FfnKind


def counts(**kw):
    base = dict(d_model=64, n_layers=8, n_dense=1, n_moe=7, n_linear_attn=6, n_mla=2, n_routed_experts=8, n_shared_experts=1,
                top_k=2, expert_hidden=32, mtp_heads=2, core_block_layers=2, recurrence_train_mean=2.0, recurrence_max=4,
                vocab_size=512, max_context=1024)
    base.update(kw)
    return base


def test_constants_and_types():
    assert M.LINEAR_TO_MLA == 3 and [k.value for k in A] == ["linear", "mla"] and [k.value for k in Fk] == ["dense", "moe"]
    assert str(A.MLA) == "mla" and issubclass(M.ModelDefError, ValueError)
    row = M.SglangLayer(0, A.LINEAR, Fk.DENSE, False)
    with pytest.raises(dataclasses.FrozenInstanceError):
        row.index = 1
    bare = M.SglangModelDef(**counts())
    assert bare.layers == () and bare.max_racks == 4


@pytest.mark.parametrize("n_layers", [1, 3, 4, 8, 12, 61])
def test_attention_pattern_is_three_linear_then_one_softmax(n_layers):
    kinds = [M.attention_kind(i, n_layers) for i in range(n_layers)]
    assert kinds[0] is A.LINEAR
    assert kinds == [A.MLA if i % 4 == 3 else A.LINEAR for i in range(n_layers)]
    for i in range(n_layers - 4):
        assert kinds[i] is kinds[i + 4]
    for bad in (-1, n_layers, n_layers + 5):
        with pytest.raises(M.ModelDefError):
            M.attention_kind(bad, n_layers)


def test_explicit_small_sequences():
    assert [M.attention_kind(i, 8).value for i in range(8)] == ["linear", "linear", "linear", "mla"] * 2
    assert [M.ffn_kind(i, 2, 5).value for i in range(5)] == ["dense", "dense", "moe", "moe", "moe"]
    assert [M.in_core_block(i, 6, 2) for i in range(6)] == [False] * 4 + [True] * 2
    with pytest.raises(M.ModelDefError):
        M.attention_kind(0, 0)


@pytest.mark.parametrize("n_dense, n_layers", [(0, 4), (1, 8), (3, 8), (8, 8)])
def test_feed_forward_layers_are_dense_first(n_dense, n_layers):
    kinds = [M.ffn_kind(i, n_dense, n_layers) for i in range(n_layers)]
    assert kinds == [Fk.DENSE] * n_dense + [Fk.MOE] * (n_layers - n_dense)
    for bad in (-1, n_layers):
        with pytest.raises(M.ModelDefError):
            M.ffn_kind(bad, n_dense, n_layers)


@pytest.mark.parametrize("n_layers, core", [(8, 1), (8, 2), (8, 8), (12, 5)])
def test_core_block_is_the_tail_of_the_stack(n_layers, core):
    flags = [M.in_core_block(i, n_layers, core) for i in range(n_layers)]
    assert flags == [False] * (n_layers - core) + [True] * core
    for bad in (-1, n_layers):
        with pytest.raises(M.ModelDefError):
            M.in_core_block(bad, n_layers, core)


def test_from_counts_fills_and_stores():
    d = M.from_counts(**counts())
    assert [r.index for r in d.layers] == list(range(8)) and len(d.layers) == d.n_layers == 8
    assert [r.attention.value for r in d.layers] == ["linear", "linear", "linear", "mla"] * 2
    assert [r.ffn.value for r in d.layers] == ["dense"] + ["moe"] * 7 and [r.in_core_block for r in d.layers] == [False] * 6 + [True] * 2
    for k, v in counts().items():
        assert getattr(d, k) == v
    assert d.max_racks == 4 and M.from_counts(**counts(max_racks=2)).max_racks == 2
    assert M.layer_table(d) == d.layers and M.mtp_head_count(d) == 2


@pytest.mark.parametrize("kw", [
    dict(n_dense=2), dict(n_moe=6), dict(n_linear_attn=5), dict(n_mla=3), dict(n_linear_attn=4, n_mla=4), dict(mtp_heads=1),
    dict(mtp_heads=0), dict(mtp_heads=3), dict(n_dense=-1, n_moe=9), dict(core_block_layers=0), dict(core_block_layers=9),
    dict(core_block_layers=-1), dict(n_layers=0, n_dense=0, n_moe=0, n_linear_attn=0, n_mla=0), dict(top_k=9), dict(top_k=0),
    dict(d_model=0), dict(vocab_size=0), dict(recurrence_train_mean=0.0), dict(max_racks=0),
    dict(n_layers=6, n_dense=1, n_moe=5, n_linear_attn=5, n_mla=1),                      # 6 layers cannot be 3 : 1
])
def test_from_counts_rejects(kw):
    with pytest.raises(M.ModelDefError):
        M.from_counts(**counts(**kw))


def test_edge_shapes():
    all_dense = M.from_counts(**counts(n_dense=8, n_moe=0))
    assert all(r.ffn is Fk.DENSE for r in all_dense.layers)
    all_moe = M.from_counts(**counts(n_dense=0, n_moe=8))
    assert all(r.ffn is Fk.MOE for r in all_moe.layers)
    whole = M.from_counts(**counts(core_block_layers=8))
    assert all(r.in_core_block for r in whole.layers)
    last = M.from_counts(**counts(core_block_layers=1))
    assert [r.in_core_block for r in last.layers] == [False] * 7 + [True]
    four = M.from_counts(**counts(n_layers=4, n_dense=1, n_moe=3, n_linear_attn=3, n_mla=1))
    assert [r.attention.value for r in four.layers] == ["linear", "linear", "linear", "mla"]


def test_layer_table_rechecks_hand_built_definitions():
    good = M.from_counts(**counts())
    rows = list(good.layers)
    assert M.layer_table(dataclasses.replace(good, layers=tuple(rows))) == tuple(rows)
    broken = [
        tuple(rows[:-1]),                                                                               # wrong length
        tuple([dataclasses.replace(rows[0], attention=A.MLA)] + rows[1:]),                              # wrong attention
        tuple(rows[:1] + [dataclasses.replace(rows[1], ffn=Fk.DENSE)] + rows[2:]),                      # wrong feed-forward kind
        tuple(rows[:7] + [dataclasses.replace(rows[7], in_core_block=False)]),                          # wrong core flag
        tuple([dataclasses.replace(rows[0], index=5)] + rows[1:]),                                      # wrong index
    ]
    for layers in broken:
        with pytest.raises(M.ModelDefError):
            M.layer_table(dataclasses.replace(good, layers=layers))
    with pytest.raises(M.ModelDefError):
        M.mtp_head_count(dataclasses.replace(good, mtp_heads=3))


@pytest.mark.parametrize("n_layers, n_dense, core", [(4, 0, 1), (8, 3, 4), (12, 1, 6), (16, 16, 16), (64, 3, 8)])
def test_declared_counts_equal_the_filled_table(n_layers, n_dense, core):
    d = M.from_counts(**counts(n_layers=n_layers, n_dense=n_dense, n_moe=n_layers - n_dense, n_linear_attn=3 * n_layers // 4,
                               n_mla=n_layers // 4, core_block_layers=core))
    assert sum(r.attention is A.LINEAR for r in d.layers) == d.n_linear_attn and sum(r.attention is A.MLA for r in d.layers) == d.n_mla
    assert sum(r.ffn is Fk.DENSE for r in d.layers) == d.n_dense and sum(r.in_core_block for r in d.layers) == core
    assert [r.index for r in d.layers] == list(range(n_layers))


def test_presets_of_the_model_package_give_valid_tables():
    for name in ("tiny", "flagship"):
        cfg = getattr(model, f"{name}_config")()
        d = M.from_model_config(cfg)
        assert len(M.layer_table(d)) == cfg.n_layers and d.n_linear_attn == 3 * d.n_mla
