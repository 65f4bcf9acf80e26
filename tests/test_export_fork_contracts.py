"""Contracts registry, weight export codecs and layout, serving-side fork rules, model_def."""
import json

import numpy as np
import pytest
import torch

from prometheus_b200 import contracts, export, fork, model, model_def


def test_contract_goldens_validate_and_bad_payloads_fail():
    ids = [s.value for s in contracts.SchemaId]
    assert len(ids) == 16 and "prometheus.checkpoint" in ids
    for sid in ids:
        gold = contracts.load_golden(sid, 1)
        contracts.validate(gold)
        assert contracts.migrate(gold, 1) == gold and contracts.current_version(sid) == 1
    bad = contracts.load_golden("prometheus.loader_state", 1)
    bad["epoch"] = -1
    with pytest.raises(contracts.ValidationError):
        contracts.validate(bad)
    with pytest.raises(contracts.UnknownSchemaError):
        contracts.validate({"schema_id": "prometheus.nope", "schema_version": 1})
    with pytest.raises(contracts.MigrationError):
        contracts.migrate(contracts.load_golden("prometheus.packing", 1), 2)
    with pytest.raises(contracts.ValidationError):
        contracts.validate({"schema_version": 1})


def test_native_manifest_and_loader_json_match_schemas():
    from prometheus_b200 import native

    st = native.loader.LoaderState()
    st.data_mix_hash = "a" * 64
    contracts.validate(json.loads(st.to_json()))
    contracts.validate(json.loads(native.loader.Packing("p", 16).to_json()))


@pytest.mark.parametrize("dtype,tol", [("bf16", 0.0), ("fp8", 0.02), ("nvfp4", 0.3)])
def test_export_roundtrip(tmp_path, dtype, tol):
    cfg = model.tiny_config()
    params = model.init_params(cfg, 0)
    small = {"embed": params["embed"], "layers": [{"W_q": params["layers"][0]["W_q"],
                                                   "norm": params["layers"][0]["pre_attn_norm"]}]}
    ex = export.export_weights(small, export_id="e1", source_checkpoint_id="c1", tokenizer_id="tok",
                               dtype=dtype, created_at="2026-01-01T00:00:00Z", out_dir=str(tmp_path))
    assert [s.name for s in ex.shards] == ["embed", "layers.0.W_q", "layers.0.norm"]
    err = export.parity_max_abs_err(small, ex, str(tmp_path))
    scale = max(float(v.abs().max()) for v in (small["embed"], small["layers"][0]["W_q"]))
    assert err <= tol * max(scale, 1.0) + 1e-12
    side = json.loads((tmp_path / "shards.json").read_text())
    assert side["format"] == "prometheus.c1.npy-shards.v1" and len(side["shards"]) == 3
    payload = export.to_contract(ex)
    contracts.validate(payload)
    assert payload["shards"][0]["content_hash"] == \
        export._hash(np.load(tmp_path / "embed.npy"))


def test_export_codecs_and_errors(tmp_path):
    q, s = export.quantize(np.array([448.0, -448.0, 0.0], dtype=np.float32), "fp8")
    assert q.tolist() == [255, 1, 128] and float(s) == 1.0
    q4, s4 = export.quantize(np.arange(-8, 8, dtype=np.float32), "nvfp4")
    assert q4.shape == (8,) and s4.shape == (1,)
    back = export.dequantize(q4, s4, "nvfp4")
    assert back.shape == (16,) and abs(back[0] + 8.0) < 1e-6
    with pytest.raises(export.ExportError):
        export.quantize(np.array([np.inf]), "fp8")
    with pytest.raises(export.ExportError):
        export.flatten_params({"a": "str"})
    with pytest.raises(export.ExportError):
        export.export_weights({"a": np.ones(2)}, export_id="", source_checkpoint_id="c",
                              tokenizer_id="t", dtype="bf16", created_at="x", out_dir=str(tmp_path))
    hashes = export.export_fp8_e4m3({"w": torch.randn(130, 70), "b": torch.ones(4)}, str(tmp_path / "e4"))
    assert set(hashes) == {"w", "b"} and np.load(tmp_path / "e4" / "w.scale.npy").shape == (2, 1)


def test_fork_rules():
    assert fork.bucket_recurrence(3, 100).r == 4 and fork.bucket_recurrence(9, 8).r == 8
    assert fork.bucket_recurrence(40, 100).r == 16
    with pytest.raises(fork.ForkError):
        fork.bucket_recurrence(0, 1)
    assert fork.validate_latent_chunk(4).mode is fork.DecodeMode.LATENT
    with pytest.raises(fork.ForkError):
        fork.validate_latent_chunk(3)
    assert fork.decode_mode(True, False) is fork.DecodeMode.LATENT
    assert fork.decode_mode(True, True) is fork.DecodeMode.VERBAL
    assert fork.next_kv_tier(fork.KvTier.HBM) is fork.KvTier.GRACE
    assert fork.next_kv_tier(fork.KvTier.DISTRIBUTED) is None
    assert fork.swap_waiting_session(False) is fork.KvTier.GRACE
    assert fork.capture_routing(0, 1, (3, 5), 2).expert_ids == (3, 5)
    with pytest.raises(fork.ForkError):
        fork.capture_routing(0, 1, (3, 3), 2)
    assert fork.schedule_prefix_group("p", ("a", "b"), 3).depth == 3
    with pytest.raises(fork.ForkError):
        fork.schedule_prefix_group("p", ("p",), 1)
    with pytest.raises(fork.ForkError):
        fork.register_ttt("", "l")


def test_model_def_table():
    d = model_def.from_model_config(model.tiny_config())
    rows = model_def.layer_table(d)
    assert [r.attention.value for r in rows[:4]] == ["linear", "linear", "linear", "mla"]
    assert rows[0].ffn is model_def.FfnKind.DENSE and rows[1].ffn is model_def.FfnKind.MOE
    assert [r.in_core_block for r in rows] == [False] * 6 + [True] * 2
    assert model_def.mtp_head_count(d) == 2
    with pytest.raises(model_def.ModelDefError):
        model_def.from_counts(8, 8, 1, 7, 5, 3, 8, 2, 2, 16, 2, 2, 3.0, 16, 256, 128)
    with pytest.raises(model_def.ModelDefError):
        model_def.attention_kind(9, 8)
