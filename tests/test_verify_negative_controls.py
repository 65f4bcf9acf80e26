"""Negative controls of the verification stages (``prometheus_b200.verify``; reference
tests/test_v7_rl.py, test_v8_serving.py, test_v9_lab.py, test_v10_soak.py): each gate of a
stage must be able to fail. With the policy update skipped the reward does not rise, without
an injected drift the parity monitor does not halt, a write outside the grader's files is not
flagged, perturbed served weights fail the log-prob check, an idea without an effect is not
found, and a dropped task or a doubled output shows in the soak's counters."""
import json
import math

import pytest

from prometheus_b200 import native, verify as V


def test_v7_gates_and_their_controls():
    ok = V.run_v7()
    assert {k: ok[k] for k in ("reward_rises", "logprob_drift_halted", "planted_write_flagged")} == {
        "reward_rises": True, "logprob_drift_halted": True, "planted_write_flagged": True}
    json.dumps(ok)
    assert ok["mean_reward_last10"] > ok["mean_reward_first10"] + 0.2
    frozen_policy = V.run_v7(update=False)
    assert frozen_policy["reward_rises"] is False and abs(frozen_policy["mean_reward_last10"] - 0.25) < 0.2     # one arm of four pays
    assert V.run_v7(inject_drift=False)["logprob_drift_halted"] is False
    assert V.run_v7(plant_write="agent")["planted_write_flagged"] is False
    assert V.run_v7(plant_write=None)["planted_write_flagged"] is False
    assert V.V7_INJECTED_DRIFT > V.V7_PARITY_THRESHOLD > 0
    for bad in (0, -1, True, 1.5):
        with pytest.raises(V.VerifyError):
            V.run_v7(gpus=bad)
    with pytest.raises(V.VerifyError):
        V.run_v7(plant_write="somewhere")
    assert issubclass(V.VerifyError, Exception) and not issubclass(V.VerifyError, NotImplementedError)


def test_v8_fails_on_perturbed_served_weights():
    good, bad = V.run_v8(), V.run_v8(perturb=0.01)
    assert good["logprob_within_threshold"] is True and good["export_max_abs_err"] == 0.0 and good["tiered_restore_matches"] is True
    assert bad["logprob_within_threshold"] is False
    assert good["tiers"][0] == "grace" and good["tiers"][1] == "nvme"                    # a waiting session steps down one tier at a time


def test_v9_needs_a_real_effect():
    good, flat = V.run_v9(), V.run_v9(planted_effect=0.0)
    assert all(good[k] for k in ("planted_positive_found", "planted_positive_replicated", "planted_negative_recorded"))
    assert not flat["planted_positive_found"] and not flat["planted_positive_replicated"]
    assert not flat["planted_negative_recorded"]                                         # two negatives on the ledger, not exactly the planted one
    weak = V.run_v9(planted_effect=0.05)                                                 # inside the noise: no claim
    assert not weak["planted_positive_replicated"]


def test_v10_counters_see_a_dropped_task_and_a_doubled_output():
    clean = V.run_v10(hours=1.0)
    assert (clean["hours"], clean["lost_tasks"], clean["duplicated_outputs"], clean["dead_tokens"]) == (1.0, 0, 0, 0) and clean["faults_applied"] > 0
    json.dumps(clean)
    assert V.run_v10(hours=1.0, drop_task=True)["lost_tasks"] == 1
    assert V.run_v10(hours=1.0, duplicate_output=True)["duplicated_outputs"] == 1
    both = V.run_v10(hours=1.0, drop_task=True, duplicate_output=True)
    assert (both["lost_tasks"], both["duplicated_outputs"]) == (1, 1)
    for bad in (0, -1.0, math.nan, math.inf, True, "72"):
        with pytest.raises(V.VerifyError):
            V.run_v10(hours=bad)
    assert V.run_v10(hours=2.0, seed=3) == V.run_v10(hours=2.0, seed=3)                  # injected time and seeds only: no wall clock


def test_exit_checks_refuse_the_control_results(tmp_path):
    for stage, result in (("v7", V.run_v7(inject_drift=False)), ("v8", V.run_v8(perturb=0.01)), ("v9", V.run_v9(planted_effect=0.0)),
                          ("v10", dict(V.run_v10(hours=72.0, drop_task=True)))):
        d = tmp_path / stage
        d.mkdir()
        V.write_result(stage, result, d)
        with pytest.raises(native.NativeError) as e:
            V.check_exit(stage, d)
        assert e.value.kind == "ExitFailed"


def test_v4_each_fault_gate_can_fail():
    good = V.run_v4()
    assert all(good[k] for k in ("resumed_bitwise_equal", "sdc_caught_flip", "spike_rollback_skipped_shard"))
    json.dumps(good)
    assert V.run_v4(corrupt_restore=True)["resumed_bitwise_equal"] is False             # one flipped bit in the restored state
    assert V.run_v4(check_hash=False)["sdc_caught_flip"] is False                        # a flip nobody hashes goes unreported
    kept = V.run_v4(skip_bad_shard=False)
    assert kept["spike_rollback_skipped_shard"] is False and kept["resumed_bitwise_equal"] is True     # the other gates are untouched
    for bad in (0, -2, True):
        with pytest.raises(V.VerifyError):
            V.run_v4(gpus=bad)


def test_v6_each_latent_gate_can_fail():
    good = V.run_v6()
    assert all(good[k] for k in ("curriculum_no_collapse", "accuracy_rises_with_latent_budget", "thoughts_decode"))
    assert good["sweep_errors"] == sorted(good["sweep_errors"], reverse=True) and good["sweep_errors"][-1] < good["sweep_errors"][0]
    frozen = V.run_v6(freeze_budget=True)
    assert frozen["accuracy_rises_with_latent_budget"] is False and len(set(frozen["sweep_errors"])) == 1
    assert V.run_v6(pin_halt=True)["curriculum_no_collapse"] is False
    assert V.run_v6(scramble_decode=True)["thoughts_decode"] is False
    assert V.run_v6(gpus=1)["gpus"] == 1
    for bad in (0, -1, True):
        with pytest.raises(V.VerifyError):
            V.run_v6(gpus=bad)


def test_v5_curve_and_resume_gates_can_fail():
    good = V.run_v5(steps=16)
    assert good["loss_curve_matches_ladder"] and good["checkpoint_resume_ok"] and good["slope"] < 0
    assert V.run_v5(steps=16, reverse_curve=True)["loss_curve_matches_ladder"] is False
    lost = V.run_v5(steps=16, fresh_optimizer_on_resume=True)
    assert lost["checkpoint_resume_ok"] is False and lost["loss_curve_matches_ladder"] is True
    for bad in (0, -1, True):
        with pytest.raises(V.VerifyError):
            V.run_v5(gpus=bad)


def test_v2_fails_when_a_rank_is_lost_before_the_reduction():
    good, bad = V.run_v2(steps=2), V.run_v2(steps=2, drop_rank=True)
    assert good["loss_rel_diff"] < 1e-4 and good["routing_identical"] is True and good["ranks_emulated"] == 4
    assert bad["grad_rel_diff"] > 0.1 and bad["loss_rel_diff"] > 0.1
    for bad_gpus in (0, -1, True):
        with pytest.raises(V.VerifyError):
            V.run_v2(gpus=bad_gpus)


def test_v3_fails_at_one_bit_of_precision():
    import torch

    bad = V.run_v3(steps=60, crush_precision=True)
    assert bad["fp8_loss_rel_diff"] > 0.005
    if not torch.cuda.is_available():            # with a GPU the stage runs the fused trainer, which needs its 480 steps
        good = V.run_v3(steps=60)
        assert good["fp8_loss_rel_diff"] <= 0.005 and good["nvfp4_numerics_ok"] is True
    with pytest.raises(V.VerifyError):
        V.run_v3(gpus=0)
