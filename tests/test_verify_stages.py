"""Verification stages: native table / templates / exit checkers and the Python runners."""
import json

import pytest

from prometheus_b200 import native, verify
from prometheus_b200.native import NativeError

N = native.ncshare


def _kind(e):
    return e.value.kind


def test_stage_table_and_templates():
    assert N.STAGES == [f"v{i}" for i in range(11)] and N.JOB_PREFIX == "fv"
    assert N.parse_stage("V7") == "v7" and N.spec("v2")["gpus"] == 8 and N.spec("v10")["gpus"] is None
    assert [N.spec(s)["gpus"] for s in N.STAGES] == [1, 1, 8, 8, 4, 8, 4, 8, 1, 1, None]
    with pytest.raises(NativeError) as e:
        N.parse_stage("v11")
    assert _kind(e) == "UnknownStage"
    for st in N.STAGES:
        text = verify.render_job(st, "r42", "02:00:00")
        assert "fv-r42-" + st in text and "02:00:00" in text and "{{" not in text
        if st not in ("v10",):
            assert f"--gres=gpu:b200:{N.spec(st)['gpus']}" in text
    two = verify.render_v0_2node("r42", "00:30:00")
    assert "--nodes=2" in two and "gpu:b200:4" in two and "{{" not in two and "node_facts.txt" in two
    for args in (("v1", "", "1:00", 1), ("v1", "r", "", 1), ("v1", "r", "1:00", 0)):
        with pytest.raises(NativeError) as e:
            N.render_job(*args, str(verify.TEMPLATE_DIR))
        assert _kind(e) == "Other"


NCCL = """# nThread 1 nGpus 8
#       size         count      type   redop    root     time   algbw   busbw #wrong     time   algbw   busbw #wrong
     1048576        262144     float     sum      -1    45.21   23.19   40.59      0    44.80   23.41   40.96      0
  1073741824     268435456     float     sum      -1   2592.1  414.23  724.91      0   2590.0  414.57  725.50      0
# Out of bounds values : 0 OK
"""


def test_busbw_parser_and_kvm_facts():
    assert N.parse_busbw_gbps(NCCL) == 724.91
    for bad in ("", "# only comments\n", "a b c d e f g h i\n"):
        with pytest.raises(NativeError):
            N.parse_busbw_gbps(bad)
    assert N.kvm_available("crw-rw---- 1 root kvm 10, 232 /dev/kvm\n") is True
    assert N.kvm_available("# host a\n/dev/kvm: no such file\n") is False
    assert N.kvm_available("kvm: yes") is True and N.kvm_available("KVM: absent") is False
    assert N.kvm_available("/dev/kvm: character special file") is True
    for bad in ("", "nvme: none\n", "/dev/kvm is mentioned vaguely", "kvm: maybe"):
        with pytest.raises(NativeError):
            N.kvm_available(bad)


GOOD = {
    "v1": {"logits_max_diff": 1e-6, "grad_ok": True, "overfit_ok": True},
    "v2": {"loss_rel_diff": 0.0, "routing_identical": True},
    "v3": {"fp8_loss_rel_diff": 0.004, "nvfp4_numerics_ok": True},
    "v4": {"resumed_bitwise_equal": True, "sdc_caught_flip": True, "spike_rollback_skipped_shard": True},
    "v5": {"loss_curve_matches_ladder": True, "checkpoint_resume_ok": True},
    "v6": {"curriculum_no_collapse": True, "accuracy_rises_with_latent_budget": True, "thoughts_decode": True},
    "v7": {"reward_rises": True, "logprob_drift_halted": True, "planted_write_flagged": True},
    "v8": {"logprob_within_threshold": True, "tiered_restore_matches": True},
    "v9": {"planted_positive_found": True, "planted_positive_replicated": True, "planted_negative_recorded": True},
    "v10": {"hours": 72.0, "lost_tasks": 0, "duplicated_outputs": 0, "dead_tokens": 0},
}


def test_exit_checkers(tmp_path):
    with pytest.raises(NativeError) as e:
        N.check_exit("v1", str(tmp_path / "nope"))
    assert _kind(e) == "MissingOutput"
    for st, good in GOOD.items():
        d = tmp_path / st
        with pytest.raises(NativeError) as e:
            d.mkdir()
            N.check_exit(st, str(d))
        assert _kind(e) == "MissingOutput"
        verify.write_result(st, good, d)
        verify.check_exit(st, d)
        for key, val in good.items():
            broken = dict(good)
            del broken[key]
            (d / f"{st}.json").write_text(json.dumps(broken))
            with pytest.raises(NativeError) as e:
                N.check_exit(st, str(d))
            assert _kind(e) == "MissingOutput"
            wrong = dict(good, **{key: "yes"})
            (d / f"{st}.json").write_text(json.dumps(wrong))
            with pytest.raises(NativeError) as e:
                N.check_exit(st, str(d))
            assert _kind(e) == "ExitFailed"
            failing = dict(good, **{key: (False if val is True else (1 if val == 0 else (71.0 if key == "hours" else 1.0)))})
            (d / f"{st}.json").write_text(json.dumps(failing))
            with pytest.raises(NativeError) as e:
                N.check_exit(st, str(d))
            assert _kind(e) == "ExitFailed", (st, key)
        (d / f"{st}.json").write_text("[1]")
        with pytest.raises(NativeError) as e:
            N.check_exit(st, str(d))
        assert _kind(e) == "ExitFailed"
    v0 = tmp_path / "v0"
    v0.mkdir()
    with pytest.raises(NativeError) as e:
        N.check_exit("v0", str(v0))
    assert _kind(e) == "MissingOutput"
    (v0 / "busbw_gbps").write_text(NCCL)
    with pytest.raises(NativeError) as e:
        N.check_exit("v0", str(v0))
    assert _kind(e) == "MissingOutput"
    (v0 / "node_facts.txt").write_text("/dev/kvm: no such file\n")
    N.check_exit("v0", str(v0))                       # kvm absent is a known answer: passes
    (v0 / "busbw_gbps").write_text("412.5\n")
    N.check_exit("v0", str(v0))
    (v0 / "busbw_gbps").write_text("fast\n")
    with pytest.raises(NativeError) as e:
        N.check_exit("v0", str(v0))
    assert _kind(e) == "ExitFailed"
    (v0 / "busbw_gbps").write_text("412.5\n")
    (v0 / "node_facts.txt").write_text("nothing relevant\n")
    with pytest.raises(NativeError) as e:
        N.check_exit("v0", str(v0))
    assert _kind(e) == "ExitFailed"


@pytest.mark.parametrize("stage", ["v2", "v3", "v6", "v7", "v9", "v10"])
def test_runners_meet_their_own_exit_criteria(stage, tmp_path):
    import torch

    # with a GPU present v3 runs the fused trainer, which needs its default step count
    kw = {"steps": 6} if stage == "v2" else ({"steps": 60} if stage == "v3" and not torch.cuda.is_available() else {})
    result = verify.run_stage(stage, **kw)
    verify.write_result(stage, result, tmp_path)
    verify.check_exit(stage, tmp_path)


def test_cli_round_trip(tmp_path, capsys):
    from prometheus_b200.verify.__main__ import main

    assert main(["--stage", "v9", "--out", str(tmp_path), "--check", "v9"]) == 0
    assert "exit criterion met" in capsys.readouterr().out
    with pytest.raises(verify.VerifyError):
        verify.run_stage("v0")


def test_allreduce_bench_table_is_parseable_on_two_cpu_ranks():
    import subprocess
    import sys

    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", "-m",
                          "prometheus_b200.parallel.allreduce_bench", "--min-bytes", "4096", "--max-bytes", "65536",
                          "--iters", "3", "--warmup", "1"], capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    rows = [l for l in out.stdout.splitlines() if l.strip() and not l.startswith("#")]
    assert len(rows) == 3 and all(r.split()[8] == "0" for r in rows)          # #wrong == 0
    assert N.parse_busbw_gbps(out.stdout) == float(rows[-1].split()[7]) > 0
