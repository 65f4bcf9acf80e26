"""Host-side chaos runner and the Slurm client (C++), against the contracts of the reference's
harness/chaos and harness/slurm crates. Nothing here touches a GPU: faults are simulated on
event-log replicas, and the scheduler is a fake `ssh` script."""
import json
import os
import stat

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

CH, SL = native.chaos, native.slurm


def _kind(e):
    return e.value.kind


def test_chaos_world_faults_recovery_and_invariants(tmp_path):
    with pytest.raises(NativeError) as e:
        CH.World.create(str(tmp_path / "w1"), 1)
    assert _kind(e) == "TooFewReplicas"
    w = CH.World.create(str(tmp_path / "w"), 3, 4, 7)
    assert w.replicas() == ["0", "1", "2"] and w.processes() == ["coordinator", "worker-0", "worker-1", "worker-2"]
    w.enqueue_task("t0", 0)
    w.enqueue_task("t1", 0)
    assert w.invariants().lost_tasks == 2
    # a partition keeps events from replica 0 away from replica 1
    w.inject(CH.Fault("partition", "0", "1"))
    w.enqueue_task("t2", 1)
    assert (w.log_len("0"), w.log_len("1")) == (4, 3)
    w.inject(CH.Fault("heal_partition", "0", "1"))
    # kill drops every in-memory handle; nothing can be written until recovery replays the disk
    w.inject(CH.Fault("kill", "coordinator"))
    with pytest.raises(NativeError):
        w.enqueue_task("t3", 2)
    w.recover()
    assert w.replica_event_types("0")[-1] == "chaos.recover"
    for t in ("t0", "t1", "t2"):
        w.complete_task(t, 1, b"ok", 3)
    assert w.invariants().hold()
    w.complete_task("t0", 1, b"again", 4)                      # same attempt twice = duplicate
    assert w.invariants().duplicated_outputs == 1
    # corruption: the replica is skipped by recovery and by the invariants, bytes are garbage
    w.inject(CH.Fault("disk_corrupt", "2"))
    assert open(os.path.join(w.replica_dir("2"), "events.jsonl"), "rb").read() == b"{broken hash chain\n"
    with pytest.raises(NativeError) as e:
        w.log_len("2")
    assert _kind(e) == "Disk"
    w.recover()
    with pytest.raises(NativeError) as e:
        w.inject(CH.Fault("clock_skew", "0", delta_ms=30_001))
    assert _kind(e) == "ClockSkewBound"
    w.inject(CH.Fault("clock_skew", "0", delta_ms=-30_000))
    w.inject(CH.Fault("node_replace", "1", "9"))
    assert w.replicas() == ["0", "1", "2", "9"]
    for bad, kind in ((CH.Fault("kill", "nobody"), "NoProcess"), (CH.Fault("node_loss", "77"), "NoReplica")):
        with pytest.raises(NativeError) as e:
            w.inject(bad)
        assert _kind(e) == kind
    assert json.loads(CH.Fault("partition", "0", "1", True).to_json()) == \
        {"partition": {"from": "0", "to": "1", "asymmetric": True}}
    assert json.loads(CH.Fault("token_expiry").to_json()) == "token_expiry" and len(CH.FAULT_KINDS) == 18
    # a world reopened from disk rebuilds its bookkeeping; torn files are refused
    w2 = CH.World.create(str(tmp_path / "w2"), 2)
    w2.enqueue_task("a", 0)
    again = CH.World.open(str(tmp_path / "w2"), 2)
    assert again.invariants().lost_tasks == 1
    with open(os.path.join(w2.replica_dir("0"), "events.jsonl"), "ab") as f:
        f.write(b'{"torn":')
    with pytest.raises(NativeError) as e:
        CH.World.open(str(tmp_path / "w2"), 2)
    assert _kind(e) == "Log"


@pytest.mark.parametrize("gate,n", [("D0", 1000), ("D1", 2), ("D2", 4), ("D3", 3), ("D4", 3), ("D5", 2)])
def test_chaos_gates_hold_invariants(tmp_path, gate, n):
    w = CH.World.create(str(tmp_path / gate), 2, 4, 3)
    rep = CH.run_gate(w, gate)
    assert (rep.gate, rep.faults_applied, rep.recovered) == (gate, n, True) and rep.invariants.hold()
    assert len(CH.faults_for(gate)) == (1 if gate == "D0" else n)


def test_chaos_soak_covers_72_injected_hours(tmp_path):
    w = CH.World.create(str(tmp_path / "soak"), 3, 4, 11)
    rep = CH.run_gate(w, "Soak")
    assert rep.gate == "Soak" and rep.invariants.hold() and rep.faults_applied == 16
    assert w.now() == CH.SOAK_MS
    assert len(CH.faults_for("Soak")) == 15
    with pytest.raises(NativeError):
        CH.run_gate(w, "D9")


FAKE_SSH = r"""#!/bin/sh
# fake cluster: $1 is the cluster name, the rest is the remote command
shift
log="$FAKE_SLURM_DIR/calls"
echo "$@" >> "$log"
case "$1" in
  squeue) cat "$FAKE_SLURM_DIR/squeue" 2>/dev/null ;;
  sbatch) if [ -f "$FAKE_SLURM_DIR/sbatch_fail" ]; then echo "sbatch: error" >&2; exit 1; fi
          echo "Submitted batch job 4242" ;;
  sacct)  if [ -f "$FAKE_SLURM_DIR/hang" ]; then sleep 5; fi
          cat "$FAKE_SLURM_DIR/sacct_out" 2>/dev/null ;;
  scancel) echo "$2" >> "$FAKE_SLURM_DIR/cancelled" ;;
esac
"""


def test_slurm_client_against_a_fake_cluster(tmp_path, monkeypatch):
    fake = tmp_path / "ssh"
    fake.write_text(FAKE_SSH)
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PROMETHEUS_SLURM_SSH", str(fake))
    monkeypatch.setenv("FAKE_SLURM_DIR", str(tmp_path))
    c = SL.Client(SL.ClientConfig(state_dir=str(tmp_path / "state"), query_timeout_ms=400))
    with pytest.raises(NativeError) as e:
        c.submit("run1", "v3", "job.sh", "00:30:00", 8)
    assert _kind(e) == "BadGpuCount"
    (tmp_path / "squeue").write_text("1 gpu fv-a user R 0:10\n2 gpu fv-b user PD 0:00\n3 gpu other user R 1:00\n")
    with pytest.raises(NativeError) as e:
        c.submit("run1", "v3", "job.sh", "00:30:00", 2)
    assert _kind(e) == "ConcurrentCap"
    (tmp_path / "squeue").write_text("1 gpu fv-a user R 0:10\n4 gpu fv-c user CG 0:10\n")
    jid = c.submit("run1", "v3", "job.sh", "00:30:00", 2)
    assert jid == "4242"
    run = tmp_path / "state" / "runs" / "run1"
    assert (run / "job-name").read_text() == "fv-v3\n" and (run / "job-ids").read_text() == "4242\n"
    calls = (tmp_path / "calls").read_text().splitlines()
    assert calls[-1] == "sbatch -J fv-v3 -t 00:30:00 -p gpu --gres=gpu:b200:2 job.sh"
    # sbatch failure: the name file exists (written first), no id recorded
    (tmp_path / "sbatch_fail").write_text("x")
    with pytest.raises(NativeError) as e:
        c.submit("run2", "v4", "job.sh", "00:10:00", 1)
    assert _kind(e) == "Submit"
    assert (tmp_path / "state" / "runs" / "run2" / "job-name").read_text() == "fv-v4\n"
    assert (tmp_path / "state" / "runs" / "run2" / "job-ids").read_text() == ""
    # state parsing; unknown text maps to Unknown
    for text, want in (("  COMPLETED \n", "Completed"), ("CANCELLED+\n", "Cancelled"), ("weird\n", "Unknown"),
                       ("", "Unknown")):
        (tmp_path / "sacct_out").write_text(text)
        assert c.state("4242") == want
    (tmp_path / "sacct_out").write_text("RUNNING\n")
    assert SL.parse_state("OUT_OF_MEMORY") == "OutOfMemory" and SL.parse_state("NODE_FAIL x") == "NodeFail"
    assert SL.parse_state("nope") is None and SL.parse_state("  ") is None
    assert SL.is_terminal("Timeout") and not SL.is_terminal("Unknown")
    assert SL.count_live_fv("9 p fv-x u RUNNING\n8 p fvx u R\n7 p fv u pd\n") == 2
    # wait: non-terminal until the budget ends, then the job is cancelled
    assert c.wait("4242", 150) == "Cancelled"
    assert "4242" in (tmp_path / "cancelled").read_text().split()
    # a hung sacct is killed after the timeout and reported as such
    (tmp_path / "hang").write_text("x")
    with pytest.raises(NativeError) as e:
        c.state("4242")
    assert _kind(e) == "QueryTimeout"
    (tmp_path / "hang").unlink()
    # reap only what was recorded
    (run / "job-ids").write_text("4242\nnot-a-number\n77\n")
    (tmp_path / "cancelled").write_text("")
    c.reap_tracked("run1")
    assert (tmp_path / "cancelled").read_text().split() == ["4242", "77"]
    c.reap_tracked("no-such-run")
