"""Behaviour list of the Slurm client (C++ ``native.slurm``; reference
harness/slurm/tests/{submit,query,cancel,wait,paths,parse}.rs) against a fake cluster made of
shell scripts: allowed GPU counts, the cap on live jobs, what is on disk before ``sbatch``
runs, the exact command lines (a cancel names one id, never a user), waiting, fetching, and
the parsing of scheduler text compared with a Python model on random noise."""
import random
import stat
import time

import pytest

from prometheus_b200 import native
from prometheus_b200.native import NativeError

S = native.slurm

FAKE_SSH = r"""#!/bin/sh
shift
echo "$@" >> "$FAKE_DIR/calls"
case "$1" in
  squeue) cat "$FAKE_DIR/squeue" 2>/dev/null ;;
  sbatch) if [ -f "$FAKE_DIR/sbatch_fail" ]; then echo "sbatch: error: down" >&2; exit 1; fi
          cat "$FAKE_DIR/sbatch_out" 2>/dev/null || echo "Submitted batch job 9001" ;;
  sacct)  if [ -f "$FAKE_DIR/hang" ]; then sleep 5; fi
          n=$(cat "$FAKE_DIR/polls" 2>/dev/null || echo 0); n=$((n + 1)); echo $n > "$FAKE_DIR/polls"
          if [ -f "$FAKE_DIR/done_after" ] && [ $n -ge $(cat "$FAKE_DIR/done_after") ]; then echo COMPLETED; else cat "$FAKE_DIR/sacct_out" 2>/dev/null; fi ;;
  scancel) echo "$@" >> "$FAKE_DIR/cancelled" ;;
esac
exit 0
"""

FAKE_RSYNC = r"""#!/bin/sh
echo "$@" >> "$FAKE_DIR/rsync_calls"
for last; do :; done
if [ -f "$FAKE_DIR/rsync_fail" ]; then exit 23; fi
echo artifact > "$last/metrics.json"
"""


def err(call):
    with pytest.raises(NativeError) as e:
        call()
    return e.value


@pytest.fixture
def cluster(tmp_path, monkeypatch):
    for name, body in (("ssh", FAKE_SSH), ("rsync", FAKE_RSYNC)):
        f = tmp_path / "bin" / name
        f.parent.mkdir(exist_ok=True)
        f.write_text(body)
        f.chmod(f.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PROMETHEUS_SLURM_SSH", str(tmp_path / "bin" / "ssh"))
    monkeypatch.setenv("PATH", f"{tmp_path / 'bin'}:" + __import__("os").environ["PATH"])
    monkeypatch.setenv("FAKE_DIR", str(tmp_path))
    client = S.Client(S.ClientConfig(cluster="fakecluster", remote_root="/work/p", state_dir=str(tmp_path / "state"), query_timeout_ms=400))
    return client, tmp_path


def calls(d):
    return (d / "calls").read_text().splitlines() if (d / "calls").exists() else []


# ------------------------------------------------------------------------------ submit
def test_constants_names_and_paths(cluster):
    c, d = cluster
    assert (S.ALLOWED_GPUS, S.MAX_CONCURRENT_JOBS, S.JOB_PREFIX, S.QUERY_TIMEOUT_MS) == ([1, 2, 4], 2, "fv", 45_000)
    assert c.job_ids_path("run-7") == str(d / "state" / "runs" / "run-7" / "job-ids")


@pytest.mark.parametrize("gpus", [0, 3, 5, 8, 16])
def test_other_gpu_counts_are_refused_before_anything_is_sent(cluster, gpus):
    c, d = cluster
    assert err(lambda: c.submit("r", "x", "job.sh", "00:10:00", gpus)).kind == "BadGpuCount"
    assert calls(d) == [] and not (d / "state").exists()


@pytest.mark.parametrize("gpus", [1, 2, 4])
def test_submit_command_line_and_bookkeeping(cluster, gpus):
    c, d = cluster
    (d / "sbatch_out").write_text("some banner\nSubmitted batch job 31337 on cluster x\n")
    assert c.submit("run1", "abc", "train.sbatch", "01:30:00", gpus) == "31337"
    assert calls(d) == ["squeue --noheader", f"sbatch -J fv-abc -t 01:30:00 -p gpu --gres=gpu:b200:{gpus} train.sbatch"]   # a hard wall time, always
    run = d / "state" / "runs" / "run1"
    assert (run / "job-name").read_text() == "fv-abc\n" and (run / "job-ids").read_text() == "31337\n"
    (d / "sbatch_out").write_text("Submitted batch job 31338\n")
    c.submit("run1", "abc", "train.sbatch", "00:05:00", gpus)
    assert (run / "job-ids").read_text() == "31337\n31338\n"                                  # ids accumulate per run


def test_live_job_cap_counts_only_this_frameworks_running_or_pending_jobs(cluster):
    c, d = cluster
    (d / "squeue").write_text("1 gpu fv-a me R 0:10\n2 gpu fv-b me PD 0:00\n3 gpu someone-else me R 9:00\n")
    assert err(lambda: c.submit("r", "x", "job.sh", "00:10:00", 1)).kind == "ConcurrentCap"
    assert calls(d) == ["squeue --noheader"] and not (d / "state" / "runs" / "r" / "job-name").exists()
    (d / "squeue").write_text("1 gpu fv-a me R 0:10\n2 gpu fv-b me CG 0:00\n3 gpu other me R 9:00\n4 gpu other2 me PD 0:00\n")
    assert c.submit("r", "x", "job.sh", "00:10:00", 1) == "9001"                               # one live job of ours: allowed


def test_the_job_name_is_on_disk_before_sbatch_runs(cluster):
    c, d = cluster
    (d / "sbatch_fail").write_text("x")
    assert err(lambda: c.submit("r2", "y", "job.sh", "00:10:00", 2)).kind == "Submit"
    run = d / "state" / "runs" / "r2"
    assert (run / "job-name").read_text() == "fv-y\n" and (run / "job-ids").read_text() == ""  # a crash here can still be cleaned up by name
    (d / "sbatch_fail").unlink()
    (d / "sbatch_out").write_text("queued, no number given\n")
    assert err(lambda: c.submit("r3", "z", "job.sh", "00:10:00", 2)).kind == "Submit"
    assert (d / "state" / "runs" / "r3" / "job-ids").read_text() == ""


# ------------------------------------------------------------------------------ query / cancel / wait / fetch
def test_state_queries_never_hang(cluster):
    c, d = cluster
    for text, want in (("RUNNING\n", "Running"), ("PENDING\n", "Pending"), ("  COMPLETED  \n", "Completed"), ("CANCELLED by 1000\n", "Cancelled"),
                       ("TIMEOUT+\n", "Timeout"), ("", "Unknown"), ("COMPLETING\n", "Unknown"), ("what\n", "Unknown")):
        (d / "sacct_out").write_text(text)
        assert c.state("55") == want
    assert any(line.startswith("sacct") and "55" in line.split() or "-j" in line for line in calls(d))
    (d / "hang").write_text("x")
    t0 = time.monotonic()
    assert err(lambda: c.state("55")).kind == "QueryTimeout" and time.monotonic() - t0 < 3    # the configured limit, not the scheduler's mood


def test_cancel_names_exactly_one_job(cluster):
    c, d = cluster
    c.cancel("4242")
    assert (d / "cancelled").read_text().splitlines() == ["scancel 4242"]
    assert all("-u" not in line.split() and "--user" not in line for line in calls(d))         # never a whole user's jobs
    (d / "state" / "runs" / "mine").mkdir(parents=True)
    (d / "state" / "runs" / "other").mkdir(parents=True)
    (d / "state" / "runs" / "mine" / "job-ids").write_text("10\n\nnot-an-id\n 11 \n12abc\n13\n")
    (d / "state" / "runs" / "other" / "job-ids").write_text("99\n")
    (d / "cancelled").write_text("")
    c.reap_tracked("mine")
    assert (d / "cancelled").read_text().splitlines() == ["scancel 10", "scancel 13"]          # only clean ids of that run
    c.reap_tracked("never-submitted")
    assert (d / "cancelled").read_text().splitlines() == ["scancel 10", "scancel 13"]


def test_wait_returns_the_terminal_state_or_cancels_at_the_limit(cluster):
    c, d = cluster
    (d / "sacct_out").write_text("RUNNING\n")
    (d / "done_after").write_text("3")
    assert c.wait("77", 20_000) == "Completed" and not (d / "cancelled").exists()
    (d / "done_after").unlink()
    assert c.wait("78", 200) == "Cancelled"
    assert (d / "cancelled").read_text().splitlines() == ["scancel 78"]


def test_fetch_copies_the_runs_directory(cluster):
    c, d = cluster
    dest = d / "out" / "deep"
    c.fetch("run9", str(dest))
    assert (dest / "metrics.json").read_text() == "artifact\n"
    assert (d / "rsync_calls").read_text().split()[-2:] == ["fakecluster:/work/p/run9/", str(dest)]
    (d / "rsync_fail").write_text("x")
    err(lambda: c.fetch("run9", str(dest)))


# ------------------------------------------------------------------------------ parsing
STATES = {"PENDING": "Pending", "RUNNING": "Running", "COMPLETED": "Completed", "FAILED": "Failed", "CANCELLED": "Cancelled", "CANCELED": "Cancelled",
          "TIMEOUT": "Timeout", "PREEMPTED": "Preempted", "NODE_FAIL": "NodeFail", "OUT_OF_MEMORY": "OutOfMemory"}


def model_parse(raw):
    tokens = raw.split()
    return STATES.get(tokens[0].rstrip("+").upper()) if tokens else None


def test_parse_state_table_and_terminal_states():
    for token, want in STATES.items():
        assert S.parse_state(token) == want == S.parse_state(f"  {token.lower()}+  trailing words\nSECOND LINE")
    for raw in ("", "   \n\t", "COMPLETING", "SUSPENDED", "BOOT_FAIL", "COMPLETED|", "+", "RUN NING", "JobState=RUNNING"):
        assert S.parse_state(raw) is None
    assert [s for s in list(dict.fromkeys(STATES.values())) + ["Unknown"] if not S.is_terminal(s)] == ["Pending", "Running", "Unknown"]


def test_random_scheduler_text_agrees_with_the_model():
    rng = random.Random(0)
    pieces = list(STATES) + ["completing", "running", "Cancelled", "+", "++", " ", "\n", "\t", "by", "123", "x", "NODE_FAIL+", "|"]
    for _ in range(500):
        raw = "".join(rng.choice(pieces) + rng.choice(["", " ", "+", "\n"]) for _ in range(rng.randint(0, 4)))
        assert S.parse_state(raw) == model_parse(raw), repr(raw)


def model_live(text):
    n = 0
    for line in text.split("\n"):
        f = line.split()
        n += any(x == "fv" or x.startswith("fv-") for x in f) and any(x.upper() in ("R", "PD", "RUNNING", "PENDING") for x in f)
    return n


def test_count_live_jobs_agrees_with_the_model():
    assert S.count_live_fv("") == 0 and S.count_live_fv("1 gpu fv-a me R 0:01") == 1 and S.count_live_fv("1 gpu fva me R\n2 gpu xfv-a me R\n") == 0
    assert S.count_live_fv("1 gpu fv-a me CG\n2 gpu fv-b me F\n3 gpu fv-c me pd\n4 gpu fv-d me Running\n") == 2
    rng = random.Random(1)
    words = ["fv-a", "fv", "fvx", "other", "R", "PD", "CG", "r", "pending", "RUNNING", "gpu", "17", "0:10", "xfv-1"]
    for _ in range(300):
        text = "\n".join(rng.choice([" ", "\t", "  "]).join(rng.choice(words) for _ in range(rng.randint(0, 6))) for _ in range(rng.randint(0, 5)))
        assert S.count_live_fv(text) == model_live(text), repr(text)
