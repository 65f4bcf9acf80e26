"""``harness`` operator command line: ``python -m prometheus_b200.native.harness [--json] status``.

Opens the release state under ``--ops-dir`` and the control-plane replicas under ``--raft-dir``
(both are replayed from their own logs) and prints the dispatcher's answer; exit status 1 with
the message on standard error for anything else
(reference: harness/ops/src/bin/harness.rs, prometheus_ops::cli at harness/ops/src/lib.rs:727).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

from . import NativeError, ops, raft

USAGE = "usage: harness [--json] status --ops-dir DIR --raft-dir DIR [--nodes N]\n"


def dispatch(argv: list[str]) -> str:
    ap = argparse.ArgumentParser(prog="harness", add_help=False)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--ops-dir")
    ap.add_argument("--raft-dir")
    ap.add_argument("--nodes", type=int, default=raft.MIN_VOTERS)
    ap.add_argument("-h", "--help", action="store_true")
    ap.add_argument("command", nargs="*")
    a = ap.parse_args(argv)
    if a.help or not a.command:
        return USAGE
    if a.command != ["status"]:
        raise ValueError("unknown command: " + " ".join(a.command))
    if not a.ops_dir or not a.raft_dir:
        raise ValueError("harness status needs --ops-dir and --raft-dir")
    state = ops.Ops.open(a.ops_dir) if Path(a.ops_dir).exists() else ops.Ops.create(a.ops_dir)
    if (Path(a.raft_dir) / "0").exists():          # replicas exist: replay node 0 from its own log
        cluster = raft.Cluster.open(str(Path(a.raft_dir) / "0"), "0")
    else:
        group = raft.LocalGroup.start(a.nodes, a.raft_dir)
        group.tick(0)
        cluster = group.get(0)
    return state.cli((["--json"] if a.json else []) + ["status"], cluster)


def main(argv=None) -> int:
    try:
        out = dispatch(list(sys.argv[1:] if argv is None else argv))
    except (ValueError, NativeError) as err:
        print(err, file=sys.stderr)
        return 1
    sys.stdout.write(out if out.endswith("\n") else out + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
