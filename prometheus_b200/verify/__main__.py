"""Command line of the verification stages (see the package docstring)."""
import argparse
import json
import sys

from . import check_exit, render_job, run_stage, write_result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m prometheus_b200.verify")
    ap.add_argument("--stage", help="run this stage's runner and write <out>/<stage>.json")
    ap.add_argument("--check", help="apply the exit checker of this stage to <out>")
    ap.add_argument("--render", help="print the job script of this stage")
    ap.add_argument("--out", default="verify-out")
    ap.add_argument("--gpus", type=int)
    ap.add_argument("--hours", type=float)
    ap.add_argument("--run-id", default="run")
    ap.add_argument("--walltime", default="01:00:00")
    a = ap.parse_args(argv)
    if a.render:
        print(render_job(a.render, a.run_id, a.walltime, a.gpus))
    if a.stage:
        kw = {}
        if a.gpus is not None and a.stage.lower() != "v10":
            kw["gpus"] = a.gpus
        if a.hours is not None:
            kw["hours"] = a.hours
        result = run_stage(a.stage, **kw)
        print(json.dumps(result, sort_keys=True))
        write_result(a.stage, result, a.out)
    if a.check:
        check_exit(a.check, a.out)
        print(f"{a.check}: exit criterion met")
    return 0


if __name__ == "__main__":
    sys.exit(main())
