#!/bin/bash
# V10: harness chaos soak while the V5-V9 jobs run (shared allocation, no GPU of its own).
# Exit criterion is read from $OUT/v10.json by the stage checker.
#SBATCH -J fv-{{RUN_ID}}-v10
#SBATCH -t {{WALLTIME}}
#SBATCH -p cpu
#SBATCH --nodes=1
#SBATCH --ntasks=1
#SBATCH --output=fv-{{RUN_ID}}-v10-%j.out
#SBATCH --error=fv-{{RUN_ID}}-v10-%j.err
set -euo pipefail

ROOT="${PROMETHEUS_ROOT:-${SLURM_SUBMIT_DIR:-$PWD}}"
OUT="${VERIFY_OUTPUT_DIR:-$ROOT/verify-out/{{RUN_ID}}/v10}"
mkdir -p "$OUT"
cd "$ROOT"
python -m prometheus_b200._build --native-only
python -m prometheus_b200.verify --stage v10 --hours "${SOAK_HOURS:-72}" --out "$OUT"
python -m prometheus_b200.verify --check v10 --out "$OUT"
