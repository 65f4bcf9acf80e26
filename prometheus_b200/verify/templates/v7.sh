#!/bin/bash
# V7: RL loss, staleness, routing replay, weight sync, parity halt, reward-hacking controls
# Exit criterion is read from $OUT/v7.json by the stage checker, never from a summary.
#SBATCH -J fv-{{RUN_ID}}-v7
#SBATCH -t {{WALLTIME}}
#SBATCH -p gpu
#SBATCH --gres=gpu:b200:{{GPUS}}
#SBATCH --nodes=1
#SBATCH --ntasks=1
#SBATCH --output=fv-{{RUN_ID}}-v7-%j.out
#SBATCH --error=fv-{{RUN_ID}}-v7-%j.err
set -euo pipefail

ROOT="${PROMETHEUS_ROOT:-${SLURM_SUBMIT_DIR:-$PWD}}"
OUT="${VERIFY_OUTPUT_DIR:-$ROOT/verify-out/{{RUN_ID}}/v7}"
mkdir -p "$OUT"
cd "$ROOT"

# the job fails closed unless the kernels are built for this GPU and a GPU is visible
python -m prometheus_b200._build
python - <<'PY'
import torch
assert torch.cuda.is_available(), "no GPU visible to the job"
print("gpu:", torch.cuda.get_device_name(0), "count:", torch.cuda.device_count())
PY

python -m prometheus_b200.verify --stage v7 --gpus {{GPUS}} --out "$OUT"
python -m prometheus_b200.verify --check v7 --out "$OUT"
