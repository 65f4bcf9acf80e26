#!/bin/bash
# V0, second allocation: 2 boxes x 4 GPUs. All-reduce bandwidth inside one box and across both,
# /dev/kvm and NVMe facts, queue wait. Writes busbw_gbps and node_facts.txt.
#SBATCH -J fv-{{RUN_ID}}-v0-2node
#SBATCH -t {{WALLTIME}}
#SBATCH -p gpu
#SBATCH --gres=gpu:b200:4
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --output=fv-{{RUN_ID}}-v0-%j.out
#SBATCH --error=fv-{{RUN_ID}}-v0-%j.err
set -euo pipefail

ROOT="${PROMETHEUS_ROOT:-${SLURM_SUBMIT_DIR:-$PWD}}"
OUT="${VERIFY_OUTPUT_DIR:-$ROOT/verify-out/{{RUN_ID}}/v0}"
mkdir -p "$OUT"
cd "$ROOT"

{
  echo "job_id=${SLURM_JOB_ID:-none}"
  echo "submit_time=${SLURM_JOB_SUBMIT_TIME:-unknown}"
  echo "start_time=$(date -u +%Y-%m-%dT%H:%M:%SZ)"
  echo "nodelist=${SLURM_JOB_NODELIST:-$(hostname)}"
} > "$OUT/queue_wait.txt"

python -m prometheus_b200._build

# scheduler dry run of a dummy script
DUMMY="$OUT/test_only.sh"
printf '#!/bin/bash\n#SBATCH -J fv-{{RUN_ID}}-dry\n#SBATCH -t 00:01:00\ntrue\n' > "$DUMMY"
if command -v sbatch >/dev/null 2>&1; then
  sbatch --test-only "$DUMMY" > "$OUT/test_only.txt" 2>&1 || true
fi

# all-reduce bus bandwidth over the GPUs of this allocation (table in the nccl-tests layout)
# inside one box (4 ranks on the batch host) ...
python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 4 \
  -m prometheus_b200.parallel.allreduce_bench --max-bytes 1073741824 > "$OUT/all_reduce_intra.txt"
# ... and across both boxes (8 ranks); busbw_gbps is the two-box measurement
HEAD="$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n1)"
srun --ntasks-per-node=1 python -m torch.distributed.run --nnodes=2 --nproc-per-node 4 \
  --rdzv-backend c10d --rdzv-endpoint "$HEAD:29500" \
  -m prometheus_b200.parallel.allreduce_bench --max-bytes 1073741824 > "$OUT/all_reduce.txt"
cp "$OUT/all_reduce.txt" "$OUT/busbw_gbps"

# facts from every allocated node, not only the batch host
srun --ntasks-per-node=1 bash -c 'echo "# host $(hostname)"; if [[ -e /dev/kvm ]]; then ls -l /dev/kvm; else echo "/dev/kvm: no such file"; fi; lsblk -d -o NAME,ROTA,SIZE,MODEL 2>/dev/null | grep -i nvme || echo "nvme: none"' > "$OUT/node_facts.txt"

python -m prometheus_b200.verify --check v0 --out "$OUT"
