#!/bin/bash
#SBATCH --job-name={job_name}
#SBATCH --nodes={num_nodes}
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=56
#SBATCH --mem=0
#SBATCH --exclusive
#SBATCH --partition={partition}
#SBATCH --account={account}
#SBATCH --time={time}
#SBATCH --output={dump_dir}/{job_name}/logs/%j.out
#SBATCH --error={dump_dir}/{job_name}/logs/%j.err

# One task per node; each task starts one process per GPU through torchrun (scripts/slurm/in_container.sh).
set -euo pipefail

JOB_DIR="{dump_dir}/{job_name}"
CONTAINER="{container}"

# newest log is always reachable as latest.out / latest.err
ln -sfn "$SLURM_JOB_ID.out" "$JOB_DIR/logs/latest.out"
ln -sfn "$SLURM_JOB_ID.err" "$JOB_DIR/logs/latest.err"

export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export MASTER_PORT=$((20000 + SLURM_JOB_ID % 20000))
export NNODES=$SLURM_JOB_NUM_NODES
export GPUS_PER_NODE=8
export JOB_DIR

echo "job $SLURM_JOB_ID on $NNODES nodes, rendezvous at $MASTER_ADDR:$MASTER_PORT"

if [ -n "$CONTAINER" ]; then
  srun --kill-on-bad-exit=1 singularity exec --nv -B "$PWD" "$CONTAINER" \
    bash scripts/slurm/in_container.sh train.py "$JOB_DIR"
else
  srun --kill-on-bad-exit=1 bash scripts/slurm/in_container.sh train.py "$JOB_DIR"
fi
