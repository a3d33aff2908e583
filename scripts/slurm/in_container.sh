#!/bin/bash
# Per-node launcher: environment for NCCL over NVLink/NVSwitch (+ InfiniBand between nodes), the
# NCCL flight recorder, optional preflight knobs, then torchrun with one process per GPU.
# usage: in_container.sh <script> <job_dir>
set -euo pipefail
SCRIPT="$1"; shift
JOB_DIR="$1"; shift || true

if [ -f .venv/bin/activate ]; then source .venv/bin/activate; fi

# --- NCCL
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}
export NCCL_NVLS_ENABLE=${NCCL_NVLS_ENABLE:-1}          # in-switch reductions on NVSwitch systems
export NCCL_SOCKET_IFNAME=${NCCL_SOCKET_IFNAME:-^lo,docker}
export TORCH_NCCL_ASYNC_ERROR_HANDLING=3                # keep the communicator so the recorder can dump

# --- flight recorder: dump collective history of every rank when a collective times out
export TORCH_NCCL_DUMP_ON_TIMEOUT=1
export TORCH_NCCL_DEBUG_INFO_TEMP_FILE="$JOB_DIR/logs/nccl_trace_rank_"
export TORCH_FR_BUFFER_SIZE=2000
export TORCH_NCCL_ENABLE_TIMING=1

# --- optional link check before training (see nccl_preflight.py)
export RUN_NCCL_PREFLIGHT=${RUN_NCCL_PREFLIGHT:-0}
export NCCL_PREFLIGHT_MAX_MB=${NCCL_PREFLIGHT_MAX_MB:-256}
export NCCL_PREFLIGHT_REPORT_DIR=${NCCL_PREFLIGHT_REPORT_DIR:-$JOB_DIR/logs}

export OMP_NUM_THREADS=${OMP_NUM_THREADS:-7}
NODE_RANK=${SLURM_NODEID:-0}
LOG_DIR="$JOB_DIR/logs/node_${NODE_RANK}"
mkdir -p "$LOG_DIR"

exec torchrun \
  --nnodes="${NNODES:-1}" --nproc_per_node="${GPUS_PER_NODE:-8}" --node_rank="$NODE_RANK" \
  --rdzv_backend=c10d --rdzv_endpoint="${MASTER_ADDR:-127.0.0.1}:${MASTER_PORT:-29500}" \
  --rdzv_id="${SLURM_JOB_ID:-0}" \
  --local-ranks-filter 0 --tee 3 --log-dir "$LOG_DIR" \
  "$SCRIPT" "$JOB_DIR" "$@"
