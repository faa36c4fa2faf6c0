#!/usr/bin/env bash
# Launch a script on every GPU of this node (and, with NNODES>1, of several nodes).
#   bash launch.sh examples/llm_training/train_fsdp2.py --model_name llama3.2-1b
# Environment: GPUS_PER_NODE (default: all visible), NNODES (1), NODE_RANK (0), MASTER_ADDR (127.0.0.1),
# MASTER_PORT (29500), ODC_SYMMETRIC_SIZE (address space reserved per rank, default 64G; physical
# memory is mapped as buffers are allocated), PROFILED=1 (wrap in nsys when it is installed),
# MAX_RESTARTS (0): how often the launcher restarts all ranks after one of them failed (a trainer given
# --checkpoint-dir then resumes from its newest checkpoint).
set -euo pipefail
GPUS_PER_NODE=${GPUS_PER_NODE:-$(python - <<'PY'
import torch; print(max(torch.cuda.device_count(), 1))
PY
)}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export LOCAL_WORLD_SIZE=${GPUS_PER_NODE}
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-16}
export ODC_SYMMETRIC_SIZE=${ODC_SYMMETRIC_SIZE:-${NVSHMEM_SYMMETRIC_SIZE:-64G}}
export TORCH_CPP_LOG_LEVEL=${TORCH_CPP_LOG_LEVEL:-ERROR}
CMD=(python -m torch.distributed.run --nnodes="${NNODES}" --node-rank="${NODE_RANK}" --nproc-per-node="${GPUS_PER_NODE}"
     --master-addr "${MASTER_ADDR}" --master-port "${MASTER_PORT}" "$@")
if [[ "${PROFILED:-0}" == "1" ]] && command -v nsys >/dev/null; then
  exec nsys profile --trace=cuda,nvtx --capture-range=cudaProfilerApi -o "${RUN_NAME:-odc_b200}" "${CMD[@]}"
fi
# Each attempt is a fresh launcher (new rendezvous store, new processes); ODC_LAUNCH_ATTEMPT tells the job which one.
attempt=0
while true; do
  rc=0
  ODC_LAUNCH_ATTEMPT=${attempt} "${CMD[@]}" || rc=$?
  if [[ ${rc} -eq 0 || ${attempt} -ge ${MAX_RESTARTS:-0} ]]; then
    exit ${rc}
  fi
  attempt=$((attempt + 1))
  echo "launch.sh: attempt ${attempt} of ${MAX_RESTARTS} after exit code ${rc}" >&2
  sleep "${RESTART_DELAY_S:-2}"
done
