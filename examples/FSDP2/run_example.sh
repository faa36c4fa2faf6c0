#!/usr/bin/env bash
# ODC=1|0  HPZ=1|0  HSDP=1|0  NUM_GPUS_PER_NODE=2  bash examples/FSDP2/run_example.sh [script] [example flags]
# Runs the toy FSDP2 example (default: example.py --mixed-precision) on NUM_GPUS_PER_NODE GPUs of this node.
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
export ODC=${ODC:-1}
export GPUS_PER_NODE=${NUM_GPUS_PER_NODE:-2}
export ODC_SYMMETRIC_SIZE=${ODC_SYMMETRIC_SIZE:-${NVSHMEM_SYMMETRIC_SIZE:-5G}}
SCRIPT=${1:-$HERE/example.py}
[[ $# -gt 0 ]] && shift
[[ $# -eq 0 ]] && set -- --mixed-precision
echo "Launching ${SCRIPT} on ${GPUS_PER_NODE} GPUs (ODC=${ODC})"
exec bash "$ROOT/launch.sh" "$SCRIPT" "$@"
