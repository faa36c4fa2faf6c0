#!/usr/bin/env bash
# ODC=1|0  FSDP2=1|0  HPZ=1|0  HSDP=1|0  bash examples/llm_training/run.sh [trainer flags]
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
export ODC=${ODC:-1} HPZ=${HPZ:-0} HSDP=${HSDP:-0}
if [[ "${HSDP}" == "1" ]]; then export ODC_SYMMETRIC_SIZE=${ODC_SYMMETRIC_SIZE:-10G}; else export ODC_SYMMETRIC_SIZE=${ODC_SYMMETRIC_SIZE:-64G}; fi
SCRIPT=train_fsdp2.py
[[ "${FSDP2:-1}" == "0" ]] && SCRIPT=train_fsdp1.py
cd "$HERE" && exec bash "$ROOT/launch.sh" "$HERE/$SCRIPT" "$@"
