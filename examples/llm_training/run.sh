#!/usr/bin/env bash
# ODC=1|0  FSDP2=1|0  HPZ=1|0  HSDP=1|0  ENGINE=fused  HF=1  bash examples/llm_training/run.sh [trainer flags]
# HF=1: train_hf.py (a transformers model class under the patch; needs --hf-checkpoint <folder>)
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
export ODC=${ODC:-1} HPZ=${HPZ:-0} HSDP=${HSDP:-0}
if [[ "${HSDP}" == "1" ]]; then export ODC_SYMMETRIC_SIZE=${ODC_SYMMETRIC_SIZE:-10G}; else export ODC_SYMMETRIC_SIZE=${ODC_SYMMETRIC_SIZE:-64G}; fi
SCRIPT=train_fsdp2.py
[[ "${FSDP2:-1}" == "0" ]] && SCRIPT=train_fsdp1.py
[[ "${HF:-0}" == "1" ]] && SCRIPT=train_hf.py
cd "$HERE" && exec bash "$ROOT/launch.sh" "$HERE/$SCRIPT" "$@"
