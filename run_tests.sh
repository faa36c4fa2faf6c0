#!/usr/bin/env bash
# Build the extension, then run the CPU tests and (when a GPU is visible) the GPU tests.
set -euo pipefail
cd "$(dirname "$0")"
python -m odc_b200.build
python -m pytest tests -q -m "not gpu" "$@"
if python -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  python -m pytest tests -q -m gpu "$@"
fi
