#!/usr/bin/env bash
# Unit tests.  CPU tier always (multi-rank paths run as gloo processes spawned by the tests); the
# GPU tier when a device is visible (multi-GPU tests skip themselves on fewer devices).
set -euo pipefail
cd "$(dirname "$0")/.."
python -m slapo_b200.csrc.build
python -m pytest tests -x -q -m "not gpu"
if python -c "import torch, sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
    python -m pytest tests -x -q -m gpu
fi
