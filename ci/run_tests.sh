#!/usr/bin/env bash
# Build the native extension and run the test suite.
#   ci/run_tests.sh          CPU tests (gloo ranks spawned by the tests themselves)
#   ci/run_tests.sh gpu      GPU tests on the visible B200(s)
#   ci/run_tests.sh lint     static checks only (ci/lint.py)
set -euo pipefail
cd "$(dirname "$0")/.."
if [ "${1:-cpu}" = "lint" ]; then
    exec python ci/lint.py
fi
python ci/lint.py
python -m slapo_b200.csrc.build
if [ "${1:-cpu}" = "gpu" ]; then
    python -m pytest tests -x -q -m gpu
else
    python -m pytest tests -x -q -m "not gpu"
fi
