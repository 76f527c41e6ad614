#!/usr/bin/env bash
# Container entry point: report the environment, then run the given command from the repo root.
set -euo pipefail
cd "$(dirname "$0")/.."
python benchmark/bench_single_node.py env || true
exec "$@"
