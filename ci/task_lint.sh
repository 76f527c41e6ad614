#!/usr/bin/env bash
# Static checks (unused imports, line length, stand-alone comments): ci/lint.py over the tree.
set -euo pipefail
cd "$(dirname "$0")/.."
python ci/lint.py
