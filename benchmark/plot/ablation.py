"""Ablation: throughput of one model / layout as optimisations are switched on one by one
(horizontal order = order of the input lines).

    python benchmark/plot/ablation.py ablation.jsonl [ablation.svg]

Every input line is a benchmark record (see ``single_device.py``) with an extra ``"label"`` key
naming the variant, e.g. the ``bench.py`` line of a run with ``SLAPO_B200_LIBRARY_GEMM=1`` labelled
"library GEMM".  Parity: benchmark/plot/ablation.py of the reference (Fig. 10)."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import records  # noqa: E402
import svg  # noqa: E402


def main(argv):
    if not argv:
        print(__doc__)
        return 1
    rows = [r for r in records.read_records(argv[0]) if r["samples_per_sec"] > 0]
    labels = [r["label"] or f'{r["impl"]} {r["layout"]}' for r in rows]
    base = rows[0]["samples_per_sec"] if rows else 1.0
    for lab, r in zip(labels, rows):
        print(f'{lab}: {r["samples_per_sec"]:.1f} samples/s ({r["samples_per_sec"] / base:.2f} x)')
    out = argv[1] if len(argv) > 1 else "ablation.svg"
    title = f'{rows[0]["model"]}, {rows[0]["gpus"]} GPUs' if rows else ""
    svg.bar_chart(labels, ["samples / s"], {"samples / s": [r["samples_per_sec"] for r in rows]},
                  title=title, ylabel="samples / s", path=out)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
