"""Throughput over the number of GPUs of one node, one line per (model, arm), plus the weak-scaling
efficiency table (throughput at N GPUs / (N x throughput at the smallest N)).

    python benchmark/plot/single_node.py results.jsonl|results.tsv [single_node.svg]

Input as for ``single_device.py`` (``bench.py`` lines at 1, 2, 4, 8 GPUs of both arms) or the TSV of
``bench_single_node.py sweep``.  Parity: benchmark/plot/single_node.py of the reference (Fig. 8)."""
from __future__ import annotations

import collections
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import records  # noqa: E402
import svg  # noqa: E402


def collect(rows):
    best = collections.defaultdict(dict)
    for r in rows:
        key = f'{r["model"]} ({r["impl"]})'
        if r["samples_per_sec"] > best[key].get(r["gpus"], 0.0):
            best[key][r["gpus"]] = r["samples_per_sec"]
    return {k: sorted(v.items()) for k, v in best.items() if v}


def efficiency(points):
    n0, t0 = points[0]
    return [(n, t / (t0 / n0 * n)) for n, t in points]


def main(argv):
    if not argv:
        print(__doc__)
        return 1
    data = collect(records.read_records(argv[0]))
    for name, pts in data.items():
        eff = dict(efficiency(pts))
        print(name + ": " + ", ".join(f"{n} GPUs {t:.1f} samples/s (eff {eff[n]:.2f})" for n, t in pts))
    out = argv[1] if len(argv) > 1 else "single_node.svg"
    ticks = sorted({n for pts in data.values() for n, _ in pts})
    svg.line_chart(data, title="one node of B200s, bf16", xlabel="GPUs", ylabel="samples / s", path=out,
                   xticks=ticks)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
