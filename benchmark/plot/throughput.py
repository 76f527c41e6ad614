"""Plot the TSV written by ``bench_single_node.py sweep``: throughput per model over the GPU
count, one line per layout (matplotlib optional: without it the table is printed).

    python benchmark/plot/throughput.py results.tsv [out.png]
"""
from __future__ import annotations

import collections
import sys


def read(path):
    rows = []
    with open(path, encoding="utf-8") as fh:
        header = fh.readline().rstrip("\n").split("\t")
        for line in fh:
            cells = line.rstrip("\n").split("\t")
            if len(cells) == len(header):
                rows.append(dict(zip(header, cells)))
    return rows


def series(rows):
    out = collections.defaultdict(list)
    for r in rows:
        try:
            thr = float(r["samples_per_sec"])
        except ValueError:          # "oom" / "fail"
            continue
        out[r["model"]].append((int(r["gpus"]), thr, r["layout"]))
    return {m: sorted(v) for m, v in out.items()}


def main(argv):
    if not argv:
        print(__doc__)
        return 1
    data = series(read(argv[0]))
    for model, pts in data.items():
        base = pts[0][1] / pts[0][0]
        print(model)
        for n, thr, layout in pts:
            print(f"  {n} GPUs  {layout:12s} {thr:10.1f} samples/s  scaling {thr / (base * n):.2f}")
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return 0
    fig, ax = plt.subplots(figsize=(6, 4))
    for model, pts in data.items():
        ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", label=model)
    ax.set_xlabel("GPUs")
    ax.set_ylabel("samples / s")
    ax.set_xscale("log", base=2)
    ax.legend(fontsize=7)
    fig.tight_layout()
    fig.savefig(argv[1] if len(argv) > 1 else "throughput.png", dpi=150)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
