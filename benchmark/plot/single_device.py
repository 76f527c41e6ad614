"""Single-GPU throughput per model, this framework against the reference arm (grouped bars).

    python benchmark/plot/single_device.py results.jsonl [single_device.svg]

``results.jsonl``: one JSON object per line - the lines printed by ``bench.py`` (both ``--impl``
arms, any ``--model``) and / or by ``python -m slapo_b200.bench.train``; rows of more than one GPU
are ignored.  Parity: benchmark/plot/single_device.py of the reference (Fig. 7 of its paper)."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import records  # noqa: E402
import svg  # noqa: E402


def collect(rows):
    rows = [r for r in rows if r["gpus"] == 1]
    models = sorted({r["model"] for r in rows})
    impls = sorted({r["impl"] for r in rows})
    values = {i: [None] * len(models) for i in impls}
    for r in rows:      # the best run of a (model, impl) pair
        cur = values[r["impl"]][models.index(r["model"])]
        if r["samples_per_sec"] > 0 and (cur is None or r["samples_per_sec"] > cur):
            values[r["impl"]][models.index(r["model"])] = r["samples_per_sec"]
    return models, impls, values


def main(argv):
    if not argv:
        print(__doc__)
        return 1
    models, impls, values = collect(records.read_records(argv[0]))
    for m_i, model in enumerate(models):
        cells = ", ".join(f"{i} {values[i][m_i]:.1f}" for i in impls if values[i][m_i] is not None)
        print(f"{model}: {cells}")
    out = argv[1] if len(argv) > 1 else "single_device.svg"
    svg.bar_chart(models, impls, values, title="one B200, bf16", ylabel="samples / s", path=out)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
