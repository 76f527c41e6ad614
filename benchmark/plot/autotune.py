"""The auto-tuner's walk through (checkpoint ratio, batch size): every evaluated point with its
throughput (circle area), failed points (out of memory) as crosses, the visiting order as a line
and the best point marked.

    python benchmark/plot/autotune.py tune_db.json [autotune.svg]

``tune_db.json`` is what ``python -m slapo_b200.autotune.tune --db tune_db.json ...`` writes.
Parity: benchmark/plot/autotune.py of the reference (Fig. 11)."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import records  # noqa: E402
import svg  # noqa: E402


def draw(points, path):
    cv = svg.Canvas(title="auto-tuning trace", xlabel="checkpoint ratio", ylabel="batch size")
    xs = [c.get("ckpt_ratio", 0.0) for c, _, _ in points] or [0.0, 1.0]
    ys = [c.get("batch_size", 0) for c, _, _ in points] or [0, 1]
    ymap = cv.y_axis(0.0, max(ys) * 1.1)
    xmap = cv.x_axis_numeric(min(xs + [0.0]), max(xs + [1.0]))
    top = max([t for _, t, _ in points] or [1.0]) or 1.0
    mapped = [(xmap(c.get("ckpt_ratio", 0.0)), ymap(c.get("batch_size", 0))) for c, _, _ in points]
    if len(mapped) > 1:
        cv.polyline(mapped, "#bbb", 1.0)
    best = max(range(len(points)), key=lambda i: points[i][1]) if points else None
    for i, ((x, y), (_, thr, code)) in enumerate(zip(mapped, points)):
        if code != 0 or thr <= 0:
            cv.line(x - 4, y - 4, x + 4, y + 4, "#a00", 1.5)
            cv.line(x - 4, y + 4, x + 4, y - 4, "#a00", 1.5)
        else:
            cv.circle(x, y, 3 + 9 * (thr / top) ** 0.5, svg.PALETTE[2 if i == best else 0])
            cv.text(x + 8, y - 8, f"{thr:.0f}", size=9)
    return cv.save(path) if path else cv.render()


def main(argv):
    if not argv:
        print(__doc__)
        return 1
    points = records.read_tuner_db(argv[0])
    for cfg, thr, code in points:
        print(cfg, f"{thr:.1f} samples/s" if code == 0 and thr > 0 else "failed")
    out = argv[1] if len(argv) > 1 else "autotune.svg"
    draw(points, out)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
