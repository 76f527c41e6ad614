"""The search space of a tuning configuration as the auto-tuner enumerates it: every valid
(checkpoint ratio, batch size) point and their hull.

    python benchmark/plot/search_space.py examples/bert/tune_cfg.py [polygon.svg] [key=value ...]

``key=value`` pairs are the training-script arguments that the configuration's ``get_bs_range`` /
``is_valid`` read (e.g. ``model_name=bert-large gpus=8``).  Parity: benchmark/plot/search_space.py
of the reference (Fig. 6)."""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import svg  # noqa: E402


def enumerate_space(config_file, script_args):
    from slapo_b200.autotune.tune import CKPT_RATIOS, load_config

    config = load_config(config_file)
    lo, hi, step = config.get_bs_range(script_args)
    is_valid = getattr(config, "is_valid", None)
    pts = []
    for bs in range(lo, hi + 1, step):
        for ratio in CKPT_RATIOS:
            cfg = {"batch_size": bs, "ckpt_ratio": ratio}
            if is_valid is None or is_valid(script_args, cfg):
                pts.append((ratio, bs))
    return pts


def hull(points):
    """Convex hull (monotone chain) of 2-D points."""
    pts = sorted(set(points))
    if len(pts) <= 2:
        return pts

    def cross(o, a, b):
        return (a[0] - o[0]) * (b[1] - o[1]) - (a[1] - o[1]) * (b[0] - o[0])

    lower, upper = [], []
    for p in pts:
        while len(lower) >= 2 and cross(lower[-2], lower[-1], p) <= 0:
            lower.pop()
        lower.append(p)
    for p in reversed(pts):
        while len(upper) >= 2 and cross(upper[-2], upper[-1], p) <= 0:
            upper.pop()
        upper.append(p)
    return lower[:-1] + upper[:-1]


def main(argv):
    if not argv:
        print(__doc__)
        return 1
    out = "polygon.svg"
    script_args = {}
    for a in argv[1:]:
        if "=" in a:
            k, v = a.split("=", 1)
            script_args[k] = int(v) if v.isdigit() else v
        else:
            out = a
    pts = enumerate_space(argv[0], script_args)
    print(f"{len(pts)} points")
    cv = svg.Canvas(title="search space", xlabel="checkpoint ratio", ylabel="batch size")
    ymap = cv.y_axis(0.0, max([b for _, b in pts] or [1]) * 1.1)
    xmap = cv.x_axis_numeric(0.0, 1.0)
    if len(pts) > 2:
        cv.polygon([(xmap(x), ymap(y)) for x, y in hull(pts)], svg.PALETTE[0])
    for x, y in pts:
        cv.circle(xmap(x), ymap(y), 2.5, svg.PALETTE[0])
    cv.save(out)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
