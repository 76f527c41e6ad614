"""A small chart writer that needs nothing but the standard library: grouped bar charts, line
charts and scatter plots as SVG text.  The plotting scripts of this folder use it so that figures
can be produced on a training box that has no matplotlib.

Parity: the figure scripts of the reference (benchmark/plot/*.py) draw with matplotlib; the
charts here carry the same information."""
from __future__ import annotations

PALETTE = ["#4C72B0", "#DD8452", "#55A868", "#C44E52", "#8172B3", "#937860", "#DA8BC3", "#8C8C8C"]


def _esc(text):
    return str(text).replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;")


def _ticks(lo, hi, n=5):
    """About ``n`` round tick values covering [lo, hi] (steps of 1, 2, 2.5 or 5 x 10^k)."""
    import math

    if hi <= lo:
        hi = lo + 1.0
    raw = (hi - lo) / max(n, 1)
    mag = 10.0 ** math.floor(math.log10(raw))
    step = next(m * mag for m in (1, 2, 2.5, 5, 10) if m * mag >= raw)
    v = math.floor(lo / step) * step
    out = []
    while v <= hi + 1e-9 * step:
        if v >= lo - 1e-9 * step:
            out.append(round(v, 10))
        v += step
    return out or [lo, hi]


class Canvas:
    def __init__(self, width=720, height=420, title="", xlabel="", ylabel=""):
        self.w, self.h = width, height
        self.left, self.right, self.top, self.bottom = 70, 20, 40 if title else 20, 60
        self.parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" '
                      f'viewBox="0 0 {width} {height}" font-family="sans-serif" font-size="12">',
                      f'<rect width="{width}" height="{height}" fill="white"/>']
        if title:
            self.text(width / 2, 22, title, size=14, anchor="middle")
        if xlabel:
            self.text(self.left + self.plot_w / 2, height - 12, xlabel, anchor="middle")
        if ylabel:
            mid = self.top + self.plot_h / 2
            self.parts.append(f'<text x="16" y="{mid}" text-anchor="middle" '
                              f'transform="rotate(-90 16 {mid})">{_esc(ylabel)}</text>')

    plot_w = property(lambda self: self.w - self.left - self.right)
    plot_h = property(lambda self: self.h - self.top - self.bottom)

    def text(self, x, y, s, size=12, anchor="start", color="#222"):
        self.parts.append(f'<text x="{x:.1f}" y="{y:.1f}" font-size="{size}" text-anchor="{anchor}" '
                          f'fill="{color}">{_esc(s)}</text>')

    def line(self, x1, y1, x2, y2, color="#222", width=1.0, dash=None):
        d = f' stroke-dasharray="{dash}"' if dash else ""
        self.parts.append(f'<line x1="{x1:.1f}" y1="{y1:.1f}" x2="{x2:.1f}" y2="{y2:.1f}" '
                          f'stroke="{color}" stroke-width="{width}"{d}/>')

    def rect(self, x, y, w, h, color):
        self.parts.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{max(w, 0):.1f}" '
                          f'height="{max(h, 0):.1f}" fill="{color}"/>')

    def circle(self, x, y, r, color):
        self.parts.append(f'<circle cx="{x:.1f}" cy="{y:.1f}" r="{r:.1f}" fill="{color}"/>')

    def polyline(self, pts, color, width=2.0):
        path = " ".join(f"{x:.1f},{y:.1f}" for x, y in pts)
        self.parts.append(f'<polyline points="{path}" fill="none" stroke="{color}" stroke-width="{width}"/>')

    def polygon(self, pts, color, opacity=0.3):
        path = " ".join(f"{x:.1f},{y:.1f}" for x, y in pts)
        self.parts.append(f'<polygon points="{path}" fill="{color}" fill-opacity="{opacity}" '
                          f'stroke="{color}"/>')

    def y_axis(self, lo, hi, fmt="{:g}"):
        ticks = _ticks(lo, hi)
        lo, hi = min(lo, ticks[0]), max(hi, ticks[-1])

        def ymap(v):
            return self.top + self.plot_h * (1 - (v - lo) / (hi - lo))

        for t in ticks:
            self.line(self.left, ymap(t), self.left + self.plot_w, ymap(t), "#ddd")
            self.text(self.left - 6, ymap(t) + 4, fmt.format(t), anchor="end")
        self.line(self.left, self.top, self.left, self.top + self.plot_h)
        return ymap

    def x_axis_numeric(self, lo, hi, ticks=None, fmt="{:g}"):
        ticks = ticks if ticks is not None else _ticks(lo, hi)
        lo, hi = min(lo, ticks[0]), max(hi, ticks[-1])
        if hi <= lo:
            hi = lo + 1

        def xmap(v):
            return self.left + self.plot_w * (v - lo) / (hi - lo)

        base = self.top + self.plot_h
        self.line(self.left, base, self.left + self.plot_w, base)
        for t in ticks:
            self.line(xmap(t), base, xmap(t), base + 4)
            self.text(xmap(t), base + 18, fmt.format(t), anchor="middle")
        return xmap

    def legend(self, labels, colors=None):
        x = self.left + 10
        for i, lab in enumerate(labels):
            color = (colors or PALETTE)[i % len(colors or PALETTE)]
            self.rect(x, self.top + 6 + 16 * i, 10, 10, color)
            self.text(x + 15, self.top + 15 + 16 * i, lab, size=11)

    def render(self):
        return "\n".join(self.parts + ["</svg>"]) + "\n"

    def save(self, path):
        with open(path, "w", encoding="utf-8") as fh:
            fh.write(self.render())
        return path


def bar_chart(groups, series, values, title="", ylabel="", path=None, annotate=True):
    """``values[series_name][group_index]`` (None = missing) as grouped bars."""
    cv = Canvas(title=title, ylabel=ylabel)
    top = max([v for s in series for v in values[s] if v is not None] or [1.0])
    ymap = cv.y_axis(0.0, top * 1.1)
    gw = cv.plot_w / max(len(groups), 1)
    bw = gw * 0.8 / max(len(series), 1)
    base = cv.top + cv.plot_h
    cv.line(cv.left, base, cv.left + cv.plot_w, base)
    for gi, g in enumerate(groups):
        x0 = cv.left + gi * gw + gw * 0.1
        for si, s in enumerate(series):
            v = values[s][gi]
            if v is None:
                cv.text(x0 + si * bw + bw / 2, base - 4, "x", anchor="middle", color="#a00")
                continue
            cv.rect(x0 + si * bw, ymap(v), bw * 0.92, base - ymap(v), PALETTE[si % len(PALETTE)])
            if annotate:
                cv.text(x0 + si * bw + bw / 2, ymap(v) - 3, f"{v:.3g}", size=9, anchor="middle")
        cv.text(cv.left + gi * gw + gw / 2, base + 18, g, anchor="middle")
    cv.legend(series)
    return cv.save(path) if path else cv.render()


def line_chart(xs_by_series, title="", xlabel="", ylabel="", path=None, xticks=None):
    """``xs_by_series[name] = [(x, y), ...]`` as one line per series."""
    cv = Canvas(title=title, xlabel=xlabel, ylabel=ylabel)
    allx = [x for pts in xs_by_series.values() for x, _ in pts] or [0.0, 1.0]
    ally = [y for pts in xs_by_series.values() for _, y in pts] or [0.0, 1.0]
    ymap = cv.y_axis(0.0, max(ally) * 1.1)
    xmap = cv.x_axis_numeric(min(allx), max(allx), ticks=xticks)
    for i, (name, pts) in enumerate(xs_by_series.items()):
        color = PALETTE[i % len(PALETTE)]
        mapped = [(xmap(x), ymap(y)) for x, y in sorted(pts)]
        cv.polyline(mapped, color)
        for x, y in mapped:
            cv.circle(x, y, 3, color)
    cv.legend(list(xs_by_series))
    return cv.save(path) if path else cv.render()
