"""Figures of benchmark results without a plotting library: a figure is a list of panels, a panel holds line and
bar series, and ``save_figure`` writes one self-contained SVG (text, so it diffs and needs no display). Series
colours come from a ``Palette`` that keeps one colour per name across figures, so "ours" is the same blue in
the scaling plot and in the kernel plot.

    python -m kohakuwullm_b200.bench.plotting results/ --out results/throughput.svg
    python -m kohakuwullm_b200.bench.plotting results/ --scaling --out results/scaling.svg

    python -m kohakuwullm_b200.bench.plotting out/sweep --metrics train/loss throughput/tokens_per_s --out out/sweep/curves.svg

The command reads the result files ``bench.sweep.load_rows`` reads (one JSON line per run) and draws either bars of
the metric per file or, with ``--scaling``, the metric over the number of GPUs with the ideal line of the smallest
run; with ``--metrics`` it reads the per-step ``*.jsonl`` files of the trainers' JSONL sink instead and draws one panel
per metric with one line per run. Reference: src/kohakuwullm/bench/core/plotting.py:1-134 (matplotlib styling helpers for its bench scripts).
"""

from __future__ import annotations

import argparse
import math
import os
import sys
from dataclasses import dataclass, field
from xml.sax.saxutils import escape

# Okabe-Ito colour-blind-safe ramp
CATEGORICAL = ("#0072B2", "#D55E00", "#009E73", "#CC79A7", "#E69F00", "#56B4E9", "#F0E442", "#7F7F7F")

PANEL_W, PANEL_H = 520, 360
MARGIN_L, MARGIN_R, MARGIN_T, MARGIN_B = 64, 16, 34, 52


class Palette:
    """Name -> colour, assigned in order of first use and stable afterwards."""

    def __init__(self, colors=CATEGORICAL) -> None:
        self.colors = tuple(colors)
        self.assigned: dict[str, str] = {}

    def color(self, key: str) -> str:
        if key not in self.assigned:
            self.assigned[key] = self.colors[len(self.assigned) % len(self.colors)]
        return self.assigned[key]


def si_format(value: float) -> str:
    """1536 -> ``1.5k``, 2e6 -> ``2M``; fractions keep their digits (0.25 -> ``0.25``)."""
    for unit, scale in (("T", 1e12), ("G", 1e9), ("M", 1e6), ("k", 1e3)):
        if abs(value) >= scale:
            return f"{value / scale:.1f}".rstrip("0").rstrip(".") + unit
    return f"{value:.4g}"      # 7 -> "7", 0.25 -> "0.25", 11.145 -> "11.14" (tick labels of a flat curve must differ)


def nice_ticks(lo: float, hi: float, count: int = 5) -> list[float]:
    """Round tick values (1, 2 or 5 times a power of ten apart) covering ``[lo, hi]``."""
    if not math.isfinite(lo) or not math.isfinite(hi):
        return [0.0, 1.0]
    if hi <= lo:
        hi = lo + (abs(lo) if lo else 1.0)
    raw = (hi - lo) / max(count, 1)
    mag = 10.0 ** math.floor(math.log10(raw))
    step = next(s * mag for s in (1, 2, 5, 10) if s * mag >= raw)
    first = math.floor(lo / step) * step
    ticks, t = [], first
    while t < hi + 0.5 * step:
        ticks.append(round(t, 12))
        t += step
    return ticks


def log_ticks(lo: float, hi: float, base: float) -> list[float]:
    lo, hi = max(lo, 1e-300), max(hi, 1e-300)
    a, b = math.floor(math.log(lo, base) + 1e-9), math.ceil(math.log(hi, base) - 1e-9)
    return [base ** e for e in range(a, max(b, a + 1) + 1)]


@dataclass
class Series:
    kind: str                 # "line" | "bar"
    name: str
    xs: list
    ys: list
    color: str
    dashed: bool = False
    labels: bool = False      # print each bar's value above it


@dataclass
class Panel:
    title: str = ""
    xlabel: str = ""
    ylabel: str = ""
    logx: bool = False        # base 2, as sizes and GPU counts double
    logy: bool = False        # base 10
    legend: bool = True
    label_format: str = "{:.0f}"
    series: list = field(default_factory=list)

    def line(self, name: str, xs, ys, color: str, dashed: bool = False) -> None:
        self.series.append(Series("line", name, list(xs), list(ys), color, dashed))

    def bars(self, name: str, categories, ys, color: str, labels: bool = True) -> None:
        self.series.append(Series("bar", name, [str(c) for c in categories], list(ys), color, labels=labels))

    # -- drawing --------------------------------------------------------------------------------------------------

    def _scale(self, lo: float, hi: float, log: bool, base: float, px0: float, px1: float):
        if log:
            tf = lambda v: math.log(max(v, 1e-300), base)
            lo, hi = tf(lo), tf(hi)
        else:
            tf = lambda v: v
        span = (hi - lo) or 1.0
        return lambda v: px0 + (tf(v) - lo) / span * (px1 - px0)

    def render(self, ox: float, oy: float) -> list[str]:
        x0, x1 = ox + MARGIN_L, ox + PANEL_W - MARGIN_R
        y0, y1 = oy + PANEL_H - MARGIN_B, oy + MARGIN_T          # y0 is the bottom edge in pixels
        out = [f'<rect x="{x0:.1f}" y="{y1:.1f}" width="{x1 - x0:.1f}" height="{y0 - y1:.1f}" fill="white" '
               f'stroke="#333333" stroke-width="0.8"/>']
        if self.title:
            out.append(f'<text x="{(x0 + x1) / 2:.1f}" y="{oy + 20:.1f}" text-anchor="middle" font-weight="bold" '
                       f'font-size="13">{escape(self.title)}</text>')
        out.append(f'<text x="{(x0 + x1) / 2:.1f}" y="{oy + PANEL_H - 10:.1f}" text-anchor="middle">'
                   f'{escape(self.xlabel)}</text>')
        out.append(f'<text transform="translate({ox + 14:.1f},{(y0 + y1) / 2:.1f}) rotate(-90)" text-anchor="middle">'
                   f'{escape(self.ylabel)}</text>')
        bars = [s for s in self.series if s.kind == "bar"]
        lines = [s for s in self.series if s.kind == "line"]
        values = [y for s in self.series for y in s.ys if y is not None and math.isfinite(y)]
        if not values:
            out.append(f'<text x="{(x0 + x1) / 2:.1f}" y="{(y0 + y1) / 2:.1f}" text-anchor="middle" '
                       f'fill="#7F7F7F">no data</text>')
            return out
        positive = [v for v in values if v > 0]
        if self.logy and positive:
            yticks = log_ticks(min(positive), max(positive), 10.0)
        else:
            yticks = nice_ticks(min(0.0, min(values)) if bars else min(values), max(values))
        sy = self._scale(yticks[0], yticks[-1], self.logy and bool(positive), 10.0, y0, y1)
        for t in yticks:
            py = sy(t)
            out.append(f'<line x1="{x0:.1f}" x2="{x1:.1f}" y1="{py:.1f}" y2="{py:.1f}" stroke="#DDDDDD" '
                       f'stroke-width="0.6"/>')
            out.append(f'<text x="{x0 - 6:.1f}" y="{py + 3.5:.1f}" text-anchor="end" font-size="10">'
                       f'{si_format(t)}</text>')
        if bars:
            cats: list[str] = []
            for s in bars:
                cats += [c for c in s.xs if c not in cats]
            slot = (x1 - x0) / max(len(cats), 1)
            width = slot * 0.8 / len(bars)
            base_px = sy(max(yticks[0], 0.0) if not self.logy else yticks[0])
            for ci, c in enumerate(cats):
                cx = x0 + slot * (ci + 0.5)
                out.append(f'<text x="{cx:.1f}" y="{y0 + 14:.1f}" text-anchor="middle" font-size="10">'
                           f'{escape(c)}</text>')
                for bi, s in enumerate(bars):
                    if c not in s.xs:
                        continue                      # a configuration that was not run leaves a gap, not a zero
                    v = s.ys[s.xs.index(c)]
                    if v is None or not math.isfinite(v):
                        continue
                    bx = cx - slot * 0.4 + bi * width
                    top = sy(v)
                    out.append(f'<rect x="{bx:.1f}" y="{min(top, base_px):.1f}" width="{width:.1f}" '
                               f'height="{abs(base_px - top):.1f}" fill="{s.color}"><title>{escape(s.name)}: '
                               f'{v:g}</title></rect>')
                    if s.labels:
                        out.append(f'<text x="{bx + width / 2:.1f}" y="{top - 3:.1f}" text-anchor="middle" '
                                   f'font-size="9">{escape(self.label_format.format(v))}</text>')
        if lines:
            xs_all = [x for s in lines for x in s.xs]
            if self.logx:
                xticks = log_ticks(min(xs_all), max(xs_all), 2.0)
            else:
                xticks = nice_ticks(min(xs_all), max(xs_all))
            sx = self._scale(xticks[0], xticks[-1], self.logx, 2.0, x0, x1)
            if not bars:
                for t in xticks:
                    px = sx(t)
                    out.append(f'<line x1="{px:.1f}" x2="{px:.1f}" y1="{y0:.1f}" y2="{y1:.1f}" stroke="#DDDDDD" '
                               f'stroke-width="0.6"/>')
                    out.append(f'<text x="{px:.1f}" y="{y0 + 14:.1f}" text-anchor="middle" font-size="10">'
                               f'{si_format(t)}</text>')
            for s in lines:
                pts = [(sx(x), sy(y)) for x, y in zip(s.xs, s.ys) if y is not None and math.isfinite(y)
                       and (not self.logy or y > 0)]
                if not pts:
                    continue
                path = " ".join(f"{px:.1f},{py:.1f}" for px, py in pts)
                dash = ' stroke-dasharray="5,4"' if s.dashed else ""
                out.append(f'<polyline points="{path}" fill="none" stroke="{s.color}" stroke-width="1.8"{dash}/>')
                if not s.dashed:
                    out += [f'<circle cx="{px:.1f}" cy="{py:.1f}" r="2.6" fill="{s.color}"/>' for px, py in pts]
        if self.legend and len(self.series) > 1:
            for i, s in enumerate(self.series):
                ly = y1 + 12 + 14 * i
                out.append(f'<rect x="{x0 + 8:.1f}" y="{ly - 8:.1f}" width="10" height="10" fill="{s.color}"/>')
                out.append(f'<text x="{x0 + 22:.1f}" y="{ly + 1:.1f}" font-size="10">{escape(s.name)}</text>')
        return out


class Figure:
    """``rows x cols`` panels; ``panels`` is always a flat list, row by row."""

    def __init__(self, rows: int = 1, cols: int = 1) -> None:
        self.rows, self.cols = rows, cols
        self.panels = [Panel() for _ in range(rows * cols)]

    def svg(self) -> str:
        w, h = self.cols * PANEL_W, self.rows * PANEL_H
        body = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" viewBox="0 0 {w} {h}" '
                f'font-family="sans-serif" font-size="11">', f'<rect width="{w}" height="{h}" fill="white"/>']
        for i, panel in enumerate(self.panels):
            body += panel.render((i % self.cols) * PANEL_W, (i // self.cols) * PANEL_H)
        body.append("</svg>")
        return "\n".join(body) + "\n"


def save_figure(fig: Figure, path: str) -> str:
    """Writes the SVG (the extension is replaced by ``.svg``) through a temporary file and returns its path."""
    path = os.path.splitext(path)[0] + ".svg"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w") as fh:
        fh.write(fig.svg())
    os.replace(tmp, path)
    return path


# -- figures of result rows ---------------------------------------------------------------------------------------

def _series_name(row: dict) -> str:
    model = row.get("preset") or (row.get("config") or {}).get("model", "?")
    return f"{model} ({row.get('impl', 'ours')})"


def throughput_figure(rows: list[dict], key: str = "value", palette: Palette | None = None) -> Figure:
    """One bar per clean result file; contended and out-of-memory rows are left out (they are not measurements)."""
    palette = palette or Palette()
    fig = Figure()
    p = fig.panels[0]
    p.title, p.xlabel, p.ylabel, p.label_format = "throughput", "run", key, "{:,.0f}"
    by_name: dict[str, tuple[list, list]] = {}
    for r in rows:
        v = r.get(key, r.get("tokens_per_s"))
        if r.get("status", "clean") != "clean" or not isinstance(v, (int, float)):
            continue
        cats, ys = by_name.setdefault(_series_name(r), ([], []))
        cats.append(os.path.splitext(r.get("file", f"run{len(cats)}"))[0])
        ys.append(float(v))
    for name, (cats, ys) in by_name.items():
        p.bars(name, cats, ys, palette.color(name))
    return fig


def scaling_figure(rows: list[dict], key: str = "value", palette: Palette | None = None) -> Figure:
    """Metric over GPU count per (model, implementation), with the ideal line through each series' smallest run,
    and beside it the efficiency relative to that line."""
    palette = palette or Palette()
    fig = Figure(1, 2)
    left, right = fig.panels
    left.title, left.xlabel, left.ylabel, left.logx, left.logy = "scaling", "GPUs", key, True, True
    right.title, right.xlabel, right.ylabel, right.logx = "efficiency vs smallest run", "GPUs", "fraction", True
    groups: dict[str, dict[int, float]] = {}
    for r in rows:
        v, n = r.get(key, r.get("tokens_per_s")), r.get("n_gpus")
        if r.get("status", "clean") != "clean" or not isinstance(v, (int, float)) or not isinstance(n, int):
            continue
        best = groups.setdefault(_series_name(r), {})
        best[n] = max(best.get(n, 0.0), float(v))
    for name, by_n in groups.items():
        ns = sorted(by_n)
        color = palette.color(name)
        left.line(name, ns, [by_n[n] for n in ns], color)
        left.line(name + " ideal", ns, [by_n[ns[0]] * n / ns[0] for n in ns], color, dashed=True)
        right.line(name, ns, [by_n[n] / (by_n[ns[0]] * n / ns[0]) for n in ns], color)
    return fig


def load_metric_curves(directory: str, pattern: str = "*.jsonl") -> dict[str, dict[str, tuple[list, list]]]:
    """``{file stem: {metric: (steps, values)}}`` from the per-step metric files a ``JsonlReporter`` writes (one JSON
    object per report with a ``step`` and any number of scalar metrics)."""
    import glob
    import json

    runs: dict[str, dict[str, tuple[list, list]]] = {}
    for path in sorted(glob.glob(os.path.join(directory, pattern))):
        curves: dict[str, tuple[list, list]] = {}
        with open(path) as fh:
            for line in fh:
                try:
                    row = json.loads(line)
                except ValueError:
                    continue                      # a line cut short by a killed run
                step = row.get("step")
                if not isinstance(step, int):
                    continue
                for k, v in row.items():
                    if k not in ("step", "t") and isinstance(v, (int, float)) and math.isfinite(v):
                        xs, ys = curves.setdefault(k, ([], []))
                        xs.append(step)
                        ys.append(float(v))
        if curves:
            runs[os.path.splitext(os.path.basename(path))[0]] = curves
    return runs


def curves_figure(runs: dict, metrics: list[str], palette: Palette | None = None, logy: bool = False) -> Figure:
    """One panel per metric, one line per run: loss and throughput of the points of a sweep side by side."""
    palette = palette or Palette()
    fig = Figure(1, max(len(metrics), 1))
    for panel, metric in zip(fig.panels, metrics):
        panel.title, panel.xlabel, panel.ylabel, panel.logy = metric, "step", metric.split("/")[-1], logy
        for run, curves in runs.items():
            if metric in curves:
                panel.line(run, curves[metric][0], curves[metric][1], palette.color(run))
    return fig


def main(argv=None) -> int:
    from kohakuwullm_b200.bench.sweep import load_rows

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("directory")
    ap.add_argument("--pattern", default="*.json")
    ap.add_argument("--key", default="value")
    ap.add_argument("--scaling", action="store_true")
    ap.add_argument("--metrics", nargs="+", help="plot these per-step metrics of *.jsonl metric files, one panel each")
    ap.add_argument("--logy", action="store_true")
    ap.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    if args.metrics:
        runs = load_metric_curves(args.directory, args.pattern if args.pattern != "*.json" else "*.jsonl")
        print(f"wrote {save_figure(curves_figure(runs, args.metrics, logy=args.logy), args.out)} from {len(runs)} runs")
        return 0
    rows = load_rows(args.directory, args.pattern)
    fig = (scaling_figure if args.scaling else throughput_figure)(rows, args.key)
    print(f"wrote {save_figure(fig, args.out)} from {len(rows)} rows")
    return 0


if __name__ == "__main__":
    sys.exit(main())
