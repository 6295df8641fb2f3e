"""Figures from benchmark results, written as stand-alone SVG (no plotting library needed).

The reference draws its figures with matplotlib / seaborn (benchmark/plotting/
plot_microbenchmark_results.py:380-399 grouped bars of ms per batch per framework,
plot_e2e_results.py iteration-time bars, plot_loss_curve.py overlaid loss curves,
plot_dryrun_results.py communication volume and imbalance against block size).  The same four
figures are produced here from the tables that ``run_experiments`` / ``dry_run`` / ``parse_logs``
write:

    python -m dcp_b200.bench.plotting microbench results/summary.csv --out microbench.svg
    python -m dcp_b200.bench.plotting e2e results/summary.csv --out e2e.svg
    python -m dcp_b200.bench.plotting loss run_a.log run_b.log --out loss.svg
    python -m dcp_b200.bench.plotting dryrun dry.json --metric modelled_pipeline_ms --out dryrun.svg
"""
from __future__ import annotations

import argparse
import csv
import json
import math
from typing import Dict, List, Sequence, Tuple
from xml.sax.saxutils import escape

from .parse_logs import parse_loss_curve

PALETTE = ["#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#76b7b2", "#edc948", "#b07aa1", "#9c755f"]
W, H, ML, MR, MT, MB = 760, 420, 70, 150, 40, 70          # canvas and margins


def _nice_ticks(lo: float, hi: float, n: int = 5) -> List[float]:
    if hi <= lo:
        hi = lo + 1.0
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m for m in (1, 2, 2.5, 5, 10) if m * mag >= raw), default=10) * mag
    start = math.floor(lo / step) * step
    ticks, t = [], start
    while t <= hi + 1e-9 * step:
        ticks.append(round(t, 10))
        t += step
    if ticks[-1] < hi:
        ticks.append(round(ticks[-1] + step, 10))
    return ticks


def _frame(title: str, ylabel: str, xlabel: str, ticks: Sequence[float], y_of) -> List[str]:
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="12">',
           f'<rect width="{W}" height="{H}" fill="white"/>',
           f'<text x="{W / 2}" y="20" text-anchor="middle" font-size="15">{escape(title)}</text>',
           f'<text x="16" y="{(MT + H - MB) / 2}" text-anchor="middle" transform="rotate(-90 16 {(MT + H - MB) / 2})">'
           f'{escape(ylabel)}</text>',
           f'<text x="{(ML + W - MR) / 2}" y="{H - 12}" text-anchor="middle">{escape(xlabel)}</text>']
    for t in ticks:
        y = y_of(t)
        out.append(f'<line x1="{ML}" y1="{y:.1f}" x2="{W - MR}" y2="{y:.1f}" stroke="#dddddd"/>')
        out.append(f'<text x="{ML - 6}" y="{y + 4:.1f}" text-anchor="end">{t:g}</text>')
    out.append(f'<line x1="{ML}" y1="{MT}" x2="{ML}" y2="{H - MB}" stroke="black"/>')
    out.append(f'<line x1="{ML}" y1="{H - MB}" x2="{W - MR}" y2="{H - MB}" stroke="black"/>')
    return out


def _legend(names: Sequence[str]) -> List[str]:
    out = []
    for i, n in enumerate(names):
        y = MT + 10 + 18 * i
        out.append(f'<rect x="{W - MR + 12}" y="{y - 9}" width="12" height="12" fill="{PALETTE[i % len(PALETTE)]}"/>')
        out.append(f'<text x="{W - MR + 30}" y="{y + 1}">{escape(str(n))}</text>')
    return out


def bar_chart_svg(groups: Dict[str, Dict[str, float]], title: str, ylabel: str, xlabel: str = "") -> str:
    """Grouped bars: ``groups[group][series] = value`` (missing combinations leave a gap)."""
    series = sorted({s for g in groups.values() for s in g})
    top = max([v for g in groups.values() for v in g.values() if v is not None] + [1e-9])
    ticks = _nice_ticks(0.0, top)
    y_of = lambda v: H - MB - (v - ticks[0]) / (ticks[-1] - ticks[0]) * (H - MB - MT)
    out = _frame(title, ylabel, xlabel, ticks, y_of)
    gw = (W - ML - MR) / max(len(groups), 1)
    bw = gw * 0.8 / max(len(series), 1)
    for gi, (gname, vals) in enumerate(groups.items()):
        x0 = ML + gi * gw + gw * 0.1
        for si, sname in enumerate(series):
            v = vals.get(sname)
            if v is None:
                continue
            y = y_of(v)
            out.append(f'<rect class="bar" x="{x0 + si * bw:.1f}" y="{y:.1f}" width="{bw * 0.92:.1f}" '
                       f'height="{H - MB - y:.1f}" fill="{PALETTE[si % len(PALETTE)]}"><title>{escape(gname)} / '
                       f'{escape(sname)}: {v:g}</title></rect>')
        out.append(f'<text x="{ML + gi * gw + gw / 2:.1f}" y="{H - MB + 16}" text-anchor="middle">{escape(str(gname))}</text>')
    return "\n".join(out + _legend(series) + ["</svg>"])


def line_chart_svg(series: Dict[str, Sequence[Tuple[float, float]]], title: str, ylabel: str, xlabel: str = "") -> str:
    """One polyline per series of (x, y) points."""
    pts = [p for s in series.values() for p in s]
    xs, ys = [p[0] for p in pts] or [0.0], [p[1] for p in pts] or [0.0]
    xt, yt = _nice_ticks(min(xs), max(xs)), _nice_ticks(min(min(ys), 0.0) if min(ys) >= 0 else min(ys), max(ys))
    x_of = lambda v: ML + (v - xt[0]) / (xt[-1] - xt[0]) * (W - ML - MR)
    y_of = lambda v: H - MB - (v - yt[0]) / (yt[-1] - yt[0]) * (H - MB - MT)
    out = _frame(title, ylabel, xlabel, yt, y_of)
    for t in xt:
        out.append(f'<text x="{x_of(t):.1f}" y="{H - MB + 16}" text-anchor="middle">{t:g}</text>')
    for i, (name, s) in enumerate(series.items()):
        path = " ".join(f"{x_of(x):.1f},{y_of(y):.1f}" for x, y in s)
        out.append(f'<polyline class="line" fill="none" stroke="{PALETTE[i % len(PALETTE)]}" stroke-width="2" points="{path}"/>')
    return "\n".join(out + _legend(list(series)) + ["</svg>"])


def _rows(path: str) -> List[dict]:
    if path.endswith(".json"):
        data = json.load(open(path))
        return data["cells"] if isinstance(data, dict) and "cells" in data else data
    return list(csv.DictReader(open(path)))


def _num(v):
    try:
        return float(v)
    except (TypeError, ValueError):
        return None


def microbench_figure(rows: Sequence[dict]) -> str:
    """ms per batch: one group per (mask, length distribution), one bar per framework."""
    groups: Dict[str, Dict[str, float]] = {}
    for r in rows:
        if r.get("kind", "attention") != "attention" or r.get("status", "ok") != "ok":
            continue
        vals = [_num(v) for k, v in r.items() if k.startswith("ms_per_batch_") and _num(v) is not None]
        if vals:
            g = groups.setdefault(f"{r.get('mask', '')} / {r.get('length_dist', '')}", {})
            name = f"{r.get('framework', 'dcp')} bs{r.get('block_size', '')}" if r.get("framework") == "dcp" else r["framework"]
            g[name] = min(g.get(name, float("inf")), sum(vals))
    return bar_chart_svg(groups, "Attention forward + backward", "ms per batch (max over ranks)")


def e2e_figure(rows: Sequence[dict]) -> str:
    groups: Dict[str, Dict[str, float]] = {}
    for r in rows:
        v = _num(r.get("ms_per_iteration"))
        if r.get("kind") == "train" and v is not None:
            groups.setdefault(f"{r.get('mask', '')} / {r.get('length_dist', '')}", {})[f"bs{r.get('block_size', '')}"] = v
    return bar_chart_svg(groups, "Training iteration time", "ms per iteration")


def loss_figure(logs: Dict[str, str]) -> str:
    return line_chart_svg({name: list(enumerate(parse_loss_curve(text))) for name, text in logs.items()},
                          "Training loss", "loss", "iteration")


def dryrun_figure(rows: Sequence[dict], metric: str = "modelled_pipeline_ms") -> str:
    """``metric`` against block size, one line per (mask, length distribution, stages)."""
    series: Dict[str, List[Tuple[float, float]]] = {}
    for r in rows:
        v, b = _num(r.get(metric)), _num(r.get("block_size"))
        if v is not None and b is not None:
            series.setdefault(f"{r.get('mask', '')} {r.get('length_dist', '')} s{r.get('n_stages', '')}", []).append((b, v))
    return line_chart_svg({k: sorted(v) for k, v in series.items()}, f"Planner dry run: {metric}", metric, "block size")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("figure", choices=["microbench", "e2e", "loss", "dryrun"])
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("--metric", default="modelled_pipeline_ms")
    ap.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    if args.figure == "loss":
        svg = loss_figure({p: open(p).read() for p in args.inputs})
    else:
        rows = [r for p in args.inputs for r in _rows(p)]
        svg = {"microbench": microbench_figure, "e2e": e2e_figure}[args.figure](rows) if args.figure != "dryrun" \
            else dryrun_figure(rows, args.metric)
    with open(args.out, "w") as f:
        f.write(svg)


if __name__ == "__main__":
    main()
