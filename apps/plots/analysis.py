"""Load the ``metrics.jsonl`` files of training runs (with the run's ``config.yaml`` next to them) into
one pandas frame, and draw a metric against the step.

Same frame layout as apps/plots/analysis.py:50-63 of the reference: one row per logged step, columns
``params/<flattened config>`` and ``metrics/<flattened metric>``. Plotting uses plotly when it is installed
and otherwise writes a small self-contained SVG, so the module works on a machine without a graphics stack.

    python -m apps.plots.analysis "runs/**/metrics.jsonl" --y loss/out --out loss.svg
"""
from __future__ import annotations

import argparse
import glob
import json
from pathlib import Path
from typing import Iterable, List, Optional

import pandas as pd

from lingua_b200.config import load_yaml


def load_raw_jsonl(path) -> List[dict]:
    """One dict per line; a line that does not parse is reported and skipped."""
    rows = []
    with open(path) as f:
        for i, line in enumerate(f):
            line = line.strip()
            if not line:
                continue
            try:
                rows.append(json.loads(line))
            except json.JSONDecodeError:
                print(f"Error decoding line {i + 1} in file {path}")
    return rows


def get_metrics(path) -> pd.DataFrame:
    path = Path(path)
    cfg_file = path.parent / "config.yaml"
    params = load_yaml(cfg_file) if cfg_file.exists() else {}
    rows = [{"params": params, "metrics": r} for r in load_raw_jsonl(path)]
    df = pd.json_normalize(rows, sep="/")
    df["run"] = path.parent.name
    return df


def get_merged_df(pattern: str) -> pd.DataFrame:
    files = sorted(glob.glob(pattern, recursive=True))
    if not files:
        raise FileNotFoundError(f"no file matches {pattern!r}")
    return pd.concat([get_metrics(f) for f in files], ignore_index=True)


def _svg_lines(series: Iterable, title: str, logy: bool, width=720, height=420) -> str:
    import math

    series = [(name, [(x, y) for x, y in pts if y == y and (not logy or y > 0)]) for name, pts in series]
    series = [(n, p) for n, p in series if p]
    if not series:
        return f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}"/>'
    fy = (lambda v: math.log10(v)) if logy else (lambda v: v)
    xs = [x for _, p in series for x, _ in p]
    ys = [fy(y) for _, p in series for _, y in p]
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    x1, y1 = (x1 if x1 > x0 else x0 + 1), (y1 if y1 > y0 else y0 + 1)
    L, R, T, B = 60, 20, 30, 40
    sx = lambda x: L + (x - x0) / (x1 - x0) * (width - L - R)
    sy = lambda y: height - B - (fy(y) - y0) / (y1 - y0) * (height - T - B)
    colors = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e", "#8c564b"]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="11">',
           f'<rect width="100%" height="100%" fill="white"/><text x="{width / 2}" y="18" text-anchor="middle">{title}</text>',
           f'<line x1="{L}" y1="{height - B}" x2="{width - R}" y2="{height - B}" stroke="black"/>',
           f'<line x1="{L}" y1="{T}" x2="{L}" y2="{height - B}" stroke="black"/>']
    for k in range(5):
        yv = y0 + (y1 - y0) * k / 4
        label = f"{10 ** yv:.3g}" if logy else f"{yv:.3g}"
        yp = height - B - (height - T - B) * k / 4
        out.append(f'<text x="{L - 5}" y="{yp + 4}" text-anchor="end">{label}</text>')
        xv = x0 + (x1 - x0) * k / 4
        out.append(f'<text x="{L + (width - L - R) * k / 4}" y="{height - B + 15}" text-anchor="middle">{xv:.6g}</text>')
    for i, (name, pts) in enumerate(series):
        d = " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in pts)
        c = colors[i % len(colors)]
        out.append(f'<polyline fill="none" stroke="{c}" stroke-width="1.5" points="{d}"/>')
        out.append(f'<text x="{width - R - 5}" y="{T + 14 * (i + 1)}" text-anchor="end" fill="{c}">{name}</text>')
    out.append("</svg>")
    return "\n".join(out)


def plot_metric(df: pd.DataFrame, y: str = "loss/out", x: str = "global_step", out: Optional[str] = None,
                logy: bool = True) -> str:
    """Line per run of ``metrics/<y>`` over ``metrics/<x>``; returns the path written (html with plotly, else svg)."""
    xc, yc = f"metrics/{x}", f"metrics/{y}"
    d = df.dropna(subset=[xc, yc])
    try:
        import plotly.express as px  # optional

        fig = px.line(d, x=xc, y=yc, color="run")
        if logy:
            fig.update_yaxes(type="log")
        out = out or "metric.html"
        fig.write_html(out)
        return out
    except ImportError:
        series = [(run, list(zip(g[xc].tolist(), g[yc].tolist()))) for run, g in d.groupby("run")]
        out = out or "metric.svg"
        Path(out).write_text(_svg_lines(series, y, logy))
        return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("pattern", help='glob of metrics files, e.g. "dumps/**/metrics.jsonl"')
    ap.add_argument("--y", default="loss/out")
    ap.add_argument("--x", default="global_step")
    ap.add_argument("--out", default=None)
    ap.add_argument("--linear", action="store_true")
    a = ap.parse_args(argv)
    df = get_merged_df(a.pattern)
    print(plot_metric(df, a.y, a.x, a.out, logy=not a.linear))


if __name__ == "__main__":
    main()
