"""Animate probe statistics over depth and training time as one standalone HTML page.

Input: folders of probe dumps written by ``lingua_b200.probe.AutoProbeD`` (one JSON object per line:
``{"data": {"<module path>::<what>": {"mean", "std", "quantiles", ...}}, "meta": {...}, "quantiles": [...]}``), one folder
per run. For each requested tensor-name pattern (``layers.{}.attention.wq::out``-style, ``{}`` is
the layer index) the page shows the quantile bands of that tensor at every depth and steps through the
dumps in time. This is what apps/plots/probe_animation.py:134-192 of the reference renders with matplotlib;
here the page is drawn by a few lines of inline JavaScript on an SVG, so neither matplotlib nor a display
is needed.

    python -m apps.plots.probe_animation dump/probe --pattern "layers.{}.attention.wo::out" --out probe.html
"""
from __future__ import annotations

import argparse
import json
import re
from pathlib import Path
from typing import Dict, List, Sequence


def load_probe_folder(folder) -> List[dict]:
    """All dumps of one run, ordered by global step (falls back to file order)."""
    rows = []
    for f in sorted(Path(folder).glob("*.json*")):
        for line in f.read_text().splitlines():
            line = line.strip()
            if line:
                rows.append(json.loads(line))
    rows.sort(key=lambda r: (r.get("meta") or {}).get("global_step", 0))
    return rows


def num_layers(dump: dict) -> int:
    idx = [int(m.group(1)) for k in dump["data"] for m in [re.search(r"layers\.(\d+)\.", k)] if m]
    return max(idx) + 1 if idx else 0


def depth_series(dumps: Sequence[dict], pattern: str) -> Dict[str, list]:
    """For every dump: per layer the quantile vector of the tensor named by ``pattern`` (``name::what``)."""
    name, _, what = pattern.partition("::")
    what = what or "out"
    L = num_layers(dumps[0]) if dumps else 0
    frames, steps = [], []
    for d in dumps:
        per_layer = []
        for layer in range(L):
            stats = d["data"].get(f"{name.format(layer)}::{what}")
            q = (stats or {}).get("quantiles")
            per_layer.append(q if q is not None else None)
        frames.append(per_layer)
        steps.append((d.get("meta") or {}).get("global_step", len(steps)))
    qs = dumps[0].get("quantiles", []) if dumps else []
    return {"pattern": pattern, "frames": frames, "steps": steps, "quantiles": qs}


_PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>probe animation</title>
<style>body{font-family:sans-serif} svg{border:1px solid #ccc;margin:4px}</style></head><body>
<div><button id="play">play / pause</button> <input id="t" type="range" min="0" value="0" style="width:60%">
<span id="lab"></span></div><div id="plots"></div>
<script>
const RUNS = __DATA__;
const COLORS = ["#1f77b4","#d62728","#2ca02c","#9467bd","#ff7f0e"];
const W = 520, H = 300, L = 50, B = 30, T = 20, R = 10;
const nT = Math.max(...RUNS.flatMap(r => r.series.map(s => s.frames.length)));
document.getElementById("t").max = Math.max(0, nT - 1);
const plots = document.getElementById("plots");
const nP = RUNS[0].series.length;
const svgs = [];
for (let p = 0; p < nP; p++) {
  const s = document.createElementNS("http://www.w3.org/2000/svg", "svg");
  s.setAttribute("width", W); s.setAttribute("height", H); plots.appendChild(s); svgs.push(s);
}
function range(p) {
  let lo = Infinity, hi = -Infinity;
  for (const r of RUNS) for (const f of r.series[p].frames) for (const q of f) if (q) { lo = Math.min(lo, ...q); hi = Math.max(hi, ...q); }
  if (!isFinite(lo)) { lo = 0; hi = 1; } if (hi <= lo) hi = lo + 1; return [lo, hi];
}
const ranges = [...Array(nP).keys()].map(range);
function draw(t) {
  for (let p = 0; p < nP; p++) {
    const [lo, hi] = ranges[p]; const s = svgs[p]; s.innerHTML = "";
    const depth = RUNS[0].series[p].frames[0].length;
    const sx = i => L + (W - L - R) * (depth > 1 ? i / (depth - 1) : 0.5), sy = v => H - B - (H - B - T) * (v - lo) / (hi - lo);
    let h = `<text x="${W / 2}" y="14" text-anchor="middle" font-size="12">${RUNS[0].series[p].pattern}</text>` +
            `<text x="4" y="${T + 8}" font-size="10">${hi.toPrecision(3)}</text><text x="4" y="${H - B}" font-size="10">${lo.toPrecision(3)}</text>` +
            `<text x="${W / 2}" y="${H - 8}" text-anchor="middle" font-size="10">depth</text>`;
    RUNS.forEach((r, ri) => {
      const fr = r.series[p].frames[Math.min(t, r.series[p].frames.length - 1)]; const c = COLORS[ri % COLORS.length];
      const nq = (fr.find(q => q) || []).length;
      for (let a = 0; a < Math.floor(nq / 2); a++) {
        let up = [], dn = [];
        fr.forEach((q, i) => { if (q) { up.push(`${sx(i)},${sy(q[nq - 1 - a])}`); dn.unshift(`${sx(i)},${sy(q[a])}`); } });
        h += `<polygon points="${up.concat(dn).join(" ")}" fill="${c}" fill-opacity="${0.08 + 0.1 * a}" stroke="none"/>`;
      }
      if (nq % 2) { const mid = []; fr.forEach((q, i) => { if (q) mid.push(`${sx(i)},${sy(q[(nq - 1) / 2])}`); });
        h += `<polyline points="${mid.join(" ")}" fill="none" stroke="${c}" stroke-width="1.5"/>`; }
      h += `<text x="${W - R - 4}" y="${T + 12 * (ri + 1)}" text-anchor="end" font-size="10" fill="${c}">${r.name}</text>`;
    });
    s.innerHTML = h;
  }
  const st = RUNS[0].series[0].steps; document.getElementById("lab").textContent = "step " + st[Math.min(t, st.length - 1)];
}
let timer = null; const slider = document.getElementById("t");
slider.oninput = () => draw(+slider.value);
document.getElementById("play").onclick = () => { if (timer) { clearInterval(timer); timer = null; } else timer = setInterval(() => { slider.value = (+slider.value + 1) % nT; draw(+slider.value); }, 500); };
draw(0);
</script></body></html>"""


def render(probe_folders: Sequence[str], patterns: Sequence[str], out: str, subsample: int = 1) -> str:
    runs = []
    for folder in probe_folders:
        dumps = load_probe_folder(folder)[::max(1, subsample)]
        if not dumps:
            raise FileNotFoundError(f"no probe dump found in {folder}")
        runs.append({"name": Path(folder).name, "series": [depth_series(dumps, p) for p in patterns]})
    Path(out).parent.mkdir(parents=True, exist_ok=True)
    Path(out).write_text(_PAGE.replace("__DATA__", json.dumps(runs)))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("probe_folders", nargs="+")
    ap.add_argument("--pattern", action="append", default=None,
                    help='tensor pattern "name::what" with {} for the layer index; may be repeated')
    ap.add_argument("--out", default="render_out/probe.html")
    ap.add_argument("--subsample", type=int, default=1)
    a = ap.parse_args(argv)
    pats = a.pattern or ["layers.{}.attention.wo::out", "layers.{}.feed_forward.w2::out"]
    print(render(a.probe_folders, pats, a.out, a.subsample))


if __name__ == "__main__":
    main()
