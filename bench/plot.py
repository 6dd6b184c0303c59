#!/usr/bin/env python
"""Plots of benchmark output as stand-alone SVG files (no matplotlib, no display needed).

    python bench/plot.py curves  sweep.jsonl  -o busbw.svg     # bus bandwidth against message size
    python bench/plot.py phases  sweep.jsonl  -o phases.svg    # where a kernel's time goes

`curves` reads the JSON lines of bench/sweep.py (one line per configuration and size) and the
tables of bench/hx_perf (lines of numbers under a "# hx_perf ..." header) and draws one curve
per configuration on a logarithmic size axis. `phases` reads the JSON lines that bench/sweep.py
prints under HXCCL_TRACE=1 (field "trace_us": mean time per CTA and call in each phase of the
kernel) and draws one stacked bar per (configuration, size).

Takes the place of the reference's scripts/plot_b_timeline.py:1-162, which draws timelines from
an nsys export; nsys is not part of this environment, the library's own phase timers are.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from typing import Dict, List, Tuple

COLORS = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f"]
PHASES = ["in", "sigA", "waitA", "mid", "sigB", "waitB", "out"]


def human(nbytes: float) -> str:
    for unit, k in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
        if nbytes >= k:
            return f"{nbytes / k:g}{unit}"
    return f"{nbytes:g}"


def read_rows(path: str) -> List[dict]:
    """JSON lines as they are; hx_perf tables become rows with config = the header's settings."""
    rows, header = [], None
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if line.startswith("{"):
                try:
                    rows.append(json.loads(line))
                except json.JSONDecodeError:
                    pass
            elif line.startswith("# hx_perf"):
                header = " ".join(w for w in line[9:].split() if w.split("=")[0] in ("op", "type", "red", "ranks"))
            elif header and not line.startswith("#"):
                parts = line.split()
                if len(parts) == 5:
                    rows.append({"config": header, "bytes": int(parts[0]), "us": float(parts[2]),
                                 "busbw_GBps": float(parts[4])})
    return rows


class Svg:
    def __init__(self, w: int, h: int):
        self.w, self.h, self.items = w, h, []

    def add(self, s: str) -> None:
        self.items.append(s)

    def text(self, x, y, s, size=11, anchor="start", rot=None, fill="#222") -> None:
        tr = f' transform="rotate({rot} {x} {y})"' if rot is not None else ""
        s = str(s).replace("&", "&amp;").replace("<", "&lt;")
        self.add(f'<text x="{x:.1f}" y="{y:.1f}" font-size="{size}" text-anchor="{anchor}" fill="{fill}" '
                 f'font-family="sans-serif"{tr}>{s}</text>')

    def line(self, x0, y0, x1, y1, color="#999", width=1.0, dash=None) -> None:
        d = f' stroke-dasharray="{dash}"' if dash else ""
        self.add(f'<line x1="{x0:.1f}" y1="{y0:.1f}" x2="{x1:.1f}" y2="{y1:.1f}" stroke="{color}" '
                 f'stroke-width="{width}"{d}/>')

    def dump(self) -> str:
        return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.w}" height="{self.h}" '
                f'viewBox="0 0 {self.w} {self.h}"><rect width="100%" height="100%" fill="white"/>'
                + "".join(self.items) + "</svg>\n")


def nice_ceiling(v: float) -> float:
    if v <= 0:
        return 1.0
    mag = 10 ** math.floor(math.log10(v))
    for m in (1, 2, 2.5, 5, 10):
        if v <= m * mag:
            return m * mag
    return 10 * mag


def plot_curves(rows: List[dict], title: str) -> str:
    series: Dict[str, List[Tuple[int, float]]] = {}
    for r in rows:
        if "bytes" in r and "busbw_GBps" in r:
            series.setdefault(str(r.get("config", "default")), []).append((int(r["bytes"]), float(r["busbw_GBps"])))
    if not series:
        raise SystemExit("no rows with 'bytes' and 'busbw_GBps' found")
    W, H, L, R, T, B = 860, 480, 70, 230, 40, 60
    svg = Svg(W, H)
    xs = [b for pts in series.values() for b, _ in pts]
    lo, hi = math.log2(max(1, min(xs))), math.log2(max(2, max(xs)))
    hi = hi if hi > lo else lo + 1
    top = nice_ceiling(max(v for pts in series.values() for _, v in pts))
    px = lambda b: L + (math.log2(max(1, b)) - lo) / (hi - lo) * (W - L - R)  # noqa: E731
    py = lambda v: H - B - v / top * (H - T - B)  # noqa: E731
    svg.text(L, 22, title, size=14)
    for k in range(6):
        v = top * k / 5
        svg.line(L, py(v), W - R, py(v), "#ddd")
        svg.text(L - 6, py(v) + 4, f"{v:g}", anchor="end")
    e = math.ceil(lo)
    step = max(1, round((hi - lo) / 10))
    while e <= hi:
        svg.line(px(2 ** e), H - B, px(2 ** e), H - B + 4, "#555")
        svg.text(px(2 ** e), H - B + 18, human(2 ** e), anchor="middle")
        e += step
    svg.line(L, H - B, W - R, H - B, "#555")
    svg.line(L, T, L, H - B, "#555")
    svg.text((L + W - R) / 2, H - 14, "message size (bytes)", anchor="middle")
    svg.text(18, (T + H - B) / 2, "bus bandwidth (GB/s)", anchor="middle", rot=-90)
    for i, (name, pts) in enumerate(sorted(series.items())):
        pts.sort()
        c = COLORS[i % len(COLORS)]
        path = " ".join(f"{'M' if j == 0 else 'L'}{px(b):.1f},{py(v):.1f}" for j, (b, v) in enumerate(pts))
        svg.add(f'<path d="{path}" fill="none" stroke="{c}" stroke-width="2"/>')
        for b, v in pts:
            svg.add(f'<circle cx="{px(b):.1f}" cy="{py(v):.1f}" r="3" fill="{c}"/>')
        svg.line(W - R + 14, T + 14 + 18 * i, W - R + 38, T + 14 + 18 * i, c, 2)
        svg.text(W - R + 44, T + 18 + 18 * i, name[:30])
    return svg.dump()


def plot_phases(rows: List[dict], title: str) -> str:
    bars = [(f"{r.get('config', 'default')} @ {human(r['bytes'])}", r["trace_us"]) for r in rows if "trace_us" in r]
    if not bars:
        raise SystemExit("no rows with 'trace_us' found (run bench/sweep.py with HXCCL_TRACE=1)")
    W, L, R, T, rowh = 900, 260, 40, 60, 26
    H = T + rowh * len(bars) + 50
    svg = Svg(W, H)
    svg.text(20, 22, title, size=14)
    top = nice_ceiling(max(sum(float(t.get(p, 0)) for p in PHASES) for _, t in bars))
    px = lambda v: L + v / top * (W - L - R)  # noqa: E731
    for i, p in enumerate(PHASES):
        svg.add(f'<rect x="{L + 80 * i}" y="32" width="12" height="12" fill="{COLORS[i]}"/>')
        svg.text(L + 80 * i + 16, 43, p)
    for k in range(6):
        v = top * k / 5
        svg.line(px(v), T, px(v), H - 40, "#ddd")
        svg.text(px(v), H - 24, f"{v:g}", anchor="middle")
    svg.text((L + W - R) / 2, H - 8, "microseconds per call (mean over CTAs)", anchor="middle")
    for j, (name, t) in enumerate(bars):
        y, x = T + rowh * j, 0.0
        svg.text(L - 8, y + 16, name[:38], anchor="end")
        for i, p in enumerate(PHASES):
            v = float(t.get(p, 0))
            svg.add(f'<rect x="{px(x):.1f}" y="{y + 4}" width="{max(0.0, px(x + v) - px(x)):.1f}" height="{rowh - 8}" '
                    f'fill="{COLORS[i]}"><title>{p}: {v:g} us</title></rect>')
            x += v
        if "all" in t:
            svg.line(px(float(t["all"])), y + 2, px(float(t["all"])), y + rowh - 2, "#000", 1.5, "3,2")
    return svg.dump()


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kind", choices=["curves", "phases"])
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("-o", "--out", default="-")
    ap.add_argument("--title", default="")
    args = ap.parse_args()
    rows = [r for p in args.inputs for r in read_rows(p)]
    svg = (plot_curves if args.kind == "curves" else plot_phases)(rows, args.title or " ".join(args.inputs))
    if args.out == "-":
        sys.stdout.write(svg)
    else:
        with open(args.out, "w") as f:
            f.write(svg)
    return 0


if __name__ == "__main__":
    sys.exit(main())
