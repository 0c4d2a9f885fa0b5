"""Draws the figures under docs/ from measured sweep rows, as plain SVG (no
plotting library needed).

    python docs/make_plots.py docs/data/sweep8_fairring_ordinary.json docs/data/sweep8_nccl.json docs/allreduce_busbw_8gpu.svg \\
        --title "all-reduce, 8 x B200, fp32, ordinary tensors"

The input is what ``python -m fairring_b200.bench.sweep --json`` (or
``baseline/ref_sweep.py --json``) writes: ``{"rows": [{"backend", "dtype",
"bytes", "busbw_gbs" | "us"}, ...]}``; several files may be given and are
merged.  One line per (backend, dtype); x = message size (log2), y = bus GB/s
(or microseconds with ``--y us``).
"""

from __future__ import annotations

import argparse
import json
import math
import sys

COLORS = ["#d62728", "#1f77b4", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f"]


def human(n: int) -> str:
    for unit, k in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if n >= k:
            v = n / k
            return f"{v:g} {unit}"
    return f"{n} B"


def line_chart(series: dict[str, list[tuple[float, float]]], title: str, ylabel: str, logy: bool) -> str:
    W, H, L, R, T, B = 860, 480, 70, 230, 40, 60
    xs = sorted({x for pts in series.values() for x, _ in pts})
    ys = [y for pts in series.values() for _, y in pts if y > 0]
    if not xs or not ys:
        raise SystemExit("nothing to plot")
    x0, x1 = math.log2(xs[0]), math.log2(xs[-1])
    if logy:
        y0, y1 = math.log10(min(ys)), math.log10(max(ys))
    else:
        y0, y1 = 0.0, max(ys) * 1.05
    if x1 == x0:
        x1 += 1
    if y1 == y0:
        y1 += 1

    def px(x):
        return L + (math.log2(x) - x0) / (x1 - x0) * (W - L - R)

    def py(y):
        v = math.log10(y) if logy else y
        return H - B - (v - y0) / (y1 - y0) * (H - T - B)

    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" viewBox="0 0 {W} {H}" '
           f'font-family="sans-serif" font-size="12">',
           f'<rect width="{W}" height="{H}" fill="white"/>',
           f'<text x="{L}" y="22" font-size="15" font-weight="bold">{title}</text>']
    # grid: every second power of two on x
    for i, x in enumerate(xs):
        if len(xs) > 12 and i % 2:
            continue
        out.append(f'<line x1="{px(x):.1f}" y1="{T}" x2="{px(x):.1f}" y2="{H - B}" stroke="#e5e5e5"/>')
        out.append(f'<text x="{px(x):.1f}" y="{H - B + 16}" text-anchor="middle">{human(int(x))}</text>')
    ticks = []
    if logy:
        e = math.floor(y0)
        while e <= math.ceil(y1):
            for m in (1, 2, 5):
                v = m * 10 ** e
                if 10 ** y0 <= v <= 10 ** y1:
                    ticks.append(v)
            e += 1
    else:
        step = 10 ** math.floor(math.log10(y1 / 5))
        for m in (1, 2, 5, 10):
            if y1 / (step * m) <= 8:
                step *= m
                break
        v = 0.0
        while v <= y1:
            ticks.append(v)
            v += step
    for v in ticks:
        if v <= 0 and logy:
            continue
        out.append(f'<line x1="{L}" y1="{py(v):.1f}" x2="{W - R}" y2="{py(v):.1f}" stroke="#e5e5e5"/>')
        out.append(f'<text x="{L - 6}" y="{py(v) + 4:.1f}" text-anchor="end">{v:g}</text>')
    out.append(f'<rect x="{L}" y="{T}" width="{W - L - R}" height="{H - T - B}" fill="none" stroke="#444"/>')
    out.append(f'<text x="16" y="{(H - B + T) / 2:.0f}" transform="rotate(-90 16 {(H - B + T) / 2:.0f})" '
               f'text-anchor="middle">{ylabel}</text>')
    out.append(f'<text x="{(L + W - R) / 2:.0f}" y="{H - 14}" text-anchor="middle">message size</text>')
    for i, (name, pts) in enumerate(series.items()):
        col = COLORS[i % len(COLORS)]
        pts = sorted(p for p in pts if p[1] > 0)
        d = " ".join(f"{'M' if j == 0 else 'L'}{px(x):.1f},{py(y):.1f}" for j, (x, y) in enumerate(pts))
        out.append(f'<path d="{d}" fill="none" stroke="{col}" stroke-width="2"/>')
        for x, y in pts:
            out.append(f'<circle cx="{px(x):.1f}" cy="{py(y):.1f}" r="2.5" fill="{col}"/>')
        ly = T + 14 + 18 * i
        out.append(f'<line x1="{W - R + 12}" y1="{ly - 4}" x2="{W - R + 36}" y2="{ly - 4}" stroke="{col}" stroke-width="2"/>')
        out.append(f'<text x="{W - R + 42}" y="{ly}">{name}</text>')
    out.append("</svg>")
    return "\n".join(out) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("inputs_and_output", nargs="+", help="one or more JSON files, then the SVG to write")
    ap.add_argument("--title", default="all-reduce bus bandwidth")
    ap.add_argument("--y", choices=["busbw", "us"], default="busbw")
    ap.add_argument("--dtype", default="", help="only rows of this dtype")
    ap.add_argument("--min-bytes", type=int, default=0)
    ap.add_argument("--max-bytes", type=int, default=1 << 62)
    ap.add_argument("--rename", action="append", default=[], help="old=new label, repeatable")
    args = ap.parse_args(argv)
    *inputs, output = args.inputs_and_output
    rename = dict(r.split("=", 1) for r in args.rename)
    series: dict[str, list[tuple[float, float]]] = {}
    for path in inputs:
        with open(path) as f:
            data = json.load(f)
        for r in data["rows"] if isinstance(data, dict) else data:
            if "bytes" not in r or not (args.min_bytes <= r["bytes"] <= args.max_bytes):
                continue
            if args.dtype and r.get("dtype", args.dtype) != args.dtype:
                continue
            name = r.get("backend") or r.get("variant") or r.get("part", "?")
            if not args.dtype and "dtype" in r:
                name = f"{name} {r['dtype']}"
            name = rename.get(name, name)
            y = r.get("busbw_gbs", r.get("busbw")) if args.y == "busbw" else r.get("us")
            if y is None:
                continue
            series.setdefault(name, []).append((float(r["bytes"]), float(y)))
    svg = line_chart(series, args.title, "bus GB/s" if args.y == "busbw" else "microseconds per call",
                     logy=args.y == "us")
    with open(output, "w") as f:
        f.write(svg)
    print(f"wrote {output}: {len(series)} series")
    return 0


if __name__ == "__main__":
    sys.exit(main())
