"""Turns a sweep CSV (``mccs_b200.utils.sweep``) into the table the evaluation needs:
per collective, dtype and message size, the service's time and bus bandwidth (``auto``
row when present, else the best variant), the best single variant, NCCL on the same
buffers, their ratio, and the fraction of the NVLink roofline. Counterpart of the
reference's ``eval/single-app/collect.py`` + ``eval/plot/single_app/main.py``.

    python -m mccs_b200.utils.report sweep.csv --link-gbs 770 > summary.md
    python -m mccs_b200.utils.report sweep.csv --svg curves.svg      # bus bandwidth vs. size, service and NCCL

The figure is written as plain SVG (no plotting package is needed): one panel per
(collective, dtype), message size on a log axis, the link bandwidth as a dashed line.
"""
from __future__ import annotations

import argparse
import csv
import sys
from collections import defaultdict


def human(n: int) -> str:
    for unit, div in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if n >= div:
            v = n / div
            return f"{v:g} {unit}"
    return f"{n} B"


def write_svg(path: str, groups, link_gbs: float) -> None:
    """Bus bandwidth over message size: best service variant and NCCL, one panel per
    (collective, dtype, GPU count)."""
    import math
    panels = defaultdict(dict)     # (coll, dtype, n) -> size -> (service busBW, nccl busBW or None)
    for (coll, dtype, n, size), rs in groups.items():
        mine = [float(r["busbw_GBps"]) for r in rs if r["algo"] != "nccl"]
        nccl = [float(r["busbw_GBps"]) for r in rs if r["algo"] == "nccl"]
        if mine:
            panels[(coll, dtype, n)][size] = (max(mine), nccl[0] if nccl else None)
    W, H, L, R, T, B = 560, 300, 60, 20, 30, 45
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H * max(len(panels), 1)}" font-family="sans-serif" font-size="11">']
    for pi, (key, pts) in enumerate(sorted(panels.items())):
        y0 = pi * H
        sizes = sorted(pts)
        lo, hi = math.log2(sizes[0]), math.log2(max(sizes[-1], sizes[0] * 2))
        top = max(link_gbs, max(max(v[0], v[1] or 0) for v in pts.values())) * 1.08

        def X(s):
            return L + (math.log2(s) - lo) / (hi - lo) * (W - L - R)

        def Y(v):
            return y0 + H - B - v / top * (H - T - B)
        out.append(f'<text x="{L}" y="{y0 + 18}" font-size="13">{key[0]} {key[1]}, {key[2]} GPUs: bus bandwidth (GB/s) vs. message size</text>')
        out.append(f'<rect x="{L}" y="{y0 + T}" width="{W - L - R}" height="{H - T - B}" fill="none" stroke="#888"/>')
        for frac in (0.25, 0.5, 0.75, 1.0):
            v = top * frac
            out.append(f'<line x1="{L}" x2="{W - R}" y1="{Y(v):.1f}" y2="{Y(v):.1f}" stroke="#ddd"/>')
            out.append(f'<text x="{L - 6}" y="{Y(v) + 4:.1f}" text-anchor="end">{v:.0f}</text>')
        for s in sizes[::2]:
            out.append(f'<text x="{X(s):.1f}" y="{y0 + H - B + 14}" text-anchor="middle">{human(s).replace(" ", "")}</text>')
        out.append(f'<line x1="{L}" x2="{W - R}" y1="{Y(link_gbs):.1f}" y2="{Y(link_gbs):.1f}" stroke="#c33" stroke-dasharray="5,4"/>')
        out.append(f'<text x="{W - R - 4}" y="{Y(link_gbs) - 4:.1f}" text-anchor="end" fill="#c33">link {link_gbs:.0f}</text>')
        for idx, (name, colour) in enumerate((("service", "#1668c1"), ("NCCL", "#777"))):
            line = [(X(s), Y(pts[s][idx])) for s in sizes if pts[s][idx] is not None]
            if not line:
                continue
            out.append(f'<polyline fill="none" stroke="{colour}" stroke-width="2" points="' + " ".join(f"{x:.1f},{y:.1f}" for x, y in line) + '"/>')
            for x, y in line:
                out.append(f'<circle cx="{x:.1f}" cy="{y:.1f}" r="2.5" fill="{colour}"/>')
            out.append(f'<text x="{L + 10 + 70 * idx}" y="{y0 + T + 14}" fill="{colour}">{name}</text>')
    out.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(out))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--svg", default="", help="also write the bandwidth curves to this SVG file")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured NVLink bandwidth per direction per GPU")
    a = ap.parse_args()
    rows = list(csv.DictReader(open(a.csv)))
    groups = defaultdict(list)
    for r in rows:
        groups[(r["coll"], r["dtype"], int(r["n"]), int(r["bytes"]))].append(r)
    if a.svg:
        write_svg(a.svg, groups, a.link_gbs)
    print("| collective | dtype | GPUs | size | service | CTAs | time µs | busBW GB/s | best variant | its busBW | NCCL busBW | service/NCCL | of NVLink roofline |")
    print("|---|---|---|---|---|---|---|---|---|---|---|---|---|")
    for (coll, dtype, n, size), rs in sorted(groups.items(), key=lambda kv: (kv[0][0], kv[0][1], kv[0][2], kv[0][3])):
        mine = [r for r in rs if r["algo"] != "nccl"]
        nccl = [r for r in rs if r["algo"] == "nccl"]
        if not mine:
            continue
        best = min(mine, key=lambda r: float(r["ms"]))
        svc = best
        nb = float(nccl[0]["busbw_GBps"]) if nccl else None
        bus = float(svc["busbw_GBps"])
        # The roofline of a bus-bandwidth figure is the link bandwidth itself: busBW is
        # defined so that a ring moving data at link speed scores exactly the link speed.
        roof = bus / a.link_gbs
        print(f"| {coll} | {dtype} | {n} | {human(size)} | {svc['algo']} | {svc['ctas']} | {float(svc['ms']) * 1e3:.1f} | {bus:.1f} | "
              f"{best['algo']} | {float(best['busbw_GBps']):.1f} | {nb:.1f} | {bus / nb:.2f} | {roof:.2f} |" if nb else
              f"| {coll} | {dtype} | {n} | {human(size)} | {svc['algo']} | {svc['ctas']} | {float(svc['ms']) * 1e3:.1f} | {bus:.1f} | "
              f"{best['algo']} | {float(best['busbw_GBps']):.1f} | - | - | {roof:.2f} |")
    return 0


if __name__ == "__main__":
    sys.exit(main())
