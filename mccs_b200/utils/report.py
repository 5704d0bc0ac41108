"""Turns a sweep CSV (``mccs_b200.utils.sweep``) into the table the evaluation needs:
per collective, dtype and message size, the service's time and bus bandwidth (``auto``
row when present, else the best variant), the best single variant, NCCL on the same
buffers, their ratio, and the fraction of the NVLink roofline. Counterpart of the
reference's ``eval/single-app/collect.py`` + ``eval/plot/single_app/main.py`` (text
instead of a figure).

    python -m mccs_b200.utils.report sweep.csv --link-gbs 770 > summary.md
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured NVLink bandwidth per direction per GPU")
    a = ap.parse_args()
    rows = list(csv.DictReader(open(a.csv)))
    groups = defaultdict(list)
    for r in rows:
        groups[(r["coll"], r["dtype"], int(r["n"]), int(r["bytes"]))].append(r)
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
