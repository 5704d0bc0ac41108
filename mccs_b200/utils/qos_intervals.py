"""Offline planner for time-window QoS schedules: given the compute and communication
phase lengths of a premium job and of a victim job, lay the premium job's
communication windows on a periodic timeline and first-fit the victim's windows into
the gaps. Same algorithm as the reference's ``eval/multi-app/interval.py:4-33``; the
result is what goes into ``[qos_schedule]`` of the daemon configuration (or a
``qos_set`` admin request).

    python -m mccs_b200.utils.qos_intervals --premium 200:310000:110000 --victim 201:230000:35000

prints the TOML fragment (times in microseconds).
"""
from __future__ import annotations

import argparse
import math
from typing import List, Tuple

Interval = Tuple[int, int]


def calculate_intervals(premium_comp: int, premium_comm: int, victim_comp: int, victim_comm: int,
                        epoch: int | None = None) -> Tuple[List[Interval], List[Interval], int]:
    """Windows (start, end) for the premium and the victim job and the epoch length.

    The premium job communicates for ``premium_comm`` then computes for
    ``premium_comp``, repeating; the epoch defaults to the least common multiple of
    the two jobs' iteration times so that the schedule is periodic for both.
    """
    if epoch is None:
        epoch = math.lcm(premium_comp + premium_comm, victim_comp + victim_comm)
    premium: List[Interval] = []
    t = 0
    while t < epoch:
        premium.append((t, min(t + premium_comm, epoch)))
        t += premium_comm + premium_comp
    gaps = [(premium[i][1], premium[i + 1][0] if i + 1 < len(premium) else epoch) for i in range(len(premium))]
    victim: List[Interval] = []
    t = 0
    for start, end in gaps:
        t = max(t, start)
        while t + victim_comm <= end:
            victim.append((t, t + victim_comm))
            t += victim_comm + victim_comp
    return premium, victim, epoch


def to_toml(epoch: int, schedule: dict) -> str:
    out = ["[qos_schedule]", f"epoch_microsecs = {epoch}"]
    for comm_id, ivs in schedule.items():
        out += [f"[qos_schedule.schedule.{comm_id}]", "intervals = [" + ", ".join(f"[{a}, {b}]" for a, b in ivs) + "]",
                'mode = "Allow"']
    return "\n".join(out) + "\n"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--premium", required=True, help="comm_id:compute_us:comm_us")
    ap.add_argument("--victim", required=True, help="comm_id:compute_us:comm_us")
    ap.add_argument("--epoch", type=int, default=None)
    a = ap.parse_args()
    pid, pcomp, pcomm = (int(x) for x in a.premium.split(":"))
    vid, vcomp, vcomm = (int(x) for x in a.victim.split(":"))
    prem, vic, epoch = calculate_intervals(pcomp, pcomm, vcomp, vcomm, a.epoch)
    print(to_toml(epoch, {pid: prem, vid: vic}), end="")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
