"""Real-workload co-location: the VGG and the two GPT traces of the reference's figure 9,
replayed by ``traffic_gen`` side by side under three policies, job completion times out.

The reference runs VGG (574,668,960 B fp16 AllReduce after 160 ms of compute, 101 iterations,
4 GPUs) next to two GPT jobs (83,886,080 B after 6 ms, 1501 and 3001 iterations, 2 GPUs each) on
hosts whose NICs they share, under "fair" (no policy), "qosv1" (a premium route for VGG) and
"qosv2" (qosv1 plus a time-window schedule that keeps the GPT jobs off the wire while VGG
communicates): ``eval/multi-app/gen_traffic_gen_config.py:213-260``, ``workloads/setup-4_*.toml``,
results in ``eval/plot/real_workload/jct.csv``. Inside one NVSwitch box jobs on disjoint GPUs
do not meet at all, so the default placement here makes them share GPUs (VGG on 0-3, GPT_1 on
0-1, GPT_2 on 2-3: SMs and link bandwidth of every GPU are contended); ``--placement reference``
keeps the reference's disjoint placement on eight GPUs. The policies map to this service's
arbiter: qosv1 = VGG gets weight 4 and a high-priority stream, qosv2 = that plus Allow windows
laid out by :mod:`mccs_b200.utils.qos_intervals` from the jobs' compute and communication times.

    python -m mccs_b200.utils.colocate_traces --scale 0.25 --out jct.json

``--scale`` multiplies the iteration counts (1.0 = the reference's). Prints one JSON object:
per policy and job the completion time in ms and the mean iteration time, next to the
reference's published means.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile
from typing import Dict, List

from .. import _lib, daemon
from .qos_intervals import calculate_intervals, to_toml

JOBS = {   # name: (communicator id, bytes, compute us, iterations in the reference)
    "vgg": (200, 574668960, 160000, 101),
    "gpt_1": (201, 83886080, 6000, 1501),
    "gpt_2": (202, 83886080, 6000, 3001),
}
PLACEMENT = {
    "shared": {"vgg": [0, 1, 2, 3], "gpt_1": [0, 1], "gpt_2": [2, 3]},
    "reference": {"vgg": [0, 1, 2, 3], "gpt_1": [4, 6], "gpt_2": [5, 7]},
}
REFERENCE_JCT_MS = {   # eval/plot/real_workload/jct.csv, means of 10 runs on the reference's testbed
    "fair": {"vgg": 34684, "gpt_1": 39084, "gpt_2": 69768},
    "qosv1": {"vgg": 30636, "gpt_1": 51501, "gpt_2": 85552},
    "qosv2": {"vgg": 30621, "gpt_1": 44483, "gpt_2": 99970},
}


def policy_config(policy: str, vgg_comm_us: int, gpt_comm_us: int, time_scale: float = 1.0) -> str:
    if policy == "fair":
        return ""
    text = f"[qos.tenants.{JOBS['vgg'][0]}]\nweight = 4.0\npriority = 1\n"
    if policy == "qosv2":
        vgg_compute = max(int(JOBS["vgg"][2] * time_scale), 1)
        gpt_compute = max(int(JOBS["gpt_1"][2] * time_scale), 1)
        premium, victim, epoch = calculate_intervals(vgg_compute, vgg_comm_us, gpt_compute, gpt_comm_us, epoch=vgg_compute + vgg_comm_us)
        text += to_toml(epoch, {JOBS["vgg"][0]: premium, JOBS["gpt_1"][0]: victim, JOBS["gpt_2"][0]: victim})
    return text


def run_policy(policy: str, place: Dict[str, List[int]], scale: float, work: str, host: bool, vgg_comm_us: int,
               gpt_comm_us: int, timeout: float, size_scale: float = 1.0, time_scale: float = 1.0) -> dict:
    prefix = os.path.join(work, policy)
    os.makedirs(prefix, exist_ok=True)
    cfg = daemon.default_config(prefix, listen_port=-1, host_devices=8, force_host=host) + policy_config(policy, vgg_comm_us, gpt_comm_us, time_scale)
    with open(prefix + "/mccs.toml", "w") as f:
        f.write(cfg)
    sp = daemon.spawn(prefix + "/mccs.toml", env={"MCCS_LOG": "warn"})
    procs = []
    try:
        env = dict(os.environ, MCCS_CONTROL=sp.control, MCCS_LOG="error")
        for name, (cid, size, compute, iters) in JOBS.items():
            trace = f"{prefix}/{name}.toml"
            size = max(int(size * size_scale) // 16 * 16, 16)
            compute = max(int(compute * time_scale), 1)
            with open(trace, "w") as f:
                f.write(f"communicator_id = {cid}\ncuda_devices = {place[name]}\n[[traces]]\nsize = {size}\ntype = \"all_reduce\"\n"
                        f"compute_interval = {compute}\n")
            n_iter = max(int(iters * scale), 22)
            for rank in range(len(place[name])):
                cmd = [os.path.join(_lib.NATIVE_DIR, "traffic_gen"), "--rank", str(rank), "--config", trace, "--iters", str(n_iter),
                       "--name", name]
                procs.append((name, rank, n_iter, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
        out: Dict[str, dict] = {}
        for name, rank, n_iter, p in procs:
            try:
                so, se = p.communicate(timeout=timeout)
            except subprocess.TimeoutExpired:
                p.kill()
                so, se = p.communicate()
            if p.returncode != 0:
                raise RuntimeError(f"{policy}/{name} rank {rank} exit {p.returncode}: {se[-1000:]}")
            if rank == 0:
                m = re.search(r"run time: (\d+) ms", so)
                mm = re.search(r"\(mean, median, min, max\) = \(([\d.]+), ([\d.]+)", so)
                out[name] = {"jct_ms": int(m.group(1)) if m else None, "iterations": n_iter,
                             "mean_iter_ms": float(mm.group(1)) if mm else None, "median_iter_ms": float(mm.group(2)) if mm else None,
                             "reference_jct_ms": REFERENCE_JCT_MS[policy][name]}
        return out
    finally:
        for _, _, _, p in procs:
            if p.poll() is None:
                p.kill()
        sp.stop()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--policies", default="fair,qosv1,qosv2")
    ap.add_argument("--placement", default="shared", choices=sorted(PLACEMENT))
    ap.add_argument("--scale", type=float, default=0.25, help="fraction of the reference's iteration counts")
    ap.add_argument("--vgg-comm-us", type=int, default=2000, help="VGG's AllReduce time alone, for the window schedule")
    ap.add_argument("--gpt-comm-us", type=int, default=400, help="a GPT job's AllReduce time alone")
    ap.add_argument("--host", action="store_true", help="host backend (a dry run of the tool without GPUs)")
    ap.add_argument("--size-scale", type=float, default=1.0, help="multiplies the message sizes (dry runs)")
    ap.add_argument("--time-scale", type=float, default=1.0, help="multiplies the compute intervals (dry runs)")
    ap.add_argument("--timeout", type=float, default=900.0)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    place = PLACEMENT[a.placement]
    res = {"placement": a.placement, "devices": place, "scale": a.scale, "size_scale": a.size_scale, "time_scale": a.time_scale,
           "policies": {}}
    with tempfile.TemporaryDirectory(prefix="mccs-colocate-") as work:
        for policy in a.policies.split(","):
            res["policies"][policy] = run_policy(policy, place, a.scale, work, a.host, a.vgg_comm_us, a.gpt_comm_us, a.timeout,
                                                 a.size_scale, a.time_scale)
    text = json.dumps(res, indent=1)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
