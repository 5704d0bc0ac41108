"""Multi-tenant benchmark: several applications share the GPUs of the box and loop
batches of back-to-back AllReduces, under QoS weights, with a live reconfiguration in
the middle of the run.

Default scenario (the reference's counterpart is
``eval/multi-app`` settings 1-4 plus ``eval/dynamic-config``): four applications —
A and B on two GPUs each, C and D on four GPUs each, overlapping A's and B's GPUs —
each iteration = 16 back-to-back fp32 AllReduces of 8 MB, weights 2:1:1:1, and at
iteration 500 application C's rings are re-ordered and its channel count changed
without restarting anything. Reports per-application iteration time (device-timed)
and a weighted fairness index.

    python -m mccs_b200.utils.multi_tenant --iters 1000                 # through the service
    python -m mccs_b200.utils.multi_tenant --iters 1000 --backend nccl  # each app an NCCL group

One orchestrator process hosts the daemon and starts one process per application
rank; with ``--backend nccl`` the same workers use torch.distributed/NCCL instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from typing import Dict, List

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def default_apps(ngpu: int) -> List[dict]:
    if ngpu >= 8:
        place = {"A": [0, 1], "B": [2, 3], "C": [0, 2, 4, 6], "D": [1, 3, 5, 7]}
    elif ngpu >= 4:
        place = {"A": [0, 1], "B": [2, 3], "C": [0, 1, 2, 3], "D": [0, 1, 2, 3]}
    elif ngpu >= 2:
        place = {"A": [0, 1], "B": [0, 1], "C": [0, 1], "D": [0, 1]}
    else:
        place = {"A": [0], "B": [0]}
    weights = {"A": 2.0, "B": 1.0, "C": 1.0, "D": 1.0}
    return [{"name": k, "comm_id": 900 + i, "devices": v, "weight": weights[k]} for i, (k, v) in enumerate(place.items())]


def reference_setting(k: int) -> List[dict]:
    """Placements of the reference's multi-application settings 1-4
    (``eval/multi-app/gen_config.py:154-413``: four hosts with two GPUs each, jobs that share
    hosts but never a GPU), with host i of the testbed mapped to the GPU pair (2i, 2i+1) of
    one box. The jobs are equals (weight 1); the reference runs one 128 MB AllReduce per
    iteration (``--batch 1 --bytes 134217728``)."""
    place = {
        1: {"blue": [0, 1, 2, 3], "red": [4, 5, 6, 7]},                      # two 4-GPU jobs on disjoint host pairs
        2: {"blue": [0, 4, 2, 6], "green": [1, 3], "red": [5, 7]},            # a 4-GPU job on every host + two 2-GPU jobs
        3: {"blue": [0, 4, 2, 6], "red": [1, 5, 3, 7]},                       # two 4-GPU jobs on the same four hosts
        4: {"blue": [0, 1, 2, 3], "green": [4, 6], "red": [5, 7]},            # a 4-GPU job on two hosts + two 2-GPU jobs on the others
    }[k]
    return [{"name": n, "comm_id": 910 + 10 * k + i, "devices": d, "weight": 1.0} for i, (n, d) in enumerate(place.items())]


def worker(a) -> int:
    import torch
    import torch.distributed as dist
    dev = a.device
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(dev)
    store = dist.TCPStore("127.0.0.1", a.store_port, is_master=False, timeout=__import__("datetime").timedelta(seconds=300))
    count = a.bytes // 4
    if a.backend == "mccs":
        import mccs_b200 as M
        M.init(os.environ["MCCS_CONTROL"])
        bufs = [M.Buffer(a.bytes, dev) for _ in range(a.batch)]
        ts = [b.tensor(torch.float32, count) for b in bufs]
        comm = M.Communicator(a.comm_id, a.rank, a.nranks, device=dev)

        def one_iteration():
            with M.group():
                for t in ts:
                    comm.all_reduce(t, op="avg")     # averages keep the values bounded over thousands of rounds
    else:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(a.group_port)
        dist.init_process_group("nccl" if cuda else "gloo", rank=a.rank, world_size=a.nranks,
                                device_id=torch.device(f"cuda:{dev}") if cuda else None)
        ts = [torch.empty(count, dtype=torch.float32, device=f"cuda:{dev}" if cuda else "cpu") for _ in range(a.batch)]

        def one_iteration():
            for t in ts:
                dist.all_reduce(t, op=dist.ReduceOp.AVG)
    g = torch.Generator().manual_seed(a.rank)
    for t in ts:
        t.copy_(torch.rand(count, generator=g) * 2 - 1)
    for _ in range(5):
        one_iteration()
    if cuda:
        torch.cuda.synchronize()
    # all applications start together
    store.add("ready", 1)
    while int(store.add("ready", 0)) < a.total_ranks:
        time.sleep(0.001)
    events = []
    t_host0 = time.perf_counter()
    for it in range(a.iters):
        if a.reconfig_at >= 0 and it == a.reconfig_at and a.rank == 0 and a.backend == "mccs":
            import mccs_b200 as M
            n = a.nranks
            rings = [list(reversed(range(n))), list(range(n)), [(i * 3) % n for i in range(n)] if n % 3 else list(range(n))]
            rings = [r for r in rings if sorted(r) == list(range(n))]
            rep = M.reconfigure(a.admin_port, [{"communicator_id": a.comm_id,
                                                "channels": [{"channel_id": i, "ring": r} for i, r in enumerate(rings)]}])
            assert rep.get("status") == "ok", rep
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            one_iteration()
            e1.record()
            events.append((e0, e1))
            if it % 64 == 63:
                e1.synchronize()      # bound the number of iterations queued ahead
        else:
            t0 = time.perf_counter()
            one_iteration()
            events.append((time.perf_counter() - t0) * 1e3)
    if cuda:
        torch.cuda.synchronize()
        times = [e0.elapsed_time(e1) for e0, e1 in events]
    else:
        times = events
    wall = time.perf_counter() - t_host0
    ok = all(bool(torch.isfinite(t[:16]).all()) for t in ts)
    out = {"app": a.app, "rank": a.rank, "mean_ms": statistics.fmean(times), "median_ms": statistics.median(times),
           "p99_ms": sorted(times)[int(len(times) * 0.99) - 1], "wall_s": wall, "finite": ok,
           "mean_before_ms": statistics.fmean(times[:a.reconfig_at]) if a.reconfig_at > 0 else None,
           "mean_after_ms": statistics.fmean(times[a.reconfig_at:]) if a.reconfig_at > 0 else None}
    if a.backend == "mccs":
        q = comm.query()
        out["config_epoch"] = q["config_epoch"]
        out["async_error"] = q["async_error"]
        out["launch"] = comm.launch_mode
        comm.destroy()
    else:
        dist.destroy_process_group()
    print("RESULT " + json.dumps(out), flush=True)
    return 0


def orchestrate(a) -> int:
    import torch
    import torch.distributed as dist
    ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if a.apps:
        apps = json.loads(a.apps)
    elif a.setting:
        apps = reference_setting(a.setting)
        if ngpu and ngpu < 8:
            raise SystemExit("the reference's settings place jobs on eight GPUs")
    else:
        apps = default_apps(max(ngpu, a.host_devices if ngpu == 0 else ngpu))
    total = sum(len(x["devices"]) for x in apps)
    import datetime
    store = dist.TCPStore("127.0.0.1", 0, is_master=True, timeout=datetime.timedelta(seconds=300), wait_for_workers=False)
    env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
    admin_port = 0
    if a.backend == "mccs":
        import mccs_b200 as M
        tenants = "\n".join(f"[qos.tenants.{x['comm_id']}]\nweight = {x['weight']}" for x in apps)
        prefix = f"/tmp/mccs-mt-{os.getuid()}-{os.getpid()}"
        cfg = M.daemon.default_config(prefix, listen_port=-1, host_devices=8, sync=a.sync) + ("" if a.no_qos else tenants + "\n")
        M.daemon.start_embedded(cfg)
        admin_port = M.daemon.embedded_admin_port()
        env["MCCS_CONTROL"] = prefix + "/control.sock"
        if a.no_qos:
            M.daemon.embedded_admin({"cmd": "qos_set", "enabled": False})
    procs = []
    for ai, app in enumerate(apps):
        for r, dev in enumerate(app["devices"]):
            cmd = [sys.executable, "-m", "mccs_b200.utils.multi_tenant", "--worker", "--app", app["name"],
                   "--comm-id", str(app["comm_id"]), "--rank", str(r), "--nranks", str(len(app["devices"])),
                   "--device", str(dev), "--iters", str(a.iters), "--batch", str(a.batch), "--bytes", str(a.bytes),
                   "--backend", a.backend, "--store-port", str(store.port), "--total-ranks", str(total),
                   "--group-port", str(29700 + ai), "--admin-port", str(admin_port),
                   "--reconfig-at", str(a.reconfig_at if app["name"] == a.reconfig_app else -1)]
            procs.append((app["name"], subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    results: Dict[str, List[dict]] = {}
    failed = False
    for name, p in procs:
        try:
            out, err = p.communicate(timeout=a.timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, err = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"[{name}] exit {p.returncode}\n{err[-2000:]}\n")
        for line in out.splitlines():
            if line.startswith("RESULT "):
                results.setdefault(name, []).append(json.loads(line[7:]))
    summary = {"backend": a.backend, "qos": not a.no_qos and a.backend == "mccs", "setting": a.setting, "iters": a.iters, "batch": a.batch,
               "bytes": a.bytes, "apps": {}}
    for app in apps:
        rs = results.get(app["name"], [])
        if not rs:
            continue
        mean = max(r["mean_ms"] for r in rs)         # the slowest rank defines the app's iteration time
        summary["apps"][app["name"]] = {
            "devices": app["devices"], "weight": app["weight"], "iter_ms": mean,
            "median_ms": max(r["median_ms"] for r in rs), "p99_ms": max(r["p99_ms"] for r in rs),
            "busbw_GBps": a.batch * a.bytes / mean / 1e6 * 2 * (len(app["devices"]) - 1) / max(len(app["devices"]), 1),
            "before_ms": rs[0].get("mean_before_ms"), "after_ms": rs[0].get("mean_after_ms"),
            "config_epoch": rs[0].get("config_epoch"), "async_error": rs[0].get("async_error"), "launch": rs[0].get("launch"),
            "finite": all(r["finite"] for r in rs),
        }
    # Jain's index over weight-normalised throughput (1.0 = shares exactly follow the weights)
    xs = [1.0 / v["iter_ms"] / v["weight"] for v in summary["apps"].values()]
    if xs:
        summary["weighted_fairness"] = sum(xs) ** 2 / (len(xs) * sum(x * x for x in xs))
    if a.backend == "mccs":
        import mccs_b200 as M
        summary["qos_stats"] = M.daemon.embedded_admin({"cmd": "stats"})["stats"]["qos"]["tenants"]
        M.daemon.stop_embedded()
    print(json.dumps(summary))
    return 1 if failed else 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--backend", default="mccs", choices=["mccs", "nccl"])
    ap.add_argument("--iters", type=int, default=1000)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--bytes", type=int, default=8 << 20)
    ap.add_argument("--reconfig-at", type=int, default=500)
    ap.add_argument("--reconfig-app", default="C")
    ap.add_argument("--apps", default="", help="JSON list of {name, comm_id, devices, weight}")
    ap.add_argument("--setting", type=int, default=0, choices=[0, 1, 2, 3, 4],
                    help="placement of the reference's multi-application setting 1-4 instead of the default scenario")
    ap.add_argument("--no-qos", action="store_true")
    ap.add_argument("--sync", default="auto", choices=["auto", "memops", "events"])
    ap.add_argument("--host-devices", type=int, default=4)
    ap.add_argument("--timeout", type=float, default=900.0)
    # worker-only
    ap.add_argument("--app", default="")
    ap.add_argument("--comm-id", type=int, default=0)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--nranks", type=int, default=1)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--store-port", type=int, default=0)
    ap.add_argument("--total-ranks", type=int, default=1)
    ap.add_argument("--group-port", type=int, default=29700)
    ap.add_argument("--admin-port", type=int, default=0)
    a = ap.parse_args()
    return worker(a) if a.worker else orchestrate(a)


if __name__ == "__main__":
    sys.exit(main())
