"""Where does the time of a small collective go? Runs back-to-back AllReduces (or
AllGathers) of one small size through the service with the daemon's tracer on, then
splits the per-call period into its stages from the daemon's trace and the kernels'
own ``globaltimer`` stamps:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m mccs_b200.utils.latency --bytes 64K --iters 300

    period            CUDA events on the client's stream, per call, max over ranks
    rendezvous        request taken from a rank's ring -> all ranks arrived and planned
    wait for clients  planned -> every client's stream has reached the collective
    launch            gates passed -> kernel (and the "done" write) queued
    kernel            device time between the kernel's first and last instruction
    hand-over         device time from the end of one kernel to the start of the next:
                      "done" reaches the client's stream, its next "submitted" reaches
                      the proxy, the launch reaches the GPU

The reference only has commented-out timing hints in its daemon loop
(src/mccs/src/daemon/engine.rs:284-309). Without a GPU the same script runs on the
host backend (gloo ranks), where only the host-side stages mean anything.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from typing import Dict, List

import torch
import torch.distributed as dist

import mccs_b200 as M
from mccs_b200.utils.sweep import parse_size


def summarise(events: List[dict], comm_id: int, skip: int) -> Dict[str, dict]:
    """Per-stage statistics (µs) from chrome-trace events of one communicator."""
    stages: Dict[str, List[float]] = {"rendezvous": [], "wait for clients": [], "launch": []}
    device: Dict[int, List[tuple]] = {}
    for e in events:
        if e.get("pid") != comm_id:
            continue
        name = e["name"]
        if name.startswith("device "):
            device.setdefault(int(e["tid"]) - 1000, []).append((float(e["ts"]), float(e["dur"])))
            continue
        seq = int(name.rsplit("#", 1)[1])
        if seq < skip:
            continue
        if name.startswith("rendezvous"):
            stages["rendezvous"].append(float(e["dur"]))
        elif name.startswith("wait for clients"):
            stages["wait for clients"].append(float(e["dur"]))
        elif name.startswith("admit+launch"):
            stages["launch"].append(float(e["dur"]))
    kernel: List[float] = []
    gap: List[float] = []
    for _, spans in device.items():
        spans = sorted(set(spans))[skip:]
        kernel += [d for _, d in spans]
        gap += [spans[i + 1][0] - (spans[i][0] + spans[i][1]) for i in range(len(spans) - 1)]
    stages["kernel"] = kernel
    stages["hand-over"] = [g for g in gap if g >= 0]

    def stat(xs: List[float]) -> dict:
        if not xs:
            return {"n": 0}
        xs = sorted(xs)
        return {"n": len(xs), "median_us": statistics.median(xs), "mean_us": statistics.fmean(xs),
                "p90_us": xs[int(len(xs) * 0.9) - 1] if len(xs) >= 10 else xs[-1]}
    return {k: stat(v) for k, v in stages.items()}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", default="64K")
    ap.add_argument("--coll", default="allreduce", choices=["allreduce", "allgather", "reducescatter"])
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--iters", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--sync", default="auto", choices=["auto", "memops", "events"])
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of a table")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    dev = local_rank
    if cuda:
        torch.cuda.set_device(dev)
    if n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl" if cuda else "gloo", device_id=torch.device(f"cuda:{dev}") if cuda else None)

    def barrier():
        if n > 1:
            dist.barrier()

    prefix = f"/tmp/mccs-lat-{os.getuid()}-{os.environ.get('MASTER_PORT', '0')}"
    spawned = None
    if local_rank == 0:
        os.makedirs(prefix, exist_ok=True)
        with open(prefix + "/mccs.toml", "w") as f:
            f.write(M.daemon.default_config(prefix, listen_port=-1, sync=args.sync, trace=True, host_devices=max(n, 1),
                                            force_host=not cuda))
        spawned = M.daemon.spawn(prefix + "/mccs.toml")
        with open(prefix + "/admin_port", "w") as f:
            f.write(str(spawned.admin_port))
    barrier()
    M.init(prefix + "/control.sock")
    admin_port = int(open(prefix + "/admin_port").read())

    nbytes = parse_size(args.bytes)
    is_ar = args.coll == "allreduce"
    is_rs = args.coll == "reducescatter"     # --bytes is then the whole input of a rank
    count = nbytes // 4 if is_ar else max(nbytes // 4 // n, 1) if is_rs else nbytes // n
    send = M.Buffer(max(nbytes, 16), dev)
    recv = M.Buffer(max(nbytes, 16), dev)
    comm_id = 0x1A7
    comm = M.Communicator(comm_id, rank, n, device=dev)
    if is_rs:
        s, r = send.tensor(torch.float32, count * n), recv.tensor(torch.float32, count)
    else:
        s = send.tensor(torch.float32, count) if is_ar else send.tensor(torch.uint8, count)
        r = recv.tensor(torch.float32, count) if is_ar else recv.tensor(torch.uint8, count * n)
    s.fill_(1)

    def call():
        if is_ar:
            comm.all_reduce(s, r, algo=args.algo)
        elif is_rs:
            comm.reduce_scatter(s, r, algo=args.algo)
        else:
            comm.all_gather(s, r, algo=args.algo)

    for _ in range(args.warmup):
        call()
    if cuda:
        torch.cuda.synchronize()
    barrier()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        period_us = e0.elapsed_time(e1) * 1e3 / args.iters
    else:
        import time
        t0 = time.perf_counter()
        for _ in range(args.iters):
            call()
        period_us = (time.perf_counter() - t0) * 1e6 / args.iters
    if n > 1:
        t = torch.tensor([period_us], dtype=torch.float64, device=f"cuda:{dev}" if cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        period_us = float(t.item())
    variant, ctas = comm.last_plan()
    barrier()
    if rank == 0:
        rep = M.admin_request(admin_port, {"cmd": "trace", "enabled": False, "inline": True})
        stages = summarise(rep["trace"]["traceEvents"], comm_id, args.warmup)
        out = {"coll": args.coll, "bytes": nbytes, "n": n, "variant": variant, "ctas": ctas,
               "backend": M.backend(), "launch": comm.launch_mode, "period_us": period_us, "stages": stages}
        if args.json:
            print(json.dumps(out))
        else:
            print(f"{args.coll} {nbytes} B on {n} rank(s), {variant} x{ctas}, {M.backend()} backend: "
                  f"{period_us:.1f} us per call")
            for k, v in stages.items():
                if v["n"]:
                    print(f"  {k:18s} median {v['median_us']:8.1f}  mean {v['mean_us']:8.1f}  p90 {v['p90_us']:8.1f} us  (n={v['n']})")
                else:
                    print(f"  {k:18s} no samples")
    barrier()
    comm.destroy()
    send.free()
    recv.free()
    M.finalize()
    barrier()
    if spawned is not None:
        spawned.stop()
    if n > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
