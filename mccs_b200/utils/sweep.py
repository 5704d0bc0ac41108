"""Collective sweep and tuner: AllReduce / AllGather time versus message size for
every kernel variant and a range of CTA counts, next to NCCL on the same buffers
with the same timing (CUDA events on the launching stream, max over ranks).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m mccs_b200.utils.sweep --out sweep.csv --tuning tuning.json

It is the counterpart of the reference's single-app evaluation
(``eval/single-app/gen_config.py:141-147`` sizes, ``collect.py`` CSV) and of its NCCL
baseline runs (``nccl-tests-mccs/microbenchmark/run_nccl_once.sh``), with the
nccl-tests protocol: sizes 32 KiB to 1 GiB in powers of two, 20 warm-up
and 100 timed iterations for the final numbers (``--mode final``), fewer for the tuning
pass (``--mode tune``) whose result is a tuning table the daemon loads
(``[b200] tuning_file``).

CTA counts are set through the service's live reconfiguration (``ctas`` of a
communicator pattern), so the sweep also exercises that path.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

import mccs_b200 as M
from mccs_b200.utils.timing import bus_factor

AR_ALGOS = ["ar_oneshot", "ar_twoshot", "ar_nvls_oneshot", "ar_nvls_twoshot", "ar_hybrid", "ar_ring"]
AG_ALGOS = ["ag_pull", "ag_push", "ag_nvls", "ag_ring"]
RS_ALGOS = ["rs_direct", "rs_nvls"]
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mult = 1
    for suf, m in (("K", 1 << 10), ("M", 1 << 20), ("G", 1 << 30)):
        if s.endswith(suf):
            mult, s = m, s[:-1]
    return int(float(s) * mult)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", default="32K", help="smallest message")
    ap.add_argument("--max-bytes", default="1G", help="largest message")
    ap.add_argument("--colls", default="allreduce,allgather")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--mode", default="tune", choices=["tune", "final"])
    ap.add_argument("--ctas", default="4,8,16,32,64,128")
    ap.add_argument("--algos", default="")
    ap.add_argument("--warmup", type=int, default=0)
    ap.add_argument("--iters", type=int, default=0)
    ap.add_argument("--out", default="sweep.csv")
    ap.add_argument("--tuning", default="")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--auto-only", action="store_true", help="final mode: measure only the service's own choice (and NCCL)")
    ap.add_argument("--in-place", action="store_true")
    ap.add_argument("--sync", default="auto", choices=["auto", "memops", "events"])
    ap.add_argument("--daemon", default="standalone", choices=["standalone", "embedded"],
                    help="stand-alone mccsd (every rank an outside client) or hosted by local rank 0")
    ap.add_argument("--merge-into", default="", help="also merge the new tuning rows into this JSON file")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n = int(os.environ.get("WORLD_SIZE", "1"))
    # Without a GPU the same script runs over gloo against the host backend (timing on the
    # host clock; the "nccl" column is then gloo): useful to check the tool, not the numbers.
    cuda = torch.cuda.is_available()
    dev = local_rank
    tdev = f"cuda:{dev}" if cuda else "cpu"
    if cuda:
        torch.cuda.set_device(local_rank)
    if n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl" if cuda else "gloo", device_id=torch.device(tdev) if cuda else None)

    def barrier():
        if n > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if n == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=tdev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    prefix = f"/tmp/mccs-sweep-{os.getuid()}-{os.environ.get('MASTER_PORT', '0')}"
    port_file = prefix + "/admin_port"
    spawned = None
    describe = ""
    if local_rank == 0:
        os.makedirs(prefix, exist_ok=True)
        # a tuning pass starts from the built-in table, a final pass uses the measured one
        tuning = "" if args.mode == "tune" else None
        if args.daemon == "embedded":
            M.daemon.start_embedded(prefix=prefix, listen_port=-1, sync=args.sync, tuning_file=tuning)
            port, describe = M.daemon.embedded_admin_port(), M.daemon.describe_embedded()
        else:
            # the deployment shape: a stand-alone mccsd, every rank an outside client
            with open(prefix + "/mccs.toml", "w") as f:
                f.write(M.daemon.default_config(prefix, listen_port=-1, sync=args.sync, tuning_file=tuning))
            spawned = M.daemon.spawn(prefix + "/mccs.toml")
            port, describe = spawned.admin_port, f"stand-alone mccsd ({spawned.backend})"
        with open(port_file, "w") as f:
            f.write(str(port))
    barrier()
    M.init(prefix + "/control.sock")
    admin_port = int(open(port_file).read())
    nvls = True
    if rank == 0:
        stats = M.admin_request(admin_port, {"cmd": "stats"})["stats"]
        nvls = "nvls=on" in stats["backend"]
        print(f"# {describe}: {stats['backend']}", flush=True)
    if n > 1:
        flag = torch.tensor([1 if nvls else 0], device=tdev)
        dist.broadcast(flag, 0)
        nvls = bool(flag.item())

    lo, hi = parse_size(args.min_bytes), parse_size(args.max_bytes)
    sizes = []
    s = lo
    while s <= hi:
        sizes.append(s)
        s *= 2
    # final mode: 20 warm-up and 100 timed calls per point (the median of five groups of 20, see time_ms)
    warm = args.warmup or (20 if args.mode == "final" else 5)
    iters = args.iters or (100 if args.mode == "final" else 20)
    cta_list = [int(x) for x in args.ctas.split(",")] if args.mode == "tune" else [0]
    comm_id = 0x5EE9
    comm = M.Communicator(comm_id, rank, n, device=dev)
    max_bytes = hi
    colls = args.colls.split(",")
    send_buf = M.Buffer(max_bytes, dev)
    recv_buf = M.Buffer(max_bytes, dev)

    def set_ctas(k: int) -> None:
        barrier()
        if rank == 0:
            rep = M.reconfigure(admin_port, [{"communicator_id": comm_id, "ctas": k if k > 0 else -1}])
            assert rep.get("status") == "ok", rep
        barrier()

    def time_ms(fn) -> float:
        for _ in range(warm):
            fn()
        if not cuda:
            import time
            barrier()
            t0 = time.perf_counter()
            for _ in range(iters):
                fn()
            return max_over_ranks((time.perf_counter() - t0) * 1e3 / iters)
        # The timed calls run back to back in `batches` groups, each bracketed by its own pair of
        # events; the figure is the median group (MAX over ranks per group). One mean over all
        # calls lets a single multi-millisecond stall of a shared host (seen for the service and
        # for NCCL alike) pass for the cost of a collective.
        batches = 5 if iters >= 50 else 1
        per = iters // batches
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(batches + 1)]
        stream = torch.cuda.current_stream()
        barrier()
        torch.cuda.synchronize()
        evs[0].record(stream)
        for b in range(batches):
            for _ in range(per):
                fn()
            evs[b + 1].record(stream)
        torch.cuda.synchronize()
        means = sorted(max_over_ranks(evs[b].elapsed_time(evs[b + 1]) / per) for b in range(batches))
        return means[len(means) // 2]

    rows: List[dict] = []
    best: Dict[Tuple[str, int], Tuple[float, str, int]] = {}
    for coll in colls:
        is_ar = coll == "allreduce"
        is_rs = coll == "reducescatter"
        algos = [a for a in (AR_ALGOS if is_ar else RS_ALGOS if is_rs else AG_ALGOS) if nvls or ("nvls" not in a and a != "ar_hybrid")]
        if args.algos:
            algos = [a for a in algos if a in args.algos.split(",")]
        if args.mode == "final":
            algos = ["auto"] + ([] if args.auto_only else algos)
        if n == 1:
            algos = ["auto"]
        for dname in (args.dtypes.split(",") if is_ar or is_rs else ["bytes"]):
            tdtype = DTYPES.get(dname, torch.uint8)
            esz = torch.empty((), dtype=tdtype).element_size()
            for size in sizes:
                # `size` is the message size nccl-tests reports: the reduced buffer for
                # all-reduce, the total gathered bytes for all-gather, the whole input of a
                # rank for reduce-scatter.
                per_rank = size if is_ar else size // n
                per_rank = per_rank // 16 * 16
                if per_rank == 0:
                    continue
                total = per_rank if is_ar else per_rank * n
                count = per_rank // esz
                send = send_buf.tensor(tdtype, count * n if is_rs else count)
                if is_ar:
                    recv = send if args.in_place else recv_buf.tensor(tdtype, count)
                elif is_rs:
                    recv = send[rank * count:(rank + 1) * count] if args.in_place else recv_buf.tensor(tdtype, count)
                else:
                    recv = recv_buf.tensor(tdtype, count * n)
                if tdtype.is_floating_point:
                    g = torch.Generator(device=tdev).manual_seed(rank)
                    ne = send.numel()
                    send.copy_((torch.rand(min(ne, 1 << 22), generator=g, device=tdev) * 2 - 1)
                               .to(tdtype).repeat((ne + (1 << 22) - 1) // (1 << 22))[:ne])
                if n > 1 and not args.no_nccl and (cuda or not is_rs):   # gloo (the CPU dry run) has no reduce-scatter
                    src = send
                    if is_ar:
                        dst = torch.empty_like(src)

                        def nccl_fn():
                            dist.all_reduce(dst)
                    elif is_rs:
                        dst = torch.empty(count, dtype=tdtype, device=tdev)

                        def nccl_fn():
                            dist.reduce_scatter_tensor(dst, src)
                    else:
                        dst = torch.empty(count * n, dtype=tdtype, device=tdev)

                        def nccl_fn():
                            dist.all_gather_into_tensor(dst, src)
                    ms = time_ms(nccl_fn)
                    rows.append({"coll": coll, "dtype": dname, "bytes": total, "algo": "nccl", "ctas": 0,
                                 "ms": ms, "algbw_GBps": total / ms / 1e6,
                                 "busbw_GBps": total / ms / 1e6 * bus_factor(coll, n), "n": n})
                    del dst
                for algo in algos:
                    if algo in ("ar_oneshot", "ar_nvls_oneshot") and (total > (8 << 20) or args.in_place):
                        continue
                    if "ring" in algo and total > (64 << 20):
                        continue   # the FIFO ring is a fall-back path: not worth minutes of sweep time
                    for k in (cta_list if "ring" not in algo else [0]):
                        set_ctas(k)

                        def fn():
                            if is_ar:
                                comm.all_reduce(send, recv, algo=algo)
                            elif is_rs:
                                comm.reduce_scatter(send, recv, algo=algo)
                            else:
                                comm.all_gather(send, recv, algo=algo)
                        try:
                            ms = time_ms(fn)
                        except Exception as e:  # noqa: BLE001
                            if rank == 0:
                                print(f"# {coll} {dname} {total} {algo} ctas={k}: {e}", flush=True)
                            raise
                        variant, ctas = comm.last_plan()
                        row = {"coll": coll, "dtype": dname, "bytes": total, "algo": variant, "ctas": ctas,
                               "ms": ms, "algbw_GBps": total / ms / 1e6,
                               "busbw_GBps": total / ms / 1e6 * bus_factor(coll, n), "n": n}
                        rows.append(row)
                        if variant == algo or algo == "auto":
                            # The tuning table is indexed by message bytes; keep the best of
                            # the 16-bit runs (the common case) and of any dtype otherwise.
                            key = (coll, total)
                            if key not in best or ms < best[key][0]:
                                best[key] = (ms, variant, ctas)
                if rank == 0:
                    last = [r for r in rows if r["bytes"] == total and r["coll"] == coll and r["dtype"] == dname]
                    top = min((r for r in last if r["algo"] != "nccl"), key=lambda r: r["ms"], default=None)
                    nc = next((r for r in last if r["algo"] == "nccl"), None)
                    if top:
                        print(f"{coll} {dname} {total:>11d} B  best {top['algo']:>16s} x{top['ctas']:<3d} "
                              f"{top['ms'] * 1e3:9.1f} us  bus {top['busbw_GBps']:7.1f} GB/s"
                              + (f"  | nccl {nc['ms'] * 1e3:9.1f} us bus {nc['busbw_GBps']:7.1f} GB/s" if nc else ""),
                              flush=True)
    set_ctas(0)
    if rank == 0:
        with open(args.out, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=["coll", "dtype", "n", "bytes", "algo", "ctas", "ms", "algbw_GBps", "busbw_GBps"])
            w.writeheader()
            for r in rows:
                w.writerow(r)
        if args.tuning and args.mode == "tune":
            table: Dict[str, Dict[str, list]] = {"allreduce": {}, "allgather": {}, "reducescatter": {}}
            for coll in colls:
                ent = sorted((b, v) for (c, b), v in best.items() if c == coll)
                table[coll][str(n)] = [[b, v[1], v[2], 512] for b, v in ent]
                if table[coll][str(n)]:
                    table[coll][str(n)][-1][0] = -1
            with open(args.tuning, "w") as f:
                json.dump(table, f, indent=1)
            if args.merge_into:
                merged = {"allreduce": {}, "allgather": {}, "reducescatter": {}}
                if os.path.exists(args.merge_into):
                    with open(args.merge_into) as f:
                        merged.update(json.load(f))
                for coll in table:
                    merged.setdefault(coll, {}).update({k: v for k, v in table[coll].items() if v})
                with open(args.merge_into, "w") as f:
                    json.dump(merged, f, indent=1)
    comm.destroy()
    send_buf.free()
    recv_buf.free()
    M.finalize()
    barrier()
    if local_rank == 0:
        if spawned is not None:
            spawned.stop()
        else:
            M.daemon.stop_embedded()
    if n > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
