#!/usr/bin/env python
"""Headline benchmark: AllReduce algorithm bandwidth of a 512 MiB 16-bit message
through the managed service, the configuration of the reference's single-app figure
(``eval/plot/single_app/allreduce_8gpu.csv``: fp16, 512 MiB, 8 GPUs, MCCS algBW
5.99 GB/s on 4x2 RTX 3090 over 50 Gb/s RoCE).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

One step = one AllReduce(sum) of ``--size-mb`` MiB of bf16 per rank, out of place,
issued through the public client API (libmccs -> daemon -> sm_100a kernel). The local
rank 0 starts a stand-alone ``mccsd`` (the deployment the service is made for: one daemon
per box, applications in their own processes); every rank is a client. Timing: CUDA
events on the launching stream around exactly K steps, barrier + synchronise on both
sides, MAX over ranks. The message (512 MiB) is larger than the 126 MB L2, so no
flush is needed between iterations. The ``e2e`` figure adds, every step, the
host->device copy of the input from pinned memory and a device->host read of the head
of the result. After the timed steps a sample spread over the whole output (first and last
elements, the shard boundaries, evenly spaced windows) is compared with a plain fp32 sum of
the ranks' inputs; a mismatch makes the run fail.

``--impl reference`` runs the reference's own NCCL baseline harness
(``nccl-tests-mccs`` built unmodified into ``baseline/_ref``) for the same message.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

BASELINE_ALGBW_GBPS = 5.99   # MCCS, AllReduce fp16 512 MiB, 8 GPUs, as published by the reference (RTX 3090 testbed)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="mccs", choices=["mccs", "reference"])
    p.add_argument("--size-mb", type=float, default=512.0)
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    p.add_argument("--coll", default="allreduce", choices=["allreduce", "allgather"])
    p.add_argument("--algo", default="auto")
    p.add_argument("--no-nccl", action="store_true", help="skip the same-harness NCCL measurement")
    return p.parse_args()


def job_config(args, nbytes: int, n: int) -> dict:
    """The work of one step, in the same words for both arms."""
    return {"model": f"{args.coll} sum, {nbytes / 2**20:g} MiB {args.dtype} per rank, out of place",
            "global_batch": nbytes * n, "seq_len": 1, "parallelism": f"dp{n}"}


def reference_e2e(args, rank: int, world: int, size: int):
    """End-to-end figure for the reference arm. Its harness (nccl-tests) has no per-step host
    copy, so the same NCCL library is driven through torch.distributed here: pinned host ->
    device copy of the input, all_reduce, device -> host read of the head of the result, every
    step. Nothing of this repository is on that path."""
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        return None
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    tdtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    esz = torch.empty((), dtype=tdtype).element_size()
    count = size // esz
    pinned = torch.empty(count, dtype=tdtype, pin_memory=True)
    pinned.fill_(0.5)
    src = torch.empty(count, dtype=tdtype, device="cuda")
    d2h = min(count, 32768)
    host = torch.empty(d2h, dtype=tdtype, pin_memory=True)
    is_ar = args.coll == "allreduce"
    dst = src if is_ar else torch.empty(count * world, dtype=tdtype, device="cuda")

    def step():
        src.copy_(pinned, non_blocking=True)
        if world > 1:
            dist.all_reduce(src) if is_ar else dist.all_gather_into_tensor(dst, src)
        elif not is_ar:
            dst.copy_(src)
        host.copy_(dst[:d2h], non_blocking=True)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.destroy_process_group()
    total = size if is_ar else size * world
    return {"value": total / ms / 1e6, "unit": "GB/s", "ms_per_step": ms, "h2d_bytes_per_step": size,
            "d2h_bytes_per_step": d2h * esz,
            "how": "pinned H2D copy + NCCL collective via torch.distributed (the library the reference harness links) + D2H read"}


def reference_arm(args, rank: int) -> int:
    """The reference's NCCL baseline harness, unmodified, single process, -g N. The ranks
    other than 0 of a torchrun launch only take part in the end-to-end figure, after the
    harness has finished (they block in the process-group rendezvous until rank 0 joins)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    size = int(args.size_mb * 1024 * 1024)
    out = {"impl": "reference"}
    if rank == 0:
        out.update(run_reference_harness(args, size))
    try:
        e2e = reference_e2e(args, rank, world, size)
        if e2e and "unavailable" not in out:
            out["e2e"] = e2e
    except Exception as e:  # noqa: BLE001
        out["e2e_unavailable"] = str(e)[:200]
    if rank == 0:
        print(json.dumps(out))
    return 0


def run_reference_harness(args, size: int) -> dict:
    exe = os.path.join(REPO, "baseline", "_ref", "nccl-tests-mccs", "build",
                       "all_reduce_perf" if args.coll == "allreduce" else "all_gather_perf")
    if not os.path.exists(exe):
        return {"unavailable": "the reference is a Rust workspace (no setup.py/pyproject; needs cargo, libibverbs, "
                               "gdrcopy) and its nccl-tests-mccs harness is not built in baseline/_ref"}
    dt = {"bf16": "bfloat16", "fp16": "half", "fp32": "float"}[args.dtype]
    env = dict(os.environ)
    import glob
    libs = glob.glob(os.path.join(sys.prefix, "lib", "python*", "site-packages", "nvidia", "*", "lib"))
    libs.append("/usr/local/cuda/lib64")
    env["LD_LIBRARY_PATH"] = ":".join(libs + [env.get("LD_LIBRARY_PATH", "")])
    cmd = [exe, "-g", str(args.gpus), "-b", str(size), "-e", str(size), "-d", dt, "-n", str(args.steps),
           "-w", str(max(args.warmup, 3)), "-c", "0"]
    try:
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"nccl-tests-mccs failed to run: {e}"}
    alg, t_us = None, None
    for line in res.stdout.splitlines():
        f = line.split()
        # size count type redop root | time algbw busbw #wrong | time algbw busbw #wrong (out of place, then in place)
        if len(f) >= 8 and f[0].isdigit() and int(f[0]) == size:
            try:
                t_us, alg = float(f[-8]), float(f[-7])
            except (ValueError, IndexError):
                pass
    if alg is None:
        tail = (res.stderr.strip() or res.stdout.strip())[-200:].replace("\n", " | ")
        return {"unavailable": "nccl-tests-mccs produced no result row: " + tail}
    return {
        "ms_per_step": t_us / 1000.0,
        "metric": f"{args.coll}_algbw_GBps", "value": alg, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": alg / BASELINE_ALGBW_GBPS, "dtype": args.dtype, "data": "synthetic",
        "config": job_config(args, size, args.gpus),
        "detail": {"harness": "NCCL via the reference's nccl-tests-mccs, host-timed by that harness, single process -g N"},
    }


def main() -> int:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return reference_arm(args, rank)

    import torch
    import torch.distributed as dist

    import mccs_b200 as M
    from mccs_b200.utils.timing import ClockSampler, bus_factor

    n = world
    if n != args.gpus and rank == 0:
        print(f"bench.py: WORLD_SIZE={world} differs from --gpus {args.gpus}; using {world}", file=sys.stderr)
    have_cuda = torch.cuda.is_available()
    if have_cuda:
        torch.cuda.set_device(local_rank)
    if n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if have_cuda:
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        else:
            dist.init_process_group("gloo")

    def barrier():
        if n > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if n == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local_rank}" if have_cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    port = os.environ.get("MASTER_PORT", "0")
    prefix = f"/tmp/mccs-bench-{os.getuid()}-{port}-{os.environ.get('TORCHELASTIC_RUN_ID', os.getppid() if n > 1 else os.getpid())}"
    control = prefix + "/control.sock"
    spawned = None
    if local_rank == 0:
        os.makedirs(prefix, exist_ok=True)
        with open(prefix + "/mccs.toml", "w") as f:
            f.write(M.daemon.default_config(prefix, channel_count=2, host_devices=max(n, 1), listen_port=-1,
                                            force_host=not have_cuda))
        spawned = M.daemon.spawn(prefix + "/mccs.toml")
    barrier()
    M.init(control)
    backend = M.backend()
    dev = local_rank

    tdtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    esz = torch.empty((), dtype=tdtype).element_size()
    nbytes = int(args.size_mb * 1024 * 1024)
    if backend == "host":
        nbytes = min(nbytes, 8 << 20)   # CPU dry run of the script only
    count = nbytes // esz
    is_ar = args.coll == "allreduce"
    send_buf = M.Buffer(nbytes, dev)
    recv_buf = M.Buffer(nbytes if is_ar else nbytes * n, dev)
    send = send_buf.tensor(tdtype, count)
    recv = recv_buf.tensor(tdtype, count if is_ar else count * n)
    gen = torch.Generator(device="cpu").manual_seed(rank)
    pinned = torch.empty(count, dtype=tdtype, pin_memory=have_cuda)
    chunk = 1 << 24
    for off in range(0, count, chunk):   # U(-1, 1), seed = rank
        m = min(chunk, count - off)
        pinned[off:off + m] = (torch.rand(m, generator=gen) * 2 - 1).to(tdtype)
    send.copy_(pinned)
    comm = M.Communicator(0xB200, rank, n, device=dev)

    def step():
        if is_ar:
            comm.all_reduce(send, recv, algo=args.algo)
        else:
            comm.all_gather(send, recv, algo=args.algo)

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    # clocks are sampled from before the warm-up to after the last timed step
    sampler = ClockSampler(dev, period_ms=100) if (have_cuda and local_rank == 0) else None
    if sampler:
        sampler.start()
    for _ in range(warmup):
        step()
    if have_cuda:
        torch.cuda.synchronize()

    # What is checked after the timed steps: windows of the output spread over the whole
    # buffer (its first and last elements, both sides of every shard boundary, evenly spaced
    # ones in between) against a plain fp32 sum of all ranks' inputs at the same places.
    win = min(count, 4096)
    starts = {0, count - win}
    for k in range(1, 32):
        starts.add(min(count - win, (count * k // 32) // 8 * 8))
    for r in range(1, n):
        edge = count * r // n
        starts.add(max(0, min(count - win, edge - win // 2)))
    starts = sorted(starts)
    idx = torch.cat([torch.arange(s0, s0 + win) for s0 in starts]).to(send.device)

    def verify() -> bool:
        if have_cuda:
            torch.cuda.synchronize()
        mine = send[idx].float()
        if n > 1:
            gathered = [torch.empty_like(mine) for _ in range(n)]
            dist.all_gather(gathered, mine)
        else:
            gathered = [mine]
        good = True
        if is_ar:
            want = torch.stack(gathered).sum(0)
            got = recv[idx].float()
            tol = 1e-5 if tdtype == torch.float32 else 2e-2
            good = bool(torch.allclose(got, want, rtol=tol, atol=tol * n)) and bool(torch.isfinite(got).all())
        else:
            for r in range(n):
                good = good and bool(torch.equal(recv[idx + r * count].float(), gathered[r]))
        flag = torch.tensor([1.0 if good else 0.0], dtype=torch.float64, device=send.device)
        if n > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item() > 0.5)

    # the warm-up results must not be what passes the check
    recv.fill_(float("nan"))
    if have_cuda:
        torch.cuda.synchronize()

    def timed(fn) -> float:
        if not have_cuda:
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                fn()
            dt = (time.perf_counter() - t0) * 1000 / steps
            barrier()
            return max_over_ranks(dt)
        stream = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    ms = timed(step)
    ok = verify()
    variant, ctas = comm.last_plan()
    launch_mode = comm.launch_mode

    # End to end: input arrives from pinned host memory and the result is read back, every step.
    d2h_elems = min(count, 32768)
    result_host = torch.empty(d2h_elems, dtype=tdtype, pin_memory=have_cuda)

    def e2e_step():
        send.copy_(pinned, non_blocking=True)
        step()
        result_host.copy_(recv[:d2h_elems], non_blocking=True)

    for _ in range(2):
        e2e_step()
    recv.fill_(float("nan"))
    ms_e2e = timed(e2e_step)
    ok = verify() and ok
    clocks = sampler.stop() if sampler else None

    # Same harness, NCCL (the baseline the service has to match on this box).
    nccl = None
    if n > 1 and have_cuda and not args.no_nccl:
        src = torch.empty(count, dtype=tdtype, device=f"cuda:{dev}").copy_(send)
        if is_ar:
            def nccl_step():
                dist.all_reduce(src)
        else:
            dst = torch.empty(count * n, dtype=tdtype, device=f"cuda:{dev}")

            def nccl_step():
                dist.all_gather_into_tensor(dst, src)
        for _ in range(warmup):
            nccl_step()
        ms_nccl = timed(nccl_step)
        total = nbytes if is_ar else nbytes * n
        nccl = {"ms_per_step": ms_nccl, "algbw_GBps": total / ms_nccl / 1e6,
                "busbw_GBps": total / ms_nccl / 1e6 * bus_factor(args.coll, n)}

    total_bytes = nbytes if is_ar else nbytes * n
    alg = total_bytes / ms / 1e6          # GB/s
    alg_e2e = total_bytes / ms_e2e / 1e6
    comm.destroy()
    send_buf.free()
    recv_buf.free()
    M.finalize()
    barrier()
    if spawned is not None:
        spawned.stop()
    if rank == 0:
        out = {
            "metric": f"{args.coll}_algbw_GBps", "value": alg, "unit": "GB/s", "n_gpus": n, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": alg / BASELINE_ALGBW_GBPS, "dtype": args.dtype, "data": "synthetic",
            "impl": "mccs",
            "busbw_GBps": alg * bus_factor(args.coll, n),
            "config": job_config(args, nbytes, n),
            "detail": {
                "path": "libmccs client -> stand-alone mccsd -> sm_100a kernel",
                "variant": variant, "ctas": ctas, "backend": backend, "launch": launch_mode,
                "l2": "inputs larger than L2 (no flush)", "timing": "CUDA events, max over ranks",
                "verified": ok, "verified_elements": int(idx.numel()),
            },
            "clocks": clocks,
            "e2e": {"value": alg_e2e, "unit": "GB/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": d2h_elems * esz},
            # one collective kernel per rank and step (launched by each rank's own library when
            # "launch" is "client", by the daemon's proxy threads otherwise)
            "gpu_launches": steps * n,
            "nccl_same_harness": nccl,
        }
        print(json.dumps(out))
    if n > 1:
        dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
