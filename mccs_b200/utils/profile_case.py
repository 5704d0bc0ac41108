"""A small, self-contained workload for profilers: N ranks on cuda:0 (one cooperative
launch per collective, so a kernel replay by the profiler sees every rank), a few
collectives of one variant, then exit.

    python -m mccs_b200.utils.profile_case --algo ar_twoshot --ranks 4 --mb 256 --dtype bf16 --iters 3
    ncu --set full --clock-control none -k regex:ar_twoshot -s 1 -c 2 -o prof \
        python -m mccs_b200.utils.profile_case --algo ar_twoshot --ranks 4 --mb 256

The buffers are larger than the L2 (126 MB) by default, so DRAM counters mean
something, and stay within a few GB in total.
"""
from __future__ import annotations

import argparse
import os
import sys
import threading

import torch

import mccs_b200 as M


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--algo", default="ar_twoshot")
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--mb", type=float, default=256.0, help="message size per rank in MiB")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--ctas", type=int, default=0)
    a = ap.parse_args()
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    M.daemon.start_embedded(prefix=f"/tmp/mccs-prof-{os.getpid()}", listen_port=-1)
    if M.backend() != "cuda":
        print("profile_case needs a GPU", file=sys.stderr)
        return 1
    n = a.ranks
    nbytes = int(a.mb * 1024 * 1024)
    esz = torch.empty((), dtype=dtype).element_size()
    is_ar = a.algo.startswith("ar_") or a.algo == "auto"
    count = nbytes // esz
    errors = []
    ready = threading.Barrier(n)

    def rank_fn(r: int) -> None:
        try:
            torch.cuda.set_device(0)
            torch.cuda.set_stream(torch.cuda.Stream())
            send = M.Buffer(nbytes, 0)
            recv = M.Buffer(nbytes if is_ar else nbytes * n, 0)
            s = send.tensor(dtype, count)
            s.copy_(((torch.rand(min(count, 1 << 20)) * 2 - 1).to(dtype)).repeat((count + (1 << 20) - 1) // (1 << 20))[:count])
            comm = M.Communicator(77, r, n, device=0)
            if a.ctas and r == 0:
                M.reconfigure(M.daemon.embedded_admin_port(), [{"communicator_id": 77, "ctas": a.ctas}])
            ready.wait()
            for _ in range(a.iters):
                if is_ar:
                    comm.all_reduce(s, recv.tensor(dtype, count), algo=a.algo)
                else:
                    comm.all_gather(s, recv.tensor(dtype, count * n), algo=a.algo)
            torch.cuda.synchronize()
            if r == 0:
                print("plan:", comm.last_plan(), flush=True)
            ready.wait()
            comm.destroy()
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    ths = [threading.Thread(target=rank_fn, args=(r,)) for r in range(n)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    M.finalize()
    M.daemon.stop_embedded()
    if errors:
        raise errors[0]
    return 0


if __name__ == "__main__":
    sys.exit(main())
