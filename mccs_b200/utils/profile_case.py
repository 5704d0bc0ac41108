"""A small, self-contained workload for profilers: N ranks on cuda:0 (one cooperative
launch per collective, so a kernel replay by the profiler sees every rank), a few
collectives of one variant, then exit.

    python -m mccs_b200.utils.profile_case --algo ar_twoshot --ranks 4 --mb 256 --dtype bf16 --iters 3
    ncu --set full --clock-control none -k regex:ar_twoshot -s 1 -c 2 -o prof \
        python -m mccs_b200.utils.profile_case --algo ar_twoshot --ranks 4 --mb 256

The buffers are larger than the L2 (126 MB) by default, so DRAM counters mean
something, and stay within a few GB in total. ``--fuse K`` splits the message into K
independent AllReduces issued as one group with fused launches switched on, which is
how the fused kernels (``ar_twoshot_batch``) are reached; ``--algo rs_direct`` runs a
ReduceScatter of the ``--mb`` input. Rank 0 checks the last result
against a plain fp32 sum (or the concatenation) of the ranks' inputs.
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
    ap.add_argument("--fuse", type=int, default=1, help="members per fused launch (AllReduce only)")
    a = ap.parse_args()
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    M.daemon.start_embedded(prefix=f"/tmp/mccs-prof-{os.getpid()}", listen_port=-1,
                            extra=f"fuse_allreduce = {a.fuse}" if a.fuse > 1 else "")
    if M.backend() != "cuda":
        print("profile_case needs a GPU", file=sys.stderr)
        return 1
    n = a.ranks
    nbytes = int(a.mb * 1024 * 1024)
    esz = torch.empty((), dtype=dtype).element_size()
    is_ar = a.algo.startswith("ar_") or a.algo == "auto"
    is_rs = a.algo.startswith("rs_")      # --mb is then the whole input of a rank; each rank keeps 1/ranks of it
    count = nbytes // esz
    block = count // n // 64 * 64         # reduce-scatter: elements per block, 128-byte multiples
    errors = []
    ready = threading.Barrier(n)
    inputs = [None] * n
    parts = max(a.fuse, 1) if is_ar else 1
    part = count // parts // 64 * 64      # elements per member, 128-byte multiples

    def rank_fn(r: int) -> None:
        try:
            torch.cuda.set_device(0)
            torch.cuda.set_stream(torch.cuda.Stream())
            send = M.Buffer(nbytes, 0)
            recv = M.Buffer(nbytes if is_ar or is_rs else nbytes * n, 0)
            s = send.tensor(dtype, count)
            s.copy_(((torch.rand(min(count, 1 << 20)) * 2 - 1).to(dtype)).repeat((count + (1 << 20) - 1) // (1 << 20))[:count])
            inputs[r] = s
            r_all = recv.tensor(dtype, count if is_ar or is_rs else count * n)
            comm = M.Communicator(77, r, n, device=0)
            if a.ctas and r == 0:
                M.reconfigure(M.daemon.embedded_admin_port(), [{"communicator_id": 77, "ctas": a.ctas}])
            ready.wait()
            for _ in range(a.iters):
                if is_ar and parts > 1:
                    with M.group():
                        for k in range(parts):
                            comm.all_reduce(s[k * part:(k + 1) * part], r_all[k * part:(k + 1) * part], algo=a.algo)
                elif is_ar:
                    comm.all_reduce(s, r_all, algo=a.algo)
                elif is_rs:
                    comm.reduce_scatter(s[:block * n], r_all[:block], algo=a.algo)
                else:
                    comm.all_gather(s, r_all, algo=a.algo)
            torch.cuda.synchronize()
            ready.wait()
            if r == 0:
                print("plan:", comm.last_plan(), flush=True)
                m = min(part * parts if is_ar else count, 1 << 22)   # compare the head of the buffers
                if is_rs:
                    m = min(block, 1 << 22)
                    want = torch.stack([x[:m].float() for x in inputs]).sum(0)       # rank 0 keeps block 0
                    tol = 1e-5 if dtype == torch.float32 else 2e-2
                    good = bool(torch.allclose(r_all[:m].float(), want, rtol=tol, atol=tol * n))
                elif is_ar:
                    want = torch.stack([x[:m].float() for x in inputs]).sum(0)
                    tol = 1e-5 if dtype == torch.float32 else 2e-2
                    good = bool(torch.allclose(r_all[:m].float(), want, rtol=tol, atol=tol * n))
                else:
                    good = all(bool(torch.equal(r_all[q * count:q * count + m], inputs[q][:m])) for q in range(n))
                st = M.daemon.embedded_admin({"cmd": "stats"})["stats"]["communicators"]["77"]
                print(f"check: {'ok' if good else 'MISMATCH'}  fused_launches={st['fused_launches']} "
                      f"fused_members={st['fused_members']}", flush=True)
                if not good:
                    errors.append(RuntimeError("result mismatch"))
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
