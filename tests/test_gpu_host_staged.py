"""The host-staged transport on a GPU, and the allocation hook under a real CUDA program.

Host-staged is this service's form of the reference's intra-host shared-memory transport
(src/mccs/src/transport/shm/transporter.rs:39-181): every hop of the ring goes through
FIFO slots and flags in pinned host memory instead of peer device memory. The test is the
plumbing check the reference's proto apps make (src/mccs_examples/allreduce_proto/src/main.rs:75-116):
a stand-alone daemon with `[b200] transport = "host_staged"`, two client processes, a ring
AllReduce of 262 144 fp32 values drawn from N(0,1) and a ring AllGather of 65 536 values
`rank * 1e6 + index` per rank, compared with numpy at rtol 1e-5. With one GPU both ranks sit
on cuda:0 (one cooperative launch by the daemon), with two or more each rank has its own.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import NATIVE, REPO, write_config

pytestmark = pytest.mark.gpu

CLIENT = r"""
import os, sys, json
import numpy as np, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); dev = int(os.environ["DEV"])
torch.cuda.set_device(dev)
rng = np.random.default_rng(0)
inputs = [rng.standard_normal(262144).astype(np.float32) for _ in range(n)]     # every process draws all ranks' data
send = M.Buffer(262144 * 4, dev); recv = M.Buffer(262144 * 4 * n, dev)
comm = M.Communicator(7100, rank, n, device=dev)
s = send.tensor(torch.float32, 262144); d = recv.tensor(torch.float32, 262144)
s.copy_(torch.from_numpy(inputs[rank]))
res = {}
for rep in range(70):          # more than the daemon queues ahead of the GPU (48): it must see every kernel's completion word
    comm.all_reduce(s, d)
torch.cuda.synchronize()
res["ar_plan"] = comm.last_plan()[0]
want = np.sum(np.stack(inputs).astype(np.float64), axis=0)
res["ar_ok"] = bool(np.allclose(d.cpu().numpy(), want, rtol=1e-5, atol=1e-6))
g_in = send.tensor(torch.float32, 65536); g_out = recv.tensor(torch.float32, 65536 * n)
g_in.copy_(torch.arange(65536, dtype=torch.float32) + rank * 1e6)
comm.all_gather(g_in, g_out)
torch.cuda.synchronize()
res["ag_plan"] = comm.last_plan()[0]
want = np.concatenate([np.arange(65536, dtype=np.float32) + r * 1e6 for r in range(n)])
res["ag_ok"] = bool(np.allclose(g_out.cpu().numpy(), want, rtol=1e-5))
# in place, and a size that needs several trips around the FIFO (4 MiB of slots per channel)
big_buf = M.Buffer(24 << 20, dev)        # the object owns the memory: it must outlive its tensors
big = big_buf.tensor(torch.float32, 6 << 20)
big.fill_(float(rank + 1))
comm.all_reduce(big)
torch.cuda.synchronize()
res["big_ok"] = bool(torch.all(big == float(n * (n + 1) // 2)))
q = comm.query()
res["async_error"] = q["async_error"]; res["device_error"] = q["device_error"]; res["launch"] = comm.launch_mode
comm.destroy()
print("RESULT", json.dumps(res), flush=True)
"""


def test_host_staged_transport_two_ranks(tmp_path):
    from mccs_b200 import daemon
    ngpu = torch.cuda.device_count()
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), transport="host_staged", listen_port=-1,
                       wait_timeout_ms=5000)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        assert sp.backend == "cuda"
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE="2", MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="30000")
        procs = [subprocess.Popen([sys.executable, "-c", CLIENT], env=dict(env, RANK=str(r), DEV=str(r if ngpu >= 2 else 0)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
        for p in procs:
            out, err = p.communicate(timeout=240)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["ar_plan"] == "ar_ring" and res["ag_plan"] == "ag_ring"     # the FIFO variants are the transport
            assert res["ar_ok"] and res["ag_ok"] and res["big_ok"]
            assert res["async_error"] == 0 and res["device_error"] == 0
            assert res["launch"] == "daemon"        # pinned host FIFOs are not exported to clients
    finally:
        sp.stop()


PRELOAD_APP = r"""
// An application that knows nothing of mccsMalloc: plain cudaMalloc / cudaMemcpy / cudaFree,
// then a collective on those pointers. Run with LD_PRELOAD=libmccs_preload.so.
#include <cuda_runtime.h>
#include <stdio.h>
#include <vector>
#include "mccs.h"
int main() {
  const size_t n = 1 << 20;   // 4 MiB per buffer: above the hook's threshold
  float *a = nullptr, *b = nullptr, *small = nullptr;
  if (cudaMalloc((void**)&a, n * 4) || cudaMalloc((void**)&b, n * 4) || cudaMalloc((void**)&small, 1024)) return 2;
  uint64_t id = 0;
  const int big_ours = mccsMemInfo(a, &id, nullptr, nullptr) == mccsSuccess && mccsMemInfo(b, &id, nullptr, nullptr) == mccsSuccess;
  const int small_ours = mccsMemInfo(small, &id, nullptr, nullptr) == mccsSuccess;
  std::vector<float> h(n);
  for (size_t i = 0; i < n; i++) h[i] = (float)(i % 1000) * 0.5f;
  if (cudaMemcpy(a, h.data(), n * 4, cudaMemcpyHostToDevice)) return 3;
  mccsComm_t comm = nullptr;
  if (mccsCommInitRank(&comm, 7200, 0, 1, 0, nullptr) != mccsSuccess) return 4;
  cudaStream_t s; cudaStreamCreate(&s);
  if (mccsAllReduce(comm, a, b, n, mccsFloat32, mccsSum, s) != mccsSuccess) return 5;
  if (cudaStreamSynchronize(s)) return 6;
  std::vector<float> out(n);
  if (cudaMemcpy(out.data(), b, n * 4, cudaMemcpyDeviceToHost)) return 7;
  int same = 1;
  for (size_t i = 0; i < n; i++) if (out[i] != h[i]) { same = 0; break; }
  mccsCommDestroy(comm);
  const int freed = cudaFree(a) == 0 && cudaFree(b) == 0 && cudaFree(small) == 0;
  const int gone = mccsMemInfo(a, &id, nullptr, nullptr) != mccsSuccess;
  printf("big_ours=%d small_ours=%d same=%d freed=%d gone=%d\n", big_ours, small_ours, same, freed, gone);
  return 0;
}
"""


def test_preload_hook_under_a_cuda_program(tmp_path):
    """`libmccs_preload.so` in front of the real CUDA runtime: the program's large
    cudaMalloc results are service memory and usable in a collective as they are."""
    import shutil
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc on this machine to build the CUDA program")
    from mccs_b200 import daemon
    (tmp_path / "app.cu").write_text(PRELOAD_APP)
    inc = os.path.join(REPO, "csrc", "include")
    build = subprocess.run([nvcc, "-cudart", "shared", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + inc, "-o", str(tmp_path / "app"),
                            str(tmp_path / "app.cu"), "-L" + NATIVE, "-lmccs", "-Xlinker", "-rpath," + NATIVE],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    cfg = write_config(os.path.join(str(tmp_path), "mccs.toml"), os.path.join(str(tmp_path), "sock"), listen_port=-1)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        env = dict(os.environ, LD_PRELOAD=os.path.join(NATIVE, "libmccs_preload.so"), MCCS_CONTROL=sp.control,
                   MCCS_PRELOAD_MIN_BYTES=str(1 << 20), MCCS_LOG="error")
        res = subprocess.run([str(tmp_path / "app")], env=env, capture_output=True, text=True, timeout=120)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "big_ours=1 small_ours=0 same=1 freed=1 gone=1" in res.stdout, res.stdout + res.stderr
    finally:
        sp.stop()


FUSED_CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); dev = int(os.environ["DEV"]); port = int(os.environ["ADMIN_PORT"])
torch.cuda.set_device(dev)
bufs = [M.Buffer((1 << 20) + 4096 * k, dev) for k in range(6)]
ts = [b.tensor(torch.float32, (1 << 18) + 1024 * k) for k, b in enumerate(bufs)]     # six members of different sizes
comm = M.Communicator(7300, rank, n, device=dev)
bad = []
for rnd in range(4):
    for k, t in enumerate(ts):
        t.fill_(float(rank + 1 + k + rnd))
    with M.group():                       # queued together: the daemon may carry them in one launch
        for t in ts:
            comm.all_reduce(t, algo="ar_twoshot")
    torch.cuda.synchronize()
    for k, t in enumerate(ts):
        want = float(sum(r + 1 + k + rnd for r in range(n)))
        if not bool(torch.all(t == want)):
            bad.append((rnd, k, float(t[0]), want))
q = comm.query()
st = M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"]["7300"]
comm.destroy()
print("RESULT", json.dumps({"bad": bad[:4], "async_error": q["async_error"], "device_error": q["device_error"],
                            "fused_launches": st["fused_launches"], "fused_members": st["fused_members"], "launch": comm.launch_mode}), flush=True)
"""


def test_fused_launches_on_a_gpu(tmp_path):
    """`[b200] fuse_allreduce = 4` with daemon launches: AllReduces queued together in a group
    go out as fused kernels (one pair of cross-rank barriers for up to four of them), and every
    member's result is right. Two ranks; on one GPU both sit on cuda:0 (cooperative launch)."""
    from mccs_b200 import daemon
    ngpu = torch.cuda.device_count()
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, wait_timeout_ms=5000,
                       extra='launch = "daemon"\nfuse_allreduce = 4')
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE="2", MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="30000",
                   ADMIN_PORT=str(sp.admin_port))
        procs = [subprocess.Popen([sys.executable, "-c", FUSED_CLIENT], env=dict(env, RANK=str(r), DEV=str(r if ngpu >= 2 else 0)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
        for p in procs:
            out, err = p.communicate(timeout=240)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
            assert res["launch"] == "daemon"
            assert res["fused_launches"] > 0 and res["fused_members"] >= res["fused_launches"]
    finally:
        sp.stop()
