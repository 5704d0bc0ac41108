"""Client-side launch on GPUs: `[b200] launch = "client"` with the CUDA backend. One client
process per GPU; each maps its peers' buffers, signal pads, status blocks and FIFOs
(exported VMM handles, shared registered host memory), loads `libmccs_kernels.so` and
launches its own rank's kernel on its own stream from the plan the daemon published.

This is what the daemon's default (`[b200] launch = "auto"`) gives every communicator whose
ranks are separate processes on separate GPUs, so the first case runs with the default
configuration and checks that the mode was chosen. With one GPU only the single-rank copy
can be launched by a client; several ranks on one GPU stay with the daemon's cooperative
launch by design. The second case adds the in-switch variants, for which each client maps
the multicast objects the daemon created and bound (`client_nvls`, on by default).
"""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import REPO, write_config

pytestmark = pytest.mark.gpu

CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); port = int(os.environ["ADMIN_PORT"])
torch.cuda.set_device(rank)
DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "i32": torch.int32}
def inputs(dt, count, salt):
    g = torch.Generator().manual_seed(1000 * salt + count)
    return [torch.randint(-4, 5, (count,), generator=g).to(dt) for _ in range(n)]
send = M.Buffer(8 << 20, rank); recv = M.Buffer(16 << 20, rank)
comm = M.Communicator(6300, rank, n, device=rank)
bad, seen, salt = [], set(), 0
def allreduce(algo, dname, count, op="sum", in_place=False):
    global salt
    salt += 1
    dt = DT[dname]
    xs = inputs(dt, count, salt)
    s = send.tensor(dt, count); s.copy_(xs[rank])
    d = s if in_place else recv.tensor(dt, count)
    comm.all_reduce(s, None if in_place else d, op=op, algo=algo)
    acc = torch.stack([x.double() for x in xs])
    want = {"sum": acc.sum(0), "max": acc.max(0).values, "avg": acc.sum(0) / n}[op]
    tol = {"bf16": 0.05 * n, "f16": 0.01 * n}.get(dname, 1e-6)
    if not torch.allclose(d.double().cpu(), want, rtol=0, atol=tol):
        bad.append(("allreduce", algo, dname, count, op, in_place))
    seen.add(comm.last_plan()[0])
def allgather(algo, nbytes):
    global salt
    salt += 1
    xs = [((torch.arange(nbytes) * (r + 3) + salt) % 251).to(torch.uint8) for r in range(n)]
    out = recv.tensor(torch.uint8, nbytes * n)
    s = send.tensor(torch.uint8, nbytes); s.copy_(xs[rank])
    comm.all_gather(s, out, algo=algo)
    if not torch.equal(out.cpu(), torch.cat(xs)):
        bad.append(("allgather", algo, nbytes))
    seen.add(comm.last_plan()[0])
def reduce_scatter(algo, dname, count, in_place=False):
    global salt
    salt += 1
    dt = DT[dname]
    xs = inputs(dt, count * n, salt)
    s = send.tensor(dt, count * n); s.copy_(xs[rank])
    d = s[rank * count:(rank + 1) * count] if in_place else recv.tensor(dt, count)
    comm.reduce_scatter(s, d, algo=algo)
    want = torch.stack([x.double() for x in xs]).sum(0)[rank * count:(rank + 1) * count]
    tol = {"bf16": 0.05 * n, "f16": 0.01 * n}.get(dname, 1e-6)
    if not torch.allclose(d.double().cpu(), want, rtol=0, atol=tol):
        bad.append(("reduce_scatter", algo, dname, count, in_place))
    seen.add(comm.last_plan()[0])
if n > 1:
    for dname, count in (("f32", 1), ("f32", 4096), ("bf16", 3001), ("i32", 257), ("bf16", 1 << 18)):
        reduce_scatter("rs_direct", dname, count)
    reduce_scatter("auto", "f32", 8192, in_place=True)
    if os.environ.get("NVLS") == "1":
        for dname, count in (("f32", 4096), ("bf16", 1 << 18)):
            reduce_scatter("rs_nvls", dname, count)
ar = ("ar_oneshot", "ar_twoshot", "ar_ring", "auto") if n > 1 else ("auto",)
ag = ("ag_pull", "ag_push", "ag_ring", "auto") if n > 1 else ("auto",)
for algo in ar:
    for dname, count in (("f32", 1), ("f32", 4099), ("bf16", 3001), ("i32", 257), ("f16", 2048), ("bf16", 1 << 20)):
        allreduce(algo, dname, count)
    allreduce(algo, "f32", 1000, op="avg")
    allreduce(algo, "i32", 500, op="max")
    if algo != "ar_oneshot":
        allreduce(algo, "f32", 5000, in_place=True)
for algo in ag:
    for nbytes in (16, 1000, 40000, 1 << 20):
        allgather(algo, nbytes)
if os.environ.get("NVLS") == "1" and n > 1:
    # the in-switch variants: each client maps the multicast objects the daemon bound
    for algo in ("ar_nvls_oneshot", "ar_nvls_twoshot", "ar_hybrid"):
        for dname, count in (("f32", 4), ("f32", 4100), ("bf16", 3000), ("f16", 2048), ("bf16", 1 << 20)):
            allreduce(algo, dname, count)
        allreduce(algo, "f32", 8192, in_place=True)
    for nbytes in (16, 4096, 1 << 20):
        allgather("ag_nvls", nbytes)
# 200 collectives back to back on poisoned outputs, checked on the device after every one
# (the ordering stress of tests/test_gpu_collectives.py, here with kernels launched by the
# clients and, in the second case, through the multicast mappings each client made itself)
if n > 1:
    cnt = 300000
    bad_count = torch.zeros((), dtype=torch.int64, device="cuda")
    sa = send.tensor(torch.float32, cnt); da = recv.tensor(torch.float32, cnt)
    stress = ("ar_nvls_twoshot", "ar_twoshot") if os.environ.get("NVLS") == "1" else ("ar_twoshot",)
    for algo in stress:
        for it in range(200):
            sa.fill_(float(rank + 1) + 0.25 * it); da.fill_(float("nan"))
            comm.all_reduce(sa, da, algo=algo)
            bad_count += (da != float(n * (n + 1) // 2) + 0.25 * it * n).sum()
    sg = send.tensor(torch.uint8, cnt); dg = recv.tensor(torch.uint8, cnt * n)
    for algo in (("ag_nvls", "ag_push") if os.environ.get("NVLS") == "1" else ("ag_push",)):
        for it in range(200):
            sg.fill_((rank * 31 + it) % 251); dg.fill_(255)
            comm.all_gather(sg, dg, algo=algo)
            for q in range(n):
                bad_count += (dg[q * cnt:(q + 1) * cnt] != (q * 31 + it) % 251).sum()
    torch.cuda.synchronize()
    if int(bad_count.item()) != 0:
        bad.append(("stress", int(bad_count.item())))
# back to back on the stream without looking at the results in between
t = send.tensor(torch.float32, 1 << 16)
t.fill_(1.0)
for _ in range(50):
    comm.all_reduce(t, op="avg")
torch.cuda.synchronize()
if not bool(torch.all(t == 1.0)):
    bad.append(("chain",))
q = comm.query()
st = M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"]["6300"]
comm.destroy()
print("RESULT", json.dumps({"bad": bad, "seen": sorted(seen), "async_error": q["async_error"], "device_error": q["device_error"],
                            "client_launch": st["client_launch"], "completed": st["completed"]}), flush=True)
"""


@pytest.mark.parametrize("nvls", [False, True])
def test_client_side_launch_on_gpus(tmp_path, nvls):
    from mccs_b200 import daemon
    n = min(torch.cuda.device_count(), 4)
    if nvls and n < 2:
        pytest.skip("multicast needs two GPUs")
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, wait_timeout_ms=2000,
                       extra='launch = "client"\nclient_nvls = true' if nvls else "client_nvls = false")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn", "NCCL_NVLS_ENABLE": "0"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="error",
                   ADMIN_PORT=str(sp.admin_port), MCCS_WC_TIMEOUT_MS="60000", NVLS="1" if nvls else "0")
        procs = [subprocess.Popen([sys.executable, "-c", CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        for p in procs:
            out, err = p.communicate(timeout=600)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
            assert res["client_launch"] is True
            if nvls:
                assert {"ar_nvls_oneshot", "ar_nvls_twoshot", "ar_hybrid", "ag_nvls"} <= set(res["seen"])
            if n > 1:
                assert {"ar_oneshot", "ar_twoshot", "ar_ring", "ag_pull", "ag_push", "ag_ring"} <= set(res["seen"])
            else:
                assert set(res["seen"]) == {"local_copy"}
    finally:
        sp.stop()


SLICE_CLIENT = r"""
import os, sys, json, time, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); cid = int(os.environ["COMM"]); n = 2
torch.cuda.set_device(rank)
count = 8 << 20                                         # 32 MiB of fp32: eight slices of 4 MiB under this daemon's policy
buf = M.Buffer(count * 4, rank); out = M.Buffer(count * 4, rank)
comm = M.Communicator(cid, rank, n, device=rank)
x = buf.tensor(torch.float32, count); y = out.tensor(torch.float32, count)
base = (torch.arange(count, dtype=torch.float32, device="cuda") % 97)
port = int(os.environ["ADMIN_PORT"])
for _ in range(600):                                    # start together with the other tenant
    if {"6201", "6202"} <= set(M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"]):
        break
    time.sleep(0.05)
bad = torch.zeros((), dtype=torch.int64, device="cuda")
for it in range(40):
    x.copy_(base + float(rank + it + cid % 7))
    y.fill_(float("nan"))
    comm.all_reduce(x, y, algo="ar_twoshot")
    bad += (y != base * 2 + float(1 + 2 * (it + cid % 7))).sum()
torch.cuda.synchronize()
q = comm.query()
mode = comm.launch_mode
comm.destroy()
print("RESULT", json.dumps({"bad": int(bad.item()), "async_error": q["async_error"], "device_error": q["device_error"], "launch": mode}), flush=True)
"""


def test_time_slices_under_client_launch_on_gpus(tmp_path):
    """Two tenants on the same two GPUs, kernels launched by the clients: large AllReduces are
    cut into time slices, the daemon hands out one plan per admitted slice, and every result is
    exact although the two tenants' slices interleave on the links."""
    import mccs_b200 as M
    from mccs_b200 import daemon
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, wait_timeout_ms=5000, trace=True)
    with open(cfg, "a") as f:
        f.write("\n[qos]\nmax_outstanding_bytes = 8388608\nactive_window_us = 3000000\n[qos.tenants.6201]\nweight = 2.0\n[qos.tenants.6202]\nweight = 1.0\n")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="60000",
                   ADMIN_PORT=str(sp.admin_port))
        procs = [subprocess.Popen([sys.executable, "-c", SLICE_CLIENT], env=dict(env, RANK=str(r), COMM=str(c)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for c in (6201, 6202) for r in range(2)]
        for p in procs:
            out, err = p.communicate(timeout=300)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == 0 and res["async_error"] == 0 and res["device_error"] == 0 and res["launch"] == "client"
        events = M.admin_request(sp.admin_port, {"cmd": "trace", "enabled": False, "inline": True})["trace"]["traceEvents"]
        assert max(e.get("args", {}).get("slices", 1) for e in events) > 1, "no collective was sliced"
    finally:
        sp.stop()


FUSED_CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); port = int(os.environ["ADMIN_PORT"])
torch.cuda.set_device(rank)
bufs = [M.Buffer((4 << 20) + 4096 * k, rank) for k in range(12)]
ts = [b.tensor(torch.float32, (1 << 20) + 1024 * k) for k, b in enumerate(bufs)]     # twelve members of different sizes
comm = M.Communicator(7400, rank, n, device=rank)
bad = []
for rnd in range(6):
    for k, t in enumerate(ts):
        t.fill_(float(rank + 1 + k + rnd))
    with M.group():                       # posted together; the plans are taken at the end of the group
        for t in ts:
            comm.all_reduce(t, algo="ar_twoshot")
    torch.cuda.synchronize()
    for k, t in enumerate(ts):
        want = float(sum(r + 1 + k + rnd for r in range(n)))
        if not bool(torch.all(t == want)):
            bad.append((rnd, k, float(t[0]), want))
# a single call outside a group still works as before
ts[0].fill_(1.0)
comm.all_reduce(ts[0])
torch.cuda.synchronize()
if not bool(torch.all(ts[0] == float(n))):
    bad.append(("single",))
q = comm.query()
st = M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"]["7400"]
mode = comm.launch_mode
comm.destroy()
print("RESULT", json.dumps({"bad": bad[:4], "async_error": q["async_error"], "device_error": q["device_error"],
                            "fused_launches": st["fused_launches"], "fused_members": st["fused_members"], "launch": mode}), flush=True)
"""


def test_fused_launches_under_client_launch_on_gpus(tmp_path):
    """`fuse_allreduce = 8` with kernels launched by the clients: the AllReduces of a group are
    posted together, the daemon carries up to eight of them in one plan (a head and its
    followers), and each client builds and launches the fused kernel itself."""
    from mccs_b200 import daemon
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs two GPUs")
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, wait_timeout_ms=5000,
                       extra="fuse_allreduce = 8")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="30000",
                   ADMIN_PORT=str(sp.admin_port))
        procs = [subprocess.Popen([sys.executable, "-c", FUSED_CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        for p in procs:
            out, err = p.communicate(timeout=240)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0 and res["launch"] == "client"
            assert res["fused_launches"] > 0 and res["fused_members"] > res["fused_launches"]
    finally:
        sp.stop()
