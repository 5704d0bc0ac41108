"""The whole service on a machine without a GPU, with the REAL kernels: the daemon's host
backend runs the kernels' own sources on the SIMT emulator (`[b200] host_kernels =
"emulated"`) instead of its plain loops. What this adds over the other host tests is the
daemon's side of the device contract: barrier epochs and tickets handed out per collective
and per slice, ring step counters and FIFO placement across collectives, ring orders
frozen at plan time, live reconfiguration between kernels, fused launches and the
host-staged transport's FIFO ring."""
import json
import os
import subprocess
import sys

import pytest

from helpers import REPO, write_config

CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); port = int(os.environ["ADMIN_PORT"])
torch.manual_seed(1234)                     # every rank can compute every rank's input
DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "i32": torch.int32, "i64": torch.int64, "f64": torch.float64}
def inputs(dt, count, salt):
    g = torch.Generator().manual_seed(1000 * salt + count)
    return [torch.randint(-4, 5, (count,), generator=g).to(dt) for _ in range(n)]
send = M.Buffer(1 << 20, rank); recv = M.Buffer(1 << 21, rank)
CID = 6100
comm = M.Communicator(CID, rank, n, device=rank)
bad = []
seen = set()
salt = 0
def allreduce(algo, dname, count, op="sum", in_place=False):
    global salt
    salt += 1
    dt = DT[dname]
    xs = inputs(dt, count, salt)
    s = send.tensor(dt, count); s.copy_(xs[rank])
    d = s if in_place else recv.tensor(dt, count)
    comm.all_reduce(s, None if in_place else d, op=op, algo=algo)
    acc = torch.stack([x.double() for x in xs])
    want = {"sum": acc.sum(0), "max": acc.max(0).values, "min": acc.min(0).values, "avg": acc.sum(0) / n, "prod": acc.prod(0)}[op]
    tol = {"bf16": 0.05 * n, "f16": 0.01 * n}.get(dname, 1e-6)
    if not torch.allclose(d.double(), want, rtol=0, atol=tol):
        bad.append(("allreduce", algo, dname, count, op, in_place))
    seen.add(comm.last_plan()[0])
def allgather(algo, nbytes, in_place=False):
    global salt
    salt += 1
    xs = [((torch.arange(nbytes) * (r + 3) + salt) % 251).to(torch.uint8) for r in range(n)]
    out = recv.tensor(torch.uint8, nbytes * n)
    s = out[rank * nbytes:(rank + 1) * nbytes] if in_place else send.tensor(torch.uint8, nbytes)
    s.copy_(xs[rank])
    comm.all_gather(s, out, algo=algo)
    if not torch.equal(out, torch.cat(xs)):
        bad.append(("allgather", algo, nbytes, in_place))
    seen.add(comm.last_plan()[0])

def reduce_scatter(algo, dname, count, op="sum", in_place=False):
    global salt
    salt += 1
    dt = DT[dname]
    xs = inputs(dt, count * n, salt)
    s = send.tensor(dt, count * n); s.copy_(xs[rank])
    d = s[rank * count:(rank + 1) * count] if in_place else recv.tensor(dt, count)
    comm.reduce_scatter(s, d, op=op, algo=algo)
    acc = torch.stack([x.double() for x in xs])[:, rank * count:(rank + 1) * count]
    want = {"sum": acc.sum(0), "max": acc.max(0).values, "avg": acc.sum(0) / n}[op]
    tol = {"bf16": 0.05 * n, "f16": 0.01 * n}.get(dname, 1e-6)
    if not torch.allclose(d.double(), want, rtol=0, atol=tol):
        bad.append(("reduce_scatter", algo, dname, count, op, in_place))
    seen.add(comm.last_plan()[0])

if os.environ.get("HOST_STAGED") == "1":
    # the host-staged transport has ring kernels only, and reduce-scatter has no ring form
    try:
        reduce_scatter("auto", "f32", 64)
        bad.append(("reduce_scatter accepted on the host-staged transport",))
    except Exception as e:
        if getattr(e, "code", None) != -9: bad.append(("reduce_scatter", str(e)))
    # the refusal ended the communicator; a new one takes a new id (the old id stays taken until
    # every rank has let go of it)
    comm.destroy(); CID = 6101; comm = M.Communicator(CID, rank, n, device=rank)
for algo in () if os.environ.get("HOST_STAGED") == "1" else ("rs_direct", "auto") + (("rs_nvls",) if os.environ.get("NVLS") == "1" else ()):
    for dname, count in (("f32", 1), ("f32", 1028), ("bf16", 3000), ("i32", 257), ("f64", 100), ("f16", 2048), ("f32", 4099)):
        reduce_scatter(algo, dname, count)
    reduce_scatter(algo, "f32", 1000, op="avg")
    reduce_scatter(algo, "i32", 500, op="max")
    reduce_scatter(algo, "f32", 2048, in_place=True)
for algo in ("ar_oneshot", "ar_twoshot", "ar_ring", "auto"):
    for dname, count in (("f32", 1), ("f32", 4099), ("bf16", 3001), ("i32", 257), ("f64", 100), ("i64", 33), ("f16", 2048)):
        allreduce(algo, dname, count)
    allreduce(algo, "f32", 1000, op="avg")
    allreduce(algo, "i32", 500, op="max")
    if algo != "ar_oneshot":
        allreduce(algo, "f32", 5000, in_place=True)
if os.environ.get("NVLS") == "1":
    # the in-switch variants on emulated multicast regions (floating-point sums; anything
    # else asked of them is answered by a variant that can do it)
    for algo in ("ar_nvls_oneshot", "ar_nvls_twoshot", "ar_hybrid"):
        for dname, count in (("f32", 4), ("f32", 4100), ("bf16", 3000), ("f16", 2048), ("f32", 4099), ("i32", 256)):
            allreduce(algo, dname, count)
        allreduce(algo, "f32", 1000, op="avg")
        allreduce(algo, "f32", 8192, in_place=True)
        allreduce(algo, "f32", 512, op="max")
    for nbytes in (16, 4096, 40000, 1000):
        allgather("ag_nvls", nbytes)
for algo in ("ag_pull", "ag_push", "ag_ring", "auto"):
    for nbytes in (16, 1000, 40000):
        allgather(algo, nbytes)
    allgather(algo, 4096, in_place=True)
# many FIFO loops through the ring, then a live change of the ring order and channel count,
# then the ring again: step counters and FIFO slots carry over between the launches
allreduce("ar_ring", "f32", 150000)
if rank == 0:
    ring = list(reversed(range(n)))
    rep = M.reconfigure(port, [{"communicator_id": CID, "channels": [{"channel_id": 0, "ring": ring}, {"channel_id": 1, "ring": list(range(n))}, {"channel_id": 2, "ring": ring}]}])
    assert rep.get("status") == "ok", rep
for _ in range(3):
    allreduce("ar_ring", "f32", 70000)
    allgather("ag_ring", 30000)
# a burst: 8 independent all-reduces in one group (fused launches are on in this daemon)
bufs = [M.Buffer(8192, rank) for _ in range(8)]
ts = [b.tensor(torch.float32, 100 + 37 * i) for i, b in enumerate(bufs)]
for i, t in enumerate(ts):
    t.fill_(float(rank + i))
with M.group():
    for t in ts:
        comm.all_reduce(t, algo="ar_twoshot")
for i, t in enumerate(ts):
    if not bool(torch.all(t == float(sum(range(n)) + n * i))):
        bad.append(("group", i))
q = comm.query()
st = M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"][str(CID)]
comm.destroy()
print("RESULT", json.dumps({"bad": bad, "seen": sorted(seen), "async_error": q["async_error"], "device_error": q["device_error"],
                            "fused_members": st["fused_members"], "epoch": st["config_epoch"],
                            "client_launch": st["client_launch"], "completed": st["completed"]}), flush=True)
"""


def _run(tmp_path, n, extra, client_env=None, **kw):
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=n, listen_port=-1, force_host=True,
                       wait_timeout_ms=20000, extra='host_kernels = "emulated"\nfuse_allreduce = 8\n' + extra, **kw)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        assert "SIMT emulator" in json.dumps(__import__("mccs_b200").admin_request(sp.admin_port, {"cmd": "stats"}))
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="error",
                   ADMIN_PORT=str(sp.admin_port), MCCS_WC_TIMEOUT_MS="60000")
        env.update(client_env or {})
        procs = [subprocess.Popen([sys.executable, "-c", CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        results = []
        for p in procs:
            out, err = p.communicate(timeout=600)
            assert p.returncode == 0, err[-3000:]
            results.append(json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:]))
        return results
    finally:
        sp.stop()


@pytest.mark.parametrize("n,sync", [(2, "auto"), (4, "auto"), (3, "memops")])
def test_service_with_the_real_kernels_on_the_emulator(tmp_path, n, sync):
    """`sync = "memops"`: the same, with the semaphore protocol instead of events (and with
    it the fused kernels' start-barrier skip and in-kernel completion word, which only
    apply to semaphore-ordered ranks)."""
    extra = "single_through_fused = true\nskip_start_barrier = true\nkernel_writes_done = true" if sync == "memops" else ""
    for res in _run(tmp_path, n, extra, sync=sync):
        assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
        # every emulated variant really ran
        assert {"ar_oneshot", "ar_twoshot", "ar_ring", "ag_pull", "ag_push", "ag_ring", "rs_direct"} <= set(res["seen"])
        assert res["epoch"] == 1 and res["fused_members"] >= 2 and res["client_launch"] is False


@pytest.mark.parametrize("n", [2, 4])
def test_in_switch_variants_on_emulated_multicast(tmp_path, n):
    """The NVLS kernels through the whole service without a GPU: the host backend binds
    emulated multicast regions (an address range that stands for the same offsets of every
    rank's buffer), so the multicast cache, the feasibility rules and the multicast
    addresses in the kernels' arguments are exercised as on a GPU."""
    for res in _run(tmp_path, n, "", client_env={"NVLS": "1"}):
        assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
        assert {"ar_nvls_oneshot", "ar_nvls_twoshot", "ar_hybrid", "ag_nvls", "rs_nvls"} <= set(res["seen"])


def test_host_staged_transport_with_the_real_ring_kernels(tmp_path):
    """`transport = "host_staged"`: only the FIFO ring variants are legal, whatever is asked for."""
    for res in _run(tmp_path, 3, "", transport="host_staged", client_env={"HOST_STAGED": "1"}):
        assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
        assert set(res["seen"]) <= {"ar_ring", "ag_ring"}


SLICE_CLIENT = r"""
import os, sys, json, time, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); cid = int(os.environ["COMM"]); n = 2
count = 1 << 20                                         # 4 MiB of fp32: above the 1 MiB slice size of this daemon
buf = M.Buffer(count * 4, rank); out = M.Buffer(count * 4, rank)
comm = M.Communicator(cid, rank, n, device=rank)
x = buf.tensor(torch.float32, count); y = out.tensor(torch.float32, count)
ok = True
# start together with the other tenant: wait until both communicators exist
port = int(os.environ["ADMIN_PORT"])
for _ in range(600):
    if {"6201", "6202"} <= set(M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"]):
        break
    time.sleep(0.05)
for it in range(12):
    x.copy_(torch.arange(count, dtype=torch.float32) % 97 + rank + it + cid)
    comm.all_reduce(x, y, algo="ar_twoshot")
    want = (torch.arange(count, dtype=torch.float32) % 97) * 2 + 1 + 2 * (it + cid)
    ok &= bool(torch.equal(y, want))
q = comm.query()
comm.destroy()
print("RESULT", json.dumps({"ok": ok, "async_error": q["async_error"], "device_error": q["device_error"]}), flush=True)
"""


@pytest.mark.parametrize("launch", ["daemon", "client"])
def test_time_sliced_allreduce_with_the_real_kernels(tmp_path, launch):
    """Two tenants on the same two devices: large all-reduces are cut into slices (each its
    own launch with its own barrier epochs and ticket) and still give the right sums. With
    client-side launch the daemon hands out one plan per admitted slice and the client
    library launches them one after another."""
    import mccs_b200 as M
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=2, listen_port=-1, force_host=True,
                       wait_timeout_ms=20000, trace=True, extra=f'host_kernels = "emulated"\nlaunch = "{launch}"')
    with open(cfg, "a") as f:
        f.write("\n[qos]\nmax_outstanding_bytes = 2097152\nactive_window_us = 3000000\n[qos.tenants.6201]\nweight = 2.0\n[qos.tenants.6202]\nweight = 1.0\n")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="60000",
                   ADMIN_PORT=str(sp.admin_port))
        procs = [subprocess.Popen([sys.executable, "-c", SLICE_CLIENT], env=dict(env, RANK=str(r), COMM=str(c)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for c in (6201, 6202) for r in range(2)]
        for p in procs:
            out, err = p.communicate(timeout=600)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["ok"] and res["async_error"] == 0 and res["device_error"] == 0
        events = M.admin_request(sp.admin_port, {"cmd": "trace", "enabled": False, "inline": True})["trace"]["traceEvents"]
        assert max(e.get("args", {}).get("slices", 1) for e in events) > 1, "no collective was sliced"
    finally:
        sp.stop()


@pytest.mark.parametrize("n", [2, 4])
def test_client_side_launch(tmp_path, n):
    """`[b200] launch = "client"`: the daemon collects the ranks' requests, plans, admits and
    hands out epochs and tickets as always, but gives the plan back to each rank's client
    library, which maps its peers' buffers, pads, status blocks and FIFOs and runs its
    rank's kernel itself (here on the emulator, one process per rank meeting through
    shared memory). Same scenario as above: every variant, ring reconfiguration, groups."""
    for res in _run(tmp_path, n, 'launch = "client"'):
        assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
        assert {"ar_oneshot", "ar_twoshot", "ar_ring", "ag_pull", "ag_push", "ag_ring"} <= set(res["seen"])
        assert res["epoch"] == 1 and res["client_launch"] is True and res["completed"] > 50
        # the burst of eight grouped all-reduces went out as fused launches, built by each
        # client from the head's plan and its followers' buffers
        assert res["fused_members"] >= 2


def test_client_side_launch_of_the_in_switch_variants(tmp_path):
    """`client_nvls = true`: plans name multicast regions; each client maps them (here: builds
    the emulated region over its own mappings of the ranks' buffers) and launches the NVLS,
    hybrid and multicast all-gather kernels itself."""
    for res in _run(tmp_path, 4, 'launch = "client"\nclient_nvls = true', client_env={"NVLS": "1"}):
        assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
        assert {"ar_nvls_oneshot", "ar_nvls_twoshot", "ar_hybrid", "ag_nvls"} <= set(res["seen"])
        assert res["client_launch"] is True


GROUP_CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); port = int(os.environ["ADMIN_PORT"])
comm = M.Communicator(6500, rank, n, device=rank)
bufs = [M.Buffer(4096, rank) for _ in range(40)]
ts = [b.tensor(torch.float32, 64 + 8 * (i % 5)) for i, b in enumerate(bufs)]
gat_buf = M.Buffer(256 * n, rank)           # the object owns the memory: it must outlive its tensors
gat = gat_buf.tensor(torch.uint8, 256 * n)
bad = []
for rnd in range(3):
    for i, t in enumerate(ts):
        t.fill_(float(rank + i + rnd))
    gat[rank * 256:(rank + 1) * 256] = rank + 1 + rnd
    with M.group():
        # more members than the plan ring holds (the library takes plans as it goes), an
        # all-gather in the middle (never fused), a max in between sums (ends a fused run)
        for i, t in enumerate(ts[:25]):
            comm.all_reduce(t, algo="ar_twoshot")
        comm.all_gather(gat[rank * 256:(rank + 1) * 256], gat)
        comm.all_reduce(ts[25], op="max", algo="ar_twoshot")
        for t in ts[26:]:
            comm.all_reduce(t, algo="ar_twoshot")
    for i, t in enumerate(ts):
        want = float(n - 1 + i + rnd) if i == 25 else float(sum(range(n)) + n * (i + rnd))
        if not bool(torch.all(t == want)):
            bad.append((rnd, i, float(t[0]), want))
    if [int(gat[r * 256]) for r in range(n)] != [r + 1 + rnd for r in range(n)]:
        bad.append((rnd, "gather"))
# dependent members must not share a launch: out of one is the input of the next
a, b, c = ts[0], ts[1], ts[2]
a.fill_(1.0)
with M.group():
    comm.all_reduce(a, a, algo="ar_twoshot")          # a = n
    comm.all_reduce(a, a, algo="ar_twoshot")          # a = n * n
if not bool(torch.all(a == float(n * n))):
    bad.append(("dependent", float(a[0])))
q = comm.query()
st = M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"]["6500"]
comm.destroy()
print("RESULT", json.dumps({"bad": bad[:5], "async_error": q["async_error"], "device_error": q["device_error"],
                            "fused_launches": st["fused_launches"], "fused_members": st["fused_members"],
                            "client_launch": st["client_launch"], "completed": st["completed"]}), flush=True)
"""


@pytest.mark.parametrize("launch", ["client", "daemon"])
def test_large_and_mixed_groups_with_fused_launches(tmp_path, launch):
    """Groups that are larger than the plan ring, contain collectives that cannot be fused and
    members that depend on each other: fused where allowed, right everywhere."""
    from mccs_b200 import daemon
    n = 3
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=n, listen_port=-1, force_host=True,
                       wait_timeout_ms=20000, extra=f'host_kernels = "emulated"\nfuse_allreduce = 8\nlaunch = "{launch}"')
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="error",
                   ADMIN_PORT=str(sp.admin_port), MCCS_WC_TIMEOUT_MS="60000")
        procs = [subprocess.Popen([sys.executable, "-c", GROUP_CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        for p in procs:
            out, err = p.communicate(timeout=600)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == [] and res["async_error"] == 0 and res["device_error"] == 0
            assert res["client_launch"] is (launch == "client")
            assert res["fused_launches"] > 0 and res["completed"] > 0
    finally:
        sp.stop()


OPEN_GROUP_CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
comm = M.Communicator(6600, rank, n, device=rank)
other = M.Communicator(6601, rank, n, device=rank)
bufs = [M.Buffer(4096, rank) for _ in range(6)]
ts = [b.tensor(torch.float32, 128) for b in bufs]
res = {}
for i, t in enumerate(ts):
    t.fill_(float(rank + i))
M.client._lib.shim().mccsGroupStart()
for t in ts[:3]:
    comm.all_reduce(t, algo="ar_twoshot")
res["plan_inside"] = comm.last_plan()[0]          # flushes: the three run now, inside the open group
res["inside_ok"] = all(bool(torch.all(t == float(sum(range(n)) + n * i))) for i, t in enumerate(ts[:3]))
comm.all_reduce(ts[3], algo="ar_twoshot")
ts[3] = None
bufs[3].free()                                     # a free inside the group settles what names the memory first
other.all_reduce(ts[4], algo="ar_twoshot")
other.destroy()                                    # so does destroying a communicator with requests pending
comm.all_reduce(ts[5], algo="ar_twoshot")
res["group_end"] = int(M.client._lib.shim().mccsGroupEnd())
res["after_ok"] = all(bool(torch.all(ts[i] == float(sum(range(n)) + n * i))) for i in (4, 5))
# ranks that disagree inside a fused group: every rank gets the error when the group ends, the
# requests before the bad one have run, nothing waits for ever
a, b, c = ts[0], ts[1], ts[2]
a.fill_(1.0); b.fill_(1.0); c.fill_(1.0)
M.client._lib.shim().mccsGroupStart()
comm.all_reduce(a, algo="ar_twoshot")
comm.all_reduce(b, count=64 if rank == 1 else 128, algo="ar_twoshot")
comm.all_reduce(c, algo="ar_twoshot")
res["mismatch_rc"] = int(M.client._lib.shim().mccsGroupEnd())
res["first_ran"] = bool(torch.all(a == float(n)))
comm.destroy()
print("RESULT", json.dumps(res), flush=True)
"""


def test_open_groups_settle_before_free_destroy_and_queries(tmp_path):
    """Client-side launch with fused launches on: requests of an open group are only posted.
    Reading the last plan, freeing a buffer and destroying a communicator inside the group each
    launch what is pending first; a group whose ranks disagree ends with an error on every rank."""
    from mccs_b200 import daemon
    n = 2
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=n, listen_port=-1, force_host=True,
                       wait_timeout_ms=5000, extra='host_kernels = "emulated"\nfuse_allreduce = 8\nlaunch = "client"')
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "error"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="off", MCCS_WC_TIMEOUT_MS="30000")
        procs = [subprocess.Popen([sys.executable, "-c", OPEN_GROUP_CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        for p in procs:
            out, err = p.communicate(timeout=300)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["plan_inside"] == "ar_twoshot" and res["inside_ok"]
            assert res["group_end"] == 0 and res["after_ok"]
            assert res["mismatch_rc"] != 0 and res["first_ran"]
    finally:
        sp.stop()
