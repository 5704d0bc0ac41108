"""The stream-memory-operation protocol between client library and daemon — "submitted"
and "done" semaphores in a shared page, requests that are counted instead of answered,
launches gated on every rank's semaphore, deferred and grouped waits — on a machine
without a GPU: with `[b200] sync = "memops"` the host backend hands out semaphore pages
and does the "stream memory operations" on the CPU, and the library writes and awaits the
semaphores itself. On a GPU box the same code paths run with cuStreamWriteValue64 /
cuStreamWaitValue64 in their place."""
import json
import os
import subprocess
import sys

import pytest

from helpers import REPO, write_config

CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); cid = int(os.environ.get("COMM", "6300"))
weight = float(cid % 7 + 1)
bad = []
bufs = [M.Buffer(1 << 16, rank) for _ in range(20)]
comm = M.Communicator(cid, rank, n, device=rank)
x = bufs[0].tensor(torch.float32, 4096); y = bufs[1].tensor(torch.float32, 4096)
# 1. plain calls: more than the request ring holds, more than the in-flight bound
for i in range(300):
    x.fill_(float(rank + i))
    comm.all_reduce(x, y)
    if float(y[7]) != float(sum(range(n)) + n * i): bad.append(("plain", i, float(y[7])))
# 2. all-gather, in place
g = bufs[2].tensor(torch.uint8, 512 * n)
g[rank * 512:(rank + 1) * 512] = rank + 1
comm.all_gather(g[rank * 512:(rank + 1) * 512], g)
if [int(g[r * 512]) for r in range(n)] != [r + 1 for r in range(n)]: bad.append(("allgather",))
# 3. groups: one wait at the end, members on independent buffers (fused launches are on)
ts = [b.tensor(torch.float32, 64 + 8 * i) for i, b in enumerate(bufs[3:19])]
for rnd in range(5):
    for i, t in enumerate(ts): t.fill_(float(rank + i + rnd))
    with M.group():
        for t in ts: comm.all_reduce(t)
    for i, t in enumerate(ts):
        if not bool(torch.all(t == float(sum(range(n)) + n * (i + rnd)))): bad.append(("group", rnd, i))
# 4. deferred waiting: calls only post, one wait covers them
comm.set_deferred_wait(True)
for i, t in enumerate(ts): t.fill_(float(rank * 2 + i))
for t in ts: comm.all_reduce(t, op="max")
comm.wait()
for i, t in enumerate(ts):
    if not bool(torch.all(t == float((n - 1) * 2 + i))): bad.append(("deferred", i))
comm.set_deferred_wait(False)
comm.flush()
q = comm.query()
# 5. a mismatch is an error on every rank, reported by the failing call itself
err = None
try:
    comm.all_reduce(x, y, count=100 + rank)
except Exception as e:
    err = getattr(e, "code", None)
comm.destroy()
print("RESULT", json.dumps({"bad": bad[:5], "launched": q["launched"], "async_error": q["async_error"], "mismatch": err}), flush=True)
"""


def _spawn_daemon(tmp_path, n, extra=""):
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=n, listen_port=-1, force_host=True,
                       sync="memops", wait_timeout_ms=5000, extra="fuse_allreduce = 4\n" + extra)
    return daemon.spawn(cfg, env={"MCCS_LOG": "warn"})


@pytest.mark.parametrize("n", [1, 2, 4])
def test_memop_protocol_on_the_host_backend(tmp_path, n):
    sp = _spawn_daemon(tmp_path, n)
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="30000")
        procs = [subprocess.Popen([sys.executable, "-c", CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        for p in procs:
            out, err = p.communicate(timeout=300)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == [] and res["async_error"] == 0
            assert res["launched"] == 300 + 1 + 5 * 16 + 16
            if n > 1:
                assert res["mismatch"] == -8        # mccsMismatch
    finally:
        sp.stop()


def test_memop_mode_tenants_share_devices(tmp_path):
    """Three tenants on overlapping devices in mem-op mode, all at once."""
    sp = _spawn_daemon(tmp_path, 4)
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="60000")
        procs = []
        for cid, n in ((6301, 4), (6302, 2), (6303, 3)):
            for r in range(n):
                procs.append(subprocess.Popen([sys.executable, "-c", CLIENT], env=dict(env, RANK=str(r), WORLD_SIZE=str(n), COMM=str(cid)),
                                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
        for p in procs:
            out, err = p.communicate(timeout=600)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["bad"] == [] and res["async_error"] == 0 and res["mismatch"] == -8
    finally:
        sp.stop()


WAITER = r"""
import os, sys, time, torch
import mccs_b200 as M
rank = int(os.environ["RANK"])
buf = M.Buffer(1 << 16, rank)
x = buf.tensor(torch.float32, 4096)
comm = M.Communicator(6400, rank, 2, device=rank)
if rank == 1:
    print("JOINED", flush=True)
    time.sleep(600)          # never posts: rank 0's request stays queued in the daemon
comm.set_deferred_wait(True)
comm.all_reduce(x)           # returns at once; the "wait for done" is what blocks below
print("POSTED", flush=True)
t0 = time.time()
code = 0
try:
    comm.wait()              # the daemon dies while this waits for the "done" semaphore
except Exception as e:
    code = getattr(e, "code", -999)
first = time.time() - t0
later = 0
try:
    comm.all_reduce(x)
except Exception as e:
    later = getattr(e, "code", -999)
print("RESULT", code, later, round(first, 2), flush=True)
"""


def test_daemon_death_releases_a_waiter_in_memop_mode(tmp_path):
    """A caller whose stream already waits for a collective's "done" semaphore must not be
    left waiting for ever when the daemon is killed: the library notices the closed control
    socket, satisfies the wait itself and fails the communicator with mccsNotConnected."""
    import time
    sp = _spawn_daemon(tmp_path, 2)
    procs = []
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="fatal", MCCS_WC_TIMEOUT_MS="120000")
        procs = [subprocess.Popen([sys.executable, "-c", WAITER], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(2)]
        assert procs[1].stdout.readline().strip() == "JOINED"
        assert procs[0].stdout.readline().strip() == "POSTED"
        time.sleep(0.5)
        sp.proc.kill()           # no goodbye, no clean-up
        t0 = time.time()
        out, err = procs[0].communicate(timeout=60)
        took = time.time() - t0
        line = [l for l in out.splitlines() if l.startswith("RESULT ")]
        assert line, err[-2000:]
        code, later, _ = line[0].split()[1:]
        assert int(code) == -12 and int(later) == -12          # mccsNotConnected, now and from then on
        assert took < 20, f"the waiter needed {took:.1f}s, the 120 s completion timeout must not be what released it"
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        sp.stop()
