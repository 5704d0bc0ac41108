"""Service behaviour beyond plain collectives, all on the host backend (no GPU):
live reconfiguration, pause/resume with queued work, QoS windows, tracing, the admin
endpoint, and the failure paths — every failure is made on the host (a client that
exits, a rank that never joins), never by faulting a device."""
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import pytest
import torch

from helpers import NATIVE, REPO, fresh_comm_id, run_ranks, write_config


def _host(M):
    if M.backend() != "host":
        pytest.skip("host-backend test")


def test_live_reconfiguration_mid_run(service):
    """Four ranks run batches of 16 back-to-back all-reduces; at iteration 5 the ring
    order, the channel count and the algorithm are replaced while the job runs.
    Results before and after are identical and no rank restarts anything."""
    M = service
    _host(M)
    n, cid, count, iters = 4, fresh_comm_id(), 2048, 10
    port = M.daemon.embedded_admin_port()
    sync = threading.Barrier(n)

    def rank_fn(r):
        bufs = [M.Buffer(count * 4, r) for _ in range(16)]
        ts = [b.tensor(torch.float32, count) for b in bufs]
        c = M.Communicator(cid, r, n, device=r)
        plans, sums = [], []
        for it in range(iters):
            for i, t in enumerate(ts):
                t.fill_(float(r + i + it))
            if it == 5:
                sync.wait()
                if r == 0:
                    rep = M.reconfigure(port, [{"communicator_id": cid, "allreduce_algo": "ar_ring", "ctas": 3,
                                                "channels": [{"channel_id": 0, "ring": [3, 2, 1, 0]},
                                                             {"channel_id": 1, "ring": [0, 2, 1, 3]},
                                                             {"channel_id": 2, "ring": [1, 3, 0, 2]}]}])
                    assert rep["status"] == "ok", rep
                sync.wait()
            with M.group():
                for t in ts:
                    c.all_reduce(t)
            plans.append(c.last_plan())
            sums.append([float(t[0]) for t in ts])
        q = c.query()
        sync.wait()
        c.destroy()
        return plans, sums, q

    outs = run_ranks(n, rank_fn)
    for plans, sums, q in outs:
        for it in range(iters):
            assert sums[it] == [float(sum(r + i + it for r in range(n))) for i in range(16)]
        assert plans[4][0] != "ar_ring"
        assert plans[5] == ("ar_ring", 1) or plans[5][0] == "ar_ring"   # small messages use one channel
        assert q["config_epoch"] == 1 and q["async_error"] == 0
    stats = M.daemon.embedded_admin({"cmd": "stats"})["stats"]
    assert str(cid) not in stats["communicators"]          # destroyed


def test_reconfiguration_is_validated(service):
    M = service
    _host(M)
    cid = fresh_comm_id()

    def rank_fn(r):
        c = M.Communicator(cid, r, 2, device=r)
        if r == 0:
            bad = M.daemon.embedded_admin({"comm_patterns_reconfig": [
                {"communicator_id": cid, "channels": [{"channel_id": 0, "ring": [0, 0]}]}]}, type_=1)
            unknown = M.daemon.embedded_admin({"comm_patterns_reconfig": [{"communicator_id": 999999, "ctas": 2}]}, type_=1)
            algo = M.daemon.embedded_admin({"comm_patterns_reconfig": [{"communicator_id": cid, "allreduce_algo": "nope"}]}, type_=1)
            res = (bad, unknown, algo)
        else:
            res = None
        time.sleep(0.2)
        q = c.query()
        c.destroy()
        return res, q

    outs = run_ranks(2, rank_fn)
    bad, unknown, algo = outs[0][0]
    assert bad["status"] == "error" and "permutation" in bad["error"]
    assert unknown["status"] == "error"
    assert algo["status"] == "error"
    assert outs[0][1]["config_epoch"] == 0


def test_pause_queues_and_resume_replays(service):
    """While a communicator is paused its collectives are queued, not failed
    (the reference queues all-reduces that arrive during a reconfiguration,
    src/mccs/src/proxy/engine.rs:1045-1047), and run in order after resume."""
    M = service
    _host(M)
    n, cid = 2, fresh_comm_id()
    done = [0] * n
    gate = threading.Barrier(n + 1)

    def rank_fn(r):
        buf = M.Buffer(4096, r)
        t = buf.tensor(torch.float32, 1024)
        t.fill_(1.0)
        c = M.Communicator(cid, r, n, device=r)
        gate.wait()          # main thread pauses the communicator here
        gate.wait()
        for _ in range(3):
            c.all_reduce(t)
            done[r] += 1
        c.destroy()
        return float(t[0])

    results = {}
    th = threading.Thread(target=lambda: results.update(out=run_ranks(n, rank_fn)))
    th.start()
    gate.wait()
    assert M.daemon.embedded_admin({"cmd": "pause", "communicator_id": cid})["status"] == "ok"
    gate.wait()
    time.sleep(0.4)
    assert done == [0, 0]                       # queued behind the pause
    assert M.daemon.embedded_admin({"cmd": "resume", "communicator_id": cid})["status"] == "ok"
    th.join(30)
    assert done == [3, 3]
    assert results["out"] == [8.0, 8.0]         # 1 -> 2 -> 4 -> 8


def test_qos_window_schedule_gates_a_tenant(service):
    """The reference's Allow-window schedule (qos_schedule in mccs.toml): a tenant that
    may only send during the first 10 ms of every 60 ms epoch needs several epochs for
    a burst that otherwise takes microseconds."""
    M = service
    _host(M)
    n, cid = 2, fresh_comm_id()
    rep = M.daemon.embedded_admin({"cmd": "qos_set", "epoch_microsecs": 60000,
                                   "schedule": {str(cid): {"intervals": [[0, 10000]], "mode": "Allow"}}})
    assert rep["status"] == "ok"

    def rank_fn(r):
        buf = M.Buffer(4096, r)
        t = buf.tensor(torch.float32, 1024)
        t.fill_(1.0)
        c = M.Communicator(cid, r, n, device=r)
        t0 = time.time()
        stamps = []
        for _ in range(6):
            c.all_reduce(t)
            stamps.append((time.time() * 1e6) % 60000)
        c.destroy()
        return stamps, time.time() - t0, float(t[0])

    try:
        outs = run_ranks(n, rank_fn)
        stats = M.daemon.embedded_admin({"cmd": "stats"})["stats"]["qos"]["tenants"][str(cid)]
    finally:
        M.daemon.embedded_admin({"cmd": "qos_set", "epoch_microsecs": 0, "schedule": {}})
    for stamps, _, val in outs:
        assert val == 64.0
        # every completion falls inside (or just after) the allowed window
        assert all(s < 25000 for s in stamps), stamps
    assert stats["admitted"] == 6


def test_trace_records_collectives(service):
    M = service
    _host(M)
    assert M.daemon.embedded_admin({"cmd": "trace", "enabled": True, "clear": True})["status"] == "ok"
    cid = fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(1 << 16, r)
        c = M.Communicator(cid, r, 2, device=r)
        for _ in range(5):
            c.all_reduce(buf.tensor(torch.float32, 1000))
        c.destroy()

    run_ranks(2, rank_fn)
    rep = M.daemon.embedded_admin({"cmd": "trace", "enabled": False, "inline": True})
    events = rep["trace"]["traceEvents"]
    mine = [e for e in events if e["pid"] == cid]
    assert len(mine) >= 10 and all(e["ph"] == "X" and e["dur"] >= 0 for e in mine)
    assert any("rendezvous" in e["name"] for e in mine)


def test_admin_over_tcp(service):
    M = service
    _host(M)
    port = M.daemon.embedded_admin_port()
    assert port > 0
    rep = M.admin_request(port, {"cmd": "stats"})
    assert rep["status"] == "ok" and "qos" in rep["stats"] and rep["stats"]["clients"] >= 1
    assert M.admin_request(port, {"cmd": "no-such-command"})["status"] == "error"
    table = M.admin_request(port, {"cmd": "tuning_get"})["tuning"]
    assert "allreduce" in table and "8" in table["allreduce"]
    assert M.admin_request(port, {"cmd": "tuning_set", "tuning": {"allreduce": {"2": [[-1, "ar_twoshot", 7, 256]]}}})["status"] == "ok"
    cid = fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(1 << 20, r)
        c = M.Communicator(cid, r, 2, device=r)
        c.all_reduce(buf.tensor(torch.float32, 1 << 18))
        plan = c.last_plan()
        c.destroy()
        return plan

    try:
        assert run_ranks(2, rank_fn) == [("ar_twoshot", 7)] * 2
    finally:
        M.admin_request(port, {"cmd": "tuning_set", "tuning": table})


# ---------------------------------------------------------------------------------------------
# failure paths, each in its own daemon so that nothing leaks into other tests
# ---------------------------------------------------------------------------------------------
@pytest.fixture()
def private_daemon():
    from mccs_b200 import daemon
    d = tempfile.mkdtemp(prefix="mccs-ft-")
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=4, listen_port=-1,
                       force_host=True, extra="init_timeout_ms = 6000")   # well above the start-up skew of two client processes on a busy machine
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    yield sp
    sp.stop()


CLIENT = r"""
import os, sys, time, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); mode = os.environ["MODE"]
buf = M.Buffer(4096, rank)
t = buf.tensor(torch.float32, 1024); t.fill_(1.0)
try:
    c = M.Communicator(4242, rank, n, device=rank)
except Exception as e:
    print("INIT_ERROR", getattr(e, "code", None), flush=True); sys.exit(0)
c.all_reduce(t)
print("FIRST_OK", float(t[0]), flush=True)
if mode == "die" and rank == 1:
    os._exit(17)                      # no goodbye, no destroy: the daemon only sees the socket close
time.sleep(0.5)
t0 = time.time()
try:
    c.all_reduce(t)
    c.flush()
    print("SECOND_OK", flush=True)
except Exception as e:
    print("SECOND_ERROR", getattr(e, "code", None), round(time.time() - t0, 2), flush=True)
"""


def _spawn_clients(control, n, mode, ranks=None):
    env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=control, WORLD_SIZE=str(n), MODE=mode, MCCS_LOG="error",
               MCCS_WC_TIMEOUT_MS="20000")
    return [subprocess.Popen([sys.executable, "-c", CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                             stderr=subprocess.PIPE, text=True) for r in (ranks if ranks is not None else range(n))]


def test_client_death_turns_into_an_error_for_its_peers(private_daemon):
    procs = _spawn_clients(private_daemon.control, 2, "die")
    outs = [p.communicate(timeout=60) for p in procs]
    assert procs[1].returncode == 17
    assert "FIRST_OK 2.0" in outs[0][0]
    # the survivor is told that its peer is gone (-10), well inside the completion timeout
    line = [l for l in outs[0][0].splitlines() if l.startswith("SECOND_")][0]
    assert line.startswith("SECOND_ERROR -10"), outs[0]
    assert float(line.split()[2]) < 10
    # and the daemon keeps serving new communicators
    procs = _spawn_clients(private_daemon.control, 2, "ok")
    outs = [p.communicate(timeout=60) for p in procs]
    assert all("SECOND_OK" in o[0] for o in outs), outs


def test_rank_that_never_joins_times_out(private_daemon):
    procs = _spawn_clients(private_daemon.control, 2, "ok", ranks=[0])
    out, err = procs[0].communicate(timeout=60)
    assert "INIT_ERROR -6" in out, out + err       # mccsTimeout after init_timeout_ms


def test_example_apps_end_to_end(private_daemon, tmp_path):
    """The C++ apps against a stand-alone daemon: hello, the two correctness probes,
    both benchmarks, the trace replayer and the reconfiguration tool."""
    env = dict(os.environ, MCCS_CONTROL=private_daemon.control, MCCS_LOG="error")

    def run(args, **kw):
        return subprocess.run(args, env=env, capture_output=True, text=True, timeout=120, **kw)

    def run_ranks_app(name, n, extra):
        procs = [subprocess.Popen([os.path.join(NATIVE, name), "--rank", str(r), "--num-ranks", str(n),
                                   "--cuda-device-idx", str(r)] + extra, env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(n)]
        outs = [p.communicate(timeout=120) for p in procs]
        for p, o in zip(procs, outs):
            assert p.returncode == 0, o
        return outs

    r = run([os.path.join(NATIVE, "mccs_hello")])
    assert r.returncode == 0 and "round trip ok" in r.stdout
    outs = run_ranks_app("allreduce_proto", 4, ["--size", "65536", "--communicator", "42"])
    assert all("passed" in o[0] for o in outs)
    outs = run_ranks_app("allgather_proto", 3, ["--size", "65536", "--communicator", "43"])
    assert all("passed" in o[0] for o in outs)
    outs = run_ranks_app("reducescatter_proto", 3, ["--size", "49152", "--communicator", "48"])
    assert all("passed" in o[0] for o in outs)
    outs = run_ranks_app("allreduce_bench", 2, ["--size", "262144", "--communicator", "44", "--round", "5", "--epoch", "2"])
    assert outs[0][0].count("Algorithm bandwidth") == 2 and "Bus bandwidth" in outs[0][0]
    outs = run_ranks_app("allgather_bench", 2, ["--size", "65536", "--communicator", "45", "--round", "5"])
    assert "Algorithm bandwidth" in outs[0][0]

    trace = tmp_path / "trace.toml"
    trace.write_text('communicator_id = 200\ncuda_devices = [0, 1]\n[[traces]]\nsize = 65536\ntype = "all_reduce"\n'
                     'compute_interval = 500\n[[traces]]\nsize = 4096\ntype = "all_gather"\ncompute_interval = 100\n'
                     '[[traces]]\nsize = 32768\ntype = "reduce_scatter"\ncompute_interval = 100\n')
    csv = tmp_path / "times.csv"
    procs = [subprocess.Popen([os.path.join(NATIVE, "traffic_gen"), "--rank", str(rk), "--config", str(trace), "--iters", "30",
                               "--save-path", str(csv), "--name", "vgg"], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for rk in range(2)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "[vgg] Rank 0: run time:" in outs[0][0]
    assert len(csv.read_text().splitlines()) == 1 + 9      # header + iterations after the first 21 are dropped

    patch = tmp_path / "patch.toml"
    patch.write_text(f'mccs_addrs = ["127.0.0.1"]\nmccs_port = {private_daemon.admin_port}\n'
                     '[[comm_patterns_reconfig]]\ncommunicator_id = 600\n'
                     'channels = [ { channel_id = 0, ring = [1, 0] } ]\n')
    r = run([os.path.join(NATIVE, "ring_config"), "--config", str(patch)])
    assert "no communicator 600" in r.stdout          # reached the daemon, which rejected the unknown id
    r = run([os.path.join(NATIVE, "ring_config"), "--stats", "--port", str(private_daemon.admin_port)])
    assert r.returncode == 0 and json.loads(r.stdout.split(": ", 1)[1])["status"] == "ok"


def test_committed_tuning_table_is_accepted(service):
    """The measured size -> (variant, CTAs) table that ships with the package loads into
    the planner unchanged (every variant name known, every launch shape in range)."""
    import json
    M = service
    port = M.daemon.embedded_admin_port()
    with open(M.daemon.TUNING_FILE) as f:
        shipped = json.load(f)
    before = M.admin_request(port, {"cmd": "tuning_get"})["tuning"]
    try:
        assert M.admin_request(port, {"cmd": "tuning_set", "tuning": shipped})["status"] == "ok"
        after = M.admin_request(port, {"cmd": "tuning_get"})["tuning"]
        for kind in ("allreduce", "allgather"):
            for n, rows in shipped[kind].items():
                assert [r[1:3] for r in after[kind][n]] == [r[1:3] for r in rows]
                assert after[kind][n][-1][0] == -1
    finally:
        M.admin_request(port, {"cmd": "tuning_set", "tuning": before})


def test_hwinfo_reports_devices_and_peer_matrix(service):
    M = service
    hw = M.admin_request(M.daemon.embedded_admin_port(), {"cmd": "hwinfo"})["hwinfo"]
    n = len(hw["devices"])
    assert n >= 1 and hw["backend"] in ("host", "cuda")
    for d in hw["devices"]:
        assert len(d["peer_access"]) == n and d["peer_access"][d["index"]] is True


# ---------------------------------------------------------------------------------------------
# fused launches: consecutive queued AllReduces of one communicator in one kernel
# ---------------------------------------------------------------------------------------------
FUSION_CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"])
sizes = [1, 7, 256, 1000, 4096, 65539, 300, 12, 2048, 5, 33, 100000, 64, 8, 77, 1024]
bufs = [M.Buffer(max(s, 4) * 4, rank) for s in sizes]
c = M.Communicator(5151, rank, n, device=rank)
ok = True
for rnd in range(3):
    ts = [b.tensor(torch.float32, s) for b, s in zip(bufs, sizes)]
    for i, t in enumerate(ts):
        t.copy_(torch.arange(t.numel(), dtype=torch.float32) % 13 + rank + i + rnd)
    with M.group():
        for i, t in enumerate(ts):
            if i == 9:
                # a different operator in the middle: ends one batch, starts another
                c.all_reduce(t, op="max")
            else:
                c.all_reduce(t)
    for i, (t, s) in enumerate(zip(ts, sizes)):
        base = torch.arange(s, dtype=torch.float32) % 13 + i + rnd
        want = base + (n - 1) if i == 9 else base * n + sum(range(n))
        ok &= bool(torch.equal(t, want))
    # the same buffers again, one by one (nothing to fuse with)
    c.all_reduce(ts[2])
    ok &= bool(torch.equal(ts[2], (torch.arange(256, dtype=torch.float32) % 13 + 2 + rnd) * n * n + sum(range(n)) * n))
# members that depend on each other (the same buffer four times) must not share a launch
dep = bufs[4].tensor(torch.float32, 4096)
dep.fill_(1.0)
with M.group():
    for _ in range(4):
        c.all_reduce(dep)
ok &= bool(torch.all(dep == float(n) ** 4))
q = c.query()
st = M.admin_request(int(os.environ["ADMIN_PORT"]), {"cmd": "stats"})["stats"]["communicators"]["5151"]
c.destroy()
print("RESULT", json.dumps({"ok": ok, "launched": q["launched"], "async_error": q["async_error"],
                            "fused_launches": st["fused_launches"], "fused_members": st["fused_members"]}), flush=True)
"""


def test_consecutive_allreduces_share_one_launch(tmp_path):
    """With `fuse_allreduce = 8` a burst of queued AllReduces with the same type and
    operator goes out as fused launches (the reference's plan.rs:122-141), results are
    those of the separate collectives, and a change of operator splits the batch."""
    import json
    from mccs_b200 import daemon
    import mccs_b200 as M
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=4, listen_port=-1,
                       force_host=True,
                       extra="fuse_allreduce = 8\nsingle_through_fused = true\nskip_start_barrier = true\nkernel_writes_done = true")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        n = 4
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), MCCS_LOG="error",
                   ADMIN_PORT=str(sp.admin_port))
        procs = [subprocess.Popen([sys.executable, "-c", FUSION_CLIENT], env=dict(env, RANK=str(r)),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(n)]
        outs = [p.communicate(timeout=120) for p in procs]
        fused = []
        for p, (out, err) in zip(procs, outs):
            assert p.returncode == 0, err[-2000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["ok"] and res["async_error"] == 0
            assert res["launched"] == 3 * 17 + 4
            fused.append((res["fused_launches"], res["fused_members"]))
        # every fused launch carries 1..8 members (lone two-shot AllReduces also take the fused
        # kernel in this configuration), and the bursts did get fused
        launches, members = max(fused)
        assert launches >= 1 and launches < members <= 8 * launches, fused
    finally:
        sp.stop()


# ---------------------------------------------------------------------------------------------
# LD_PRELOAD allocation hook, against a stand-in CUDA runtime (no GPU needed)
# ---------------------------------------------------------------------------------------------
FAKE_CUDART = r"""
#include <stdlib.h>
int cudaMalloc(void** p, size_t n) { *p = malloc(n); return *p ? 0 : 2; }
int cudaFree(void* p) { free(p); return 0; }
int cudaGetDevice(int* d) { *d = 1; return 0; }
"""

PRELOAD_APP = r"""
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
int cudaMalloc(void**, size_t);
int cudaFree(void*);
typedef int (*meminfo_fn)(const void*, uint64_t*, uint64_t*, uint64_t*);
int main(void) {
  void *big = 0, *small = 0;
  if (cudaMalloc(&big, 2u << 20) || cudaMalloc(&small, 1024)) return 2;
  memset(big, 7, 2u << 20);                      /* service memory is ordinary shared memory on the host backend */
  meminfo_fn info = (meminfo_fn)dlsym(RTLD_DEFAULT, "mccsMemInfo");
  if (!info) return 3;
  uint64_t id = 0, off = 0, size = 0;
  int big_ours = info(big, &id, &off, &size) == 0;
  int small_ours = info(small, 0, 0, 0) == 0;
  printf("big_ours=%d size=%llu small_ours=%d\n", big_ours, (unsigned long long)size, small_ours);
  if (cudaFree(big) || cudaFree(small)) return 4;
  printf("big_after_free=%d\n", info(big, 0, 0, 0) == 0);
  return 0;
}
"""


def test_preload_hook_routes_large_allocations_to_the_service(private_daemon, tmp_path):
    from helpers import NATIVE
    (tmp_path / "fake_cudart.c").write_text(FAKE_CUDART)
    (tmp_path / "app.c").write_text(PRELOAD_APP)
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(tmp_path / "libfakecudart.so"), str(tmp_path / "fake_cudart.c")],
                   check=True)
    subprocess.run(["gcc", "-o", str(tmp_path / "app"), str(tmp_path / "app.c"), "-L" + str(tmp_path), "-lfakecudart",
                    "-ldl", "-Wl,-rpath," + str(tmp_path)], check=True)
    env = dict(os.environ, LD_PRELOAD=os.path.join(NATIVE, "libmccs_preload.so"), MCCS_CONTROL=private_daemon.control,
               MCCS_PRELOAD_MIN_BYTES=str(1 << 20), MCCS_LOG="error")
    res = subprocess.run([str(tmp_path / "app")], env=env, capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    # the 2 MiB request came from the service (device 1, as the runtime reported), the 1 KiB one did not
    assert "big_ours=1" in res.stdout and "small_ours=0" in res.stdout and "big_after_free=0" in res.stdout
    size = int(res.stdout.split("size=")[1].split()[0])
    assert size >= 2 << 20


CHAOS_CLIENT = r"""
import os, sys, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = int(os.environ["WORLD_SIZE"]); cid = int(os.environ["COMM"])
buf = M.Buffer(1 << 16, rank)
t = buf.tensor(torch.float32, 4096); t.fill_(1.0)
try:
    c = M.Communicator(cid, rank, n, device=rank)
except Exception as e:
    print("INIT_ERROR", getattr(e, "code", None), flush=True); sys.exit(0)
print("READY", flush=True)
try:
    for i in range(10 ** 7):
        t.fill_(1.0)
        if i % 7 == 3:
            with M.group():
                for _ in range(4):
                    c.all_reduce(t, op="max")
        else:
            c.all_reduce(t)
        if float(t[0]) not in (1.0, float(n)):
            print("BAD", float(t[0]), flush=True); sys.exit(3)
except Exception as e:
    print("ERROR", getattr(e, "code", None), flush=True)
"""


@pytest.mark.parametrize("launch", ["daemon", "client"])
def test_clients_killed_at_random_leave_the_daemon_clean(tmp_path, launch):
    """Three rounds of: a few ranks hammer a communicator, one of them is killed without
    warning at a random moment; the others get an error (never a wrong value, never a
    hang), the same communicator id is usable again right afterwards, and at the end the
    daemon holds no client, communicator or allocation."""
    import random
    import signal
    import time
    import mccs_b200 as M
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=4, listen_port=-1, force_host=True,
                       wait_timeout_ms=3000, extra=f"init_timeout_ms = 15000\nfuse_allreduce = 4\nlaunch = \"{launch}\"")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "error"})
    rng = random.Random(11)
    try:
        for rnd in range(3):
            n = rng.choice([2, 3, 4])
            env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, WORLD_SIZE=str(n), COMM="8000", MCCS_LOG="error",
                       MCCS_WC_TIMEOUT_MS="8000")
            procs = [subprocess.Popen([sys.executable, "-c", CHAOS_CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True) for r in range(n)]
            # wait until every rank is in its loop, then strike at a random moment
            for p in procs:
                assert p.stdout.readline().startswith("READY")
            time.sleep(rng.uniform(0.05, 0.8))
            victim = rng.randrange(n)
            procs[victim].send_signal(signal.SIGKILL)
            for r, p in enumerate(procs):
                out, err = p.communicate(timeout=30)
                assert "BAD" not in out
                if r != victim:
                    assert "ERROR" in out, (rnd, r, out, err[-500:])
            assert sp.proc.poll() is None, "the daemon died"
        # A session leaves the client count first and gives its memory back last, after the
        # streams that may still touch it have drained: allow that a moment.
        deadline = time.time() + 10
        while True:
            st = M.admin_request(sp.admin_port, {"cmd": "stats"})["stats"]
            if (st["clients"], st["communicators"], st["allocations"]) == (0, {}, 0) or time.time() > deadline:
                break
            time.sleep(0.1)
        assert st["clients"] == 0 and st["communicators"] == {} and st["allocations"] == 0
    finally:
        sp.stop()


TRANSPORT_CLIENT = r"""
import os, sys, json, torch
import mccs_b200 as M
rank = int(os.environ["RANK"]); devs = json.loads(os.environ["DEVS"]); cid = int(os.environ["COMM"]); port = int(os.environ["ADMIN_PORT"])
n = len(devs); dev = devs[rank]
a, b = M.Buffer(1 << 20, dev), M.Buffer(1 << 20, dev)
s, d = a.tensor(torch.float32, 100000), b.tensor(torch.float32, 100000)
s.fill_(float(rank + 1))
comm = M.Communicator(cid, rank, n, device=dev)
comm.all_reduce(s, d)
ar_plan = comm.last_plan()[0]
comm.all_reduce(s, d, algo="ar_twoshot")            # a request the connections may not be able to carry
asked_plan = comm.last_plan()[0]
ok = bool(torch.all(d == float(n * (n + 1) // 2)))
g = b.tensor(torch.uint8, 4096 * n)               # reuses the output buffer
comm.all_gather(a.tensor(torch.uint8, 4096), g)
ag_plan = comm.last_plan()[0]
st = M.admin_request(port, {"cmd": "stats"})["stats"]["communicators"][str(cid)]
comm.destroy()
print("RESULT", json.dumps({"ok": ok, "ar": ar_plan, "asked": asked_plan, "ag": ag_plan, "transport": st["transport"],
                            "host_staged": st["host_staged"]}), flush=True)
"""


def test_transport_is_chosen_per_connection(tmp_path):
    """A box on which one pair of GPUs has no peer access (host backend, `host_no_peer_access`):
    a communicator that contains the pair gets host-staged connections for it and peer-memory
    connections for the rest, keeps its scratch in host memory and runs the FIFO rings whatever
    is asked for; a communicator without the pair is untouched. (The reference picks a
    transporter per connection the same way, src/mccs/src/transport/setup.rs:346-361.)"""
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), host_devices=4, listen_port=-1, force_host=True,
                       extra="host_no_peer_access = [[1, 2]]")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        for cid, devs, want in ((8101, [0, 1, 2, 3], "mixed"), (8102, [0, 1, 3], "peer")):
            env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="error", DEVS=json.dumps(devs), COMM=str(cid),
                       ADMIN_PORT=str(sp.admin_port))
            procs = [subprocess.Popen([sys.executable, "-c", TRANSPORT_CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True) for r in range(len(devs))]
            for p in procs:
                out, err = p.communicate(timeout=120)
                assert p.returncode == 0, err[-2000:]
                res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
                assert res["ok"]
                if want == "mixed":
                    assert res["transport"] == "host_staged x2, nvlink_p2p x10" and res["host_staged"] is True
                    assert res["ar"] == "ar_ring" and res["asked"] == "ar_ring" and res["ag"] == "ag_ring"
                else:
                    assert res["transport"] == "nvlink_p2p" and res["host_staged"] is False
                    assert res["asked"] == "ar_twoshot" and "ring" not in res["ar"] and "ring" not in res["ag"]
    finally:
        sp.stop()


@pytest.mark.parametrize("launch", ["daemon", "client"])
def test_daemon_holds_nothing_after_many_client_lifetimes(tmp_path, launch):
    """A service runs for months: after hundreds of client lifetimes (connect, allocate, create a
    communicator, run, destroy, leave; some of them killed in the middle of their traffic) the
    daemon has as many open descriptors and memory mappings as before, and no more memory."""
    import signal
    import time
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, host_devices=2, force_host=True,
                       extra=f'launch = "{launch}"\ninit_timeout_ms = 3000')     # client: pads, status blocks and peers' buffers are handed out as descriptors too
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "error"})
    pid = sp.proc.pid

    def snapshot():
        fds = len(os.listdir(f"/proc/{pid}/fd"))
        rss = int([l for l in open(f"/proc/{pid}/status") if l.startswith("VmRSS")][0].split()[1])
        maps = sum(1 for _ in open(f"/proc/{pid}/maps"))
        return fds, rss, maps

    env = dict(os.environ, MCCS_CONTROL=sp.control, MCCS_LOG="error")

    def polite(k):
        ps = [subprocess.Popen([os.path.join(NATIVE, "allreduce_proto"), "--rank", str(r), "--num-ranks", "2", "--cuda-device-idx", str(r),
                                "--communicator", str(4000 + k % 7), "--size", "65536"], env=env, stdout=subprocess.DEVNULL,
                               stderr=subprocess.DEVNULL) for r in range(2)]
        return [p.wait(timeout=60) for p in ps]

    def killed(k):
        trace = os.path.join(d, "t.toml")
        with open(trace, "w") as f:
            f.write('communicator_id = 4100\ncuda_devices = [0, 1]\n[[traces]]\nsize = 262144\ntype = "all_reduce"\ncompute_interval = 50\n')
        ps = [subprocess.Popen([os.path.join(NATIVE, "traffic_gen"), "--rank", str(r), "--config", trace, "--iters", "1000000"], env=env,
                               stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for r in range(2)]
        time.sleep(0.15)
        ps[k % 2].send_signal(signal.SIGKILL)      # no goodbye; its peer ends with an error
        for p in ps:
            p.wait(timeout=60)

    try:
        for k in range(10):
            assert polite(k) == [0, 0]
        killed(0)
        time.sleep(0.5)
        before = snapshot()
        for k in range(120):
            assert polite(k) == [0, 0]
        for k in range(12):
            killed(k)
        deadline = time.time() + 10
        while time.time() < deadline:
            after = snapshot()
            if after[0] == before[0] and after[2] == before[2]:
                break
            time.sleep(0.2)
        assert after[0] == before[0] and after[2] == before[2], (before, after)
        assert after[1] <= before[1] + 2048, (before, after)          # kB
        assert sp.proc.poll() is None
    finally:
        sp.stop()


LIFETIMES_CLIENT = r"""
import os, torch, gc
import mccs_b200 as M
rank = int(os.environ["RANK"]); n = 2
def snap():
    return len(os.listdir("/proc/self/fd")), sum(1 for _ in open("/proc/self/maps")), int([l for l in open("/proc/self/status") if l.startswith("VmRSS")][0].split()[1])
def life(k):
    buf = M.Buffer(1 << 16, rank); t = buf.tensor(torch.float32, 4096); t.fill_(1.0)
    c = M.Communicator(5000 + k, rank, n, device=rank)
    for _ in range(3): c.all_reduce(t)
    with M.group():
        c.all_reduce(t); c.all_reduce(t)
    g = M.Buffer(1 << 12, rank)
    c.all_gather(g.tensor(torch.uint8, 1024)[:512] if False else g.tensor(torch.uint8, 2048)[rank * 1024:(rank + 1) * 1024], g.tensor(torch.uint8, 2048))
    c.destroy(); del t; buf.free(); g.free()
for k in range(20): life(k)
gc.collect(); a = snap()
for k in range(20, 120): life(k)
gc.collect(); b = snap()
import json; print("RESULT", json.dumps({"before": a, "after": b}), flush=True)
M.finalize()
"""


@pytest.mark.parametrize("launch", ["daemon", "client"])
def test_client_library_holds_nothing_after_many_communicator_lifetimes(tmp_path, launch):
    """The other side of the same question: a long-lived application that creates and destroys
    communicators and buffers (100 times here, with collectives and groups in between) ends
    with the descriptors and mappings it started with; with client launches that includes
    the peers' buffers, pads and status blocks mapped per communicator."""
    import json
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, host_devices=2, force_host=True,
                       extra=f'launch = "{launch}"')
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "error"})
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="error", LAUNCH=launch)
        procs = [subprocess.Popen([sys.executable, "-c", LIFETIMES_CLIENT], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True) for r in range(2)]
        for p in procs:
            out, err = p.communicate(timeout=300)
            assert p.returncode == 0, err[-3000:]
            res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][0][7:])
            assert res["after"][0] == res["before"][0] and res["after"][1] <= res["before"][1] + 2, res     # descriptors, mappings
            assert res["after"][2] <= res["before"][2] + 8192, res                                         # resident kB
    finally:
        sp.stop()


def test_per_client_limits(tmp_path):
    """`[limits]`: what one client may hold. Beyond the bounds an allocation answers out of
    memory and a communicator is refused, what the client already holds keeps working, freeing
    makes room again, and a connection beyond `max_clients` is turned away."""
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, host_devices=2, force_host=True,
                       extra="[limits]\nmax_clients = 2\nmax_allocations_per_client = 3\nmax_bytes_per_client = 1048576\n"
                             "max_communicators_per_client = 2")
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "error"})
    code = r"""
import os, sys, torch, json
import mccs_b200 as M
res = {}
a = M.Buffer(400000, 0); b = M.Buffer(400000, 0)
try:
    M.Buffer(400000, 0); res["bytes"] = "allowed"
except M.MccsError as e:
    res["bytes"] = e.code                       # 1.2 MB > max_bytes_per_client
c = M.Buffer(1000, 0)
try:
    M.Buffer(1000, 0); res["count"] = "allowed"
except M.MccsError as e:
    res["count"] = e.code                       # a fourth allocation
c.free()
d = M.Buffer(1000, 0); res["after_free"] = "ok"  # freeing made room
c1 = M.Communicator(1, 0, 1, device=0); c2 = M.Communicator(2, 0, 1, device=0)
try:
    M.Communicator(3, 0, 1, device=0); res["comms"] = "allowed"
except M.MccsError as e:
    res["comms"] = e.code
t = a.tensor(torch.float32, 1000); t.fill_(3.0); c1.all_reduce(t, b.tensor(torch.float32, 1000))
res["still_works"] = float(b.tensor(torch.float32, 1000)[7])
c2.destroy(); c3 = M.Communicator(3, 0, 1, device=0); res["after_destroy"] = "ok"
print("RESULT", json.dumps(res), flush=True)
sys.stdin.readline()          # stays connected until the test lets it go
"""
    try:
        env = dict(os.environ, PYTHONPATH=REPO, MCCS_CONTROL=sp.control, MCCS_LOG="off")
        first = subprocess.Popen([sys.executable, "-c", code], env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        line = first.stdout.readline()
        res = json.loads(line[7:])
        assert res == {"bytes": -2, "count": -2, "after_free": "ok", "comms": -2, "still_works": 3.0, "after_destroy": "ok"}, res
        # the first client is still connected; a second fits, a third does not
        hello = os.path.join(NATIVE, "mccs_hello")
        second = subprocess.Popen([sys.executable, "-c", "import sys, mccs_b200 as M; M.init(); print('IN', flush=True); sys.stdin.readline()"],
                                  env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        assert second.stdout.readline().startswith("IN")
        third = subprocess.run([hello], env=env, capture_output=True, text=True, timeout=60)
        assert third.returncode != 0
        for p in (second, first):
            p.stdin.close()
            p.wait(timeout=30)
        deadline = time.time() + 15          # the daemon notices the closed connections at its next look
        while True:
            fourth = subprocess.run([hello], env=env, capture_output=True, text=True, timeout=60)      # room again
            if fourth.returncode == 0 or time.time() > deadline:
                break
            time.sleep(0.2)
        assert fourth.returncode == 0, fourth.stdout + fourth.stderr
    finally:
        sp.stop()


@pytest.mark.parametrize("launch", ["daemon", "client"])
def test_clients_killed_on_a_busy_machine_do_not_take_the_daemon_down(tmp_path, launch):
    """A client that dies takes its memory with it while a surviving rank's proxy may be in the
    middle of a launch that reads it (it had looked at the communicator a moment before it was
    failed). The daemon lets such launches end and waits for every rank's stream before it
    releases the memory. Forty kills at varying moments with the machine's cores kept busy,
    which is what it took to hit the window."""
    import signal
    import time
    from mccs_b200 import daemon
    d = str(tmp_path)
    # (a victim that is killed before it has joined leaves its peer waiting for the init timeout)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, host_devices=2, force_host=True,
                       extra=f'launch = "{launch}"\ninit_timeout_ms = 3000')
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "off"})
    env = dict(os.environ, MCCS_CONTROL=sp.control, MCCS_LOG="off")
    trace = os.path.join(d, "t.toml")
    with open(trace, "w") as f:
        f.write('communicator_id = 4100\ncuda_devices = [0, 1]\n[[traces]]\nsize = 262144\ntype = "all_reduce"\ncompute_interval = 50\n')
    burners = [subprocess.Popen([sys.executable, "-c", "import time\nt = time.time()\nwhile time.time() - t < 60: pass"]) for _ in range(6)]
    try:
        for k in range(40):
            ps = [subprocess.Popen([os.path.join(NATIVE, "traffic_gen"), "--rank", str(r), "--config", trace, "--iters", "1000000"], env=env,
                                   stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for r in range(2)]
            time.sleep(0.05 + (k % 5) * 0.04)
            ps[k % 2].send_signal(signal.SIGKILL)
            for p in ps:
                p.wait(timeout=60)
            assert sp.proc.poll() is None, f"the daemon died after {k + 1} kills"
        # and it still serves
        ok = [subprocess.Popen([os.path.join(NATIVE, "allreduce_proto"), "--rank", str(r), "--num-ranks", "2", "--cuda-device-idx", str(r),
                                "--communicator", "4101", "--size", "65536"], env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
              for r in range(2)]
        assert [p.wait(timeout=60) for p in ok] == [0, 0]
    finally:
        for b in burners:
            b.kill()
        sp.stop()


@pytest.mark.parametrize("launch", ["daemon", "client"])
def test_ranks_killed_anywhere_in_their_lifetime(tmp_path, launch):
    """Forty short jobs of two to four ranks; in each, one or two ranks are killed at a random
    moment between their start and their end: while connecting, allocating, joining the
    communicator, in a collective, in their clean-up. The daemon stays up, gives every
    descriptor back and serves the next job."""
    import random
    import signal
    import time
    from mccs_b200 import daemon
    d = str(tmp_path)
    cfg = write_config(os.path.join(d, "mccs.toml"), os.path.join(d, "sock"), listen_port=-1, host_devices=4, force_host=True,
                       extra=f'launch = "{launch}"\ninit_timeout_ms = 2000')
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "off"})
    env = dict(os.environ, MCCS_CONTROL=sp.control, MCCS_LOG="off", MCCS_WC_TIMEOUT_MS="5000")
    rng = random.Random(5)

    def job(n, comm, size):
        return [subprocess.Popen([os.path.join(NATIVE, "allreduce_proto"), "--rank", str(r), "--num-ranks", str(n), "--cuda-device-idx", str(r),
                                  "--communicator", str(comm), "--size", str(size)], env=env, stdout=subprocess.DEVNULL,
                                 stderr=subprocess.DEVNULL) for r in range(n)]

    try:
        fds_before = None
        for k in range(40):
            n = rng.choice([2, 3, 4])
            ps = job(n, 6000 + k % 3, 1048576)
            time.sleep(rng.uniform(0.0, 0.08))
            for victim in rng.sample(range(n), rng.choice([1, 1, 2])):
                ps[victim].send_signal(signal.SIGKILL)
            for p in ps:
                p.wait(timeout=60)
            assert sp.proc.poll() is None, f"the daemon died in round {k}"
            if k == 10:
                time.sleep(0.5)
                fds_before = len(os.listdir(f"/proc/{sp.proc.pid}/fd"))
        deadline = time.time() + 10
        while time.time() < deadline and len(os.listdir(f"/proc/{sp.proc.pid}/fd")) != fds_before:
            time.sleep(0.2)
        assert len(os.listdir(f"/proc/{sp.proc.pid}/fd")) == fds_before
        assert [p.wait(timeout=60) for p in job(2, 6100, 65536)] == [0, 0]
    finally:
        sp.stop()
