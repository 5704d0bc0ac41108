"""Tooling: the benchmark launcher (dependency order, weak services, output files,
teardown) and the QoS interval planner."""
import os
import subprocess
import sys

from helpers import REPO


def test_qos_interval_planner_matches_reference_algorithm():
    from mccs_b200.utils.qos_intervals import calculate_intervals, to_toml
    prem, vic, epoch = calculate_intervals(premium_comp=300, premium_comm=100, victim_comp=150, victim_comm=50)
    assert epoch == 400                                    # lcm(400, 200)
    assert prem == [(0, 100)]
    assert vic == [(100, 150), (300, 350)]                 # first fit into the gap [100, 400)
    # windows never overlap
    for a, b in prem:
        for c, d in vic:
            assert b <= c or d <= a
    text = to_toml(epoch, {7: prem, 8: vic})
    sys.path.insert(0, REPO)
    import tomllib
    parsed = tomllib.loads(text)
    assert parsed["qos_schedule"]["epoch_microsecs"] == 400
    assert parsed["qos_schedule"]["schedule"]["8"]["intervals"] == [[100, 150], [300, 350]]


def test_launcher_runs_workers_in_dependency_order(tmp_path):
    marker = tmp_path / "order.txt"
    spec = tmp_path / "bench.toml"
    spec.write_text(f'''
name = "unit"
[[worker]]
bin = "python"
args = "-c \\"import time; open(r'{marker}', 'a').write('service\\\\n'); time.sleep(60)\\""
weak = true
dependencies = []
[[worker]]
bin = "python"
args = "-c \\"open(r'{marker}', 'a').write('job1\\\\n'); print('hello from job1')\\""
dependencies = [0]
delay = 4.0
[[worker]]
bin = "python"
args = "-c \\"open(r'{marker}', 'a').write('job2\\\\n')\\""
dependencies = [1]
''')
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.launcher", "--benchmark", str(spec), "--output-dir", str(out),
                          "--timeout", "30"], env=dict(os.environ, PYTHONPATH=REPO), capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    assert marker.read_text().split() == ["service", "job1", "job2"]
    assert "hello from job1" in (out / "unit" / "1_python.stdout").read_text()


def test_latency_breakdown_tool_on_host_backend():
    """The per-stage latency report runs end to end (two gloo ranks, host backend) and
    its host-side stages add up to less than the measured period."""
    import json
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="warn")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "mccs_b200.utils.latency",
                          "--bytes", "4K", "--iters", "100", "--warmup", "10", "--json"],
                         env=env, capture_output=True, text=True, timeout=300, cwd=REPO)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["n"] == 2 and out["backend"] == "host" and out["period_us"] > 0
    st = out["stages"]
    assert st["rendezvous"]["n"] == 200 and st["launch"]["n"] == 200
    assert st["rendezvous"]["median_us"] + st["launch"]["median_us"] < 5 * out["period_us"] + 50


def test_report_table_and_svg(tmp_path):
    """Sweep CSV -> markdown table (service vs NCCL, roofline fraction) and SVG curves."""
    import xml.dom.minidom
    csv_path = tmp_path / "s.csv"
    rows = ["coll,dtype,n,bytes,algo,ctas,ms,algbw_GBps,busbw_GBps"]
    for i, size in enumerate([1 << 20, 1 << 24, 1 << 28]):
        rows.append(f"allreduce,bf16,8,{size},nccl,0,{0.03 * 4 ** i},{size / (0.03 * 4 ** i) / 1e6},{size / (0.03 * 4 ** i) / 1e6 * 1.75}")
        rows.append(f"allreduce,bf16,8,{size},ar_nvls_twoshot,16,{0.04 * 3 ** i},{size / (0.04 * 3 ** i) / 1e6},{size / (0.04 * 3 ** i) / 1e6 * 1.75}")
        rows.append(f"allreduce,bf16,8,{size},ar_twoshot,32,{0.05 * 4 ** i},{size / (0.05 * 4 ** i) / 1e6},{size / (0.05 * 4 ** i) / 1e6 * 1.75}")
    csv_path.write_text("\n".join(rows) + "\n")
    svg = tmp_path / "c.svg"
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.report", str(csv_path), "--svg", str(svg)],
                         capture_output=True, text=True, cwd=REPO, env=dict(os.environ, PYTHONPATH=REPO), timeout=60)
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("| allreduce")]
    assert len(lines) == 3 and all("ar_nvls_twoshot" in l for l in lines)
    assert "| 0.75 |" in lines[0]            # 1 MiB: 0.03 ms NCCL vs 0.04 ms service
    doc = xml.dom.minidom.parse(str(svg))
    assert len(doc.getElementsByTagName("polyline")) == 2


import pytest


@pytest.mark.parametrize("sync", ["events", "memops"])
def test_multi_tenant_tool_on_host_backend(sync):
    """Four applications on overlapping devices, QoS weights, a live reconfiguration of one
    of them in the middle: every rank finishes without error and the reconfigured
    application reports the new configuration epoch."""
    import json
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.multi_tenant", "--iters", "30", "--reconfig-at", "15",
                          "--bytes", "65536", "--batch", "4", "--host-devices", "4", "--timeout", "200", "--sync", sync],
                         capture_output=True, text=True, cwd=REPO, env=dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error"),
                         timeout=400)
    assert res.returncode == 0, res.stderr[-3000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert set(out["apps"]) == {"A", "B", "C", "D"}
    for name, app in out["apps"].items():
        assert app["finite"] and app["async_error"] == 0, (name, app)
    assert out["apps"]["C"]["config_epoch"] == 1 and out["apps"]["A"]["config_epoch"] == 0
    assert all(t["admitted"] == 35 * 4 for t in out["qos_stats"].values())


def test_multi_tenant_tool_with_client_side_launch():
    """The same four applications with `[b200] launch = "client"`: every rank's library runs
    its own kernels (on the emulator) while weights, admission and the live reconfiguration
    stay with the daemon."""
    import json
    env = dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error", MCCS_B200_EXTRA='launch = "client"')
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.multi_tenant", "--iters", "20", "--reconfig-at", "10",
                          "--bytes", "65536", "--batch", "4", "--host-devices", "4", "--timeout", "300", "--sync", "events"],
                         capture_output=True, text=True, cwd=REPO, env=env, timeout=500)
    assert res.returncode == 0, res.stderr[-3000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    for name, app in out["apps"].items():
        assert app["finite"] and app["async_error"] == 0, (name, app)
    assert out["apps"]["C"]["config_epoch"] == 1 and out["apps"]["A"]["config_epoch"] == 0
    assert all(t["admitted"] == 25 * 4 and t["outstanding_bytes"] == 0 for t in out["qos_stats"].values())


def test_bench_script_contract_on_cpu():
    """bench.py runs end to end without a GPU (host backend, reduced size) and prints the
    one JSON line with every key of the benchmark contract; the reference arm prints
    either its result or the reason it is unavailable."""
    import json
    import socket
    env = dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error")
    one = subprocess.run([sys.executable, "bench.py", "--steps", "2", "--warmup", "1"], capture_output=True, text=True,
                         cwd=REPO, env=env, timeout=300)
    assert one.returncode == 0, one.stderr[-2000:]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", str(port), "bench.py", "--gpus", "2", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, cwd=REPO, env=env, timeout=300)
    assert two.returncode == 0, two.stderr[-2000:]
    for res, n in ((one, 1), (two, 2)):
        lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
        assert len(lines) == 1                      # rank 0 prints ONE line
        out = json.loads(lines[0])
        for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                    "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
            assert key in out, key
        assert out["n_gpus"] == n and out["steps"] == 2 and out["warmup"] >= 3 and out["higher_is_better"] is True
        assert out["metric"] == "allreduce_algbw_GBps" and out["dtype"] == "bf16" and out["data"] == "synthetic"
        assert {"model", "global_batch", "seq_len", "parallelism"} <= set(out["config"])
        assert set(out["config"]) == {"model", "global_batch", "seq_len", "parallelism"}     # the same words in both arms
        assert out["config"]["parallelism"] == f"dp{n}" and out["detail"]["verified"] is True
        assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(out["e2e"])
        assert out["e2e"]["h2d_bytes_per_step"] > 0 and out["e2e"]["d2h_bytes_per_step"] > 0
        assert out["gpu_launches"] == 2 * n and out["detail"]["launch"] == "daemon"
    ref = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, cwd=REPO, env=env, timeout=300)
    assert ref.returncode == 0
    r = json.loads([l for l in ref.stdout.splitlines() if l.startswith("{")][-1])
    assert r["impl"] == "reference" and ("value" in r or "unavailable" in r)


def test_sweep_tuner_and_report_pipeline_on_cpu(tmp_path, service):
    """The sweep tool end to end without a GPU (two gloo ranks, host backend): every
    variant x CTA count is measured through the live-reconfiguration path, the tuning
    table it writes is accepted by a planner, and the report tool digests its CSV."""
    import json
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    csv_path, tuning = str(tmp_path / "sweep.csv"), str(tmp_path / "tuning.json")
    env = dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", str(port), "-m", "mccs_b200.utils.sweep", "--mode", "tune", "--dtypes", "bf16",
                          "--min-bytes", "32K", "--max-bytes", "128K", "--ctas", "2,4", "--iters", "3", "--warmup", "1",
                          "--out", csv_path, "--tuning", tuning], capture_output=True, text=True, cwd=REPO, env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    table = json.load(open(tuning))
    assert [r[0] for r in table["allreduce"]["2"]] == [32768, 65536, -1]
    assert all(r[1].startswith("ar_") for r in table["allreduce"]["2"]) and all(r[1].startswith("ag_") for r in table["allgather"]["2"])
    M = service
    admin = M.daemon.embedded_admin_port()
    before = M.admin_request(admin, {"cmd": "tuning_get"})["tuning"]
    try:
        assert M.admin_request(admin, {"cmd": "tuning_set", "tuning": table})["status"] == "ok"
    finally:
        M.admin_request(admin, {"cmd": "tuning_set", "tuning": before})
    rep = subprocess.run([sys.executable, "-m", "mccs_b200.utils.report", csv_path], capture_output=True, text=True, cwd=REPO,
                         env=env, timeout=60)
    assert rep.returncode == 0 and rep.stdout.count("| allreduce | bf16 | 2 |") == 3 and rep.stdout.count("| allgather |") == 3


def test_trace_colocation_tool_on_host_backend():
    """The real-workload co-location experiment as a dry run: the three traces side by side
    under the three policies (none, weight + priority, weight + priority + time windows),
    sizes and compute intervals scaled down; every job of every policy reports its times."""
    import json
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.colocate_traces", "--host", "--scale", "0.001", "--size-scale", "0.0005",
                          "--time-scale", "0.02", "--vgg-comm-us", "400", "--gpt-comm-us", "100", "--timeout", "120"],
                         capture_output=True, text=True, cwd=REPO, env=dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error"), timeout=400)
    assert res.returncode == 0, res.stderr[-3000:]
    out = json.loads(res.stdout[res.stdout.index("{"):])
    assert set(out["policies"]) == {"fair", "qosv1", "qosv2"}
    for policy, jobs in out["policies"].items():
        assert set(jobs) == {"vgg", "gpt_1", "gpt_2"}
        for name, job in jobs.items():
            assert job["iterations"] == 22 and job["jct_ms"] is not None and job["mean_iter_ms"] > 0, (policy, name, job)


def test_shipped_configurations_are_consistent():
    """Every file under configs/: the daemon accepts its configurations (`mccsd --check`), a
    malformed file is refused, every worker of a launch description names a program, a module
    and files that exist, every trace names devices and well-formed steps."""
    import glob
    import importlib.util
    import shlex
    import tomllib
    from helpers import NATIVE
    mccsd = os.path.join(NATIVE, "mccsd")
    for cfg in ("configs/mccs.toml", "configs/mccs_qos.toml"):
        res = subprocess.run([mccsd, "--config", os.path.join(REPO, cfg), "--check"], capture_output=True, text=True, timeout=60)
        assert res.returncode == 0 and "configuration ok" in res.stdout, res.stdout + res.stderr
    assert "2 tenant policies" in res.stdout
    bad = subprocess.run([mccsd, "--config", os.path.join(REPO, "Makefile"), "--check"], capture_output=True, text=True, timeout=60)
    assert bad.returncode == 2
    launches = [f for f in glob.glob(os.path.join(REPO, "configs/launch/*.toml")) if "worker" in tomllib.load(open(f, "rb"))]
    assert len(launches) >= 3
    for path in launches:
        spec = tomllib.load(open(path, "rb"))
        workers = spec["worker"]
        for i, w in enumerate(workers):
            assert w["bin"] == "python" or os.path.exists(os.path.join(NATIVE, "mccsd" if w["bin"] in ("mccs", "mccsd") else w["bin"])), (path, w["bin"])
            assert all(0 <= d < len(workers) and d != i for d in w.get("dependencies", [])), (path, i)
            words = shlex.split(w.get("args", ""))
            for k, word in enumerate(words):
                if word.startswith("configs/"):
                    assert os.path.exists(os.path.join(REPO, word)), (path, word)
                if word == "-m" and k + 1 < len(words):
                    assert importlib.util.find_spec(words[k + 1]) is not None, (path, words[k + 1])
    traces = glob.glob(os.path.join(REPO, "configs/workloads/*.toml"))
    assert len(traces) >= 4
    for path in traces:
        t = tomllib.load(open(path, "rb"))
        assert isinstance(t["communicator_id"], int) and len(t["cuda_devices"]) >= 1, path
        for step in t["traces"]:
            assert step["size"] > 0 and step["type"] in ("all_reduce", "all_gather", "reduce_scatter") and step["compute_interval"] >= 0, (path, step)
    patch = tomllib.load(open(os.path.join(REPO, "configs/launch/reconfig-patch.toml"), "rb"))
    assert patch["comm_patterns_reconfig"][0]["channels"][0]["ring"]


def test_clock_sampler_reads_clocks_and_throttle_reasons(tmp_path, monkeypatch):
    """The sampler that runs beside every timed region, against a stand-in `nvidia-smi`:
    median and maximum clocks, peak power, and the throttle reasons that were active."""
    import stat
    import time
    from mccs_b200.utils.timing import ClockSampler, bus_factor
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "echo '0, 1965, 1965, 250.1, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo '0, 1800, 1965, 990.5, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1700, 1965, 1001.0, 0x0000000000000004, Not Active, Active, Not Active, Active'\n"
                    "echo 'garbage line'\n"
                    "sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    s = ClockSampler(gpu_index=0)
    s.start()
    for _ in range(100):
        if len(s.lines) >= 4:
            break
        time.sleep(0.05)
    out = s.stop()
    assert out["samples"] == 3 and out["sm_mhz"] == 1800 and out["sm_max_mhz"] == 1965 and out["power_w_max"] == 1001.0
    assert out["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]
    assert bus_factor("allreduce", 8) == 1.75 and bus_factor("allgather", 8) == 0.875 and bus_factor("allreduce", 1) == 1.0
    # no nvidia-smi at all: an empty record, not an error
    monkeypatch.setenv("PATH", str(tmp_path / "nowhere"))
    s2 = ClockSampler()
    s2.start()
    assert s2.stop()["samples"] == 0


def test_every_tool_starts_and_describes_itself():
    """`--help` of every command-line tool of the package, of the training driver and of the
    benchmark script: imports resolve and the argument parsers build."""
    env = dict(os.environ, PYTHONPATH=REPO)
    mods = ["mccs_b200.utils." + m for m in ("sweep", "report", "multi_tenant", "qos_intervals", "latency", "profile_case",
                                             "launcher", "colocate_traces", "colocate_train", "metrics")] + ["mccs_b200.parallel.train"]
    procs = [subprocess.Popen([sys.executable, "-m", m, "--help"], cwd=REPO, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for m in mods]
    procs.append(subprocess.Popen([sys.executable, "bench.py", "--help"], cwd=REPO, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    for name, p in zip(mods + ["bench.py"], procs):
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0 and "usage" in out.lower(), (name, err[-1000:])
    from helpers import NATIVE
    for app in ("mccsd", "allreduce_bench", "allgather_bench", "traffic_gen", "ring_config", "mccs_hello"):
        res = subprocess.run([os.path.join(NATIVE, app), "--help"], capture_output=True, text=True, timeout=60)
        assert "usage" in (res.stdout + res.stderr).lower(), (app, res.stdout + res.stderr)


def test_metrics_exporter_serves_the_daemons_counters(service):
    """`mccs_b200.utils.metrics`: the statistics of a live daemon as Prometheus text, through
    the render function and through the HTTP endpoint a scraper would ask."""
    import threading
    import urllib.request
    import torch
    from helpers import fresh_comm_id, run_ranks
    from mccs_b200.utils import metrics
    M = service
    if M.backend() != "host":
        pytest.skip("host-backend test")
    cid = fresh_comm_id()

    def rank_fn(r):
        buf = M.Buffer(4096, r)
        c = M.Communicator(cid, r, 2, device=r)
        for _ in range(3):
            c.all_reduce(buf.tensor(torch.float32, 256))
        c.flush()
        text = metrics.scrape(M.daemon.embedded_admin_port()) if r == 0 else ""
        import time
        time.sleep(0.2)          # rank 1 keeps the communicator alive while rank 0 reads
        c.destroy()
        return text

    text = run_ranks(2, rank_fn)[0]
    assert f'mccs_comm_planned_total{{comm="{cid}"}} 3' in text
    assert f'mccs_tenant_admitted_total{{comm="{cid}"}} 3' in text
    assert f'mccs_tenant_deferred_total{{comm="{cid}",reason="window"}} 0' in text
    assert f'mccs_comm_info{{comm="{cid}",variant="' in text and "# TYPE mccs_comm_completed_total counter" in text
    assert "mccs_client_allocated_bytes{client=" in text and "mccs_client_communicators{client=" in text
    for line in text.splitlines():        # every sample line is `name{labels} number`
        if line and not line.startswith("#"):
            float(line.rsplit(" ", 1)[1])
    srv = metrics.serve(M.daemon.embedded_admin_port(), 0)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    try:
        port = srv.server_address[1]
        body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10).read().decode()
        assert "mccs_clients " in body and "mccs_allocated_bytes " in body
        with pytest.raises(Exception):
            urllib.request.urlopen(f"http://127.0.0.1:{port}/other", timeout=10)
    finally:
        srv.shutdown()
        srv.server_close()


def test_multi_tenant_tool_with_a_reference_placement():
    """`--setting 2`: the placement of the reference's second multi-application experiment (a
    four-GPU job across all host pairs next to two two-GPU jobs), on eight host devices."""
    import json
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.multi_tenant", "--setting", "2", "--iters", "12", "--reconfig-at", "0",
                          "--bytes", "65536", "--batch", "1", "--host-devices", "8", "--timeout", "200"],
                         capture_output=True, text=True, cwd=REPO, env=dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error"), timeout=400)
    assert res.returncode == 0, res.stderr[-3000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["setting"] == 2 and set(out["apps"]) == {"blue", "green", "red"}
    assert out["apps"]["blue"]["devices"] == [0, 4, 2, 6] and out["apps"]["green"]["devices"] == [1, 3]
    for name, app in out["apps"].items():
        assert app["finite"] and app["async_error"] == 0, (name, app)


def test_colocated_training_tool_dry_run():
    """`colocate_train --scenario gpt-with-resnet` as a dry run on the host backend: an
    eight-rank job and a four-rank job that shares its devices, both tenants of one daemon
    (weights and priority from the scenario), warm up apart, start their timed steps
    together and report their rates."""
    import json
    res = subprocess.run([sys.executable, "-m", "mccs_b200.utils.colocate_train", "--scenario", "gpt-with-resnet", "--steps-scale", "0.1",
                          "--warmup", "1", "--dry-run-model", "gpt2-tiny", "--timeout", "300"],
                         capture_output=True, text=True, cwd=REPO, env=dict(os.environ, PYTHONPATH=REPO, MCCS_LOG="error"), timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    jobs = out["jobs"]
    assert set(jobs) == {"gpt2-medium", "resnet50"} and jobs["gpt2-medium"]["n_gpus"] == 8 and jobs["resnet50"]["n_gpus"] == 4
    for j in jobs.values():
        assert "error" not in j and j["backend"] == "mccs" and j["ms_per_step"] > 0 and j["last_loss"] < j["first_loss"] + 0.5
