"""The C++ example apps against a stand-alone daemon on GPUs: hello, the three correctness
probes (`*_proto`), both bandwidth benchmarks and the trace replayer, i.e. the reference's
`src/mccs_examples` programs as an operator would start them. With one GPU all ranks sit on
device 0 (the daemon launches one cooperative kernel per collective); with several GPUs every
rank has its own and launches its kernels itself."""
import os
import subprocess

import pytest
import torch

from helpers import NATIVE, write_config

pytestmark = pytest.mark.gpu


def test_example_apps_on_gpus(tmp_path):
    from mccs_b200 import daemon
    ngpu = torch.cuda.device_count()
    n = min(max(ngpu, 2), 4)
    cfg = write_config(os.path.join(str(tmp_path), "mccs.toml"), os.path.join(str(tmp_path), "sock"), listen_port=-1,
                       wait_timeout_ms=5000)
    sp = daemon.spawn(cfg, env={"MCCS_LOG": "warn"})
    try:
        assert sp.backend == "cuda"
        env = dict(os.environ, MCCS_CONTROL=sp.control, MCCS_LOG="error", MCCS_WC_TIMEOUT_MS="30000")

        def run_ranks_app(name, extra):
            procs = [subprocess.Popen([os.path.join(NATIVE, name), "--rank", str(r), "--num-ranks", str(n),
                                       "--cuda-device-idx", str(r if ngpu >= n else 0)] + extra, env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(n)]
            outs = [p.communicate(timeout=180) for p in procs]
            for p, o in zip(procs, outs):
                assert p.returncode == 0, o
            return outs

        r = subprocess.run([os.path.join(NATIVE, "mccs_hello")], env=env, capture_output=True, text=True, timeout=60)
        assert r.returncode == 0 and "round trip ok" in r.stdout, r.stdout + r.stderr
        assert all("passed" in o[0] for o in run_ranks_app("allreduce_proto", ["--size", "1048576", "--communicator", "42"]))
        assert all("passed" in o[0] for o in run_ranks_app("allgather_proto", ["--size", "262144", "--communicator", "43"]))
        assert all("passed" in o[0] for o in run_ranks_app("reducescatter_proto", ["--size", "196608", "--communicator", "48"]))
        outs = run_ranks_app("allreduce_bench", ["--size", "33554432", "--size-in-byte", "--communicator", "44", "--round", "10",
                                                 "--epoch", "2"])
        assert outs[0][0].count("Algorithm bandwidth") == 2 and "Bus bandwidth" in outs[0][0]
        outs = run_ranks_app("allgather_bench", ["--size", "4194304", "--size-in-byte", "--communicator", "45", "--round", "10"])
        assert "Algorithm bandwidth" in outs[0][0]

        trace = tmp_path / "trace.toml"
        devs = list(range(n)) if ngpu >= n else [0] * n
        trace.write_text(f'communicator_id = 200\ncuda_devices = {devs}\n[[traces]]\nsize = 8388608\ntype = "all_reduce"\n'
                         'compute_interval = 500\n[[traces]]\nsize = 65536\ntype = "all_gather"\ncompute_interval = 100\n')
        procs = [subprocess.Popen([os.path.join(NATIVE, "traffic_gen"), "--rank", str(rk), "--config", str(trace), "--iters", "30",
                                   "--name", "job"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
                 for rk in range(n)]
        outs = [p.communicate(timeout=180) for p in procs]
        assert all(p.returncode == 0 for p in procs), outs
        assert "[job] Rank 0: run time:" in outs[0][0]
    finally:
        sp.stop()
