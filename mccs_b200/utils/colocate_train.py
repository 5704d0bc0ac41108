"""Co-located data-parallel training jobs on one box, through the service or over NCCL.

Scenarios (the reference replays such jobs as traces, ``workloads/setup-4_*.toml``; here the
real training loops of :mod:`mccs_b200.parallel.train` run):

    cnn              ResNet-50 on GPUs 0-3 next to VGG-16 on GPUs 4-7 (fp32, batch 64 per GPU)
    gpt              GPT-2-medium on all GPUs, alone (bf16 parameters and gradient buckets)
    gpt-with-resnet  GPT-2-medium on all 8 GPUs, high priority and weight 4, sharing GPUs 0-3
                     with a ResNet-50 job

On a box with four to seven GPUs the same scenarios run at half the width (ResNet-50 on 0-1 next
to VGG-16 on 2-3; GPT-2-medium on 0-3 sharing 0-1 with ResNet-50).

    python -m mccs_b200.utils.colocate_train --scenario cnn --backend mccs
    python -m mccs_b200.utils.colocate_train --scenario cnn --backend nccl

With ``--backend mccs`` one stand-alone ``mccsd`` serves all jobs (each job is a tenant: its
communicator id carries its QoS weight and priority). The jobs warm up on their own and start
their timed steps together. Prints one JSON object with every job's images/s or tokens/s.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import subprocess
import sys
import tempfile

from .. import daemon

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SCENARIOS = {
    "cnn": [
        {"name": "resnet50", "model": "resnet50", "devices": [0, 1, 2, 3], "comm_id": 300, "steps": 100},
        {"name": "vgg16", "model": "vgg16", "devices": [4, 5, 6, 7], "comm_id": 301, "steps": 40},
    ],
    "gpt": [
        {"name": "gpt2-medium", "model": "gpt2-medium", "devices": list(range(8)), "comm_id": 310, "steps": 30},
    ],
    "gpt-with-resnet": [
        {"name": "gpt2-medium", "model": "gpt2-medium", "devices": list(range(8)), "comm_id": 310, "steps": 30},
        {"name": "resnet50", "model": "resnet50", "devices": [0, 1, 2, 3], "comm_id": 311, "steps": 90},
    ],
}
QOS = "[qos.tenants.310]\nweight = 4.0\npriority = 1\n[qos.tenants.311]\nweight = 1.0\n"


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenario", default="cnn", choices=sorted(SCENARIOS))
    ap.add_argument("--backend", default="mccs", choices=["mccs", "nccl"])
    ap.add_argument("--steps-scale", type=float, default=1.0)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--comm-ctas", type=int, default=0)
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--dry-run-model", default="", help="every job trains this model instead of its own, with a small batch "
                    "(e.g. gpt2-tiny): a run of the tool itself, on a machine without GPUs too")
    a = ap.parse_args()
    jobs = [dict(j) for j in SCENARIOS[a.scenario]]
    import torch
    ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 8
    if 4 <= ngpu < 8:
        # a four-GPU box: the same scenarios at half the width (jobs of 2 and 4 GPUs)
        for j in jobs:
            j["devices"] = sorted({d // 2 for d in j["devices"]})
    out = {"scenario": a.scenario, "backend": a.backend, "jobs": {}}
    with tempfile.TemporaryDirectory(prefix="mccs-cotrain-") as work:
        env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
        sp = None
        if a.backend == "mccs":
            with open(work + "/mccs.toml", "w") as f:
                f.write(daemon.default_config(work + "/sock", listen_port=-1) + QOS)
            sp = daemon.spawn(work + "/mccs.toml", env={"MCCS_LOG": "warn"})
            env["MCCS_CONTROL"] = sp.control
        procs = []
        try:
            for j in jobs:
                cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(len(j["devices"])),
                       "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m", "mccs_b200.parallel.train",
                       "--model", j["model"], "--backend", a.backend, "--comm-id", str(j["comm_id"]),
                       "--devices", ",".join(map(str, j["devices"])), "--steps", str(max(int(j["steps"] * a.steps_scale), 2)),
                       "--warmup", str(a.warmup), "--name", j["name"], "--sync-dir", work + "/sync", "--sync-jobs", str(len(jobs))]
                if a.dry_run_model:
                    cmd[cmd.index("--model") + 1] = a.dry_run_model
                    cmd += ["--batch", "2", "--seq", "32", "--bucket-mb", "0.05"]
                if a.backend == "mccs":
                    cmd += ["--control", sp.control]
                    if a.comm_ctas > 0:
                        cmd += ["--comm-ctas", str(a.comm_ctas), "--admin-port", str(sp.admin_port)]
                procs.append((j, subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
            rc = 0
            for j, p in procs:
                try:
                    so, se = p.communicate(timeout=a.timeout)
                except subprocess.TimeoutExpired:
                    p.kill()
                    so, se = p.communicate()
                line = [l for l in so.splitlines() if l.startswith("{")]
                if p.returncode != 0 or not line:
                    rc = 1
                    out["jobs"][j["name"]] = {"error": se[-1500:]}
                else:
                    out["jobs"][j["name"]] = json.loads(line[-1])
        finally:
            for _, p in procs:
                if p.poll() is None:
                    p.kill()
            if sp is not None:
                sp.stop()
    print(json.dumps(out))
    return rc


if __name__ == "__main__":
    sys.exit(main())
