"""Benchmark launcher: starts the workers of a TOML description in dependency order,
tees their output to files, enforces a timeout and tears everything down.

It reads the format of the reference's launcher (``launcher/src/main.rs:44-67``;
e.g. ``eval/dynamic-config/launch-ring-reconfig.toml``):

    name = "setup4-dynamic"
    [[worker]]
    bin = "mccsd"                      # a name in mccs_b200/_native, or "python", or a path
    args = "--config configs/mccs.toml"
    weak = true                        # a service: not waited for, terminated at the end
    dependencies = []
    [[worker]]
    bin = "traffic_gen"
    args = "--rank 0 --config configs/workloads/gpt.toml --iters 100 --name gpt"
    dependencies = [0]                 # start after worker 0 is up
    delay = 2.0                        # optional: seconds to wait after the dependencies

The reference runs workers over ssh on four hosts; inside one box every worker is a
local process (``host`` is accepted and ignored). ``env = { KEY = "value" }`` adds
environment variables per worker.

    python -m mccs_b200.utils.launcher --benchmark configs/launch/reconfig.toml --output-dir /tmp/out
"""
from __future__ import annotations

import argparse
import os
import shlex
import signal
import subprocess
import sys
import time
from typing import List

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
NATIVE = os.path.join(REPO, "mccs_b200", "_native")


def load_toml(path: str) -> dict:
    import tomllib
    with open(path, "rb") as f:
        return tomllib.load(f)


def resolve_bin(name: str) -> List[str]:
    if name == "python":
        return [sys.executable]
    if name in ("mccs", "mccsd"):
        return [os.path.join(NATIVE, "mccsd")]
    cand = os.path.join(NATIVE, name)
    if os.path.exists(cand):
        return [cand]
    return [name]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--benchmark", "-b", required=True)
    ap.add_argument("--output-dir", "-o", default="/tmp/mccs-launcher")
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--silent", action="store_true")
    args = ap.parse_args()
    spec = load_toml(args.benchmark)
    workers = spec.get("worker", [])
    name = spec.get("name", os.path.splitext(os.path.basename(args.benchmark))[0])
    out_dir = os.path.join(args.output_dir, name)
    os.makedirs(out_dir, exist_ok=True)
    procs: List[subprocess.Popen | None] = [None] * len(workers)
    started = [0.0] * len(workers)
    files = []
    deadline = time.time() + args.timeout
    rc = 0

    def ready(i: int) -> bool:
        for d in workers[i].get("dependencies", []):
            if procs[d] is None:
                return False
            # a service needs a moment to come up; a job must have finished
            if workers[d].get("weak", False):
                if time.time() - started[d] < float(workers[i].get("delay", 1.0)):
                    return False
            elif procs[d].poll() is None:
                return False
        return True

    try:
        while time.time() < deadline:
            for i, w in enumerate(workers):
                if procs[i] is None and ready(i):
                    cmd = resolve_bin(w["bin"]) + shlex.split(w.get("args", ""))
                    env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
                    env.setdefault("USER", os.environ.get("LOGNAME", "user"))   # what the daemon assumes when unset
                    for k, v in w.get("env", {}).items():
                        v = str(v)
                        for name, val in env.items():
                            v = v.replace("${" + name + "}", val)
                        env[k] = v
                    tag = f"{i}_{os.path.basename(w['bin'])}"
                    so = open(os.path.join(out_dir, tag + ".stdout"), "w")
                    se = open(os.path.join(out_dir, tag + ".stderr"), "w")
                    files += [so, se]
                    procs[i] = subprocess.Popen(cmd, cwd=REPO, env=env, stdout=so, stderr=se, start_new_session=True)
                    started[i] = time.time()
                    if not args.silent:
                        print(f"[launcher] started #{i}: {' '.join(cmd)}", flush=True)
            strong = [i for i, w in enumerate(workers) if not w.get("weak", False)]
            if all(procs[i] is not None and procs[i].poll() is not None for i in strong):
                break
            for i in strong:
                p = procs[i]
                if p is not None and p.poll() not in (None, 0):
                    rc = p.returncode
            if rc:
                break
            time.sleep(0.05)
        else:
            print("[launcher] timeout", file=sys.stderr)
            rc = 124
        for i in [i for i, w in enumerate(workers) if not w.get("weak", False)]:
            if procs[i] is not None and procs[i].returncode not in (None, 0):
                rc = rc or procs[i].returncode
    finally:
        # terminate what is still running: each worker was started in its own process group
        for p in procs:
            if p is not None and p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        t_end = time.time() + 10
        for p in procs:
            if p is not None:
                try:
                    p.wait(max(0.1, t_end - time.time()))
                except subprocess.TimeoutExpired:
                    os.killpg(p.pid, signal.SIGKILL)
        for f in files:
            f.close()
    if not args.silent:
        print(f"[launcher] outputs in {out_dir}, exit {rc}", flush=True)
    return rc


if __name__ == "__main__":
    sys.exit(main())
