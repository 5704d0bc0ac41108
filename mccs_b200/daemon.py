"""Starting and stopping the service daemon from Python.

Two ways, both ending with a control socket that clients connect to:

* :func:`start_embedded` runs the daemon as native threads inside the calling
  process (``libmccs_daemon.so``). The launcher rank of a ``torchrun`` job does this
  so that no separate service has to be started by hand; the kernels are then
  launched from this process.
* :func:`spawn` starts the stand-alone ``mccsd`` binary the way the reference is
  run (``mccs --host <idx> --config mccs.toml``, ``src/mccs/src/main.rs:16-24``).

The configuration is the reference's ``mccs.toml`` schema plus a ``[b200]`` table;
see ``csrc/daemon/config.h``.
"""
from __future__ import annotations

import json
import os
import subprocess
import time
from typing import Optional

from . import _lib

_embedded_path: Optional[str] = None


TUNING_FILE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "tuning_b200.json")


def default_config(prefix: str, *, transport: str = "auto", nvls: bool = True, channel_count: int = 2,
                   wait_timeout_ms: int = 10000, host_devices: int = 8, force_host: bool = False,
                   listen_port: int = -1, trace: bool = False, sync: str = "auto", tuning_file: Optional[str] = None,
                   extra: str = "") -> str:
    """TOML text of a daemon configuration with its sockets under ``prefix``.

    The size -> (variant, CTAs) table measured on B200 (``configs/tuning_b200.json``,
    written by ``python -m mccs_b200.utils.sweep --tuning``) is loaded when present;
    pass ``tuning_file=""`` for the built-in defaults. ``MCCS_B200_EXTRA`` (environment)
    adds lines to the ``[b200]`` table of every configuration built here, e.g.
    ``MCCS_B200_EXTRA='fuse_allreduce = 8;skip_start_barrier = true'`` (``;`` separates lines),
    which is how the benchmark tools are pointed at an experimental setting.
    """
    if tuning_file is None:
        tuning_file = TUNING_FILE if os.path.exists(TUNING_FILE) else ""
    wait_timeout_ms = int(os.environ.get("MCCS_WAIT_TIMEOUT_MS", wait_timeout_ms))
    env_extra = os.environ.get("MCCS_B200_EXTRA", "")
    if env_extra:
        # before `extra`, which may open another table
        extra = "\n".join([line.strip() for line in env_extra.split(";") if line.strip()] + [extra])
    tuning_line = f'tuning_file = "{tuning_file}"' if tuning_file else ""
    return f"""
listen_port = {listen_port}
mccs_daemon_prefix = "{prefix}"
[control]
prefix = "{prefix}"
path = "control.sock"
[comm_default_config]
buffer_sizes = [4194304]
channel_count = {channel_count}
[b200]
transport = "{transport}"
nvls = {"true" if nvls else "false"}
wait_timeout_ms = {wait_timeout_ms}
host_devices = {host_devices}
force_host_backend = {"true" if force_host else "false"}
trace = {"true" if trace else "false"}
sync = "{sync}"
{tuning_line}
{extra}
"""


def start_embedded(config_toml: Optional[str] = None, *, prefix: Optional[str] = None, **kw) -> str:
    """Start the in-process daemon (idempotent) and return its control socket path.

    Also points this process's client shim at it through ``MCCS_CONTROL``.
    """
    global _embedded_path
    lib = _lib.daemon_lib()
    if config_toml is None:
        prefix = prefix or f"/tmp/mccs-{os.getuid()}-{os.getpid()}"
        config_toml = default_config(prefix, **kw)
    rc = lib.mccsd_start(config_toml.encode())
    if rc != 0:
        raise RuntimeError(f"embedded mccs daemon failed to start (status {rc})")
    _embedded_path = lib.mccsd_control_path().decode()
    os.environ["MCCS_CONTROL"] = _embedded_path
    return _embedded_path


def stop_embedded() -> None:
    global _embedded_path
    if _embedded_path is not None:
        _lib.daemon_lib().mccsd_stop()
        _embedded_path = None


def embedded_admin(body: dict, type_: int = 2) -> dict:
    """Admin request to the in-process daemon without going through TCP."""
    out = _lib.daemon_lib().mccsd_admin(type_, json.dumps(body).encode())
    return json.loads(out.decode())


def embedded_admin_port() -> int:
    return int(_lib.daemon_lib().mccsd_admin_port())


def embedded_backend() -> str:
    k = _lib.daemon_lib().mccsd_backend_kind()
    return {0: "host", 1: "cuda"}.get(k, "none")


def describe_embedded() -> str:
    return _lib.daemon_lib().mccsd_describe().decode()


class SpawnedDaemon:
    """A stand-alone ``mccsd`` child process."""

    def __init__(self, proc: subprocess.Popen, control: str, admin_port: int, backend: str):
        self.proc = proc
        self.control = control
        self.admin_port = admin_port
        self.backend = backend

    def stop(self, timeout: float = 10.0) -> int:
        if self.proc.poll() is None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                self.proc.wait()
        return self.proc.returncode

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()


def spawn(config_path: str, *, env: Optional[dict] = None, timeout: float = 120.0) -> SpawnedDaemon:
    """Start ``mccsd --config config_path`` and wait until it accepts clients."""
    exe = os.environ.get("MCCSD") or os.path.join(_lib.NATIVE_DIR, "mccsd")   # MCCSD: another build, e.g. a sanitizer one
    if not os.path.exists(exe):
        raise FileNotFoundError(f"{exe} is missing: run `make -j` at the repository root")
    e = dict(os.environ)
    if env:
        e.update(env)
    proc = subprocess.Popen([exe, "--config", config_path], stdout=subprocess.PIPE, env=e, text=True)
    deadline = time.time() + timeout
    while time.time() < deadline:
        line = proc.stdout.readline()
        if not line:
            if proc.poll() is not None:
                raise RuntimeError(f"mccsd exited with {proc.returncode} before it was ready")
            continue
        if line.startswith("MCCSD_READY"):
            fields = dict(f.split("=", 1) for f in line.split()[1:])
            return SpawnedDaemon(proc, fields["control"], int(fields["admin_port"]), fields["backend"])
    proc.kill()
    raise TimeoutError("mccsd did not become ready")
