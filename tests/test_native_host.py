"""Runs the C++ unit tests of the host-side native code (IPC rings, fd passing,
TOML/JSON, configuration schema, planner, ring step accounting, QoS arbiter)."""
import os
import subprocess

from helpers import NATIVE


def test_host_unit_tests():
    res = subprocess.run([os.path.join(NATIVE, "host_tests")], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout
