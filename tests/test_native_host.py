"""Runs the C++ unit tests of the host-side native code (IPC rings, fd passing,
TOML/JSON, configuration schema, planner, ring step accounting, QoS arbiter)."""
import os
import subprocess

from helpers import NATIVE


def test_host_unit_tests():
    res = subprocess.run([os.path.join(NATIVE, "host_tests")], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout


def _sanitizer_run(target):
    """Builds and runs the in-process daemon + clients + operator stress test under a
    sanitizer; skipped where the system compiler has no sanitizer runtime."""
    import shutil

    import pytest
    from helpers import REPO
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    probe = subprocess.run([cxx, "-fsanitize=" + ("thread" if target == "tsan" else "address"), "-x", "c++", "-",
                            "-o", "/dev/null"], input="int main(){return 0;}", capture_output=True, text=True)
    if probe.returncode != 0:
        pytest.skip("no sanitizer runtime for " + cxx)
    res = subprocess.run(["make", target, "SAN_CXX=" + cxx], cwd=REPO, capture_output=True, text=True, timeout=900)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    assert "stress_host: 0 failure(s)" in out
    assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out and "runtime error" not in out
    if target == "asan":
        assert "no crash" in out      # the parser fuzzing ran to its end


def test_thread_sanitizer_stress():
    _sanitizer_run("tsan")


def test_address_sanitizer_stress():
    _sanitizer_run("asan")


def test_kernels_on_the_simt_emulator():
    """The collective kernels' own source, compiled for the host against the SIMT emulator
    in csrc/tests/sim: every variant, 2-8 ranks, odd sizes, in place, fused launches,
    per-rank pipelining, and the bounded-wait error paths."""
    from helpers import REPO
    res = subprocess.run(["make", "simtest"], cwd=REPO, capture_output=True, text=True, timeout=900)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    assert ", 0 failed" in out
