import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200 box)")


def _native_ready() -> bool:
    d = os.path.join(REPO, "mccs_b200", "_native")
    return all(os.path.exists(os.path.join(d, f)) for f in ("libmccs.so", "libmccs_daemon.so", "libmccs_kernels.so", "mccsd", "host_tests", "reducescatter_proto"))


@pytest.fixture(scope="session", autouse=True)
def native_build():
    """The native libraries are build products (git-ignored): build them once when a
    fresh checkout runs the tests."""
    if not _native_ready():
        import __graft_entry__
        __graft_entry__.build()
    yield


@pytest.fixture(scope="session")
def service():
    """One in-process daemon for the whole test session: CUDA backend when the marker
    selection runs on a GPU box, host backend otherwise. Short device wait bound so
    that fault-path tests finish quickly."""
    import mccs_b200 as M
    prefix = f"/tmp/mccs-pytest-{os.getuid()}-{os.getpid()}"
    extra = '[qos.tenants.901]\nweight = 2.0\n'
    M.daemon.start_embedded(prefix=prefix, listen_port=-1, wait_timeout_ms=2000, host_devices=8, extra="")
    M.init(prefix + "/control.sock")
    yield M
    M.finalize()
    M.daemon.stop_embedded()
