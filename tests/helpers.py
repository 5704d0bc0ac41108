"""Test helpers: ranks as threads of the test process, subprocess clients."""
from __future__ import annotations

import os
import subprocess
import sys
import threading
from typing import Callable, Dict, List, Optional

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NATIVE = os.path.join(REPO, "mccs_b200", "_native")

_next_comm_id = [1000]


def fresh_comm_id() -> int:
    _next_comm_id[0] += 1
    return _next_comm_id[0]


def run_ranks(n: int, fn: Callable[[int], object], timeout: float = 120.0) -> List[object]:
    """Run fn(rank) on n threads (the shim releases the GIL while it waits), re-raise
    the first failure, return the per-rank results."""
    results: Dict[int, object] = {}
    errors: List[BaseException] = []

    def wrap(r: int) -> None:
        try:
            results[r] = fn(r)
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=wrap, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout)
        if t.is_alive():
            raise TimeoutError("a rank did not finish")
    if errors:
        raise errors[0]
    return [results[r] for r in range(n)]


def run_python(code: str, env: Optional[dict] = None, timeout: float = 120.0) -> subprocess.CompletedProcess:
    e = dict(os.environ)
    e["PYTHONPATH"] = REPO + os.pathsep + e.get("PYTHONPATH", "")
    if env:
        e.update(env)
    return subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=timeout)


def popen_python(code: str, env: Optional[dict] = None) -> subprocess.Popen:
    e = dict(os.environ)
    e["PYTHONPATH"] = REPO + os.pathsep + e.get("PYTHONPATH", "")
    if env:
        e.update(env)
    return subprocess.Popen([sys.executable, "-c", code], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)


def write_config(path: str, prefix: str, **kw) -> str:
    from mccs_b200.daemon import default_config
    os.makedirs(os.path.dirname(path), exist_ok=True)
    with open(path, "w") as f:
        f.write(default_config(prefix, **kw))
    return path
