"""Measurement helpers shared by bench.py and the sweep: device timing with CUDA
events (max over ranks), clock sampling during the timed region, bus-bandwidth
factors.

The reference times on the host (``Instant`` around the launch loop plus one stream
synchronise, rank 0 only: ``src/mccs_examples/allreduce_bench/src/main.rs:147-169``);
here every number is taken on the device and reduced with MAX over the ranks.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Callable, List, Optional

import torch

_CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def bus_factor(coll: str, n: int) -> float:
    """algBW -> busBW factor, the one nccl-tests and the reference use
    (``allreduce_bench/src/main.rs:168-169``, ``allgather_bench/src/main.rs:161-176``)."""
    if n <= 1:
        return 1.0
    return 2.0 * (n - 1) / n if coll == "allreduce" else (n - 1) / n


class ClockSampler:
    """Samples ``nvidia-smi`` every 200 ms while a timed region runs."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.lines: List[str] = []
        self._thread: Optional[threading.Thread] = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_CLOCK_QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            assert self.proc is not None and self.proc.stdout is not None
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self._thread is not None:
            self._thread.join(2)
        sm, sm_max, power, reasons = [], [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                sm_max.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(sm_max) if sm_max else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def device_time_ms(fn: Callable[[], None], steps: int, stream: Optional[torch.cuda.Stream] = None,
                   barrier: Optional[Callable[[], None]] = None) -> float:
    """Milliseconds per step of ``steps`` back-to-back calls of ``fn``, timed with CUDA
    events on the launching stream, with a barrier and a device synchronise on both
    sides of the timed region."""
    stream = stream or torch.cuda.current_stream()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return start.elapsed_time(stop) / steps
