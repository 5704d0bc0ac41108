"""Parallelism: data parallel is the one strategy the reference's workloads use (and
only as traces); see :mod:`mccs_b200.parallel.ddp`."""
from .ddp import DataParallel

__all__ = ["DataParallel"]
