"""Parallelism: data parallel is the one strategy the reference's workloads use (and
only as traces); see :mod:`mccs_b200.parallel.ddp`. :mod:`mccs_b200.parallel.zero` adds
the sharded-optimizer form of it on top of the service's ReduceScatter."""
from .ddp import DataParallel
from .zero import ShardedDataParallel

__all__ = ["DataParallel", "ShardedDataParallel"]
