"""Data-parallel training with sharded optimizer state (ZeRO stage 1) over the service.

The reference's workloads are plain data parallel: every rank all-reduces every gradient
and keeps a full optimizer (``workloads/setup-4_vgg.toml``). With ReduceScatter in the
service (``csrc/kernels/scatter.cuh``) the same step needs half the gradient traffic and
1/n of the optimizer state:

* gradients live in flat buckets in service memory, as in :class:`DataParallel`, padded so
  that a bucket splits into ``nranks`` equal, 128-byte aligned parts;
* when a bucket's last gradient has been accumulated it is reduce-scattered in place (average
  fused into the kernel) on the side stream while backward continues: rank r ends up with
  the averaged gradient of part r only;
* parameters live in flat buckets of the same layout; the optimizer made by
  :meth:`make_optimizer` owns one flat parameter per bucket, rank r's part, whose ``.grad``
  is the matching part of the gradient bucket, so its state covers 1/n of the model;
* :meth:`step` runs that optimizer and all-gathers the updated parts in place, after which
  every rank holds the same full parameters again.

The optimizer sees flat parts, not the module's tensors: per-tensor options (weight-decay
exclusions, per-layer learning rates) are not expressible; element-wise optimizers (SGD with
momentum, Adam, AdamW with one setting) give the same result as their unsharded form.
"""
from __future__ import annotations

from typing import List, Type

import torch

from ..client import Buffer, Communicator
from .ddp import DataParallel, _Bucket


class ShardedDataParallel(DataParallel):
    """:class:`DataParallel` with reduce-scattered gradients and a sharded optimizer."""

    def __init__(self, module: torch.nn.Module, comm: Communicator, bucket_mb: float = 25.0,
                 broadcast_parameters: bool = True, algo: str = "auto"):
        super().__init__(module, comm, bucket_mb=bucket_mb, broadcast_parameters=broadcast_parameters, algo=algo)
        n, r = comm.nranks, comm.rank
        self._param_buffers: List[Buffer] = []
        self._param_flats: List[torch.Tensor] = []
        with torch.no_grad():
            for b in self.buckets:
                esz = b.flat.element_size()
                buf = Buffer(max(b.padded * esz, 256), self._device)
                flat = buf.tensor(b.flat.dtype, b.padded)
                flat.zero_()
                for p, off in zip(b.params, b.offsets):
                    view = flat[off:off + p.numel()].as_strided(p.shape, p.stride())
                    view.copy_(p.detach())
                    p.data = view          # the module now computes on the flat bucket
                self._param_buffers.append(buf)
                self._param_flats.append(flat)
        self._part = [b.padded // n for b in self.buckets]
        self._rank = r

    def _bucket_multiple(self) -> int:
        return self.comm.nranks * 64      # equal parts, each a multiple of 128 bytes for 16-bit types

    def _part_of(self, flat: torch.Tensor, i: int) -> torch.Tensor:
        s = self._part[i]
        return flat[self._rank * s:(self._rank + 1) * s]

    def _reduce(self, bucket: _Bucket) -> None:
        self._launched += 1
        if self.comm.nranks == 1 or not self._sync:
            return
        i = self.buckets.index(bucket)
        mine = self._part_of(bucket.flat, i)
        if self._cuda:
            bucket.ready_event.record(torch.cuda.current_stream(self._device))
            self._stream.wait_event(bucket.ready_event)
            self.comm.reduce_scatter(bucket.flat, mine, op="avg", stream=self._stream)
        else:
            self.comm.reduce_scatter(bucket.flat, mine, op="avg")

    def make_optimizer(self, cls: Type[torch.optim.Optimizer], **kwargs) -> torch.optim.Optimizer:
        """An optimizer of type ``cls`` over this rank's parts of the parameter buckets."""
        shards = []
        for i, (b, pflat) in enumerate(zip(self.buckets, self._param_flats)):
            p = torch.nn.Parameter(self._part_of(pflat, i), requires_grad=True)
            p.grad = self._part_of(b.flat, i)
            shards.append(p)
        self._shards = shards
        return cls(shards, **kwargs)

    def step(self, optimizer: torch.optim.Optimizer) -> None:
        """Optimizer step on this rank's parts, then every rank's part to everybody."""
        optimizer.step()
        if self.comm.nranks == 1:
            return
        for i, pflat in enumerate(self._param_flats):
            mine = self._part_of(pflat, i)
            self.comm.all_gather(mine, pflat, nbytes=mine.numel() * mine.element_size())
        self.comm.wait()

    def optimizer_state_elements(self) -> int:
        """Parameter elements this rank's optimizer keeps state for (1/nranks of the model)."""
        return sum(self._part)

    def release(self) -> None:
        # hand the parameters back as ordinary tensors before the buckets go away
        with torch.no_grad():
            for b in self.buckets:
                for p in b.params:
                    p.data = p.data.clone()
        super().release()
        for buf in self._param_buffers:
            buf.free()
        self._param_buffers = []
        self._param_flats = []
