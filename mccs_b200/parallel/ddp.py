"""Data-parallel training over the service: bucketed gradient AllReduce that
overlaps with backward.

The reference evaluates "real workloads" as traces of one monolithic AllReduce per
iteration with a sleep for the compute phase and a stream synchronise after every
operation (``workloads/setup-4_vgg.toml``, ``src/mccs_examples/traffic_gen/src/main.rs:171-204``).
This module runs the real thing: gradients live in flat buckets of ``bucket_mb`` MB
(25 MB, torch DDP's default) that are allocated in service
memory, each parameter's ``.grad`` is a view into its bucket, and as soon as the last
gradient of a bucket has been accumulated the bucket is all-reduced in place on a
side stream while backward continues on the compute stream. The averaging is fused
into the collective kernel (``SumPostDiv``), so no elementwise kernel follows it.
"""
from __future__ import annotations

import contextlib
from typing import Iterable, List, Optional

import torch

from ..client import Buffer, Communicator, backend


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter], dtype: torch.dtype, device: int, cuda: bool, multiple: int = 1):
        self.params = params
        self.numel = sum(p.numel() for p in params)
        esz = torch.empty((), dtype=dtype).element_size()
        # 256-byte slots keep every view aligned for the 16-byte vector path
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() * esz + 255) // 256 * 256 // esz
        self.padded = (off + multiple - 1) // multiple * multiple   # sharded subclasses cut the bucket into equal parts
        self.buffer = Buffer(max(self.padded * esz, 256), device)
        self.flat = self.buffer.tensor(dtype, self.padded)
        self.flat.zero_()
        self.pending = len(params)
        self.ready_event = torch.cuda.Event() if cuda else None


class DataParallel:
    """Wraps a module for data-parallel training with the mccs service.

    ``comm`` is this rank's :class:`~mccs_b200.client.Communicator`. Call
    :meth:`finish` after ``loss.backward()`` and before the optimizer step.
    """

    def __init__(self, module: torch.nn.Module, comm: Communicator, bucket_mb: float = 25.0,
                 broadcast_parameters: bool = True, algo: str = "auto"):
        self.module = module
        self.comm = comm
        self.algo = algo
        self._cuda = backend() == "cuda"
        self._device = comm.device
        # High priority: the CTAs of a bucket's kernel wait for their peers on the other GPUs, so
        # they should get SMs as soon as backward's kernels release some, not after its queue.
        self._stream = torch.cuda.Stream(device=self._device, priority=-1) if self._cuda else None
        params = [p for p in module.parameters() if p.requires_grad]
        if broadcast_parameters and comm.nranks > 1:
            self._broadcast(params)
        # Buckets follow the reverse parameter order, the order in which backward
        # produces gradients, so the first buckets complete early.
        self.buckets: List[_Bucket] = []
        limit = int(bucket_mb * 1024 * 1024)
        cur: List[torch.nn.Parameter] = []
        cur_bytes = 0
        cur_dtype: Optional[torch.dtype] = None
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > limit or p.dtype != cur_dtype):
                self.buckets.append(_Bucket(cur, cur_dtype, self._device, self._cuda, self._bucket_multiple()))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            self.buckets.append(_Bucket(cur, cur_dtype, self._device, self._cuda, self._bucket_multiple()))
        self._launched = 0
        self._sync = True
        # Bucket reductions are issued from a side stream and only their sum total is
        # awaited, once, at the end of backward: no per-bucket wait is queued anywhere.
        self.comm.set_deferred_wait(True)
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                # same strides as the parameter (channels-last weights keep that layout)
                p.grad = b.flat[off:off + p.numel()].as_strided(p.shape, p.stride())
                p.register_post_accumulate_grad_hook(self._make_hook(b))

    def _bucket_multiple(self) -> int:
        """Element count every bucket is padded to a multiple of."""
        return 1

    # -- parameter broadcast (rank 0's values) through an all-gather ----------------
    def _broadcast(self, params: Iterable[torch.nn.Parameter]) -> None:
        n, r = self.comm.nranks, self.comm.rank
        for p in params:
            nb = p.numel() * p.element_size()
            nb16 = (nb + 15) // 16 * 16
            buf = Buffer(nb16 * n, self._device)
            full = buf.bytes_tensor()
            mine = full[r * nb16:r * nb16 + nb]
            with torch.no_grad():
                mine.copy_(p.detach().reshape(-1).view(torch.uint8))
                self.comm.all_gather(full[r * nb16:(r + 1) * nb16], full, nbytes=nb16)
                p.copy_(full[:nb].view(p.dtype).view_as(p))
            if self._cuda:
                torch.cuda.current_stream(self._device).synchronize()
            buf.free()

    def _make_hook(self, bucket: _Bucket):
        def hook(param: torch.nn.Parameter) -> None:
            bucket.pending -= 1
            if bucket.pending == 0:
                self._reduce(bucket)
        return hook

    def _reduce(self, bucket: _Bucket) -> None:
        self._launched += 1
        if self.comm.nranks == 1 or not self._sync:
            return
        if self._cuda:
            # The side stream picks up after the gradients written so far.
            bucket.ready_event.record(torch.cuda.current_stream(self._device))
            self._stream.wait_event(bucket.ready_event)
            self.comm.all_reduce(bucket.flat, op="avg", algo=self.algo, stream=self._stream)
        else:
            self.comm.all_reduce(bucket.flat, op="avg", algo=self.algo)

    def finish(self) -> None:
        """Wait (on the compute stream) for all gradient reductions of this step."""
        for b in self.buckets:
            if b.pending != 0:
                # Some parameter of this bucket got no gradient in this step (unused in the
                # forward pass): reduce it now so that all ranks issue the same collectives.
                self._reduce(b)
            b.pending = len(b.params)
        if self.comm.nranks > 1 and self._sync:
            self.comm.wait()          # the compute stream waits for all bucket reductions of this step
        self._launched = 0

    @contextlib.contextmanager
    def no_sync(self):
        """Gradient accumulation, as torch DDP's ``no_sync``: backward passes inside the block
        only add to the gradient buckets, nothing is reduced; the first backward after the
        block reduces the accumulated sums. Call :meth:`finish` after every backward, inside
        the block too (it then only re-arms the buckets), and :meth:`zero_grad` once per
        optimizer step."""
        self._sync = False
        try:
            yield self
        finally:
            self._sync = True

    def zero_grad(self) -> None:
        """Zero the gradient buckets (keeps ``.grad`` views in place)."""
        for b in self.buckets:
            b.flat.zero_()

    def __call__(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def gradient_bytes(self) -> int:
        return sum(b.numel * b.flat.element_size() for b in self.buckets)

    def release(self) -> None:
        self.comm.set_deferred_wait(False)
        for b in self.buckets:
            for p in b.params:
                p.grad = None
            b.buffer.free()
        self.buckets = []
