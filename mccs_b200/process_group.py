"""``torch.distributed`` backend "mccs": collectives of a process group served by the
managed collective communication daemon.

    import mccs_b200.process_group            # registers the backend
    dist.init_process_group("mccs", rank=r, world_size=n)   # MCCS_CONTROL names the daemon
    dist.all_reduce(t)

The reference has no framework layer (its "workloads" are traffic traces replayed by
``src/mccs_examples/traffic_gen``); this backend is what lets real PyTorch jobs be
tenants of the service. Every rank of the group is one client of the daemon and owns
one communicator rank (``src/libmccs/src/communicator.rs:15-45``).

Tensors that live in service memory (allocated with :func:`empty` / :class:`Buffer`, or
through :func:`mem_pool`) are used in place: the kernel reads and writes them directly.
Other tensors are staged through a service buffer on the caller's stream (one copy in,
one copy out). Collectives are stream ordered: when a call returns, the work is
enqueued on the caller's current stream. The returned ``Work`` wraps a future that is
completed at once and, for CUDA tensors, knows their devices: it carries an event recorded
behind the collective, so ``work.wait()`` (or a callback chained to the future) on any
stream waits for the collective the way it would for the ``nccl`` backend.
"""
from __future__ import annotations

import os
import threading
import weakref
from typing import Optional

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import (AllgatherOptions, AllreduceOptions, AllToAllOptions, BarrierOptions, BroadcastOptions,
                                        GatherOptions, ReduceOp, ReduceOptions, ReduceScatterOptions, ScatterOptions,
                                        _create_work_from_future)
from torch.futures import Future

from . import _lib, client
from .client import Buffer, Communicator

_OP_NAMES = {
    ReduceOp.SUM: "sum", ReduceOp.PRODUCT: "prod", ReduceOp.MIN: "min", ReduceOp.MAX: "max", ReduceOp.AVG: "avg",
}


def _op_name(op) -> str:
    try:
        return _OP_NAMES[op]
    except (KeyError, TypeError):
        pass
    for k, v in _OP_NAMES.items():
        if op == k:
            return v
    raise NotImplementedError(f"reduce op {op} is not supported by the mccs backend")


def _allreduce_options(op) -> AllreduceOptions:
    o = AllreduceOptions()
    o.reduceOp = op
    return o


def _cuda_devices(result) -> list:
    found = set()

    def visit(x) -> None:
        if isinstance(x, torch.Tensor):
            if x.is_cuda:
                found.add(x.device)
        elif isinstance(x, (list, tuple)):
            for y in x:
                visit(y)

    visit(result)
    return sorted(found, key=lambda d: d.index or 0)


def _done(result) -> "dist.Work":
    """A finished ``Work`` for a collective that has been enqueued on the caller's current
    stream. For CUDA results the future is told their devices: completing it then records an
    event on those devices' current streams, and whoever waits for it (on any stream) waits
    for that event, that is for the collective."""
    devices = _cuda_devices(result)
    try:
        fut: Future = Future(devices=devices) if devices else Future()
    except Exception:          # a torch build whose futures take no devices: stream order alone then
        fut = Future()
    fut.set_result(result)
    return _create_work_from_future(fut)


from .ops import all_gather as _ops_all_gather, all_reduce as _ops_all_reduce, arena as _arena, in_service_memory  # noqa: E402
from .ops import reduce_scatter as _ops_reduce_scatter  # noqa: E402


def empty(numel: int, dtype: torch.dtype, device: int = 0):
    """A 1-D tensor in service memory plus the :class:`Buffer` that keeps it alive."""
    esz = torch.empty((), dtype=dtype).element_size()
    buf = Buffer(max(numel * esz, 16), device)
    return buf.tensor(dtype, numel), buf


_pool_allocator = None


def mem_pool():
    """A ``torch.cuda.MemPool`` whose blocks come from the daemon, for code that cannot
    allocate its communication buffers explicitly:

        with torch.cuda.use_mem_pool(mccs_b200.process_group.mem_pool()):
            grads = torch.empty(n, device="cuda")     # usable in place by collectives
    """
    global _pool_allocator
    if _pool_allocator is None:
        path = os.path.join(_lib.NATIVE_DIR, "libmccs.so")
        _pool_allocator = torch.cuda.memory.CUDAPluggableAllocator(path, "mccs_torch_malloc", "mccs_torch_free")
    return torch.cuda.MemPool(_pool_allocator.allocator())


_groups: "weakref.WeakSet[ProcessGroupMCCS]" = weakref.WeakSet()


def shutdown() -> None:
    """Shuts down every process group of this backend that is still alive in this process
    (``dist.destroy_process_group()`` drops the group object without telling a backend written
    in Python): call it before the process ends, while its CUDA context is still there."""
    for g in list(_groups):
        g.shutdown()


class ProcessGroupMCCS(dist.ProcessGroup):
    """One rank of a process group whose collectives run in the mccs daemon."""

    def __init__(self, store, rank: int, size: int, timeout=None, device: Optional[int] = None,
                 comm_id: Optional[int] = None):
        super().__init__(rank, size)
        self._rank, self._size = rank, size
        client.init(os.environ.get("MCCS_CONTROL") or None)
        self._cuda = client.backend() == "cuda"
        if device is None:
            device = torch.cuda.current_device() if self._cuda else rank % max(client.device_count(), 1)
        self._device = int(device)
        # All ranks must name the same communicator: rank 0 picks the id, the store carries it.
        if comm_id is None:
            if rank == 0:
                comm_id = int.from_bytes(os.urandom(4), "little") & 0x7FFFFFFF
                store.set("mccs_comm_id", str(comm_id))
            else:
                comm_id = int(store.get("mccs_comm_id").decode())
        self.comm_id = comm_id
        self._comm = Communicator(comm_id, rank, size, device=self._device)
        self._lock = threading.Lock()
        self._closed = False
        _groups.add(self)

    # -- helpers: the functional collectives of mccs_b200.ops do the work, in place for tensors
    # in service memory, through the communicator's staging arena otherwise -------------------
    def _sync(self) -> None:
        if self._cuda:
            torch.cuda.current_stream(self._device).synchronize()

    def _all_reduce_flat(self, t: torch.Tensor, op: str) -> None:
        """t: contiguous tensor, reduced in place."""
        _ops_all_reduce(self._comm, t, op=op)

    def _all_gather_flat(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        """out: contiguous, size * inp.numel() elements of the same dtype."""
        _ops_all_gather(self._comm, inp, out)

    # -- c10d interface --------------------------------------------------------------
    def getBackendName(self) -> str:
        return "mccs"

    def size(self) -> int:
        return self._size

    def rank(self) -> int:
        return self._rank

    def allreduce(self, tensors, opts=AllreduceOptions()):
        tensors = tensors if isinstance(tensors, (list, tuple)) else [tensors]
        op = _op_name(opts.reduceOp)
        for t in tensors:
            if t.is_contiguous():
                self._all_reduce_flat(t, op)
            else:
                c = t.contiguous()
                self._all_reduce_flat(c, op)
                t.copy_(c)
        return _done(list(tensors))

    def allreduce_coalesced(self, tensors, opts=AllreduceOptions()):
        return self.allreduce(tensors, opts)

    def broadcast(self, tensors, opts=BroadcastOptions()):
        tensors = tensors if isinstance(tensors, (list, tuple)) else [tensors]
        root = opts.rootRank
        for t in tensors:
            if t.numel() == 0:
                continue
            # The service has AllReduce and AllGather (as the reference). A broadcast is the
            # integer sum of the root's bytes and zeros: exact for every dtype, in place, and
            # 2(n-1)/n of the message per GPU instead of the n-fold traffic of a gather.
            flat = t.contiguous()
            raw = flat.view(torch.uint8).reshape(-1) if flat.dtype != torch.uint8 else flat.reshape(-1)
            words = raw.view(torch.int32) if raw.numel() % 4 == 0 and raw.data_ptr() % 4 == 0 else raw
            if self._rank != root:
                words.zero_()
            self._all_reduce_flat(words, "sum")
            if flat.data_ptr() != t.data_ptr():
                t.copy_(flat)
        return _done(list(tensors))

    def allgather(self, output_tensors, input_tensors, opts=AllgatherOptions()):
        for outs, inp in zip(output_tensors, input_tensors):
            flat = torch.empty((self._size,) + tuple(inp.shape), dtype=inp.dtype, device=inp.device)
            self._all_gather_flat(flat, inp)
            for r, o in enumerate(outs):
                o.copy_(flat[r])
        return _done(output_tensors)

    def _allgather_base(self, output_tensor, input_tensor, opts=AllgatherOptions()):
        if output_tensor.is_contiguous():
            self._all_gather_flat(output_tensor, input_tensor)
        else:
            tmp = torch.empty(output_tensor.shape, dtype=output_tensor.dtype, device=output_tensor.device)
            self._all_gather_flat(tmp, input_tensor)
            output_tensor.copy_(tmp)
        return _done(output_tensor)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=AllgatherOptions()):
        for o, i in zip(outputs, inputs):
            self._allgather_base(o, i, opts)
        return _done(outputs)

    def _reduce_scatter_flat(self, out: torch.Tensor, full: torch.Tensor, op: str) -> None:
        """full: contiguous, size blocks of out.numel() elements; out receives this rank's block."""
        _ops_reduce_scatter(self._comm, full, out, op=op)

    def reduce_scatter(self, output_tensors, input_tensors, opts=ReduceScatterOptions()):
        op = _op_name(opts.reduceOp)
        for out, ins in zip(output_tensors, input_tensors):
            full = torch.stack([i.contiguous() for i in ins])
            self._reduce_scatter_flat(out, full, op)
        return _done(output_tensors)

    def _reduce_scatter_base(self, output_tensor, input_tensor, opts=ReduceScatterOptions()):
        self._reduce_scatter_flat(output_tensor, input_tensor.contiguous(), _op_name(opts.reduceOp))
        return _done(output_tensor)

    # The rooted and the personalised collectives are composed from the service's three (the
    # reference has AllReduce and AllGather only): every rank moves what the un-rooted
    # collective moves, which is n times what a native gather / scatter / all-to-all would.
    # They are here so that code written against torch.distributed runs; the hot paths of
    # data-parallel training do not use them.
    def reduce(self, tensors, opts=ReduceOptions()):
        tensors = tensors if isinstance(tensors, (list, tuple)) else [tensors]
        op = _op_name(opts.reduceOp)
        for t in tensors:
            if self._rank == opts.rootRank:
                self.allreduce([t], _allreduce_options(opts.reduceOp))
            else:
                self._all_reduce_flat(t.contiguous().clone(), op)     # takes part; its own tensor stays as it is
        return _done(list(tensors))

    def gather(self, output_tensors, input_tensors, opts=GatherOptions()):
        for i, inp in enumerate(input_tensors):
            flat = torch.empty((self._size,) + tuple(inp.shape), dtype=inp.dtype, device=inp.device)
            self._all_gather_flat(flat, inp.contiguous())
            if self._rank == opts.rootRank:
                for r, o in enumerate(output_tensors[i]):
                    o.copy_(flat[r])
        return _done(output_tensors)

    def scatter(self, output_tensors, input_tensors, opts=ScatterOptions()):
        for i, out in enumerate(output_tensors):
            if self._rank == opts.rootRank:
                full = torch.stack([t.contiguous() for t in input_tensors[i]])
            else:
                full = torch.empty((self._size,) + tuple(out.shape), dtype=out.dtype, device=out.device)
            b = BroadcastOptions()
            b.rootRank = opts.rootRank
            self.broadcast([full], b)
            out.copy_(full[self._rank])
        return _done(output_tensors)

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=AllToAllOptions()):
        if output_split_sizes or input_split_sizes:
            raise NotImplementedError("all_to_all_single with unequal splits is not supported by the mccs backend")
        n = self._size
        if input.numel() % n or output.numel() != input.numel():
            raise ValueError("all_to_all_single needs equal splits: numel divisible by the group size, output as large as input")
        k = input.numel() // n
        everything = torch.empty((n, n, k), dtype=input.dtype, device=input.device)      # [source rank][destination][k]
        self._all_gather_flat(everything, input.contiguous())
        res = everything[:, self._rank, :].reshape(output.shape)
        output.copy_(res)
        return _done(output)

    def alltoall(self, output_tensors, input_tensors, opts=AllToAllOptions()):
        shapes = {tuple(t.shape) for t in list(output_tensors) + list(input_tensors)}
        if len(shapes) != 1:
            raise NotImplementedError("all_to_all with tensors of different shapes is not supported by the mccs backend")
        inp = torch.stack([t.contiguous() for t in input_tensors]).reshape(-1)
        out = torch.empty_like(inp)
        self.alltoall_base(out, inp, [], [], opts)
        for r, o in enumerate(output_tensors):
            o.copy_(out.reshape((self._size,) + tuple(o.shape))[r])
        return _done(output_tensors)

    def barrier(self, opts=BarrierOptions()):
        dev = f"cuda:{self._device}" if self._cuda else "cpu"
        t = torch.zeros(4, dtype=torch.float32, device=dev)
        self._all_reduce_flat(t, "sum")
        self._sync()
        return _done(None)

    # -- extras ---------------------------------------------------------------------------
    @property
    def communicator(self) -> Communicator:
        return self._comm

    def shutdown(self) -> None:
        """Waits for this rank's collectives, then gives the staging memory and the
        communicator back to the service. Safe to call more than once."""
        if self._closed:
            return
        self._closed = True
        self._sync()
        _arena(self._comm).release()
        self._comm.destroy()

    def __repr__(self) -> str:
        return f"ProcessGroupMCCS(rank={self._rank}, size={self._size}, comm_id={self.comm_id})"


def _create(store, rank, size, timeout):
    return ProcessGroupMCCS(store, rank, size, timeout)


dist.Backend.register_backend("mccs", _create, devices=["cpu", "cuda"])

__all__ = ["ProcessGroupMCCS", "empty", "mem_pool", "in_service_memory", "shutdown"]
