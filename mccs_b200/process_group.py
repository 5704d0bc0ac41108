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
enqueued and the caller's current stream waits for it, so the returned ``Work`` is
already complete in the sense PyTorch's stream semantics need.
"""
from __future__ import annotations

import os
import threading
from ctypes import byref, c_uint64, c_void_p
from typing import List, Optional

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import (AllgatherOptions, AllreduceOptions, BarrierOptions, BroadcastOptions,
                                        ReduceOp, ReduceScatterOptions, _create_work_from_future)
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


def _done(result) -> "dist.Work":
    fut: Future = Future()
    fut.set_result(result)
    return _create_work_from_future(fut)


def in_service_memory(t: torch.Tensor) -> bool:
    """True when the tensor's storage was allocated by the daemon."""
    if t.numel() == 0:
        return False
    mem_id, off, size = c_uint64(), c_uint64(), c_uint64()
    return _lib.shim().mccsMemInfo(c_void_p(t.data_ptr()), byref(mem_id), byref(off), byref(size)) == 0


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
        self._staging: Optional[Buffer] = None
        self._lock = threading.Lock()

    # -- helpers -------------------------------------------------------------------
    def _stage(self, nbytes: int) -> Buffer:
        if self._staging is None or self._staging.nbytes < nbytes:
            if self._staging is not None:
                self._sync()
                self._staging.free()
            self._staging = Buffer(max(nbytes, 1 << 20) * 2, self._device)
        return self._staging

    def _sync(self) -> None:
        if self._cuda:
            torch.cuda.current_stream(self._device).synchronize()

    def _usable_in_place(self, t: torch.Tensor) -> bool:
        return t.is_contiguous() and in_service_memory(t) and t.dtype in client.DTYPES

    def _all_reduce_flat(self, t: torch.Tensor, op: str) -> None:
        """t: contiguous tensor; reduced in place (through staging when needed)."""
        if t.numel() == 0:
            return
        if self._usable_in_place(t):
            self._comm.all_reduce(t, op=op)
            return
        dtype = t.dtype
        work_dtype = dtype if dtype in client.DTYPES else torch.float32
        nbytes = t.numel() * torch.empty((), dtype=work_dtype).element_size()
        with self._lock:
            st = self._stage(nbytes).tensor(work_dtype, t.numel())
            st.copy_(t.reshape(-1), non_blocking=True)
            self._comm.all_reduce(st, op=op)
            t.reshape(-1).copy_(st, non_blocking=True)

    def _all_gather_flat(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        """out: contiguous, size * inp.numel() elements of the same dtype."""
        nb = inp.numel() * inp.element_size()
        if nb == 0:
            return
        if self._usable_in_place(out) and inp.is_contiguous() and in_service_memory(inp):
            self._comm.all_gather(inp, out, nbytes=nb)
            return
        with self._lock:
            stage = self._stage(nb * self._size)
            full = stage.bytes_tensor()[:nb * self._size]
            mine = full[self._rank * nb:(self._rank + 1) * nb]
            mine.copy_(inp.contiguous().view(torch.uint8).reshape(-1), non_blocking=True)
            self._comm.all_gather(mine, full, nbytes=nb)      # in place inside the staging buffer
            out.view(torch.uint8).reshape(-1).copy_(full, non_blocking=True)

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
        """full: contiguous, size * out.numel() elements; out receives the reduction of this
        rank's block. Through the service's own reduce-scatter (half the traffic of the
        all-reduce this used to be); tensors outside service memory are staged."""
        n = out.numel()
        if n == 0:
            return
        if self._usable_in_place(full) and self._usable_in_place(out) and out.dtype == full.dtype:
            self._comm.reduce_scatter(full, out, op=op)
            return
        dtype = full.dtype
        work_dtype = dtype if dtype in client.DTYPES else torch.float32
        esz = torch.empty((), dtype=work_dtype).element_size()
        with self._lock:
            st = self._stage(n * self._size * esz).tensor(work_dtype, n * self._size)
            st.copy_(full.reshape(-1), non_blocking=True)
            mine = st[self._rank * n:(self._rank + 1) * n]
            self._comm.reduce_scatter(st, mine, op=op)           # in place inside the staging buffer
            out.reshape(-1).copy_(mine, non_blocking=True) if out.is_contiguous() else out.copy_(mine.reshape(out.shape))

    def reduce_scatter(self, output_tensors, input_tensors, opts=ReduceScatterOptions()):
        op = _op_name(opts.reduceOp)
        for out, ins in zip(output_tensors, input_tensors):
            full = torch.stack([i.contiguous() for i in ins])
            self._reduce_scatter_flat(out, full, op)
        return _done(output_tensors)

    def _reduce_scatter_base(self, output_tensor, input_tensor, opts=ReduceScatterOptions()):
        self._reduce_scatter_flat(output_tensor, input_tensor.contiguous(), _op_name(opts.reduceOp))
        return _done(output_tensor)

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
        self._sync()
        if self._staging is not None:
            self._staging.free()
            self._staging = None
        self._comm.destroy()

    def __repr__(self) -> str:
        return f"ProcessGroupMCCS(rank={self._rank}, size={self._size}, comm_id={self.comm_id})"


def _create(store, rank, size, timeout):
    return ProcessGroupMCCS(store, rank, size, timeout)


dist.Backend.register_backend("mccs", _create, devices=["cpu", "cuda"])

__all__ = ["ProcessGroupMCCS", "empty", "mem_pool", "in_service_memory"]
