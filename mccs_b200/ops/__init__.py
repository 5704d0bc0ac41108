"""Collective operations on tensors, functional form.

``all_reduce`` / ``all_gather`` / ``reduce_scatter`` are the stream-ordered collectives of a
:class:`mccs_b200.Communicator` (the reference's ``libmccs::all_reduce`` /
``all_gather``, src/libmccs/src/collectives.rs:15-138) written as plain functions, with
the kernel variant as a keyword: what runs is one of the hand-written sm_100a kernels of
``csrc/kernels`` (``VARIANTS``), planned by the daemon and launched by the client library or
the daemon. Unlike the communicator's methods they take any tensor: one that lives in service
memory is used where it is, anything else is staged through a per-communicator arena (which is
what the ``torch.distributed`` backend builds on).

``local_all_reduce_no_alloc`` calls the kernels directly, without daemon or communicator:
the allocation-free single-GPU AllReduce of ``csrc/include/mccs_noalloc.h``.

On a machine with a GPU these functions never fall back to PyTorch code: a missing
native library is an error.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Sequence

import torch

from .. import _lib
from ..client import ALGOS, DTYPES, Buffer, Communicator, backend

VARIANTS = {
    "auto": "the planner's choice from the measured size -> (variant, CTAs) table",
    "ar_oneshot": "AllReduce: every rank loads all peers' data over NVLink, reduces in fp32, stores locally (small messages, out of place)",
    "ar_twoshot": "AllReduce: rank r reduces shard r from all peers (loads) and stores it into every rank's output",
    "ar_nvls_oneshot": "AllReduce: multimem.ld_reduce of the whole buffer on every rank (sum in the NVSwitch)",
    "ar_nvls_twoshot": "AllReduce: multimem.ld_reduce of the own shard + multimem.st broadcast",
    "ar_hybrid": "AllReduce: head of the buffer through the switch, the rest by peer loads/stores, in one kernel",
    "ar_ring": "AllReduce: FIFO-staged ring with a configurable order per channel (also the host-staged transport)",
    "ag_pull": "AllGather: every rank loads its peers' shards",
    "ag_push": "AllGather: every rank stores its shard into every peer",
    "ag_nvls": "AllGather: multimem.st of the own shard",
    "ag_ring": "AllGather: FIFO-staged ring",
    "rs_direct": "ReduceScatter: every rank loads its block from all peers and reduces it (the reducing half of ar_twoshot)",
    "rs_nvls": "ReduceScatter: multimem.ld_reduce of the own block",
    "local_copy": "single-rank communicator: device copy",
}
assert set(VARIANTS) == set(ALGOS)


def in_service_memory(t: torch.Tensor) -> bool:
    """True when the tensor's storage was handed out by the daemon (``Buffer``, the memory
    pool, the ``LD_PRELOAD`` hook): the kernels can then read and write it where it is."""
    if t.numel() == 0:
        return False
    mem_id, off, size = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
    return _lib.shim().mccsMemInfo(ctypes.c_void_p(t.data_ptr()), ctypes.byref(mem_id), ctypes.byref(off), ctypes.byref(size)) == 0


def usable_in_place(t: torch.Tensor) -> bool:
    return t.is_contiguous() and t.dtype in DTYPES and in_service_memory(t)


class _Arena:
    """Staging memory of one communicator for tensors that do not live in service memory:
    one service buffer that grows on demand, used under a lock (one staged collective of a
    communicator at a time; the copies in and out are stream ordered like the collective)."""

    def __init__(self, comm: Communicator):
        self.comm = comm
        self.buffer: Optional[Buffer] = None
        self.lock = threading.Lock()

    def get(self, nbytes: int) -> Buffer:
        if self.buffer is None or self.buffer.nbytes < nbytes:
            if self.buffer is not None:
                if backend() == "cuda":
                    torch.cuda.synchronize(self.comm.device)    # work that still uses the old buffer, on whichever stream
                self.buffer.free()
            self.buffer = Buffer(max(nbytes, 1 << 20) * 2, self.comm.device)
        return self.buffer

    def release(self) -> None:
        if self.buffer is not None:
            self.buffer.free()
            self.buffer = None


def arena(comm: Communicator) -> _Arena:
    a = getattr(comm, "_ops_arena", None)
    if a is None:
        a = _Arena(comm)
        comm._ops_arena = a
    return a


def all_reduce(comm: Communicator, send: torch.Tensor, recv: Optional[torch.Tensor] = None, *, op: str = "sum",
               scale: float = 1.0, algo: str = "auto", stream=None) -> torch.Tensor:
    """AllReduce of ``send`` into ``recv`` (in place when ``recv`` is None) over ``comm``.
    Tensors in service memory (:class:`mccs_b200.Buffer`) are used where they are; any other
    tensor (ordinary CUDA memory, unsupported element type such as bool, non-contiguous) is
    staged through the communicator's arena: one copy in, the collective in place, one copy
    out, all on the caller's stream. Returns the output tensor; like a kernel launch, the call
    returns before the result exists."""
    out = send if recv is None else recv
    if send.numel() == 0:
        return out
    if usable_in_place(send) and (recv is None or usable_in_place(recv)):
        comm.all_reduce(send, recv, op=op, scale=scale, algo=algo, stream=stream)
        return out
    work = send.dtype if send.dtype in DTYPES else torch.float32
    n = send.numel()
    ar = arena(comm)
    with ar.lock:
        st = ar.get(n * torch.empty((), dtype=work).element_size()).tensor(work, n)
        st.copy_(send.reshape(-1), non_blocking=True)
        comm.all_reduce(st, op=op, scale=scale, algo=algo, stream=stream)
        # (a copy to ordinary host memory is left blocking: the caller may read it at once)
        out.copy_(st.view(out.shape) if out.dtype == work else st.to(out.dtype).view(out.shape), non_blocking=out.is_cuda)
    return out


def all_gather(comm: Communicator, send: torch.Tensor, recv: torch.Tensor, *, algo: str = "auto", stream=None) -> torch.Tensor:
    """AllGather: rank r's ``send`` lands at ``recv[r * send.numel():]`` on every rank
    (``recv`` holds ``nranks * send.numel()`` elements of the same type). Staged like
    :func:`all_reduce` when a tensor is not in service memory."""
    nb = send.numel() * send.element_size()
    if nb == 0:
        return recv
    if usable_in_place(recv) and send.is_contiguous() and in_service_memory(send):
        comm.all_gather(send, recv, nbytes=nb, algo=algo, stream=stream)
        return recv
    n, r = comm.nranks, comm.rank
    ar = arena(comm)
    with ar.lock:
        full = ar.get(nb * n).bytes_tensor()[:nb * n]
        mine = full[r * nb:(r + 1) * nb]
        mine.copy_(send.contiguous().view(torch.uint8).reshape(-1), non_blocking=True)
        comm.all_gather(mine, full, nbytes=nb, algo=algo, stream=stream)      # in place inside the staging buffer
        if recv.is_contiguous():
            recv.view(torch.uint8).reshape(-1).copy_(full, non_blocking=recv.is_cuda)
        else:
            recv.copy_(full.view(recv.dtype).view(recv.shape), non_blocking=recv.is_cuda)
    return recv


def reduce_scatter(comm: Communicator, send: torch.Tensor, recv: torch.Tensor, *, op: str = "sum", scale: float = 1.0,
                   algo: str = "auto", stream=None) -> torch.Tensor:
    """ReduceScatter: ``send`` holds ``nranks`` blocks of ``recv.numel()`` elements; ``recv``
    receives the reduction of this rank's block (in place when it is that block of ``send``).
    Staged like :func:`all_reduce` when a tensor is not in service memory."""
    if recv.numel() == 0:
        return recv
    if usable_in_place(send) and usable_in_place(recv):
        comm.reduce_scatter(send, recv, op=op, scale=scale, algo=algo, stream=stream)
        return recv
    work = send.dtype if send.dtype in DTYPES else torch.float32
    n, blk = comm.nranks, recv.numel()
    esz = torch.empty((), dtype=work).element_size()
    ar = arena(comm)
    with ar.lock:
        st = ar.get(n * blk * esz).tensor(work, n * blk)
        st.copy_(send.reshape(-1), non_blocking=True)
        mine = st[comm.rank * blk:(comm.rank + 1) * blk]
        comm.reduce_scatter(st, mine, op=op, scale=scale, algo=algo, stream=stream)     # in place in the staging buffer
        recv.copy_(mine.view(recv.shape) if recv.dtype == work else mine.to(recv.dtype).view(recv.shape), non_blocking=recv.is_cuda)
    return recv


def local_all_reduce_no_alloc(inputs: Sequence[torch.Tensor], outputs: Optional[Sequence[torch.Tensor]] = None,
                              stream=None) -> Sequence[torch.Tensor]:
    """Sum of up to 8 equally shaped f32 / f16 / bf16 tensors on the CURRENT CUDA device,
    written to every output (in place when ``outputs`` is None), by the two-shot kernel in
    one cooperative launch. Allocates nothing, neither here nor in the native code: usable
    while a memory pool is frozen. Overlapping calls on one device race (they share one
    scratch array); make the first call on a device outside stream capture."""
    if not inputs:
        raise ValueError("no tensors")
    outs = list(inputs) if outputs is None else list(outputs)
    first = inputs[0]
    if len(outs) != len(inputs) or len(inputs) > 8:
        raise ValueError("need as many outputs as inputs, at most 8")
    for t in list(inputs) + outs:
        if not t.is_cuda or t.device != first.device or t.dtype != first.dtype or t.numel() != first.numel() or not t.is_contiguous():
            raise ValueError("tensors must be contiguous CUDA tensors of one device, dtype and size")
    if first.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("float32, float16 or bfloat16 only")
    lib = _lib.daemon_lib()          # raises when the native library is missing: no silent fallback
    fn = lib.mccsLocalAllReduceNoAlloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_size_t,
                   ctypes.c_int, ctypes.c_void_p]
    n = len(inputs)
    ins = (ctypes.c_void_p * n)(*[t.data_ptr() for t in inputs])
    ous = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
    s = torch.cuda.current_stream(first.device) if stream is None else stream
    with torch.cuda.device(first.device):
        rc = fn(ins, ous, n, first.numel(), DTYPES[first.dtype], ctypes.c_void_p(s.cuda_stream))
    if rc != 0:
        raise RuntimeError(f"mccsLocalAllReduceNoAlloc failed with CUDA error {rc}")
    return outs


__all__ = ["VARIANTS", "all_reduce", "all_gather", "reduce_scatter", "in_service_memory", "usable_in_place", "arena",
           "local_all_reduce_no_alloc"]
