"""Python client of the service: buffers, communicators, collectives.

Thin object layer over the C API (``csrc/include/mccs.h``). It follows the
reference's client calls one to one — ``cuda_malloc`` / ``init_communicator_rank``
/ ``register_stream`` / ``all_gather`` / ``all_reduce``
(``src/libmccs/src/lib.rs:23-27``) — and adds what a PyTorch user needs: buffers
that are torch tensors, dtype mapping, an admin client.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import byref, c_uint32, c_uint64, c_void_p
from typing import Optional, Sequence, Union

import torch

from . import _lib
from ._lib import check

# mccsDataType_t
DTYPES = {
    torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4,
    torch.float16: 6, torch.float32: 7, torch.float64: 8, torch.bfloat16: 9,
}
if hasattr(torch, "uint32"):
    DTYPES[torch.uint32] = 3
if hasattr(torch, "uint64"):
    DTYPES[torch.uint64] = 5

OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "premulsum": 4, "avg": 5, "sumpostdiv": 5}

ALGOS = {
    "auto": 0, "ar_oneshot": 1, "ar_twoshot": 2, "ar_nvls_oneshot": 3, "ar_nvls_twoshot": 4,
    "ar_ring": 5, "ag_pull": 6, "ag_push": 7, "ag_nvls": 8, "ag_ring": 9, "local_copy": 10, "ar_hybrid": 11,
    "rs_direct": 12, "rs_nvls": 13,
}
ALGO_NAMES = {v: k for k, v in ALGOS.items()}


def init(control_path: Optional[str] = None) -> None:
    """Connect to the daemon (otherwise done lazily with MCCS_CONTROL / MCCS_PREFIX)."""
    check(_lib.shim().mccsInit(control_path.encode() if control_path else None), "mccsInit")


def finalize() -> None:
    _lib.shim().mccsFinalize()


def backend() -> str:
    """'cuda' or 'host' (a daemon without GPUs serving host shared memory)."""
    k = _lib.shim().mccsBackendKind()
    if k < 0:
        raise RuntimeError("not connected to an mccs daemon")
    return "cuda" if k == 1 else "host"


def device_count() -> int:
    return int(_lib.shim().mccsDeviceCount())


class _CudaArrayView:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


class Buffer:
    """Device memory allocated by the daemon and mapped into this process."""

    def __init__(self, nbytes: int, device: int = 0):
        p = c_void_p()
        check(_lib.shim().mccsMalloc(byref(p), int(device), int(nbytes)), "mccsMalloc")
        self.ptr = int(p.value)
        self.nbytes = int(nbytes)
        self.device = int(device)
        self._freed = False
        self._is_cuda = backend() == "cuda"
        self._bytes: Optional[torch.Tensor] = None

    def bytes_tensor(self) -> torch.Tensor:
        """The whole buffer as a uint8 tensor aliasing the daemon-owned memory."""
        if self._bytes is None:
            if self._is_cuda:
                self._bytes = torch.as_tensor(_CudaArrayView(self.ptr, self.nbytes), device=f"cuda:{self.device}")
            else:
                raw = (ctypes.c_uint8 * self.nbytes).from_address(self.ptr)
                self._bytes = torch.frombuffer(raw, dtype=torch.uint8)
        return self._bytes

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        if numel is None:
            numel = (self.nbytes - offset_bytes) // esz
        b = self.bytes_tensor()[offset_bytes:offset_bytes + numel * esz]
        return b.view(dtype)

    def mem_info(self):
        mem_id, off, size = c_uint64(), c_uint64(), c_uint64()
        check(_lib.shim().mccsMemInfo(c_void_p(self.ptr), byref(mem_id), byref(off), byref(size)), "mccsMemInfo")
        return mem_id.value, off.value, size.value

    def free(self) -> None:
        if not self._freed:
            self._freed = True
            self._bytes = None
            _lib.shim().mccsFree(c_void_p(self.ptr))

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _ptr(x: Union[torch.Tensor, Buffer, int]) -> int:
    if isinstance(x, torch.Tensor):
        return x.data_ptr()
    if isinstance(x, Buffer):
        return x.ptr
    return int(x)


def _stream_handle(stream) -> Optional[int]:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


def _refuse_capture() -> None:
    """A collective takes its barrier epoch and its ticket from the daemon at the call: a CUDA
    graph that captured one would replay stale values. Refused here, loudly, instead of giving
    wrong results at replay."""
    try:
        capturing = torch.cuda.is_current_stream_capturing()
    except Exception:      # no usable CUDA runtime in this process: nothing can be capturing
        capturing = False
    if capturing:
        raise _lib.MccsError(-9, "a collective inside CUDA graph capture")


class Communicator:
    """One rank of a communicator (``init_communicator_rank`` in the reference)."""

    def __init__(self, unique_id: int, rank: int, nranks: int, device: int = 0, root_addr: str = "127.0.0.1"):
        h = c_void_p()
        check(_lib.shim().mccsCommInitRank(byref(h), int(unique_id), int(rank), int(nranks), int(device),
                                           root_addr.encode()), "mccsCommInitRank")
        self._h = h
        self.unique_id, self.rank, self.nranks, self.device = int(unique_id), int(rank), int(nranks), int(device)
        self._is_cuda = backend() == "cuda"

    @property
    def handle(self) -> int:
        return int(_lib.shim().mccsCommHandle(self._h))

    def _stream(self, stream) -> Optional[int]:
        if self._is_cuda:
            _refuse_capture()
        if stream is not None:
            return _stream_handle(stream)
        if self._is_cuda:
            return int(torch.cuda.current_stream(self.device).cuda_stream)
        return None

    def all_reduce(self, send, recv=None, *, count: Optional[int] = None, dtype: Optional[torch.dtype] = None,
                   op: str = "sum", scale: float = 1.0, algo: str = "auto", stream=None) -> None:
        """AllReduce ``count`` elements; in place when ``recv`` is None."""
        if recv is None:
            recv = send
        if isinstance(send, torch.Tensor):
            dtype = dtype or send.dtype
            count = send.numel() if count is None else count
        if dtype is None or count is None:
            raise ValueError("dtype and count are needed for raw pointers")
        check(_lib.shim().mccsAllReduceEx(self._h, c_void_p(_ptr(send)), c_void_p(_ptr(recv)), int(count),
                                          DTYPES[dtype], OPS[op.lower()], float(scale), ALGOS[algo],
                                          c_void_p(self._stream(stream))), "mccsAllReduce")

    def all_gather(self, send, recv, *, nbytes: Optional[int] = None, algo: str = "auto", stream=None) -> None:
        """AllGather ``nbytes`` per rank into ``recv`` (``nranks * nbytes`` bytes)."""
        if nbytes is None:
            if not isinstance(send, torch.Tensor):
                raise ValueError("nbytes is needed for raw pointers")
            nbytes = send.numel() * send.element_size()
        check(_lib.shim().mccsAllGatherEx(self._h, c_void_p(_ptr(send)), c_void_p(_ptr(recv)), int(nbytes),
                                          ALGOS[algo], c_void_p(self._stream(stream))), "mccsAllGather")

    def reduce_scatter(self, send, recv, *, count: Optional[int] = None, dtype: Optional[torch.dtype] = None,
                       op: str = "sum", scale: float = 1.0, algo: str = "auto", stream=None) -> None:
        """ReduceScatter: ``send`` holds ``nranks * count`` elements, ``recv`` receives the
        reduction of block ``rank`` (``count`` elements). In place when ``recv`` is the
        rank's own block of ``send``. The reference has no such call."""
        if isinstance(recv, torch.Tensor):
            dtype = dtype or recv.dtype
            count = recv.numel() if count is None else count
        if dtype is None or count is None:
            raise ValueError("dtype and count are needed for raw pointers")
        check(_lib.shim().mccsReduceScatterEx(self._h, c_void_p(_ptr(send)), c_void_p(_ptr(recv)), int(count),
                                              DTYPES[dtype], OPS[op.lower()], float(scale), ALGOS[algo],
                                              c_void_p(self._stream(stream))), "mccsReduceScatter")

    def set_deferred_wait(self, on: bool) -> None:
        """With deferred waiting a collective call does not make the caller's stream wait
        for it; :meth:`wait` places that wait where the results are needed."""
        check(_lib.shim().mccsCommSetDeferredWait(self._h, 1 if on else 0), "mccsCommSetDeferredWait")

    def wait(self, stream=None) -> None:
        """Make ``stream`` (default: the current stream) wait for every collective
        submitted on this communicator so far."""
        check(_lib.shim().mccsCommWait(self._h, c_void_p(self._stream(stream))), "mccsCommWait")

    def flush(self) -> None:
        """Wait until the daemon has launched everything posted so far; raise the first
        error a request reported (collective calls may return before the daemon has
        even seen them)."""
        check(_lib.shim().mccsCommFlush(self._h), "mccsCommFlush")

    def query(self) -> dict:
        _lib.shim().mccsCommFlush(self._h)
        info = _lib.CommInfo()
        check(_lib.shim().mccsCommQuery(self._h, byref(info)), "mccsCommQuery")
        return {f: getattr(info, f) for f, _ in info._fields_}

    def last_plan(self):
        v, c = c_uint32(), c_uint32()
        _lib.shim().mccsCommLastPlan(self._h, byref(v), byref(c))
        return ALGO_NAMES.get(v.value, str(v.value)), int(c.value)

    @property
    def launch_mode(self) -> str:
        """'daemon' (the service launches the kernels) or 'client' (this process does, on the
        caller's stream, from the plan the service made)."""
        return "client" if _lib.shim().mccsCommLaunchMode(self._h) == 1 else "daemon"

    def destroy(self) -> None:
        if self._h is not None and self._h.value:
            _lib.shim().mccsCommDestroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class group:
    """``with group():`` submits the enclosed collectives back to back (GroupCall)."""

    def __enter__(self):
        check(_lib.shim().mccsGroupStart(), "mccsGroupStart")
        return self

    def __exit__(self, *exc):
        rc = _lib.shim().mccsGroupEnd()
        if exc[0] is None:
            check(rc, "mccsGroupEnd")


def admin_request(port: int, body: dict, *, host: str = "127.0.0.1", type_: int = 2) -> dict:
    """One request to a daemon's admin port (reconfiguration: ``type_=1``)."""
    buf = ctypes.create_string_buffer(1 << 22)
    check(_lib.shim().mccsAdminRequest(host.encode(), int(port), int(type_), json.dumps(body).encode(), buf,
                                       len(buf)), "mccsAdminRequest")
    return json.loads(buf.value.decode())


def reconfigure(port: int, patterns: Sequence[dict], *, host: str = "127.0.0.1") -> dict:
    """Live reconfiguration: ring order per channel, algorithm, CTA count.

    ``patterns`` uses the reference's shape
    ``{"communicator_id": id, "channels": [{"channel_id": 0, "ring": [...]}, ...]}``
    (``eval/dynamic-config/reconfig-patch.toml``) plus optional ``allreduce_algo``,
    ``allgather_algo`` and ``ctas``.
    """
    return admin_request(port, {"comm_patterns_reconfig": list(patterns)}, host=host, type_=1)
