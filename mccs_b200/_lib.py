"""ctypes bindings of the two native libraries.

``libmccs.so`` is the client shim every application loads (C API in
``csrc/include/mccs.h``; it mirrors the reference's Rust crate
``src/libmccs/src/lib.rs:23-27``). ``libmccs_daemon.so`` holds the service itself
(daemon + sm_100a kernels) and is only loaded by a process that hosts the daemon
in-process instead of talking to a separate ``mccsd``.

Both live in ``mccs_b200/_native`` and are built by ``make`` at the repository root
(``__graft_entry__.build()`` runs it). Nothing here falls back to a Python
implementation: a missing library is an ImportError naming the build command.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, byref, c_char_p, c_float, c_int, c_int32, c_size_t,
                    c_uint32, c_uint64, c_void_p)

NATIVE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_native")


def _load(name: str) -> ctypes.CDLL:
    path = os.path.join(NATIVE_DIR, name)
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build the native code with `make -j` at the repository root "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`)")
    # RTLD_LOCAL: nothing else in the process should resolve symbols against these libraries
    return ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)


class CommInfo(Structure):
    _fields_ = [("async_error", c_int32), ("device_error", c_uint32), ("launched", c_uint64),
                ("completed", c_uint64), ("last_variant", c_uint32), ("last_ctas", c_uint32),
                ("config_epoch", c_uint64)]


_shim = None
_daemon = None


def shim() -> ctypes.CDLL:
    global _shim
    if _shim is not None:
        return _shim
    lib = _load("libmccs.so")
    lib.mccsInit.argtypes = [c_char_p]
    lib.mccsInit.restype = c_int
    lib.mccsFinalize.restype = c_int
    lib.mccsBackendKind.restype = c_int
    lib.mccsDeviceCount.restype = c_int
    lib.mccsMalloc.argtypes = [POINTER(c_void_p), c_int, c_size_t]
    lib.mccsMalloc.restype = c_int
    lib.mccsFree.argtypes = [c_void_p]
    lib.mccsFree.restype = c_int
    lib.mccsMemInfo.argtypes = [c_void_p, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint64)]
    lib.mccsMemInfo.restype = c_int
    lib.mccsCommInitRank.argtypes = [POINTER(c_void_p), c_uint32, c_int, c_int, c_int, c_char_p]
    lib.mccsCommInitRank.restype = c_int
    lib.mccsCommDestroy.argtypes = [c_void_p]
    lib.mccsCommDestroy.restype = c_int
    lib.mccsCommHandle.argtypes = [c_void_p]
    lib.mccsCommHandle.restype = c_uint64
    lib.mccsRegisterStream.argtypes = [c_int, c_void_p]
    lib.mccsRegisterStream.restype = c_int
    lib.mccsAllReduceEx.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_float,
                                    c_int, c_void_p]
    lib.mccsAllReduceEx.restype = c_int
    lib.mccsReduceScatterEx.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_float,
                                        c_int, c_void_p]
    lib.mccsReduceScatterEx.restype = c_int
    lib.mccsAllGatherEx.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]
    lib.mccsAllGatherEx.restype = c_int
    lib.mccsGroupStart.restype = c_int
    lib.mccsGroupEnd.restype = c_int
    lib.mccsCommQuery.argtypes = [c_void_p, POINTER(CommInfo)]
    lib.mccsCommQuery.restype = c_int
    lib.mccsCommSetDeferredWait.argtypes = [c_void_p, c_int]
    lib.mccsCommSetDeferredWait.restype = c_int
    lib.mccsCommWait.argtypes = [c_void_p, c_void_p]
    lib.mccsCommWait.restype = c_int
    lib.mccsCommFlush.argtypes = [c_void_p]
    lib.mccsCommFlush.restype = c_int
    lib.mccsCommLastPlan.argtypes = [c_void_p, POINTER(c_uint32), POINTER(c_uint32)]
    lib.mccsCommLastPlan.restype = c_int
    lib.mccsCommLaunchMode.argtypes = [c_void_p]
    lib.mccsCommLaunchMode.restype = c_int
    lib.mccsGetErrorString.argtypes = [c_int]
    lib.mccsGetErrorString.restype = c_char_p
    lib.mccsAlgoName.argtypes = [c_int]
    lib.mccsAlgoName.restype = c_char_p
    lib.mccsAdminRequest.argtypes = [c_char_p, c_int, c_int, c_char_p, c_char_p, c_size_t]
    lib.mccsAdminRequest.restype = c_int
    _shim = lib
    return lib


def daemon_lib() -> ctypes.CDLL:
    global _daemon
    if _daemon is not None:
        return _daemon
    lib = _load("libmccs_daemon.so")
    lib.mccsd_start.argtypes = [c_char_p]
    lib.mccsd_start.restype = c_int
    lib.mccsd_start_file.argtypes = [c_char_p]
    lib.mccsd_start_file.restype = c_int
    lib.mccsd_stop.restype = None
    lib.mccsd_control_path.restype = c_char_p
    lib.mccsd_admin_port.restype = c_int
    lib.mccsd_backend_kind.restype = c_int
    lib.mccsd_describe.restype = c_char_p
    lib.mccsd_admin.argtypes = [c_int, c_char_p]
    lib.mccsd_admin.restype = c_char_p
    _daemon = lib
    return lib


class MccsError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        msg = shim().mccsGetErrorString(code).decode()
        super().__init__(f"{what}: {msg} ({code})")


def check(code: int, what: str) -> None:
    if code != 0:
        raise MccsError(code, what)


__all__ = ["shim", "daemon_lib", "check", "MccsError", "CommInfo", "NATIVE_DIR", "byref"]
