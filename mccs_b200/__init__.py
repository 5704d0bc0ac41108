"""mccs_b200: a managed collective communication service for one 8xB200 NVSwitch box.

Layers (bottom up): sm_100a collective kernels and the service daemon
(``csrc/``, loaded as ``_native/libmccs_daemon.so`` or run as ``_native/mccsd``),
the client shim ``_native/libmccs.so`` (C API ``csrc/include/mccs.h``), this
package's object API (:mod:`mccs_b200.client`), a ``torch.distributed`` backend
(:mod:`mccs_b200.process_group`) and data-parallel training drivers
(:mod:`mccs_b200.parallel`, :mod:`mccs_b200.models`).
"""
from .client import (ALGOS, Buffer, Communicator, admin_request, backend, device_count, finalize, group, init,
                     reconfigure)
from ._lib import MccsError
from . import daemon

__all__ = ["ALGOS", "Buffer", "Communicator", "MccsError", "admin_request", "backend", "device_count", "finalize", "group",
           "init", "reconfigure", "daemon"]
__version__ = "0.1.0"
