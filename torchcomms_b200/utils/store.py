"""Store helpers used for bootstrap.

``create_prefix_store(prefix)`` connects to (rank 0: hosts) the TCPStore at
``MASTER_ADDR:MASTER_PORT`` and scopes it by ``prefix``; ``dup_prefix_store``
opens a second store on a port of its own, published through an existing one,
for users that must not share a server with the bootstrap traffic.

Parity: comms/torchcomms/utils/_store_manager.pyi (``_create_prefix_store``,
``_dup_prefix_store``; comms/torchcomms/utils/StoreManager.cpp:11-80).
"""
from __future__ import annotations

from datetime import timedelta
from typing import Optional

from .. import _comms

_DEFAULT = timedelta(seconds=600)


def create_prefix_store(prefix: str, timeout: Optional[timedelta] = None):
    return _comms._create_prefix_store(prefix, timeout or _DEFAULT)


def dup_prefix_store(prefix: str, bootstrap_store, timeout: Optional[timedelta] = None):
    return _comms._dup_prefix_store(prefix, bootstrap_store, timeout or _DEFAULT)


_create_prefix_store = create_prefix_store
_dup_prefix_store = dup_prefix_store
