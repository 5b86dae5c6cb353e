"""zyx_b200 — a B200 (sm_100a) compute backend for the zyx ML library's hot path.

The product is the shared library `libzyxb.so` (C ABI in include/zyxb.h) built from
zyx_b200/csrc.  `backend` mirrors zyx's MemoryPool/Device interface over that ABI and `ops`
offers host-array convenience calls; both fail loudly when the library is missing.
"""
from . import _lib
from .backend import Backend, BackendError, Device, MemoryPool  # noqa: F401

__all__ = ["Backend", "BackendError", "Device", "MemoryPool", "_lib"]
