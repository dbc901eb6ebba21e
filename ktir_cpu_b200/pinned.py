"""Page-locked host arrays, so host<->device copies run at PCIe speed.

``pinned_empty`` gives callers an input/output array in pinned memory;
:class:`PinnedPool` recycles the buffers behind the fresh result arrays that
``execute_function`` returns (a buffer goes back to the pool when its array is
garbage-collected, so callers still own what they were handed).
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, List, Tuple

import numpy as np


class _Lease:
    """Owns one pinned buffer; numpy arrays built on it keep it alive through ``base``."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.buf = (C.c_char * max(nbytes, 1)).from_address(ptr)


def _wrap(lease: _Lease, shape, dtype) -> np.ndarray:
    dtype = np.dtype(dtype)
    n = int(np.prod(shape)) if len(shape) else 1
    arr = np.frombuffer(lease.buf, dtype=dtype, count=n).reshape(shape)
    return arr


def pinned_empty(dev, shape, dtype) -> np.ndarray:
    """An uninitialised array in page-locked memory, freed when the array is collected."""
    dtype = np.dtype(dtype)
    nbytes = max(int(np.prod(shape)) * dtype.itemsize, 1)
    ptr = dev.alloc_host(nbytes)
    lease = _Lease(ptr, nbytes)
    weakref.finalize(lease.buf, _free, dev, ptr)
    return _wrap(lease, tuple(shape), dtype)


def _free(dev, ptr):
    try:
        if dev.h:
            dev.free_host(ptr)
    except Exception:
        pass


class PinnedPool:
    """Recycled page-locked buffers (sizes rounded up to a power of two).  At most ``max_bytes`` are
    kept page-locked; past that ``empty`` hands out an ordinary NumPy array, which still works as a
    result array but is copied to synchronously and more slowly — raise ``max_bytes`` for calls
    whose live results exceed it."""

    def __init__(self, dev, max_bytes: int = 8 << 30):
        self.dev = dev
        self.max_bytes = max_bytes
        self.total = 0
        self.free: Dict[int, List[int]] = {}

    def _recycle(self, ptr: int, nbytes: int):
        self.free.setdefault(nbytes, []).append(ptr)

    def empty(self, shape, dtype) -> np.ndarray:
        dtype = np.dtype(dtype)
        nbytes = max(int(np.prod(shape)) * dtype.itemsize, 1)
        cap = 1 << (nbytes - 1).bit_length()
        lst = self.free.get(cap)
        if lst:
            ptr = lst.pop()
        elif self.total + cap <= self.max_bytes:
            ptr = self.dev.alloc_host(cap)
            self.total += cap
        else:
            return np.empty(shape, dtype)
        lease = _Lease(ptr, cap)
        weakref.finalize(lease.buf, self._recycle, ptr, cap)
        return _wrap(lease, tuple(shape), dtype)

    def close(self):
        for lst in self.free.values():
            for p in lst:
                _free(self.dev, p)
        self.free = {}
