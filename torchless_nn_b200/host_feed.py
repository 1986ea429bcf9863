"""Double-buffered host feed (pinned host buffers, a copy stream) for batch loops.

The reference uploads every batch synchronously (``xp.array(batch)``, network.py:117,152).  ``HostFeed`` overlaps
the upload of batch i+1 with the compute of batch i: ``batches(data, batch_size)`` yields device arrays that alias
the feeder's two device buffers, each valid until the next one is requested."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import backend
from ._lib import lib, check
from .device_array import DeviceArray


class HostFeed:
    def __init__(self, bytes_per_batch: int):
        self.bytes = int(bytes_per_batch)
        self._version = 0           # device arrays yielded by batches() use the feeder as their root (see DeviceArray.version)
        self.handle = C.c_void_p()
        check(lib.tlnn_feed_create(backend.ctx(), self.bytes, C.byref(self.handle)))
        self._host = []
        for slot in (0, 1):
            p = C.c_void_p()
            check(lib.tlnn_feed_host(self.handle, slot, C.byref(p)))
            self._host.append(np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(self.bytes,)))

    def close(self):
        if self.handle:
            lib.tlnn_feed_destroy(self.handle)
            self.handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _submit(self, slot: int, batch: np.ndarray):
        check(lib.tlnn_feed_host_wait(self.handle, slot))          # the slot's previous copy has left the host buffer
        raw = np.ascontiguousarray(batch).view(np.uint8).reshape(-1)
        if raw.size > self.bytes:
            raise ValueError(f"batch of {raw.size} bytes for a feeder of {self.bytes}")
        self._host[slot][:raw.size] = raw
        check(lib.tlnn_feed_submit(self.handle, slot, raw.size))

    def batches(self, data, batch_size: int, dtype):
        """Yield (start, stop, device array) for consecutive slices of ``data``; the next slice is already on its way
        to the device while the caller works on the current one."""
        n = len(data)
        starts = list(range(0, n, batch_size))
        if not starts:
            return
        dtype = np.dtype(dtype)

        def cut(i):
            return np.asarray(data[i:min(i + batch_size, n)], dtype=dtype)
        cur = cut(starts[0])
        self._submit(0, cur)
        for k, i in enumerate(starts):
            slot = k & 1
            nxt = None
            if k + 1 < len(starts):
                nxt = cut(starts[k + 1])
                self._submit(slot ^ 1, nxt)
            dev = C.c_void_p()
            check(lib.tlnn_feed_acquire(self.handle, slot, C.byref(dev)))
            yield i, min(i + batch_size, n), DeviceArray(cur.shape, dtype, ptr=dev.value, root=self)
            check(lib.tlnn_feed_release(self.handle, slot))
            cur = nxt
