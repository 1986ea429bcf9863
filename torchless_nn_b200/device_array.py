"""Device-resident arrays: the objects that stand where ``xp.ndarray`` stands in the reference.

A ``DeviceArray`` is an opaque handle on memory owned by libtlnn.so plus a shape and a dtype (float32 for
activations and parameters, int32 for token ids and arg-max results).  It offers what callers of the forward path
use on reference arrays: ``shape`` / ``dtype`` / ``ndim`` / ``size``, ``get()`` (demo.ipynb:1535,1707), basic
indexing for the ``predict(x)[0, -1]`` idiom (demo.ipynb:1530), in-place loading (``p[...] = a``, ``p *= 0``,
``p += a``: demo.ipynb:1725-1726), ``fill`` (utils.py:45-52), ``reshape`` views, ``a + b`` (utils.py:84-85), and
``__cuda_array_interface__`` for zero-copy interop.  Every in-place change bumps a version counter so that cached
re-laid-out copies of a weight are rebuilt.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import lib, check
from . import backend

_DTYPES = {np.dtype(np.float32): _lib.F32, np.dtype(np.int32): _lib.I32, np.dtype(np.int64): _lib.I64,
           np.dtype(np.uint8): _lib.U8}


def _shape_tuple(shape) -> tuple:
    if isinstance(shape, (int, np.integer)):
        return (int(shape),)
    return tuple(int(s) for s in shape)


class DeviceArray:
    __slots__ = ("ptr", "shape", "dtype", "_root", "_owner", "_version", "__weakref__")

    def __init__(self, shape, dtype=np.float32, ptr=None, root=None):
        self.shape = _shape_tuple(shape)
        self.dtype = np.dtype(dtype)
        if self.dtype not in _DTYPES:
            raise TypeError(f"unsupported device dtype {self.dtype}")
        self._version = 0
        if ptr is None:
            p = C.c_void_p()
            check(lib.tlnn_alloc(backend.ctx(), self.nbytes, C.byref(p)))
            self.ptr = p.value
            self._owner = True
            self._root = self
        else:
            self.ptr = int(ptr)
            self._owner = False
            self._root = root if root is not None else self

    # ---- basic properties
    @property
    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def nbytes(self) -> int:
        return self.size * self.dtype.itemsize

    @property
    def version(self) -> int:
        return self._root._version

    def _touch(self):
        self._root._version += 1

    def __len__(self):
        return self.shape[0]

    def __repr__(self):
        return f"DeviceArray(shape={self.shape}, dtype={self.dtype}, ptr=0x{self.ptr:x})"

    def __del__(self):
        try:
            if self._owner and self.ptr and backend._ctx is not None:
                lib.tlnn_free(backend._ctx, self.ptr)
        except Exception:
            pass

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": self.dtype.str, "data": (self.ptr, False), "version": 3,
                "strides": None, "stream": int(lib.tlnn_stream(backend.ctx()) or 0) or None}

    # ---- host <-> device
    @classmethod
    def from_numpy(cls, a) -> "DeviceArray":
        a = np.ascontiguousarray(a)
        out = cls(a.shape, a.dtype)
        check(lib.tlnn_h2d(backend.ctx(), out.ptr, a.ctypes.data, a.nbytes))
        # the copy is asynchronous only for pinned sources; pageable sources are staged before the call returns
        return out

    def get(self) -> np.ndarray:
        """Copy to a new NumPy array (waits for the stream; surfaces device-side errors)."""
        out = np.empty(self.shape, dtype=self.dtype)
        check(lib.tlnn_d2h(backend.ctx(), out.ctypes.data, self.ptr, self.nbytes))
        return out

    def __array__(self, dtype=None, copy=None):
        a = self.get()
        return a if dtype is None else a.astype(dtype)

    def copy(self) -> "DeviceArray":
        out = DeviceArray(self.shape, self.dtype)
        check(lib.tlnn_d2d(backend.ctx(), out.ptr, self.ptr, self.nbytes))
        return out

    def astype(self, dtype) -> "DeviceArray":
        if np.dtype(dtype) == self.dtype:
            return self.copy()
        return DeviceArray.from_numpy(self.get().astype(dtype))

    # ---- views
    def reshape(self, *shape) -> "DeviceArray":
        if len(shape) == 1 and not isinstance(shape[0], (int, np.integer)):
            shape = tuple(shape[0])
        shape = list(int(s) for s in shape)
        if shape.count(-1) > 1:
            raise ValueError("can only specify one unknown dimension")
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1], dtype=np.int64))
            shape[shape.index(-1)] = self.size // max(known, 1)
        if int(np.prod(shape, dtype=np.int64)) != self.size:
            raise ValueError(f"cannot reshape array of size {self.size} into shape {tuple(shape)}")
        return DeviceArray(shape, self.dtype, ptr=self.ptr, root=self._root)

    def _normalised_key(self, key):
        """``key`` as one entry per axis (Ellipsis expanded, trailing axes filled with full slices), or None when it
        holds anything other than integers and slices."""
        if not isinstance(key, tuple):
            key = (key,)
        n_ell = sum(1 for k in key if k is Ellipsis)
        if n_ell > 1:
            return None
        if n_ell:
            i = next(j for j, k in enumerate(key) if k is Ellipsis)
            key = key[:i] + (slice(None),) * (self.ndim - (len(key) - 1)) + key[i + 1:]
        if len(key) > self.ndim:
            raise IndexError(f"too many indices for array: array is {self.ndim}-dimensional, but {len(key)} were indexed")
        key = key + (slice(None),) * (self.ndim - len(key))
        for k in key:
            if isinstance(k, (bool, np.bool_)) or not isinstance(k, (int, np.integer, slice)):
                return None
        return key

    def _basic_offsets(self, key):
        """Flat element offsets selected by integers and slices, computed from the strides axis by axis: the host
        builds an array the size of the SELECTION, never of the whole array (``predict(x)[0, -1]`` on a
        (64, 2048, 50257) array touches 50257 offsets).  Returns None for advanced (array, boolean) indices."""
        key = self._normalised_key(key)
        if key is None:
            return None
        strides = [1] * self.ndim
        for ax in range(self.ndim - 2, -1, -1):
            strides[ax] = strides[ax + 1] * self.shape[ax + 1]
        base, axes = 0, []
        for ax, k in enumerate(key):
            n = self.shape[ax]
            if isinstance(k, slice):
                axes.append(np.arange(*k.indices(n), dtype=np.int64) * strides[ax])
            else:
                i = int(k) + n if k < 0 else int(k)
                if not 0 <= i < n:
                    raise IndexError(f"index {int(k)} is out of bounds for axis {ax} with size {n}")
                base += i * strides[ax]
        out = np.full((), base, dtype=np.int64)
        for a in axes:
            out = out[..., None] + a
        return out

    def _flat_index(self, key) -> np.ndarray:
        """Flat element offsets selected by a NumPy basic or advanced index (host-side arithmetic)."""
        idx = self._basic_offsets(key)
        if idx is not None:
            return idx
        return np.arange(self.size, dtype=np.int64).reshape(self.shape)[key]

    def __getitem__(self, key):
        if key is Ellipsis or (isinstance(key, slice) and key == slice(None)):
            return self
        idx = self._flat_index(key)
        out_shape = idx.shape
        flat = np.ascontiguousarray(idx.reshape(-1))
        # one contiguous run is a plain copy; anything else goes through the gather kernel
        if flat.size <= 1 or (int(flat[-1]) - int(flat[0]) == flat.size - 1 and np.all(np.diff(flat) == 1)):
            out = DeviceArray(out_shape, self.dtype)
            if flat.size:
                check(lib.tlnn_d2d(backend.ctx(), out.ptr, self.ptr + int(flat[0]) * self.dtype.itemsize, out.nbytes))
            return out
        if self.dtype != np.float32:
            return DeviceArray.from_numpy(self.get().reshape(-1)[flat].reshape(out_shape))
        out = DeviceArray(out_shape, self.dtype)
        dev_idx = DeviceArray.from_numpy(flat)
        check(lib.tlnn_gather_f32(backend.ctx(), self.ptr, dev_idx.ptr, out.ptr, flat.size))
        return out

    def __setitem__(self, key, value):
        full = key is Ellipsis or (isinstance(key, slice) and key == slice(None))
        if full and isinstance(value, DeviceArray):
            if value.shape != self.shape or value.dtype != self.dtype:
                raise ValueError(f"could not broadcast input array from shape {value.shape} into shape {self.shape}")
            check(lib.tlnn_d2d(backend.ctx(), self.ptr, value.ptr, self.nbytes))
        elif full:
            a = np.ascontiguousarray(np.broadcast_to(np.asarray(value, dtype=self.dtype), self.shape))
            check(lib.tlnn_h2d(backend.ctx(), self.ptr, a.ctypes.data, a.nbytes))
        else:
            host = self.get()
            host[key] = value.get() if isinstance(value, DeviceArray) else value
            check(lib.tlnn_h2d(backend.ctx(), self.ptr, host.ctypes.data, host.nbytes))
        self._touch()

    # ---- in-place arithmetic used by weight loading and optimiser-free parameter edits
    def _need_f32(self):
        if self.dtype != np.float32:
            raise TypeError("in-place arithmetic is implemented for float32 arrays")

    def fill(self, value):
        self._need_f32()
        check(lib.tlnn_axpby_f32(backend.ctx(), self.ptr, 0.0, None, float(value), self.size))
        self._touch()

    def __imul__(self, scalar):
        self._need_f32()
        check(lib.tlnn_axpby_f32(backend.ctx(), self.ptr, float(scalar), None, 0.0, self.size))
        self._touch()
        return self

    def __iadd__(self, other):
        self._need_f32()
        if isinstance(other, (int, float, np.floating, np.integer)):
            check(lib.tlnn_axpby_f32(backend.ctx(), self.ptr, 1.0, None, float(other), self.size))
        else:
            o = other if isinstance(other, DeviceArray) else as_device(
                np.ascontiguousarray(np.broadcast_to(np.asarray(other, dtype=np.float32), self.shape)))
            if o.shape != self.shape:
                raise ValueError(f"operands could not be broadcast together with shapes {self.shape} {o.shape}")
            check(lib.tlnn_axpby_f32(backend.ctx(), self.ptr, 1.0, o.ptr, 1.0, self.size))
        self._touch()
        return self

    def __add__(self, other):
        self._need_f32()
        o = other if isinstance(other, DeviceArray) else as_device(
            np.ascontiguousarray(np.broadcast_to(np.asarray(other, dtype=np.float32), self.shape)))
        if o.shape != self.shape:
            raise ValueError(f"operands could not be broadcast together with shapes {self.shape} {o.shape}")
        out = DeviceArray(self.shape, np.float32)
        check(lib.tlnn_add_f32(backend.ctx(), self.ptr, o.ptr, out.ptr, self.size))
        return out

    __radd__ = __add__


def zeros(shape, dtype=np.float32) -> DeviceArray:
    out = DeviceArray(shape, dtype)
    check(lib.tlnn_memset(backend.ctx(), out.ptr, 0, out.nbytes))
    return out


def as_device(x, dtype=None) -> DeviceArray:
    """Device handle for ``x``: a DeviceArray passes through, host data is copied to the device."""
    if isinstance(x, DeviceArray):
        return x
    a = np.asarray(x) if dtype is None else np.asarray(x, dtype=dtype)
    if a.dtype == np.float64:
        a = a.astype(np.float32)
    return DeviceArray.from_numpy(a)


def as_token_ids(x) -> DeviceArray:
    """Token ids on the device.  Any integer dtype is accepted (the demo uses uint8: demo.ipynb:1524); a
    non-integer dtype raises IndexError as ``table[input]`` does in the reference."""
    if isinstance(x, DeviceArray):
        if x.dtype.kind not in "iu":
            raise IndexError("arrays used as indices must be of integer type")
        return x
    a = np.asarray(x)
    if a.dtype.kind not in "iu":
        raise IndexError("arrays used as indices must be of integer (or boolean) type")
    if a.dtype not in (np.dtype(np.int32), np.dtype(np.uint8), np.dtype(np.int64)):
        a = a.astype(np.int64)
    return DeviceArray.from_numpy(a)


def argmax_last(a: DeviceArray) -> DeviceArray:
    """First index of the maximum over the last axis (numpy.argmax semantics), int32 on the device."""
    if a.dtype != np.float32:
        raise TypeError("argmax expects a float32 array")
    cols = a.shape[-1]
    rows = a.size // cols
    out = DeviceArray(a.shape[:-1], np.int32)
    check(lib.tlnn_argmax_fwd(backend.ctx(), a.ptr, cols, out.ptr, rows, cols))
    return out
