"""Backend selector with the B200 runtime.

Mirrors the reference's ``backend.py`` (backend.py:1-34): the runtime is chosen once per process from the
``XP_RUNTIME`` environment variable and the same names are exported - ``runtime``, ``xp``, ``FLOAT_TYPE``,
``init_random_tensor``, ``init_zeros_tensor``.  The reference accepts ``CUDA`` (CuPy) and ``CPU`` (NumPy); this
module adds ``B200`` and implements only that value: ``xp`` is a small namespace whose arrays live in device memory
owned by libtlnn.so, and every layer's ``forward`` calls the library through ctypes.  There is no NumPy, PyTorch or
CuPy fallback: without the library or without a B200 the first device operation raises.

Arithmetic mode (the reference's CUDA path runs float32 storage with TF32 tensor-op math, backend.py:9,16):
``TLNN_PRECISION=tf32`` (default) keeps float32 storage and rounds GEMM operands to TF32;
``TLNN_PRECISION=bf16`` stores GEMM weights and operands as bf16 with float32 accumulation and a float32 residual
stream.  ``set_precision`` changes it at run time; prepared weights are rebuilt on demand.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib
from ._lib import lib, check

runtime = os.environ.get("XP_RUNTIME", "B200")
if runtime != "B200":
    raise AssertionError(
        f"XP_RUNTIME={runtime!r}: torchless_nn_b200 implements the 'B200' runtime only "
        "(the reference's own modules provide 'CUDA' and 'CPU')")

FLOAT_TYPE = np.float32

_PRECISIONS = {"tf32": _lib.PREC_TF32, "fp32": _lib.PREC_TF32, "bf16": _lib.PREC_BF16}
_precision = os.environ.get("TLNN_PRECISION", "tf32").lower()
if _precision not in _PRECISIONS:
    raise AssertionError(f"TLNN_PRECISION={_precision!r}: expected one of {sorted(_PRECISIONS)}")


def set_precision(name: str) -> None:
    global _precision
    name = name.lower()
    if name not in _PRECISIONS:
        raise ValueError(f"unknown precision {name!r}: expected one of {sorted(_PRECISIONS)}")
    _precision = name


def precision() -> str:
    return "tf32" if _precision == "fp32" else _precision


def precision_code() -> int:
    return _PRECISIONS[_precision]


_ctx = None


def device_index() -> int:
    """One process drives one GPU: TLNN_DEVICE, else the launcher's LOCAL_RANK, else 0."""
    return int(os.environ.get("TLNN_DEVICE", os.environ.get("LOCAL_RANK", "0")))


def ctx():
    """The process-wide engine context (created on first use)."""
    global _ctx
    if _ctx is None:
        h = C.c_void_p()
        check(lib.tlnn_init(device_index(), C.byref(h)))
        _ctx = h
    return _ctx


def synchronize() -> None:
    check(lib.tlnn_sync(ctx()))


def launch_count(reset: bool = False) -> int:
    return int(lib.tlnn_launch_count(ctx(), 1 if reset else 0))


def shutdown() -> None:
    global _ctx
    if _ctx is not None:
        lib.tlnn_shutdown(_ctx)
        _ctx = None


# The module-level generator is unseeded, as in the reference (backend.py:28).
rng = np.random.default_rng()


def init_random_tensor(size):
    """Standard-normal float32 tensor on the device (backend.py:30-31)."""
    from .device_array import DeviceArray
    return DeviceArray.from_numpy(rng.standard_normal(size, dtype=FLOAT_TYPE))


def init_zeros_tensor(size):
    """Zero float32 tensor on the device (backend.py:33-34)."""
    from .device_array import zeros
    return zeros(size, FLOAT_TYPE)


class _XP:
    """The slice of the array-module API that callers of the forward path use (demo.ipynb:1524-1533, 1576;
    network.py:135,158): array creation from host data, zeros, argmax, concatenate of token columns."""
    float32 = np.float32
    int32 = np.int32
    uint8 = np.uint8
    pi = np.pi

    @staticmethod
    def array(obj, dtype=None):
        from .device_array import DeviceArray, as_device
        if isinstance(obj, DeviceArray):
            return obj.copy() if dtype is None or np.dtype(dtype) == obj.dtype else obj.astype(dtype)
        return as_device(np.array(obj, dtype=dtype))

    asarray = array

    @staticmethod
    def zeros(shape, dtype=np.float32):
        from .device_array import zeros
        return zeros(shape, dtype)

    @staticmethod
    def argmax(a, axis=-1):
        from .device_array import argmax_last
        if axis not in (-1, a.ndim - 1):
            raise ValueError("argmax is implemented over the last axis only")
        return argmax_last(a)

    @staticmethod
    def asnumpy(a):
        return a.get() if hasattr(a, "get") else np.asarray(a)


xp = _XP()
