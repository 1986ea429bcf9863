"""Layer interface and the Residual wrapper, B200 runtime.

Mirror of the reference's ``utils.py`` (Layer: utils.py:8-52, Residual: utils.py:55-104) for the forward path.
Differences that follow from scope, not from taste: gradients, moments and variances are training state, so
``register_param`` records ``None`` placeholders instead of allocating three zero tensors per parameter
(utils.py:34-41 would triple weight memory), and ``backward`` raises ``NotImplementedError`` everywhere.
"""
from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import lib, check
from . import backend
from .backend import xp, FLOAT_TYPE, init_random_tensor, init_zeros_tensor  # noqa: F401  (same exports as the reference)
from .device_array import DeviceArray, as_device


class Layer:

    def __init__(self):
        self.input = None
        self.output = None

        self.parameters = []
        self.gradients = []
        self.moments = []
        self.variances = []

        self.eval_mode = False
        self.is_embed_layer_back = False

    def forward(self, *input):
        raise NotImplementedError

    def backward(self, *input):
        raise NotImplementedError("the B200 runtime implements the forward path only; train with the reference runtime")

    def set_eval(self, eval_mode):
        self.eval_mode = eval_mode

    def register_param(self, parameter):
        self.parameters.append(parameter)
        self.gradients.append(None)
        self.moments.append(None)
        self.variances.append(None)
        return None

    def zero_grad(self):
        for grad in self.gradients:
            if grad is not None:
                grad.fill(0)

    def zero_adam(self):
        for moment, variance in zip(self.moments, self.variances):
            if moment is not None:
                moment.fill(0)
            if variance is not None:
                variance.fill(0)


class PreparedWeight:
    """A GEMM weight in the layout and type the tensor cores read: (out, in) with the contraction dimension
    contiguous, bf16 or TF32-rounded float32.  Built lazily from the float32 parameter the layer owns and rebuilt
    when that parameter is modified in place or the arithmetic mode changes."""

    def __init__(self, param: DeviceArray, transpose: bool):
        self.param = param
        self.transpose = transpose
        self._key = None
        self._buf = None
        self._ptr = 0

    def ptr(self) -> int:
        prec = backend.precision_code()
        key = (self.param.version, prec, self.param.ptr)
        if key != self._key:
            rows, cols = self.param.shape
            nbytes = rows * cols * (2 if prec == _lib.PREC_BF16 else 4)
            # raw device bytes: kept as a uint8 array so that the handle frees itself
            self._buf = DeviceArray((nbytes,), np.uint8)
            check(lib.tlnn_weight_prepare(backend.ctx(), self.param.ptr, rows, cols, 1 if self.transpose else 0, prec,
                                          self._buf.ptr))
            self._ptr = self._buf.ptr
            self._key = key
        return self._ptr


def linear(x: DeviceArray, weight: PreparedWeight, bias, n_out: int, act: int = _lib.ACT_NONE) -> DeviceArray:
    """x @ W + b on the last axis of a float32 device array of any rank."""
    k = x.shape[-1]
    m = x.size // k if k else 0
    out = DeviceArray(x.shape[:-1] + (n_out,), np.float32)
    check(lib.tlnn_linear_fwd(backend.ctx(), backend.precision_code(), x.ptr, k, weight.ptr(),
                              bias.ptr if bias is not None else None, act, None, 0, out.ptr, n_out, m, n_out, k))
    return out


class Residual(Layer):
    """Runs a sub-list of layers and adds the input back (utils.py:76-88).  Only ``mode="add"`` is on the
    transformer forward path; ``"concat"`` belongs to the convolutional demo and is not implemented here."""

    def __init__(self, layers: list, mode="add", concat_axis=1):
        super(Residual, self).__init__()
        self.layers = layers
        self.mode = mode
        assert self.mode in {"add", "concat"}
        self.concat_axis = concat_axis
        for layer in layers:
            self.parameters = self.parameters + layer.parameters
            self.gradients = self.gradients + layer.gradients
            self.moments = self.moments + layer.moments
            self.variances = self.variances + layer.variances

    def forward(self, input):
        self.input = as_device(input, np.float32)
        x = self.input
        for layer in self.layers:
            x = layer.forward(x)
        if self.mode == "add":
            self.output = self.input + x
        else:
            raise NotImplementedError("Residual(mode='concat') is outside the transformer forward path")
        return self.output

    def set_eval(self, eval_mode):
        for layer in self.layers:
            layer.set_eval(eval_mode)
