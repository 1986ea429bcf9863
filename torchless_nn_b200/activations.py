"""Activation layers, B200 runtime (mirror of the reference's ``activations.py``).

Inside ``TransformerFeedForward`` the activation is fused into the first GEMM's epilogue; the classes here are the
stand-alone layers (``Network([... , SoftMax()])``, demo.ipynb:1216,1499) and also name the activation for the
fused path through ``ACT_CODE``.
"""
from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import lib, check
from . import backend
from .backend import xp, FLOAT_TYPE  # noqa: F401
from .device_array import DeviceArray, as_device
from .utils import Layer


class _Elementwise(Layer):
    ACT_CODE = _lib.ACT_NONE

    def forward(self, input):
        self.input = as_device(input, np.float32)
        self.output = DeviceArray(self.input.shape, np.float32)
        check(lib.tlnn_activation_fwd(backend.ctx(), self.ACT_CODE, self.input.ptr, self.output.ptr, self.input.size))
        return self.output


class ReLU(_Elementwise):
    """max(x, 0) (activations.py:10-13)."""
    ACT_CODE = _lib.ACT_RELU


class GeLU(_Elementwise):
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) (activations.py:24-28)."""
    ACT_CODE = _lib.ACT_GELU


class SiLU(_Elementwise):
    """x (1 + tanh(x / 2)) / 2 (activations.py:41-45)."""
    ACT_CODE = _lib.ACT_SILU


class SoftMax(Layer):
    """exp((x - max) / temperature) / sum over the last axis (activations.py:57-64).  ``temperature`` may be
    changed after construction (demo.ipynb:1650)."""

    def __init__(self, temperature=FLOAT_TYPE(1.0)):
        super(SoftMax, self).__init__()
        self.temperature = temperature

    def forward(self, input):
        self.input = as_device(input, np.float32)
        cols = self.input.shape[-1]
        rows = self.input.size // cols
        self.output = DeviceArray(self.input.shape, np.float32)
        check(lib.tlnn_softmax_fwd(backend.ctx(), self.input.ptr, self.output.ptr, rows, cols, float(self.temperature)))
        return self.output
