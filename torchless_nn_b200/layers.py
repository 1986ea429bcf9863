"""Transformer layers, B200 runtime (mirror of the reference's ``layers.py`` for the forward path).

Constructors keep the reference's names, positional order and defaults; parameters are float32 device arrays with
the reference's shapes and initial distributions; ``forward`` takes one array (NumPy or device) and returns a device
array, also stored in ``self.output``.  Each ``forward`` is one call into libtlnn.so.  The convolutional layers of
the reference (layers.py:5-192) are not on the transformer path and are not provided.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import lib, check
from . import backend
from .backend import xp, FLOAT_TYPE, init_random_tensor, init_zeros_tensor  # noqa: F401
from .device_array import DeviceArray, as_device
from .utils import Layer, PreparedWeight, linear


def _scaled_normal(shape, divisor):
    a = backend.rng.standard_normal(shape, dtype=FLOAT_TYPE) / FLOAT_TYPE(divisor)
    return DeviceArray.from_numpy(a.astype(FLOAT_TYPE))


class Dense(Layer):
    """input @ W + b, W stored (in, out) (layers.py:195-209)."""

    def __init__(self, input_size, output_size):
        super(Dense, self).__init__()
        self.weights = _scaled_normal((input_size, output_size), (0.5 * input_size) ** 0.5)
        self.bias = init_zeros_tensor(output_size)
        self.weight_grads = self.register_param(self.weights)
        self.bias_grads = self.register_param(self.bias)
        self._w = PreparedWeight(self.weights, transpose=True)

    def forward(self, input):
        self.input = as_device(input, np.float32)
        if self.input.shape[-1] != self.weights.shape[0]:
            raise ValueError(f"matmul: input has width {self.input.shape[-1]}, weight expects {self.weights.shape[0]}")
        self.output = linear(self.input, self._w, self.bias, self.weights.shape[1])
        return self.output

    def forward_tokens(self, input):
        """arg-max over the outputs without materialising them (used when Dense is a language-model head)."""
        x = as_device(input, np.float32)
        d, v = self.weights.shape
        rows = x.size // d
        tokens = DeviceArray(x.shape[:-1], np.int32)
        check(lib.tlnn_logits_fwd(backend.ctx(), backend.precision_code(), x.ptr, self._w.ptr(), self.bias.ptr, None,
                                  tokens.ptr, rows, d, v))
        return tokens


class Dropout(Layer):
    """Identity in evaluation mode or at rate 0, returning its input object (layers.py:225-233).  The random-mask
    mode is training behaviour and raises."""

    def __init__(self, dropout_rate):
        super(Dropout, self).__init__()
        self.dropout_rate = dropout_rate
        self.dropout_neurons = None

    def forward(self, input):
        self.input = input
        if self.dropout_rate > 0.0 and self.eval_mode is False:
            raise NotImplementedError("dropout masks are training behaviour; call set_eval(True) or use rate 0")
        self.output = self.input
        return self.output


class MultiHeadAttention(Layer):
    """Multi-head self-attention (layers.py:241-307): fused QKV projection, scaled scores, optional decoder mask,
    softmax, weighted sum, output projection - two tensor-core GEMMs around one fused attention kernel."""

    def __init__(self, embedding_dim, context_length, num_heads, decoder=False,
                 attn_dropout_rate=0.0, res_dropout_rate=0.0):
        super(MultiHeadAttention, self).__init__()
        self.embedding_dim = embedding_dim
        self.context_length = context_length
        self.num_heads = num_heads
        self.heads_dim = embedding_dim // num_heads
        self.is_decoder = decoder

        self.attn_dropout = Dropout(attn_dropout_rate)
        self.res_dropout = Dropout(res_dropout_rate)

        self.qkv_weights = _scaled_normal((embedding_dim, 3 * embedding_dim), (0.5 * embedding_dim) ** 0.5)
        self.qkv_bias = init_zeros_tensor(3 * embedding_dim)
        self.out_weights = _scaled_normal((embedding_dim, embedding_dim), (0.5 * embedding_dim) ** 0.5)
        self.out_bias = init_zeros_tensor(embedding_dim)

        self.qkv_weight_grads = self.register_param(self.qkv_weights)
        self.qkv_bias_grads = self.register_param(self.qkv_bias)
        self.out_weight_grads = self.register_param(self.out_weights)
        self.out_bias_grads = self.register_param(self.out_bias)

        self._wqkv = PreparedWeight(self.qkv_weights, transpose=True)
        self._wo = PreparedWeight(self.out_weights, transpose=True)

    def _check_dropout(self):
        for drop in (self.attn_dropout, self.res_dropout):
            if drop.dropout_rate > 0.0 and drop.eval_mode is False:
                raise NotImplementedError("dropout masks are training behaviour; call set_eval(True) or use rate 0")

    def forward(self, input):
        self._check_dropout()
        self.input = as_device(input, np.float32)
        if self.input.ndim != 3 or self.input.shape[2] != self.embedding_dim:
            raise ValueError(f"attention expects (B, T, {self.embedding_dim}), got {self.input.shape}")
        B, T, Cc = self.input.shape
        if self.is_decoder and T > self.context_length:
            raise ValueError(f"operands could not be broadcast together: sequence length {T} exceeds the mask "
                             f"({self.context_length}, {self.context_length})")
        self.output = DeviceArray((B, T, Cc), np.float32)
        check(lib.tlnn_attention_fwd(backend.ctx(), backend.precision_code(), self.input.ptr, self._wqkv.ptr(),
                                     self.qkv_bias.ptr, self._wo.ptr(), self.out_bias.ptr, self.output.ptr,
                                     B, T, Cc, self.num_heads, 1 if self.is_decoder else 0))
        return self.output

    def set_eval(self, eval_mode):
        self.attn_dropout.set_eval(eval_mode)
        self.res_dropout.set_eval(eval_mode)


class TransformerFeedForward(Layer):
    """act(x W1 + b1) W2 + b2 with hidden width 4 d (layers.py:346-375); ``activation`` is a class, as in the
    reference, and is fused into the first GEMM."""

    def __init__(self, num_channels, activation, res_dropout_rate=0.0):
        super(TransformerFeedForward, self).__init__()
        self.activation = activation()
        self.dropout = Dropout(res_dropout_rate)
        self.weights1 = _scaled_normal((num_channels, 4 * num_channels), (0.5 * num_channels) ** 0.5)
        self.bias1 = init_zeros_tensor(4 * num_channels)
        self.weights2 = _scaled_normal((4 * num_channels, num_channels), (2 * num_channels) ** 0.5)
        self.bias2 = init_zeros_tensor(num_channels)
        self.weight_grads1 = self.register_param(self.weights1)
        self.bias_grads1 = self.register_param(self.bias1)
        self.weight_grads2 = self.register_param(self.weights2)
        self.bias_grads2 = self.register_param(self.bias2)
        self._w1 = PreparedWeight(self.weights1, transpose=True)
        self._w2 = PreparedWeight(self.weights2, transpose=True)

    def act_code(self) -> int:
        code = getattr(self.activation, "ACT_CODE", None)
        if code is None:
            raise NotImplementedError(f"activation {type(self.activation).__name__} has no fused epilogue")
        return code

    def forward(self, input):
        if self.dropout.dropout_rate > 0.0 and self.dropout.eval_mode is False:
            raise NotImplementedError("dropout masks are training behaviour; call set_eval(True) or use rate 0")
        self.input = as_device(input, np.float32)
        d = self.weights1.shape[0]
        if self.input.shape[-1] != d:
            raise ValueError(f"feed-forward expects width {d}, got {self.input.shape}")
        rows = self.input.size // d
        self.output = DeviceArray(self.input.shape, np.float32)
        check(lib.tlnn_ffn_fwd(backend.ctx(), backend.precision_code(), self.input.ptr, self._w1.ptr(), self.bias1.ptr,
                               self._w2.ptr(), self.bias2.ptr, self.act_code(), self.output.ptr, rows, d))
        return self.output

    def set_eval(self, eval_mode):
        self.dropout.set_eval(eval_mode)


class LayerNorm(Layer):
    """Per-row normalisation with affine (layers.py:394-428), eps 1e-5."""

    def __init__(self, num_channels):
        super(LayerNorm, self).__init__()
        self.channels = num_channels
        self.eps = FLOAT_TYPE(1e-5)
        self.gamma = init_zeros_tensor(num_channels)
        self.gamma.fill(1)
        self.beta = init_zeros_tensor(num_channels)
        self.gamma_grads = self.register_param(self.gamma)
        self.beta_grads = self.register_param(self.beta)

    def forward(self, input):
        self.input = as_device(input, np.float32)
        if self.input.shape[-1] != self.channels:
            raise ValueError(f"operands could not be broadcast together with shapes {self.input.shape} ({self.channels},)")
        rows = self.input.size // self.channels
        self.output = DeviceArray(self.input.shape, np.float32)
        check(lib.tlnn_layernorm_fwd(backend.ctx(), self.input.ptr, self.gamma.ptr, self.beta.ptr, float(self.eps),
                                     self.output.ptr, rows, self.channels))
        return self.output


class TransformerBlock(Layer):
    """Pre-LN block: y = x + attn(ln1(x)); out = y + ffn(ln2(y)) (layers.py:444-467).  ``forward`` is a single
    library call that runs LayerNorm -> QKV GEMM -> attention -> output GEMM (+residual) -> LayerNorm ->
    GEMM (+activation) -> GEMM (+residual) on one stream."""

    def __init__(self, embed_dim, context_length, num_heads, activation, decoder=False,
                 attn_dropout_rate=0.0, res_dropout_rate=0.0):
        super(TransformerBlock, self).__init__()
        self.pre_attn_norm = LayerNorm(embed_dim)
        self.attn_block = MultiHeadAttention(embed_dim, context_length, num_heads, decoder=decoder,
                                             attn_dropout_rate=attn_dropout_rate, res_dropout_rate=res_dropout_rate)
        self.pre_ffn_norm = LayerNorm(embed_dim)
        self.ffn = TransformerFeedForward(embed_dim, activation, res_dropout_rate=res_dropout_rate)
        subs = (self.pre_attn_norm, self.attn_block, self.pre_ffn_norm, self.ffn)
        self.parameters = [p for s in subs for p in s.parameters]
        self.gradients = [g for s in subs for g in s.gradients]
        self.moments = [m for s in subs for m in s.moments]
        self.variances = [v for s in subs for v in s.variances]

    def block_params(self) -> _lib.BlockParams:
        a, f = self.attn_block, self.ffn
        return _lib.BlockParams(self.pre_attn_norm.gamma.ptr, self.pre_attn_norm.beta.ptr, a._wqkv.ptr(), a.qkv_bias.ptr,
                                a._wo.ptr(), a.out_bias.ptr, self.pre_ffn_norm.gamma.ptr, self.pre_ffn_norm.beta.ptr,
                                f._w1.ptr(), f.bias1.ptr, f._w2.ptr(), f.bias2.ptr)

    def forward(self, input):
        self.attn_block._check_dropout()
        self.input = as_device(input, np.float32)
        d = self.attn_block.embedding_dim
        if self.input.ndim != 3 or self.input.shape[2] != d:
            raise ValueError(f"transformer block expects (B, T, {d}), got {self.input.shape}")
        B, T, _ = self.input.shape
        if self.attn_block.is_decoder and T > self.attn_block.context_length:
            raise ValueError(f"operands could not be broadcast together: sequence length {T} exceeds the mask "
                             f"({self.attn_block.context_length}, {self.attn_block.context_length})")
        self.output = DeviceArray((B, T, d), np.float32)
        p = self.block_params()
        check(lib.tlnn_block_fwd(backend.ctx(), backend.precision_code(), self.input.ptr, C.byref(p), self.ffn.act_code(),
                                 self.output.ptr, B, T, d, self.attn_block.num_heads,
                                 1 if self.attn_block.is_decoder else 0))
        return self.output

    def set_eval(self, eval_mode):
        self.attn_block.set_eval(eval_mode)
        self.ffn.set_eval(eval_mode)
