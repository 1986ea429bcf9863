"""GPT and ViT adapter layers, B200 runtime (mirror of the reference's ``transformer_adapters.py``, forward path)."""
from __future__ import annotations

import numpy as np

from . import _lib
from ._lib import lib, check
from . import backend
from .backend import xp, FLOAT_TYPE, init_random_tensor, init_zeros_tensor  # noqa: F401
from .device_array import DeviceArray, as_device, as_token_ids
from .utils import Layer, PreparedWeight, linear
from .layers import Dropout  # noqa: F401  (re-exported by the reference module too)


def _scaled_normal(shape, divisor):
    a = backend.rng.standard_normal(shape, dtype=FLOAT_TYPE) / divisor
    return DeviceArray.from_numpy(a.astype(FLOAT_TYPE))


class VitProjector(Layer):
    """Patchify + linear projection + class/register tokens + positional embeddings
    (transformer_adapters.py:6-55).  Patch features are ordered (row in patch, column in patch, channel)."""

    def __init__(self, input_size: tuple, patch_size: tuple, embedding_dim, num_registers=0):
        super(VitProjector, self).__init__()
        self.batch_size = 0
        self.channels, self.height, self.width = input_size
        self.patch_size = patch_size
        self.patches_height = self.height // self.patch_size[0]
        self.patches_width = self.width // self.patch_size[1]
        self.sequence_length = self.patches_height * self.patches_width
        self.token_dim = self.patch_size[0] * self.patch_size[1] * self.channels
        self.embedding_dim = embedding_dim
        self.cls_reg_size = 1 + num_registers

        self.projection = _scaled_normal((self.token_dim, self.embedding_dim), self.token_dim ** 0.5)
        self.cls_reg_tokens = _scaled_normal((self.cls_reg_size, self.embedding_dim), self.embedding_dim ** 0.5)
        self.positional_embeddings = init_zeros_tensor((self.cls_reg_size + self.sequence_length, self.embedding_dim))

        self.projection_grads = self.register_param(self.projection)
        self.cls_reg_token_grads = self.register_param(self.cls_reg_tokens)
        self.positional_embeddings_grads = self.register_param(self.positional_embeddings)
        self._proj = PreparedWeight(self.projection, transpose=True)

    def forward(self, input):
        self.input = as_device(input, np.float32)
        want = (self.channels, self.height, self.width)
        if self.input.ndim != 4 or self.input.shape[1:] != want:
            raise ValueError(f"cannot reshape array of shape {self.input.shape} into patches of a {want} image")
        self.batch_size = self.input.shape[0]
        T = self.cls_reg_size + self.sequence_length
        self.output = DeviceArray((self.batch_size, T, self.embedding_dim), np.float32)
        check(lib.tlnn_vit_project_fwd(backend.ctx(), backend.precision_code(), self.input.ptr, self._proj.ptr(),
                                       self.cls_reg_tokens.ptr, self.positional_embeddings.ptr, self.output.ptr,
                                       self.batch_size, self.channels, self.height, self.width,
                                       self.patch_size[0], self.patch_size[1], self.embedding_dim, self.cls_reg_size - 1))
        return self.output


class VitMLPHead(Layer):
    """Linear layer on the class token: x[:, 0, :] @ W + b (transformer_adapters.py:76-95)."""

    def __init__(self, in_channels, out_channels):
        super(VitMLPHead, self).__init__()
        self.weights = _scaled_normal((in_channels, out_channels), in_channels ** 0.5)
        self.bias = init_zeros_tensor(out_channels)
        self.weight_grads = self.register_param(self.weights)
        self.bias_grads = self.register_param(self.bias)
        self._w = PreparedWeight(self.weights, transpose=True)

    def forward(self, input):
        self.input = as_device(input, np.float32)
        d, n_out = self.weights.shape
        if self.input.ndim != 3 or self.input.shape[2] != d:
            raise ValueError(f"ViT head expects (B, T, {d}), got {self.input.shape}")
        B, T, _ = self.input.shape
        self.output = DeviceArray((B, n_out), np.float32)
        check(lib.tlnn_vit_head_fwd(backend.ctx(), backend.precision_code(), self.input.ptr, self._w.ptr(), self.bias.ptr,
                                    self.output.ptr, B, T, d, n_out))
        return self.output


class GPTEmbeddingTable:
    """Token table shared by the embedding and the tied output layer (transformer_adapters.py:108-116)."""

    def __init__(self, vocab_size, embed_size):
        self.vocab_size = vocab_size
        self.embed_size = embed_size
        self.table = init_random_tensor((vocab_size, embed_size))
        self.table_grads = None
        self.table_moments = None
        self.table_vars = None
        # (V, d) already has the contraction dimension contiguous: no transpose for the tied head
        self._as_head = PreparedWeight(self.table, transpose=False)


class GPTEmbedFront(Layer):
    """table[ids] + positional[:T] (transformer_adapters.py:119-153), learned or sinusoidal positions."""

    def __init__(self, embedding_table: GPTEmbeddingTable, context_length, positional_embedding="learned"):
        super(GPTEmbedFront, self).__init__()
        assert positional_embedding == "learned" or positional_embedding == "sinusoidal"
        self.positional_embedding = positional_embedding
        self.context_length = context_length
        d = embedding_table.embed_size
        if self.positional_embedding == "sinusoidal":
            # float64 on the host exactly as the reference builds it, then cast (transformer_adapters.py:128-135)
            pos = np.arange(context_length)[:, None]
            i = np.arange(d)[None, :]
            t = pos / 10000 ** (2 * (i // 2) / d)
            t[:, 0::2] = np.sin(t[:, 0::2])
            t[:, 1::2] = np.cos(t[:, 1::2])
            self.pos_embedding_table = DeviceArray.from_numpy(t.astype(FLOAT_TYPE))
        else:
            self.pos_embedding_table = init_zeros_tensor((context_length, d))
            self.pos_embedding_table_grads = self.register_param(self.pos_embedding_table)
        self.embedding_table = embedding_table
        self.parameters.append(self.embedding_table.table)
        self.gradients.append(None)
        self.moments.append(None)
        self.variances.append(None)

    def forward(self, input):
        self.input = as_token_ids(input)
        if self.input.ndim != 2:
            raise ValueError(f"token ids must be (B, T), got {self.input.shape}")
        B, T = self.input.shape
        if T > self.context_length:
            raise ValueError(f"operands could not be broadcast together with shapes ({B},{T},{self.embedding_table.embed_size}) "
                             f"({self.context_length},{self.embedding_table.embed_size})")
        d, V = self.embedding_table.embed_size, self.embedding_table.vocab_size
        self.output = DeviceArray((B, T, d), np.float32)
        check(lib.tlnn_embed_fwd(backend.ctx(), self.input.ptr, _ids_code(self.input), self.embedding_table.table.ptr,
                                 self.pos_embedding_table.ptr, self.output.ptr, B, T, d, V))
        # an out-of-range id raises IndexError here, as table[input] does in the reference
        check(lib.tlnn_check(backend.ctx()))
        return self.output


def _ids_code(ids: DeviceArray) -> int:
    return {np.dtype(np.int32): _lib.I32, np.dtype(np.int64): _lib.I64, np.dtype(np.uint8): _lib.U8}[ids.dtype]


class GPTEmbedBack(Layer):
    """Tied output layer: x @ table.T, no bias (transformer_adapters.py:167-177)."""

    def __init__(self, embedding_table: GPTEmbeddingTable):
        super(GPTEmbedBack, self).__init__()
        self.embedding_table = embedding_table
        self.is_embed_layer_back = False

    def forward(self, input):
        self.input = as_device(input, np.float32)
        d, V = self.embedding_table.embed_size, self.embedding_table.vocab_size
        if self.input.shape[-1] != d:
            raise ValueError(f"matmul: input has width {self.input.shape[-1]}, table expects {d}")
        self.output = linear(self.input, self.embedding_table._as_head, None, V)
        return self.output

    def forward_tokens(self, input):
        """arg-max over the vocabulary taken inside the GEMM epilogue; the logits are never written."""
        x = as_device(input, np.float32)
        d, V = self.embedding_table.embed_size, self.embedding_table.vocab_size
        rows = x.size // d
        tokens = DeviceArray(x.shape[:-1], np.int32)
        check(lib.tlnn_logits_fwd(backend.ctx(), backend.precision_code(), x.ptr, self.embedding_table._as_head.ptr(),
                                  None, None, tokens.ptr, rows, d, V))
        return tokens
