"""Sequential container, B200 runtime (mirror of the reference's ``network.py`` for the forward path).

``predict`` keeps the reference's meaning: apply every layer's ``forward`` in order and return the last output
(network.py:33-39).  Two additions serve the inference workloads the reference drives from user code:

* ``predict_tokens(ids)``: greedy next-token ids for every position.  For the GPT recipe
  (GPTEmbedFront, [Dropout], decoder TransformerBlocks, LayerNorm, GPTEmbedBack | Dense) the whole forward is one
  library call with the arg-max fused into the head GEMM, so the (B, T, V) logits are never written.
* ``generate_greedy(prompts, new_tokens)``: the notebook's generation loop (demo.ipynb:1520-1535) with arg-max
  in place of sampling, on a per-layer KV cache instead of re-running the window for every token.

Training (``train``, ``evaluate``'s loss, AdamW: network.py:51-160) belongs to the reference runtimes.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import lib, check
from . import backend
from .backend import xp, FLOAT_TYPE  # noqa: F401
from .device_array import DeviceArray, as_device, as_token_ids, argmax_last
from .utils import Layer
from .layers import *  # noqa: F401,F403
from .layers import Dropout, LayerNorm, TransformerBlock, Dense
from .transformer_adapters import *  # noqa: F401,F403
from .transformer_adapters import GPTEmbedFront, GPTEmbedBack, _ids_code


class GPTPlan:
    """The tlnn_gpt_model description of a layer list that follows the GPT recipe."""

    def __init__(self, front, blocks, final_norm, head):
        self.front, self.blocks, self.final_norm, self.head = front, blocks, final_norm, head

    @staticmethod
    def match(layers):
        ls = [l for l in layers if not isinstance(l, Dropout)]
        if len(ls) < 3 or not isinstance(ls[0], GPTEmbedFront) or not isinstance(ls[-2], LayerNorm):
            return None
        if not isinstance(ls[-1], (GPTEmbedBack, Dense)):
            return None
        blocks = ls[1:-2]
        if not all(isinstance(b, TransformerBlock) and b.attn_block.is_decoder for b in blocks):
            return None
        if blocks and len({(b.attn_block.embedding_dim, b.attn_block.num_heads, b.ffn.act_code()) for b in blocks}) != 1:
            return None
        return GPTPlan(ls[0], blocks, ls[-2], ls[-1])

    def model(self):
        """Build the C struct; the returned tuple keeps the block array alive."""
        f = self.front
        d, V = f.embedding_table.embed_size, f.embedding_table.vocab_size
        arr = (_lib.BlockParams * max(len(self.blocks), 1))()
        for i, b in enumerate(self.blocks):
            arr[i] = b.block_params()
        if isinstance(self.head, GPTEmbedBack):
            head_t, head_b = self.head.embedding_table._as_head.ptr(), None
            if self.head.embedding_table.embed_size != d:
                raise ValueError("tied head width differs from the model width")
        else:
            head_t, head_b = self.head._w.ptr(), self.head.bias.ptr
            V = self.head.weights.shape[1]
        heads = self.blocks[0].attn_block.num_heads if self.blocks else 1
        act = self.blocks[0].ffn.act_code() if self.blocks else _lib.ACT_NONE
        m = _lib.GPTModel(f.embedding_table.vocab_size, f.context_length, d, heads, len(self.blocks), act,
                          backend.precision_code(), f.embedding_table.table.ptr, f.pos_embedding_table.ptr,
                          arr, self.final_norm.gamma.ptr, self.final_norm.beta.ptr, head_t, head_b)
        return m, arr, V


class Network:

    def __init__(self, layers: list):
        self.layers = layers

    def predict(self, input):
        return self._forward(input)

    def _forward(self, input):
        for layer in self.layers:
            input = layer.forward(input)
        return input

    def _backward(self, gradient):
        raise NotImplementedError("the B200 runtime implements the forward path only")

    def set_eval(self, eval_mode):
        for layer in self.layers:
            layer.set_eval(eval_mode)
            layer.zero_grad()

    # ---- additions ------------------------------------------------------------------------------------------
    def _check_eval(self):
        for layer in self.layers:
            if isinstance(layer, Dropout) and layer.dropout_rate > 0.0 and layer.eval_mode is False:
                raise NotImplementedError("dropout masks are training behaviour; call set_eval(True) first")

    def predict_logits(self, input):
        """Same result as ``predict`` for the GPT recipe, as one fused library call (no per-layer outputs kept)."""
        plan = GPTPlan.match(self.layers)
        if plan is None:
            return self.predict(input)
        self._check_eval()
        ids = as_token_ids(input)
        B, T = ids.shape
        if T > plan.front.context_length:
            raise ValueError(f"sequence length {T} exceeds the context length {plan.front.context_length}")
        m, keep, V = plan.model()
        logits = DeviceArray((B, T, V), np.float32)
        check(lib.tlnn_gpt_prefill(backend.ctx(), C.byref(m), ids.ptr, _ids_code(ids), B, T, logits.ptr, None))
        return logits

    def predict_tokens(self, input):
        """arg-max of ``predict(input)`` over the last axis, int32 on the device."""
        plan = GPTPlan.match(self.layers)
        if plan is not None:
            self._check_eval()
            ids = as_token_ids(input)
            B, T = ids.shape
            if T > plan.front.context_length:
                raise ValueError(f"sequence length {T} exceeds the context length {plan.front.context_length}")
            m, keep, V = plan.model()
            tokens = DeviceArray((B, T), np.int32)
            check(lib.tlnn_gpt_prefill(backend.ctx(), C.byref(m), ids.ptr, _ids_code(ids), B, T, None, tokens.ptr))
            return tokens
        return argmax_last(self.predict(input))

    def generate_greedy(self, prompts, new_tokens: int):
        """Greedy continuation of every prompt row by ``new_tokens`` tokens; returns (B, T0 + new_tokens) int32 on
        the device.  Prompt plus continuation must fit the context length (the notebook's sliding window beyond it,
        demo.ipynb:1528, is not implemented)."""
        plan = GPTPlan.match(self.layers)
        if plan is None:
            raise ValueError("generate_greedy needs the GPT layer recipe")
        self._check_eval()
        ids = as_token_ids(prompts)
        B, T0 = ids.shape
        if new_tokens < 1:
            raise ValueError("new_tokens must be positive")
        if T0 + new_tokens > plan.front.context_length:
            raise ValueError(f"prompt ({T0}) + new tokens ({new_tokens}) exceed the context length "
                             f"{plan.front.context_length}")
        m, keep, V = plan.model()
        first = DeviceArray((B,), np.int32)
        dec = C.c_void_p()
        check(lib.tlnn_decode_begin(backend.ctx(), C.byref(m), ids.ptr, _ids_code(ids), B, T0, T0 + new_tokens,
                                    first.ptr, C.byref(dec)))
        try:
            new = DeviceArray((B, new_tokens), np.int32)
            if new_tokens > 1:
                rest = DeviceArray((B, new_tokens - 1), np.int32)
                check(lib.tlnn_decode_run(dec, first.ptr, new_tokens - 1, rest.ptr))
                host = np.concatenate([first.get()[:, None], rest.get()], axis=1)
            else:
                host = first.get()[:, None]
        finally:
            lib.tlnn_decode_end(dec)
        prompt_host = ids.get().astype(np.int32)
        return DeviceArray.from_numpy(np.concatenate([prompt_host, host.astype(np.int32)], axis=1))
