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
from .transformer_adapters import GPTEmbedFront, GPTEmbedBack, VitProjector, VitMLPHead, _ids_code


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
        table = ls[0].embedding_table
        if isinstance(ls[-1], Dense) and tuple(ls[-1].weights.shape) != (table.embed_size, table.vocab_size):
            return None          # a head of another width runs layer by layer
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
            # the C description has one vocabulary size: the id bound of the table and the width of the head product
            if tuple(self.head.weights.shape) != (d, V):
                raise ValueError(f"the fused GPT call needs a Dense head of shape ({d}, {V}); this one is "
                                 f"{tuple(self.head.weights.shape)}")
            head_t, head_b = self.head._w.ptr(), self.head.bias.ptr
        heads = self.blocks[0].attn_block.num_heads if self.blocks else 1
        act = self.blocks[0].ffn.act_code() if self.blocks else _lib.ACT_NONE
        m = _lib.GPTModel(f.embedding_table.vocab_size, f.context_length, d, heads, len(self.blocks), act,
                          backend.precision_code(), f.embedding_table.table.ptr, f.pos_embedding_table.ptr,
                          arr, self.final_norm.gamma.ptr, self.final_norm.beta.ptr, head_t, head_b)
        return m, arr, V


class ViTPlan:
    """The tlnn_vit_model description of a layer list that follows the ViT recipe (VitProjector, [Dropout], encoder
    TransformerBlocks, LayerNorm, VitMLPHead)."""

    def __init__(self, front, blocks, final_norm, head):
        self.front, self.blocks, self.final_norm, self.head = front, blocks, final_norm, head

    @staticmethod
    def match(layers):
        ls = [l for l in layers if not isinstance(l, Dropout)]
        if len(ls) < 3 or not isinstance(ls[0], VitProjector) or not isinstance(ls[-2], LayerNorm):
            return None
        if not isinstance(ls[-1], VitMLPHead):
            return None
        blocks = ls[1:-2]
        if not all(isinstance(b, TransformerBlock) and not b.attn_block.is_decoder for b in blocks):
            return None
        d = ls[0].embedding_dim
        if blocks and {(b.attn_block.embedding_dim, b.attn_block.num_heads, b.ffn.act_code()) for b in blocks} != \
                {(d, blocks[0].attn_block.num_heads, blocks[0].ffn.act_code())}:
            return None
        if ls[-1].weights.shape[0] != d or ls[-2].gamma.shape[-1] != d:
            return None
        return ViTPlan(ls[0], blocks, ls[-2], ls[-1])

    def model(self):
        """Build the C struct; the returned tuple keeps the block array alive."""
        f = self.front
        arr = (_lib.BlockParams * max(len(self.blocks), 1))()
        for i, b in enumerate(self.blocks):
            arr[i] = b.block_params()
        heads = self.blocks[0].attn_block.num_heads if self.blocks else 1
        act = self.blocks[0].ffn.act_code() if self.blocks else _lib.ACT_NONE
        n_out = self.head.weights.shape[1]
        m = _lib.ViTModel(f.channels, f.height, f.width, f.patch_size[0], f.patch_size[1], f.embedding_dim, heads,
                          len(self.blocks), act, backend.precision_code(), f.cls_reg_size - 1, n_out,
                          f._proj.ptr(), f.cls_reg_tokens.ptr, f.positional_embeddings.ptr, arr,
                          self.final_norm.gamma.ptr, self.final_norm.beta.ptr, self.head._w.ptr(), self.head.bias.ptr)
        return m, arr, n_out


def _rows(x, lo, hi):
    """Rows [lo, hi) of a batch: a view for device arrays (rows are contiguous), a slice for host arrays."""
    if isinstance(x, DeviceArray):
        per_row = int(np.prod(x.shape[1:], dtype=np.int64)) * x.dtype.itemsize
        return DeviceArray((hi - lo,) + tuple(x.shape[1:]), x.dtype, ptr=x.ptr + lo * per_row, root=x._root)
    return np.asarray(x)[lo:hi]


class CrossEntropy:
    """The criterion ``Network.evaluate`` takes (network.py:11-25).  Only ``loss`` has a meaning on the forward path:
    ``-sum(log(probs[label] + 1e-7))`` over a batch of probabilities; ``gradients`` belongs to training."""

    def __init__(self, num_classes):
        self.num_classes = int(num_classes)

    def gradients(self, logits, labels):
        raise NotImplementedError("the B200 runtime implements the forward path only")

    def loss(self, probs, labels):
        probs = as_device(probs, np.float32)
        V = probs.shape[-1]
        rows = probs.size // V
        y = as_token_ids(np.asarray(labels.get() if isinstance(labels, DeviceArray) else labels).reshape(rows))
        acc = DeviceArray((16,), np.uint8)
        check(lib.tlnn_memset(backend.ctx(), acc.ptr, 0, 16))
        check(lib.tlnn_eval_batch_fwd(backend.ctx(), probs.ptr, V, y.ptr, _ids_code(y), rows, V, acc.ptr, acc.ptr + 8))
        return float(acc.get()[:8].view(np.float64)[0])

    def num_samples(self, labels):
        return int(np.prod(np.shape(labels)))


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

    def predict_logits(self, input, comm=None):
        """Same result as ``predict`` for the GPT and the ViT recipes, as one fused library call (no per-layer outputs
        kept; a repeated call on the same buffers replays a captured CUDA graph).
        With ``comm`` every rank runs its slice of the batch rows and the logits are all-gathered (see
        ``predict_tokens``); for large vocabularies prefer gathering tokens."""
        if comm is not None and comm.world > 1:
            from .comm import sharded_rows
            return sharded_rows(comm, len(input), lambda lo, hi: self.predict_logits(_rows(input, lo, hi)),
                                comm.allgather_logits)
        vit = ViTPlan.match(self.layers)
        if vit is not None:
            self._check_eval()
            img = as_device(input, np.float32)
            want = (vit.front.channels, vit.front.height, vit.front.width)
            if img.ndim != 4 or img.shape[1:] != want:
                raise ValueError(f"cannot reshape array of shape {img.shape} into patches of a {want} image")
            m, keep, n_out = vit.model()
            scores = DeviceArray((img.shape[0], n_out), np.float32)
            check(lib.tlnn_vit_forward(backend.ctx(), C.byref(m), img.ptr, img.shape[0], scores.ptr))
            return scores
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

    def predict_tokens(self, input, comm=None):
        """arg-max of ``predict(input)`` over the last axis, int32 on the device.

        With ``comm`` (a ``torchless_nn_b200.comm.Communicator``) the call is collective: every rank passes the same
        global batch, runs the contiguous slice of rows it owns and receives the tokens of the whole batch, gathered
        over NCCL in row order."""
        if comm is not None and comm.world > 1:
            from .comm import sharded_rows
            return sharded_rows(comm, len(input), lambda lo, hi: self.predict_tokens(_rows(input, lo, hi)),
                                comm.allgather_tokens)
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
        return argmax_last(self.predict_logits(input))

    def evaluate(self, test_data, test_labels, criterion=None, batch_size=64, prefetch=True):
        """network.py:145-160: mean cross-entropy and accuracy of ``predict`` over ``test_data`` in batches.  The
        arg-max, its comparison with the labels and the loss terms stay on the device; two numbers come back at the
        end.  ``criterion`` is accepted for signature compatibility (its ``loss`` is what is computed).  With
        ``prefetch`` the next batch is copied from pinned host memory on a second stream while the current one is
        computed (the reference uploads each batch synchronously, network.py:152)."""
        from .host_feed import HostFeed
        self.set_eval(True)
        n = len(test_data)
        labels = np.asarray(test_labels)
        acc = DeviceArray((16,), np.uint8)
        check(lib.tlnn_memset(backend.ctx(), acc.ptr, 0, 16))
        first = np.asarray(test_data[0:1])
        is_ids = np.issubdtype(first.dtype, np.integer)
        in_dtype = (first.dtype if first.dtype in (np.dtype(np.int32), np.dtype(np.uint8), np.dtype(np.int64)) else np.dtype(np.int64)) \
            if is_ids else np.dtype(np.float32)

        def plain():
            for i in range(0, n, batch_size):
                hi = min(i + batch_size, n)
                x = np.asarray(test_data[i:hi], dtype=in_dtype)
                yield i, hi, (as_token_ids(x) if is_ids else as_device(x))

        feed = HostFeed(int(np.prod(first.shape[1:])) * in_dtype.itemsize * batch_size) if (prefetch and n > 0) else None
        source = feed.batches(test_data, batch_size, in_dtype) if feed else plain()
        try:
            for i, hi, x in source:
                self._evaluate_batch(x, labels[i:hi], acc)
        finally:
            if feed:
                backend.synchronize()
                feed.close()
        host = acc.get()
        total = float(np.prod(labels.shape))
        return float(host[:8].view(np.float64)[0]) / total, float(host[8:].view(np.int64)[0]) / total

    def _evaluate_batch(self, x, batch_labels, acc):
        """One batch of ``evaluate``: forward, then loss terms and correct arg-max count added on the device."""
        y_hat = self.predict(x)
        V = y_hat.shape[-1]
        rows = y_hat.size // V
        y = as_token_ids(np.ascontiguousarray(batch_labels).reshape(rows))
        check(lib.tlnn_eval_batch_fwd(backend.ctx(), y_hat.ptr, V, y.ptr, _ids_code(y), rows, V, acc.ptr, acc.ptr + 8))

    def generate(self, seed_tokens, length: int, uniforms=None, seed=None, use_cache: bool = True):
        """The notebook's ``GPT.generate`` (demo.ipynb:1520-1535) for every row of ``seed_tokens``: each step crops
        the tokens to the last ``context_length`` (the sliding window of demo.ipynb:1528, positions restart at the
        crop), runs the model, takes the probabilities of the last position and draws the next token as
        ``random.choice(arange(V), p=probs)`` does on the NumPy runtime: the first index whose normalised prefix sum
        exceeds a uniform number.  ``uniforms`` (length, B) supplies those numbers; by default they come from
        ``numpy.random.default_rng(seed)``.  The model's output must be probabilities (a trailing ``SoftMax``), as in
        the notebook; a model that ends in logits gets ``SoftMax()`` applied.  Returns (B, T0 + length) int32 on the
        host.

        Steps that need no crop run on the per-layer KV cache (``tlnn_decode_run_sampled``; ``use_cache=False`` forces
        the window path); once the window slides, positions restart at the crop, the cache no longer applies and every
        step re-runs the window like the reference, with only the last position going through the row-wise tail of the
        model (final LayerNorm, head, SoftMax): B x V probabilities per step instead of B x T x V."""
        from .activations import SoftMax
        self._check_eval()
        tokens = np.asarray(as_token_ids(seed_tokens).get()).astype(np.int32)
        if tokens.ndim != 2 or tokens.shape[1] < 1:
            raise ValueError("generate needs a (B, T0 >= 1) array of token ids")
        B = tokens.shape[0]
        front = self.layers[0]
        if not isinstance(front, GPTEmbedFront):
            raise ValueError("generate needs a model that starts with GPTEmbedFront")
        context = front.context_length
        if uniforms is None:
            uniforms = np.random.default_rng(seed).random((length, B))
        uniforms = np.ascontiguousarray(np.asarray(uniforms, dtype=np.float64).reshape(length, B))
        # the row-wise tail starts after the last attention block
        split = max(i for i, l in enumerate(self.layers) if isinstance(l, TransformerBlock)) + 1 \
            if any(isinstance(l, TransformerBlock) for l in self.layers) else 1
        body, tail = self.layers[:split], self.layers[split:]
        ends_in_probs = bool(tail) and isinstance(tail[-1], SoftMax)
        extra = None if ends_in_probs else SoftMax()
        u_dev = DeviceArray((B * 8,), np.uint8)          # B doubles (the device array type has no float64)
        picked = DeviceArray((B,), np.int32)
        first_step = 0
        # While prompt + continuation fit the context nothing is cropped, so the per-layer KV cache gives the same
        # tokens without re-running the window: those steps go through the decoder (one CUDA graph replay each).
        core = self.layers[:-1] if ends_in_probs else self.layers
        plan = GPTPlan.match(core) if use_cache else None
        cached = min(length, context - tokens.shape[1]) if plan is not None else 0
        if plan is not None and plan.blocks:
            ab = plan.blocks[0].attn_block
            if ab.embedding_dim // ab.num_heads not in (32, 64, 128):      # head sizes of the decode attention kernel
                cached = 0
        if cached >= 1:
            temperature = float(tail[-1].temperature) if ends_in_probs else 1.0
            m, keep, V = plan.model()
            ids = as_token_ids(tokens)
            T0 = tokens.shape[1]
            first = DeviceArray((B,), np.int32)
            dec = C.c_void_p()
            check(lib.tlnn_decode_begin(backend.ctx(), C.byref(m), ids.ptr, _ids_code(ids), B, T0, T0 + cached,
                                        first.ptr, C.byref(dec)))
            try:
                check(lib.tlnn_decode_first_sampled(dec, temperature, uniforms[0].ctypes.data, first.ptr))
                new = [first.get().reshape(B, 1)]
                if cached > 1:
                    rest = DeviceArray((B, cached - 1), np.int32)
                    check(lib.tlnn_decode_run_sampled(dec, first.ptr, cached - 1, temperature,
                                                      uniforms[1:cached].ctypes.data, rest.ptr))
                    new.append(rest.get())
            finally:
                lib.tlnn_decode_end(dec)
            tokens = np.concatenate([tokens] + [n.astype(np.int32) for n in new], axis=1)
            first_step = cached
        for step in range(first_step, length):
            window = tokens[:, max(0, tokens.shape[1] - context):]
            x = as_token_ids(window)
            for layer in body:
                x = layer.forward(x)
            T, d = x.shape[1], x.shape[2]
            last = x[:, T - 1:T, :] if T > 1 else x
            for layer in tail:
                last = layer.forward(last)
            if extra is not None:
                last = extra.forward(last)
            V = last.shape[-1]
            check(lib.tlnn_h2d(backend.ctx(), u_dev.ptr, uniforms[step].ctypes.data, uniforms[step].nbytes))
            check(lib.tlnn_sample_fwd(backend.ctx(), last.ptr, V, u_dev.ptr, picked.ptr, B, V))
            tokens = np.concatenate([tokens, picked.get().reshape(B, 1).astype(np.int32)], axis=1)
        return tokens

    def _last_position(self, window):
        """Output of the model at the last position of every row of ``window`` (B, T): the blocks run on the whole
        window, the row-wise tail (final LayerNorm, head, ...) on the last position only."""
        split = max((i for i, l in enumerate(self.layers) if isinstance(l, TransformerBlock)), default=0) + 1
        x = as_token_ids(window)
        for layer in self.layers[:split]:
            x = layer.forward(x)
        T = x.shape[1]
        last = x[:, T - 1:T, :] if T > 1 else x
        for layer in self.layers[split:]:
            last = layer.forward(last)
        return last

    def generate_greedy(self, prompts, new_tokens: int, comm=None):
        """Greedy continuation of every prompt row by ``new_tokens`` tokens; returns (B, T0 + new_tokens) int32 on
        the device.  While prompt plus continuation fit the context the steps run on the per-layer KV cache (one CUDA
        graph replay per token).  Beyond it the notebook's sliding window applies (demo.ipynb:1528): the tokens are
        cropped to the last ``context_length``, positions restart at the crop, and every step re-runs the window as
        the reference does, with the arg-max of the last position appended.

        With ``comm`` the call is collective: every rank passes the same prompts, decodes the rows it owns on its own
        cache and receives all rows, gathered once at the end."""
        if comm is not None and comm.world > 1:
            from .comm import sharded_rows
            return sharded_rows(comm, len(prompts), lambda lo, hi: self.generate_greedy(_rows(prompts, lo, hi), new_tokens),
                                comm.allgather_tokens)
        plan = GPTPlan.match(self.layers)
        if plan is None:
            raise ValueError("generate_greedy needs the GPT layer recipe")
        self._check_eval()
        ids = as_token_ids(prompts)
        B, T0 = ids.shape
        if new_tokens < 1:
            raise ValueError("new_tokens must be positive")
        if T0 < 1:
            raise ValueError("generate_greedy needs prompts of at least one token")
        context = plan.front.context_length
        tokens = ids.get().astype(np.int32)
        cached = max(0, min(new_tokens, context - T0))
        if cached >= 1:
            m, keep, V = plan.model()
            first = DeviceArray((B,), np.int32)
            dec = C.c_void_p()
            check(lib.tlnn_decode_begin(backend.ctx(), C.byref(m), ids.ptr, _ids_code(ids), B, T0, T0 + cached,
                                        first.ptr, C.byref(dec)))
            try:
                new = [first.get()[:, None]]
                if cached > 1:
                    rest = DeviceArray((B, cached - 1), np.int32)
                    check(lib.tlnn_decode_run(dec, first.ptr, cached - 1, rest.ptr))
                    new.append(rest.get())
            finally:
                lib.tlnn_decode_end(dec)
            tokens = np.concatenate([tokens] + [n.astype(np.int32) for n in new], axis=1)
        for _ in range(cached, new_tokens):
            window = tokens[:, max(0, tokens.shape[1] - context):]
            nxt = argmax_last(self._last_position(window)).get().reshape(B, 1)
            tokens = np.concatenate([tokens, nxt.astype(np.int32)], axis=1)
        return DeviceArray.from_numpy(tokens)
