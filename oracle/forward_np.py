"""CPU oracle: a NumPy restatement of the reference library's transformer
forward pass (luke-skynet/torchless-nn, ``XP_RUNTIME=CPU``).

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the tests, the smoke
check and the benchmark's CPU-baseline legs may import it; the CUDA engine
never does.

Pinning: the reference ships no tests or golden vectors for this path, so the
restatement is pinned against the reference's own code executed on the CPU:
``tests/golden/make_golden.py`` imports the reference, runs ``Network.predict``
on canonical seeded weights and inputs, stores the results as fixtures, and
``tests/test_oracle_golden.py`` checks every function here against them.

Every function works on float32 C-contiguous arrays, performs the same array
operations in the same order as the reference line it cites (same temporaries,
same broadcasting, same non-contiguous views), so that its rounding behaviour
and its CPU cost are those of the reference's NumPy path.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------- activations
def gelu_tanh(x):
    """activations.py:24-28 - 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))."""
    t = np.tanh((2 / np.pi) ** 0.5 * (x + 0.044715 * x ** 3))
    return 0.5 * x * (1 + t)


def silu_tanh(x):
    """activations.py:41-45 - x (1 + tanh(x/2)) / 2."""
    return x * ((1 + np.tanh(x / 2)) / 2)


def relu(x):
    """activations.py:10-13."""
    return np.maximum(x, 0)


ACTIVATIONS = {"gelu": gelu_tanh, "silu": silu_tanh, "relu": relu}


def softmax_t(x, temperature=F32(1.0)):
    """activations.py:57-64 - max-subtracted softmax over the last axis with a
    temperature divisor applied after the subtraction."""
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp((x - m) / temperature)
    return e / np.sum(e, axis=-1, keepdims=True)


# --------------------------------------------------------------------------- layers
def layer_norm(x, gamma, beta, eps=F32(1e-5)):
    """layers.py:415-428 - mean, biased variance, (var + eps) ** 0.5,
    centre / std, then gamma * normed + beta."""
    mean = np.mean(x, axis=-1, keepdims=True)
    var = np.var(x, axis=-1, keepdims=True)
    centred = x - mean
    std = (var + eps) ** F32(0.5)
    return gamma * (centred / std) + beta


def causal_mask(context):
    """layers.py:254-256 - 0 on and below the diagonal, -1e9 above it."""
    m = np.tril(np.ones((context, context)))
    return np.where(m == 0, -1e9, 0.0).astype(F32, copy=False)


def attention(x, wqkv, bqkv, wo, bo, heads, mask=None):
    """layers.py:281-307 - fused QKV projection, split into heads (K kept
    transposed), scores divided by sqrt(head_dim), additive mask, softmax over
    keys, weighted sum of V, merge heads, output projection."""
    B, T, C = x.shape
    hd = C // heads
    qkv = x @ wqkv + bqkv
    q, k, v = np.split(qkv, 3, axis=2)
    q = q.reshape((B, T, heads, hd)).transpose(0, 2, 1, 3)
    k_t = k.reshape((B, T, heads, hd)).transpose(0, 2, 3, 1)
    v = v.reshape((B, T, heads, hd)).transpose(0, 2, 1, 3)
    scores = (q @ k_t) / F32(hd ** 0.5)
    if mask is not None:
        scores += mask[:T, :T]
    m = np.max(scores, axis=-1, keepdims=True)
    e = np.exp(scores - m)
    p = e / np.sum(e, axis=-1, keepdims=True)
    merged = (p @ v).transpose(0, 2, 1, 3).reshape(B, T, C)
    return merged @ wo + bo


def feed_forward(x, w1, b1, w2, b2, act="gelu"):
    """layers.py:369-375 - act(x W1 + b1) W2 + b2, hidden width 4 d."""
    return ACTIVATIONS[act](x @ w1 + b1) @ w2 + b2


def block(x, p, heads, mask=None, act="gelu"):
    """layers.py:463-467 - pre-LN residual block.  ``p`` holds the block's
    twelve tensors in registration order (layers.py:458)."""
    g1, be1, wqkv, bqkv, wo, bo, g2, be2, w1, b1, w2, b2 = p
    y = x + attention(layer_norm(x, g1, be1), wqkv, bqkv, wo, bo, heads, mask)
    return y + feed_forward(layer_norm(y, g2, be2), w1, b1, w2, b2, act)


def dense(x, w, b):
    """layers.py:206-209 - x @ W + b with W stored (in, out)."""
    return x @ w + b


def embed_front(ids, tok_table, pos_table):
    """transformer_adapters.py:148-153 - table[ids] + pos[:T]."""
    return tok_table[ids] + pos_table[:ids.shape[1], :]


def sinusoidal_table(context, d):
    """transformer_adapters.py:128-135 - pos / 10000^(2 (i // 2) / d), sine on
    even columns and cosine on odd columns, computed in float64 then cast."""
    pos = np.arange(context)[:, None]
    i = np.arange(d)[None, :]
    t = pos / 10000 ** (2 * (i // 2) / d)
    t[:, 0::2] = np.sin(t[:, 0::2])
    t[:, 1::2] = np.cos(t[:, 1::2])
    return t.astype(F32, copy=False)


def tied_logits(x, tok_table):
    """transformer_adapters.py:174-177 - x @ table.T (no bias)."""
    return x @ tok_table.transpose()


def vit_project(img, projection, cls_reg, pos, patch):
    """transformer_adapters.py:34-55 - cut the image into patches whose feature
    order is (row in patch, column in patch, channel), project, put the class
    and register tokens in front, add the positional embeddings."""
    B, C, H, W = img.shape
    ph, pw = H // patch[0], W // patch[1]
    r = img.reshape((B, C, ph, patch[0], pw, patch[1]))
    tokens = r.transpose(0, 2, 4, 3, 5, 1).reshape(B, ph * pw, patch[0] * patch[1] * C)
    emb = tokens @ projection
    emb = np.concatenate([np.tile(cls_reg, (B, 1, 1)), emb], axis=1)
    return emb + pos


def vit_head(x, w, b):
    """transformer_adapters.py:89-95 - linear layer on the class token."""
    return x[:, 0, :] @ w + b


# --------------------------------------------------------------------------- whole models
def _blocks(params, start, n_layers):
    return [params[start + 12 * i: start + 12 * (i + 1)] for i in range(n_layers)]


def gpt_forward(spec, params, ids, act="gelu", upto=None):
    """Network.predict (network.py:33-39) on the GPT recipe: GPTEmbedFront,
    L decoder blocks, LayerNorm, then GPTEmbedBack (tied) or Dense (untied).
    ``params`` is the flat canonical list.  Returns float32 logits (B, T, V).
    ``upto='hidden'`` returns the final-LayerNorm output instead."""
    pos, tok = params[0], params[1]
    x = embed_front(ids, tok, pos)
    mask = causal_mask(spec.context)
    for p in _blocks(params, 2, spec.layers):
        x = block(x, p, spec.heads, mask, act)
    k = 2 + 12 * spec.layers
    x = layer_norm(x, params[k], params[k + 1])
    if upto == "hidden":
        return x
    if spec.tied_head:
        return tied_logits(x, tok)
    return dense(x, params[k + 2], params[k + 3])


def vit_forward(spec, params, img, act="gelu"):
    """Network.predict on the ViT recipe: VitProjector, L encoder blocks (no
    mask), LayerNorm, VitMLPHead.  Returns float32 logits (B, classes)."""
    x = vit_project(img, params[0], params[1], params[2], spec.patch)
    for p in _blocks(params, 3, spec.layers):
        x = block(x, p, spec.heads, None, act)
    k = 3 + 12 * spec.layers
    x = layer_norm(x, params[k], params[k + 1])
    return vit_head(x, params[k + 2], params[k + 3])


def forward(spec, params, x, **kw):
    return gpt_forward(spec, params, x, **kw) if spec.kind == "gpt" else vit_forward(spec, params, x, **kw)


def greedy_decode(spec, params, prompts, new_tokens):
    """Greedy form of the notebook's generation loop (demo.ipynb:1520-1535):
    crop to the last ``context`` tokens, run the whole window through the model,
    take the last position's argmax, append.  No cache - this is the
    reference's algorithm and costs one full forward per token."""
    tokens = np.array(prompts)
    for _ in range(new_tokens):
        window = tokens[:, max(0, tokens.shape[1] - spec.context):]
        nxt = np.argmax(gpt_forward(spec, params, window)[:, -1], axis=-1)
        tokens = np.concatenate((tokens, nxt[:, None].astype(tokens.dtype)), axis=1)
    return tokens


# --------------------------------------------------------------------------- comparison rules
def top2(logits):
    """Per row: (argmax, top value, runner-up value)."""
    a = np.argmax(logits, axis=-1)
    flat = logits.reshape(-1, logits.shape[-1])
    top = np.take_along_axis(flat, a.reshape(-1, 1), axis=1)[:, 0]
    masked = flat.copy()
    masked[np.arange(flat.shape[0]), a.reshape(-1)] = -np.inf
    second = masked.max(axis=1)
    return a, top.reshape(a.shape), second.reshape(a.shape)


def tokens_match(got, ref_argmax, ref_top, ref_second, tol_abs):
    """Greedy-token rule: tokens must be identical except at positions where
    the reference's own top-2 logits differ by less than the tolerance."""
    got = np.asarray(got).reshape(ref_argmax.shape)
    differ = got != ref_argmax
    excused = (ref_top - ref_second) < tol_abs
    return bool(np.all(~differ | excused)), int(differ.sum()), int((differ & ~excused).sum())


def choice_index(probs, u):
    """numpy.random.RandomState.choice(arange(V), p=probs) for a given uniform number u (the NumPy runtime of
    demo.ipynb:1530): cdf = cumsum(p) in double, cdf /= cdf[-1], first index with cdf > u."""
    cdf = np.cumsum(np.asarray(probs, dtype=np.float64))
    cdf /= cdf[-1]
    return int(min(np.searchsorted(cdf, u, side="right"), len(cdf) - 1))


def sample_generate(forward_probs, seed_tokens, length, context, uniforms):
    """demo.ipynb:1520-1535 (GPT.generate) for B rows: crop to the last ``context`` tokens, run the model
    (``forward_probs(ids) -> (B, T, V)`` probabilities), draw the next token of every row from the last position.
    Returns (tokens (B, T0 + length), margins (length, B)) where a margin is the distance of the uniform number to
    the nearest boundary of the chosen cell of the cdf: draws with a tiny margin may legitimately differ between two
    implementations whose probabilities differ in the last digits."""
    tokens = np.asarray(seed_tokens).astype(np.int64)
    B = tokens.shape[0]
    margins = np.zeros((length, B))
    for step in range(length):
        window = tokens[:, max(0, tokens.shape[1] - context):]
        probs = forward_probs(window)[:, -1]
        nxt = np.zeros((B, 1), dtype=np.int64)
        for b in range(B):
            cdf = np.cumsum(probs[b].astype(np.float64))
            cdf /= cdf[-1]
            i = choice_index(probs[b], uniforms[step, b])
            lo = cdf[i - 1] if i > 0 else 0.0
            margins[step, b] = min(uniforms[step, b] - lo, cdf[i] - uniforms[step, b])
            nxt[b, 0] = i
        tokens = np.concatenate([tokens, nxt], axis=1)
    return tokens, margins
