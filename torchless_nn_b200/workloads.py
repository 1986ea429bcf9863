"""Model recipes, canonical seeded weights and synthetic inputs for the five
benchmark configurations of the transformer forward path.

Nothing here touches a GPU.  The same functions feed the CUDA engine, the CPU
oracle and the script that generates the golden fixtures, so that all three
see identical weights and inputs.

Parameter order follows the reference library's own registration order, so a
flat list produced here can be written straight into the ``parameters`` lists
of a reference ``Network``:

* ``GPTEmbedFront.parameters`` = [positional table, token table]
  (transformer_adapters.py:137-143),
* ``TransformerBlock.parameters`` = [ln1 gamma, ln1 beta, Wqkv, bqkv, Wo, bo,
  ln2 gamma, ln2 beta, W1, b1, W2, b2] (layers.py:458),
* ``LayerNorm.parameters`` = [gamma, beta] (layers.py:403-407),
* ``Dense.parameters`` / ``VitMLPHead.parameters`` = [W, b]
  (layers.py:200-204, transformer_adapters.py:81-87),
* ``VitProjector.parameters`` = [projection, cls/register tokens, positional
  embeddings] (transformer_adapters.py:26-32),
* ``GPTEmbedBack`` owns no parameter of its own: it aliases the token table
  (transformer_adapters.py:169-172).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass(frozen=True)
class GPTSpec:
    """Decoder-only transformer: embedding, L pre-LN blocks, final LN, head."""
    name: str
    vocab: int
    context: int
    d_model: int
    heads: int
    layers: int
    tied_head: bool          # True: GPTEmbedBack (x @ table.T); False: Dense(d, vocab)
    precision: str           # "tf32" or "bf16"
    batch: int
    seq_len: int
    input_seed: int
    input_dist: str          # "uniform" or "zipf"
    kind: str = field(default="gpt", init=False)

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads

    def n_params(self) -> int:
        d, L, V = self.d_model, self.layers, self.vocab
        per_block = 2 * d + (3 * d * d + 3 * d) + (d * d + d) + 2 * d + (4 * d * d + 4 * d) + (4 * d * d + d)
        n = self.context * d + V * d + L * per_block + 2 * d
        if not self.tied_head:
            n += d * V + V
        return n

    def flops_per_token(self, causal: bool = True, seq_len: int | None = None) -> float:
        """Algorithmic multiply-add work (2 FLOP each) of one token's forward:
        24 d^2 per layer for the four weight GEMMs, 2 (T+1) d per layer for
        causal attention (the mean of 4 (t+1) d over positions), 2 d V for the
        head.  Softmax, LayerNorm and GeLU are not counted."""
        T = self.seq_len if seq_len is None else seq_len
        d, L, V = self.d_model, self.layers, self.vocab
        attn = 2.0 * (T + 1) * d if causal else 4.0 * T * d
        return L * (24.0 * d * d + attn) + 2.0 * d * V


@dataclass(frozen=True)
class ViTSpec:
    """Encoder-only vision transformer on C x H x W images."""
    name: str
    image: tuple          # (C, H, W)
    patch: tuple          # (ph, pw)
    d_model: int
    heads: int
    layers: int
    classes: int
    precision: str
    batch: int
    input_seed: int
    registers: int = 0
    kind: str = field(default="vit", init=False)

    @property
    def n_patches(self) -> int:
        return (self.image[1] // self.patch[0]) * (self.image[2] // self.patch[1])

    @property
    def tokens(self) -> int:
        return 1 + self.registers + self.n_patches

    @property
    def token_dim(self) -> int:
        return self.patch[0] * self.patch[1] * self.image[0]

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads

    def flops_per_image(self) -> float:
        d, L, T = self.d_model, self.layers, self.tokens
        return (self.n_patches * 2.0 * self.token_dim * d
                + T * L * (24.0 * d * d + 4.0 * T * d) + 2.0 * d * self.classes)


CONFIGS = {
    # char-level GPT, FP32 / TF32, untied Dense head
    "c1": GPTSpec("c1", vocab=65, context=128, d_model=128, heads=4, layers=4, tied_head=False,
                  precision="tf32", batch=32, seq_len=128, input_seed=1, input_dist="uniform"),
    # ViT on 32x32x3 images, 4x4 patches
    "c2": ViTSpec("c2", image=(3, 32, 32), patch=(4, 4), d_model=192, heads=6, layers=6, classes=10,
                  precision="tf32", batch=256, input_seed=2),
    # GPT-2-small shape, BF16 weights, FP32 accumulation, prefill
    "c3": GPTSpec("c3", vocab=50257, context=1024, d_model=768, heads=12, layers=12, tied_head=True,
                  precision="bf16", batch=16, seq_len=1024, input_seed=3, input_dist="zipf"),
    # greedy decode on the c3 model: 64 prompts of 128 tokens, 256 new tokens each
    "c4": GPTSpec("c4", vocab=50257, context=1024, d_model=768, heads=12, layers=12, tied_head=True,
                  precision="bf16", batch=64, seq_len=128, input_seed=4, input_dist="zipf"),
    # GPT-2-medium shape prefill, global batch 64 x 2048, sharded by batch over the GPUs
    "c5": GPTSpec("c5", vocab=50257, context=2048, d_model=1024, heads=16, layers=24, tied_head=True,
                  precision="bf16", batch=64, seq_len=2048, input_seed=5, input_dist="zipf"),
}
C4_NEW_TOKENS = 256

WEIGHT_SEED = 0
WEIGHT_STD = np.float32(0.02)


def param_shapes(spec) -> list[tuple[str, tuple]]:
    """(name, shape) of every distinct parameter in canonical order."""
    out: list[tuple[str, tuple]] = []
    d = spec.d_model
    if spec.kind == "gpt":
        out.append(("pos_table", (spec.context, d)))
        out.append(("tok_table", (spec.vocab, d)))
    else:
        out.append(("projection", (spec.token_dim, d)))
        out.append(("cls_reg_tokens", (1 + spec.registers, d)))
        out.append(("vit_pos", (spec.tokens, d)))
    for i in range(spec.layers):
        p = f"block{i}."
        out += [(p + "ln1_gamma", (d,)), (p + "ln1_beta", (d,)),
                (p + "wqkv", (d, 3 * d)), (p + "bqkv", (3 * d,)),
                (p + "wo", (d, d)), (p + "bo", (d,)),
                (p + "ln2_gamma", (d,)), (p + "ln2_beta", (d,)),
                (p + "w1", (d, 4 * d)), (p + "b1", (4 * d,)),
                (p + "w2", (4 * d, d)), (p + "b2", (d,))]
    out += [("lnf_gamma", (d,)), ("lnf_beta", (d,))]
    if spec.kind == "gpt":
        if not spec.tied_head:
            out += [("head_w", (d, spec.vocab)), ("head_b", (spec.vocab,))]
    else:
        out += [("head_w", (d, spec.classes)), ("head_b", (spec.classes,))]
    return out


def seeded_params(spec, seed: int = WEIGHT_SEED) -> list[np.ndarray]:
    """Canonical weights: one ``default_rng(seed)`` stream walked in parameter
    order; every parameter with two or more dimensions is N(0, 0.02) in
    float32, one-dimensional parameters keep the constructor values of the
    reference (biases and LayerNorm beta 0, LayerNorm gamma 1)."""
    rng = np.random.default_rng(seed)
    params = []
    for name, shape in param_shapes(spec):
        if len(shape) >= 2:
            params.append(rng.standard_normal(shape, dtype=np.float32) * WEIGHT_STD)
        elif name.endswith("gamma"):
            params.append(np.ones(shape, dtype=np.float32))
        else:
            params.append(np.zeros(shape, dtype=np.float32))
    return params


def zipf_probabilities(vocab: int, s: float = 1.1) -> np.ndarray:
    """Bounded Zipf law over token ids: p[k] proportional to (k+1)^-s."""
    p = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    return p / p.sum()


def token_ids(vocab: int, shape: tuple, seed: int, dist: str) -> np.ndarray:
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        return rng.integers(0, vocab, size=shape).astype(np.int32)
    if dist == "zipf":
        return rng.choice(vocab, size=shape, p=zipf_probabilities(vocab)).astype(np.int32)
    raise ValueError(f"unknown token distribution {dist!r}")


def images(shape: tuple, seed: int) -> np.ndarray:
    """Pixels uniform in [0,1), normalised per channel with mean 0.5, std 0.25."""
    x = np.random.default_rng(seed).random(shape, dtype=np.float32)
    return ((x - np.float32(0.5)) / np.float32(0.25)).astype(np.float32)


def make_inputs(spec, batch: int | None = None) -> np.ndarray:
    """The configuration's input batch (or its first ``batch`` rows: the
    generators draw row-major, so a prefix of rows is generated by drawing the
    full shape and slicing)."""
    if spec.kind == "gpt":
        x = token_ids(spec.vocab, (spec.batch, spec.seq_len), spec.input_seed, spec.input_dist)
    else:
        x = images((spec.batch,) + tuple(spec.image), spec.input_seed)
    return x if batch is None else x[:batch]


def shard_rows(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous batch slice [lo, hi) owned by ``rank`` of ``world``; the
    first ``n_rows % world`` ranks take one extra row."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)
