"""Generate the golden fixtures in this directory by running the UNMODIFIED
reference library (luke-skynet/torchless-nn) on its NumPy path.

    XP_RUNTIME=CPU python tests/golden/make_golden.py --reference /path/to/torchless-nn [c1 c2 layers c3 c4 c5 ckpt eval]

The reference checkout is only needed to (re)generate fixtures; tests read the
committed ``.npz`` files.  For each configuration the script builds the
reference ``Network`` from the recipe, overwrites its parameters in place with
the canonical seeded weights (``torchless_nn_b200.workloads.seeded_params``),
calls ``set_eval(True)`` and ``predict`` on the canonical inputs, and stores
what the parity tests need.  It also checks the NumPy oracle
(``oracle/forward_np.py``) against the reference's output and records the
largest difference in each fixture (``oracle_max_abs_diff``).

Full logits of the large-vocabulary configurations would be hundreds of MB, so
for those the fixture keeps, per position: the arg-max token, the top and
runner-up logit (needed for the tie rule), and the logits at a fixed sample of
positions x vocabulary columns.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

os.environ["XP_RUNTIME"] = "CPU"
sys.dont_write_bytecode = True

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from torchless_nn_b200 import workloads as wl   # noqa: E402
from oracle import forward_np as onp            # noqa: E402


def load_reference(path):
    sys.path.insert(0, path)
    import network, layers, activations, transformer_adapters  # noqa: F401
    return network, layers, activations, transformer_adapters


def build_reference_net(ref, spec):
    network, layers, activations, ta = ref
    if spec.kind == "gpt":
        tab = ta.GPTEmbeddingTable(spec.vocab, spec.d_model)
        ls = [ta.GPTEmbedFront(tab, spec.context)]
        ls += [layers.TransformerBlock(spec.d_model, spec.context, spec.heads, activations.GeLU, decoder=True)
               for _ in range(spec.layers)]
        ls.append(layers.LayerNorm(spec.d_model))
        ls.append(ta.GPTEmbedBack(tab) if spec.tied_head else layers.Dense(spec.d_model, spec.vocab))
    else:
        ls = [ta.VitProjector(tuple(spec.image), tuple(spec.patch), spec.d_model, spec.registers)]
        ls += [layers.TransformerBlock(spec.d_model, 0, spec.heads, activations.GeLU)
               for _ in range(spec.layers)]
        ls += [layers.LayerNorm(spec.d_model), ta.VitMLPHead(spec.d_model, spec.classes)]
    return network.Network(ls)


def load_seeded(net, params):
    """Write the canonical weights into the reference network in place,
    visiting each distinct array once in registration order."""
    seen, it = set(), iter(params)
    for layer in net.layers:
        for p in layer.parameters:
            if id(p) in seen:
                continue
            seen.add(id(p))
            src = next(it)
            assert p.shape == src.shape, (p.shape, src.shape)
            p[...] = src
    assert next(it, None) is None
    net.set_eval(True)


SAMPLE_POS = 64
SAMPLE_COLS = 256


def sampled(logits2d, seed):
    rng = np.random.default_rng(seed)
    rows = np.sort(rng.choice(logits2d.shape[0], size=min(SAMPLE_POS, logits2d.shape[0]), replace=False))
    # a third of the sampled columns from the head of the Zipf law, the rest anywhere
    head = rng.choice(min(512, logits2d.shape[1]), size=SAMPLE_COLS // 4, replace=False)
    rest = rng.choice(logits2d.shape[1], size=SAMPLE_COLS - SAMPLE_COLS // 4, replace=False)
    cols = np.unique(np.concatenate([head, rest]))
    return rows.astype(np.int32), cols.astype(np.int32), logits2d[np.ix_(rows, cols)].astype(np.float32)


def summarise(logits):
    a, top, second = onp.top2(logits)
    return dict(argmax=a.astype(np.int32), top=top.astype(np.float32), second=second.astype(np.float32),
                max_abs=np.float32(np.abs(logits).max()))


def gen_small(ref, name):
    spec = wl.CONFIGS[name]
    params = wl.seeded_params(spec)
    x = wl.make_inputs(spec)
    net = build_reference_net(ref, spec)
    load_seeded(net, params)
    t0 = time.time()
    y = net.predict(x)
    dt = time.time() - t0
    yo = onp.forward(spec, params, x)
    diff = float(np.abs(y - yo).max())
    out = dict(summarise(y), oracle_max_abs_diff=np.float32(diff), ref_seconds=np.float32(dt))
    if name == "c1":
        out["logits"] = y[:8].astype(np.float32)
        out["embed0"] = net.layers[0].output[:2].astype(np.float32)
        out["block0_out"] = net.layers[1].output[:2].astype(np.float32)
        out["hidden"] = net.layers[-2].output[:2].astype(np.float32)
    else:
        out["logits"] = y.astype(np.float32)
        out["embed0"] = net.layers[0].output[:2].astype(np.float32)
        out["block0_out"] = net.layers[1].output[:2].astype(np.float32)
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print(name, "ref", round(dt, 2), "s  oracle diff", diff, "max|logit|", out["max_abs"])


def gen_large(ref, name, rows):
    """Whole sequences of a large configuration, one at a time (batch rows are independent).  ``rows`` are GLOBAL row
    indices of the configuration's batch: sequence ``s`` of the fixture is global row ``rows[s]`` (stored as
    ``global_rows``), so that every rank of a batch-sharded run owns at least one pinned sequence."""
    spec = wl.CONFIGS[name]
    params = wl.seeded_params(spec)
    x = wl.make_inputs(spec)
    net = build_reference_net(ref, spec)
    load_seeded(net, params)
    out = {}
    diffs, secs = [], []
    for s, r in enumerate(rows):
        t0 = time.time()
        y = net.predict(x[r:r + 1])[0]
        secs.append(time.time() - t0)
        if s == 0:
            yo = onp.gpt_forward(spec, params, x[r:r + 1])[0]
            diffs.append(float(np.abs(y - yo).max()))
        sm = summarise(y)
        pos, cols, vals = sampled(y, seed=1000 + s)
        for k, v in sm.items():
            out[f"seq{s}_{k}"] = v
        out[f"seq{s}_rows"], out[f"seq{s}_cols"], out[f"seq{s}_vals"] = pos, cols, vals
        if s < 2:
            out[f"seq{s}_hidden_rows"] = net.layers[-2].output[0][pos].astype(np.float32)
        print(name, "seq", s, "global row", r, round(secs[-1], 1), "s", "max|logit|", sm["max_abs"], flush=True)
    out["n_seq"] = np.int32(len(rows))
    out["global_rows"] = np.asarray(rows, dtype=np.int32)
    out["oracle_max_abs_diff"] = np.float32(max(diffs))
    out["ref_seconds_per_seq"] = np.float32(np.mean(secs))
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print(name, "oracle diff", max(diffs))


def gen_decode(ref, n_prompts=2, steps=24):
    """Literal stepwise loop of the reference (one full forward per token,
    demo.ipynb:1526-1533, with arg-max in place of sampling) on the first
    prompts of the decode configuration."""
    spec = wl.CONFIGS["c4"]
    params = wl.seeded_params(spec)
    prompts = wl.make_inputs(spec, n_prompts)
    net = build_reference_net(ref, spec)
    load_seeded(net, params)
    tokens = np.array(prompts)
    tops, seconds = [], []
    for _ in range(steps):
        window = tokens[:, max(0, tokens.shape[1] - spec.context):]
        last = net.predict(window)[:, -1]
        a, top, second = onp.top2(last)
        tops.append(top)
        seconds.append(second)
        tokens = np.concatenate((tokens, a[:, None].astype(tokens.dtype)), axis=1)
    last_abs = float(np.abs(last).max())
    tok_oracle = onp.greedy_decode(spec, params, prompts, 4)
    assert np.array_equal(tok_oracle, tokens[:, :prompts.shape[1] + 4])
    np.savez_compressed(os.path.join(HERE, "c4.npz"), tokens=tokens.astype(np.int32),
                        top=np.stack(tops, 1).astype(np.float32), second=np.stack(seconds, 1).astype(np.float32),
                        max_abs=np.float32(last_abs), n_prompts=np.int32(n_prompts), steps=np.int32(steps))
    print("c4 tokens", tokens[:, -steps:])


def gen_layers(ref):
    """Single-layer forwards at small and awkward shapes."""
    network, layers, activations, ta = ref
    rng = np.random.default_rng(7)
    out = {}

    def rnd(*shape, scale=1.0):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)

    # LayerNorm, rows of width 128 / 192 / 768 / 1000
    for d in (128, 192, 768, 1000):
        ln = layers.LayerNorm(d)
        ln.gamma[...] = rnd(d) * 0.1 + 1
        ln.beta[...] = rnd(d) * 0.1
        x = rnd(3, 17, d, scale=2.0) + np.float32(0.5)
        out[f"ln{d}_x"], out[f"ln{d}_g"], out[f"ln{d}_b"] = x, ln.gamma.copy(), ln.beta.copy()
        out[f"ln{d}_y"] = ln.forward(x)
        assert np.abs(out[f"ln{d}_y"] - onp.layer_norm(x, ln.gamma, ln.beta)).max() == 0
    # attention: causal and bidirectional, hd 32 and 64, T = 1, 17, 65, 128
    for tag, d, H, T, dec in (("a", 128, 4, 17, True), ("b", 128, 4, 128, True), ("c", 192, 6, 65, False),
                              ("d", 128, 2, 1, True), ("e", 256, 4, 100, True), ("f", 128, 2, 33, False)):
        at = layers.MultiHeadAttention(d, 128, H, decoder=dec)
        at.qkv_weights[...] = rnd(d, 3 * d, scale=0.08)
        at.qkv_bias[...] = rnd(3 * d, scale=0.05)
        at.out_weights[...] = rnd(d, d, scale=0.08)
        at.out_bias[...] = rnd(d, scale=0.05)
        at.set_eval(True)
        x = rnd(2, T, d)
        y = at.forward(x)
        for k, v in (("x", x), ("wqkv", at.qkv_weights), ("bqkv", at.qkv_bias), ("wo", at.out_weights),
                     ("bo", at.out_bias), ("y", y)):
            out[f"attn_{tag}_{k}"] = np.array(v, dtype=np.float32)
        out[f"attn_{tag}_meta"] = np.array([d, H, T, int(dec)], dtype=np.int32)
        yo = onp.attention(x, at.qkv_weights, at.qkv_bias, at.out_weights, at.out_bias, H,
                           onp.causal_mask(128) if dec else None)
        assert np.abs(y - yo).max() == 0
    # feed-forward with each activation
    for act_name, act_cls in (("gelu", activations.GeLU), ("silu", activations.SiLU), ("relu", activations.ReLU)):
        d = 96
        ff = layers.TransformerFeedForward(d, act_cls)
        ff.weights1[...] = rnd(d, 4 * d, scale=0.1)
        ff.bias1[...] = rnd(4 * d, scale=0.1)
        ff.weights2[...] = rnd(4 * d, d, scale=0.1)
        ff.bias2[...] = rnd(d, scale=0.1)
        ff.set_eval(True)
        x = rnd(2, 19, d)
        y = ff.forward(x)
        for k, v in (("x", x), ("w1", ff.weights1), ("b1", ff.bias1), ("w2", ff.weights2), ("b2", ff.bias2), ("y", y)):
            out[f"ffn_{act_name}_{k}"] = np.array(v, dtype=np.float32)
        assert np.abs(y - onp.feed_forward(x, ff.weights1, ff.bias1, ff.weights2, ff.bias2, act_name)).max() == 0
    # activations on their own, and softmax with temperatures
    x = rnd(5, 131, scale=3.0)
    out["act_x"] = x
    out["act_gelu"] = activations.GeLU().forward(x)
    out["act_silu"] = activations.SiLU().forward(x)
    out["act_relu"] = activations.ReLU().forward(x)
    for i, (V, temp) in enumerate(((65, 1.0), (50257, 0.7), (10, 2.0), (1001, 1.0))):
        x = rnd(3, V, scale=2.0)
        sm = activations.SoftMax(np.float32(temp))
        out[f"softmax{i}_x"], out[f"softmax{i}_t"], out[f"softmax{i}_y"] = x, np.float32(temp), sm.forward(x)
        assert np.abs(out[f"softmax{i}_y"] - onp.softmax_t(x, np.float32(temp))).max() == 0
    # Dense on 2-D and 3-D inputs
    dn = layers.Dense(40, 65)
    dn.weights[...] = rnd(40, 65, scale=0.2)
    dn.bias[...] = rnd(65, scale=0.2)
    x2, x3 = rnd(7, 40), rnd(2, 5, 40)
    out.update(dense_w=dn.weights.copy(), dense_b=dn.bias.copy(), dense_x2=x2, dense_y2=dn.forward(x2),
               dense_x3=x3, dense_y3=dn.forward(x3))
    # GPT embedding front (learned and sinusoidal) and tied head
    tab = ta.GPTEmbeddingTable(97, 48)
    tab.table[...] = rnd(97, 48)
    fr = ta.GPTEmbedFront(tab, 32)
    fr.pos_embedding_table[...] = rnd(32, 48)
    ids = rng.integers(0, 97, size=(3, 21))
    out.update(emb_table=tab.table.copy(), emb_pos=fr.pos_embedding_table.copy(), emb_ids=ids.astype(np.int64),
               emb_y=fr.forward(ids), emb_y_u8=fr.forward(ids.astype(np.uint8)))
    fs = ta.GPTEmbedFront(tab, 32, positional_embedding="sinusoidal")
    out.update(emb_sin_pos=fs.pos_embedding_table.copy(), emb_sin_y=fs.forward(ids))
    assert np.array_equal(fs.pos_embedding_table, onp.sinusoidal_table(32, 48))
    bk = ta.GPTEmbedBack(tab)
    xb = rnd(3, 21, 48)
    out.update(back_x=xb, back_y=bk.forward(xb))
    # ViT projector with and without register tokens, and the class-token head
    for tag, regs in (("r0", 0), ("r2", 2)):
        vp = ta.VitProjector((3, 16, 24), (4, 4), 64, regs)
        vp.projection[...] = rnd(48, 64, scale=0.1)
        vp.cls_reg_tokens[...] = rnd(1 + regs, 64, scale=0.1)
        vp.positional_embeddings[...] = rnd(1 + regs + 24, 64, scale=0.1)
        img = rnd(3, 3, 16, 24)
        out.update({f"vitp_{tag}_proj": vp.projection.copy(), f"vitp_{tag}_cls": vp.cls_reg_tokens.copy(),
                    f"vitp_{tag}_pos": vp.positional_embeddings.copy(), f"vitp_{tag}_img": img,
                    f"vitp_{tag}_y": vp.forward(img)})
        assert np.abs(out[f"vitp_{tag}_y"] - onp.vit_project(img, vp.projection, vp.cls_reg_tokens,
                                                             vp.positional_embeddings, (4, 4))).max() == 0
    vh = ta.VitMLPHead(64, 10)
    vh.weights[...] = rnd(64, 10, scale=0.2)
    vh.bias[...] = rnd(10, scale=0.2)
    xh = rnd(5, 25, 64)
    out.update(vith_w=vh.weights.copy(), vith_b=vh.bias.copy(), vith_x=xh, vith_y=vh.forward(xh))
    # one whole block with SiLU, bidirectional (the notebook's encoder variant)
    blk = layers.TransformerBlock(64, 0, 2, activations.SiLU)
    ps = []
    for p in blk.parameters:
        p[...] = rnd(*p.shape, scale=0.1) + (1 if (p.ndim == 1 and np.all(p == 1)) else 0)
        ps.append(p.copy())
    blk.set_eval(True)
    xb = rnd(2, 11, 64)
    yb = blk.forward(xb)
    for i, p in enumerate(ps):
        out[f"block_silu_p{i}"] = p
    out.update(block_silu_x=xb, block_silu_y=yb)
    assert np.abs(yb - onp.block(xb, ps, 2, None, "silu")).max() == 0
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **out)
    print("layers:", len(out), "arrays")


def notebook_helpers(reference_path, ref):
    """``save_weights`` / ``load_weights`` as the reference's notebook defines them, executed from the checkout."""
    import json
    import pickle
    nb = json.load(open(os.path.join(reference_path, "demo.ipynb")))
    ns = {"pickle": pickle, "xp": np, "np": np}
    for cell in nb["cells"]:
        src = "".join(cell["source"])
        if cell["cell_type"] == "code" and "def save_weights" in src and "def load_weights" in src:
            exec(compile(src, "demo.ipynb:save_weights", "exec"), ns)
            return ns["save_weights"], ns["load_weights"]
    raise SystemExit("demo.ipynb: save_weights / load_weights not found")


def gen_checkpoint(reference_path, ref):
    """A tiny tied-head GPT saved by the reference's own ``save_weights``; logits of the reference on a small batch."""
    network, layers, activations, ta = ref
    spec = wl.GPTSpec("ckpt", vocab=40, context=16, d_model=32, heads=2, layers=2, tied_head=True, precision="tf32",
                      batch=3, seq_len=12, input_seed=11, input_dist="uniform")
    net = build_reference_net(ref, spec)
    params = wl.seeded_params(spec, 77)
    seen, it = set(), iter(params)
    for layer in net.layers:
        for prm in layer.parameters:
            if id(prm) in seen:
                continue
            seen.add(id(prm))
            prm[...] = next(it)
    net.set_eval(True)
    save_weights, _ = notebook_helpers(reference_path, ref)

    class HostArray(np.ndarray):
        # the notebook calls CuPy's .get() on every parameter; on the NumPy path the array is already on the host
        def get(self):
            return np.asarray(self)

    class View:
        def __init__(self, layer):
            self.parameters = [prm.view(HostArray) for prm in layer.parameters]
    View.__name__ = "View"

    class Saved:
        layers = []
    for layer in net.layers:
        v = type(type(layer).__name__, (View,), {})(layer)      # keeps type(layer).__name__ for the file's "name"
        Saved.layers.append(v)
    save_weights(Saved, os.path.join(HERE, "ckpt_tiny.pkl"))
    ids = wl.make_inputs(spec)
    logits = np.asarray(net.predict(ids), dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "ckpt_tiny.npz"), ids=ids, logits=logits,
                        spec=np.array([spec.vocab, spec.context, spec.d_model, spec.heads, spec.layers]))
    print("ckpt_tiny: logits", logits.shape, "file", os.path.getsize(os.path.join(HERE, "ckpt_tiny.pkl")), "bytes")


def gen_evaluate(ref):
    """The demo's ViT recipe in small (demo.ipynb: VitProjector with register tokens, SiLU blocks with dropout rates,
    LayerNorm, VitMLPHead, SiLU, Dropout, Dense, SoftMax) through the reference's own ``Network.evaluate``."""
    network, layers, activations, ta = ref
    E, H = 64, 2
    net = network.Network(
        [ta.VitProjector((3, 16, 16), (2, 2), E, num_registers=2)]
        + [layers.TransformerBlock(E, 0, H, activations.SiLU, attn_dropout_rate=0.1, res_dropout_rate=0.1) for _ in range(2)]
        + [layers.LayerNorm(E), ta.VitMLPHead(E, 32), activations.SiLU(), layers.Dropout(0.1), layers.Dense(32, 10),
           activations.SoftMax()])
    rng = np.random.default_rng(123)
    params, seen = [], set()
    for layer in net.layers:
        for prm in layer.parameters:
            if id(prm) in seen:
                continue
            seen.add(id(prm))
            if prm.ndim == 1 and prm.shape[0] in (E, 4 * E, 3 * E, 32, 10):
                new = rng.standard_normal(prm.shape) * 0.1 + (1.0 if np.all(np.asarray(prm) == 1) else 0.0)
            else:
                new = rng.standard_normal(prm.shape) / np.sqrt(prm.shape[0] if prm.ndim > 1 else 1.0) * 0.7
            prm[...] = new.astype(np.float32)
            params.append(np.array(prm, dtype=np.float32))
    images = rng.standard_normal((20, 3, 16, 16)).astype(np.float32)
    labels = rng.integers(0, 10, size=20).astype(np.int64)
    loss, acc = net.evaluate(images, labels, network.CrossEntropy(10), batch_size=8)
    probs = np.asarray(net.predict(images), dtype=np.float32)
    out = {f"p{i}": a for i, a in enumerate(params)}
    np.savez_compressed(os.path.join(HERE, "eval_tiny.npz"), images=images, labels=labels, loss=np.float64(loss),
                        accuracy=np.float64(acc), probs=probs, n_params=np.int64(len(params)), **out)
    print("eval_tiny: loss", float(loss), "accuracy", float(acc), "params", len(params))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("what", nargs="*", default=["layers", "c1", "c2"])
    a = ap.parse_args()
    ref = load_reference(a.reference)
    for w in a.what:
        if w == "layers":
            gen_layers(ref)
        elif w in ("c1", "c2"):
            gen_small(ref, w)
        elif w == "c3":
            gen_large(ref, "c3", [0, 1, 2, 4, 6, 8, 10, 12, 14])      # rows 0 and 1, then one per rank of an 8-way shard
        elif w == "c5":
            gen_large(ref, "c5", [0, 8, 16, 24, 32, 40, 48, 56])      # one sequence per rank of an 8-way shard
        elif w == "c4":
            gen_decode(ref)
        elif w == "ckpt":
            gen_checkpoint(a.reference, ref)
        elif w == "eval":
            gen_evaluate(ref)
        else:
            raise SystemExit(f"unknown target {w}")


if __name__ == "__main__":
    main()
