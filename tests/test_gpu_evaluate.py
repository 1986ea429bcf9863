"""Network.evaluate (network.py:145-160) on the demo's ViT recipe in small: register tokens, SiLU blocks with dropout
rates, VitMLPHead -> SiLU -> Dropout -> Dense -> SoftMax.  ``golden/eval_tiny.npz`` holds the parameters, inputs, and
the loss / accuracy / probabilities the reference's own ``evaluate`` and ``predict`` produced (make_golden.py eval)."""
import numpy as np
import pytest

from conftest import rel_err, TOL

pytestmark = pytest.mark.gpu


def _build(g):
    from torchless_nn_b200 import activations as act
    from torchless_nn_b200 import layers as L
    from torchless_nn_b200 import transformer_adapters as ta
    from torchless_nn_b200.network import Network
    E, H = 64, 2
    net = Network(
        [ta.VitProjector((3, 16, 16), (2, 2), E, num_registers=2)]
        + [L.TransformerBlock(E, 0, H, act.SiLU, attn_dropout_rate=0.1, res_dropout_rate=0.1) for _ in range(2)]
        + [L.LayerNorm(E), ta.VitMLPHead(E, 32), act.SiLU(), L.Dropout(0.1), L.Dense(32, 10), act.SoftMax()])
    arrays = [g[f"p{i}"] for i in range(int(g["n_params"]))]
    it, seen = iter(arrays), set()
    for layer in net.layers:
        for p in layer.parameters:
            if id(p) in seen:
                continue
            seen.add(id(p))
            a = next(it)
            assert tuple(p.shape) == tuple(a.shape)
            p[...] = a
    assert next(it, None) is None
    return net


@pytest.mark.parametrize("prec", ["tf32", "bf16"])
def test_evaluate_matches_the_reference(engine, golden, prec):
    from torchless_nn_b200.network import CrossEntropy
    g = golden("eval_tiny")
    engine.set_precision(prec)
    try:
        net = _build(g)
        net.set_eval(True)
        probs = net.predict(g["images"]).get()
        assert rel_err(probs, g["probs"]) < TOL[prec]
        loss, acc = net.evaluate(g["images"], g["labels"], CrossEntropy(10), batch_size=8)
        assert abs(loss - float(g["loss"])) < (5e-3 if prec == "tf32" else 5e-2) * float(g["loss"])
        # arg-max may only differ where the reference's two best classes are closer than the tolerance
        top2 = np.sort(g["probs"], axis=1)[:, -2:]
        shaky = int(((top2[:, 1] - top2[:, 0]) < TOL[prec] * g["probs"].max()).sum())
        assert abs(acc - float(g["accuracy"])) <= shaky / len(g["labels"]) + 1e-12
        # the criterion on its own: one batch, sum of -log(p[label] + 1e-7)
        ce = CrossEntropy(10).loss(g["probs"], g["labels"])
        want = float(-np.sum(np.log(g["probs"][np.arange(len(g["labels"])), g["labels"]] + np.float32(1e-7))))
        assert abs(ce - want) < 1e-4 * abs(want)
    finally:
        engine.set_precision("tf32")


def test_label_out_of_range_is_an_index_error(engine):
    from torchless_nn_b200 import backend
    from torchless_nn_b200.network import CrossEntropy
    engine.set_precision("tf32")
    p = np.full((4, 10), 0.1, dtype=np.float32)
    with pytest.raises(IndexError):
        CrossEntropy(10).loss(p, np.array([1, 2, 10, 3]))
        backend.synchronize()


def test_prefetched_batches_equal_plain_uploads(engine, golden):
    """The double-buffered feeder delivers every batch (ragged last one included) bit for bit, and evaluate gives the
    same two numbers with and without it."""
    from torchless_nn_b200.host_feed import HostFeed
    from torchless_nn_b200.network import CrossEntropy
    g = golden("eval_tiny")
    engine.set_precision("tf32")
    data = g["images"]
    per = int(np.prod(data.shape[1:])) * 4
    with HostFeed(per * 8) as feed:
        seen = []
        for lo, hi, dev in feed.batches(data, 8, np.float32):
            assert dev.shape == data[lo:hi].shape
            assert np.array_equal(dev.get(), data[lo:hi])
            seen.append((lo, hi))
    assert seen == [(0, 8), (8, 16), (16, 20)]
    net = _build(g)
    a = net.evaluate(data, g["labels"], CrossEntropy(10), batch_size=8, prefetch=True)
    b = net.evaluate(data, g["labels"], CrossEntropy(10), batch_size=8, prefetch=False)
    assert a == b
