"""Weight interchange with the reference's pickle layout (demo.ipynb save_weights / load_weights).  The fixture
``golden/ckpt_tiny.pkl`` was written by the reference's own ``save_weights`` (see golden/make_golden.py, target
``ckpt``); ``golden/ckpt_tiny.npz`` holds the reference's logits for that model."""
import os
import pickle

import numpy as np
import pytest

from conftest import rel_err, TOL

HERE = os.path.dirname(os.path.abspath(__file__))
CKPT = os.path.join(HERE, "golden", "ckpt_tiny.pkl")


def _spec():
    from torchless_nn_b200 import workloads as wl
    g = np.load(os.path.join(HERE, "golden", "ckpt_tiny.npz"))
    vocab, context, d, heads, layers = (int(v) for v in g["spec"])
    spec = wl.GPTSpec("ckpt", vocab=vocab, context=context, d_model=d, heads=heads, layers=layers, tied_head=True,
                      precision="tf32", batch=3, seq_len=12, input_seed=11, input_dist="uniform")
    return spec, g


def test_fixture_layout():
    from torchless_nn_b200.checkpoint import read_checkpoint
    entries = read_checkpoint(CKPT)
    assert [e["name"] for e in entries] == ["GPTEmbedFront", "TransformerBlock", "TransformerBlock", "LayerNorm", "GPTEmbedBack"]
    # the tied head registers no parameter of its own: the table belongs to the embedding front
    assert [len(e["parameters"]) for e in entries] == [2, 12, 12, 2, 0]
    assert all(a.dtype == np.float32 for e in entries for a in e["parameters"])


def test_loader_refuses_anything_but_arrays(tmp_path):
    from torchless_nn_b200.checkpoint import read_checkpoint
    bad = tmp_path / "bad.pkl"
    bad.write_bytes(pickle.dumps([{"name": "Dense", "parameters": [print]}]))
    with pytest.raises(pickle.UnpicklingError):
        read_checkpoint(bad)
    odd = tmp_path / "odd.pkl"
    odd.write_bytes(pickle.dumps({"name": "Dense"}))
    with pytest.raises(ValueError):
        read_checkpoint(odd)


@pytest.mark.gpu
def test_reference_checkpoint_runs_and_round_trips(engine, tmp_path):
    from torchless_nn_b200.checkpoint import load_weights, save_weights, read_checkpoint
    from torchless_nn_b200.models import build_network
    spec, g = _spec()
    engine.set_precision("tf32")
    net = build_network(spec)
    load_weights(net, CKPT)
    net.set_eval(True)
    logits = net.predict(g["ids"])
    logits = logits.get() if hasattr(logits, "get") else np.asarray(logits)
    assert logits.shape == g["logits"].shape
    assert rel_err(logits, g["logits"]) < TOL["tf32"]
    out = tmp_path / "again.pkl"
    save_weights(net, out)
    a, b = read_checkpoint(CKPT), read_checkpoint(out)
    assert [e["name"] for e in a] == [e["name"] for e in b]
    for ea, eb in zip(a, b):
        assert len(ea["parameters"]) == len(eb["parameters"])
        for x, y in zip(ea["parameters"], eb["parameters"]):
            assert np.array_equal(x, y)


@pytest.mark.gpu
def test_strict_loading_reports_mismatches(engine):
    from torchless_nn_b200 import workloads as wl
    from torchless_nn_b200.checkpoint import load_weights
    from torchless_nn_b200.models import build_network
    spec, _ = _spec()
    wider = wl.GPTSpec("ckpt", vocab=spec.vocab, context=spec.context, d_model=64, heads=2, layers=2, tied_head=True,
                       precision="tf32", batch=3, seq_len=12, input_seed=11, input_dist="uniform")
    with pytest.raises(ValueError):
        load_weights(build_network(wider), CKPT)
    deeper = wl.GPTSpec("ckpt", vocab=spec.vocab, context=spec.context, d_model=32, heads=2, layers=3, tied_head=True,
                        precision="tf32", batch=3, seq_len=12, input_seed=11, input_dist="uniform")
    with pytest.raises(ValueError):
        load_weights(build_network(deeper), CKPT)
