"""CPU tests: the NumPy oracle against the golden fixtures that the reference library itself produced
(tests/golden/make_golden.py).  The oracle restates the reference's array operations one for one, so the match is
expected to be exact; a tiny slack covers BLAS builds that block differently."""
import numpy as np
import pytest

from oracle import forward_np as onp
from torchless_nn_b200 import workloads as wl

EXACT = 5e-6


def test_fixtures_record_bit_identical_oracle(golden):
    for name in ("c1", "c2", "c3", "c5"):
        assert float(golden(name)["oracle_max_abs_diff"]) == 0.0


def test_c1_oracle_matches_reference(golden):
    g = golden("c1")
    spec = wl.CONFIGS["c1"]
    params = wl.seeded_params(spec)
    x = wl.make_inputs(spec)
    y = onp.forward(spec, params, x)
    assert np.abs(y[:8] - g["logits"]).max() < EXACT
    assert np.array_equal(np.argmax(y, -1), g["argmax"])
    assert np.array_equal(onp.embed_front(x[:2], params[1], params[0]), g["embed0"])
    assert abs(float(np.abs(y).max()) - float(g["max_abs"])) < EXACT


def test_c2_oracle_matches_reference(golden):
    g = golden("c2")
    spec = wl.CONFIGS["c2"]
    y = onp.forward(spec, wl.seeded_params(spec), wl.make_inputs(spec, 32))
    assert np.abs(y - g["logits"][:32]).max() < EXACT


def test_c3_oracle_prefix_matches_reference(golden):
    """The model is causal, so the logits of a prefix equal the stored logits of the full sequence."""
    g = golden("c3")
    spec = wl.CONFIGS["c3"]
    T = 160
    x = wl.make_inputs(spec, 1)[:, :T]
    y = onp.gpt_forward(spec, wl.seeded_params(spec), x)[0]
    rows = g["seq0_rows"]
    keep = rows < T
    got = y[np.ix_(rows[keep], g["seq0_cols"])]
    assert np.abs(got - g["seq0_vals"][keep]).max() < 1e-4
    tol = 2e-3 * float(g["seq0_max_abs"])
    ok, _, bad = onp.tokens_match(np.argmax(y, -1), g["seq0_argmax"][:T], g["seq0_top"][:T], g["seq0_second"][:T], tol)
    assert ok, bad


def test_c4_oracle_greedy_matches_reference(golden):
    g = golden("c4")
    spec = wl.CONFIGS["c4"]
    prompts = wl.make_inputs(spec, int(g["n_prompts"]))
    assert np.array_equal(prompts, g["tokens"][:, :spec.seq_len])
    out = onp.greedy_decode(spec, wl.seeded_params(spec), prompts[:1], 3)
    assert np.array_equal(out, g["tokens"][:1, :spec.seq_len + 3])


def test_layer_fixtures(golden):
    g = golden("layers")
    for d in (128, 192, 768, 1000):
        assert np.array_equal(onp.layer_norm(g[f"ln{d}_x"], g[f"ln{d}_g"], g[f"ln{d}_b"]), g[f"ln{d}_y"])
    for tag in "abcdef":
        d, H, T, dec = (int(v) for v in g[f"attn_{tag}_meta"])
        y = onp.attention(g[f"attn_{tag}_x"], g[f"attn_{tag}_wqkv"], g[f"attn_{tag}_bqkv"], g[f"attn_{tag}_wo"],
                          g[f"attn_{tag}_bo"], H, onp.causal_mask(128) if dec else None)
        assert np.abs(y - g[f"attn_{tag}_y"]).max() < EXACT
    for act in ("gelu", "silu", "relu"):
        y = onp.feed_forward(g[f"ffn_{act}_x"], g[f"ffn_{act}_w1"], g[f"ffn_{act}_b1"], g[f"ffn_{act}_w2"],
                             g[f"ffn_{act}_b2"], act)
        assert np.abs(y - g[f"ffn_{act}_y"]).max() < EXACT
        assert np.array_equal(onp.ACTIVATIONS[act](g["act_x"]), g[f"act_{act}"])
    for i in range(4):
        assert np.array_equal(onp.softmax_t(g[f"softmax{i}_x"], np.float32(g[f"softmax{i}_t"])), g[f"softmax{i}_y"])
    assert np.abs(onp.dense(g["dense_x3"], g["dense_w"], g["dense_b"]) - g["dense_y3"]).max() < EXACT
    assert np.array_equal(onp.embed_front(g["emb_ids"], g["emb_table"], g["emb_pos"]), g["emb_y"])
    assert np.array_equal(onp.embed_front(g["emb_ids"].astype(np.uint8), g["emb_table"], g["emb_pos"]), g["emb_y_u8"])
    assert np.array_equal(onp.sinusoidal_table(32, 48), g["emb_sin_pos"])
    assert np.abs(onp.tied_logits(g["back_x"], g["emb_table"]) - g["back_y"]).max() < EXACT
    for tag in ("r0", "r2"):
        y = onp.vit_project(g[f"vitp_{tag}_img"], g[f"vitp_{tag}_proj"], g[f"vitp_{tag}_cls"], g[f"vitp_{tag}_pos"], (4, 4))
        assert np.abs(y - g[f"vitp_{tag}_y"]).max() < EXACT
    assert np.abs(onp.vit_head(g["vith_x"], g["vith_w"], g["vith_b"]) - g["vith_y"]).max() < EXACT
    ps = [g[f"block_silu_p{i}"] for i in range(12)]
    assert np.abs(onp.block(g["block_silu_x"], ps, 2, None, "silu") - g["block_silu_y"]).max() < EXACT


def test_tie_rule():
    ref_arg = np.array([3, 5, 7])
    top = np.array([1.0, 1.0, 1.0], dtype=np.float32)
    second = np.array([0.5, 0.999, 0.2], dtype=np.float32)
    ok, n, bad = onp.tokens_match(np.array([3, 9, 7]), ref_arg, top, second, 0.01)
    assert ok and n == 1 and bad == 0
    ok, n, bad = onp.tokens_match(np.array([4, 5, 7]), ref_arg, top, second, 0.01)
    assert not ok and bad == 1


def test_workload_generators():
    p = wl.zipf_probabilities(50257)
    assert abs(p.sum() - 1) < 1e-12 and p[0] > p[1] > p[100]
    a = wl.token_ids(50257, (4, 64), 3, "zipf")
    b = wl.token_ids(50257, (4, 64), 3, "zipf")
    assert np.array_equal(a, b) and a.dtype == np.int32 and a.min() >= 0 and a.max() < 50257
    assert np.array_equal(wl.make_inputs(wl.CONFIGS["c3"], 2), wl.make_inputs(wl.CONFIGS["c3"])[:2])
    img = wl.images((2, 3, 32, 32), 2)
    assert img.dtype == np.float32 and img.min() >= -2.0 and img.max() < 2.0
    assert wl.CONFIGS["c3"].n_params() == 124_439_808
    assert wl.CONFIGS["c5"].n_params() == 355_871_744
    assert wl.CONFIGS["c1"].n_params() == 826_433
    assert round(wl.CONFIGS["c5"].flops_per_token()) == 807_618_560
    assert round(wl.CONFIGS["c3"].flops_per_token()) == 265_956_864
    assert [wl.shard_rows(64, r, 8) for r in (0, 7)] == [(0, 8), (56, 64)]
    assert [wl.shard_rows(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        wl.shard_rows(8, 4, 4)


def test_choice_rule_is_numpys():
    """The sampling oracle restates numpy.random.RandomState.choice(arange(V), p=p) - what `xp.random.choice` is on the
    reference's NumPy runtime (demo.ipynb:1530) - for a given uniform number: pinned against NumPy itself."""
    from oracle import forward_np as onp
    rng = np.random.default_rng(0)
    for V in (5, 65, 1000):
        p = rng.random(V) ** 3
        p /= p.sum()
        for seed in range(25):
            u = np.random.RandomState(seed).random_sample()
            want = np.random.RandomState(seed).choice(np.arange(V), p=p)
            assert onp.choice_index(p, u) == want
