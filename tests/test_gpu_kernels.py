"""GPU parity tests, layer by layer, through the C ABI (via the Layer classes), against the NumPy oracle and the
golden fixtures produced by the reference.  Tolerances are the ones the task states: float32/TF32 results within
2e-3 of max|reference|, bf16 within 3e-2, embedding gather bit-exact."""
import numpy as np
import pytest

from conftest import rel_err, TOL
from oracle import forward_np as onp

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["tf32", "bf16"])
def prec(request, engine):
    engine.set_precision(request.param)
    yield request.param
    engine.set_precision("tf32")


def _load(arr, dev):
    dev[...] = arr


# ----------------------------------------------------------------------------- GEMM through Dense
@pytest.mark.parametrize("M,K,N", [(1, 8, 1), (7, 40, 65), (128, 64, 256), (130, 72, 10), (300, 128, 384),
                                   (4096, 128, 65), (1000, 768, 2304), (257, 3072, 768), (513, 192, 576),
                                   (2048, 1024, 1000)])
def test_dense_matches_numpy(engine, prec, M, K, N):
    from torchless_nn_b200.layers import Dense
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    w = (rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    layer = Dense(K, N)
    _load(w, layer.weights)
    _load(b, layer.bias)
    y = layer.forward(x).get()
    ref = x.astype(np.float64) @ w.astype(np.float64) + b
    assert y.shape == (M, N)
    assert rel_err(y, ref) < TOL[prec]


@pytest.mark.parametrize("M,K,N", [(10240, 256, 1024), (9999, 192, 1184), (12800, 64, 800)])
def test_dense_many_tiles_pair_kernel(engine, M, K, N):
    """Shapes with at least as many 256 x 256 tiles as SMs take the CTA-pair GEMM in bf16 mode (ragged M, ragged N)."""
    from torchless_nn_b200.layers import Dense
    engine.set_precision("bf16")
    try:
        rng = np.random.default_rng(M + K + N)
        w = (rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
        b = rng.standard_normal(N, dtype=np.float32)
        x = rng.standard_normal((M, K), dtype=np.float32)
        layer = Dense(K, N)
        _load(w, layer.weights)
        _load(b, layer.bias)
        y = layer.forward(x).get()
        ref = x @ w + b
        assert rel_err(y, ref) < TOL["bf16"]
    finally:
        engine.set_precision("tf32")


@pytest.mark.parametrize("M,K,N", [(64, 768, 768), (64, 3072, 768), (100, 1024, 256), (10240, 256, 1024), (300, 128, 384)])
def test_linear_in_place_residual(engine, M, K, N):
    """residual == out: the product is added to the buffer in place (TMA reduce-add epilogue in bf16 mode; with few
    tiles the contraction is split over several CTAs).  Through the C ABI, against NumPy."""
    import ctypes as C
    from torchless_nn_b200 import _lib, backend
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.device_array import DeviceArray
    from torchless_nn_b200.utils import PreparedWeight
    engine.set_precision("bf16")
    try:
        rng = np.random.default_rng(M * 3 + K + N)
        w = (rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
        b = rng.standard_normal(N, dtype=np.float32)
        a = rng.standard_normal((M, K), dtype=np.float32)
        x = rng.standard_normal((M, N), dtype=np.float32)
        wd, bd, ad, xd = (DeviceArray.from_numpy(v) for v in (w, b, a, x))
        pw = PreparedWeight(wd, transpose=True)
        for _ in range(2):                      # twice: x += a w + b, then once more on the result
            check(lib.tlnn_linear_fwd(backend.ctx(), backend.precision_code(), ad.ptr, K, pw.ptr(), bd.ptr, _lib.ACT_NONE,
                                      xd.ptr, N, xd.ptr, N, M, N, K))
        ref = x + 2.0 * (a @ w + b)
        assert rel_err(xd.get(), ref) < TOL["bf16"]
    finally:
        engine.set_precision("tf32")


@pytest.mark.parametrize("M,K,N,prec", [(16640, 192, 192, "tf32"), (16000, 96, 200, "tf32"), (16640, 192, 192, "bf16")])
def test_linear_one_round_of_wide_tiles(engine, M, K, N, prec):
    """130 row blocks and 129 to 256 columns: one round of 256-wide tiles on most SMs is chosen over two rounds of
    128-wide ones.  Bias and residual through the C ABI, against NumPy."""
    from torchless_nn_b200 import _lib, backend
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.device_array import DeviceArray
    from torchless_nn_b200.utils import PreparedWeight
    engine.set_precision(prec)
    try:
        rng = np.random.default_rng(M + K + N)
        w = (rng.standard_normal((K, N), dtype=np.float32) / np.sqrt(K)).astype(np.float32)
        b = rng.standard_normal(N, dtype=np.float32)
        a = rng.standard_normal((M, K), dtype=np.float32)
        x = rng.standard_normal((M, N), dtype=np.float32)
        wd, bd, ad, xd = (DeviceArray.from_numpy(v) for v in (w, b, a, x))
        yd = DeviceArray.from_numpy(np.zeros((M, N), dtype=np.float32))
        pw = PreparedWeight(wd, transpose=True)
        check(lib.tlnn_linear_fwd(backend.ctx(), backend.precision_code(), ad.ptr, K, pw.ptr(), bd.ptr, _lib.ACT_NONE,
                                  xd.ptr, N, yd.ptr, N, M, N, K))
        assert rel_err(yd.get(), x + a @ w + b) < TOL[prec]
    finally:
        engine.set_precision("tf32")


def test_suite_with_pair_kernel_forced():
    """TLNN_GEMM_PAIR=force routes every bf16 product through the CTA-pair kernel: the layer tests must still pass."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, TLNN_GEMM_PAIR="force")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                        os.path.join(root, "tests", "test_gpu_kernels.py"),
                        "-k", "dense_matches_numpy or ffn_golden or block_golden or attention_golden"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_dense_golden(engine, prec, golden):
    from torchless_nn_b200.layers import Dense
    g = golden("layers")
    layer = Dense(40, 65)
    _load(g["dense_w"], layer.weights)
    _load(g["dense_b"], layer.bias)
    assert rel_err(layer.forward(g["dense_x2"]).get(), g["dense_y2"]) < TOL[prec]
    y3 = layer.forward(g["dense_x3"])
    assert y3.shape == g["dense_y3"].shape
    assert rel_err(y3.get(), g["dense_y3"]) < TOL[prec]


def test_dense_weight_edit_invalidates_prepared_copy(engine):
    from torchless_nn_b200.layers import Dense
    layer = Dense(16, 8)
    x = np.ones((4, 16), dtype=np.float32)
    w = np.full((16, 8), 0.5, dtype=np.float32)
    _load(w, layer.weights)
    y0 = layer.forward(x).get()
    layer.weights *= 0
    layer.weights += w * 2
    y1 = layer.forward(x).get()
    assert np.allclose(y0, 8.0) and np.allclose(y1, 16.0)


# ----------------------------------------------------------------------------- embedding (bit-exact)
def test_embedding_bit_exact(engine, golden):
    from torchless_nn_b200.transformer_adapters import GPTEmbeddingTable, GPTEmbedFront
    g = golden("layers")
    tab = GPTEmbeddingTable(97, 48)
    _load(g["emb_table"], tab.table)
    fr = GPTEmbedFront(tab, 32)
    _load(g["emb_pos"], fr.pos_embedding_table)
    for ids in (g["emb_ids"], g["emb_ids"].astype(np.int32), g["emb_ids"].astype(np.uint8)):
        assert np.array_equal(fr.forward(ids).get(), g["emb_y"])
    fs = GPTEmbedFront(tab, 32, positional_embedding="sinusoidal")
    assert np.array_equal(fs.pos_embedding_table.get(), g["emb_sin_pos"])
    assert np.array_equal(fs.forward(g["emb_ids"]).get(), g["emb_sin_y"])


def test_embedding_odd_width_and_negative_ids(engine):
    from torchless_nn_b200.transformer_adapters import GPTEmbeddingTable, GPTEmbedFront
    rng = np.random.default_rng(0)
    tab = GPTEmbeddingTable(11, 7)
    t = rng.standard_normal((11, 7), dtype=np.float32)
    p = rng.standard_normal((5, 7), dtype=np.float32)
    _load(t, tab.table)
    fr = GPTEmbedFront(tab, 5)
    _load(p, fr.pos_embedding_table)
    ids = np.array([[0, -1, 10, 3, 5]], dtype=np.int64)
    assert np.array_equal(fr.forward(ids).get(), onp.embed_front(ids, t, p))


def test_embedding_errors(engine):
    from torchless_nn_b200.transformer_adapters import GPTEmbeddingTable, GPTEmbedFront
    fr = GPTEmbedFront(GPTEmbeddingTable(10, 8), 4)
    with pytest.raises(IndexError):
        fr.forward(np.array([[1, 10]], dtype=np.int32))          # id out of range
    with pytest.raises(IndexError):
        fr.forward(np.array([[1.0, 2.0]], dtype=np.float32))     # float ids
    with pytest.raises(ValueError):
        fr.forward(np.zeros((1, 5), dtype=np.int32))             # longer than the context
    assert fr.forward(np.zeros((1, 4), dtype=np.int32)).shape == (1, 4, 8)   # context still usable afterwards


# ----------------------------------------------------------------------------- LayerNorm / softmax / activations
@pytest.mark.parametrize("d", [128, 192, 768, 1000])
def test_layernorm_golden(engine, golden, d):
    from torchless_nn_b200.layers import LayerNorm
    g = golden("layers")
    ln = LayerNorm(d)
    _load(g[f"ln{d}_g"], ln.gamma)
    _load(g[f"ln{d}_b"], ln.beta)
    y = ln.forward(g[f"ln{d}_x"]).get()
    assert np.abs(y - g[f"ln{d}_y"]).max() < 2e-5


def test_layernorm_odd_width(engine):
    from torchless_nn_b200.layers import LayerNorm
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 3, 37), dtype=np.float32) * 3 + 1
    ln = LayerNorm(37)
    y = ln.forward(x).get()
    assert np.abs(y - onp.layer_norm(x, np.ones(37, np.float32), np.zeros(37, np.float32))).max() < 2e-5
    with pytest.raises(ValueError):
        ln.forward(np.zeros((2, 36), dtype=np.float32))


@pytest.mark.parametrize("i", [0, 1, 2, 3])
def test_softmax_golden(engine, golden, i):
    from torchless_nn_b200.activations import SoftMax
    g = golden("layers")
    sm = SoftMax()
    sm.temperature = float(g[f"softmax{i}_t"])       # mutated after construction, as the notebook does
    y = sm.forward(g[f"softmax{i}_x"]).get()
    ref = g[f"softmax{i}_y"]
    assert np.abs(y - ref).max() <= 1e-6 + 1e-4 * ref.max()
    assert np.allclose(y.sum(-1), 1.0, atol=1e-4)


def test_activations_golden(engine, golden):
    from torchless_nn_b200 import activations
    g = golden("layers")
    for name, cls in (("gelu", activations.GeLU), ("silu", activations.SiLU), ("relu", activations.ReLU)):
        y = cls().forward(g["act_x"]).get()
        assert np.abs(y - g[f"act_{name}"]).max() < 1e-5


def test_argmax_first_maximum(engine):
    from torchless_nn_b200.backend import xp
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 50257), dtype=np.float32)
    x[2, 100] = x[2, 40000] = 9.0          # tie: first index wins
    x[3, 50256] = 10.0
    a = xp.argmax(xp.array(x), axis=-1).get()
    assert np.array_equal(a, np.argmax(x, axis=-1))
    small = rng.standard_normal((3, 5, 10), dtype=np.float32)
    assert np.array_equal(xp.argmax(xp.array(small)).get(), np.argmax(small, -1))


# ----------------------------------------------------------------------------- attention / feed-forward / block
@pytest.mark.parametrize("tag", list("abcdef"))
def test_attention_golden(engine, prec, golden, tag):
    from torchless_nn_b200.layers import MultiHeadAttention
    g = golden("layers")
    d, H, T, dec = (int(v) for v in g[f"attn_{tag}_meta"])
    at = MultiHeadAttention(d, 128, H, decoder=bool(dec))
    _load(g[f"attn_{tag}_wqkv"], at.qkv_weights)
    _load(g[f"attn_{tag}_bqkv"], at.qkv_bias)
    _load(g[f"attn_{tag}_wo"], at.out_weights)
    _load(g[f"attn_{tag}_bo"], at.out_bias)
    at.set_eval(True)
    y = at.forward(g[f"attn_{tag}_x"]).get()
    assert y.shape == g[f"attn_{tag}_y"].shape
    assert rel_err(y, g[f"attn_{tag}_y"]) < TOL[prec]


@pytest.mark.parametrize("B,T,d,H,causal", [(2, 300, 128, 2, True), (1, 257, 256, 2, False), (3, 64, 64, 2, True),
                                            (1, 1024, 128, 2, True), (2, 129, 256, 2, True),
                                            (4, 512, 256, 4, True), (1, 2048, 64, 1, True), (5, 193, 128, 2, False),
                                            (2, 1000, 192, 3, True), (37, 200, 64, 1, True)])
def test_attention_long_and_ragged(engine, prec, B, T, d, H, causal):
    from torchless_nn_b200.layers import MultiHeadAttention
    rng = np.random.default_rng(T + d)
    at = MultiHeadAttention(d, max(1024, T), H, decoder=causal)
    ws = [rng.standard_normal(p.shape, dtype=np.float32) * np.float32(0.08) for p in at.parameters]
    for p, w in zip(at.parameters, ws):
        _load(w, p)
    x = rng.standard_normal((B, T, d), dtype=np.float32)
    y = at.forward(x).get()
    ref = onp.attention(x, *ws, H, onp.causal_mask(max(1024, T)) if causal else None)
    assert rel_err(y, ref) < TOL[prec]


@pytest.mark.parametrize("B,T,d,H,causal", [(2, 50, 32, 2, True), (3, 33, 32, 4, False), (1, 130, 64, 4, True),
                                            (2, 65, 64, 2, False), (2, 65, 64, 2, True), (1, 257, 64, 2, False),
                                            (2, 100, 128, 2, True), (1, 36, 64, 1, False), (1, 132, 128, 2, False),
                                            (128, 65, 192, 6, False), (40, 128, 256, 8, True), (96, 40, 128, 8, True)])
def test_attention_small_heads_float32(engine, B, T, d, H, causal):
    """Head dimensions 8 and 16 exist in float32 / TF32 mode only (thread-per-query kernel); lengths one to four past a
    multiple of 32 (a ViT's class token) send their last queries to the warp-per-query rows of that kernel.  The large
    batches have enough warps for one thread per query; the others split each query's keys over four lanes."""
    from torchless_nn_b200.layers import MultiHeadAttention
    engine.set_precision("tf32")
    rng = np.random.default_rng(T + d + H)
    at = MultiHeadAttention(d, max(256, T), H, decoder=causal)
    ws = [rng.standard_normal(p.shape, dtype=np.float32) * np.float32(0.1) for p in at.parameters]
    for p, w in zip(at.parameters, ws):
        _load(w, p)
    x = rng.standard_normal((B, T, d), dtype=np.float32)
    y = at.forward(x).get()
    ref = onp.attention(x, *ws, H, onp.causal_mask(max(256, T)) if causal else None)
    assert rel_err(y, ref) < TOL["tf32"]


@pytest.mark.parametrize("act", ["gelu", "silu", "relu"])
def test_ffn_golden(engine, prec, golden, act):
    from torchless_nn_b200 import activations
    from torchless_nn_b200.layers import TransformerFeedForward
    g = golden("layers")
    cls = {"gelu": activations.GeLU, "silu": activations.SiLU, "relu": activations.ReLU}[act]
    ff = TransformerFeedForward(96, cls)
    for name, p in (("w1", ff.weights1), ("b1", ff.bias1), ("w2", ff.weights2), ("b2", ff.bias2)):
        _load(g[f"ffn_{act}_{name}"], p)
    y = ff.forward(g[f"ffn_{act}_x"]).get()
    assert rel_err(y, g[f"ffn_{act}_y"]) < TOL[prec]


def test_block_golden_silu_bidirectional(engine, prec, golden):
    from torchless_nn_b200 import activations
    from torchless_nn_b200.layers import TransformerBlock
    g = golden("layers")
    blk = TransformerBlock(64, 0, 2, activations.SiLU)
    for i, p in enumerate(blk.parameters):
        _load(g[f"block_silu_p{i}"], p)
    blk.set_eval(True)
    y = blk.forward(g["block_silu_x"]).get()
    assert rel_err(y, g["block_silu_y"]) < TOL[prec]
    assert blk.input.shape == (2, 11, 64) and blk.output.dtype == np.float32


# ----------------------------------------------------------------------------- ViT adapters, tied head
@pytest.mark.parametrize("tag,regs", [("r0", 0), ("r2", 2)])
def test_vit_projector_golden(engine, prec, golden, tag, regs):
    from torchless_nn_b200.transformer_adapters import VitProjector
    g = golden("layers")
    vp = VitProjector((3, 16, 24), (4, 4), 64, regs)
    _load(g[f"vitp_{tag}_proj"], vp.projection)
    _load(g[f"vitp_{tag}_cls"], vp.cls_reg_tokens)
    _load(g[f"vitp_{tag}_pos"], vp.positional_embeddings)
    y = vp.forward(g[f"vitp_{tag}_img"]).get()
    assert y.shape == g[f"vitp_{tag}_y"].shape
    assert rel_err(y, g[f"vitp_{tag}_y"]) < TOL[prec]
    # class / register rows involve no product: exact
    assert np.array_equal(y[:, :1 + regs], g[f"vitp_{tag}_y"][:, :1 + regs])


def test_vit_head_golden(engine, prec, golden):
    from torchless_nn_b200.transformer_adapters import VitMLPHead
    g = golden("layers")
    vh = VitMLPHead(64, 10)
    _load(g["vith_w"], vh.weights)
    _load(g["vith_b"], vh.bias)
    assert rel_err(vh.forward(g["vith_x"]).get(), g["vith_y"]) < TOL[prec]


def test_tied_head_golden_and_tokens(engine, prec, golden):
    from torchless_nn_b200.transformer_adapters import GPTEmbeddingTable, GPTEmbedBack
    g = golden("layers")
    tab = GPTEmbeddingTable(97, 48)
    _load(g["emb_table"], tab.table)
    bk = GPTEmbedBack(tab)
    y = bk.forward(g["back_x"]).get()
    assert rel_err(y, g["back_y"]) < TOL[prec]
    tok = bk.forward_tokens(g["back_x"]).get()
    assert np.array_equal(tok, np.argmax(y, axis=-1))       # fused arg-max agrees with the logits it came from


# ----------------------------------------------------------------------------- device arrays
def test_device_array_api(engine):
    from torchless_nn_b200.backend import xp
    rng = np.random.default_rng(9)
    a = rng.standard_normal((4, 6, 10), dtype=np.float32)
    d = xp.array(a)
    assert d.shape == a.shape and d.dtype == np.float32 and d.ndim == 3 and d.size == a.size
    assert np.array_equal(d[0, -1].get(), a[0, -1])
    assert np.array_equal(d[:, -1].get(), a[:, -1])
    assert np.array_equal(d[1:3, ::2, 3].get(), a[1:3, ::2, 3])
    assert np.array_equal(d.reshape(24, 10).get(), a.reshape(24, 10))
    assert np.array_equal((d + d).get(), a + a)
    d *= 0
    d += a
    assert np.array_equal(d.get(), a)
    d.fill(2)
    assert np.all(d.get() == 2)
    d[...] = a
    assert np.array_equal(np.asarray(d), a)
    z = xp.zeros((3, 2))
    assert np.all(z.get() == 0)


# ----------------------------------------------------------------------------- failure handling
def test_expired_wait_is_reported_and_the_context_survives(engine):
    """A device-side wait that nothing satisfies gives up after its limit (60 ms here), the kernel returns, the next
    synchronisation raises RuntimeError with the time-out status, and the same context computes correctly afterwards."""
    import time
    from torchless_nn_b200 import backend
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.layers import Dense
    engine.set_precision("bf16")
    try:
        backend.synchronize()
        t0 = time.time()
        check(lib.tlnn_selftest_wait(backend.ctx(), 60))
        with pytest.raises(RuntimeError) as info:
            backend.synchronize()
        assert time.time() - t0 < 5.0
        assert "status -5" in str(info.value) and "site 900" in str(info.value)      # TLNN_ERR_TIMEOUT from the self-test
        backend.synchronize()                       # the error has been consumed
        layer = Dense(64, 32)
        x = np.random.default_rng(0).standard_normal((50, 64), dtype=np.float32)
        w = np.random.default_rng(1).standard_normal((64, 32), dtype=np.float32) / 8
        _load(w, layer.weights)
        _load(np.zeros(32, dtype=np.float32), layer.bias)
        assert rel_err(layer.forward(x).get(), x @ w) < TOL["bf16"]
    finally:
        engine.set_precision("tf32")


# ----------------------------------------------------------------------------- Residual wrapper, profiling, misc ABI
def test_residual_add_around_feed_forward(engine, prec, golden):
    """Residual(mode="add") (utils.py:76-88) on device arrays: x + feed_forward(x), against the reference's own
    feed-forward output from the fixture."""
    from torchless_nn_b200 import activations
    from torchless_nn_b200.layers import TransformerFeedForward
    from torchless_nn_b200.utils import Residual
    g = golden("layers")
    ff = TransformerFeedForward(96, activations.GeLU)
    for name, p in (("w1", ff.weights1), ("b1", ff.bias1), ("w2", ff.weights2), ("b2", ff.bias2)):
        _load(g[f"ffn_gelu_{name}"], p)
    res = Residual([ff], mode="add")
    res.set_eval(True)
    x = g["ffn_gelu_x"]
    y = res.forward(x)
    want = x + g["ffn_gelu_y"]
    assert y.shape == x.shape and rel_err(y.get(), want) < TOL[prec]
    params = [g[f"ffn_gelu_{n}"] for n in ("w1", "b1", "w2", "b2")]
    assert rel_err(y.get(), x + onp.feed_forward(x, *params, act="gelu")) < TOL[prec]
    assert res.output is y and np.array_equal(res.input.get(), x)
    assert len(res.parameters) == 4 and res.parameters[0] is ff.weights1
    with pytest.raises(NotImplementedError):
        Residual([ff], mode="concat").forward(x)


def test_profiling_entry_points(engine):
    """tlnn_prof_begin/end time a region with CUDA events; tlnn_prof_classes/table give per-kernel-class launches and
    times; tlnn_device_info and tlnn_d2h_async are part of the same ABI."""
    import ctypes as C
    from torchless_nn_b200 import _lib, backend
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.layers import LayerNorm
    ctx = backend.ctx()
    sm, total, free = C.c_int(), C.c_size_t(), C.c_size_t()
    check(lib.tlnn_device_info(ctx, C.byref(sm), C.byref(total), C.byref(free)))
    assert sm.value >= 100 and 0 < free.value <= total.value and total.value > 100 << 30
    ln = LayerNorm(256)
    x = np.random.default_rng(3).standard_normal((512, 256), dtype=np.float32)
    ln.forward(x)
    ms = C.c_float(-1.0)
    check(lib.tlnn_prof_begin(ctx))
    check(lib.tlnn_prof_classes(ctx, 1))
    before = backend.launch_count()
    for _ in range(3):
        y = ln.forward(x)
    check(lib.tlnn_prof_end(ctx, C.byref(ms)))
    rows = (_lib.ProfRow * 32)()
    n = lib.tlnn_prof_table(ctx, rows, 32)
    check(lib.tlnn_prof_classes(ctx, 0))
    assert ms.value > 0.0 and backend.launch_count() - before >= 3
    table = {r.name.decode(): (r.launches, r.ms) for r in rows[:n]}
    assert any(k.startswith("layernorm") and v[0] == 3 and v[1] > 0 for k, v in table.items()), table
    # asynchronous copy back into pinned memory, completed by tlnn_sync
    hp = C.c_void_p()
    check(lib.tlnn_host_alloc(y.nbytes, C.byref(hp)))
    try:
        host = np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_float)), shape=y.shape)
        host[...] = 0
        check(lib.tlnn_d2h_async(ctx, hp, y.ptr, y.nbytes))
        check(lib.tlnn_sync(ctx))
        assert np.array_equal(host, y.get())
    finally:
        lib.tlnn_host_free(hp)
