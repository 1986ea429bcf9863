"""CPU tests of the boundary: the shared library loads, exports every symbol the header declares, validates its
arguments on the host before touching a device, and fails loudly without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tlnn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tlnn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from torchless_nn_b200 import _lib
    names = _declared()
    assert len(names) >= 40
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} is declared in tlnn.h but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == names
    assert _lib.lib.tlnn_version() >= 100


def test_status_codes_map_to_reference_exception_classes():
    from torchless_nn_b200 import _lib
    for code, exc in ((_lib.ERR_VALUE, ValueError), (_lib.ERR_INDEX, IndexError), (_lib.ERR_CUDA, RuntimeError),
                      (_lib.ERR_NOMEM, MemoryError), (_lib.ERR_TIMEOUT, RuntimeError), (_lib.ERR_NULL, ValueError)):
        with pytest.raises(exc):
            _lib.check(code)
    _lib.check(_lib.OK)


def test_null_and_bad_arguments_are_rejected_on_the_host():
    from torchless_nn_b200 import _lib
    lib = _lib.lib
    assert lib.tlnn_init(0, None) == _lib.ERR_NULL
    assert lib.tlnn_sync(None) == _lib.ERR_NULL
    assert lib.tlnn_layernorm_fwd(None, None, None, None, 1e-5, None, 1, 8) == _lib.ERR_NULL
    assert lib.tlnn_gpt_prefill(None, None, None, 2, 1, 1, None, None) == _lib.ERR_NULL
    assert b"null" in lib.tlnn_last_error()
    assert lib.tlnn_launch_count(None, 0) == 0
    assert lib.tlnn_decode_end(None) in (_lib.OK, _lib.ERR_NULL)


def test_no_gpu_means_an_error_not_a_fallback():
    """On a machine without a GPU the engine refuses to start; nothing computes on the CPU."""
    from torchless_nn_b200 import _lib
    h = C.c_void_p()
    status = _lib.lib.tlnn_init(0, C.byref(h))
    if status == _lib.OK:
        _lib.lib.tlnn_shutdown(h)
        pytest.skip("a GPU is present")
    assert status == _lib.ERR_CUDA
    with pytest.raises(RuntimeError):
        _lib.check(status)


def test_backend_rejects_other_runtimes(monkeypatch):
    import importlib
    import torchless_nn_b200.backend as be
    monkeypatch.setenv("XP_RUNTIME", "CPU")
    with pytest.raises(AssertionError):
        importlib.reload(be)
    monkeypatch.setenv("XP_RUNTIME", "B200")
    importlib.reload(be)
    assert be.runtime == "B200" and be.FLOAT_TYPE is np.float32
    with pytest.raises(ValueError):
        be.set_precision("fp8")


def test_mirror_modules_export_the_reference_names():
    from torchless_nn_b200 import layers, activations, transformer_adapters, network, utils, backend
    for mod, names in ((layers, ["Dense", "Dropout", "MultiHeadAttention", "TransformerFeedForward", "LayerNorm",
                                 "TransformerBlock"]),
                       (activations, ["ReLU", "GeLU", "SiLU", "SoftMax"]),
                       (transformer_adapters, ["VitProjector", "VitMLPHead", "GPTEmbeddingTable", "GPTEmbedFront",
                                               "GPTEmbedBack"]),
                       (network, ["Network"]), (utils, ["Layer", "Residual"]),
                       (backend, ["xp", "FLOAT_TYPE", "runtime", "init_random_tensor", "init_zeros_tensor"])):
        for n in names:
            assert hasattr(mod, n), (mod.__name__, n)
    import inspect
    sig = inspect.signature(layers.TransformerBlock.__init__)
    assert list(sig.parameters)[1:] == ["embed_dim", "context_length", "num_heads", "activation", "decoder",
                                        "attn_dropout_rate", "res_dropout_rate"]
    sig = inspect.signature(layers.MultiHeadAttention.__init__)
    assert list(sig.parameters)[1:] == ["embedding_dim", "context_length", "num_heads", "decoder",
                                        "attn_dropout_rate", "res_dropout_rate"]
    sig = inspect.signature(transformer_adapters.VitProjector.__init__)
    assert list(sig.parameters)[1:] == ["input_size", "patch_size", "embedding_dim", "num_registers"]


def test_product_code_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "torchless_nn_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f"{f} imports the oracle"
                assert "oracle/" not in text and "oracle." not in text, f"{f} reaches into the oracle"


def test_fused_gpt_call_refuses_a_head_of_another_width():
    """The C description of a GPT has one vocabulary size, used both as the id bound and as the head width: a Dense
    head of any other shape must not reach the fused call (it would write past the logits buffer)."""
    from torchless_nn_b200.network import GPTPlan

    class Table:
        vocab_size, embed_size = 65, 128

    class Front:
        embedding_table, context_length = Table(), 128

    class Head:
        class weights:
            shape = (128, 70)

    from torchless_nn_b200 import layers
    plan = GPTPlan(Front(), [], None, Head())
    with pytest.raises(ValueError, match="Dense head"):
        plan.model()


def test_basic_indexing_offsets_match_numpy_and_stay_selection_sized():
    """Device-array indexing computes flat offsets from the strides, axis by axis (no array the size of the whole
    tensor is built on the host): checked against NumPy on a stand-in object, no device needed."""
    from torchless_nn_b200.device_array import DeviceArray

    class Shape:
        def __init__(self, shape):
            self.shape, self.ndim = shape, len(shape)

        def _normalised_key(self, key):
            return DeviceArray._normalised_key(self, key)

    shape = (4, 5, 6)
    a = np.arange(np.prod(shape)).reshape(shape)
    for key in [(0, -1), (slice(None), -1), (1,), (1, slice(2, 4)), (Ellipsis, 2), (2, Ellipsis), -1, slice(1, 4),
                (slice(None), slice(4, 5), slice(None)), (slice(None, None, -1), 0), (slice(2, 2),), (3, 4, 5)]:
        got = DeviceArray._basic_offsets(Shape(shape), key)
        assert got.shape == a[key].shape and np.array_equal(got, a[key]), key
    assert DeviceArray._basic_offsets(Shape(shape), (np.array([0, 1]),)) is None      # advanced index: other path
    with pytest.raises(IndexError):
        DeviceArray._basic_offsets(Shape(shape), (4,))
    big = Shape((64, 2048, 50257))                                                    # the predict(x)[0, -1] idiom
    got = DeviceArray._basic_offsets(big, (0, -1))
    assert got.shape == (50257,) and got[0] == 2047 * 50257


def test_vit_recipe_is_recognised_only_when_it_is_the_recipe():
    """The whole-model ViT call is taken only for VitProjector, [Dropout], encoder blocks of one width, LayerNorm,
    VitMLPHead; anything else runs layer by layer.  Checked on stand-in layers (no device needed)."""
    from torchless_nn_b200 import network
    from torchless_nn_b200.network import ViTPlan

    def stand_in(cls, **attrs):
        obj = cls.__new__(cls)
        obj.__dict__.update(attrs)
        return obj

    class Act:
        def __init__(self, code): self.code = code
        def act_code(self): return self.code

    class Shape:
        def __init__(self, *shape): self.shape = shape

    def block(d, heads, decoder=False, act=1):
        attn = type("A", (), {"embedding_dim": d, "num_heads": heads, "is_decoder": decoder})()
        return stand_in(network.TransformerBlock, attn_block=attn, ffn=Act(act))

    proj = stand_in(network.VitProjector, embedding_dim=192)
    norm = stand_in(network.LayerNorm, gamma=Shape(192))
    head = stand_in(network.VitMLPHead, weights=Shape(192, 10))
    drop = stand_in(network.Dropout, dropout_rate=0.0, eval_mode=True)
    good = [proj, drop, block(192, 6), block(192, 6), norm, head]
    assert ViTPlan.match(good) is not None
    assert ViTPlan.match([proj, norm, head]) is not None                        # no blocks at all
    assert ViTPlan.match([proj, block(192, 6, decoder=True), norm, head]) is None   # a causal block is not the ViT recipe
    assert ViTPlan.match([proj, block(192, 6), block(192, 3), norm, head]) is None  # blocks that differ
    assert ViTPlan.match([proj, block(128, 4), norm, head]) is None                 # a width other than the projector's
    assert ViTPlan.match([proj, block(192, 6), norm, stand_in(network.VitMLPHead, weights=Shape(128, 10))]) is None
    assert ViTPlan.match([proj, block(192, 6), head]) is None                       # no final LayerNorm
    assert ViTPlan.match(good[1:]) is None                                          # no projector
