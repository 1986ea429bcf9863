"""The allocation-free arg-max head (tlnn_logits_tokens_noalloc) against the regular entry point.

Some hosts cannot allocate device memory when they call into the library - their own allocator owns the GPU, or the
call sits in a loop that must not stall - so this one entry point works out of an array compiled into the library.
The test calls it through the C ABI twice in a row, with different inputs, and requires the tokens to equal those of
tlnn_logits_fwd, which proves that leftovers of the first call do not leak into the second.  It lives in a file that
sorts last so that a run stopping at the first failure has already exercised everything else.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_bytes(ctx) -> int:
    import ctypes as C
    from torchless_nn_b200._lib import lib, check
    free = C.c_size_t()
    check(lib.tlnn_sync(ctx))
    check(lib.tlnn_device_info(ctx, None, None, C.byref(free)))
    return int(free.value)


@pytest.mark.parametrize("prec", ["bf16", "tf32"])
def test_noalloc_head_matches_regular_head_twice(engine, prec):
    from torchless_nn_b200 import _lib
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.device_array import DeviceArray
    from torchless_nn_b200.utils import PreparedWeight

    engine.set_precision(prec)
    try:
        ctx = engine.ctx()
        code = engine.precision_code()
        rng = np.random.default_rng(11)
        d, vocab = 256, 5003
        table = DeviceArray.from_numpy(rng.standard_normal((vocab, d), dtype=np.float32) * np.float32(0.05))
        head = PreparedWeight(table, transpose=False)
        bias = DeviceArray.from_numpy(rng.standard_normal(vocab, dtype=np.float32) * np.float32(0.01))
        for rows in (300, 77):                      # two calls in a row share the built-in scratch
            x = DeviceArray.from_numpy(rng.standard_normal((rows, d), dtype=np.float32))
            want = DeviceArray((rows,), np.int32)
            got = DeviceArray((rows,), np.int32)
            check(lib.tlnn_logits_fwd(ctx, code, x.ptr, head.ptr(), bias.ptr, None, want.ptr, rows, d, vocab))
            check(lib.tlnn_logits_tokens_noalloc(ctx, code, x.ptr, head.ptr(), bias.ptr, got.ptr, rows, d, vocab))
            w, g = want.get(), got.get()
            assert np.array_equal(g, w)
            # the promise itself: a warmed call leaves the device's free memory exactly where it was
            before = _free_bytes(ctx)
            check(lib.tlnn_logits_tokens_noalloc(ctx, code, x.ptr, head.ptr(), bias.ptr, got.ptr, rows, d, vocab))
            check(lib.tlnn_sync(ctx))
            assert _free_bytes(ctx) == before
            assert np.array_equal(got.get(), w)
            # and both agree with a float64 product wherever the top-2 gap is clear of the mode's rounding
            ref = x.get().astype(np.float64) @ table.get().astype(np.float64).T + bias.get()
            order = np.sort(ref, axis=1)
            clear = (order[:, -1] - order[:, -2]) > (3e-2 if prec == "bf16" else 2e-3) * np.abs(ref).max()
            assert np.array_equal(g[clear], np.argmax(ref, axis=1)[clear])
    finally:
        engine.set_precision("tf32")


def test_noalloc_head_refuses_shapes_beyond_its_scratch(engine):
    from torchless_nn_b200 import _lib
    from torchless_nn_b200._lib import lib
    from torchless_nn_b200.device_array import DeviceArray
    ctx = engine.ctx()
    d, vocab, rows = 1024, 50257, 1 << 16            # 64 Ki rows need far more than the built-in 16 MiB
    dummy = DeviceArray((16,), np.float32)            # never dereferenced: the size check comes first
    tokens = DeviceArray((16,), np.int32)
    status = lib.tlnn_logits_tokens_noalloc(ctx, _lib.PREC_BF16, dummy.ptr, dummy.ptr, None, tokens.ptr, rows, d, vocab)
    assert status == _lib.ERR_VALUE
    assert b"scratch" in lib.tlnn_last_error()
    with pytest.raises(ValueError):
        _lib.check(status)
