"""Bandwidth check of the row kernels (embedding gather, LayerNorm, SoftMax, arg-max) through the C ABI.

    python -m torchless_nn_b200.rowbench [embed|layernorm|softmax|argmax|all] [--rows N] [--cols N] [--iters K]

Each kernel is timed with CUDA events on the engine's stream over K launches after warm-up, on operands larger than
the 126 MB L2 unless the defaults are overridden, and reported as achieved GB/s of its algorithmic bytes (what the
reference's array operations must read and write at least once: transformer_adapters.py:150-151, layers.py:419-427,
activations.py:60-63, network.py:135).  The same invocations are what the ncu summaries under profiles/ were taken on.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import numpy as np

os.environ.setdefault("XP_RUNTIME", "B200")


def _time(fn, iters: int) -> float:
    from . import backend
    from ._lib import lib, check
    ctx = backend.ctx()
    for _ in range(3):
        fn()
    backend.synchronize()
    ms = C.c_float()
    check(lib.tlnn_prof_begin(ctx))
    for _ in range(iters):
        fn()
    check(lib.tlnn_prof_end(ctx, C.byref(ms)))
    return float(ms.value) / iters


def bench_embed(rows: int, cols: int, iters: int) -> dict:
    """rows = tokens (B x T with T = 1024), cols = model width; Zipf(1.1) ids over a 50257-row table."""
    from . import backend, workloads as wl
    from ._lib import lib, check, I32
    from .device_array import DeviceArray
    T = 1024
    B = max(rows // T, 1)
    vocab = 50257
    rng = np.random.default_rng(0)
    table = DeviceArray.from_numpy(rng.standard_normal((vocab, cols), dtype=np.float32))
    pos = DeviceArray.from_numpy(rng.standard_normal((T, cols), dtype=np.float32))
    ids = DeviceArray.from_numpy(wl.token_ids(vocab, (B, T), 3, "zipf"))
    out = DeviceArray((B, T, cols), np.float32)
    ctx = backend.ctx()
    ms = _time(lambda: check(lib.tlnn_embed_fwd(ctx, ids.ptr, I32, table.ptr, pos.ptr, out.ptr, B, T, cols, vocab)), iters)
    touched = len(np.unique(ids.get()))
    algo = B * T * cols * 4 + B * T * 4 + touched * cols * 4 + T * cols * 4       # output + ids + touched table rows + positions
    return {"kernel": "embed_kernel", "shape": [B, T, cols], "ms": ms, "algorithmic_bytes": algo, "gbs": algo / ms / 1e6}


def bench_layernorm(rows: int, cols: int, iters: int) -> dict:
    from . import backend
    from ._lib import lib, check
    from .device_array import DeviceArray
    rng = np.random.default_rng(1)
    x = DeviceArray.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32))
    g = DeviceArray.from_numpy(np.ones(cols, dtype=np.float32))
    b = DeviceArray.from_numpy(np.zeros(cols, dtype=np.float32))
    out = DeviceArray((rows, cols), np.float32)
    ctx = backend.ctx()
    ms = _time(lambda: check(lib.tlnn_layernorm_fwd(ctx, x.ptr, g.ptr, b.ptr, 1e-5, out.ptr, rows, cols)), iters)
    algo = rows * cols * 8
    return {"kernel": "layernorm_warp_kernel (float32 out)", "shape": [rows, cols], "ms": ms, "algorithmic_bytes": algo,
            "gbs": algo / ms / 1e6}


def bench_softmax(rows: int, cols: int, iters: int) -> dict:
    from . import backend
    from ._lib import lib, check
    from .device_array import DeviceArray
    rng = np.random.default_rng(2)
    x = DeviceArray.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32))
    out = DeviceArray((rows, cols), np.float32)
    ctx = backend.ctx()
    ms = _time(lambda: check(lib.tlnn_softmax_fwd(ctx, x.ptr, out.ptr, rows, cols, 1.0)), iters)
    algo = rows * cols * 8
    return {"kernel": "softmax_kernel", "shape": [rows, cols], "ms": ms, "algorithmic_bytes": algo, "gbs": algo / ms / 1e6}


def bench_argmax(rows: int, cols: int, iters: int) -> dict:
    from . import backend
    from ._lib import lib, check
    from .device_array import DeviceArray
    rng = np.random.default_rng(3)
    x = DeviceArray.from_numpy(rng.standard_normal((rows, cols), dtype=np.float32))
    out = DeviceArray((rows,), np.int32)
    ctx = backend.ctx()
    ms = _time(lambda: check(lib.tlnn_argmax_fwd(ctx, x.ptr, cols, out.ptr, rows, cols)), iters)
    algo = rows * cols * 4 + rows * 4
    return {"kernel": "argmax_kernel", "shape": [rows, cols], "ms": ms, "algorithmic_bytes": algo, "gbs": algo / ms / 1e6}


DEFAULTS = {"embed": (65536, 768), "layernorm": (131072, 1024), "softmax": (2048, 50257), "argmax": (2048, 50257)}
BENCH = {"embed": bench_embed, "layernorm": bench_layernorm, "softmax": bench_softmax, "argmax": bench_argmax}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all", choices=["all"] + sorted(BENCH))
    ap.add_argument("--rows", type=int, default=0)
    ap.add_argument("--cols", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args(argv)
    peak = 6546.6
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f)["hbm_gbs"])
    except Exception:
        pass
    for name in (sorted(BENCH) if a.which == "all" else [a.which]):
        rows, cols = DEFAULTS[name]
        r = BENCH[name](a.rows or rows, a.cols or cols, a.iters)
        r["frac_of_measured_copy_rate"] = r["gbs"] / peak
        print(json.dumps(r), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
