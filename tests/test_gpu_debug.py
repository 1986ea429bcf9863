"""GPU tests of the memory-safety aids that stand in for a memory checker: canary-padded allocations
(`tlnn_debug_canaries` / `tlnn_debug_check`) and the debug build of the library (`libtlnn_debug.so`, device-side bounds
checks in the stores of the GEMM, attention and decode kernels).  Both run in child processes so that a deliberately
overwritten canary does not count against the session-wide check in conftest.py.  Nothing here faults: the overwrite
stays inside the padded allocation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CANARY = r'''
import ctypes as C, gc, os, sys
sys.path.insert(0, os.environ["TLNN_ROOT"])
os.environ.setdefault("XP_RUNTIME", "B200")
import numpy as np
from torchless_nn_b200 import backend
from torchless_nn_b200._lib import lib, check
from torchless_nn_b200.device_array import DeviceArray
ctx = backend.ctx()
def state():
    bad, live = C.c_longlong(), C.c_longlong()
    check(lib.tlnn_debug_check(ctx, C.byref(bad), C.byref(live)))
    return bad.value, live.value
before = DeviceArray((8,), np.float32)                 # allocated before canaries are on: not guarded
check(lib.tlnn_debug_canaries(ctx, 1))
a = DeviceArray((25,), np.float32)                     # 100 bytes, padded to 112, then 256 canary bytes
b = DeviceArray((64,), np.float32)
assert state() == (0, 2)
check(lib.tlnn_memset(ctx, a.ptr, 0, 100))             # inside the block
a[...] = np.arange(25, dtype=np.float32)
assert state() == (0, 2)
check(lib.tlnn_memset(ctx, a.ptr, 0, 116))             # four bytes into the canary (still inside the padded allocation)
assert state() == (1, 2)
del a                                                  # the overwritten canary is counted when the block is freed, once
gc.collect()                                           # (a device array refers to itself as the root of its views)
assert state() == (1, 1)
del b
gc.collect()
assert state() == (1, 0)
check(lib.tlnn_debug_canaries(ctx, 0))
c = DeviceArray((4,), np.float32)
assert state() == (1, 0)
print("CANARY OK")
'''

FORWARD = r'''
import json, os, sys
sys.path.insert(0, os.environ["TLNN_ROOT"])
os.environ.setdefault("XP_RUNTIME", "B200")
import numpy as np
from torchless_nn_b200 import _lib, backend, workloads as wl
from torchless_nn_b200.models import build_seeded
assert os.path.basename(_lib.LIB_PATH) == os.environ["EXPECT_LIB"], _lib.LIB_PATH
out = {}
spec, net = build_seeded("c1")                          # TF32 GEMMs, float32 attention, untied head
x = wl.make_inputs(spec, 4)
out["c1_tokens"] = net.predict_tokens(x).get().tolist()
out["c1_decode"] = net.generate_greedy(x[:, :20], 8).get().tolist()
small = wl.GPTSpec("dbg", vocab=1000, context=384, d_model=256, heads=4, layers=2, tied_head=True, precision="bf16",
                   batch=3, seq_len=320, input_seed=7, input_dist="zipf")
spec, net = build_seeded(small)                         # bf16: pair/one-CTA GEMMs, tcgen05 attention (hd 64, T >= 192)
x = wl.make_inputs(spec)
out["bf16_tokens"] = net.predict_tokens(x).get().tolist()
out["bf16_logits_sum"] = float(np.abs(net.predict(x).get()).sum())
out["bf16_decode"] = net.generate_greedy(x[:, :40], 6).get().tolist()      # persistent decode kernel when TLNN_DECODE_FUSED=1
backend.synchronize()                                   # a recorded bounds violation would raise IndexError here
print("RESULT " + json.dumps(out))
'''


def _run(script, tmp_path, **env):
    path = tmp_path / "child.py"
    path.write_text(script)
    r = subprocess.run([sys.executable, str(path)], env=dict(os.environ, TLNN_ROOT=ROOT, **env), capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


def test_canary_behind_every_allocation_detects_an_overrun(tmp_path):
    assert "CANARY OK" in _run(CANARY, tmp_path)


def test_debug_build_runs_clean_and_agrees_with_the_regular_build(tmp_path):
    assert os.path.exists(os.path.join(ROOT, "torchless_nn_b200", "libtlnn_debug.so")), \
        "build it with `python -m torchless_nn_b200.build --debug`"
    res = {}
    for name, env in (("regular", dict(TLNN_DEBUG="0", EXPECT_LIB="libtlnn.so")),
                      ("debug", dict(TLNN_DEBUG="1", EXPECT_LIB="libtlnn_debug.so"))):
        out = _run(FORWARD, tmp_path, TLNN_DECODE_FUSED="1", **env)
        res[name] = json.loads(out.split("RESULT ", 1)[1])
    # the checks only guard stores: results are the same numbers (the second feed-forward product of the persistent
    # decode kernel adds its four K ranges in no fixed order, so its tokens are compared up to the first fork only)
    for key in ("c1_tokens", "c1_decode", "bf16_tokens"):
        assert res["regular"][key] == res["debug"][key], key
    assert abs(res["regular"]["bf16_logits_sum"] - res["debug"]["bf16_logits_sum"]) <= 1e-3 * res["regular"]["bf16_logits_sum"]
    a, b = np.array(res["regular"]["bf16_decode"]), np.array(res["debug"]["bf16_decode"])
    assert a.shape == b.shape == (3, 46) and np.array_equal(a[:, :41], b[:, :41])
