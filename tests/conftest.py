import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
os.environ.setdefault("XP_RUNTIME", "B200")

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def golden():
    cache = {}

    def load(name):
        if name not in cache:
            cache[name] = np.load(os.path.join(GOLDEN, name + ".npz"))
        return cache[name]
    return load


@pytest.fixture(scope="session")
def engine():
    """The device context; a GPU test fails (not skips) when the library or the GPU is missing.  The whole GPU session
    runs with canary-padded allocations (no memory checker is available on the test machines): every device array is
    followed by 256 bytes of a known pattern, verified when it is freed, after every test and at the end."""
    import ctypes as C
    from torchless_nn_b200 import backend
    from torchless_nn_b200._lib import lib, check
    ctx = backend.ctx()
    check(lib.tlnn_debug_canaries(ctx, 1))
    yield backend
    backend.synchronize()
    bad, live = C.c_longlong(), C.c_longlong()
    check(lib.tlnn_debug_check(ctx, C.byref(bad), C.byref(live)))
    assert bad.value == 0, f"{bad.value} device allocations were written past their end during the session"


@pytest.fixture(autouse=True)
def _canaries_intact_after_each_gpu_test(request):
    yield
    if request.node.get_closest_marker("gpu") is None or "engine" not in request.fixturenames:
        return
    import ctypes as C
    from torchless_nn_b200 import backend
    from torchless_nn_b200._lib import lib, check
    bad, live = C.c_longlong(), C.c_longlong()
    check(lib.tlnn_debug_check(backend.ctx(), C.byref(bad), C.byref(live)))
    assert bad.value == 0, f"{request.node.name}: {bad.value} device allocations were written past their end ({live.value} guarded)"


def rel_err(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


TOL = {"tf32": 2e-3, "bf16": 3e-2}
