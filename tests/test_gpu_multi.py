"""GPU tests of the batch-sharded product path: `Network.predict_tokens(..., comm=)`, `predict_logits(..., comm=)` and
`generate_greedy(..., comm=)` over the library's NCCL communicator (`tlnn_comm_*`, `tlnn_allgather_*`).

A communicator of one rank runs on any box.  The two-rank cases start one child process per GPU and are skipped on a
box with a single GPU; every rank checks the gathered result of the whole batch against the NumPy oracle, so a rank
that wrote its rows to the wrong place fails the test."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import TOL
from oracle import forward_np as onp
from torchless_nn_b200 import workloads as wl

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count() -> int:
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=60).stdout
        return sum(1 for ln in out.splitlines() if ln.startswith("GPU "))
    except Exception:
        return 1


def test_single_rank_communicator(engine):
    from torchless_nn_b200.comm import Communicator
    from torchless_nn_b200.device_array import DeviceArray
    from torchless_nn_b200.models import build_seeded
    comm = Communicator(0, 1, Communicator.unique_id())
    try:
        assert (comm.rank, comm.world) == (0, 1)
        local = DeviceArray.from_numpy(np.arange(12, dtype=np.int32).reshape(3, 4))
        assert np.array_equal(comm.allgather_tokens(local).get(), local.get())
        assert np.array_equal(comm.allgather_tokens(local, [3]).get(), local.get())
        with pytest.raises(ValueError):
            comm.allgather_tokens(local, [2])                       # does not describe this rank's rows
        with pytest.raises(TypeError):
            comm.allgather_logits(local)                            # int32 passed where float32 is expected
        comm.barrier()
        assert comm.max_over_ranks(3.5) == 3.5
        spec, net = build_seeded("c1")
        x = wl.make_inputs(spec, 3)
        assert np.array_equal(net.predict_tokens(x, comm=comm).get(), net.predict_tokens(x).get())
    finally:
        comm.close()
        engine.set_precision("tf32")


def test_injected_init_failure_is_reported(engine, monkeypatch):
    """Host-side fault injection: the refusal comes back as a status and a message, before any GPU or network work."""
    from torchless_nn_b200.comm import Communicator
    ident = Communicator.unique_id()
    monkeypatch.setenv("TLNN_COMM_FAIL_INIT", "1")
    with pytest.raises(RuntimeError, match="TLNN_COMM_FAIL_INIT"):
        Communicator(0, 1, ident)
    monkeypatch.delenv("TLNN_COMM_FAIL_INIT")
    Communicator(0, 1, ident).close()                               # the context is untouched by the refusal


WORKER = r'''
import os, sys
import numpy as np
sys.path.insert(0, os.environ["TLNN_ROOT"])
os.environ.setdefault("XP_RUNTIME", "B200")
from torchless_nn_b200 import workloads as wl
from torchless_nn_b200.comm import Communicator
from torchless_nn_b200.models import build_seeded
from oracle import forward_np as onp

comm = Communicator.from_env(timeout_s=120)
rank, world = comm.rank, comm.world
spec, net = build_seeded("c1")
params = wl.seeded_params(spec)
ok = True
for n_rows in (8, 7):                                # an even split and a ragged one
    x = wl.make_inputs(spec, n_rows)
    ref = onp.forward(spec, params, x)
    tol = 2e-3 * float(np.abs(ref).max())
    tokens = net.predict_tokens(x, comm=comm).get()
    a, top, second = onp.top2(ref)
    good, n_diff, n_bad = onp.tokens_match(tokens, a, top, second, tol)
    logits = net.predict_logits(x, comm=comm).get()
    ok = ok and tokens.shape == (n_rows, spec.seq_len) and good and float(np.abs(logits - ref).max()) < tol
    # the gathered rows equal what this rank computes for the whole batch alone
    ok = ok and bool(np.array_equal(tokens, net.predict_tokens(x).get()))
# decode: every rank keeps the cache of its own prompts, rows gathered once at the end
prompts = wl.make_inputs(spec, 6)[:, :16]
out = net.generate_greedy(prompts, 12, comm=comm).get()
alone = net.generate_greedy(prompts, 12).get()
ok = ok and out.shape == (6, 28) and bool(np.array_equal(out, alone))
ok = ok and comm.max_over_ranks(float(rank + 1)) == float(world)
comm.barrier()
comm.close()
print("RANK", rank, "OK" if ok else "MISMATCH", flush=True)
sys.exit(0 if ok else 1)
'''


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_ranks_shard_gather_and_decode(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), TLNN_ROOT=ROOT,
                   TLNN_RDZV_FILE=str(tmp_path / "rdzv"))
        env.pop("TLNN_DEVICE", None)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"RANK {rank} OK" in out
