"""CPU tests of the multi-rank host logic: batch sharding and the token all-gather, run as two gloo ranks.
The GPU path shards the global batch by contiguous rows and gathers int32 arg-max tokens; the same functions are
exercised here with the oracle standing in for the engine (no GPU is touched)."""
import os
import socket
import subprocess
import sys

import numpy as np

from torchless_nn_b200 import workloads as wl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["TLNN_ROOT"])
from torchless_nn_b200 import workloads as wl
from oracle import forward_np as onp

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
spec = wl.CONFIGS["c1"]
params = wl.seeded_params(spec)
ids = wl.make_inputs(spec, 8)
lo, hi = wl.shard_rows(len(ids), rank, world)
local = np.argmax(onp.forward(spec, params, ids[lo:hi]), axis=-1).astype(np.int32)
t_local = torch.from_numpy(np.ascontiguousarray(local))
t_all = torch.empty((len(ids), ids.shape[1]), dtype=torch.int32)
dist.all_gather_into_tensor(t_all.view(-1), t_local.view(-1))
full = np.argmax(onp.forward(spec, params, ids), axis=-1).astype(np.int32)
ok = bool(np.array_equal(t_all.numpy(), full))
# timing reduction used by the benchmark: the maximum over ranks
t = torch.tensor([float(rank + 1)], dtype=torch.float64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)
ok = ok and t.item() == float(world)
dist.barrier()
dist.destroy_process_group()
print("RANK", rank, "OK" if ok else "MISMATCH", flush=True)
sys.exit(0 if ok else 1)
'''


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), TLNN_ROOT=ROOT, OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"RANK {rank} OK" in out


def test_shards_cover_the_batch_exactly_once():
    for n_rows in (64, 16, 10, 3):
        for world in (1, 2, 4, 8):
            spans = [wl.shard_rows(n_rows, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n_rows
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_reference_arm_exits_quietly_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "0"], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""
