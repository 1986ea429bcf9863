"""CPU tests of the multi-rank host logic, run as two gloo ranks.
`Network.predict_tokens(..., comm=)` shards the global batch by contiguous rows and gathers int32 arg-max tokens through
`torchless_nn_b200.comm.sharded_rows`; that function is driven here with a gloo communicator of the same shape and the
oracle standing in for the engine (no GPU is touched), on an even and on a ragged split.  The file rendezvous that
hands rank 0's communicator identifier to the other ranks is tested with real processes."""
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
from torchless_nn_b200.comm import sharded_rows, shard_counts
from oracle import forward_np as onp

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")


class GlooComm:
    # the two members and the gather signature of torchless_nn_b200.comm.Communicator, over gloo and host arrays
    def __init__(self):
        self.rank, self.world = rank, world

    def allgather_tokens(self, local, rows_per_rank):
        assert rows_per_rank[self.rank] == local.shape[0]
        # one broadcast per rank, as the library does for ragged shards
        parts = [torch.from_numpy(np.ascontiguousarray(local)) if r == self.rank
                 else torch.empty((n,) + local.shape[1:], dtype=torch.int32) for r, n in enumerate(rows_per_rank)]
        for r, part in enumerate(parts):
            dist.broadcast(part, src=r)
        return torch.cat(parts).numpy()


comm = GlooComm()
spec = wl.CONFIGS["c1"]
params = wl.seeded_params(spec)
ok = True
for n_rows in (8, 7):            # an even split and a ragged one (4 + 3)
    ids = wl.make_inputs(spec, n_rows)
    seen = []

    def run_local(lo, hi):
        seen.append((lo, hi))
        return np.argmax(onp.forward(spec, params, ids[lo:hi]), axis=-1).astype(np.int32)

    got = sharded_rows(comm, n_rows, run_local, comm.allgather_tokens)
    full = np.argmax(onp.forward(spec, params, ids), axis=-1).astype(np.int32)
    ok = ok and seen == [wl.shard_rows(n_rows, rank, world)] and bool(np.array_equal(got, full))
    ok = ok and sum(shard_counts(n_rows, world)) == n_rows
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


def test_identifier_rendezvous_between_processes(tmp_path):
    """Rank 0 publishes 128 bytes atomically; another process that started earlier polls and reads exactly them."""
    base = str(tmp_path / "rdzv")
    reader = subprocess.Popen([sys.executable, "-c",
                               "import os,sys; sys.path.insert(0, os.environ['TLNN_ROOT']);"
                               "from torchless_nn_b200.comm import await_id, rendezvous_path;"
                               "sys.stdout.buffer.write(await_id(rendezvous_path(3), 30))"],
                              env=dict(os.environ, TLNN_ROOT=ROOT, TLNN_RDZV_FILE=base), stdout=subprocess.PIPE)
    from torchless_nn_b200.comm import publish_id, await_id
    ident = bytes(range(128))
    publish_id(base + ".3", ident)
    out, _ = reader.communicate(timeout=60)
    assert reader.returncode == 0 and out == ident
    import pytest
    with pytest.raises(TimeoutError):
        await_id(base + ".4", 0.05)          # nobody publishes communicator 4: bounded wait, then an error


def test_rendezvous_names_differ_per_launch(monkeypatch):
    from torchless_nn_b200 import comm
    monkeypatch.delenv("TLNN_RDZV_FILE", raising=False)
    monkeypatch.setenv("MASTER_PORT", "29511")
    a = comm.rendezvous_path(0)
    monkeypatch.setenv("MASTER_PORT", "29512")
    assert comm.rendezvous_path(0) != a and comm.rendezvous_path(1) != comm.rendezvous_path(0)
    assert str(os.getppid()) in a


def test_comm_entry_points_validate_on_the_host(monkeypatch):
    """No GPU here: the communicator calls must refuse bad arguments, and the injected init failure must surface
    before any device or network work."""
    import ctypes as C
    from torchless_nn_b200 import _lib
    lib = _lib.lib
    assert lib.tlnn_comm_unique_id(None) == _lib.ERR_NULL
    assert lib.tlnn_comm_init(None, b"\0" * 128, 0, 1, None) == _lib.ERR_NULL
    assert lib.tlnn_allgather_tokens(None, None, None, 0, None) == _lib.ERR_NULL
    assert lib.tlnn_comm_barrier(None) == _lib.ERR_NULL
    assert lib.tlnn_comm_destroy(None) == _lib.OK
    v = C.c_int()
    if lib.tlnn_comm_nccl_version(C.byref(v)) == _lib.OK:
        assert v.value >= 22000
        buf = C.create_string_buffer(128)
        assert lib.tlnn_comm_unique_id(buf) in (_lib.OK, _lib.ERR_CUDA)
