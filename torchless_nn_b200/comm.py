"""Batch-sharded replicas: one process per GPU, every rank runs a contiguous slice of the batch rows.

The reference is single-device (``Network.predict``, network.py:33-39).  Rows of an eval-mode forward are independent,
so N processes each holding a full copy of the weights split the batch by rows and exchange results only: the int32
arg-max tokens (or float32 logits) of every rank are all-gathered.  ``Communicator`` wraps the library's NCCL entry
points (``tlnn_comm_*``, ``tlnn_allgather_*``); no PyTorch is involved.

Launchers: anything that starts N processes with ``RANK``, ``WORLD_SIZE`` and ``LOCAL_RANK`` set works
(``python -m torch.distributed.run --nproc-per-node N script.py`` is one such launcher; the script itself need not
import torch).  ``Communicator.from_env()`` hands rank 0's identifier to the other ranks of the node through a file;
with any other means of exchange, create the identifier with ``Communicator.unique_id()`` on rank 0 and pass it to the
constructor on every rank.

``sharded_rows`` is the host logic shared by ``Network.predict_tokens(..., comm=)`` and
``Network.generate_greedy(..., comm=)``: slice, run the local rows, gather in rank order.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os
import tempfile
import time

import numpy as np

from .workloads import shard_rows

ID_BYTES = 128
_sequence = 0        # communicators created by from_env in this process (all ranks create them in the same order)


def _prefer_bundled_nccl() -> None:
    """The NCCL that ships inside the Python environment (package nvidia.nccl) is the one the other CUDA libraries of
    the environment were built and tested with; use it unless the caller named a library."""
    if os.environ.get("TLNN_NCCL_LIB"):
        return
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    if spec and spec.submodule_search_locations:
        for base in spec.submodule_search_locations:
            path = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(path):
                os.environ["TLNN_NCCL_LIB"] = path
                return


def rendezvous_path(sequence: int) -> str:
    """File through which rank 0 of this launch publishes communicator number ``sequence``.  The name is unique per
    launch on a node: the launcher's process id (all ranks are its children) and its rendezvous port."""
    explicit = os.environ.get("TLNN_RDZV_FILE")
    if explicit:
        return f"{explicit}.{sequence}"
    tag = f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}_{os.environ.get('TORCHELASTIC_RUN_ID', 'none')}"
    return os.path.join(tempfile.gettempdir(), f"tlnn_rdzv_{tag}.{sequence}")


def publish_id(path: str, ident: bytes) -> None:
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(ident)
    os.replace(tmp, path)          # atomic: a reader sees the whole identifier or no file


def await_id(path: str, timeout_s: float) -> bytes:
    deadline = time.monotonic() + timeout_s
    while True:
        try:
            with open(path, "rb") as f:
                data = f.read()
            if len(data) == ID_BYTES:
                return data
        except FileNotFoundError:
            pass
        if time.monotonic() > deadline:
            raise TimeoutError(f"rank 0 did not publish a communicator identifier at {path} within {timeout_s:.0f} s")
        time.sleep(0.01)


def shard_counts(n_rows: int, world: int) -> list[int]:
    return [hi - lo for lo, hi in (shard_rows(n_rows, r, world) for r in range(world))]


def sharded_rows(comm, n_rows: int, run_local, gather):
    """Run ``run_local(lo, hi)`` on this rank's rows ``[lo, hi)`` of ``n_rows`` and return
    ``gather(local_result, rows_per_rank)``: every rank's rows in rank order, i.e. in the original row order."""
    lo, hi = shard_rows(n_rows, comm.rank, comm.world)
    return gather(run_local(lo, hi), shard_counts(n_rows, comm.world))


class Communicator:
    """NCCL communicator of the engine's context in this process."""

    def __init__(self, rank: int, world: int, ident: bytes):
        from . import backend
        from ._lib import lib, check
        if len(ident) != ID_BYTES:
            raise ValueError(f"a communicator identifier has {ID_BYTES} bytes")
        _prefer_bundled_nccl()
        self.rank, self.world = int(rank), int(world)
        h = C.c_void_p()
        check(lib.tlnn_comm_init(backend.ctx(), ident, self.rank, self.world, C.byref(h)))
        self._h = h

    @staticmethod
    def unique_id() -> bytes:
        from ._lib import lib, check
        _prefer_bundled_nccl()
        buf = C.create_string_buffer(ID_BYTES)
        check(lib.tlnn_comm_unique_id(buf))
        return buf.raw

    @classmethod
    def from_env(cls, timeout_s: float = 300.0) -> "Communicator":
        global _sequence
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        path = rendezvous_path(_sequence)
        _sequence += 1
        if rank == 0:
            ident = cls.unique_id()
            if world > 1:
                publish_id(path, ident)
        else:
            ident = await_id(path, timeout_s)
        try:
            return cls(rank, world, ident)       # returns once every rank has joined: all have read the file
        finally:
            if rank == 0 and world > 1:
                try:
                    os.remove(path)
                except OSError:
                    pass

    # ---- collectives (device arrays, on the engine's stream) ------------------------------------------------------
    def _gather(self, fn, local, rows_per_rank, dtype):
        from ._lib import check
        from .device_array import DeviceArray
        if local.dtype != dtype:
            raise TypeError(f"expected a {np.dtype(dtype)} device array")
        per_row = int(np.prod(local.shape[1:], dtype=np.int64))
        if rows_per_rank is None:
            rows_per_rank = [local.shape[0]] * self.world
        if len(rows_per_rank) != self.world or rows_per_rank[self.rank] != local.shape[0]:
            raise ValueError("rows_per_rank does not describe this rank's array")
        out = DeviceArray((int(sum(rows_per_rank)),) + tuple(local.shape[1:]), dtype)
        counts = (C.c_longlong * self.world)(*[int(r) * per_row for r in rows_per_rank])
        check(fn(self._h, local.ptr, out.ptr, local.size, counts))
        return out

    def allgather_tokens(self, local, rows_per_rank=None):
        """(rows_r, ...) int32 per rank -> (sum rows, ...) int32 on every rank, rank order."""
        from ._lib import lib
        return self._gather(lib.tlnn_allgather_tokens, local, rows_per_rank, np.int32)

    def allgather_logits(self, local, rows_per_rank=None):
        from ._lib import lib
        return self._gather(lib.tlnn_allgather_logits, local, rows_per_rank, np.float32)

    def barrier(self) -> None:
        from ._lib import lib, check
        check(lib.tlnn_comm_barrier(self._h))

    def max_over_ranks(self, value: float) -> float:
        """Largest of one host number per rank (step times: a multi-GPU step takes as long as its slowest rank)."""
        from .device_array import DeviceArray
        mine = DeviceArray.from_numpy(np.array([value], dtype=np.float32))
        return float(self.allgather_logits(mine).get().max())

    def close(self) -> None:
        from ._lib import lib
        if self._h is not None:
            lib.tlnn_comm_destroy(self._h)
            self._h = None
