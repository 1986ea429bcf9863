"""Build libtlnn.so (the sm_100a engine) in-tree with nvcc.

    python -m torchless_nn_b200.build [--force] [--debug]

The library is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); nvcc cross-compiles on a
machine without a GPU.  Object files go to ``torchless_nn_b200/build/``; the shared library is written next to this
file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libtlnn.so")
SOURCES = ["api.cu", "rowops.cu", "gemm_tcgen05.cu", "attention.cu", "attention_tcgen05.cu", "attention_tf32.cu", "layers.cu", "decode.cu", "decode_fused.cu", "noalloc.cu", "comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libtlnn.so cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> str:
    """debug=True builds libtlnn_debug.so with -DTLNN_DEBUG (bounds checks in the kernels' stores)."""
    obj_dir = OBJ + ("_debug" if debug else "")
    lib_path = os.path.join(HERE, "libtlnn_debug.so") if debug else LIB
    flags = NVCC_FLAGS + (["-DTLNN_DEBUG"] if debug else [])
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "tlnn.h"))
    nvcc = _nvcc()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            jobs.append([nvcc, *flags, *(["-Xptxas", "-v"] if verbose else []), "-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=4) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        print("\n".join(logs))
    objs = [os.path.join(obj_dir, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(lib_path, objs):
        run([nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl"])
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug="--debug" in sys.argv))
