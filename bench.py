#!/usr/bin/env python
"""Benchmark of the transformer forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config c5|c3]

One "step" is one prefill of the whole workload: the GPT-2-medium-shape configuration (vocab 50257, context 2048,
width 1024, 16 heads, 24 layers, bf16 weights with float32 accumulation) on a global batch of 64 sequences of 2048
Zipf-distributed token ids, producing the arg-max token of every position.  The batch is sharded by rows over the
N ranks (one process per GPU, started by any launcher that sets RANK / WORLD_SIZE / LOCAL_RANK, e.g.
torch.distributed.run; this script does not import torch); the only collective is an NCCL all-gather of the int32
tokens, issued by the library on the engine's stream.  Total work is fixed as N grows ("scaling": "strong").

Printed by rank 0 as one JSON line:
  value      tokens/s with the token ids already resident in device memory (CUDA events on the engine's stream,
             maximum over ranks);
  e2e        the same metric through the public API (Network.predict_tokens) with host buffers: pinned host ids
             copied to the device and the tokens copied back inside the timed region, every step;
  roofline   tensor-core GEMM class: algorithmic FLOPs of a step's GEMM launches / their summed CUDA-event durations,
             against the measured cuBLAS bf16 rate in MEASURED_PEAKS.json.  The per-launch events are taken in a second,
             untimed pass: bracketing every launch serialises them and switches the captured-graph replay off, so the
             timed region runs without them;
  parity     the gathered tokens of the fixture's global rows against the reference's arg-max under the tie rule;
  decode     greedy decode tokens/s of the c4 configuration (64/N prompts and their KV cache per GPU);
  cpu_baseline  the NumPy restatement of the reference's forward, timed on the host cores on a bounded sample.

`--impl reference` times that CPU restatement alone (rank 0 only), one bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("XP_RUNTIME", "B200")

import numpy as np  # noqa: E402

from torchless_nn_b200 import workloads as wl  # noqa: E402

METRIC = "gpt_prefill_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_BF16_TFLOPS = 1590.0

def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json, sustained cuBLAS bf16)"
    except Exception:
        return FALLBACK_BF16_TFLOPS, "fallback (1.59 PFLOP/s burst, earlier measurement on this pool)"


# ------------------------------------------------------------------------------------------------ clocks sampler
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        """Only samples taken after this call count (the sampler is started early because nvidia-smi takes a
        moment to deliver its first line)."""
        self.since = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        since = getattr(self, "since", 0.0)
        for stamp, ln in self.lines:
            if stamp < since:
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU baseline
def cpu_sample(spec, params, ids_row, block_index: int):
    """One bounded sample of the reference's CPU algorithm at the workload's full context: the embedding, ONE of
    the L identical-cost blocks, the final LayerNorm and the head on one whole sequence.  Returns the seconds of
    each part; the whole-model time of that sequence is embed + L * block + tail."""
    from oracle import forward_np as onp
    x_ids = ids_row[None, :]
    t0 = time.perf_counter()
    x = onp.embed_front(x_ids, params[1], params[0])
    t1 = time.perf_counter()
    p = params[2 + 12 * block_index: 2 + 12 * (block_index + 1)]
    x = onp.block(x, p, spec.heads, onp.causal_mask(spec.context), "gelu")
    t2 = time.perf_counter()
    k = 2 + 12 * spec.layers
    h = onp.layer_norm(x, params[k], params[k + 1])
    logits = onp.tied_logits(h, params[1]) if spec.tied_head else onp.dense(h, params[k + 2], params[k + 3])
    np.argmax(logits, axis=-1)
    t3 = time.perf_counter()
    return t1 - t0, t2 - t1, t3 - t2


def cpu_threads() -> int:
    """Give the BLAS behind NumPy every core this process may run on, and say how many that is.  A launcher that
    exports OMP_NUM_THREADS=1 to its workers (torch.distributed.run does) would otherwise halve the baseline."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=n, user_api="blas")        # stays in force: the returned object is not used as a context
        got = [i.get("num_threads", 0) for i in threadpool_info() if i.get("user_api") == "blas"]
        if got:
            return int(max(got))
    except Exception:
        pass
    return n


def cpu_tokens_per_s(spec, params, ids, n_samples: int):
    rates = []
    for i in range(n_samples):
        e, b, t = cpu_sample(spec, params, ids[i % len(ids)], i % spec.layers)
        rates.append(spec.seq_len / (e + spec.layers * b + t))
    return statistics.median(rates)


CPU_SAMPLE_TEXT = ("one of the {B} sequences at the full {T}-token context through the NumPy restatement of the "
                   "reference's forward: embedding, 1 of {L} (identical-cost) blocks, final LayerNorm, head and arg-max "
                   "timed; sequence time = embed + {L} x block + tail")


def dtype_of(spec) -> str:
    """Arithmetic type of the path for this configuration: bf16 operands (float32 accumulation) or TF32."""
    return "bf16" if spec.precision == "bf16" else "tf32"


def config_dict(spec, n_gpus, batch=None):
    head = "tied head (token table)" if spec.tied_head else "untied Dense head"
    arith = "bf16 weights / fp32 accumulate" if spec.precision == "bf16" else "fp32 storage, TF32 tensor-core operands"
    dist = "Zipf(1.1)" if spec.input_dist == "zipf" else "uniform"
    return {"workload": f"{spec.name}: GPT prefill, vocab {spec.vocab}, context {spec.context}, d_model {spec.d_model}, "
                        f"{spec.heads} heads, {spec.layers} layers, FFN {4 * spec.d_model} GeLU-tanh, {head}, "
                        f"{arith}, arg-max token per position",
            "global_batch": batch or spec.batch, "seq_len": spec.seq_len, "parallelism": f"batch-sharded x{n_gpus}",
            "weights": "N(0,0.02) seed 0", "inputs": f"{dist} token ids seed {spec.input_seed}",
            "l2": "no flush: the step streams its weights and several GB of activations, far more than the 126 MB L2"
                  if spec.d_model >= 768 else "no flush: the step is launch-bound, its working set is a few MB"}


def run_reference(args, spec):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = cpu_threads()
    params = wl.seeded_params(spec)
    ids = wl.make_inputs(spec, 4)
    for i in range(args.warmup):
        cpu_sample(spec, params, ids[i % 4], i % spec.layers)
    rates, secs = [], []
    t_all = time.perf_counter()
    for i in range(args.steps):
        e, b, t = cpu_sample(spec, params, ids[i % 4], i % spec.layers)
        secs.append(e + b + t)
        rates.append(spec.seq_len / (e + spec.layers * b + t))
    wall = time.perf_counter() - t_all
    value = statistics.median(rates)
    sample = CPU_SAMPLE_TEXT.format(B=spec.batch, T=spec.seq_len, L=spec.layers)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * wall / max(args.steps, 1), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(spec, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "CPU restatement of the reference (the reference is pure Python/NumPy and cannot travel to the GPU "
                    "box); value is the median over steps of tokens/s for a whole sequence, per the sample description"}
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------------ golden checks
def golden_rows_match(name: str, tokens: np.ndarray, tol_rel: float):
    """Compare rows of a gathered (B, T) token array with the fixture the reference wrote for this configuration
    (tests/golden/<name>.npz: arg-max, top and runner-up logit of whole sequences, stored with their global row
    numbers).  Tokens must be identical except where the reference's own top-2 gap is below the tolerance.
    Returns (all rows pass, rows checked, differing tokens, unexcused differences); (None, 0, 0, 0) without a fixture."""
    path = os.path.join(ROOT, "tests", "golden", name + ".npz")
    if not os.path.exists(path):
        return None, 0, 0, 0
    g = np.load(path)
    if "argmax" in g.files:
        # a small configuration: the fixture holds the reference's result for the whole batch
        n = min(tokens.shape[0], g["argmax"].shape[0])
        tol = tol_rel * float(g["max_abs"])
        differ = tokens[:n] != g["argmax"][:n]
        excused = (g["top"][:n] - g["second"][:n]) < tol
        n_bad = int((differ & ~excused).sum())
        return bool(n_bad == 0), n, int(differ.sum()), n_bad
    rows = g["global_rows"] if "global_rows" in g.files else np.arange(int(g["n_seq"]))
    ok, n_diff, n_bad, checked = True, 0, 0, 0
    for s, r in enumerate(rows):
        if r >= tokens.shape[0]:
            continue
        p = f"seq{s}_"
        tol = tol_rel * float(g[p + "max_abs"])
        T = min(tokens.shape[1], g[p + "argmax"].shape[0])
        differ = tokens[r, :T] != g[p + "argmax"][:T]
        excused = (g[p + "top"][:T] - g[p + "second"][:T]) < tol
        n_diff += int(differ.sum())
        n_bad += int((differ & ~excused).sum())
        checked += 1
    return bool(n_bad == 0 and checked > 0), checked, n_diff, n_bad


def decode_rows_match(tokens: np.ndarray, n_prompt: int, tol_rel: float):
    """Gathered greedy continuations against the reference's literal recompute loop (tests/golden/c4.npz: the first
    prompts, a few dozen steps): equal until the first step at which the reference's own top-2 gap is below the
    tolerance (after a near-tie the two sequences may legitimately go different ways)."""
    path = os.path.join(ROOT, "tests", "golden", "c4.npz")
    if not os.path.exists(path):
        return None
    g = np.load(path)
    tol = tol_rel * float(g["max_abs"])
    for b in range(min(int(g["n_prompts"]), tokens.shape[0])):
        for t in range(min(int(g["steps"]), tokens.shape[1] - n_prompt)):
            if tokens[b, n_prompt + t] != g["tokens"][b, n_prompt + t]:
                if g["top"][b, t] - g["second"][b, t] >= tol:
                    return False
                break
    return True


# ------------------------------------------------------------------------------------------------ the engine arm
def open_ranks(args):
    """Rank, world and (for N > 1) the NCCL communicator of this process.  One process per GPU; the launcher
    (torch.distributed.run or any other) only sets RANK / WORLD_SIZE / LOCAL_RANK."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs one process per GPU: launch with `python -m torch.distributed.run "
                             "--nproc-per-node N bench.py --gpus N ...`")
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE={world}")
    os.environ["TLNN_DEVICE"] = str(local_rank)
    comm = None
    if world > 1:
        from torchless_nn_b200.comm import Communicator
        comm = Communicator.from_env()
    return rank, world, local_rank, comm


class Timer:
    """CUDA events on the engine's stream around a region, bracketed by a barrier over the ranks and a stream
    synchronise on both sides; the reported time is the maximum over ranks."""

    def __init__(self, ctx, comm):
        self.ctx, self.comm = ctx, comm

    def barrier(self):
        from torchless_nn_b200 import backend
        backend.synchronize()
        if self.comm:
            self.comm.barrier()

    def run(self, fn, steps: int) -> float:
        import ctypes as C
        from torchless_nn_b200._lib import lib, check
        ms = C.c_float()
        self.barrier()
        check(lib.tlnn_prof_begin(self.ctx))
        for _ in range(steps):
            fn()
        check(lib.tlnn_prof_end(self.ctx, C.byref(ms)))
        self.barrier()
        return self.comm.max_over_ranks(float(ms.value)) if self.comm else float(ms.value)


def class_table(ctx, fn, repeats: int = 1):
    """Per-kernel-class CUDA-event times of `repeats` runs of fn, in an untimed pass of its own: bracketing every
    launch with events serialises the launches and switches graph replay off, so it must not run inside a timed
    region.  Returns {class: (launches, ms)} per run."""
    from torchless_nn_b200 import _lib
    from torchless_nn_b200._lib import lib, check
    check(lib.tlnn_prof_classes(ctx, 1))
    for _ in range(repeats):
        fn()
    rows = (_lib.ProfRow * 96)()
    n_rows = lib.tlnn_prof_table(ctx, rows, 96)
    check(lib.tlnn_prof_classes(ctx, 0))
    return {r.name.decode(): (int(r.launches) / repeats, float(r.ms) / repeats) for r in rows[:n_rows]}


# DRAM traffic of the four weight GEMMs of one c5 block on an 8-sequence shard (16384 rows, width 1024), from an ncu
# capture of exactly that case (dram__bytes_read.sum + dram__bytes_write.sum summed over the four launches).  Every
# operand and output of these products is streamed once, so traffic grows in proportion to the rows; the weights
# (25 MB per block) are the part that does not, and they are 2 % of the figure.
GEMM_BLOCK_TRAFFIC = {"rows": 16384, "d_model": 1024, "bytes": 591.4e6}


def measure_decode(args, rank, world, comm, timer):
    """Greedy decode on the GPT-2-small-shape model (the c4 configuration): 64 prompts of 128 tokens shared out by
    rows, every rank keeps the KV cache of its own prompts, 256 new tokens each, one gather of the finished rows."""
    from torchless_nn_b200 import backend
    from torchless_nn_b200.models import build_seeded
    spec = wl.CONFIGS["c4"]
    spec, net = build_seeded(spec)
    prompts = wl.make_inputs(spec)
    new = args.new_tokens
    out = {}

    def step():
        out["tokens"] = net.generate_greedy(prompts, new, comm=comm)

    for _ in range(2):
        step()
    backend.launch_count(reset=True)
    ms = timer.run(step, args.decode_runs) / args.decode_runs
    launches = backend.launch_count() / args.decode_runs
    tokens = out["tokens"].get()
    lo, hi = wl.shard_rows(spec.batch, rank, world)
    d, L = spec.d_model, spec.layers
    w_bytes = 2.0 * (spec.n_params() - spec.context * d)                  # bf16; the tied table doubles as the head
    kv_bytes = sum(2.0 * (hi - lo) * L * (spec.seq_len + i) * d * 2 for i in range(new))
    hbm = (w_bytes * new + kv_bytes) / (ms * 1e-3) / 1e9
    peak_hbm = measured_hbm()
    res = {"metric": "gpt_greedy_decode_new_tokens_per_s", "value": spec.batch * new / (ms * 1e-3), "unit": UNIT,
           "workload": f"c4: {spec.batch} prompts x {spec.seq_len} tokens + {new} greedy tokens on the c3-shape model, "
                       f"{spec.batch}/{world} prompts and their KV cache per GPU, prompt prefill inside the timed run",
           "ms_per_run": ms, "ms_per_step": ms / new, "launches_per_run": launches,
           "hbm_gbs_per_gpu": hbm, "hbm_peak_gbs": peak_hbm, "frac_of_measured_hbm": hbm / peak_hbm,
           "algorithmic_bytes_per_gpu_per_run": w_bytes * new + kv_bytes,
           "tokens_match_golden": decode_rows_match(tokens, spec.seq_len, 3e-2) if rank == 0 else None}
    backend.set_precision(wl.CONFIGS[args.config].precision)
    return res


def measured_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def run_b200(args, spec):
    import ctypes as C
    from torchless_nn_b200 import backend, _lib
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.device_array import DeviceArray
    from torchless_nn_b200.models import build_network, load_params
    from torchless_nn_b200.network import GPTPlan

    rank, world, local_rank, comm = open_ranks(args)
    backend.set_precision(spec.precision)
    ctx = backend.ctx()
    timer = Timer(ctx, comm)
    net = build_network(spec)
    load_params(net, wl.seeded_params(spec))
    batch = args.batch or spec.batch
    ids_all = wl.make_inputs(spec, batch)
    lo, hi = wl.shard_rows(batch, rank, world)
    ids_local = np.ascontiguousarray(ids_all[lo:hi])
    B_local, T = ids_local.shape
    n_local = B_local * T
    n_global = batch * T
    tol_rel = 3e-2 if spec.precision == "bf16" else 2e-3

    plan = GPTPlan.match(net.layers)
    model, keep, V = plan.model()
    ids_dev = DeviceArray.from_numpy(ids_local)
    tok_local = DeviceArray((B_local, T), np.int32)
    tok_all = DeviceArray((batch, T), np.int32) if comm else tok_local
    counts = None
    if comm:
        from torchless_nn_b200.comm import shard_counts
        counts = (C.c_longlong * world)(*[r * T for r in shard_counts(batch, world)])

    def prefill():
        check(lib.tlnn_gpt_prefill(ctx, C.byref(model), ids_dev.ptr, _lib.I32, B_local, T, None, tok_local.ptr))

    def step_resident():
        prefill()
        if comm:
            check(lib.tlnn_allgather_tokens(comm._h, tok_local.ptr, tok_all.ptr, n_local, counts))

    # ---- device-resident throughput: the default product path (captured graph replay, no per-launch events) ---------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step_resident()
    timer.barrier()
    backend.launch_count(reset=True)
    sampler.mark()                     # clocks are counted from here to the end of the timed region
    total_ms = timer.run(step_resident, args.steps)
    launches = backend.launch_count()
    clocks = sampler.stop() if rank == 0 else None
    value = n_global * args.steps / (total_ms * 1e-3)
    resident_tokens = tok_all.get() if rank == 0 else None
    match_resident = golden_rows_match(spec.name, resident_tokens, tol_rel) if rank == 0 else None

    # ---- per-class breakdown and the GEMM roofline: a separate, untimed pass ---------------------------------------
    classes = class_table(ctx, prefill, repeats=2)
    class_ms = sum(v[1] for v in classes.values())
    gemm_ms = sum(v[1] for k, v in classes.items() if k.startswith("gemm_"))
    gemm_launches = sum(v[0] for k, v in classes.items() if k.startswith("gemm_"))
    d, L = spec.d_model, spec.layers
    gemm_flops = n_local * (L * 24.0 * d * d + 2.0 * d * spec.vocab)
    peak, peak_how = measured_peak()
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    step_ms_rank = total_ms / args.steps
    traffic = None
    if GEMM_BLOCK_TRAFFIC["bytes"] and d == GEMM_BLOCK_TRAFFIC["d_model"]:
        # mean over the 4 L block products (the head product is not part of the capture)
        traffic = GEMM_BLOCK_TRAFFIC["bytes"] * (n_local / GEMM_BLOCK_TRAFFIC["rows"]) / 4.0
    roofline = {"bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel / gemm_tcgen05_kernel (all GEMM launches of a step)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_how,
                "traffic": traffic,
                "traffic_note": "mean DRAM bytes per block GEMM launch: ncu capture of one block's four products at 16384 rows x "
                                "1024, scaled by this rank's rows" if traffic else None,
                "algorithmic_bytes_per_launch": (n_local * (d * 2.0 * 7 + d * 4.0 * 4 + 3 * d * 2.0 + 4 * d * 2.0) * L
                                                 + 12.0 * d * d * 2 * L) / (4 * L),
                "launches_per_step": gemm_launches, "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
                "measured": "CUDA events around every launch, in an untimed pass after the timed region (the events "
                            "serialise launches, so they are kept out of it)",
                "share_of_step": gemm_ms / class_ms if class_ms else None,
                "kernel_classes_ms_per_step": {k: round(v[1], 4) for k, v in sorted(classes.items())},
                "whole_step_tflops_per_gpu": spec.flops_per_token() * n_local / (step_ms_rank * 1e-3) / 1e12,
                "frac_of_nominal_2250": achieved / 2250.0}

    # ---- end to end through the public API, host buffers -----------------------------------------------------------
    hp = C.c_void_p()
    check(lib.tlnn_host_alloc(ids_all.nbytes, C.byref(hp)))
    pinned_ids = np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_int32)), shape=ids_all.shape)
    pinned_ids[...] = ids_all
    out_rows = batch if rank == 0 else B_local
    hq = C.c_void_p()
    check(lib.tlnn_host_alloc(out_rows * T * 4, C.byref(hq)))
    pinned_tok = np.ctypeslib.as_array(C.cast(hq, C.POINTER(C.c_int32)), shape=(out_rows, T))

    def step_e2e():
        # the call a user makes: the global batch in host memory, every rank uploads and runs its rows, tokens gathered
        tok = net.predict_tokens(pinned_ids, comm=comm)
        src = tok if rank == 0 else DeviceArray((B_local, T), np.int32, ptr=tok.ptr + lo * T * 4, root=tok)
        check(lib.tlnn_d2h(ctx, pinned_tok.ctypes.data, src.ptr, pinned_tok.nbytes))

    for _ in range(2):
        step_e2e()
    e2e_ms = timer.run(step_e2e, args.steps)
    e2e_value = n_global * args.steps / (e2e_ms * 1e-3)
    match_e2e = golden_rows_match(spec.name, np.array(pinned_tok), tol_rel) if rank == 0 else None
    same = bool(np.array_equal(pinned_tok, resident_tokens)) if rank == 0 else None

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dtype_of(spec), "data": "synthetic",
            "config": config_dict(spec, world, batch), "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(ids_local.nbytes),
                    "d2h_bytes_per_step": int(pinned_tok.nbytes), "ms_per_step": e2e_ms / args.steps,
                    "api": "Network.predict_tokens(global batch in pinned host memory, comm): upload of this rank's rows, "
                           "prefill, NCCL all-gather of the tokens, copy to pinned host memory",
                    "tokens_equal_resident_path": same},
            "gpu_launches": int(launches), "roofline": roofline,
            "tokens_per_s_per_gpu": value / world,
            "frac_of_nominal_bf16_whole_step": roofline["whole_step_tflops_per_gpu"] / 2250.0}
    if rank == 0:
        ok_r, n_rows, n_diff, n_bad = match_resident
        ok_e = match_e2e[0]
        line["e2e"]["tokens_match_golden"] = ok_e
        line["parity"] = {"tokens_match_golden": None if ok_r is None else bool(ok_r and ok_e),
                          "fixture_rows_checked": n_rows, "tokens_differing": n_diff, "unexcused": n_bad,
                          "rule": "gathered tokens of the fixture's global rows equal the reference's arg-max except "
                                  f"where the reference's top-2 gap is below {tol_rel} x max|logit|"}

    # The two additions below must not take the headline measurement down with them: a failure is reported in place.
    if not args.no_decode and spec.name == "c5" and not args.batch:
        try:
            line["decode"] = measure_decode(args, rank, world, comm, timer)
        except Exception as e:                                         # noqa: BLE001
            line["decode"] = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cores = cpu_threads()
            params = wl.seeded_params(spec)
            v = cpu_tokens_per_s(spec, params, ids_all[:2], 2)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": CPU_SAMPLE_TEXT.format(B=spec.batch, T=spec.seq_len, L=spec.layers)}
        except Exception as e:                                         # noqa: BLE001
            line["cpu_baseline"] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    lib.tlnn_host_free(hp)
    lib.tlnn_host_free(hq)
    if comm:
        comm.barrier()
        comm.close()
    return 0


def run_decode(args, spec):
    """`--config c4`: the decode measurement on its own, at any number of GPUs."""
    from torchless_nn_b200 import backend
    rank, world, local_rank, comm = open_ranks(args)
    ctx = backend.ctx()
    timer = Timer(ctx, comm)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.mark()
    res = measure_decode(args, rank, world, comm, timer)
    line = {"metric": res["metric"], "value": res["value"], "unit": UNIT, "n_gpus": world, "steps": args.decode_runs,
            "warmup": 2, "ms_per_step": res["ms_per_run"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": res["workload"]},
            "clocks": sampler.stop() if rank == 0 else None, "gpu_launches": int(res["launches_per_run"] * args.decode_runs),
            "roofline": {"bound": "hbm", "achieved": res["hbm_gbs_per_gpu"], "peak": res["hbm_peak_gbs"], "unit": "GB/s",
                         "frac": res["frac_of_measured_hbm"], "traffic": None},
            "decode": res}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if comm:
        comm.barrier()
        comm.close()
    return 0


def run_other(args, spec):
    """Secondary configurations (single GPU): c2 ViT images/s, c4 greedy decode tokens/s.  Same JSON skeleton; these
    lines document the other configurations and are not the headline metric."""
    import ctypes as C
    from torchless_nn_b200 import backend, _lib
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.models import build_network, load_params
    backend.set_precision(spec.precision)
    ctx = backend.ctx()
    net = build_network(spec)
    load_params(net, wl.seeded_params(spec))
    x = wl.make_inputs(spec)
    ms = C.c_float()
    if spec.kind == "vit":
        from torchless_nn_b200.backend import xp
        xd = xp.array(x)
        step = lambda: net.predict_tokens(xd)          # the whole forward as one library call, then the arg-max of the scores
        units, metric, unit = spec.batch, "vit_forward_images_per_s", "images/s"
        flops = spec.flops_per_image() * spec.batch
    elif args.sample:
        # the notebook's generation loop (sampling from the model's SoftMax output), on the KV cache
        from torchless_nn_b200.activations import SoftMax
        from torchless_nn_b200.network import Network
        rows = args.batch or spec.batch
        x = x[:rows]
        sampler = Network(net.layers + [SoftMax()])
        sampler.set_eval(True)
        uniforms = np.random.default_rng(7).random((args.new_tokens, rows))
        step = lambda: sampler.generate(x, args.new_tokens, uniforms=uniforms)
        units, metric, unit = rows * args.new_tokens, "gpt_sampled_decode_new_tokens_per_s", "tokens/s"
        flops = None
    else:
        step = lambda: net.generate_greedy(x, args.new_tokens)
        units, metric, unit = spec.batch * args.new_tokens, "gpt_greedy_decode_new_tokens_per_s", "tokens/s"
        flops = None
    for _ in range(max(args.warmup, 3)):
        step()
    backend.synchronize()
    backend.launch_count(reset=True)
    check(lib.tlnn_prof_begin(ctx))
    for _ in range(args.steps):
        step()
    check(lib.tlnn_prof_end(ctx, C.byref(ms)))
    launches = backend.launch_count()
    # a second, untimed pass with per-launch events for the per-kernel breakdown (it serialises launches)
    check(lib.tlnn_prof_classes(ctx, 1))
    step()
    rows = (_lib.ProfRow * 64)()
    n_rows = lib.tlnn_prof_table(ctx, rows, 64)
    check(lib.tlnn_prof_classes(ctx, 0))
    classes = {r.name.decode(): round(float(r.ms), 4) for r in rows[:n_rows]}
    line = {"metric": metric, "value": units * args.steps / (ms.value * 1e-3), "unit": unit, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms.value / args.steps, "higher_is_better": True,
            "dtype": "bf16" if spec.precision == "bf16" else "tf32", "data": "synthetic",
            "config": {"workload": spec.name + (f" sampled, {args.batch or spec.batch} rows" if getattr(args, "sample", False) and spec.kind == "gpt" else "")},
            "gpu_launches": int(launches), "kernel_classes_ms_per_step": classes}
    if spec.kind == "gpt":
        line["ms_per_token"] = ms.value / args.steps / args.new_tokens
    if flops:
        line["tflops"] = flops * args.steps / (ms.value * 1e-3) / 1e12
    if spec.kind == "gpt":
        # decode is weight- and cache-streaming bound: bytes = weights once per step + K/V read per step
        d, L = spec.d_model, spec.layers
        w_bytes = 2.0 * (spec.n_params() - spec.context * d)          # bf16, tied table doubles as the head
        kv = sum(2.0 * (args.batch or spec.batch if getattr(args, "sample", False) else spec.batch) * L * (spec.seq_len + i) * d * 2
                 for i in range(args.new_tokens))
        total = w_bytes * args.new_tokens + kv
        line["hbm_bytes_per_run"] = total
        line["hbm_gbs_achieved_incl_prefill_time"] = total * args.steps / (ms.value * 1e-3) / 1e9
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="c5", choices=["c5", "c3", "c1", "c2", "c4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sample", action="store_true", help="c4 only: sampled decode (the notebook's GPT.generate) instead of arg-max")
    ap.add_argument("--batch", type=int, default=0, help="rows of the global batch (default: the configuration's)")
    ap.add_argument("--no-decode", action="store_true", help="c5: skip the decode measurement added to the line")
    ap.add_argument("--decode-runs", type=int, default=3, help="timed runs of the decode measurement")
    ap.add_argument("--new-tokens", type=int, default=wl.C4_NEW_TOKENS, help="c4 only: tokens generated per prompt")
    args = ap.parse_args()
    spec = wl.CONFIGS[args.config]
    if args.impl == "reference":
        return run_reference(args, spec)
    if args.config == "c2" or (args.config == "c4" and args.sample):
        return run_other(args, spec)
    if args.config == "c4":
        return run_decode(args, spec)
    return run_b200(args, spec)


if __name__ == "__main__":
    sys.exit(main())
