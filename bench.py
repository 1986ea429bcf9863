#!/usr/bin/env python
"""Benchmark of the transformer forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config c5|c3]

One "step" is one prefill of the whole workload: the GPT-2-medium-shape configuration (vocab 50257, context 2048,
width 1024, 16 heads, 24 layers, bf16 weights with float32 accumulation) on a global batch of 64 sequences of 2048
Zipf-distributed token ids, producing the arg-max token of every position.  The batch is sharded by rows over the
N ranks (one process per GPU, launched by torch.distributed.run for N > 1); the only collective is an all-gather
of the int32 tokens.  Total work is fixed as N grows ("scaling": "strong").

Printed by rank 0 as one JSON line:
  value      tokens/s with the token ids already resident in device memory (CUDA events on the engine's stream,
             maximum over ranks);
  e2e        the same metric through the public API (Network.predict_tokens) with host buffers: pinned host ids
             copied to the device and the tokens copied back inside the timed region, every step;
  roofline   tensor-core GEMM class: algorithmic FLOPs of its launches / their summed CUDA-event durations measured
             inside the timed region, against the measured cuBLAS bf16 rate in MEASURED_PEAKS.json;
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
# dram__bytes_read.sum + dram__bytes_write.sum of the four GEMM launches of one block, from the ncu capture summarised
# in profiles/gemm_tcgen05_c3_prefill.md (c3: 16384 rows, width 768): 411.7 MB.  Traffic grows with rows x width, so a
# workload's mean launch is estimated as that figure scaled by (rows x width) / (16384 x 768), times layers, plus the
# head's operand and arg-max candidate bytes, over the number of GEMM launches.
GEMM_BLOCK_TRAFFIC_C3 = 374.8e6


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
    try:
        from threadpoolctl import threadpool_info
        n = [i.get("num_threads", 0) for i in threadpool_info() if i.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_tokens_per_s(spec, params, ids, n_samples: int):
    rates = []
    for i in range(n_samples):
        e, b, t = cpu_sample(spec, params, ids[i % len(ids)], i % spec.layers)
        rates.append(spec.seq_len / (e + spec.layers * b + t))
    return statistics.median(rates)


CPU_SAMPLE_TEXT = ("one of the {B} sequences at the full {T}-token context through the NumPy restatement of the "
                   "reference's forward: embedding, 1 of {L} (identical-cost) blocks, final LayerNorm, head and arg-max "
                   "timed; sequence time = embed + {L} x block + tail")


def config_dict(spec, n_gpus):
    return {"workload": f"{spec.name}: GPT prefill, vocab {spec.vocab}, context {spec.context}, d_model {spec.d_model}, "
                        f"{spec.heads} heads, {spec.layers} layers, FFN {4 * spec.d_model} GeLU-tanh, tied head, "
                        f"bf16 weights / fp32 accumulate, arg-max token per position",
            "global_batch": spec.batch, "seq_len": spec.seq_len, "parallelism": f"batch-sharded x{n_gpus}",
            "weights": "N(0,0.02) seed 0", "inputs": f"Zipf(1.1) token ids seed {spec.input_seed}",
            "l2": "no flush needed: 0.7 GB of bf16 weights and several GB of activations per step exceed the 126 MB L2"}


def run_reference(args, spec):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
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
    cores = cpu_threads()
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


def run_b200(args, spec):
    import ctypes as C
    from torchless_nn_b200 import backend, _lib
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.device_array import DeviceArray
    from torchless_nn_b200.models import build_network, load_params
    from torchless_nn_b200.network import GPTPlan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs one process per GPU: launch with `python -m torch.distributed.run "
                             "--nproc-per-node N bench.py --gpus N ...`")
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE={world}")
    os.environ["TLNN_DEVICE"] = str(local_rank)

    dist = None
    torch = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    backend.set_precision(spec.precision)
    ctx = backend.ctx()
    net = build_network(spec)
    load_params(net, wl.seeded_params(spec))
    ids_all = wl.make_inputs(spec)
    lo, hi = wl.shard_rows(spec.batch, rank, world)
    ids_local = np.ascontiguousarray(ids_all[lo:hi])
    B_local, T = ids_local.shape
    n_local = B_local * T
    n_global = spec.batch * T

    plan = GPTPlan.match(net.layers)
    model, keep, V = plan.model()
    ids_dev = DeviceArray.from_numpy(ids_local)
    tok_local = DeviceArray((B_local, T), np.int32)
    tok_all = DeviceArray((spec.batch, T), np.int32) if world > 1 else tok_local

    gather = None
    if world > 1:
        if spec.batch % world != 0:
            raise SystemExit("the global batch must divide evenly over the ranks for the token all-gather")
        ext = torch.cuda.ExternalStream(int(lib.tlnn_stream(ctx)), device=torch.device("cuda", local_rank))
        t_local = torch.as_tensor(tok_local, device=torch.device("cuda", local_rank))
        t_all = torch.as_tensor(tok_all, device=torch.device("cuda", local_rank))

        def gather():
            # NCCL orders the collective after the work already enqueued on the engine's stream
            with torch.cuda.stream(ext):
                dist.all_gather_into_tensor(t_all.view(-1), t_local.view(-1))

    def step_resident():
        check(lib.tlnn_gpt_prefill(ctx, C.byref(model), ids_dev.ptr, _lib.I32, B_local, T, None, tok_local.ptr))
        if gather:
            gather()

    def barrier():
        backend.synchronize()
        if dist:
            dist.barrier()
        backend.synchronize()

    def max_over_ranks(ms: float) -> float:
        if not dist:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=torch.device("cuda", local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput ---------------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_resident()
    barrier()
    check(lib.tlnn_prof_classes(ctx, 1))
    backend.launch_count(reset=True)
    ms = C.c_float()
    barrier()
    sampler.mark()                     # clocks are counted from here to the end of the timed region
    check(lib.tlnn_prof_begin(ctx))
    for _ in range(args.steps):
        step_resident()
    check(lib.tlnn_prof_end(ctx, C.byref(ms)))
    barrier()
    launches = backend.launch_count()
    clocks = sampler.stop() if rank == 0 else None
    rows = (_lib.ProfRow * 64)()
    n_rows = lib.tlnn_prof_table(ctx, rows, 64)
    check(lib.tlnn_prof_classes(ctx, 0))
    total_ms = max_over_ranks(float(ms.value))
    value = n_global * args.steps / (total_ms * 1e-3)
    classes = {r.name.decode(): (int(r.launches), float(r.ms)) for r in rows[:n_rows]}
    gemm_ms = sum(v[1] for k, v in classes.items() if k.startswith("gemm_"))
    gemm_launches = sum(v[0] for k, v in classes.items() if k.startswith("gemm_"))
    d, L = spec.d_model, spec.layers
    gemm_flops = args.steps * n_local * (L * 24.0 * d * d + 2.0 * d * spec.vocab)
    peak, peak_how = measured_peak()
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    roofline = {"bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel / gemm_tcgen05_kernel (all GEMM launches)", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": peak_how,
                "traffic": ((GEMM_BLOCK_TRAFFIC_C3 * (n_local * d) / (16384.0 * 768.0)) * L
                            + n_local * d * 2.0 + spec.vocab * d * 2.0 + n_local * 394 * 8.0) / (4 * L + 1),
                "traffic_note": "mean DRAM bytes per GEMM launch, scaled from the c3 ncu capture by rows x width",
                "algorithmic_bytes_per_launch": (n_local * (d * 2.0 * 7 + d * 4.0 * 4 + 3 * d * 2.0 + 4 * d * 2.0) * L
                                                 + 12.0 * d * d * 2 * L + n_local * d * 2.0 + spec.vocab * d * 2.0) / (4 * L + 1),
                "launches": gemm_launches,
                "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
                "share_of_step": gemm_ms / float(ms.value) if ms.value else None,
                "kernel_classes_ms_per_step": {k: round(v[1] / args.steps, 4) for k, v in sorted(classes.items())},
                "whole_step_tflops_per_gpu": spec.flops_per_token() * n_local * args.steps / (float(ms.value) * 1e-3) / 1e12,
                "frac_of_nominal_2250": achieved / 2250.0}

    # ---- end to end through the public API, host buffers -----------------------------------------------------------
    hp = C.c_void_p()
    check(lib.tlnn_host_alloc(ids_local.nbytes, C.byref(hp)))
    pinned_ids = np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_int32)), shape=ids_local.shape)
    pinned_ids[...] = ids_local
    out_rows = spec.batch if (world > 1 and rank == 0) else B_local
    hq = C.c_void_p()
    check(lib.tlnn_host_alloc(out_rows * T * 4, C.byref(hq)))
    pinned_tok = np.ctypeslib.as_array(C.cast(hq, C.POINTER(C.c_int32)), shape=(out_rows, T))

    def step_e2e():
        dev_ids = DeviceArray(ids_local.shape, np.int32)
        check(lib.tlnn_h2d(ctx, dev_ids.ptr, pinned_ids.ctypes.data, pinned_ids.nbytes))
        tok = net.predict_tokens(dev_ids)
        src = tok
        if gather:
            check(lib.tlnn_d2d(ctx, tok_local.ptr, tok.ptr, tok.nbytes))
            gather()
            src = tok_all if rank == 0 else tok_local
        check(lib.tlnn_d2h(ctx, pinned_tok.ctypes.data, src.ptr, pinned_tok.nbytes))
        return pinned_tok

    for _ in range(2):
        step_e2e()
    barrier()
    check(lib.tlnn_prof_begin(ctx))
    for _ in range(args.steps):
        step_e2e()
    ms2 = C.c_float()
    check(lib.tlnn_prof_end(ctx, C.byref(ms2)))
    barrier()
    e2e_ms = max_over_ranks(float(ms2.value))
    e2e_value = n_global * args.steps / (e2e_ms * 1e-3)
    same = bool(np.array_equal(pinned_tok[:B_local] if out_rows != B_local else pinned_tok, tok_local.get())) \
        if rank == 0 and world == 1 else None

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(spec, world), "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(ids_local.nbytes),
                    "d2h_bytes_per_step": int(pinned_tok.nbytes), "ms_per_step": e2e_ms / args.steps,
                    "api": "Network.predict_tokens(pinned host ids) + token all-gather + copy to pinned host memory",
                    "tokens_equal_resident_path": same},
            "gpu_launches": int(launches), "roofline": roofline,
            "tokens_per_s_per_gpu": value / world,
            "frac_of_nominal_bf16_whole_step": roofline["whole_step_tflops_per_gpu"] / 2250.0}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        params = wl.seeded_params(spec)
        v = cpu_tokens_per_s(spec, params, ids_all[:2], 2)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cpu_threads(), "kind": "port",
                                "sample": CPU_SAMPLE_TEXT.format(B=spec.batch, T=spec.seq_len, L=spec.layers)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    lib.tlnn_host_free(hp)
    lib.tlnn_host_free(hq)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
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
        step = lambda: xp.argmax(net.predict(xd))
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
    ap.add_argument("--batch", type=int, default=0, help="c4 --sample only: number of prompt rows (default: the config's 64)")
    ap.add_argument("--new-tokens", type=int, default=wl.C4_NEW_TOKENS, help="c4 only: tokens generated per prompt")
    args = ap.parse_args()
    spec = wl.CONFIGS[args.config]
    if args.impl == "reference":
        return run_reference(args, spec)
    if args.config in ("c2", "c4"):
        return run_other(args, spec)
    return run_b200(args, spec)


if __name__ == "__main__":
    sys.exit(main())
