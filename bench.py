#!/usr/bin/env python
"""Benchmark of the q4_0 INT4 matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the Llama-2-7B-shaped decode projections at M = 1 — 32 layers of
q/k/v/o [4096 -> 4096], gate/up [4096 -> 11008], down [11008 -> 4096], all with distinct q4_0
weights (3.64 GB of packed weights, 29x the L2), fp16 activations.  One step = one pass over all
224 projections.  The metric is algorithmic GB/s: (18 bytes per 32 weights + X + Y bytes) / time.
The same line also carries the prefill GEMM (M = 2048, K = 4096, N = 14336, bf16) in TFLOP/s, the
packer's throughput, the M sweeps of the other configurations and, on several GPUs, the sharded
70B-shaped layers with and without their collectives.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the
reference's own torch path (dequantise + matmul) on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = 32
PROJ = [("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096),
        ("gate", 4096, 11008), ("up", 4096, 11008), ("down", 11008, 4096)]
GEMM_SHAPE = (2048, 4096, 14336)          # M, K, N of the prefill configuration
SHARD_SHAPES = [("gate_up", 8192, 28672), ("down", 28672, 8192)]     # Llama-3-70B-shaped layers


def gemv_bytes(M: int, K: int, N: int) -> int:
    """Algorithmic bytes of one decode product: packed weights + activations in + out."""
    return K * N // 32 * 18 + 2 * M * K + 2 * M * N


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def recorded_traffic():
    """DRAM traffic of one captured launch (dram__bytes_read.sum + dram__bytes_write.sum), constants
    recorded from profiler captures of small cases; the bench itself never runs under a profiler.
    decode: DRAM bytes per algorithmic byte of the persistent single-row kernel;
    gemm: bytes of one M=2048, K=4096, N=14336 launch."""
    return {"decode_dram_bytes_per_algorithmic_byte": 1.00, "gemm_dram_bytes_per_launch": 87.9e6}


def cpu_model() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for ln in f:
                if ln.lower().startswith("model name"):
                    return ln.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def keep_busy(clk: ClockSampler, elapsed_ms: float, work, sync, seconds: float = 0.6) -> None:
    """Keeps the same work running a little longer when the timed region was too short for the
    100 ms clock sampler to have seen it."""
    if clk.proc is not None and elapsed_ms < 400:
        t_end = time.time() + seconds
        while time.time() < t_end:
            work()
        sync()


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the torch restatement of the reference's CPU path
# ------------------------------------------------------------------------------------------

def cpu_layer_inputs(seed: int, M: int):
    from oracle import q4_0_oracle as orc
    g = torch.Generator().manual_seed(seed)
    items = []
    for _, K, N in PROJ:
        w = torch.randn(K, N, generator=g) * 0.02
        items.append((torch.randn(M, K, generator=g).half(), orc.quantize_q4_0(w)))
    return items


def cpu_layer_pass(items) -> float:
    """One layer's seven projections through the reference's public CPU path
    (dequantise to X.dtype, torch matmul).  Returns seconds."""
    from oracle import q4_0_oracle as orc
    t0 = time.perf_counter()
    for x, blocks in items:
        orc.matmul_q4_0_public(x, blocks)
    return time.perf_counter() - t0


def cpu_matmul_only_pass(items_dense) -> float:
    """The same seven products on weights dequantised beforehand (fp32): what the reference's path
    would cost if the dequantisation were free."""
    t0 = time.perf_counter()
    for x, w in items_dense:
        torch.matmul(x, w)
    return time.perf_counter() - t0


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    M = 1
    items = cpu_layer_inputs(1002, M)
    layer_bytes = sum(gemv_bytes(M, K, N) for _, K, N in PROJ)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_layer_pass(items)
    times = [cpu_layer_pass(items) for _ in range(args.steps)]
    total = sum(times)
    value = layer_bytes * args.steps / total / 1e9
    sample = "each step = one layer (7 projections, 1/32 of the 7B stack) through dequantise + torch matmul"
    print(json.dumps({
        "impl": "reference", "metric": "q4_0_gemv_gbps_m1", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama2-7b decode projections, M=1, q4_0 weights, fp16 activations", "m": M,
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "cpu": cpu_model(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline():
    from oracle import q4_0_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    items = cpu_layer_inputs(1002, 1)
    cpu_layer_pass(items)
    best = min(cpu_layer_pass(items) for _ in range(3))
    dense = [(x.float(), orc.dequantize_q4_0(b, torch.float32)) for x, b in items]
    cpu_matmul_only_pass(dense)
    best_mm = min(cpu_matmul_only_pass(dense) for _ in range(3))
    layer_bytes = sum(gemv_bytes(1, K, N) for _, K, N in PROJ)
    return {"value": layer_bytes / best / 1e9, "unit": "GB/s", "cores": cores, "cpu": cpu_model(), "kind": "port",
            "sample": "one layer (7 projections, 1/32 of a step) through the CPU restatement of the reference's "
                      "dequantise + torch matmul path, best of 3", "seconds": best,
            "matmul_only": {"value": layer_bytes / best_mm / 1e9, "unit": "GB/s (same algorithmic bytes)", "seconds": best_mm,
                            "note": "fp32 matmul on weights dequantised beforehand: the floor of the reference's path"}}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------

def build_stack(dev, layers: int, seed: int):
    """Distinct q4_0 weights for every projection, quantized on the device (set-up, untimed)."""
    from metalops_b200 import quantization as Q
    g = torch.Generator(device=dev).manual_seed(seed)
    stack = []
    for _ in range(layers):
        for name, K, N in PROJ:
            w = torch.randn(K, N, generator=g, device=dev) * 0.02
            _, pre = Q._quantize_impl(w, False, True)
            stack.append((name, K, N, pre))
            del w
    torch.cuda.synchronize(dev)
    return stack


def build_chains(dev, stack, xs, layers):
    """The step as stage lists of the persistent kernel, four stages per layer (q|k|v, o, gate|up,
    down).  `ready`: every stage reads an input that is ready when the launch starts, the situation
    of the per-projection launches it replaces.  `dataflow`: each stage is fed by an earlier stage's
    output (q|k|v <- previous down, o <- v, gate|up <- o, down <- gate), scaled to unit variance."""
    from metalops_b200 import decode as D
    n_out = sum(N + (-N) % 8 for _, _, N, _ in stack)
    ready = D.DecodeChain(torch.float16, dev, out_capacity=n_out)
    flow = D.DecodeChain(torch.float16, dev, out_capacity=n_out)
    a4, a11 = 1.0 / (0.02 * math.sqrt(4096)), 1.0 / (0.02 * math.sqrt(11008))
    prev = xs[4096].view(-1)
    for layer in range(layers):
        q, k, v, o, ga, up, dn = [p for *_, p in stack[7 * layer: 7 * layer + 7]]
        ready.add_stage(xs[4096].view(-1), [q, k, v])
        ready.add_stage(xs[4096].view(-1), [o])
        ready.add_stage(xs[4096].view(-1), [ga, up])
        ready.add_stage(xs[11008].view(-1), [dn])
        s0 = flow.add_stage(prev, [q, k, v], alphas=[a4] * 3)
        s1 = flow.add_stage((s0, 2), [o], alphas=[a4])
        s2 = flow.add_stage((s1, 0), [ga, up], alphas=[a4] * 2)
        s3 = flow.add_stage((s2, 0), [dn], alphas=[a11])
        prev = (s3, 0)
    return ready.build(), flow.build()


def time_steps(stream, step, steps: int, warmup: int, clk_index=None, dist_barrier=None):
    """W warm-up steps, then exactly `steps` steps between two events on `stream` (plus one event
    per step for the median); returns (total ms, per-step ms list, clock summary or None)."""
    for _ in range(warmup):
        step()
    stream.synchronize()
    if dist_barrier is not None:
        dist_barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    clocks = None

    def timed():
        evs[0].record(stream)
        for i in range(steps):
            step()
            evs[i + 1].record(stream)
        stream.synchronize()

    if clk_index is not None:
        with ClockSampler(clk_index) as clk:
            timed()
            keep_busy(clk, evs[0].elapsed_time(evs[-1]), step, stream.synchronize)
        clocks = clk.summary()
    else:
        timed()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return evs[0].elapsed_time(evs[-1]), per, clocks


def run_ours(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this build has no CPU path")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    import torch.distributed as dist
    # Libraries write to file descriptor 1 (NCCL prints its version there); the one JSON line must
    # be alone on stdout, so everything else goes to stderr until the line is printed.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    barrier = dist.barrier if world > 1 else None

    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    lib = _cabi.load()
    _cabi.stream_ptr(dev)

    M = 1
    # On several GPUs every rank runs its own copy of the step on its own weights: independent
    # replicas with no communication (the sharded layers with their collectives are the `sharded`
    # object below).
    stack = build_stack(dev, args.layers, 1002 + rank)
    xs = {K: torch.randn(1, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}
    step_bytes = sum(gemv_bytes(M, K, N) for _, K, N, _ in stack)
    packed_bytes = sum(p.nbytes() for *_, p in stack)
    n_proj = len(stack)
    stream = torch.cuda.Stream(dev)
    peaks = measured_peaks()
    traffic = recorded_traffic()

    with torch.cuda.stream(stream):
        chain_ready, chain_flow = build_chains(dev, stack, xs, args.layers)

        # ---- headline: the 224 projections as one persistent launch, inputs ready at launch ----
        ms, per, clocks = time_steps(stream, chain_ready.run, args.steps, args.warmup, clk_index=local, dist_barrier=barrier)
        if Q.wait_status(dev) != 0:
            raise SystemExit("a bounded device-side wait gave up")
        if world > 1:
            dist.barrier()
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = step_bytes * world * args.steps / (ms * 1e-3) / 1e9
    per_gpu = step_bytes * args.steps / (ms * 1e-3) / 1e9

    extras = None
    if not args.skip_variants:
        extras = bench_variants(dev, stream, lib, stack, xs, chain_flow, step_bytes, peaks, args)

    # ---- end to end through the public API with host buffers ------------------------------
    e2e = None
    if not args.skip_e2e:
        e2e = bench_e2e(dev, stream, lib, stack, xs, chain_ready, step_bytes, world, args, barrier)

    gemm = quant = sweeps = batch = sharded = int4g = None
    if not args.skip_gemm:
        gemm = bench_gemm(dev, stream, lib, peaks, traffic, local)
    if rank == 0 and not args.skip_extra:
        quant = bench_quantize(dev, stream, peaks)
        if args.layers >= 4:
            batch = bench_batch(dev, stream, lib, stack)
    del chain_ready, chain_flow, stack
    torch.cuda.empty_cache()
    if rank == 0 and not args.skip_extra:
        sweeps = bench_sweeps(dev, stream, lib, peaks)
        int4g = bench_groupwise_int4(dev, stream, lib, peaks)
    if not args.skip_extra:
        sharded = bench_sharded(dev, stream, lib, rank, world, peaks)

    out = None
    if rank == 0:
        frac = per_gpu / peaks["hbm_gbs"]
        out = {
            "metric": "q4_0_gemv_gbps_m1", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "ms_per_step_median": statistics.median(per),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"llama2-7b decode projections, M={M}, q4_0 weights, fp16 activations",
                       "layers": args.layers, "projections_per_step": n_proj,
                       "packed_weight_bytes_per_gpu": packed_bytes,
                       "l2": "inputs (3.6 GB of distinct weights per step) exceed the 126 MB L2; no flush needed",
                       "launch": "one persistent launch per step over a stage list (4 stages per layer: q|k|v, o, gate|up, "
                                 "down); every stage's input is ready when the launch starts, as for the per-projection "
                                 "launches it replaces; value = bytes of the 224 projections / step time, unchanged",
                       "parallelism": ("one GPU" if world == 1 else
                                       f"{world} independent replicas of the step, one per GPU, no communication "
                                       "(see `sharded` for the sharded layers and their collectives)")},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": frac, "peak_source": peaks["source"],
                         "frac_of_nominal_8tbs": per_gpu / 8000.0,
                         "kernel": "chain_kernel", "launches": args.steps,
                         "avg_launch_us": ms * 1e3 / args.steps,
                         "traffic": traffic["decode_dram_bytes_per_algorithmic_byte"] * step_bytes,
                         "traffic_source": "constant recorded from a profiler capture of a small case, scaled by bytes"},
            "decode_variants": extras,
            "e2e": e2e, "gpu_launches": args.steps, "clocks": clocks,
        }
        for key, val in (("gemm", gemm), ("quantize", quant), ("sweeps", sweeps), ("decode_batch", batch), ("groupwise_int4", int4g),
                         ("sharded", sharded)):
            if val is not None:
                out[key] = val
        if not args.skip_cpu:
            if world == 1:
                out["cpu_baseline"] = cpu_baseline()
            else:
                out["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": os.cpu_count(), "cpu": cpu_model(), "kind": "port",
                                       "sample": "not timed while the other ranks' processes share the host cores; "
                                                 "see the reference arm (--impl reference)"}
        os.write(json_fd, (json.dumps(out) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bench_variants(dev, stream, lib, stack, xs, chain_flow, step_bytes, peaks, args):
    """The same step two other ways: with every stage fed by an earlier stage's output, and as 224
    separate launches of the per-projection entry point."""
    from metalops_b200 import _cabi
    extras = {}
    with torch.cuda.stream(stream):
        ms_f, per_f, _ = time_steps(stream, chain_flow.run, max(5, min(args.steps, 50)), 3)
        nf = len(per_f)
        extras["dataflow"] = {"gbps": step_bytes * nf / (ms_f * 1e-3) / 1e9, "frac": step_bytes * nf / (ms_f * 1e-3) / 1e9 / peaks["hbm_gbs"],
                              "ms_per_step": ms_f / nf,
                              "note": "each stage reads the output of an earlier stage (q|k|v <- down, o <- v, gate|up <- o, "
                                      "down <- gate), handed over inside the kernel"}
        ys = [torch.empty(1, N, device=dev, dtype=torch.float16) for _, _, N, _ in stack]

        def enqueue_launches():
            sp = torch.cuda.current_stream(dev).cuda_stream
            for (name, K, N, pre), y in zip(stack, ys):
                rc = lib.q4b_gemv(xs[K].data_ptr(), _cabi.F16, 1, K, pre.data.data_ptr(), K, N, y.data_ptr(), N, _cabi.FLAG_PDL, sp)
                if rc:
                    _cabi.check(rc, "q4b_gemv")

        enqueue_launches()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            enqueue_launches()
        ms_l, per_l, _ = time_steps(stream, graph.replay, max(5, min(args.steps, 50)), 3)
        nl = len(per_l)
        extras["per_projection_launches"] = {"gbps": step_bytes * nl / (ms_l * 1e-3) / 1e9,
                                             "frac": step_bytes * nl / (ms_l * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                             "ms_per_step": ms_l / nl, "launches_per_step": len(stack),
                                             "note": "q4b_gemv per projection, CUDA graph + programmatic dependent launch"}
        del graph
    return extras


def bench_e2e(dev, stream, lib, stack, xs, chain, step_bytes, world, args, barrier):
    """The step through the public API with HOST buffers: copy the inputs from pinned memory, run the
    stage list, copy all 224 outputs back, wait.  Also the older per-projection form
    (q4b_matmul_host: H2D of X, product, D2H of Y for every projection)."""
    from metalops_b200 import _cabi
    import torch.distributed as dist
    hx = {K: torch.randn(1, K, dtype=torch.float16).pin_memory() for K in (4096, 11008)}
    used = chain._out_used
    hy = torch.empty(used, dtype=torch.float16).pin_memory()

    def e2e_step():
        for K in (4096, 11008):
            xs[K].copy_(hx[K], non_blocking=True)
        chain.run()
        hy.copy_(chain.out_flat[:used], non_blocking=True)
        stream.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_step()
        if barrier is not None:
            barrier()
        n = max(3, min(args.steps, 50))
        t0 = time.perf_counter()
        for _ in range(n):
            e2e_step()
        dt = time.perf_counter() - t0
    te = torch.tensor([dt], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    out = {"value": step_bytes * world * n / float(te.item()) / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": 2 * (4096 + 11008), "d2h_bytes_per_step": 2 * used, "steps": n,
           "note": "per step: H2D of the input rows from pinned memory, one persistent launch, D2H of all 224 outputs, "
                   "stream synchronised; host wall clock"}
    # per-projection host calls (the reference's API shape: one matmul call per projection)
    ys = [torch.empty(1, N, device=dev, dtype=torch.float16) for _, _, N, _ in stack]
    hys = [torch.empty(1, N, dtype=torch.float16).pin_memory() for _, _, N, _ in stack]
    dx = {K: torch.empty(1, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}

    def per_call_step():
        sp = stream.cuda_stream
        for (name, K, N, pre), y, yh in zip(stack, ys, hys):
            rc = lib.q4b_matmul_host(hx[K].data_ptr(), dx[K].data_ptr(), _cabi.F16, 1, pre.data.data_ptr(), K, N,
                                     y.data_ptr(), yh.data_ptr(), 0, sp)
            if rc:
                _cabi.check(rc, "q4b_matmul_host")
        stream.synchronize()

    with torch.cuda.stream(stream):
        per_call_step()
        n2 = max(3, min(args.steps, 10))
        t0 = time.perf_counter()
        for _ in range(n2):
            per_call_step()
        dt2 = time.perf_counter() - t0
    out["per_projection_calls"] = {"value": step_bytes * n2 / dt2 / 1e9, "unit": "GB/s (this rank)",
                                   "h2d_bytes_per_step": sum(2 * K for _, K, _, _ in stack),
                                   "d2h_bytes_per_step": sum(2 * N for _, _, N, _ in stack),
                                   "note": "q4b_matmul_host per projection: H2D of X, kernel, D2H of Y"}
    return out


def distinct_weights(dev, K, N, min_total_bytes, seed, outliers=False, std=0.02):
    """Enough distinct q4_0 weights of one shape to exceed L2 when rotated."""
    from metalops_b200 import quantization as Q
    g = torch.Generator(device=dev).manual_seed(seed)
    one = K * N // 32 * 18
    n = max(2, -(-min_total_bytes // one))
    pres = []
    for _ in range(n):
        w = torch.randn(K, N, generator=g, device=dev) * std
        if outliers:
            idx = torch.randint(0, K * N, (K * N // 1000,), generator=g, device=dev)
            w.view(-1)[idx] = torch.where(torch.rand(idx.numel(), generator=g, device=dev) < 0.5, -0.5, 0.5)
        pres.append(Q._quantize_impl(w, False, True)[1])
        del w
    return pres


def time_launches(stream, enqueue, reps, graph=True):
    """Average device time (ms) of one of `reps` launches enqueued by `enqueue(i)`, replayed as a
    CUDA graph when it can be captured."""
    with torch.cuda.stream(stream):
        for i in range(min(reps, 4)):
            enqueue(i)
        stream.synchronize()
        g = None
        if graph:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for i in range(reps):
                        enqueue(i)
            except Exception:
                g = None
                torch.cuda.synchronize()

        def run():
            if g is not None:
                g.replay()
            else:
                for i in range(reps):
                    enqueue(i)

        run()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / reps


def bench_gemm(dev, stream, lib, peaks, traffic, local):
    """Prefill GEMM of configuration 3 (M=2048, K=4096, N=14336, bf16): a 20-launch burst and a run of
    more than a second, each with its own clock samples."""
    from metalops_b200 import _cabi
    M, K, N = GEMM_SHAPE
    pres = distinct_weights(dev, K, N, 4 * K * N // 32 * 18, 1003, outliers=True)
    g = torch.Generator(device=dev).manual_seed(1003)
    xs = [torch.randn(M, K, generator=g, device=dev).bfloat16() for _ in pres]
    ys = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in pres]
    nset = len(pres)

    def run(n):
        sp = stream.cuda_stream
        for i in range(n):
            j = i % nset
            rc = lib.q4b_gemm(xs[j].data_ptr(), _cabi.BF16, M, K, pres[j].data.data_ptr(), K, N, ys[j].data_ptr(), N, 0, sp)
            if rc:
                _cabi.check(rc, "q4b_gemm")

    flop = 2.0 * M * K * N
    with torch.cuda.stream(stream):
        run(5)
        stream.synchronize()
        d = ctypes.c_int(0)
        if lib.q4b_wait_status(stream.cuda_stream, ctypes.byref(d)):
            return {"error": f"gemm wait status detail {d.value}"}
        reps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clk:
            time.sleep(0.25)                       # the sampler's first lines describe the idle GPU
            e0.record(stream)
            run(reps)
            e1.record(stream)
            stream.synchronize()
            time.sleep(0.15)
        ms = e0.elapsed_time(e1) / reps
        # sustained: keep launching for well over a second
        n_long = max(200, int(1500.0 / ms))
        with ClockSampler(local) as clk2:
            e0.record(stream)
            run(n_long)
            e1.record(stream)
            stream.synchronize()
        ms_long = e0.elapsed_time(e1) / n_long
    tf, tf_long = flop / (ms * 1e-3) / 1e12, flop / (ms_long * 1e-3) / 1e12
    return {"metric": "q4_0_gemm_tflops_m2048", "value": tf, "unit": "TFLOP/s", "ms_per_launch": ms,
            "config": {"workload": f"prefill GEMM M={M} K={K} N={N}, bf16 activations, q4_0 weights with 0.1% outliers",
                       "l2": f"{nset} distinct weight/activation sets rotate, larger than L2"},
            "dtype": "bf16",
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "frac_of_nominal_2250": tf / 2250.0, "peak_source": peaks["source"],
                         "kernel": "gemm_wt_kernel", "traffic": traffic.get("gemm_dram_bytes_per_launch"),
                         "note": f"{reps}-launch burst against the burst cuBLAS figure"},
            "clocks": clk.summary(),
            "sustained": {"value": tf_long, "unit": "TFLOP/s", "launches": n_long, "seconds": ms_long * n_long / 1e3,
                          "frac_of_sustained_peak": tf_long / peaks["bf16_tflops_sustained"], "clocks": clk2.summary()},
            "gpu_launches": reps + n_long}


def bench_quantize(dev, stream, peaks):
    """Configuration 5's packer: fp16 [N=14336, K=4096] (nn.Linear layout, read in place) with 1% of
    the blocks all zero -> q4_0 blocks, and the same with both output forms."""
    from metalops_b200 import _cabi
    K, N = 4096, 14336
    g = torch.Generator(device=dev).manual_seed(1005)
    ws = []
    for _ in range(3):                                     # 3 x 117 MB of inputs rotate: larger than L2
        w = (torch.randn(N, K, generator=g, device=dev) * 0.02).half()
        mask = torch.rand(N, K // 32, generator=g, device=dev) < 0.01
        w.view(N, K // 32, 32)[mask] = 0
        ws.append(w)
    algo = K * N * 2 + K * N // 32 * 18
    out = {"bytes_per_launch": algo, "config": "fp16 [14336, 4096] nn.Linear layout, 1% all-zero blocks"}
    lib = _cabi.load()
    blocks = torch.empty((K // 32, N, 18), dtype=torch.uint8, device=dev)
    pre = torch.empty(lib.q4b_prepacked_bytes(K, N), dtype=torch.uint8, device=dev)
    for label, b_ptr, p_ptr in (("blocks_only", blocks.data_ptr(), None), ("streaming_layout_only", None, pre.data_ptr()),
                                ("blocks_and_streaming_layout", blocks.data_ptr(), pre.data_ptr())):
        def enqueue(i, b_ptr=b_ptr, p_ptr=p_ptr):
            rc = lib.q4b_quantize(ws[i % 3].data_ptr(), _cabi.F16, K, N, _cabi.LAYOUT_NK, b_ptr, p_ptr,
                                  torch.cuda.current_stream(dev).cuda_stream)
            if rc:
                _cabi.check(rc, "q4b_quantize")

        us = time_launches(stream, enqueue, 12) * 1e3
        gbps = algo / us / 1e3
        out[label] = {"us_per_launch": us, "gbps": gbps, "frac_of_hbm": gbps / peaks["hbm_gbs"]}
    out["note"] = ("algorithmic bytes = input + ONE 18-byte-per-block output; the last variant writes both output forms "
                   "(1.22x the bytes) in one pass")
    return out


def bench_sweeps(dev, stream, lib, peaks):
    """Configuration 5's M sweep at K=4096, N=14336 and configuration 4 on one GPU (K=8192, N=28672
    and K=28672, N=8192 at M = 1 and 128), through q4b_matmul (the dispatcher picks the kernel)."""
    from metalops_b200 import _cabi
    out = {}
    cases = [("k4096_n14336", 4096, 14336, (1, 2, 8, 32, 128, 512, 4096)),
             ("k8192_n28672", 8192, 28672, (1, 128)), ("k28672_n8192", 28672, 8192, (1, 128))]
    for label, K, N, Ms in cases:
        pres = distinct_weights(dev, K, N, 300 << 20, 2000 + K % 97)
        res = {}
        for M in Ms:
            x = torch.randn(M, K, device=dev, dtype=torch.float16)
            y = torch.empty(M, N, device=dev, dtype=torch.float16)
            reps = max(len(pres), 8 if M >= 512 else 24)

            def enqueue(i, x=x, y=y, M=M):
                p = pres[i % len(pres)]
                rc = lib.q4b_matmul(x.data_ptr(), _cabi.F16, M, K, p.data.data_ptr(), K, N, y.data_ptr(), N, _cabi.FLAG_PDL,
                                    torch.cuda.current_stream(dev).cuda_stream)
                if rc:
                    _cabi.check(rc, "q4b_matmul")

            ms = time_launches(stream, enqueue, reps)
            gb, tf = gemv_bytes(M, K, N) / (ms * 1e-3) / 1e9, 2.0 * M * K * N / (ms * 1e-3) / 1e12
            res[f"m{M}"] = {"us": ms * 1e3, "gbps": gb, "frac_of_hbm": gb / peaks["hbm_gbs"], "tflops": tf,
                            "frac_of_bf16_burst": tf / peaks["bf16_tflops"]}
        out[label] = res
        del pres
        torch.cuda.empty_cache()
    return out


def bench_groupwise_int4(dev, stream, lib, peaks):
    """The group-wise asymmetric INT4 format (K=4096, N=14336, group 128, bf16 activations) through the
    C ABI with every buffer allocated once, as matmul_int4 runs it: at M = 1 the rows' group sums
    (q4b_int4g_rowsums) and the decode kernel forming the zero-point term in its epilogue (q4b_int4g_gemv);
    at M = 2048 the term folded into the contraction (q4b_int4g_fold_rows, then q4b_int4g_gemm_fold).  Next to each the same product on the tiles alone.  Four weights rotate."""
    import metalops_b200 as mo
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    K, N, G = 4096, 14336, 128
    g = torch.Generator(device=dev).manual_seed(1006)
    sets = []
    for _ in range(4):
        w = (torch.randn(K, N, generator=g, device=dev) * 0.02).half()
        sets.append(Q.prepack_int4(*mo.quantize_int4(w, G), G))
        del w
    out = {"config": f"K={K} N={N} group {G}, bf16 activations; M=1: term formed in the decode kernel's epilogue, M=2048: folded into the contraction"}
    for M in (1, 2048):
        x = torch.randn(M, K, generator=g, device=dev).bfloat16()
        y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        rs = torch.empty(lib.q4b_int4g_rowsums_bytes(M, K, G) // 4, dtype=torch.float32, device=dev)

        rows = torch.empty((M, 64 * sets[0].fold_ktiles), dtype=torch.bfloat16, device=dev)

        def full(i, M=M, x=x, y=y, rs=rs, rows=rows):
            sp = torch.cuda.current_stream(dev).cuda_stream
            p = sets[i % 4]
            if M > 16:         # tensor-core kernels: the zero-point term folded into the contraction (what matmul_int4 does)
                rc = lib.q4b_int4g_fold_rows(x.data_ptr(), _cabi.BF16, M, K, K, G, rows.data_ptr(), sp)
                rc = rc or lib.q4b_int4g_gemm_fold(x.data_ptr(), _cabi.BF16, M, K, p.tiles.data.data_ptr(), K, N, p.fold.data_ptr(),
                                                   rows.data_ptr(), p.fold_ktiles, None, y.data_ptr(), N, 0, sp)
            else:              # decode kernels: the rows' group sums, the term formed in the product's epilogue
                rc = lib.q4b_int4g_rowsums(x.data_ptr(), _cabi.BF16, M, K, K, G, rs.data_ptr(), sp)
                rc = rc or lib.q4b_int4g_gemv(x.data_ptr(), _cabi.BF16, M, K, p.tiles.data.data_ptr(), K, N, p.corr.data_ptr(), rs.data_ptr(),
                                              G, None, y.data_ptr(), N, 0, sp)
            if rc:
                _cabi.check(rc, "group-wise INT4 matmul")

        def tiles_only(i, M=M, x=x, y=y):
            rc = lib.q4b_matmul_addend(x.data_ptr(), _cabi.BF16, M, K, sets[i % 4].tiles.data.data_ptr(), K, N, None, 0, y.data_ptr(), N, 0,
                                       torch.cuda.current_stream(dev).cuda_stream)
            if rc:
                _cabi.check(rc, "q4b_matmul_addend")

        us_full = time_launches(stream, full, 8) * 1e3
        us_tiles = time_launches(stream, tiles_only, 8) * 1e3
        out[f"m{M}"] = {"us_per_product": us_full, "us_tiles_only": us_tiles, "tflops": 2.0 * M * K * N / us_full / 1e6,
                        "weight_gbps": gemv_bytes(M, K, N) / us_full / 1e3}
    return out


def bench_batch(dev, stream, lib, stack):
    """Decode batches: the same projections at M = 4, 16 and 64 rows through q4b_matmul (decode kernel,
    tensor-memory kernel), the first four layers (455 MB of weights, larger than L2) in a CUDA
    graph.  Reported for information next to the M = 1 headline."""
    from metalops_b200 import _cabi
    sub = stack[: 4 * len(PROJ)]
    out = {}
    for M in (4, 16, 64):
        xs = {K: torch.randn(M, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}
        ys = [torch.empty(M, N, device=dev, dtype=torch.float16) for _, _, N, _ in sub]

        def enqueue(i, xs=xs, ys=ys, M=M):
            name, K, N, pre = sub[i]
            rc = lib.q4b_matmul(xs[K].data_ptr(), _cabi.F16, M, K, pre.data.data_ptr(), K, N, ys[i].data_ptr(), N, _cabi.FLAG_PDL,
                                torch.cuda.current_stream(dev).cuda_stream)
            if rc:
                _cabi.check(rc, "q4b_matmul")

        ms = time_launches(stream, enqueue, len(sub)) * len(sub)
        nbytes = sum(gemv_bytes(M, K, N) for _, K, N, _ in sub)
        flops = sum(2.0 * M * K * N for _, K, N, _ in sub)
        out[f"m{M}"] = {"gbps": nbytes / (ms * 1e-3) / 1e9, "tflops": flops / (ms * 1e-3) / 1e12,
                        "us_per_launch": ms * 1e3 / len(sub)}
    return out


def bench_sharded(dev, stream, lib, rank, world, peaks):
    """Configuration 4: the Llama-3-70B-shaped layers (K=8192, N=28672 and K=28672, N=8192, M = 1 and
    128, fp16) sharded over the ranks, strong scaling: total work is fixed, every rank holds 1/world
    of each weight.  Column-parallel over N: local product alone, with the NCCL all-gather of the
    outputs, and (M = 1) with the gather fused into the kernel's stores to peer memory.  Row-parallel
    over K for the down shape: NCCL all-reduce of fp32 partials, and (M = 1) the fused peer-store
    reduction.  Times are device times, the maximum over ranks; throughputs are whole-job."""
    import torch.distributed as dist
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    from metalops_b200 import sharding as S
    res = {"world": world, "scaling": "strong",
           "note": "algorithmic bytes / flops of the WHOLE layer over the slowest rank's device time; `local` and the `_graph` "
                   "entries replay a CUDA graph, the other variants are enqueued call by call from Python (host-driven)"}

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def whole_job(M, K, N, ms):
        gb = gemv_bytes(M, K, N) / (ms * 1e-3) / 1e9
        tf = 2.0 * M * K * N / (ms * 1e-3) / 1e12
        return {"us": ms * 1e3, "gbps": gb, "frac_of_hbm_x_world": gb / (peaks["hbm_gbs"] * world), "tflops": tf}

    for label, K, N in SHARD_SHAPES:
        entry = {}
        # ---- column-parallel: rank r holds columns [r*N/world, (r+1)*N/world) ----
        n_loc = N // world
        pres = distinct_weights(dev, K, n_loc, 300 << 20, 3000 + rank)
        for M in (1, 128):
            x = torch.randn(M, K, device=dev, dtype=torch.float16)
            y = torch.empty(M, n_loc, device=dev, dtype=torch.float16)
            full = torch.empty(world * M, n_loc, device=dev, dtype=torch.float16)
            reps = max(len(pres), 16)

            def local(i, x=x, y=y, M=M, pdl=_cabi.FLAG_PDL):
                p = pres[i % len(pres)]
                rc = lib.q4b_matmul(x.data_ptr(), _cabi.F16, M, K, p.data.data_ptr(), K, n_loc, y.data_ptr(), n_loc, pdl,
                                    torch.cuda.current_stream(dev).cuda_stream)
                if rc:
                    _cabi.check(rc, "q4b_matmul")

            def with_gather(i, x=x, y=y, M=M, full=full):
                local(i, pdl=0)
                if world > 1:
                    dist.all_gather_into_tensor(full, y)

            e = {"local": whole_job(M, K, N, max_over_ranks(time_launches(stream, local, reps)))}
            if world > 1:
                dist.barrier()
                e["nccl_all_gather"] = whole_job(M, K, N, max_over_ranks(time_launches(stream, with_gather, reps, graph=False)))
                if M == 1:
                    try:
                        fused = S.FusedGatherBuffer(N, rank, world, torch.float16, dev)

                        def fused_step(i, x=x, fused=fused):
                            fused.gemv(x, pres[i % len(pres)])
                        dist.barrier()
                        e["fused_peer_store_gather"] = whole_job(M, K, N, max_over_ranks(time_launches(stream, fused_step, reps, graph=False)))
                        dist.barrier()
                        e["fused_peer_store_gather_graph"] = whole_job(M, K, N, max_over_ranks(time_launches(stream, fused_step, reps)))
                    except Exception as ex:           # symmetric memory unavailable on this box
                        e["fused_peer_store_gather"] = {"error": str(ex)[:200]}
            entry[f"column_parallel_m{M}"] = e
        del pres
        torch.cuda.empty_cache()
        # ---- row-parallel over K (the down projection after a column-parallel gate|up) ----
        if label == "down":
            k_loc = K // world
            pres = distinct_weights(dev, k_loc, N, 300 << 20, 4000 + rank)
            for M in (1, 128):
                x = torch.randn(M, k_loc, device=dev, dtype=torch.float16)
                y = torch.empty(M, N, device=dev, dtype=torch.float16)
                acc = torch.empty(M, N, device=dev, dtype=torch.float32)
                reps = max(len(pres), 16)

                def partial(i, x=x, y=y, M=M, pdl=_cabi.FLAG_PDL):
                    p = pres[i % len(pres)]
                    rc = lib.q4b_matmul(x.data_ptr(), _cabi.F16, M, k_loc, p.data.data_ptr(), k_loc, N, y.data_ptr(), N, pdl,
                                        torch.cuda.current_stream(dev).cuda_stream)
                    if rc:
                        _cabi.check(rc, "q4b_matmul")

                def with_reduce(i, y=y, acc=acc):
                    partial(i, pdl=0)
                    if world > 1:
                        acc.copy_(y)
                        dist.all_reduce(acc)

                e = {"local": whole_job(M, K, N, max_over_ranks(time_launches(stream, partial, reps)))}
                if world > 1:
                    dist.barrier()
                    e["nccl_all_reduce_fp32"] = whole_job(M, K, N, max_over_ranks(time_launches(stream, with_reduce, reps, graph=False)))
                    if M == 1:
                        try:
                            ex = S._PeerExchange(16, world * N, dev)
                            out = torch.empty(M, N, device=dev, dtype=torch.float16)

                            def fused_reduce(i, x=x, ex=ex, out=out):
                                ex.run(x, pres[i % len(pres)], world, rank * N, world, out)
                            dist.barrier()
                            e["fused_peer_store_reduce"] = whole_job(M, K, N, max_over_ranks(time_launches(stream, fused_reduce, reps, graph=False)))
                            dist.barrier()
                            e["fused_peer_store_reduce_graph"] = whole_job(M, K, N, max_over_ranks(time_launches(stream, fused_reduce, reps)))
                        except Exception as ex_:          # symmetric memory unavailable on this box
                            e["fused_peer_store_reduce"] = {"error": str(ex_)[:200]}
                entry[f"row_parallel_m{M}"] = e
            del pres
            torch.cuda.empty_cache()
        res[label] = entry
    if world > 1:
        res["limit"] = ("at M = 1 a rank's product takes a few microseconds, so the step is bounded by the collective's latency "
                        "(NCCL launch + ring/tree steps; for the fused forms a peer store over NVLink and the readers' polling, "
                        "no barrier), not by HBM")
    return res


def run_probe(spec: str) -> None:
    """`--probe MxKxN`: six distinct weights, a warm-up launch and then one q4b_matmul launch each (fp16 activations), then the
    wait status; prints the average device time.  `--probe chain:L`: L layers of the 7B-shaped stage
    list, three runs.  `--probe quantize:NxK`: the packer on three fp16 [N, K] weights, both output
    forms.  `--probe int4g:M`: matmul_int4 (K=4096, N=14336, group 128, bf16) three times.  Small fixed cases for profiler captures."""
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    dev = torch.device("cuda", 0)
    lib = _cabi.load()
    if spec.startswith("chain:"):
        layers = int(spec.split(":")[1])
        stack = build_stack(dev, layers, 4242)
        xs = {K: torch.randn(1, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}
        ready, flow = build_chains(dev, stack, xs, layers)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ready.run()
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(3):
            ready.run()
        e1.record()
        torch.cuda.synchronize(dev)
        print(json.dumps({"probe": spec, "launches": 3, "us_per_launch": e0.elapsed_time(e1) * 1e3 / 3,
                          "bytes_per_launch": sum(gemv_bytes(1, K, N) for _, K, N, _ in stack), "wait_status": Q.wait_status(dev)}))
        return
    if spec.startswith("int4g:"):
        import metalops_b200 as mo
        M = int(spec.split(":")[1])
        K, N, G = 4096, 14336, 128
        g = torch.Generator(device=dev).manual_seed(4242)
        w = (torch.randn(K, N, generator=g, device=dev) * 0.02).half()
        p, s_, z = mo.quantize_int4(w, G)
        x = torch.randn(M, K, generator=g, device=dev).bfloat16()
        y = mo.matmul_int4(x, p, s_, z, G)                         # prepacks once, warms up
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            y = mo.matmul_int4(x, p, s_, z, G)
        e1.record()
        torch.cuda.synchronize(dev)
        print(json.dumps({"probe": spec, "launches": 3, "us_per_product": e0.elapsed_time(e1) * 1e3 / 3, "wait_status": Q.wait_status(dev)}))
        return
    if spec.startswith("quantize:"):
        N, K = (int(v) for v in spec.split(":")[1].lower().split("x"))
        g = torch.Generator(device=dev).manual_seed(4242)
        ws = [(torch.randn(N, K, generator=g, device=dev) * 0.02).half() for _ in range(3)]
        blocks = torch.empty((K // 32, N, 18), dtype=torch.uint8, device=dev)
        pre = torch.empty(lib.q4b_prepacked_bytes(K, N), dtype=torch.uint8, device=dev)
        sp = _cabi.stream_ptr(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        _cabi.check(lib.q4b_quantize(ws[0].data_ptr(), _cabi.F16, K, N, _cabi.LAYOUT_NK, blocks.data_ptr(), pre.data_ptr(), sp), "q4b_quantize")
        torch.cuda.synchronize(dev)
        e0.record()
        for w in ws:
            _cabi.check(lib.q4b_quantize(w.data_ptr(), _cabi.F16, K, N, _cabi.LAYOUT_NK, blocks.data_ptr(), pre.data_ptr(), sp), "q4b_quantize")
        e1.record()
        torch.cuda.synchronize(dev)
        print(json.dumps({"probe": spec, "launches": 3, "us_per_launch": e0.elapsed_time(e1) * 1e3 / 3}))
        return
    M, K, N = (int(v) for v in spec.lower().split("x"))
    g = torch.Generator(device=dev).manual_seed(4242)
    pres = [Q._quantize_impl(torch.randn(K, N, generator=g, device=dev) * 0.02, False, True)[1] for _ in range(6)]
    x = torch.randn(M, K, generator=g, device=dev).half()
    y = torch.empty(M, N, device=dev, dtype=torch.float16)
    sp = _cabi.stream_ptr(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _cabi.check(lib.q4b_matmul(x.data_ptr(), _cabi.F16, M, K, pres[0].data.data_ptr(), K, N, y.data_ptr(), N, 0, sp), "q4b_matmul")
    torch.cuda.synchronize(dev)                  # the first launch pays the one-time set-up
    e0.record()
    for p in pres:
        _cabi.check(lib.q4b_matmul(x.data_ptr(), _cabi.F16, M, K, p.data.data_ptr(), K, N, y.data_ptr(), N, 0, sp), "q4b_matmul")
    e1.record()
    torch.cuda.synchronize(dev)
    print(json.dumps({"probe": spec, "launches": len(pres), "us_per_launch": e0.elapsed_time(e1) * 1e3 / len(pres),
                      "wait_status": Q.wait_status(dev)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--probe", default=None, metavar="MxKxN|chain:L|quantize:NxK|int4g:M", help="run one small case and exit (profiler captures)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-gemm", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-variants", action="store_true", help="skip the data-flow and per-projection-launch forms of the step")
    ap.add_argument("--skip-extra", action="store_true", help="skip the packer, sweep, batch and sharded objects")
    args = ap.parse_args()
    if args.probe:
        run_probe(args.probe)
        return
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
