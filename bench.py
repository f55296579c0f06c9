#!/usr/bin/env python
"""Benchmark of the q4_0 INT4 matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the Llama-2-7B-shaped decode projections at M = 1 — 32 layers of
q/k/v/o [4096 -> 4096], gate/up [4096 -> 11008], down [11008 -> 4096], all with distinct q4_0
weights (3.64 GB of packed weights, 29x the L2), fp16 activations.  One step = one pass over all
224 projections.  The metric is algorithmic GB/s: (18 bytes per 32 weights + X + Y bytes) / time.
The same run also reports the prefill GEMM (M = 2048, K = 4096, N = 14336, bf16) in TFLOP/s.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of the
reference's own torch path (dequantise + matmul) on the host cores instead.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = 32
PROJ = [("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096),
        ("gate", 4096, 11008), ("up", 4096, 11008), ("down", 11008, 4096)]
GEMM_SHAPE = (2048, 4096, 14336)          # M, K, N of the prefill configuration


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
    """DRAM traffic figures taken from the committed ncu summaries (dram__bytes_read.sum +
    dram__bytes_write.sum of one captured launch; the bench never runs under a profiler).

    gemv: profiles/gemv_m1_kernel_llama7b_layer.md — DRAM bytes / algorithmic bytes measured on the
    three shapes of a layer (1.002, 1.000, 1.001), i.e. traffic grows in proportion to the bytes
    of a launch; the step's average launch is scaled by that ratio.
    gemm: profiles/gemm_tcgen05_kernel_m2048.md — 50.0 MB read + 12.1 MB written for the bench's
    M=2048, K=4096, N=14336 launch."""
    return {"gemv_dram_bytes_per_algorithmic_byte": 1.001, "gemm_dram_bytes_per_launch": 62.1e6}


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
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


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


def run_ours(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this build has no CPU path")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    lib = _cabi.load()
    _cabi.stream_ptr(dev)

    M = args.m
    flags = 0 if args.no_pdl else _cabi.FLAG_PDL
    # weak scaling: every rank owns the column shard [rank*N, (rank+1)*N) of layers that are
    # `world` times wider; per-GPU shapes (and bytes) are those of the 7B stack.
    stack = build_stack(dev, args.layers, 1002 + rank)
    xs = {K: torch.randn(M, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}
    ys = [torch.empty(M, N, device=dev, dtype=torch.float16) for _, _, N, _ in stack]
    step_bytes = sum(gemv_bytes(M, K, N) for _, K, N, _ in stack)
    launches_per_step = len(stack)

    stream = torch.cuda.Stream(dev)

    def enqueue_step():
        sp = torch.cuda.current_stream(dev).cuda_stream
        for (name, K, N, pre), y in zip(stack, ys):
            x = xs[K]
            rc = lib.q4b_gemv(x.data_ptr(), _cabi.F16, M, K, pre.data.data_ptr(), K, N, y.data_ptr(), N, flags, sp)
            if rc:
                _cabi.check(rc, "q4b_gemv")

    graph = None
    with torch.cuda.stream(stream):
        for _ in range(2):
            enqueue_step()
        stream.synchronize()
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                enqueue_step()

        def step():
            if graph is not None:
                graph.replay()
            else:
                enqueue_step()

        for _ in range(args.warmup):
            step()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clk:
            e0.record(stream)
            for _ in range(args.steps):
                step()
            e1.record(stream)
            stream.synchronize()
            if clk.proc is not None and e0.elapsed_time(e1) < 400:
                # keep the same work running a little longer so the sampler sees clocks under load
                t_end = time.time() + 0.6
                while time.time() < t_end:
                    step()
                stream.synchronize()
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1)

    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = step_bytes * world * args.steps / (ms * 1e-3) / 1e9
    per_gpu = step_bytes * args.steps / (ms * 1e-3) / 1e9
    peaks = measured_peaks()
    traffic = recorded_traffic()

    # ---- end to end through the C ABI with host buffers (H2D of X, product, D2H of Y) ------
    e2e = None
    if not args.skip_e2e:
        hx = {K: torch.randn(M, K, dtype=torch.float16).pin_memory() for K in (4096, 11008)}
        hy = [torch.empty(M, N, dtype=torch.float16).pin_memory() for _, _, N, _ in stack]
        dx = {K: torch.empty(M, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}

        def e2e_step():
            sp = stream.cuda_stream
            for (name, K, N, pre), y, yh in zip(stack, ys, hy):
                rc = lib.q4b_matmul_host(hx[K].data_ptr(), dx[K].data_ptr(), _cabi.F16, M, pre.data.data_ptr(), K, N,
                                         y.data_ptr(), yh.data_ptr(), 0, sp)
                if rc:
                    _cabi.check(rc, "q4b_matmul_host")
            stream.synchronize()

        with torch.cuda.stream(stream):
            for _ in range(min(3, args.warmup)):
                e2e_step()
            if world > 1:
                dist.barrier()
            n_e2e = max(3, min(args.steps, 20))
            t0 = time.perf_counter()
            for _ in range(n_e2e):
                e2e_step()
            dt = time.perf_counter() - t0
        te = torch.tensor([dt], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e = {"value": step_bytes * world * n_e2e / float(te.item()) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": sum(2 * M * K for _, K, _, _ in stack),
               "d2h_bytes_per_step": sum(2 * M * N for _, _, N, _ in stack), "steps": n_e2e,
               "note": "per projection: H2D of X from pinned memory, kernel, D2H of Y, through q4b_matmul_host"}

    # ---- prefill GEMM (rank 0's GPU only at N > 1: the same kernel runs on every rank) -----
    gemm = None
    batch = None
    if not args.skip_gemm:
        gemm = bench_gemm(dev, stream, lib, peaks, traffic, args)
        if rank == 0 and args.layers >= 4:
            batch = bench_batch(dev, stream, lib, stack, flags)

    out = None
    if rank == 0:
        clocks = clk.summary()
        out = {
            "metric": "q4_0_gemv_gbps_m1", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"llama2-7b decode projections, M={M}, q4_0 weights, fp16 activations",
                       "layers": args.layers, "projections_per_step": launches_per_step,
                       "packed_weight_bytes_per_gpu": sum(p.nbytes() for *_, p in stack),
                       "l2": "inputs (3.6 GB of distinct weights per step) exceed the 126 MB L2; no flush needed",
                       "launch": ("cuda graph" if graph is not None else "stream") + (", pdl" if flags else ""),
                       "parallelism": f"column-parallel x{world}, outputs kept sharded (no collective in the step)"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "frac_of_nominal_8tbs": per_gpu / 8000.0,
                         "kernel": "gemv_m1_kernel", "launches": launches_per_step * args.steps,
                         "avg_launch_us": ms * 1e3 / (launches_per_step * args.steps),
                         "traffic": (traffic.get("gemv_dram_bytes_per_algorithmic_byte") or 0) * step_bytes / launches_per_step
                         if traffic.get("gemv_dram_bytes_per_algorithmic_byte") else None},
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        }
        if gemm is not None:
            out["gemm"] = gemm
        if batch is not None:
            out["decode_batch"] = batch
    if rank == 0 and not args.skip_cpu and world >= 1:
        out["cpu_baseline"] = cpu_baseline()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def cpu_baseline():
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    items = cpu_layer_inputs(1002, 1)
    cpu_layer_pass(items)
    best = min(cpu_layer_pass(items) for _ in range(3))
    layer_bytes = sum(gemv_bytes(1, K, N) for _, K, N in PROJ)
    return {"value": layer_bytes / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "one layer (7 projections, 1/32 of a step) through the CPU restatement of the reference's "
                      "dequantise + torch matmul path, best of 3", "seconds": best}


def bench_gemm(dev, stream, lib, peaks, traffic, args):
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    M, K, N = GEMM_SHAPE
    g = torch.Generator(device=dev).manual_seed(1003)
    # several distinct weights and activations so consecutive launches do not hit in L2
    nset = 4
    pres, xs, ys = [], [], []
    for _ in range(nset):
        w = torch.randn(K, N, generator=g, device=dev) * 0.02
        idx = torch.randint(0, K * N, (K * N // 1000,), generator=g, device=dev)
        w.view(-1)[idx] = torch.where(torch.rand(idx.numel(), generator=g, device=dev) < 0.5, -0.5, 0.5)
        pres.append(Q._quantize_impl(w, False, True)[1])
        xs.append(torch.randn(M, K, generator=g, device=dev).bfloat16())
        ys.append(torch.empty(M, N, device=dev, dtype=torch.bfloat16))
        del w
    reps = 20

    def run(n):
        sp = stream.cuda_stream
        for i in range(n):
            j = i % nset
            rc = lib.q4b_gemm(xs[j].data_ptr(), _cabi.BF16, M, K, pres[j].data.data_ptr(), K, N, ys[j].data_ptr(), N, 0, sp)
            if rc:
                _cabi.check(rc, "q4b_gemm")

    with torch.cuda.stream(stream):
        run(5)
        stream.synchronize()
        detail = torch.zeros(1, dtype=torch.int32)
        import ctypes
        d = ctypes.c_int(0)
        rc = lib.q4b_wait_status(stream.cuda_stream, ctypes.byref(d))
        if rc:
            return {"error": f"gemm status {rc} detail {d.value}"}
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run(reps)
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    tf = 2.0 * M * K * N / (ms * 1e-3) / 1e12
    return {"metric": "q4_0_gemm_tflops_m2048", "value": tf, "unit": "TFLOP/s", "ms_per_launch": ms,
            "config": {"workload": f"prefill GEMM M={M} K={K} N={N}, bf16 activations, q4_0 weights with 0.1% outliers",
                       "l2": f"{nset} distinct weight/activation sets (4 x 150 MB) rotate, larger than L2"},
            "dtype": "bf16",
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "frac_of_sustained": tf / peaks["bf16_tflops_sustained"],
                         "frac_of_nominal_2250": tf / 2250.0, "peak_source": peaks["source"],
                         "kernel": "gemm_tcgen05_kernel", "traffic": traffic.get("gemm_dram_bytes_per_launch")},
            "gpu_launches": reps}


def bench_batch(dev, stream, lib, stack, flags):
    """Decode batches: the same projections at M = 4, 16 and 64 rows through q4b_matmul (decode kernel,
    tensor-memory kernel), the first four layers (455 MB of weights, larger than L2) in a CUDA
    graph.  Reported for information next to the M = 1 headline."""
    from metalops_b200 import _cabi
    sub = stack[: 4 * len(PROJ)]
    out = {}
    for M in (4, 16, 64):
        xs = {K: torch.randn(M, K, device=dev, dtype=torch.float16) for K in (4096, 11008)}
        ys = [torch.empty(M, N, device=dev, dtype=torch.float16) for _, _, N, _ in sub]

        def enqueue():
            sp = torch.cuda.current_stream(dev).cuda_stream
            for (name, K, N, pre), y in zip(sub, ys):
                rc = lib.q4b_matmul(xs[K].data_ptr(), _cabi.F16, M, K, pre.data.data_ptr(), K, N, y.data_ptr(), N, flags, sp)
                if rc:
                    _cabi.check(rc, "q4b_matmul")

        with torch.cuda.stream(stream):
            enqueue()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                enqueue()
            for _ in range(3):
                g.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 20
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1) / reps
        nbytes = sum(gemv_bytes(M, K, N) for _, K, N, _ in sub)
        flops = sum(2.0 * M * K * N for _, K, N, _ in sub)
        out[f"m{M}"] = {"gbps": nbytes / (ms * 1e-3) / 1e9, "tflops": flops / (ms * 1e-3) / 1e12,
                        "us_per_launch": ms * 1e3 / len(sub)}
    return out


def run_probe(spec: str) -> None:
    """`--probe MxKxN`: six distinct weights, one q4b_matmul launch each (fp16 activations), then the
    wait status; prints the average device time.  A small fixed case for profiler captures."""
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    M, K, N = (int(v) for v in spec.lower().split("x"))
    dev = torch.device("cuda", 0)
    lib = _cabi.load()
    g = torch.Generator(device=dev).manual_seed(4242)
    pres = [Q._quantize_impl(torch.randn(K, N, generator=g, device=dev) * 0.02, False, True)[1] for _ in range(6)]
    x = torch.randn(M, K, generator=g, device=dev).half()
    y = torch.empty(M, N, device=dev, dtype=torch.float16)
    sp = _cabi.stream_ptr(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
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
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="decode batch rows (1..16)")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--probe", default=None, metavar="MxKxN", help="run one small product six times and exit (profiler captures)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-gemm", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
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
