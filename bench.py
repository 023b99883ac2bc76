#!/usr/bin/env python
"""Benchmark of the int4 block-quantized decode linear (the configuration the headline metric,
weight HBM GB/s against the roofline, is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("int4_decode_gemv"): W [11264, 4096] int4 in 32-element blocks with f32 block scales;
activations [M, 4096] quantized per row to int8, M in {1, 4, 16}; f32 output.  One step = one pass
over `replicas` distinct copies of the weights for each M (3 * replicas launches), so that the
working set (replicas * 28.8 MB) is several times the L2 and every launch streams its weights from
HBM.  Inputs are synthetic (seeded normal draws with the stated shapes and scales).

value   = weight-side bytes streamed per second with everything resident in HBM (kernel time only)
e2e     = the same bytes per second through the public API with host buffers: every launch copies
          its activations from pinned host memory, quantizes them on the device, runs the linear
          and copies the result back; the weights stay resident (they are model parameters)
N > 1   = one process per GPU, each with its own decode streams and a replica of the weights
          (rows of the batch are independent: no collective on the data path), weak scaling.
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

N_OUT, K_IN = 11264, 4096
MS = (1, 4, 16)
METRIC, UNIT = "int4_decode_gemv_weight_bandwidth", "GB/s"


def weight_bytes() -> int:
    return N_OUT * K_IN // 2 + N_OUT * (K_IN // 32) * 4  # packed nibbles + f32 block scales


def algorithmic_bytes(m: int) -> int:
    return weight_bytes() + m * K_IN + 4 * m + 4 * m * N_OUT  # + int8 activations, row scales, f32 out


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class CpuPort:
    """The oracle's int4 linear on the host cores (OpenMP): one pass = M in {1,4,16} over one weight copy."""

    def __init__(self):
        import numpy as np

        import oracle as O
        O.build()
        self.O = O
        rng = np.random.default_rng(1)
        w = (rng.standard_normal((N_OUT, K_IN)) * 0.02).astype(np.float32)
        self.q, self.s = O.quantize_q4(w)
        self.x = {m: O.quantize_rows_i8(rng.standard_normal((m, K_IN)).astype(np.float32)) for m in MS}
        self.threads = O.num_threads()
        self.run_pass()  # warm-up

    def run_pass(self) -> float:
        t0 = time.perf_counter()
        for m in MS:
            self.O.linear_q(*self.x[m], self.q, self.s, want_partials=False)
        return time.perf_counter() - t0

    def throughput(self, budget_s: float):
        """(GB/s of weight-side bytes, passes, seconds) over about budget_s seconds."""
        t0, passes = time.perf_counter(), 0
        while passes < 1 or time.perf_counter() - t0 < budget_s:
            self.run_pass()
            passes += 1
        dt = time.perf_counter() - t0
        return passes * len(MS) * weight_bytes() / dt / 1e9, passes, dt


def run_reference(args) -> None:
    """The reference arm: xn has no int4 path and its CPU matmul (crate `gemm`, Rust) cannot be
    built here, so this times the CPU restatement of the same arithmetic on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    port = CpuPort()
    t_start = time.perf_counter()
    for _ in range(args.warmup):
        port.run_pass()
        if time.perf_counter() - t_start > 60:
            break
    per_step = []
    for _ in range(args.steps):
        per_step.append(port.run_pass())
        if time.perf_counter() - t_start > 240:
            break
    value = len(MS) * weight_bytes() / statistics.mean(per_step) / 1e9
    sample = "one pass of M in {1,4,16} over one weight copy per step (3 linears); int8 x int4 integer port, OpenMP"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": len(per_step), "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(per_step),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xint4->int32",
            "data": "synthetic", "config": {"workload": "int4_decode_gemv", "n": N_OUT, "k": K_IN, "m": list(MS)},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": port.threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def measure_decode(args, dev, world, rank, timed):
    """Decoder-stack configuration: 32 layers, d_model 4096, 32 heads x 128, gated SiLU FFN hidden 11264,
    fp8-e4m3 weights (W8A16 form), 32 independent streams per GPU each with a 3000-token bf16 KV cache.
    One step = one token for every stream, replayed as a CUDA graph.  Streams are sharded over the
    GPUs with no communication, so the whole-job figure is the sum over ranks."""
    import torch

    from xn_b200.decoder import DecoderStack
    streams, ctx = 32, 3000
    try:
        st = DecoderStack(32, 4096, 32, 11264, streams, ctx, dev, seed=4 + rank)
    except torch.cuda.OutOfMemoryError:
        return {"unavailable": "not enough free device memory for the 57 GB decode working set"}
    x = torch.randn(streams, 4096, device=dev).bfloat16()
    st.step(x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            st.step(x)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    ms = timed(graph.replay, args.decode_steps)
    per_step = ms / args.decode_steps
    b = st.bytes_per_step()
    peak, kind = measured_peak_gbs()
    return {"ms_per_step": per_step, "steps_per_s_per_gpu": 1e3 / per_step, "streams_per_gpu": streams,
            "tokens_per_s_all_gpus": world * streams * 1e3 / per_step, "context": ctx,
            "bytes_per_step_per_gpu": b["total"], "gb_per_s_per_gpu": b["total"] / (per_step * 1e-3) / 1e9,
            "frac_of_hbm_peak": b["total"] / (per_step * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}",
            "launches_per_step": st.launches_per_step(), "variant": "W8A16",
            "l2": "working set 57 GB per GPU, far larger than L2"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="xn_b200", choices=["xn_b200", "reference"])
    ap.add_argument("--replicas", type=int, default=24)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--sweeps", type=int, default=16, help="passes over all replicas and M values per step")
    ap.add_argument("--no-decode", action="store_true", help="skip the decoder-stack step measurement")
    ap.add_argument("--decode-steps", type=int, default=8)
    ap.add_argument("--decode-only", action="store_true", help="measure only the decoder-stack step (profiling aid)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    import xn_b200 as xn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        barrier()
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if args.decode_only:
        d = measure_decode(args, dev, world, rank, timed)
        if rank == 0:
            print(json.dumps({"decode_step": d}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- synthetic operands, resident in HBM ----
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    R = args.replicas
    lins = []
    for _ in range(R):
        w = torch.randn(N_OUT, K_IN, generator=g, device=dev) * 0.02
        lins.append(xn.LinearQ4.from_weight(w))
        del w
    acts = {m: xn.quantize_rows_i8(torch.randn(m, K_IN, generator=g, device=dev)) for m in MS}
    outs = {m: torch.empty(m, N_OUT, device=dev) for m in MS}
    host_x = {m: torch.randn(m, K_IN).pin_memory() for m in MS}
    host_y = {m: torch.empty(m, N_OUT).pin_memory() for m in MS}
    SWEEPS = args.sweeps
    launches_per_step = len(MS) * R * SWEEPS

    def enqueue_sweep():
        for m in MS:
            xq, xs = acts[m]
            for lin in lins:
                xn.linear_q4(xq, xs, lin.wq, N_OUT, out=outs[m])

    # A decode loop replays the same launches every token, so the step is captured once in a CUDA
    # graph and replayed: this takes host launch overhead (Python + driver) out of the kernel-time
    # measurement.  The end-to-end leg below goes through plain API calls instead.
    enqueue_sweep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(SWEEPS):
                enqueue_sweep()
    torch.cuda.synchronize()

    def step():
        graph.replay()

    # End to end: a serving loop keeps its device buffers, so the host->device copy, the activation
    # quantizer and the linear all write into preallocated tensors; every call still goes through the
    # Python API and copies its input from and its result to pinned host memory.
    dev_x = {m: torch.empty(m, K_IN, device=dev) for m in MS}
    dev_q = {m: (torch.empty(m, K_IN, dtype=torch.int8, device=dev), torch.empty(m, device=dev)) for m in MS}

    def step_e2e():
        for m in MS:
            for lin in lins:
                dev_x[m].copy_(host_x[m], non_blocking=True)
                xq, xs = xn.quantize_rows_i8(dev_x[m], out=dev_q[m])
                xn.linear_q4(xq, xs, lin.wq, N_OUT, out=outs[m])
                host_y[m].copy_(outs[m], non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the step's result is on the host

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    for _ in range(2):
        step_e2e()
    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e = timed(step_e2e, e2e_steps)

    decode = None
    if not args.no_decode:
        del lins, graph
        torch.cuda.empty_cache()
        decode = measure_decode(args, dev, world, rank, timed)

    wb = weight_bytes()
    total_weight_bytes = world * args.steps * launches_per_step * wb
    value = total_weight_bytes / (ms * 1e-3) / 1e9
    e2e_value = world * e2e_steps * len(MS) * R * wb / (ms_e2e * 1e-3) / 1e9  # one sweep per e2e step

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        launch_s = ms * 1e-3 / (args.steps * launches_per_step)
        alg = sum(algorithmic_bytes(m) for m in MS) / len(MS)
        achieved = alg / launch_s / 1e9
        cpu_baseline = None
        if world == 1:  # the CPU leg runs at N = 1 only (torchrun pins OMP to one thread per rank)
            port = CpuPort()
            cpu_gbs, passes, cpu_dt = port.throughput(args.cpu_seconds)
            cpu_baseline = {"value": cpu_gbs, "unit": UNIT, "cores": port.threads, "kind": "port",
                            "sample": f"{passes} pass(es) of M in {{1,4,16}} over one weight copy, {cpu_dt:.1f} s"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8xint4->int32", "data": "synthetic",
            "config": {"workload": "int4_decode_gemv", "n": N_OUT, "k": K_IN, "m": list(MS), "replicas": R, "sweeps_per_step": SWEEPS,
                       "launch": "one CUDA graph replay per step",
                       "l2": f"inputs larger than L2: {R} distinct weight copies = {R * wb / 1e6:.0f} MB per M",
                       "parallelism": f"streams sharded over {world} gpu(s), no collective"},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": R * sum(m * K_IN * 4 for m in MS),
                    "d2h_bytes_per_step": R * sum(m * N_OUT * 4 for m in MS), "steps": e2e_steps,
                    "ms_per_step": ms_e2e / e2e_steps},
            "gpu_launches": args.steps * launches_per_step,
            "decode_step": decode,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": 28875776,
                         "traffic_source": "dram__bytes_read+write per launch, ncu capture in profiles/linear_q4_kernel_int4_decode_gemv.md",
                         "kernel": "linear_q4_kernel",
                         "algorithmic_bytes_per_launch": alg, "us_per_launch": launch_s * 1e6},
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
