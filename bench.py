#!/usr/bin/env python
"""Benchmark of the int4 block-quantized decode linear (the configuration the headline metric,
weight HBM GB/s against the roofline, is quoted on), with the other measurements the metric names riding
on the same JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("int4_decode_gemv"): W [11264, 4096] int4 in 32-element blocks with f32 block scales;
activations [M, 4096] quantized per row to int8, M in {1, 4, 16}; f32 output.  One step = `sweeps` passes
over `replicas` distinct copies of the weights for each M (3 * replicas * sweeps launches), so that the
working set (replicas * 28.8 MB) is several times the L2 and every launch streams its weights from
HBM.  Inputs are synthetic (seeded normal draws with the stated shapes and scales).

value   = weight-side bytes streamed per second with everything resident in HBM (kernel time only)
e2e     = the same bytes per second through the host-buffer entry point (xn_mm_linear_q4_host): every call
          copies its activations from pinned host memory, quantizes them on the device, runs the linear
          and copies the result back; the weights stay resident (they are model parameters)
N > 1   = one process per GPU, each with its own decode streams and a replica of the weights
          (rows of the batch are independent: no collective on the data path), weak scaling.

Further keys of the line (each measured in this run, CUDA events, L2 flushed between timed launches):
  fp8_prefill_gemm         fp8-e4m3 transformer linears at M = 4096 (W8A8 and W8A16), TFLOP/s and roofline
  int4_prefill_gemm        the benchmark's int4 weight with 256 / 1024 / 4096 activation rows (kind::i8 tensor-memory kernel)
  f32_linear               x [16,4096] * W [11264,4096]^T in f32 on the GPU, and the host-core baseline
  decode_step              the 32-layer decoder step, 32 streams per GPU
  prefill_column_parallel  (N > 1) the same linears with the weight rows split over the ranks and the
                           outputs assembled on every rank: peer-store epilogue, NVLink multicast and NCCL routes
  prefill_stack            a 4096-token prefill of one stream through the 32-layer stack, weights split over the ranks
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


def make_config(world: int) -> dict:
    """The workload description both arms print (identical text, so the two lines compare like for like)."""
    return {"workload": "int4_decode_gemv", "n": N_OUT, "k": K_IN, "m": list(MS),
            "l2": "inputs larger than L2: the GPU arm rotates over distinct weight copies (692 MB per M), the host arm "
                  "streams a 46 MB weight through a far smaller cache",
            "parallelism": f"streams sharded over {world} gpu(s), no collective"}


class CpuPort:
    """The CPU restatement of the int4 linear on the host cores (OpenMP over output channels; AVX-512 VNNI
    when the host has it): one pass = M in {1,4,16} over one weight copy."""

    def __init__(self):
        import numpy as np

        import oracle as O
        O.build()
        self.O = O
        self.threads = O.use_all_cores()  # torchrun exports OMP_NUM_THREADS=1 to every rank
        self.kind = O.linear_q_fast_kind()
        rng = np.random.default_rng(1)
        w = (rng.standard_normal((N_OUT, K_IN)) * 0.02).astype(np.float32)
        self.w = w
        self.q, self.s = O.quantize_q4(w)
        self.x = {m: O.quantize_rows_i8(rng.standard_normal((m, K_IN)).astype(np.float32)) for m in MS}
        self.xf = rng.standard_normal((16, K_IN)).astype(np.float32)
        self.run_pass()  # warm-up

    def run_pass(self, repeats: int = 1) -> float:
        t0 = time.perf_counter()
        for _ in range(repeats):
            for m in MS:
                self.O.linear_q_fast(*self.x[m], self.q, self.s)
        return time.perf_counter() - t0

    def throughput(self, budget_s: float):
        """(GB/s of weight-side bytes, passes, seconds) over about budget_s seconds."""
        t0, passes = time.perf_counter(), 0
        while passes < 1 or time.perf_counter() - t0 < budget_s:
            self.run_pass()
            passes += 1
        dt = time.perf_counter() - t0
        return passes * len(MS) * weight_bytes() / dt / 1e9, passes, dt

    def f32_linear(self, runs: int = 10) -> dict:
        """The reference's own CPU-runnable configuration: y = x W^T in f32 (x [16,4096], W [11264,4096])."""
        self.O.linear_f32_fast(self.xf, self.w)
        ts = []
        for _ in range(runs):
            t0 = time.perf_counter()
            self.O.linear_f32_fast(self.xf, self.w)
            ts.append(time.perf_counter() - t0)
        best, med = min(ts), statistics.median(ts)
        by, fl = 185532416, 1476395008
        return {"ms_best": best * 1e3, "ms_median": med * 1e3, "gb_per_s": by / med / 1e9, "gflop_per_s": fl / med / 1e9,
                "cores": self.threads, "runs": runs, "kind": "port (f32 FMA, compiler-vectorised, OpenMP over n)"}


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
    REP = 64  # passes per step: a step is a bounded sample of the workload, about 0.1-0.5 s of host time
    per_step = []
    for _ in range(args.steps):
        per_step.append(port.run_pass(REP))
        if time.perf_counter() - t_start > 240:
            break
    value = REP * len(MS) * weight_bytes() / statistics.mean(per_step) / 1e9
    sample = (f"{REP} passes of M in {{1,4,16}} over one weight copy per step ({3 * REP} linears); int8 x int4 integer port, "
              f"{port.kind}, OpenMP on {port.threads} threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": len(per_step), "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(per_step),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xint4->int32",
            "data": "synthetic", "config": make_config(args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": port.threads, "kind": "port", "sample": sample},
            "f32_linear_cpu": port.f32_linear(),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# DRAM bytes per launch of the dominant kernel from ncu (dram__bytes_read.sum + dram__bytes_write.sum), keyed by
# instantiation; the capture and its command are summarised in profiles/linear_q4_kernel_int4_decode_gemv.md.
NCU_DRAM_BYTES_PER_LAUNCH = {"M<=8": 28874304, "M=9..16": 28927232}


class L2Flush:
    """Writes a buffer larger than the 126 MB L2 between timed launches."""

    def __init__(self, dev):
        import torch
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.zero_()


def time_launches(fn, iters: int, flush, torch) -> float:
    """Median device time in ms of one call of fn, each call bracketed by its own pair of CUDA events on the
    current stream, L2 flushed (untimed) before every call."""
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return json.load(open(p))
    except Exception:
        return {}


SHAPES = [(12288, 4096, "qkv"), (4096, 4096, "out_proj"), (22528, 4096, "ffn_up"), (4096, 11264, "ffn_down")]


def measure_fp8_prefill(dev, flush, xn, torch) -> dict:
    """fp8-e4m3 linears at M = 4096 on the tcgen05 kernel: W8A8 (one e4m3 activation piece) and W8A16 (two
    pieces, i.e. twice the tensor work for the same useful flops).  TFLOP/s counts 2*M*N*K once."""
    m = 4096
    peaks = measured_peaks()
    bf16_burst = float(peaks.get("bf16_tflops", 1590.0))
    rows = []
    g = torch.Generator(device=dev).manual_seed(2)
    for n, k, name in SHAPES:
        w = torch.randn(n, k, generator=g, device=dev) * 0.02
        wq, ws = xn.quantize_weights_fp8(w)
        del w
        x = torch.randn(m, k, generator=g, device=dev).bfloat16()
        hi, lo, xs = xn.split_rows_e4m3(x)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        st = torch.cuda.current_stream().cuda_stream
        for variant, lo_ptr in (("W8A8", None), ("W8A16", lo.data_ptr())):
            def call():
                xn._lib.check(xn.lib().xn_mm_linear_fp8_pieces(y.data_ptr(), hi.data_ptr(), lo_ptr, xs.data_ptr(),
                                                               wq.data_ptr(), ws.data_ptr(), m, n, k, st))
            ms = time_launches(call, 10, flush, torch)
            tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            nominal = 4500.0 if variant == "W8A8" else 2250.0
            rows.append({"name": name, "m": m, "n": n, "k": k, "variant": variant, "us": ms * 1e3, "tflops": tf,
                         "roofline": {"bound": "tensor", "achieved": tf, "peak": nominal, "unit": "TFLOP/s",
                                      "frac": tf / nominal, "peak_kind": "nominal dense " + ("fp8" if variant == "W8A8" else "bf16")},
                         "frac_of_measured_bf16_burst": tf / bf16_burst})
        del wq, ws, x, hi, lo, y
    out = {"rows": rows, "measured_bf16_burst_tflops": bf16_burst,
           "note": "W8A16 runs two e4m3 MMAs per product (hi + lo activation pieces); its useful flops are judged against "
                   "the bf16 peak, W8A8's against the fp8 peak"}
    # one library fp8 GEMM of the same size for context (cuBLASLt through torch; not part of the product path)
    try:
        a = torch.randn(4096, 4096, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(12288, 4096, device=dev).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)

        def lib_call():
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        ms = time_launches(lib_call, 10, flush, torch)
        out["library_fp8_gemm_4096x12288x4096_tflops"] = 2.0 * 4096 * 12288 * 4096 / (ms * 1e-3) / 1e12
    except Exception as e:  # noqa: BLE001
        out["library_fp8_gemm_4096x12288x4096_tflops"] = None
        out["library_fp8_note"] = f"torch._scaled_mm unavailable: {type(e).__name__}"
    return out


def measure_q4_prefill(dev, flush, xn, torch) -> dict:
    """The benchmark's int4 weight [11264, 4096] with many activation rows: one unpack of the q4 tiles plus one
    launch of the kind::i8 tensor-memory kernel per call (both inside the timed region).  TOP/s counts 2*M*N*K."""
    g = torch.Generator(device=dev).manual_seed(4)
    w = torch.randn(N_OUT, K_IN, generator=g, device=dev) * 0.02
    lin = xn.LinearQ4.from_weight(w)
    del w
    rows = []
    for m in (256, 1024, 4096):
        x = torch.randn(m, K_IN, generator=g, device=dev)
        xq, xs = xn.quantize_rows_i8(x)
        y = torch.empty(m, N_OUT, device=dev)
        ms = time_launches(lambda: xn.linear_q4(xq, xs, lin.wq, N_OUT, out=y), 10, flush, torch)
        tops = 2.0 * m * N_OUT * K_IN / (ms * 1e-3) / 1e12
        rows.append({"m": m, "n": N_OUT, "k": K_IN, "us": ms * 1e3, "tops": tops,
                     "decode_kernel_passes_us_estimate": (m // 16) * 8.1,
                     "roofline": {"bound": "tensor", "achieved": tops, "peak": 4500.0, "unit": "TOP/s", "frac": tops / 4500.0,
                                  "peak_kind": "nominal dense int8"}})
        del x, xq, xs, y
    return {"rows": rows,
            "note": "one MMA per 32-element block with a hand-over to the CUDA cores for the f32 block scale: bound by the "
                    "hand-over round trip and the per-block scaling, not by the tensor pipe"}


def measure_f32_linear(dev, flush, xn, torch) -> dict:
    """The CPU-runnable configuration on the GPU: x [16,4096] N(0,1), W [11264,4096] N(0,0.02), f32."""
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(16, K_IN, generator=g, device=dev)
    w = torch.randn(N_OUT, K_IN, generator=g, device=dev) * 0.02
    lin = xn.Linear(w)
    ms = time_launches(lambda: lin(x), 20, flush, torch)
    by, fl = 185532416, 1476395008
    peak, kind = measured_peak_gbs()
    ref = (x.double() @ w.double().t())
    y = lin(x)
    rms = float(ref.pow(2).mean().sqrt())
    err = float(((y.double() - ref).abs() / ref.abs().clamp_min(1e-2 * rms)).max())
    return {"us": ms * 1e3, "gb_per_s": by / (ms * 1e-3) / 1e9, "tflops": fl / (ms * 1e-3) / 1e12,
            "roofline": {"bound": "hbm", "achieved": by / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": by / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}"},
            "max_rel_err_vs_f64_floor_1e-2_rms": err}


def measure_prefill_column_parallel(dev, world, rank, xn, torch, dist) -> dict:
    """The four fp8 linears at M = 4096 with the weight rows split over the ranks and the [M, N] result assembled
    on every rank, two routes: the GEMM epilogue storing its tiles into every rank's buffer over NVLink, and a local
    GEMM + NCCL all_gather_into_tensor + re-layout.  Both are compared bit for bit with the one-GPU result."""
    from xn_b200.prefill import PeerPrefillLinear, column_parallel_gather
    m = 4096
    rows = []

    def timeit(fn, iters=10):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for n, k, name in SHAPES:
        g = torch.Generator(device=dev).manual_seed(4)  # same weights and inputs on every rank
        w = torch.randn(n, k, generator=g, device=dev) * 0.02
        wq, ws = xn.quantize_weights_fp8(w)
        del w
        x = torch.randn(m, k, generator=g, device=dev).bfloat16()
        hi, lo, xs = xn.split_rows_e4m3(x)
        full = xn.linear_fp8(x, wq, ws, 0)
        lin = PeerPrefillLinear(wq, ws, n, k, m, multicast=False)   # one plain store per peer
        y = lin.forward(hi, lo, xs, m)
        torch.cuda.synchronize()
        same_peer = bool(torch.equal(y, full))
        lin_mc = PeerPrefillLinear(wq, ws, n, k, m, multicast=True)  # one multimem.st through the NVLink multicast mapping
        same_mc, t_mc = None, None
        if lin_mc.multicast:
            lin_mc.out.zero_()
            lin_mc.hdl.barrier()  # no rank stores into a buffer that its owner is still clearing
            y_mc = lin_mc.forward(hi, lo, xs, m)
            torch.cuda.synchronize()
            same_mc = bool(torch.equal(y_mc, full))
        wl, wsl = wq[lin.a:lin.b].contiguous(), ws[lin.a:lin.b].contiguous()

        def local_linear(xx, a, b):
            out = torch.empty(m, b - a, dtype=torch.bfloat16, device=dev)
            xn._lib.check(xn.lib().xn_mm_linear_fp8_pieces(out.data_ptr(), hi.data_ptr(), lo.data_ptr(), xs.data_ptr(),
                                                           wl.data_ptr(), wsl.data_ptr(), m, b - a, k,
                                                           torch.cuda.current_stream().cuda_stream))
            return out
        y2 = column_parallel_gather(x, local_linear, n)
        same_gather = bool(torch.equal(y2, full))
        t_peer = timeit(lambda: lin.forward(hi, lo, xs, m))
        if lin_mc.multicast:
            t_mc = timeit(lambda: lin_mc.forward(hi, lo, xs, m))
        t_gather = timeit(lambda: column_parallel_gather(x, local_linear, n))
        t_full = timeit(lambda: xn.linear_fp8(x, wq, ws, 0))
        flags = torch.tensor([int(same_peer), int(same_gather), int(same_mc is not False)], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        out_bytes = 2 * m * (lin.b - lin.a) * (world - 1)
        best = min(t_peer, t_mc) if t_mc is not None else t_peer
        rows.append({"name": name, "m": m, "n": n, "k": k, "identical_peer": bool(flags[0].item()),
                     "identical_gather": bool(flags[1].item()),
                     "identical_multicast": bool(flags[2].item()) if t_mc is not None else None,
                     "ms_peer_store_epilogue": t_peer, "ms_multicast_store_epilogue": t_mc,
                     "ms_nccl_all_gather": t_gather, "ms_one_gpu": t_full, "speedup_vs_one_gpu": t_full / best,
                     "tflops_all_gpus": 2.0 * m * n * k / (best * 1e-3) / 1e12,
                     "nvlink_bytes_delivered_per_rank": out_bytes,
                     "nvlink_gb_per_s_delivered_per_rank": out_bytes / (best * 1e-3) / 1e9,
                     "nvlink_egress_bytes_per_rank": out_bytes if t_mc is None or t_peer <= t_mc else 2 * m * (lin.b - lin.a)})
        del lin, lin_mc, wq, ws, x, hi, lo, full, y, y2
        torch.cuda.empty_cache()
    return {"world": world, "rows": rows, "scaling": "strong (one 4096-token prefill split over the ranks)",
            "timing": "CUDA events, max over ranks, 10 back-to-back calls; collective: peer stores / NCCL all-gather"}


def measure_prefill_stack(args, dev, world, rank, timed, torch, dist) -> dict:
    """The prefill half of the decoder configuration: 4096 tokens of one stream through the 32-layer stack with every
    weight split by output channel over the ranks (xn_b200.prefill.PrefillStack): local attention on the rank's heads,
    four exchanges per layer (attention output, out_proj, gated FFN activations, linear_out) written into every
    rank's buffers by store epilogues / an all-gather kernel over NVLink.  Strong scaling: the work is fixed."""
    from xn_b200.prefill import PrefillStack
    T, L = 4096, args.prefill_layers
    identical = None
    if world > 1:  # two layers of the split stack against the same two layers on one rank, bit for bit
        g = torch.Generator(device=dev).manual_seed(11)
        xs = torch.randn(T, 4096, generator=g, device=dev).bfloat16()
        a = PrefillStack(2, 4096, 32, 11264, T, dev, seed=4).forward(xs).clone()
        b = PrefillStack(2, 4096, 32, 11264, T, dev, seed=4, single=True).forward(xs)
        torch.cuda.synchronize()
        flag = torch.tensor([int(torch.equal(a, b))], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        identical = bool(flag.item())
        del a, b
        torch.cuda.empty_cache()
    try:
        st = PrefillStack(L, 4096, 32, 11264, T, dev, seed=4)
    except torch.cuda.OutOfMemoryError:
        return {"unavailable": "not enough free device memory for the prefill stack"}
    g = torch.Generator(device=dev).manual_seed(12)
    x = torch.randn(T, 4096, generator=g, device=dev).bfloat16()
    st.forward(x)
    torch.cuda.synchronize()
    steps = 3
    ms = timed(lambda: st.forward(x), steps) / steps
    out = {"tokens": T, "layers": L, "ms": ms, "tokens_per_s": T / (ms * 1e-3), "tflops_all_gpus": st.flops() / (ms * 1e-3) / 1e12,
           "world": world, "scaling": "strong", "identical_to_one_gpu_two_layers": identical,
           "nvlink_bytes_out_per_rank": st.exchanged_bytes_per_rank(),
           "route": "multimem.st through an NVLink multicast mapping" if st.proj_full.mc_ptr else
                    ("plain stores into peer buffers" if world > 1 else "one rank: no exchange"),
           "variant": "W8A16", "attention": "causal, one kernel per layer for all heads of the rank (scores and probabilities in tensor memory)"}
    del st
    torch.cuda.empty_cache()
    return out


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
    side = torch.cuda.Stream()

    def time_mode(mode):
        st.attention = mode
        st.step(x)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                st.step(x)
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        ms_ = timed(graph.replay, args.decode_steps)
        del graph
        return ms_ / args.decode_steps, st.launches_per_step()

    # the same step with cache append + attention + merge + e4m3 split as ONE launch per layer (identical results,
    # fewer launches, measured slower at this size: every attention CTA then ends with a fence and an arrival)
    fused_ms, fused_launches = time_mode("fused_one_launch") if args.decode_attention == "both" else (None, None)
    per_step, launches = time_mode("separate" if args.decode_attention == "both" else args.decode_attention)
    b = st.bytes_per_step()
    peak, kind = measured_peak_gbs()
    return {"ms_per_step": per_step, "steps_per_s_per_gpu": 1e3 / per_step, "streams_per_gpu": streams,
            "tokens_per_s_all_gpus": world * streams * 1e3 / per_step, "context": ctx,
            "bytes_per_step_per_gpu": b["total"], "gb_per_s_per_gpu": b["total"] / (per_step * 1e-3) / 1e9,
            "frac_of_hbm_peak": b["total"] / (per_step * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}",
            "launches_per_step": launches, "variant": "W8A16",
            "one_launch_attention": None if fused_ms is None else
            {"ms_per_step": fused_ms, "launches_per_step": fused_launches,
             "frac_of_hbm_peak": b["total"] / (fused_ms * 1e-3) / 1e9 / peak},
            "l2": "working set 57 GB per GPU, far larger than L2"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="xn_b200", choices=["xn_b200", "reference"])
    ap.add_argument("--replicas", type=int, default=24)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--sweeps", type=int, default=112,
                    help="passes over all replicas and M values per step (a multiple of 16 beyond 16); the default makes a "
                         "step about 50 ms, i.e. a timed region above one second at 20 steps")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the f32 linear, fp8 prefill GEMM and column-parallel prefill measurements")
    ap.add_argument("--no-decode", action="store_true", help="skip the decoder-stack step measurement")
    ap.add_argument("--decode-steps", type=int, default=8)
    ap.add_argument("--decode-only", action="store_true", help="measure only the decoder-stack step (profiling aid)")
    ap.add_argument("--decode-attention", default="both", choices=["both", "separate", "fused", "fused_one_launch"],
                    help="how a layer launches cache append + attention + merge + split; 'both' times the three-launch "
                         "form (reported as the step) and the one-launch form beside it")
    ap.add_argument("--prefill-only", action="store_true", help="measure only the prefill stack (profiling aid)")
    ap.add_argument("--prefill-layers", type=int, default=32)
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

    if args.prefill_only:
        d = measure_prefill_stack(args, dev, world, rank, timed, torch, dist)
        if rank == 0:
            print(json.dumps({"prefill_stack": d}), flush=True)
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
    GS = min(args.sweeps, 16)                 # sweeps captured in one graph
    REPLAYS = max(1, args.sweeps // GS)       # graph replays per step
    SWEEPS = GS * REPLAYS
    launches_per_step = len(MS) * R * SWEEPS

    def enqueue_sweep(ms_list=MS):
        for m in ms_list:
            xq, xs = acts[m]
            for lin in lins:
                xn.linear_q4(xq, xs, lin.wq, N_OUT, out=outs[m])

    # A decode loop replays the same launches every token, so the step is captured once in a CUDA
    # graph and replayed: this takes host launch overhead (Python + driver) out of the kernel-time
    # measurement.  The end-to-end leg below goes through plain API calls instead.
    enqueue_sweep()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()

    def capture(ms_list, sweeps):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(gr, stream=side):
                for _ in range(sweeps):
                    enqueue_sweep(ms_list)
        torch.cuda.synchronize()
        return gr

    graph = capture(MS, GS)

    def step():
        for _ in range(REPLAYS):
            graph.replay()

    # End to end through the host-buffer entry point: one library call per linear copies the activations from
    # pinned host memory, quantizes them, runs the linear and copies the result back to pinned host memory.
    # The calls of a step are independent decode requests, so a serving loop spreads them over a few streams: the
    # copies of one call overlap the kernels of another (every call still pays its own copy in and copy out).
    E2E_STREAMS = [torch.cuda.Stream() for _ in range(int(os.environ.get("XN_BENCH_E2E_STREAMS", "8")))]
    host_ys = {(m, i): torch.empty(m, N_OUT).pin_memory() for m in MS for i in range(R)}

    def step_e2e():
        # the three batch sizes interleaved, as mixed requests arrive: the copy-heavy M = 16 calls overlap the others
        n = 0
        for i, lin in enumerate(lins):
            for m in MS:
                with torch.cuda.stream(E2E_STREAMS[n % len(E2E_STREAMS)]):
                    lin.forward_host(host_x[m], host_ys[(m, i)])
                n += 1
        for st_ in E2E_STREAMS:
            st_.synchronize()  # the step's results are on the host

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = timed(step, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # the same launches one M at a time: the per-M launch time behind the averaged roofline figure
    per_m = {}
    for m in MS:
        gm = capture((m,), 4)
        for _ in range(3):
            gm.replay()
        ms_m = timed(gm.replay, 10)
        per_m[m] = ms_m * 1e-3 / (10 * 4 * R)
        del gm

    for _ in range(2):
        step_e2e()
    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e_eager = timed(step_e2e, e2e_steps)

    # The same calls captured once in a CUDA graph -- copies in, quantizers, linears, copies out, forked over the
    # streams and joined -- and replayed every step, as a serving loop does with a step whose shapes repeat: what is
    # left per step is one graph launch instead of 72 x 4 driver calls from Python, and every step still copies its
    # inputs from and its results to pinned host memory.
    e2e_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(e2e_graph, stream=side):
            for st_ in E2E_STREAMS:
                st_.wait_stream(side)
            n_call = 0
            for i, lin in enumerate(lins):
                for m in MS:
                    with torch.cuda.stream(E2E_STREAMS[n_call % len(E2E_STREAMS)]):
                        lin.forward_host(host_x[m], host_ys[(m, i)])
                    n_call += 1
            for st_ in E2E_STREAMS:
                side.wait_stream(st_)
    torch.cuda.synchronize()

    def step_e2e_graph():
        e2e_graph.replay()
        torch.cuda.current_stream().synchronize()  # the step's results are on the host

    for _ in range(2):
        step_e2e_graph()
    # the replayed step must deliver what the plain calls deliver
    chk = {key: t.clone() for key, t in list(host_ys.items())[:3]}
    for t in host_ys.values():
        t.zero_()
    step_e2e_graph()
    e2e_graph_ok = all(torch.equal(host_ys[key], ref_y) for key, ref_y in chk.items())
    ms_e2e = timed(step_e2e_graph, e2e_steps) if e2e_graph_ok else ms_e2e_eager
    del e2e_graph
    del graph
    lins_keep = lins[:1]
    del lins
    torch.cuda.empty_cache()

    flush = L2Flush(dev)
    f32_linear = measure_f32_linear(dev, flush, xn, torch) if not args.no_extras else None
    fp8_prefill = measure_fp8_prefill(dev, flush, xn, torch) if not args.no_extras else None
    q4_prefill = measure_q4_prefill(dev, flush, xn, torch) if not args.no_extras else None
    del flush
    torch.cuda.empty_cache()
    prefill_cp = None
    if world > 1 and not args.no_extras:
        try:
            prefill_cp = measure_prefill_column_parallel(dev, world, rank, xn, torch, dist)
        except Exception as e:  # noqa: BLE001  (symmetric memory unavailable, ...): report, keep the line
            prefill_cp = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()

    prefill_stack = None
    if not args.no_extras and not args.no_decode:
        try:
            prefill_stack = measure_prefill_stack(args, dev, world, rank, timed, torch, dist)
        except Exception as e:  # noqa: BLE001
            prefill_stack = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()

    decode = None
    if not args.no_decode:
        del lins_keep
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
        cpu_baseline, f32_cpu = None, None
        if world == 1:  # the CPU legs run at N = 1 only
            port = CpuPort()
            cpu_gbs, passes, cpu_dt = port.throughput(args.cpu_seconds)
            cpu_baseline = {"value": cpu_gbs, "unit": UNIT, "cores": port.threads, "kind": "port",
                            "sample": f"{passes} pass(es) of M in {{1,4,16}} over one weight copy, {cpu_dt:.1f} s; {port.kind}"}
            f32_cpu = port.f32_linear()
        if f32_linear is not None:
            f32_linear["cpu_baseline"] = f32_cpu
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8xint4->int32", "data": "synthetic",
            "config": make_config(world),
            "run": {"replicas": R, "sweeps_per_step": SWEEPS, "launch": f"{REPLAYS} replay(s) of one CUDA graph of {GS} sweeps per step",
                    "weight_copies_mb_per_m": R * wb / 1e6},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": R * sum(m * K_IN * 4 for m in MS),
                    "d2h_bytes_per_step": R * sum(m * N_OUT * 4 for m in MS), "steps": e2e_steps,
                    "ms_per_step": ms_e2e / e2e_steps, "calls_per_step": len(MS) * R,
                    "api": ("LinearQ4.forward_host -> xn_mm_linear_q4_host (copy in, quantize rows, linear, copy out), "
                            "the three batch sizes interleaved and the calls spread round-robin over 8 streams; the step's "
                            "calls are captured once in a CUDA graph (copies included) and replayed per step") if e2e_graph_ok else
                           "LinearQ4.forward_host -> xn_mm_linear_q4_host, plain calls over 8 streams (graph replay differed)",
                    "plain_calls_value": world * e2e_steps * len(MS) * R * wb / (ms_e2e_eager * 1e-3) / 1e9},
            "gpu_launches": args.steps * launches_per_step,
            "fp8_prefill_gemm": fp8_prefill,
            "int4_prefill_gemm": q4_prefill,
            "f32_linear": f32_linear,
            "prefill_column_parallel": prefill_cp,
            "prefill_stack": prefill_stack,
            "decode_step": decode,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}",
                         "traffic": (2 * NCU_DRAM_BYTES_PER_LAUNCH["M<=8"] + NCU_DRAM_BYTES_PER_LAUNCH["M=9..16"]) / 3,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, recorded per "
                                           "instantiation (M <= 8: 28874304 B, M = 16: 28927232 B) and weighted by the sweep's "
                                           "launch mix (2 : 1); capture summarised in profiles/linear_q4_kernel_int4_decode_gemv.md",
                         "kernel": "linear_q4_kernel",
                         "algorithmic_bytes_per_launch": alg, "us_per_launch": launch_s * 1e6,
                         "per_m": {str(m): {"us_per_launch": per_m[m] * 1e6, "algorithmic_bytes": algorithmic_bytes(m),
                                            "achieved": algorithmic_bytes(m) / per_m[m] / 1e9,
                                            "frac": algorithmic_bytes(m) / per_m[m] / 1e9 / peak} for m in MS}},
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
