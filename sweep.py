"""Shape sweeps behind the benchmark tables: fp8 transformer linears, grouped per-codebook matmul,
the f32 linear, and the 16-bit dense GEMM, each with its roofline and (where the reference has a
GPU path) the same call through cuBLAS as xn issues it (torch.matmul -> cublasGemmEx, f32 accumulate).

    python sweep.py [--what fp8|dense|grouped|f32|conv|all] [--json out.json] [--md out.md]

Timing: CUDA events around a CUDA-graph replay of `reps` launches that rotate over enough distinct
weight copies to exceed the L2 several times for the bandwidth-bound points.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import xn_b200 as xn  # noqa: E402

NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0, "fp8_tflops": 4500.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


def time_graph(fns, reps_per_fn=1, iters=5):
    """fns: list of callables (one per operand replica). Returns seconds per call."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(reps_per_fn):
                for f in fns:
                    f()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    # let the part settle after the previous point: a bandwidth-bound point timed right behind a
    # power-capped GEMM reads 15-20 % slow (for this library and for cuBLAS alike)
    time.sleep(0.4)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (iters * reps_per_fn * len(fns))


def replicas_for(nbytes, target=600e6, lo=1, hi=32):
    return int(max(lo, min(hi, -(-target // nbytes))))


def sweep_fp8(out, dev, pk):
    shapes = [(12288, 4096, "qkv"), (4096, 4096, "out_proj"), (22528, 4096, "ffn_up"), (4096, 11264, "ffn_down")]
    for n, k, name in shapes:
        R = replicas_for(n * k)
        ws = []
        for _ in range(R):
            w = torch.randn(n, k, device=dev) * 0.02
            ws.append(xn.quantize_weights_fp8(w))
            del w
        wb = [(q.view(torch.float8_e4m3fn)) for q, _ in ws]
        for m in (1, 16, 64, 256, 1024, 4096):
            x = torch.randn(m, k, device=dev).bfloat16()
            y = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            wsp = torch.empty(xn.lib().xn_mm_linear_fp8_workspace_bytes(m, k), dtype=torch.uint8, device=dev)
            flops = 2.0 * m * n * k
            byts = n * k + 4 * n + 2 * m * k + 2 * m * n
            reps = 1 if m >= 1024 else 2
            row = {"config": "fp8_linear", "name": name, "m": m, "n": n, "k": k, "replicas": R}
            for variant, tag in ((0, "w8a16"), (1, "w8a8")):
                t_full = time_graph([lambda q=q, s=s: xn.linear_fp8(x, q, s, variant, workspace=wsp, out=y) for q, s in ws], reps)
                hi, lo, xs = xn.split_rows_e4m3(x, want_lo=(variant == 0))
                from xn_b200._lib import check
                L = xn.lib()
                st = lambda: torch.cuda.current_stream().cuda_stream
                t_mm = time_graph([lambda q=q, s=s: check(L.xn_mm_linear_fp8_pieces(
                    y.data_ptr(), hi.data_ptr(), lo.data_ptr() if lo is not None else None, xs.data_ptr(), q.data_ptr(),
                    s.data_ptr(), m, n, k, st())) for q, s in ws], reps)
                peak_t = (pk["bf16_tflops"] if variant == 0 else 2 * pk["bf16_tflops"]) * 1e12
                roof = max(byts / (pk["hbm_gbs"] * 1e9), flops / peak_t)
                row[tag] = {"us_full": t_full * 1e6, "us_matmul": t_mm * 1e6, "tflops": flops / t_mm / 1e12,
                            "gbs": byts / t_mm / 1e9, "roofline_us": roof * 1e6, "frac_of_roofline": roof / t_mm}
            # the reference's GPU path for a bf16 weight of the same shape: cuBLAS bf16 GEMM, f32 accumulate
            wbf = [torch.randn(n, k, device=dev).bfloat16() for _ in range(min(R, max(1, R // 2)))]
            t_cublas = time_graph([lambda w=w: torch.matmul(x, w.t(), out=y) for w in wbf], reps)
            row["cublas_bf16_us"] = t_cublas * 1e6
            del wbf
            out.append(row)
            print(json.dumps(row), flush=True)
        del ws, wb
        torch.cuda.empty_cache()


def sweep_dense(out, dev, pk):
    for dt in (torch.bfloat16, torch.float16):
        shapes = [(4096, 4096, 4096), (8192, 8192, 8192), (1024, 12288, 4096), (256, 12288, 4096), (64, 12288, 4096)]
        if dt == torch.bfloat16:  # the reference's decode path: unquantized bf16 weights, decode-sized m
            shapes += [(m, n, k) for (n, k) in ((12288, 4096), (4096, 4096), (22528, 4096), (4096, 11264)) for m in (1, 16, 32)]
            # a hundred-odd rows against the narrow weights: too few 128 x 256 tiles for the machine (split along k)
            shapes += [(128, 4096, 4096), (256, 4096, 4096), (256, 4096, 11264)]
        for m, n, k in shapes:
            R = replicas_for(2 * n * k, hi=8)
            ws = [(torch.randn(n, k, device=dev) * 0.05).to(dt) for _ in range(R)]
            x = torch.randn(m, k, device=dev).to(dt)
            y = torch.empty(m, n, device=dev, dtype=dt)
            flops = 2.0 * m * n * k
            byts = 2 * (n * k + m * k + m * n)
            t = time_graph([lambda w=w: xn.matmul_(y, x, w, True) for w in ws], 1)
            t_ref = time_graph([lambda w=w: torch.matmul(x, w.t(), out=y) for w in ws], 1)
            roof = max(byts / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))
            row = {"config": "dense_16bit", "dtype": str(dt), "m": m, "n": n, "k": k, "us": t * 1e6,
                   "tflops": flops / t / 1e12, "cublas_us": t_ref * 1e6, "cublas_tflops": flops / t_ref / 1e12,
                   "frac_of_roofline": roof / t}
            out.append(row)
            print(json.dumps(row), flush=True)
            del ws
        # `a.matmul(&b)` with a row-major (k, n) right-hand side: the reference's own CUDA matmul benchmark
        # (xn-core/examples/basic_cuda.rs:35-56, (32, 1, 2048) x (2048, 11264)) and square prefill-sized products
        for m, n, k in ((32, 11264, 2048), (4096, 4096, 4096), (256, 12288, 4096)):
            R = replicas_for(2 * n * k, hi=8)
            ws = [(torch.randn(k, n, device=dev) * 0.05).to(dt) for _ in range(R)]
            x = torch.randn(m, k, device=dev).to(dt)
            y = torch.empty(m, n, device=dev, dtype=dt)
            flops = 2.0 * m * n * k
            byts = 2 * (n * k + m * k + m * n)
            t = time_graph([lambda w=w: xn.matmul_(y, x, w, False) for w in ws], 1)
            t_ref = time_graph([lambda w=w: torch.matmul(x, w, out=y) for w in ws], 1)
            roof = max(byts / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))
            row = {"config": "dense_16bit_kn_rhs", "dtype": str(dt), "m": m, "n": n, "k": k, "us": t * 1e6,
                   "tflops": flops / t / 1e12, "cublas_us": t_ref * 1e6, "cublas_tflops": flops / t_ref / 1e12,
                   "frac_of_roofline": roof / t}
            out.append(row)
            print(json.dumps(row), flush=True)
            del ws


def sweep_grouped(out, dev, pk):
    G, B = 16, 64
    for n, k, name in ((1024, 1024, "stage1"), (4096, 1024, "ffn_up"), (1024, 2048, "ffn_down")):
        R = replicas_for(2 * G * n * k, hi=16)
        ws = [(torch.randn(G, n, k, device=dev) * 0.03).bfloat16() for _ in range(R)]
        x = torch.randn(B, G, k, device=dev).bfloat16()
        xt = x.transpose(0, 1)
        y = torch.empty(G, B, n, device=dev, dtype=torch.bfloat16)
        t = time_graph([lambda w=w: xn.matmul_(y, xt, w, True) for w in ws], 2)
        t_ref = time_graph([lambda w=w: torch.bmm(xt, w.transpose(1, 2), out=y) for w in ws], 2)
        byts = 2 * (G * n * k + B * G * k + B * G * n)
        row = {"config": "grouped_codebooks", "name": name, "groups": G, "b": B, "n": n, "k": k, "us": t * 1e6,
               "gbs": byts / t / 1e9, "frac_of_hbm": byts / t / 1e9 / pk["hbm_gbs"], "cublas_us": t_ref * 1e6}
        out.append(row)
        print(json.dumps(row), flush=True)
        del ws


def sweep_f32(out, dev, pk):
    m, n, k = 16, 11264, 4096
    R = 4
    ws = [torch.randn(n, k, device=dev) * 0.02 for _ in range(R)]
    x = torch.randn(m, k, device=dev)
    y = torch.empty(m, n, device=dev)
    t = time_graph([lambda w=w: xn.matmul_(y, x, w, True) for w in ws], 2)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False  # the reference keeps full-precision f32 by default
    t_ref = time_graph([lambda w=w: torch.matmul(x, w.t(), out=y) for w in ws], 2)
    torch.backends.cuda.matmul.allow_tf32 = prev
    byts = 4 * (n * k + m * k + m * n)
    row = {"config": "f32_linear", "m": m, "n": n, "k": k, "us": t * 1e6, "gbs": byts / t / 1e9,
           "frac_of_hbm": byts / t / 1e9 / pk["hbm_gbs"], "cublas_us": t_ref * 1e6}
    out.append(row)
    print(json.dumps(row), flush=True)
    # many rows: three tf32 pieces per operand on the tensor-memory kernel, repack passes included
    torch.backends.cuda.matmul.allow_tf32 = False
    for m, n, k in ((32, 11264, 4096), (64, 11264, 4096), (125, 1024, 4096), (128, 11264, 4096), (1024, 4096, 4096),
                    (4096, 4096, 4096), (4096, 11264, 4096)):
        x = torch.randn(m, k, device=dev)
        w = torch.randn(n, k, device=dev) * 0.02
        y = torch.empty(m, n, device=dev)
        t = time_graph([lambda: xn.matmul_(y, x, w, True)], 2)
        t_ref = time_graph([lambda: torch.matmul(x, w.t(), out=y)], 2)
        row = {"config": "f32_gemm", "m": m, "n": n, "k": k, "us": t * 1e6, "tflops": 2.0 * m * n * k / t / 1e12,
               "cublas_us": t_ref * 1e6, "cublas_tflops": 2.0 * m * n * k / t_ref / 1e12}
        out.append(row)
        print(json.dumps(row), flush=True)
    torch.backends.cuda.matmul.allow_tf32 = prev


def sweep_conv(out, dev, pk):
    """conv1d / conv_transpose1d at codec-encoder sizes.  Beside each point: the reference's own GPU lowering
    built from the same library calls (im2col -> cuBLAS GEMM -> transpose, xn-core/src/cuda_backend.rs:1490-1561;
    transpose -> cuBLAS GEMM -> col2im, :1783-1856) and cuDNN through torch."""
    import torch.nn.functional as F
    prev = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = False  # the reference keeps full-precision f32
    torch.backends.cudnn.allow_tf32 = False
    # batch, c_in, c_out, length, kernel, stride, padding
    conv = [(8, 512, 512, 4096, 7, 1, 3), (8, 512, 1024, 4096, 16, 8, 4), (8, 64, 64, 32768, 7, 1, 3), (32, 512, 512, 256, 3, 1, 1),
            (1, 512, 512, 64, 7, 1, 3)]
    convt = [(8, 512, 256, 512, 16, 8), (8, 1024, 512, 256, 8, 4), (1, 512, 256, 16, 16, 8)]
    for dt in (torch.bfloat16, torch.float32):
        es = 2 if dt == torch.bfloat16 else 4
        peak = pk["bf16_tflops"] if es == 2 else None
        for b, ci, co, length, ks, st, pad in conv:
            x = torch.randn(b, ci, length, device=dev, dtype=dt)
            w = (torch.randn(co, ci, ks, device=dev) / (ci * ks) ** 0.5).to(dt)
            bias = torch.randn(co, device=dev, dtype=dt)
            lo = (length + 2 * pad - (ks - 1) - 1) // st + 1
            t = time_graph([lambda: xn.ops.conv1d(x, w, bias, st, pad, 1, 1)], 4)

            def lowered():
                col = F.unfold(F.pad(x, (pad, pad)).unsqueeze(2), (1, ks), stride=(1, st)).transpose(1, 2).contiguous()
                return (torch.matmul(col, w.reshape(co, -1).t()).transpose(1, 2).contiguous() + bias.view(1, -1, 1))
            t_low = time_graph([lowered], 2)
            t_dnn = time_graph([lambda: F.conv1d(x, w, bias, st, pad)], 4)
            flops = 2.0 * b * co * ci * ks * lo
            byts = es * (b * ci * length + co * ci * ks + b * co * lo)
            roof = max(byts / (pk["hbm_gbs"] * 1e9), flops / (peak * 1e12) if peak else 0.0)
            row = {"config": "conv1d", "dtype": str(dt), "b": b, "c_in": ci, "c_out": co, "length": length, "k": ks, "stride": st,
                   "us": t * 1e6, "tflops": flops / t / 1e12, "gbs": byts / t / 1e9, "frac_of_roofline": roof / t,
                   "lowered_us": t_low * 1e6, "cudnn_us": t_dnn * 1e6}
            out.append(row)
            print(json.dumps(row), flush=True)
        for b, ci, co, length, ks, st in convt:
            x = torch.randn(b, ci, length, device=dev, dtype=dt)
            w = (torch.randn(ci, co, ks, device=dev) / ci ** 0.5).to(dt)
            bias = torch.randn(co, device=dev, dtype=dt)
            lo = (length - 1) * st + ks
            t = time_graph([lambda: xn.ops.conv_transpose1d(x, w, bias, st, 0, 0, 1)], 4)

            def lowered_t():
                col = torch.matmul(x.transpose(1, 2).contiguous(), w.reshape(ci, co * ks))          # [b, l, co*ks]
                return F.fold(col.transpose(1, 2), (1, lo), (1, ks), stride=(1, st)).squeeze(2) + bias.view(1, -1, 1)
            t_low = time_graph([lowered_t], 2)
            t_dnn = time_graph([lambda: F.conv_transpose1d(x, w, bias, st)], 4)
            flops = 2.0 * b * co * ci * ks * length
            byts = es * (b * ci * length + co * ci * ks + b * co * lo)
            roof = max(byts / (pk["hbm_gbs"] * 1e9), flops / (peak * 1e12) if peak else 0.0)
            row = {"config": "conv_transpose1d", "dtype": str(dt), "b": b, "c_in": ci, "c_out": co, "length": length, "k": ks,
                   "stride": st, "us": t * 1e6, "tflops": flops / t / 1e12, "gbs": byts / t / 1e9, "frac_of_roofline": roof / t,
                   "lowered_us": t_low * 1e6, "cudnn_us": t_dnn * 1e6}
            out.append(row)
            print(json.dumps(row), flush=True)
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = prev


def write_md(rows, path, what="all"):
    """The sweep as markdown tables (the form kept under profiles/)."""
    pk = rows[0]["peaks"]
    tag = "sweep_" + what
    L = ["# Shape sweeps (CUDA-event timing, graph replay, operands rotated over >= 600 MB of distinct weight copies)", "",
         "Command: `python sweep.py --what %s --json %s.json --md %s.md` on one B200"
         " (committed files only)." % (what, tag, tag),
         "Roofline per point = max(algorithmic bytes / measured HBM GB/s, 2MNK / peak), peak = %s cuBLAS bf16 burst" % pk["kind"],
         "(%.0f TFLOP/s) for the W8A16 and 16-bit rows and twice that for W8A8; HBM = %.0f GB/s; `frac` = roofline time / measured time."
         % (pk["bf16_tflops"], pk["hbm_gbs"]),
         "`cuBLAS bf16` = the reference's GPU path for an unquantized weight of the same shape (torch.matmul -> cublasGemmEx,"
         " f32 accumulate).", ""]
    fp8 = [r for r in rows if r.get("config") == "fp8_linear"]
    if fp8:
        L += ["## fp8-e4m3 transformer linears (bf16 activations in, bf16 out; matmul only, activation split listed separately)", "",
              "| shape (N,K) | M | W8A16 µs | TFLOP/s | GB/s | frac | W8A8 µs | TFLOP/s | frac | split µs | cuBLAS bf16 µs |",
              "|---|---|---|---|---|---|---|---|---|---|---|"]
        for r in fp8:
            a16, a8 = r["w8a16"], r["w8a8"]
            L.append("| %s (%d,%d) | %d | %.1f | %.1f | %.0f | %.2f | %.1f | %.1f | %.2f | %.1f | %.1f |" % (
                r["name"], r["n"], r["k"], r["m"], a16["us_matmul"], a16["tflops"], a16["gbs"], a16["frac_of_roofline"],
                a8["us_matmul"], a8["tflops"], a8["frac_of_roofline"], max(0.0, a16["us_full"] - a16["us_matmul"]),
                r["cublas_bf16_us"]))
        L.append("")
    dense = [r for r in rows if r.get("config") == "dense_16bit"]
    if dense:
        L += ["## 16-bit dense matmul_t (tcgen05 tiled kernel; skinny tcgen05 form for 17-64 rows; mma.sync GEMV up to 16 rows)", "",
              "| dtype | M x N x K | µs | TFLOP/s | cuBLAS µs | cuBLAS TFLOP/s | frac |", "|---|---|---|---|---|---|---|"]
        for r in dense:
            L.append("| %s | %dx%dx%d | %.1f | %.0f | %.1f | %.0f | %.2f |" % (
                r["dtype"].replace("torch.", ""), r["m"], r["n"], r["k"], r["us"], r["tflops"], r["cublas_us"],
                r["cublas_tflops"], r["frac_of_roofline"]))
        L.append("")
    kn = [r for r in rows if r.get("config") == "dense_16bit_kn_rhs"]
    if kn:
        L += ["## 16-bit matmul with a row-major (k, n) right-hand side (tcgen05 tiled kernel, B read as an MN-major operand;"
              " first row = xn-core/examples/basic_cuda.rs)", "",
              "| dtype | M x N x K | µs | TFLOP/s | cuBLAS µs | cuBLAS TFLOP/s | frac |", "|---|---|---|---|---|---|---|"]
        for r in kn:
            L.append("| %s | %dx%dx%d | %.1f | %.0f | %.1f | %.0f | %.2f |" % (
                r["dtype"].replace("torch.", ""), r["m"], r["n"], r["k"], r["us"], r["tflops"], r["cublas_us"],
                r["cublas_tflops"], r["frac_of_roofline"]))
        L.append("")
    grp = [r for r in rows if r.get("config") == "grouped_codebooks"]
    if grp:
        L += ["## Grouped per-codebook matmul (%d groups, x [%d,%d,K] viewed [%d,%d,K], W [%d,N,K] bf16, one launch)" % (
                  grp[0]["groups"], grp[0]["b"], grp[0]["groups"], grp[0]["groups"], grp[0]["b"], grp[0]["groups"]), "",
              "| stage | N | K | µs | GB/s | frac of HBM | cuBLAS bmm µs |", "|---|---|---|---|---|---|---|"]
        for r in grp:
            L.append("| %s | %d | %d | %.1f | %.0f | %.2f | %.1f |" % (r["name"], r["n"], r["k"], r["us"], r["gbs"],
                                                                     r["frac_of_hbm"], r["cublas_us"]))
        L.append("")
    for r in rows:
        if r.get("config") == "f32_linear":
            L += ["## f32 linear (x [%d,%d], W [%d,%d]; 3xTF32 tensor-core form unless XN_MM_F32_EXACT=1)" % (r["m"], r["k"], r["n"], r["k"]), "",
                  "%.1f µs, %.0f GB/s (%.2f of %s HBM); cuBLAS SGEMM without TF32 (the reference's default): %.1f µs."
                  % (r["us"], r["gbs"], r["frac_of_hbm"], pk["kind"], r["cublas_us"]), ""]
    fg = [r for r in rows if r.get("config") == "f32_gemm"]
    if fg:
        L += ["## f32 matmul_t beyond 16 rows (up to 64 rows: 3xTF32 weight-streaming kernel in passes of 16 rows; beyond: three tf32"
              " pieces per operand on kind::tf32, repack passes included, accumulator handed to f32 registers every 8 MMAs with a second-level total in tensor memory,"
              " split-k for few tiles; 125x1024x4096 is the shape of the reference's CPU benchmark)", "",
              "| M x N x K | µs | TFLOP/s | cuBLAS SGEMM (no TF32) µs | TFLOP/s |", "|---|---|---|---|---|"]
        for r in fg:
            L.append("| %dx%dx%d | %.1f | %.1f | %.1f | %.1f |" % (r["m"], r["n"], r["k"], r["us"], r["tflops"], r["cublas_us"],
                                                                 r["cublas_tflops"]))
        L.append("")
    cv = [r for r in rows if r.get("config") in ("conv1d", "conv_transpose1d")]
    if cv:
        L += ["## conv1d / conv_transpose1d (bias fused; tensor-memory GEMM over a channels-last view: bf16 on kind::f16, f32 as three tf32 pieces on kind::tf32)", "",
              "`lowered` = the reference's GPU lowering from the same library calls (im2col / col2im around a cuBLAS GEMM, f32 without TF32);"
              " `cuDNN` = torch's conv (TF32 off). frac: bf16 rows against max(HBM, tensor) roofline, f32 rows against HBM alone"
              " (no measured f32-exact tensor peak exists; 3 tf32 MMAs per product).", "",
              "| op | dtype | batch | C_in→C_out | length | kernel/stride | µs | TFLOP/s | frac | lowered µs | cuDNN µs |",
              "|---|---|---|---|---|---|---|---|---|---|---|"]
        for r in cv:
            L.append("| %s | %s | %d | %d→%d | %d | %d/%d | %.1f | %.1f | %.2f | %.1f | %.1f |" % (
                r["config"], r["dtype"].replace("torch.", ""), r["b"], r["c_in"], r["c_out"], r["length"], r["k"], r["stride"],
                r["us"], r["tflops"], r["frac_of_roofline"], r["lowered_us"], r["cudnn_us"]))
        L.append("")
    with open(path, "w") as f:
        f.write("\n".join(L))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="all")
    ap.add_argument("--json", default=None)
    ap.add_argument("--md", default=None, help="also write the tables as markdown")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    pk = peaks()
    out = [{"peaks": pk, "nominal": NOMINAL}]
    print(json.dumps(out[0]), flush=True)
    for name, fn in (("fp8", sweep_fp8), ("dense", sweep_dense), ("grouped", sweep_grouped), ("f32", sweep_f32), ("conv", sweep_conv)):
        if a.what in ("all", name):
            fn(out, dev, pk)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f, indent=1)
    if a.md:
        write_md(out, a.md, a.what)


if __name__ == "__main__":
    main()
