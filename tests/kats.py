"""The reference's known-answer tests, expressed as Backend::gemm calls on a pluggable backend.

A backend is an object with
    plan(lhs_dims, lhs_strides, rhs_dims, rhs_strides, rhs_t, dst_capacity) -> 12 gemm args (list)
    gemm(dtype_code, dst_len, lhs_flat, lhs_off, rhs_flat, rhs_off, *12 args) -> flat np.ndarray
with 16-bit data carried as uint16 bit patterns.  `OracleBackend` runs the CPU oracle;
tests/test_gemm_gpu.py supplies the one that goes through the C ABI on the GPU.
"""
from __future__ import annotations

import json
import os

import numpy as np

import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kats.json")
DT = {"f32": O.F32, "f16": O.F16, "bf16": O.BF16}


def load():
    with open(GOLDEN) as f:
        return json.load(f)


class OracleBackend:
    def plan(self, ld, ls, rd, rs, rhs_t, dst_capacity):
        code, a = O.matmul_plan(ld, ls, rd, rs, rhs_t)
        assert code == 0, code
        assert a["lhs_b"] * a["m"] * a["n"] <= dst_capacity
        return list(a.values())

    def gemm(self, dt, dst_len, lhs, lhs_off, rhs, rhs_off, *a):
        m, n, k, lb, lbs, rbs, dcs, drs, lcs, lrs, rcs, rrs = a
        return O.gemm(dt, dst_len, lhs, lhs_off, rhs, rhs_off, m, n, k, lb, lbs, rbs, (dcs, drs), (lcs, lrs), (rcs, rrs))


def view_matmul(be, dt, lhs, ld, ls, loff, rhs, rd, rs, roff, rhs_t):
    """ops::matmul_with_t on flat storages + view geometry; returns (dims, f32 values)."""
    n = rd[-2] if rhs_t else rd[-1]
    out_dims = list(ld[:-2]) + [ld[-2], n]
    dst_len = int(np.prod(out_dims))
    a = be.plan(ld, ls, rd, rs, rhs_t, dst_len)
    flat = be.gemm(dt, dst_len, O.from_f32(dt, lhs), loff, O.from_f32(dt, rhs), roff, *a)
    return out_dims, O.to_f32(dt, flat)


def run_matmul_case(be, case):
    dt = DT[case["dtype"]]
    ld, rd = case["lhs_dims"], case["rhs_dims"]
    dims, got = view_matmul(be, dt, np.array(case["lhs"], np.float32), ld, O.contiguous_strides(ld), 0,
                            np.array(case["rhs"], np.float32), rd, O.contiguous_strides(rd), 0, case["rhs_t"])
    assert dims == case["expected_dims"]
    exp = np.array(case["expected"], np.float32)
    if case["tol"] == 0.0:
        assert np.array_equal(got, exp), (case["name"], got, exp)
    else:
        assert np.all(np.abs(got - exp) < case["tol"]), (case["name"], got, exp)


def run_transposed_view(be, spec):
    dims = spec["dims"]
    q = np.arange(24, dtype=np.float32)
    k = (np.arange(24, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    st = O.contiguous_strides(dims)
    # k.transpose(2,3): dims and strides of the last two axes swapped, same storage
    kt_dims = dims[:2] + [dims[3], dims[2]]
    kt_strides = st[:2] + [st[3], st[2]]
    d1, v1 = view_matmul(be, O.F32, q, dims, st, 0, k, kt_dims, kt_strides, 0, False)
    d2, v2 = view_matmul(be, O.F32, q, dims, st, 0, k, dims, st, 0, True)
    assert d1 == d2 == [1, 2, 3, 3]
    assert np.all(np.abs(v1 - v2) < spec["tol"])
    # and against plain numpy in float64
    ref = np.einsum("bhik,bhjk->bhij", q.reshape(dims).astype(np.float64), k.reshape(dims).astype(np.float64))
    assert np.allclose(v1.reshape(ref.shape), ref, rtol=1e-5, atol=1e-4)


def _im2col1d(src, b, c, length, l_out, ks, stride, padding, dilation=1):
    col = np.zeros((b, l_out, c * ks), np.float32)
    x = src.reshape(b, c, length)
    for li in range(l_out):
        for ci in range(c):
            for kk in range(ks):
                sl = li * stride + kk * dilation
                if padding <= sl < length + padding:
                    col[:, li, ci * ks + kk] = x[:, ci, sl - padding]
    return col.reshape(-1)


def _expect(case, out):
    """Exact unless the case carries a tolerance (the reference's f16 cases assert |r - e| < 0.1)."""
    exp = np.array(case["expected"], np.float32)
    if case.get("tol"):
        assert np.all(np.abs(out.reshape(-1) - exp) < case["tol"]), (case["name"], out)
    else:
        assert np.array_equal(out.reshape(-1), exp), (case["name"], out)


def run_conv1d_case(be, case):
    b, c_in, length = case["input_dims"]
    c_out, _, ks = case["kernel_dims"]
    stride, padding = case["stride"], case["padding"]
    l_out = (length + 2 * padding - (ks - 1) - 1) // stride + 1
    k = c_in * ks
    dt = DT[case.get("dtype", "f32")]
    col = _im2col1d(np.array(case["input"], np.float32), b, c_in, length, l_out, ks, stride, padding)
    kernel = np.array(case["kernel"], np.float32)
    # xn-core/src/cpu_backend.rs:1001-1014
    res = be.gemm(dt, b * l_out * c_out, O.from_f32(dt, col), 0, O.from_f32(dt, kernel), 0, l_out, c_out, k, b, l_out * k, 0, 1,
                  c_out, 1, k, k, 1)
    out = O.to_f32(dt, res).reshape(b, l_out, c_out).transpose(0, 2, 1).copy()
    if case["bias"] is not None:
        out += np.array(case["bias"], np.float32).reshape(1, c_out, 1)
    assert list(out.shape) == case["expected_dims"]
    _expect(case, out)


def run_conv_transpose1d_case(be, case):
    b, c_in, length = case["input_dims"]
    _, c_out, ks = case["kernel_dims"]
    stride = case["stride"]
    l_out = (length - 1) * stride + ks
    dt = DT[case.get("dtype", "f32")]
    src_t = np.array(case["input"], np.float32).reshape(b, c_in, length).transpose(0, 2, 1).copy().reshape(-1)
    kernel = np.array(case["kernel"], np.float32)
    n = c_out * ks
    # xn-core/src/cpu_backend.rs:1097-1110
    col = be.gemm(dt, b * length * n, O.from_f32(dt, src_t), 0, O.from_f32(dt, kernel), 0, length, n, c_in, b, length * c_in, 0,
                  1, n, 1, c_in, 1, n)
    col = O.to_f32(dt, col).reshape(b, length, c_out, ks)
    out = np.zeros((b, c_out, l_out), np.float32)
    for li in range(length):
        for kk in range(ks):
            out[:, :, li * stride + kk] += col[:, li, :, kk]
    if case["bias"] is not None:
        out += np.array(case["bias"], np.float32).reshape(1, c_out, 1)
    assert list(out.shape) == case["expected_dims"]
    _expect(case, out)


def conv1d_f64(x, w, stride, padding, dilation, groups):
    """The definition of conv1d evaluated in float64 (independent of the oracle's lowering)."""
    b, cin, length = x.shape
    cout, cig, ks = w.shape
    lo = (length + 2 * padding - dilation * (ks - 1) - 1) // stride + 1
    xp = np.zeros((b, cin, length + 2 * padding + stride))
    xp[:, :, padding:padding + length] = x
    out = np.zeros((b, cout, lo))
    cog = cout // groups
    for g in range(groups):
        for kk in range(ks):
            sl = xp[:, g * cig:(g + 1) * cig, kk * dilation: kk * dilation + (lo - 1) * stride + 1: stride]
            out[:, g * cog:(g + 1) * cog] += np.einsum("bcl,oc->bol", sl, w[g * cog:(g + 1) * cog, :, kk].astype(np.float64))
    return out


def conv_transpose1d_f64(x, w, stride, padding, output_padding, groups):
    b, cin, length = x.shape
    _, cog, ks = w.shape
    cig = cin // groups
    full = np.zeros((b, cog * groups, (length - 1) * stride + ks + output_padding + padding))
    for g in range(groups):
        for kk in range(ks):
            full[:, g * cog:(g + 1) * cog, kk: kk + (length - 1) * stride + 1: stride] += np.einsum(
                "bcl,co->bol", x[:, g * cig:(g + 1) * cig].astype(np.float64), w[g * cig:(g + 1) * cig, :, kk].astype(np.float64))
    lo = (length - 1) * stride + ks + output_padding - 2 * padding
    return full[:, :, padding:padding + lo]


def run_all(be):
    g = load()
    for c in g["matmul"]:
        run_matmul_case(be, c)
    run_transposed_view(be, g["transposed_view"])
    for c in g["conv1d"]:
        run_conv1d_case(be, c)
    for c in g["conv_transpose1d"]:
        run_conv_transpose1d_case(be, c)
    return len(g["matmul"]) + 1 + len(g["conv1d"]) + len(g["conv_transpose1d"])


# The Backend::gemm argument tuples real call sites produce (sizes scaled down), used by both the
# oracle self-checks and the GPU parity tests.  Each entry: name, lhs dims/strides/offset,
# rhs dims/strides/offset, rhs_t.  Storage sizes are derived from the views.
def view_cases():
    cs = O.contiguous_strides
    cases = []
    # Linear::forward on [B,T,K] x W[N,K]: flattens to one GEMM (nn/linear.rs:60)
    cases.append(("linear_3d_flatten", [3, 5, 40], cs([3, 5, 40]), 0, [24, 40], cs([24, 40]), 0, True))
    # plain matmul with [K,N] rhs (cuda_tests.rs:223, basic_cuda.rs:46-56)
    cases.append(("matmul_kn", [7, 33], cs([7, 33]), 0, [33, 19], cs([33, 19]), 0, False))
    # attention q @ k^T: q [B,H,T,hd], k [B,H,ctx,hd] (batched_transformer.rs:175)
    cases.append(("attn_qk", [2, 3, 1, 16], cs([2, 3, 1, 16]), 0, [2, 3, 37, 16], cs([2, 3, 37, 16]), 0, True))
    # attention p @ v (batched_transformer.rs:190)
    cases.append(("attn_pv", [2, 3, 1, 37], cs([2, 3, 1, 37]), 0, [2, 3, 37, 16], cs([2, 3, 37, 16]), 0, False))
    # llama: q @ k.transpose(2,3) with a transposed VIEW as rhs (models/llama.rs:193-194)
    kd = [2, 2, 9, 8]
    ks_ = cs(kd)
    cases.append(("llama_qkT_view", [2, 2, 4, 8], cs([2, 2, 4, 8]), 0, [2, 2, 8, 9], [ks_[0], ks_[1], ks_[3], ks_[2]], 0, False))
    # pocket-tts: storage [b=1,t,h,d], views transpose(1,2) on both sides (xn-pocket-tts/src/transformer.rs:126-132)
    t, h, d = 6, 4, 8
    st = cs([1, t, h, d])
    vd, vs = [1, h, t, d], [st[0], st[2], st[1], st[3]]
    cases.append(("pocket_tts_noncontig_rows", vd, vs, 0, vd, vs, 0, True))
    # grouped per-codebook: x [B,G,K] viewed as [G,B,K], W [G,N,K] (one call, G groups)
    B, G, K, N = 5, 4, 24, 12
    xs = cs([B, G, K])
    cases.append(("grouped_codebooks", [G, B, K], [xs[1], xs[0], xs[2]], 0, [G, N, K], cs([G, N, K]), 0, True))
    # narrow()-ed views: non-zero storage offsets on both sides (tensor_view.rs:243)
    cases.append(("narrow_offsets", [4, 10], [30, 1], 7, [6, 10], [16, 1], 5, True))
    # degenerate sizes
    cases.append(("m1", [1, 17], cs([1, 17]), 0, [17, 9], cs([17, 9]), 0, False))
    cases.append(("n1", [5, 17], cs([5, 17]), 0, [1, 17], cs([1, 17]), 0, True))
    cases.append(("k1", [5, 1], cs([5, 1]), 0, [1, 9], cs([1, 9]), 0, False))
    # a stride pattern cuBLAS cannot express (both rhs strides > 1); valid on the reference's CPU path
    cases.append(("rhs_both_strided", [6, 8], cs([6, 8]), 0, [8, 5], [20, 2], 3, False))
    # ragged sizes across tile boundaries
    cases.append(("ragged_tiles", [2, 67, 70], cs([2, 67, 70]), 0, [2, 70, 129], cs([2, 70, 129]), 0, False))
    return cases


def storage_len(dims, strides, off):
    return off + sum((d - 1) * s for d, s in zip(dims, strides)) + 1


def reference_from_views(lhs, ld, ls, loff, rhs, rd, rs, roff, rhs_t):
    """float64 numpy result of the view matmul, independent of the oracle's gemm."""
    L = np.lib.stride_tricks.as_strided(lhs[loff:].astype(np.float64), ld, [s * 8 for s in ls])
    R = np.lib.stride_tricks.as_strided(rhs[roff:].astype(np.float64), rd, [s * 8 for s in rs])
    if rhs_t:
        R = np.swapaxes(R, -1, -2)
    return np.matmul(L, R)
