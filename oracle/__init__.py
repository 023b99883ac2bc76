"""CPU oracle for the xn matmul path -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers over ``oracle/xn_oracle.c`` (built by ``oracle/Makefile`` into
``oracle/libxn_oracle.so``).  Only the tests, the smoke check and the benchmark's CPU
legs import this package; the shipped library never does.

16-bit floats travel as ``np.uint16`` bit patterns (numpy has no bfloat16).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libxn_oracle.so")

F32, F16, BF16 = 0, 1, 2
_NP = {F32: np.float32, F16: np.uint16, BF16: np.uint16}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "xn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libxn_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.xo_bf16_to_f32.restype = C.c_float
        _lib.xo_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.xo_f32_to_bf16.restype = C.c_uint16
        _lib.xo_f32_to_bf16.argtypes = [C.c_float]
        _lib.xo_f16_to_f32.restype = C.c_float
        _lib.xo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.xo_f32_to_f16.restype = C.c_uint16
        _lib.xo_f32_to_f16.argtypes = [C.c_float]
        _lib.xo_e4m3_to_f32.restype = C.c_float
        _lib.xo_e4m3_to_f32.argtypes = [C.c_uint8]
        _lib.xo_f32_to_e4m3.restype = C.c_uint8
        _lib.xo_f32_to_e4m3.argtypes = [C.c_float]
        _lib.xo_pow2_row_scale.restype = C.c_float
        _lib.xo_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _sz(*v):
    return [C.c_size_t(int(x)) for x in v]


# ---- 16-bit helpers (vectorised in numpy, checked against the C routines in tests) ----
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    return bits.view(np.float16).astype(np.float32)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def to_f32(dtype: int, a: np.ndarray) -> np.ndarray:
    return a if dtype == F32 else (f16_to_f32(a) if dtype == F16 else bf16_to_f32(a))


def from_f32(dtype: int, a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a if dtype == F32 else (f32_to_f16(a) if dtype == F16 else f32_to_bf16(a))


# ---- gemm ----
def gemm(dtype, dst_len, lhs, lhs_off, rhs, rhs_off, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride,
         dst_strides, lhs_strides, rhs_strides, accum=0) -> np.ndarray:
    """Backend::gemm on flat storages; returns the flat dst storage of ``dst_len`` elements."""
    dst = np.zeros(dst_len, dtype=_NP[dtype])
    lib().xo_gemm(C.c_int(dtype), _p(dst), _p(lhs), *_sz(lhs_off), _p(rhs), *_sz(rhs_off),
                  *_sz(m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_strides[0], dst_strides[1],
                       lhs_strides[0], lhs_strides[1], rhs_strides[0], rhs_strides[1]),
                  C.c_int(accum))
    return dst


def gemm_f64(dtype, lhs, lhs_off, rhs, rhs_off, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride,
             lhs_strides, rhs_strides) -> np.ndarray:
    dst = np.zeros(lhs_b * m * n, dtype=np.float64)
    lib().xo_gemm_f64out(C.c_int(dtype), _p(dst), _p(lhs), *_sz(lhs_off), _p(rhs), *_sz(rhs_off),
                         *_sz(m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, lhs_strides[0],
                              lhs_strides[1], rhs_strides[0], rhs_strides[1]))
    return dst


def matmul_plan(lhs_dims, lhs_strides, rhs_dims, rhs_strides, rhs_t):
    """Returns (code, dict of the 12 gemm arguments)."""
    out = (C.c_size_t * 12)()
    la = (C.c_size_t * len(lhs_dims))(*lhs_dims)
    ls = (C.c_size_t * len(lhs_dims))(*lhs_strides)
    ra = (C.c_size_t * len(rhs_dims))(*rhs_dims)
    rs = (C.c_size_t * len(rhs_dims))(*rhs_strides)
    code = lib().xo_matmul_plan(C.c_size_t(len(lhs_dims)), la, ls, C.c_size_t(len(rhs_dims)), ra, rs,
                                C.c_int(int(rhs_t)), out)
    names = ["m", "n", "k", "lhs_b", "lhs_b_stride", "rhs_b_stride", "dst_cs", "dst_rs", "lhs_cs",
             "lhs_rs", "rhs_cs", "rhs_rs"]
    return code, dict(zip(names, [int(v) for v in out]))


def contiguous_strides(dims):
    s, acc = [], 1
    for d in reversed(dims):
        s.append(acc)
        acc *= d
    return list(reversed(s))


def matmul(dtype, lhs, lhs_dims, rhs, rhs_dims, rhs_t, lhs_strides=None, rhs_strides=None,
           lhs_off=0, rhs_off=0, accum=0):
    """ops::matmul_with_t on flat storages with explicit view geometry. Returns (dims, flat)."""
    lhs_strides = lhs_strides or contiguous_strides(lhs_dims)
    rhs_strides = rhs_strides or contiguous_strides(rhs_dims)
    code, a = matmul_plan(lhs_dims, lhs_strides, rhs_dims, rhs_strides, rhs_t)
    if code:
        raise ValueError(f"matmul shape error {code}")
    out_dims = list(lhs_dims[:-2]) + [lhs_dims[-2], a["n"]]
    dst_len = int(np.prod(out_dims))
    flat = gemm(dtype, dst_len, lhs, lhs_off, rhs, rhs_off, a["m"], a["n"], a["k"], a["lhs_b"],
                a["lhs_b_stride"], a["rhs_b_stride"], (a["dst_cs"], a["dst_rs"]),
                (a["lhs_cs"], a["lhs_rs"]), (a["rhs_cs"], a["rhs_rs"]), accum)
    return out_dims, flat


# ---- quantizers ----
def quantize_blocks(w: np.ndarray, block: int, qmax: int):
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    q = np.zeros((n, k), dtype=np.int8)
    s = np.zeros((n, k // block), dtype=np.float32)
    lib().xo_quantize_blocks(_p(w), *_sz(n, k, block), C.c_int(qmax), _p(q), _p(s))
    return q, s


def quantize_q4(w):
    return quantize_blocks(w, 32, 7)


def quantize_q8(w):
    return quantize_blocks(w, 32, 127)


def quantize_rows_i8(x):
    q, s = quantize_blocks(x, x.shape[1], 127)
    return q, s.reshape(-1)


def pack_q4(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """Logical int4 values [n,k] + block scales [n,k/32] -> the engine's q4 tiles (flat uint8)."""
    n, k = q.shape
    out = np.zeros((n + 15) // 16 * (k // 128) * 1280, dtype=np.uint8)
    lib().xo_pack_q4(_p(np.ascontiguousarray(q)), _p(np.ascontiguousarray(scales, dtype=np.float32)), *_sz(n, k), _p(out))
    return out


def pack_q8(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    n, k = q.shape
    out = np.zeros((n + 15) // 16 * (k // 128) * 2304, dtype=np.uint8)
    lib().xo_pack_q8(_p(np.ascontiguousarray(q)), _p(np.ascontiguousarray(scales, dtype=np.float32)), *_sz(n, k), _p(out))
    return out


def unpack_q4(packed: np.ndarray, n: int, k: int):
    q = np.zeros((n, k), dtype=np.int8)
    s = np.zeros((n, k // 32), dtype=np.float32)
    lib().xo_unpack_q4(_p(np.ascontiguousarray(packed)), *_sz(n, k), _p(q), _p(s))
    return q, s


def linear_q(xq, x_scale, wq, w_scale, block=32, want_partials=True):
    m, k = xq.shape
    n = wq.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    part = np.zeros((m, n, k // block), dtype=np.int32) if want_partials else None
    lib().xo_linear_q(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(x_scale, dtype=np.float32)),
                      _p(np.ascontiguousarray(wq)), _p(np.ascontiguousarray(w_scale, dtype=np.float32)),
                      *_sz(m, n, k, block), _p(part) if want_partials else None, _p(y))
    return y, part


def linear_q_fast(xq, x_scale, wq, w_scale, block=32):
    """The timed CPU baseline form of linear_q (y only; AVX-512 VNNI when the host has it)."""
    m, k = xq.shape
    n = wq.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    lib().xo_linear_q_fast(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(x_scale, dtype=np.float32)),
                           _p(np.ascontiguousarray(wq)), _p(np.ascontiguousarray(w_scale, dtype=np.float32)),
                           *_sz(m, n, k, block), _p(y))
    return y


def linear_q_fast_kind() -> str:
    return "avx512-vnni" if lib().xo_linear_q_fast_is_vnni() else "compiler-vectorised int8 dot"


def e4m3_decode_table() -> np.ndarray:
    return np.array([lib().xo_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(x.shape, dtype=np.uint8)
    lib().xo_f32_to_e4m3_vec(_p(x), *_sz(x.size), _p(out))
    return out


def quantize_fp8_channel(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    q = np.zeros((n, k), dtype=np.uint8)
    s = np.zeros(n, dtype=np.float32)
    lib().xo_quantize_fp8_channel(_p(w), *_sz(n, k), _p(q), _p(s))
    return q, s


def split_rows_e4m3(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    hi = np.zeros((m, k), dtype=np.uint8)
    lo = np.zeros((m, k), dtype=np.uint8)
    s = np.zeros(m, dtype=np.float32)
    lib().xo_split_rows_e4m3(_p(x), *_sz(m, k), _p(hi), _p(lo), _p(s))
    return hi, lo, s


def linear_fp8(x_bf16, wq, w_scale, variant=0):
    m, k = x_bf16.shape
    n = wq.shape[0]
    y = np.zeros((m, n), dtype=np.uint16)
    yf = np.zeros((m, n), dtype=np.float32)
    lib().xo_linear_fp8(_p(np.ascontiguousarray(x_bf16)), _p(np.ascontiguousarray(wq)),
                        _p(np.ascontiguousarray(w_scale, dtype=np.float32)), *_sz(m, n, k),
                        C.c_int(variant), _p(y), _p(yf))
    return y, yf


def rms_norm(dtype, src, alpha, eps):
    rows, cols = src.shape
    dst = np.zeros_like(src)
    lib().xo_rms_norm(C.c_int(dtype), _p(dst), _p(np.ascontiguousarray(src)), _p(np.ascontiguousarray(alpha)),
                      *_sz(rows, cols), C.c_float(eps))
    return dst


def softmax(dtype, src):
    rows, cols = src.shape
    dst = np.zeros_like(src)
    lib().xo_softmax(C.c_int(dtype), _p(dst), _p(np.ascontiguousarray(src)), *_sz(rows, cols))
    return dst


def silu_mul(dtype, src):
    rows, two_h = src.shape
    dst = np.zeros((rows, two_h // 2), dtype=src.dtype)
    lib().xo_silu_mul(C.c_int(dtype), _p(dst), _p(np.ascontiguousarray(src)), *_sz(rows, two_h // 2))
    return dst


def conv1d(dtype, src, kernel, stride=1, padding=0, dilation=1, groups=1):
    """Backend::conv1d of the CPU backend; src (b, c_in, l), kernel (c_out, c_in/groups, ks) in storage form."""
    b, cin, length = src.shape
    cout, _, ks = kernel.shape
    lo = (length + 2 * padding - dilation * (ks - 1) - 1) // stride + 1
    dst = np.zeros((b, cout, lo), dtype=src.dtype)
    lib().xo_conv1d(C.c_int(dtype), _p(dst), _p(np.ascontiguousarray(src)), _p(np.ascontiguousarray(kernel)),
                    *_sz(b, cin, cout, length, lo, ks, stride, padding, dilation, groups))
    return dst


def conv_transpose1d(dtype, src, kernel, stride=1, padding=0, output_padding=0, groups=1):
    """Backend::conv_transpose1d of the CPU backend; kernel (c_in, c_out/groups, ks)."""
    b, cin, length = src.shape
    _, cog, ks = kernel.shape
    cout = cog * groups
    lo = (length - 1) * stride + ks + output_padding - 2 * padding
    dst = np.zeros((b, cout, lo), dtype=src.dtype)
    lib().xo_conv_transpose1d(C.c_int(dtype), _p(dst), _p(np.ascontiguousarray(src)), _p(np.ascontiguousarray(kernel)),
                              *_sz(b, cin, cout, length, lo, ks, stride, padding, output_padding, groups))
    return dst


def linear_f32_fast(x, w):
    m, k = x.shape
    n = w.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    lib().xo_linear_f32_fast(_p(np.ascontiguousarray(x, dtype=np.float32)),
                             _p(np.ascontiguousarray(w, dtype=np.float32)), _p(y), *_sz(m, n, k))
    return y


def num_threads() -> int:
    return int(lib().xo_num_threads())


def use_all_cores() -> int:
    """Sets the OpenMP thread count to the cores this process may run on (torchrun exports OMP_NUM_THREADS=1 to
    every rank, which would otherwise pin the timed CPU legs to one thread); returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().xo_set_num_threads(C.c_int(n))
    return num_threads()


def rel_err(y: np.ndarray, ref: np.ndarray, tau_frac: float = 1e-2) -> float:
    """max |y-ref| / max(|ref|, tau) with tau = tau_frac * rms(ref); tau_frac = 1e-2 is the contracted
    parity metric and what every parity test asserts.

    Outputs are sums of zero-mean products, so some land arbitrarily close to zero and a pure
    per-element relative error is unbounded for ANY finite-precision implementation; the floor keeps the
    metric finite.  At this floor an f32 limit of 1e-4 allows an absolute error of 1e-6 of the output's
    rms -- below what a sequential f32 accumulation over k = 4096 delivers (about 5e-6 at the maximum
    over 1e5 outputs), so f32 kernels have to accumulate in short chunks folded with compensation."""
    y = np.asarray(y, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    if ref.size == 0:
        return 0.0
    tau = tau_frac * float(np.sqrt(np.mean(ref * ref))) + 1e-30
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), tau)))


def rel_err_report(y: np.ndarray, ref: np.ndarray) -> dict:
    """The contracted metric with the figures printed beside it: the maximum under the 1e-2 floor, the same
    under a ten times larger floor, and the 99.9th percentile under the contracted floor."""
    y = np.asarray(y, dtype=np.float64).reshape(-1)
    ref = np.asarray(ref, dtype=np.float64).reshape(-1)
    if ref.size == 0:
        return {"max": 0.0, "max_tau_0.1": 0.0, "p99.9": 0.0}
    rms = float(np.sqrt(np.mean(ref * ref))) + 1e-30
    e = np.abs(y - ref) / np.maximum(np.abs(ref), 1e-2 * rms)
    return {"max": float(e.max()), "max_tau_0.1": rel_err(y, ref, 1e-1), "p99.9": float(np.quantile(e, 0.999))}
