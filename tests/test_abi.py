"""CPU: the C-ABI library loads, exports every declared symbol, and its host-only entry points
(matmul lowering, q4 tile packing, argument validation) agree with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import kats

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "xn_mm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xn_mm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(xn):
    names = _declared_symbols()
    assert len(names) >= 14
    h = C.CDLL(xn.LIB_PATH)
    for n in names:
        assert hasattr(h, n), f"{n} declared in include/xn_mm.h but not exported"
    assert sorted(xn.SIGNATURES) == names, "python binding table and header disagree"
    assert xn.lib().xn_mm_abi_version() == 1


def test_no_cpu_fallback(xn):
    import torch
    with pytest.raises(xn.XnError):
        xn.matmul(torch.zeros(2, 3), torch.zeros(3, 2))


def _plan(xn, ld, ls, rd, rs, rhs_t, cap):
    out = (C.c_size_t * 12)()
    arr = lambda v: (C.c_size_t * len(v))(*v)
    code = xn.lib().xn_mm_matmul_plan(len(ld), arr(ld), arr(ls), len(rd), arr(rd), arr(rs), int(rhs_t), cap, out)
    return code, [int(v) for v in out]


def test_matmul_plan_matches_oracle_lowering(xn, oracle):
    for name, ld, ls, loff, rd, rs, roff, rhs_t in kats.view_cases():
        n = rd[-2] if rhs_t else rd[-1]
        cap = int(np.prod(list(ld[:-2]) + [ld[-2], n]))
        code, got = _plan(xn, ld, ls, rd, rs, rhs_t, cap)
        ocode, want = oracle.matmul_plan(ld, ls, rd, rs, rhs_t)
        assert code == 0 and ocode == 0, name
        assert got == list(want.values()), name
    # the flattening branch: [B,T,K] x [N,K]^T becomes one GEMM with m = B*T, lhs_b = 1 (inplace_ops.rs:414-419)
    code, a = _plan(xn, [3, 5, 40], [200, 40, 1], [24, 40], [40, 1], True, 3 * 5 * 24)
    assert code == 0 and a[:4] == [15, 24, 40, 1] and a[5] == 1
    # grouped form keeps lhs_b = G and the transposed-view strides
    code, a = _plan(xn, [4, 5, 24], [24, 96, 1], [4, 12, 24], [288, 24, 1], True, 4 * 5 * 12)
    assert code == 0 and a == [5, 12, 24, 4, 24, 288, 1, 12, 1, 96, 24, 1]


def test_matmul_plan_errors(xn, oracle):
    lib = xn.lib()
    assert _plan(xn, [3], [1], [3, 2], [2, 1], False, 100)[0] == 1          # rank < 2
    assert b"at least 2D" in lib.xn_mm_last_error()
    assert _plan(xn, [2, 3], [3, 1], [4, 2], [2, 1], False, 100)[0] == 1    # inner mismatch
    assert b"inner dimension" in lib.xn_mm_last_error()
    assert _plan(xn, [2, 2, 3], [6, 3, 1], [3, 3, 2], [6, 2, 1], False, 100)[0] == 1  # batch mismatch
    assert _plan(xn, [2, 3], [3, 1], [3, 2], [2, 1], False, 3)[0] == 1      # dst too small
    assert b"too small" in lib.xn_mm_last_error()
    assert oracle.matmul_plan([3], [1], [3, 2], [2, 1], False)[0] == 1
    assert oracle.matmul_plan([2, 3], [3, 1], [4, 2], [2, 1], False)[0] == 2
    assert oracle.matmul_plan([2, 2, 3], [6, 3, 1], [3, 3, 2], [6, 2, 1], False)[0] == 3


def test_gemm_argument_validation_happens_on_the_host(xn):
    lib = xn.lib()
    # unknown dtype is refused like the reference refuses non-float GEMMs
    assert lib.xn_mm_gemm(7, 1, 1, 0, 1, 0, *([1] * 12), None) == 2
    assert b"GEMM not supported" in lib.xn_mm_last_error()
    # null pointers
    assert lib.xn_mm_gemm(0, None, None, 0, None, 0, *([1] * 12), None) == 1
    # empty problem: nothing to do, no pointer is touched
    assert lib.xn_mm_gemm(0, None, None, 0, None, 0, 0, 4, 4, 1, 0, 0, 1, 4, 1, 4, 4, 1, None) == 0
    # quantized entry points
    assert lib.xn_mm_linear_q4(None, None, None, None, 1, 16, 100, None, None) == 1
    assert b"multiple of 128" in lib.xn_mm_last_error()
    assert lib.xn_mm_linear_q4(None, None, None, None, 0, 16, 128, None, None) == 0
    assert lib.xn_mm_linear_fp8(None, None, None, None, 1, 16, 128, 5, None, 0, None) == 1
    assert lib.xn_mm_linear_fp8(1, 1, 1, 1, 1, 16, 128, 0, 256, 10, None) == 4  # workspace too small
    assert lib.xn_mm_linear_fp8_workspace_bytes(16, 4096) == 2 * 65536 + 256


def test_q4_host_packing_matches_oracle_layout(xn, oracle):
    rng = np.random.default_rng(0)
    n, k = 41, 384
    q = rng.integers(-7, 8, size=(n, k)).astype(np.int8)
    sc = rng.standard_normal((n, k // 32)).astype(np.float32)
    lib = xn.lib()
    nbytes = lib.xn_mm_q4_packed_bytes(n, k)
    assert nbytes == 3 * 3 * 1280
    packed = np.full(nbytes, 0xAB, dtype=np.uint8)
    assert lib.xn_mm_pack_q4_host(packed.ctypes.data, q.ctypes.data, sc.ctypes.data, n, k) == 0
    assert np.array_equal(packed, oracle.pack_q4(q, sc))
    back, sback = np.zeros_like(q), np.zeros_like(sc)
    assert lib.xn_mm_unpack_q4_host(back.ctypes.data, sback.ctypes.data, packed.ctypes.data, n, k) == 0
    assert np.array_equal(back, q) and np.array_equal(sback, sc)
    bad = q.copy()
    bad[0, 0] = 9
    assert lib.xn_mm_pack_q4_host(packed.ctypes.data, bad.ctypes.data, sc.ctypes.data, n, k) == 1


def test_row_op_and_scatter_validation_on_the_host(xn):
    lib = xn.lib()
    assert lib.xn_mm_rms_norm(9, 1, 1, 1, 4, 4, 1e-5, None) == 1
    assert lib.xn_mm_rms_norm(0, None, None, None, 4, 4, 1e-5, None) == 1
    assert lib.xn_mm_rms_norm(0, None, None, None, 0, 4, 1e-5, None) == 0
    assert lib.xn_mm_softmax(2, None, None, 3, 0, None) == 0
    assert lib.xn_mm_silu_mul(2, None, None, 3, 8, None) == 1
    assert lib.xn_mm_add(1, None, None, None, 0, None) == 0
    assert lib.xn_mm_kv_append(2, None, None, 0, None, 0, 4, 8, 128, None) == 0
    assert lib.xn_mm_decode_attention(1, 1, 0, 1, 1, None, 2, 4, 16, 64, 0.1, None) == 1
    assert b"head_dim" in lib.xn_mm_last_error()
    assert lib.xn_mm_decode_attention(None, None, 0, None, None, None, 0, 4, 16, 128, 0.1, None) == 0
    import ctypes as C
    ptrs = (C.c_void_p * 2)(1, 2)
    assert lib.xn_mm_linear_fp8_pieces_scatter(ptrs, 9, 64, 0, 1, 1, 1, 1, 1, 64, 32, 128, None) == 1
    assert lib.xn_mm_linear_fp8_pieces_scatter(ptrs, 2, 40, 16, 1, 1, 1, 1, 1, 64, 32, 128, None) == 1
    assert b"do not fit" in lib.xn_mm_last_error()
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 65, 16, 128, 0, None) == 2


def test_prefill_attention_validation_on_the_host(xn):
    """xn_mm_attention_prefill refuses what its kernel cannot take before anything is launched."""
    lib = xn.lib()
    BF16, F32 = 2, 0
    ok_args = dict(ldo=256, ld=768, hs=128, heads=2, hd=128, t=64, ctx=64)

    def call(dtype=BF16, out=16, q=16, k=16, v=16, **kw):
        a = dict(ok_args, **kw)
        return lib.xn_mm_attention_prefill(dtype, out, a["ldo"], q, k, v, a["ld"], a["hs"], a["heads"], a["hd"], a["t"], a["ctx"],
                                           0.1, None)

    assert call(dtype=F32) == 1 and b"16-bit" in lib.xn_mm_last_error()
    assert call(hd=64) == 1 and b"head_dim" in lib.xn_mm_last_error()
    assert call(heads=0) == 0 and call(t=0) == 0                      # nothing to do
    assert call(q=None) == 1 and b"null" in lib.xn_mm_last_error()
    assert call(ctx=32) == 1 and b"context" in lib.xn_mm_last_error()  # fewer keys than query rows
    assert call(ld=772) == 1 and call(hs=100) == 1 and call(q=18) == 1  # 16-byte alignment of pitches and pointers
    assert call(ldo=128) == 1                                         # rows too short for two heads of 128
    assert call(hs=64) == 1 and b"overlap" in lib.xn_mm_last_error()


def test_entry_points_work_with_nvtx_ranges_switched_on():
    """XN_MM_NVTX=1 wraps every entry point in an NVTX range; without a profiler attached the ranges are no-ops and
    the host-only entry points behave as before (checked in a child process: the switch is read once)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import ctypes as C, os\n"
        "lib = C.CDLL(os.path.join(%r, 'xn_b200', 'libxn_mm.so'))\n"
        "dims = (C.c_size_t * 2)(3, 4); st = (C.c_size_t * 2)(4, 1)\n"
        "rd = (C.c_size_t * 2)(5, 4); rs = (C.c_size_t * 2)(4, 1)\n"
        "out = (C.c_size_t * 16)()\n"
        "rc = lib.xn_mm_matmul_plan(C.c_size_t(2), dims, st, C.c_size_t(2), rd, rs, 1, C.c_size_t(15), out)\n"
        "assert rc == 0, rc\n"
        "rc = lib.xn_mm_matmul_plan(C.c_size_t(2), dims, st, C.c_size_t(2), rd, rs, 0, C.c_size_t(15), out)\n"
        "assert rc != 0\n"
        "print('ok')\n" % root)
    env = dict(os.environ, XN_MM_NVTX="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr
