"""GPU: Backend::gemm through the C ABI against the oracle -- the reference's known-answer tests,
every call-site stride pattern, all three element types, and seeded larger shapes."""
import ctypes as C

import numpy as np
import pytest
import torch

import kats

pytestmark = pytest.mark.gpu
_TORCH = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}
TOL = {0: 1e-4, 1: 1e-2, 2: 1e-2}


def _to_dev(dt, flat, dev):
    t = torch.from_numpy(np.ascontiguousarray(flat))
    if dt != 0:
        t = t.view(torch.int16).view(_TORCH[dt])
    return t.to(dev)


def _to_host(dt, t):
    t = t.cpu()
    if dt != 0:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


class AbiBackend:
    """kats backend that calls xn_mm_matmul_plan / xn_mm_gemm on the device."""

    def __init__(self, xn, dev):
        self.xn, self.dev = xn, dev

    def plan(self, ld, ls, rd, rs, rhs_t, cap):
        out = (C.c_size_t * 12)()
        arr = lambda v: (C.c_size_t * len(v))(*v)
        self.xn._lib.check(self.xn.lib().xn_mm_matmul_plan(len(ld), arr(ld), arr(ls), len(rd), arr(rd), arr(rs),
                                                          int(rhs_t), cap, out))
        return [int(v) for v in out]

    def gemm(self, dt, dst_len, lhs, lhs_off, rhs, rhs_off, *a):
        dl, dr = _to_dev(dt, lhs, self.dev), _to_dev(dt, rhs, self.dev)
        # poison the output: every element must be overwritten (dst arrives uninitialised, ops.rs:697)
        dst = torch.full((dst_len,), float("nan"), dtype=_TORCH[dt], device=self.dev)
        self.xn._lib.check(self.xn.lib().xn_mm_gemm(dt, dst.data_ptr(), dl.data_ptr(), lhs_off, dr.data_ptr(), rhs_off,
                                                    *a, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        return _to_host(dt, dst)


def test_reference_kats_through_the_c_abi(xn, cuda):
    assert kats.run_all(AbiBackend(xn, cuda)) == 19


@pytest.mark.parametrize("dt", [0, 1, 2])
def test_call_site_views_match_oracle(xn, oracle, cuda, dt):
    rng = np.random.default_rng(10 + dt)
    be, ob = AbiBackend(xn, cuda), kats.OracleBackend()
    for name, ld, ls, loff, rd, rs, roff, rhs_t in kats.view_cases():
        lhs = rng.standard_normal(kats.storage_len(ld, ls, loff)).astype(np.float32)
        rhs = rng.standard_normal(kats.storage_len(rd, rs, roff)).astype(np.float32)
        lhs, rhs = oracle.to_f32(dt, oracle.from_f32(dt, lhs)), oracle.to_f32(dt, oracle.from_f32(dt, rhs))
        dims, got = kats.view_matmul(be, dt, lhs, ld, ls, loff, rhs, rd, rs, roff, rhs_t)
        _, want = kats.view_matmul(ob, dt, lhs, ld, ls, loff, rhs, rd, rs, roff, rhs_t)
        truth = kats.reference_from_views(lhs, ld, ls, loff, rhs, rd, rs, roff, rhs_t)
        assert not np.isnan(got).any(), name
        assert oracle.rel_err(got, truth) < TOL[dt], (name, oracle.rel_err(got, truth))
        assert oracle.rel_err(got, want) < 2 * TOL[dt], name


def test_python_mirror_on_torch_views(xn, oracle, cuda):
    """matmul / matmul_t / Linear on torch views (transpose, narrow, batched) vs float64."""
    g = torch.Generator(device="cpu").manual_seed(3)
    q = torch.randn(2, 3, 5, 16, generator=g).to(cuda)
    k = torch.randn(2, 3, 11, 16, generator=g).to(cuda)
    v1 = xn.matmul(q, k.transpose(2, 3))
    v2 = xn.matmul_t(q, k)
    ref = (q.double() @ k.double().transpose(2, 3)).cpu().numpy()
    assert v1.shape == (2, 3, 5, 11)
    assert oracle.rel_err(v1.cpu().numpy(), ref) < 1e-4 and oracle.rel_err(v2.cpu().numpy(), ref) < 1e-4
    w = torch.randn(24, 16, generator=g).to(cuda)
    b = torch.randn(24, generator=g).to(cuda)
    y = xn.Linear(w, b)(q)
    assert oracle.rel_err(y.cpu().numpy(), (q.double() @ w.double().T + b.double()).cpu().numpy()) < 1e-4
    big = torch.randn(8, 40, generator=g).to(cuda)
    nar = big.narrow(1, 4, 16)  # non-zero offset, row stride 40
    y2 = xn.matmul_t(nar, w)
    assert oracle.rel_err(y2.cpu().numpy(), (nar.double() @ w.double().T).cpu().numpy()) < 1e-4
    with pytest.raises(xn.XnError):
        xn.matmul(q, torch.randn(2, 3, 17, 4, device=cuda))
    with pytest.raises(xn.XnError):
        xn.matmul(q.long(), k.long().transpose(2, 3))


def test_config1_f32_linear_full_size(xn, oracle, cuda):
    """x [16,4096] N(0,1), W [11264,4096] N(0,0.02), seed 0, y = x W^T; judged against the
    f64-accumulated oracle at tolerance 1e-4."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16, 4096)).astype(np.float32)
    w = (rng.standard_normal((11264, 4096)) * 0.02).astype(np.float32)
    y = xn.matmul_t(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda)).cpu().numpy()
    truth = oracle.gemm_f64(0, x.reshape(-1), 0, w.reshape(-1), 0, 16, 11264, 4096, 1, 0, 0, (1, 4096), (4096, 1))
    rep = oracle.rel_err_report(y, truth)
    print("config 1 (f32 linear, full size) vs f64:", rep)
    assert rep["max"] < 1e-4, rep
    # the same call through Linear::forward's entry point (static weight: prefetch allowed) gives the same bits
    y2 = xn.Linear(torch.from_numpy(w).to(cuda))(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("dt", [1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 64, 8), (5, 1000, 4096), (8, 4100, 1032), (9, 272, 8192), (16, 2048, 11264),
                                   (17, 80, 520), (32, 1030, 12288), (33, 200, 4096), (64, 528, 6144)])
def test_16bit_decode_linear_tensor_core_gemv(xn, oracle, cuda, dt, m, n, k):
    """f16 / bf16 matmul_t with m <= 16 runs on the weight-streaming mma.sync kernel (1 or 2 column groups),
    more rows on the tcgen05 kernel: ragged last tile, k that is not a multiple of the 32-element step, k chunking (long k with
    many rows) and an activation view with a row pitch."""
    rng = np.random.default_rng(11 * m + n + dt)
    xfull = oracle.from_f32(dt, rng.standard_normal((m, k + 16)).astype(np.float32))
    w = oracle.from_f32(dt, (rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    xv = _to_dev(dt, xfull, cuda)[:, :k]  # rows k + 16 apart
    y = xn.matmul_t(xv, _to_dev(dt, w, cuda))
    x = np.ascontiguousarray(xfull[:, :k])
    truth = oracle.gemm_f64(dt, x.reshape(-1), 0, w.reshape(-1), 0, m, n, k, 1, 0, 0, (1, k), (k, 1))
    assert oracle.rel_err(oracle.to_f32(dt, _to_host(dt, y).reshape(-1)), truth) < TOL[dt]


@pytest.mark.parametrize("m,n,k", [(1, 256, 32), (3, 1000, 4096), (8, 4100, 1024), (9, 272, 8192), (16, 2048, 11264)])
def test_f32_decode_linear_split_tf32_path(xn, oracle, cuda, m, n, k):
    """f32 matmul_t with m <= 16, n >= 256, k % 32 == 0 runs on the tensor cores as three tf32 MMAs per
    product (hi/lo split).  The bound of the path is 1e-4; the split is expected to stay well inside it
    (about 1e-6 of the output's rms, i.e. 1e-5 in this metric).  Shapes cover both column groups, a ragged last tile, k chunking (k = 8192, 11264) and an
    activation view with a row pitch."""
    rng = np.random.default_rng(7 * m + n)
    xfull = rng.standard_normal((m, k + 32)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.03).astype(np.float32)
    xv = torch.from_numpy(xfull).to(cuda)[:, :k]  # rows k + 32 apart
    y = xn.matmul_t(xv, torch.from_numpy(w).to(cuda)).cpu().numpy()
    x = np.ascontiguousarray(xfull[:, :k])
    truth = oracle.gemm_f64(0, x.reshape(-1), 0, w.reshape(-1), 0, m, n, k, 1, 0, 0, (1, k), (k, 1))
    rep = oracle.rel_err_report(y, truth)
    print("f32 3xTF32 decode linear", (m, n, k), rep)
    assert rep["max"] < 1e-4, rep


@pytest.mark.parametrize("m,n,k,form", [(130, 70, 300, "t"), (300, 1000, 4096, "t"), (257, 264, 1028, "kn"),
                                         (128, 64, 32, "t"), (512, 200, 2052, "views"), (125, 1024, 4096, "t"),
                                         (17, 300, 1024, "kn"), (40, 512, 2048, "t"), (64, 1000, 4096, "t"), (33, 256, 96, "views"), (90, 520, 1024, "t")])
def test_f32_many_rows_tf32_piece_path(xn, oracle, cuda, m, n, k, form):
    """f32 beyond 16 rows: matmul_t form up to 96 rows runs the 3xTF32 weight-streaming kernel in passes of 16
    rows; everything else with 17+ rows runs on the tensor-memory kernel as three tf32 pieces per operand, whatever
    the operand strides (the repack normalises them), split along k when there are few output tiles; the
    accumulator is handed to f32 registers every 64 MMAs, so the result stays at f32-accumulation accuracy,
    inside the 1e-4 bar."""
    rng = np.random.default_rng(m + n + k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.03).astype(np.float32)
    xd, wd = torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda)
    if form == "t":
        y = xn.matmul_t(xd, wd)
    elif form == "kn":
        y = xn.matmul(xd, wd.t().contiguous())                      # rhs [k, n], n-contiguous
    else:
        xs = torch.zeros(m, k + 8, device=cuda)
        xs[:, :k] = xd
        y = xn.matmul(xs[:, :k], wd.t())                            # row-pitched lhs, transposed VIEW as rhs
    truth = oracle.gemm_f64(0, x.reshape(-1), 0, w.reshape(-1), 0, m, n, k, 1, 0, 0, (1, k), (k, 1))
    rep = oracle.rel_err_report(y.cpu().numpy(), truth)
    print("f32 tensor-memory matmul", (m, n, k, form), rep)
    assert rep["max"] < 1e-4, rep


def test_f32_matmul_linearity_at_prefill_size(xn, cuda):
    """2048 x 4096 x 4096 in f32 (a size the oracle would take minutes on): (a*x + y) W^T == a * x W^T + y W^T
    to f32-accumulation accuracy, and a slice of rows agrees with float64."""
    g = torch.Generator(device=cuda).manual_seed(11)
    x = torch.randn(2048, 4096, generator=g, device=cuda)
    y = torch.randn(2048, 4096, generator=g, device=cuda)
    w = torch.randn(4096, 4096, generator=g, device=cuda) * 0.02
    lhs = xn.matmul_t(2.5 * x + y, w)
    rhs = 2.5 * xn.matmul_t(x, w) + xn.matmul_t(y, w)
    assert float((lhs - rhs).abs().max()) < 1e-4 * float(rhs.abs().max())
    ref = (2.5 * x[:64] + y[:64]).double() @ w.double().t()
    assert float((lhs[:64].double() - ref).abs().max()) < 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dt,m,n,k", [(2, 64, 256, 512), (1, 33, 130, 200), (0, 130, 70, 300), (2, 1, 512, 1024),
                                      (2, 16, 384, 2048)])
def test_seeded_linear_shapes(xn, oracle, cuda, dt, m, n, k):
    rng = np.random.default_rng(100 + m)
    x = oracle.from_f32(dt, rng.standard_normal((m, k)).astype(np.float32))
    w = oracle.from_f32(dt, (rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    y = xn.matmul_t(_to_dev(dt, x, cuda), _to_dev(dt, w, cuda))
    truth = oracle.gemm_f64(dt, x.reshape(-1), 0, w.reshape(-1), 0, m, n, k, 1, 0, 0, (1, k), (k, 1))
    assert oracle.rel_err(oracle.to_f32(dt, _to_host(dt, y).reshape(-1)), truth) < TOL[dt]


def test_grouped_codebook_config_shape(xn, oracle, cuda):
    """16 groups, x [B=64,16,1024] bf16 viewed [16,64,1024], W [16,1024,1024] bf16: one call."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 16, 1024, generator=g).bfloat16().to(cuda)
    w = (torch.randn(16, 1024, 1024, generator=g) * 0.03).bfloat16().to(cuda)
    y = xn.matmul_t(x.transpose(0, 1), w)
    assert y.shape == (16, 64, 1024)
    ref = torch.einsum("bgk,gnk->gbn", x.double(), w.double()).cpu().numpy()
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < 1e-2


@pytest.mark.parametrize("dt", [1, 2])
@pytest.mark.parametrize("m,n,k", [(17, 72, 64), (128, 256, 128), (200, 328, 1032), (512, 1024, 4096), (4096, 4096, 1024)])
def test_dense_16bit_tensor_core_path(xn, oracle, cuda, dt, m, n, k):
    """Linear::forward's form (x [m,k], W [n,k], both k-contiguous) on the tcgen05 kernel; sampled
    rows/columns are recomputed by the oracle with f64 accumulation."""
    g = torch.Generator(device=cuda).manual_seed(m + n)
    x = torch.randn(m, k, generator=g, device=cuda).to(_TORCH[dt])
    w = (torch.randn(n, k, generator=g, device=cuda) * 0.05).to(_TORCH[dt])
    y = torch.full((m, n), float("nan"), dtype=_TORCH[dt], device=cuda)
    xn.matmul_(y, x, w, True)
    torch.cuda.synchronize()
    assert not torch.isnan(y).any()
    rng = np.random.default_rng(m)
    rows = np.unique(np.concatenate([[0, m - 1], rng.choice(m, size=min(40, m), replace=False)]))
    cols = np.unique(np.concatenate([[0, n - 1], rng.choice(n, size=min(96, n), replace=False)]))
    xs = _to_host(dt, x[torch.from_numpy(rows).to(cuda)].contiguous())
    ws = _to_host(dt, w[torch.from_numpy(cols).to(cuda)].contiguous())
    truth = oracle.gemm_f64(dt, xs.reshape(-1), 0, ws.reshape(-1), 0, len(rows), len(cols), k, 1, 0, 0, (1, k), (k, 1))
    got = y[torch.from_numpy(rows).to(cuda)][:, torch.from_numpy(cols).to(cuda)].float().cpu().numpy()
    assert oracle.rel_err(got, truth) < TOL[dt]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(300, 1000, 512), (128, 72, 64), (4096, 4096, 1024)])
def test_linear_bias_fused_in_the_tiled_epilogue(xn, oracle, cuda, dtype, m, n, k):
    """nn::Linear with a bias and more than 64 rows: the tiled tensor-memory kernel adds the bias to the rounded
    product in its epilogue (xn-core/src/nn/linear.rs:61-64 is matmul_t followed by broadcast_add: two roundings).
    Bit-identical to the two-launch form."""
    g = torch.Generator(device=cuda).manual_seed(m + k)
    x = torch.randn(m, k, generator=g, device=cuda).to(dtype)
    w = (torch.randn(n, k, generator=g, device=cuda) * 0.05).to(dtype)
    b = torch.randn(n, generator=g, device=cuda).to(dtype)
    y = xn.Linear(w, b)(x)
    y_plain = xn.Linear(w)(x)
    y0 = y_plain.clone()
    xn._lib.check(xn.lib().xn_mm_add_bias(xn.ops._dtype_code(y0), y0.data_ptr(), y0.data_ptr(), b.data_ptr(), m, n,
                                          torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(y, y0)
    # the product itself against f64 (the sum with the bias cancels for some elements, and two 16-bit roundings of
    # a cancelling sum are not within 1e-2 of anything: that is the reference's arithmetic, reproduced exactly above)
    rows = torch.arange(0, m, max(1, m // 37), device=cuda)
    ref = (x[rows].double() @ w.double().t()).cpu().numpy()
    assert oracle.rel_err(y_plain[rows].float().cpu().numpy(), ref) < 1e-2
    assert torch.equal(y, (y_plain.float() + b.float()).to(dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k,bias", [(256, 4096, 4096, False), (200, 1000, 2048, True), (128, 4096, 11264, False),
                                         (512, 2048, 1024, True), (65, 260, 8192, False)])
def test_few_tiles_split_along_k(xn, oracle, cuda, dtype, m, n, k, bias):
    """A hundred-odd rows against a narrow weight: the tiled kernel runs equal k chunks as its batch dimension and a
    second kernel adds the f32 tile records in k order and applies the epilogue (bias included).  Against f64 on
    sampled rows, deterministic from call to call, and the bias form bit-identical to product + broadcast_add."""
    g = torch.Generator(device=cuda).manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g, device=cuda).to(dtype)
    w = (torch.randn(n, k, generator=g, device=cuda) * 0.05).to(dtype)
    y_plain = xn.Linear(w)(x)
    y_again = xn.Linear(w)(x)
    torch.cuda.synchronize()
    assert torch.equal(y_plain, y_again)
    rows = torch.arange(0, m, max(1, m // 37), device=cuda)
    ref = (x[rows].double() @ w.double().t()).cpu().numpy()
    assert oracle.rel_err(y_plain[rows].float().cpu().numpy(), ref) < 1e-2
    # the last row and the last column are part of the product
    ref_last = (x[-1:].double() @ w.double().t()).cpu().numpy()
    assert oracle.rel_err(y_plain[-1:].float().cpu().numpy(), ref_last) < 1e-2
    # plain matmul_t (no static-weight promise) takes the same route
    y_mm = torch.empty_like(y_plain)
    xn.ops.matmul_(y_mm, x, w, True)
    torch.cuda.synchronize()
    assert torch.equal(y_mm, y_plain)
    if bias:
        b = torch.randn(n, generator=g, device=cuda).to(dtype)
        y = xn.Linear(w, b)(x)
        torch.cuda.synchronize()
        assert torch.equal(y, (y_plain.float() + b.float()).to(dtype))


def test_dense_16bit_views_with_row_pitch(xn, oracle, cuda):
    """narrow()-ed operands: row pitches larger than k, non-zero offsets (multiples of 8 elements)."""
    g = torch.Generator(device=cuda).manual_seed(5)
    xb = torch.randn(96, 320, generator=g, device=cuda).bfloat16()
    wb = (torch.randn(144, 384, generator=g, device=cuda) * 0.05).bfloat16()
    x, w = xb.narrow(1, 64, 256), wb.narrow(1, 128, 256)
    y = xn.matmul_t(x, w)
    ref = (x.double() @ w.double().T).cpu().numpy()
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < 1e-2


@pytest.mark.parametrize("dt", [1, 2])
def test_strided_batched_16bit_one_launch(xn, oracle, cuda, dt):
    """lhs_b > 1 with per-batch rhs on the tensor-core path: contiguous batches and the transposed
    (grouped per-codebook) view, plus a ragged second stage shape of the grouped configuration."""
    g = torch.Generator(device=cuda).manual_seed(11)
    a = torch.randn(5, 40, 64, generator=g, device=cuda).to(_TORCH[dt])
    b = (torch.randn(5, 24, 64, generator=g, device=cuda) * 0.1).to(_TORCH[dt])
    y = xn.matmul_t(a, b)
    ref = torch.einsum("gmk,gnk->gmn", a.double(), b.double()).cpu().numpy()
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < TOL[dt]
    x = torch.randn(64, 16, 1024, generator=g, device=cuda).to(_TORCH[dt])   # [B, G, K]
    w = (torch.randn(16, 4096, 1024, generator=g, device=cuda) * 0.03).to(_TORCH[dt])  # gated-FFN up
    y = xn.matmul_t(x.transpose(0, 1), w)
    ref = torch.einsum("bgk,gnk->gbn", x.double(), w.double()).cpu().numpy()
    assert y.shape == (16, 64, 4096)
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < TOL[dt]


@pytest.mark.parametrize("dt", [1, 2])
@pytest.mark.parametrize("m,n,k", [(32, 11264, 2048), (300, 1000, 520), (5, 200, 64), (1, 4096, 4096), (128, 72, 4096),
                                   (2048, 2048, 2048), (17, 64, 8)])
def test_16bit_matmul_with_row_major_kn_rhs_on_the_tensor_cores(xn, oracle, cuda, dt, m, n, k):
    """`a.matmul(&b)` with b = (k, n) row-major -- cuBLAS's OP_N form in the reference
    (xn-core/src/cuda_backend.rs:208-223), the shape of the reference's own bf16 benchmark
    (xn-core/examples/basic_cuda.rs:35-56: (32, 1, 2048) x (2048, 11264)) -- runs on the tcgen05 kernel with an
    MN-major B operand: ragged n and k, a single row, many tiles."""
    g = torch.Generator(device=cuda).manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g, device=cuda).to(_TORCH[dt])
    w = (torch.randn(k, n, generator=g, device=cuda) * 0.05).to(_TORCH[dt])
    y = torch.full((m, n), float("nan"), dtype=_TORCH[dt], device=cuda)
    xn.matmul_(y, x, w, False)
    torch.cuda.synchronize()
    assert not torch.isnan(y).any()
    ref = (x.double() @ w.double()).cpu().numpy()
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < TOL[dt]
    if (m, n, k) == (32, 11264, 2048):  # the reference example's other operand order: (1, 32, 2048) x (2048, 11264)
        y3 = xn.matmul(x.view(1, 32, 2048), w)
        assert torch.equal(y3.view(32, n), y)


def test_batched_attention_pv_form_with_kn_rhs(xn, oracle, cuda):
    """attn.matmul(&v) (xn-moshi/src/batched_transformer.rs:190): lhs (B*H, T, ctx), rhs (B*H, ctx, hd) row-major,
    one launch for all heads; also a narrow()-ed rhs (row pitch larger than n)."""
    g = torch.Generator(device=cuda).manual_seed(9)
    p = torch.softmax(torch.randn(6, 40, 96, generator=g, device=cuda), -1).bfloat16()
    v = torch.randn(6, 96, 128, generator=g, device=cuda).bfloat16()
    y = xn.matmul(p, v)
    ref = (p.double() @ v.double()).cpu().numpy()
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < 1e-2
    wide = torch.randn(256, 512, generator=g, device=cuda).bfloat16()
    x = torch.randn(64, 256, generator=g, device=cuda).bfloat16()
    y2 = xn.matmul(x, wide.narrow(1, 128, 200))  # rhs rows 512 apart, offset 128
    ref2 = (x.double() @ wide.narrow(1, 128, 200).double()).cpu().numpy()
    assert oracle.rel_err(y2.float().cpu().numpy(), ref2) < 1e-2


def test_gemm_is_reentrant_from_many_host_threads(xn, oracle, cuda):
    """The reference's Backend is Send + Sync and its examples/cuda_thread_test.rs hammers one device
    from 32 threads; the entry points must give the same answers under that load."""
    import threading
    g = torch.Generator(device=cuda).manual_seed(21)
    a = torch.randn(24, 96, generator=g, device=cuda)
    b = torch.randn(40, 96, generator=g, device=cuda)
    ref = (a.double() @ b.double().T).cpu().numpy()
    errs = []

    def work(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(10):
                    y = xn.matmul_t(a, b)
                st.synchronize()
            if oracle.rel_err(y.cpu().numpy(), ref) >= 1e-4:
                errs.append((i, "mismatch"))
        except Exception as e:  # noqa: BLE001
            errs.append((i, repr(e)))

    torch.cuda.synchronize()
    ts = [threading.Thread(target=work, args=(i,)) for i in range(32)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs


def test_skinny_kernel_on_concurrent_streams(xn, oracle, cuda):
    """The skinny tensor-memory kernel hands split tiles over through library-owned scratch, one buffer per
    (device, stream): threads on different streams must not disturb each other."""
    import threading
    m, n, k = 32, 640, 4096  # 5 row tiles x 64 k stages over all SMs: every tile is split
    g = torch.Generator(device=cuda).manual_seed(5)
    w = (torch.randn(n, k, generator=g, device=cuda) * 0.05).bfloat16()
    xs = [torch.randn(m, k, generator=g, device=cuda).bfloat16() for _ in range(8)]
    refs = [(x.double() @ w.double().T).cpu().numpy() for x in xs]
    errs = []

    def work(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(20):
                    y = xn.matmul_t(xs[i], w)
                st.synchronize()
            if oracle.rel_err(y.float().cpu().numpy().reshape(-1), refs[i].reshape(-1)) >= 1e-2:
                errs.append((i, "mismatch"))
        except Exception as e:  # noqa: BLE001
            errs.append((i, repr(e)))

    torch.cuda.synchronize()
    ts = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs
