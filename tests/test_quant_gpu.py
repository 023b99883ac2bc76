"""GPU: quantizers and the quantized linears through the C ABI, bit-exact where integer."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf16_bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_quantize_rows_i8_bit_exact(xn, oracle, cuda, dtype):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, 640, generator=g).to(dtype)
    x[3] = 0  # all-zero row: scale 0, q 0
    xq, xs = xn.quantize_rows_i8(x.to(cuda))
    oq, os_ = oracle.quantize_rows_i8(x.float().numpy())
    assert np.array_equal(xs.cpu().numpy(), os_) and np.array_equal(xq.cpu().numpy(), oq)


@pytest.mark.parametrize("n,k", [(48, 256), (41, 384), (11264, 4096)])
def test_quantize_weights_q4_bit_exact(xn, oracle, cuda, n, k):
    g = torch.Generator().manual_seed(2)
    w = torch.randn(n, k, generator=g) * 0.02
    w[1, 32:64] = 0
    packed = xn.quantize_weights_q4(w.to(cuda))
    q, s = oracle.quantize_q4(w.numpy())
    assert np.array_equal(packed.cpu().numpy(), oracle.pack_q4(q, s))


def _q4_case(xn, oracle, cuda, m, n, k, seed, partials=True):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    q, s = oracle.quantize_q4(w)
    xq, xs = oracle.quantize_rows_i8(x)
    want_y, want_p = oracle.linear_q(xq, xs, q, s, want_partials=partials)
    dq = torch.from_numpy(oracle.pack_q4(q, s)).to(cuda)
    dxq, dxs = torch.from_numpy(xq).to(cuda), torch.from_numpy(xs).to(cuda)
    part = torch.full((m, n, k // 32), -12345, dtype=torch.int32, device=cuda) if partials else None
    y = torch.full((m, n), float("nan"), device=cuda)
    xn.linear_q4(dxq, dxs, dq, n, partials=part, out=y)
    # the run without the debug output must give the same floats
    y2 = xn.linear_q4(dxq, dxs, dq, n)
    torch.cuda.synchronize()
    if partials:
        assert np.array_equal(part.cpu().numpy(), want_p), "int32 block sums must match bit for bit"
    assert torch.equal(y, y2)
    assert oracle.rel_err(y.cpu().numpy(), want_y) < 1e-4
    return y


@pytest.mark.parametrize("m", [1, 2, 4, 7, 8, 9, 16, 17, 33])
def test_linear_q4_small(xn, oracle, cuda, m):
    _q4_case(xn, oracle, cuda, m, 80, 512, seed=m)


@pytest.mark.parametrize("n,k", [(16, 128), (41, 384), (1000, 1024), (304, 11264)])
def test_linear_q4_ragged_and_long_k(xn, oracle, cuda, n, k):
    _q4_case(xn, oracle, cuda, 5, n, k, seed=n)
    _q4_case(xn, oracle, cuda, 13, n, k, seed=n + 1)


@pytest.mark.parametrize("m", [1, 4, 16])
def test_linear_q4_decode_config_full_size(xn, oracle, cuda, m):
    """W [11264,4096] N(0,0.02) int4/32, x [M,4096] N(0,1) int8 per row, seed 1: int32 block sums
    bit-exact, f32 output within 1e-4; then end-to-end through the device quantizers."""
    y = _q4_case(xn, oracle, cuda, m, 11264, 4096, seed=1)
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((11264, 4096)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, 4096)).astype(np.float32)
    lin = xn.LinearQ4.from_weight(torch.from_numpy(w).to(cuda))
    y2 = lin(torch.from_numpy(x).to(cuda))
    assert torch.equal(y, y2)


def test_linear_q4_is_linear_in_the_scales(xn, oracle, cuda):
    """Size-independent property: doubling x_scale doubles y exactly; zero activations give zero."""
    rng = np.random.default_rng(9)
    n, k, m = 2048, 2048, 16
    w = torch.from_numpy((rng.standard_normal((n, k)) * 0.02).astype(np.float32)).to(cuda)
    lin = xn.LinearQ4.from_weight(w)
    xq = torch.from_numpy(rng.integers(-127, 128, (m, k)).astype(np.int8)).to(cuda)
    xs = torch.rand(m, device=cuda) + 0.5
    y1 = xn.linear_q4(xq, xs, lin.wq, n)
    y2 = xn.linear_q4(xq, xs * 2, lin.wq, n)
    assert torch.equal(y1 * 2, y2)
    y0 = xn.linear_q4(torch.zeros_like(xq), xs, lin.wq, n)
    assert not y0.any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_quantize_weights_fp8_bit_exact(xn, oracle, cuda, dtype):
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(96, 1024, generator=g) * 0.02).to(dtype)
    w[5] = 0
    wq, ws = xn.quantize_weights_fp8(w.to(cuda))
    oq, os_ = oracle.quantize_fp8_channel(w.float().numpy())
    assert np.array_equal(ws.cpu().numpy(), os_) and np.array_equal(wq.cpu().numpy(), oq)


def test_e4m3_device_encoder_all_codes_and_random(xn, oracle, cuda):
    # per-row scale is a power of two, so hi = e4m3(x / s) exercises the device encoder directly
    t = oracle.e4m3_decode_table()
    vals = t[~np.isnan(t)]
    rng = np.random.default_rng(5)
    r = (rng.standard_normal(1 << 20) * np.exp(rng.standard_normal(1 << 20) * 2)).astype(np.float32)
    x = np.concatenate([vals, r]).astype(np.float32)
    x = np.clip(x, -440, 440)
    x[0] = 300.0  # row maximum in (224, 448] -> scale 1
    x = x[: x.size // 64 * 64].reshape(1, -1)
    x[0, 1] = 0.0
    hi, lo, s = xn.split_rows_e4m3(torch.from_numpy(x).to(cuda))
    assert float(s[0]) == 1.0 or np.abs(x).max() > 448
    ohi, olo, os_ = oracle.split_rows_e4m3(x)
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(hi.cpu().numpy(), ohi) and np.array_equal(lo.cpu().numpy(), olo)


def test_split_rows_e4m3_bf16_rows(xn, oracle, cuda):
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(9, 768, generator=g) * torch.tensor([1e-3, 1, 7, 100, 0.3, 1e4, 2, 5, 0]).view(9, 1)).bfloat16()
    hi, lo, s = xn.split_rows_e4m3(x.to(cuda))
    ohi, olo, os_ = oracle.split_rows_e4m3(x.float().numpy())
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(hi.cpu().numpy(), ohi) and np.array_equal(lo.cpu().numpy(), olo)


def _fp8_case(xn, oracle, cuda, m, n, k, seed, variant=0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    xb = oracle.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    wq, ws = oracle.quantize_fp8_channel(w)
    want16, want32 = oracle.linear_fp8(xb, wq, ws, variant)
    x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).to(cuda)
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda)
    xn.linear_fp8(x, torch.from_numpy(wq).to(cuda), torch.from_numpy(ws).to(cuda), variant, out=y)
    got = oracle.bf16_to_f32(_bf16_bits(y))
    assert not np.isnan(got).any()
    # BASELINE tolerance for fp8/bf16 outputs: max relative error 1e-2 against the CPU result
    err = oracle.rel_err(got, want32)
    assert err < 1e-2, err
    # the bf16 rounding of the true value differs from ours by at most one bf16 ulp
    ulp = np.abs(got - oracle.bf16_to_f32(want16)) / np.maximum(np.abs(want32), 1e-30)
    assert np.max(ulp[np.abs(want32) > 1e-2 * np.sqrt(np.mean(want32 ** 2))]) <= 2.0 ** -7
    return got


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 40])
@pytest.mark.parametrize("variant", [0, 1])
def test_linear_fp8_small(xn, oracle, cuda, m, variant):
    _fp8_case(xn, oracle, cuda, m, 72, 512, seed=m, variant=variant)


@pytest.mark.parametrize("n,k", [(16, 64), (100, 80), (333, 1040), (64, 11264)])
def test_linear_fp8_ragged(xn, oracle, cuda, n, k):
    _fp8_case(xn, oracle, cuda, 5, n, k, seed=n)
    _fp8_case(xn, oracle, cuda, 16, n, k, seed=n + 1)


@pytest.mark.parametrize("n,k", [(12288, 4096), (4096, 4096), (22528, 4096), (4096, 11264)])
@pytest.mark.parametrize("m", [1, 16])
def test_linear_fp8_transformer_shapes_decode(xn, oracle, cuda, n, k, m):
    _fp8_case(xn, oracle, cuda, m, n, k, seed=2)


def _fp8_gemm_sampled(xn, oracle, cuda, m, n, k, variant, seed=2, n_cols=192, n_rows=48):
    """Full-size run on the device; the oracle recomputes a random sample of rows x channels."""
    g = torch.Generator(device=cuda).manual_seed(seed)
    x = torch.randn(m, k, generator=g, device=cuda).bfloat16()
    w = torch.randn(n, k, generator=g, device=cuda) * 0.02
    wq, ws = xn.quantize_weights_fp8(w)
    del w
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda)
    xn.linear_fp8(x, wq, ws, variant, out=y)
    torch.cuda.synchronize()
    assert not torch.isnan(y).any()
    rng = np.random.default_rng(seed)
    rows = np.sort(rng.choice(m, size=min(n_rows, m), replace=False))
    cols = np.sort(rng.choice(n, size=min(n_cols, n), replace=False))
    # always include the corners and tile edges
    rows[0], rows[-1] = 0, m - 1
    cols[0], cols[-1] = 0, n - 1
    xb = _bf16_bits(x[torch.from_numpy(rows).to(cuda)])
    wq_s = wq[torch.from_numpy(cols).to(cuda)].cpu().numpy()
    ws_s = ws[torch.from_numpy(cols).to(cuda)].cpu().numpy()
    _, want32 = oracle.linear_fp8(xb, wq_s, ws_s, variant)
    got = y[torch.from_numpy(rows).to(cuda)][:, torch.from_numpy(cols).to(cuda)].float().cpu().numpy()
    err = oracle.rel_err(got, want32)
    assert err < 1e-2, err
    return y


@pytest.mark.parametrize("m", [64, 100, 256])
@pytest.mark.parametrize("variant", [0, 1])
def test_linear_fp8_gemm_small_shapes_full_check(xn, oracle, cuda, m, variant):
    # every output checked; ragged n and k exercise the zero-filled tile edges
    _fp8_case(xn, oracle, cuda, m, 200, 1040, seed=m, variant=variant)
    _fp8_case(xn, oracle, cuda, m, 520, 256, seed=m + 1, variant=variant)


@pytest.mark.parametrize("n,k", [(12288, 4096), (4096, 4096), (22528, 4096), (4096, 11264)])
@pytest.mark.parametrize("m", [64, 256, 1024, 4096])
def test_linear_fp8_transformer_shapes_prefill(xn, oracle, cuda, n, k, m):
    y0 = _fp8_gemm_sampled(xn, oracle, cuda, m, n, k, 0)
    if m == 256:
        # run-to-run identical, and the W8A8 form on the same shape
        y1 = _fp8_gemm_sampled(xn, oracle, cuda, m, n, k, 0)
        assert torch.equal(y0, y1)
        _fp8_gemm_sampled(xn, oracle, cuda, m, n, k, 1)


@pytest.mark.parametrize("m,n,k", [(1, 80, 512), (7, 41, 384), (16, 1000, 1024), (33, 304, 4096), (4, 11264, 4096)])
def test_linear_q8_block_int8_weights(xn, oracle, cuda, m, n, k):
    """int8 block-quantized weights (scale = max|w|/127 per 32-block): device quantizer and host packer
    bit-exact against the oracle, int32 block sums bit-exact, f32 output within 1e-4."""
    rng = np.random.default_rng(m + n)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    q, s = oracle.quantize_q8(w)
    xq, xs = oracle.quantize_rows_i8(x)
    want_y, want_p = oracle.linear_q(xq, xs, q, s)
    packed = xn.quantize_weights_q8(torch.from_numpy(w).to(cuda))
    assert np.array_equal(packed.cpu().numpy(), oracle.pack_q8(q, s))
    host = np.zeros(packed.numel(), np.uint8)
    assert xn.lib().xn_mm_pack_q8_host(host.ctypes.data, q.ctypes.data, s.ctypes.data, n, k) == 0
    assert np.array_equal(host, packed.cpu().numpy())
    part = torch.full((m, n, k // 32), -12345, dtype=torch.int32, device=cuda)
    dxq, dxs = torch.from_numpy(xq).to(cuda), torch.from_numpy(xs).to(cuda)
    y = xn.linear_q8(dxq, dxs, packed, n, partials=part)
    y2 = xn.linear_q8(dxq, dxs, packed, n)
    torch.cuda.synchronize()
    assert np.array_equal(part.cpu().numpy(), want_p)
    assert torch.equal(y, y2)
    assert oracle.rel_err(y.cpu().numpy(), want_y) < 1e-4


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,n,k", [(160, 80, 512), (200, 200, 384), (300, 1000, 1024), (161, 41, 4096)])
def test_linear_q_many_rows_tensor_memory_path(xn, oracle, cuda, bits, m, n, k):
    """From 160 rows on the block-quantized linears unpack the weight once and run kind::i8 tensor-memory MMAs with
    one hand-over per 32-block: f32 output within 1e-4 of the oracle and within 5e-5 of the decode kernel (f32 sums over the blocks in a different order) (which
    the debug output of the block sums selects), exact linearity in the activation scales."""
    rng = np.random.default_rng(bits * 1000 + m)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    q, s = (oracle.quantize_q4 if bits == 4 else oracle.quantize_q8)(w)
    xq, xs = oracle.quantize_rows_i8(x)
    want_y, want_p = oracle.linear_q(xq, xs, q, s)
    packed = torch.from_numpy((oracle.pack_q4 if bits == 4 else oracle.pack_q8)(q, s)).to(cuda)
    dxq, dxs = torch.from_numpy(xq).to(cuda), torch.from_numpy(xs).to(cuda)
    linear = xn.linear_q4 if bits == 4 else xn.linear_q8
    y = torch.full((m, n), float("nan"), device=cuda)
    linear(dxq, dxs, packed, n, out=y)
    part = torch.empty((m, n, k // 32), dtype=torch.int32, device=cuda)
    y_decode = linear(dxq, dxs, packed, n, partials=part)
    torch.cuda.synchronize()
    assert np.array_equal(part.cpu().numpy(), want_p)
    assert oracle.rel_err(y.cpu().numpy(), want_y) < 1e-4
    assert oracle.rel_err(y.cpu().numpy(), y_decode.cpu().numpy()) < 5e-5
    assert torch.equal(linear(dxq, dxs * 2, packed, n), y * 2)


def test_linear_q4_prefill_size_matches_the_decode_kernel(xn, oracle, cuda):
    """W [11264, 4096] int4, 1024 rows: the tensor-memory path against 64 passes of the decode kernel (whose block sums
    are pinned bit for bit to the oracle at this size) and against the oracle itself on sampled rows."""
    rng = np.random.default_rng(1)
    n, k, m = 11264, 4096, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    lin = xn.LinearQ4.from_weight(torch.from_numpy(w).to(cuda))
    xq, xs = xn.quantize_rows_i8(torch.from_numpy(x).to(cuda))
    y = xn.linear_q4(xq, xs, lin.wq, n)
    y_decode = torch.cat([xn.linear_q4(xq[i : i + 16], xs[i : i + 16], lin.wq, n) for i in range(0, m, 16)])
    torch.cuda.synchronize()
    assert oracle.rel_err(y.cpu().numpy(), y_decode.cpu().numpy()) < 2e-4  # two f32 summation orders over 128 blocks
    rows = [0, 517, 1023]
    q, s = oracle.quantize_q4(w)
    oxq, oxs = oracle.quantize_rows_i8(x[rows])
    want, _ = oracle.linear_q(oxq, oxs, q, s, want_partials=False)
    assert oracle.rel_err(y[rows].cpu().numpy(), want) < 1e-4


def test_quantized_checkpoint_feeds_the_kernels_unchanged(xn, oracle, cuda, tmp_path):
    """Weights quantized on the host, written to a quantized safetensors file, read back and uploaded as
    stored give bit-identical packed bytes to the device quantizers, and the linears run from them."""
    import os

    from xn_b200 import checkpoint as ck

    rng = np.random.default_rng(21)
    w4 = (rng.standard_normal((304, 512)) * 0.02).astype(np.float32)
    w8 = (rng.standard_normal((200, 384)) * 0.05).astype(np.float32)
    path = os.path.join(tmp_path, "m.safetensors")
    ck.save_quantized(path, {"a": w4, "b": w8}, {"a": "q4", "b": "fp8"})
    linears, _ = ck.load_quantized(path)
    la = ck.linear_from_entry(linears["a"], cuda)
    lb = ck.linear_from_entry(linears["b"], cuda)
    assert torch.equal(la.wq.cpu(), xn.quantize_weights_q4(torch.from_numpy(w4).to(cuda)).cpu())
    dq, ds = xn.quantize_weights_fp8(torch.from_numpy(w8).to(cuda))
    assert torch.equal(lb.wq.cpu(), dq.cpu()) and torch.equal(lb.ws.cpu(), ds.cpu())
    x = rng.standard_normal((5, 512)).astype(np.float32)
    y = la(torch.from_numpy(x).to(cuda)).cpu().numpy()
    xq, xs = oracle.quantize_rows_i8(x)
    q, s = oracle.quantize_q4(w4)
    ref, _ = oracle.linear_q(xq, xs, q, s)
    assert oracle.rel_err(y, ref) < 1e-4
