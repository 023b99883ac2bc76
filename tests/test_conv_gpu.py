"""GPU: conv1d / conv_transpose1d through the C ABI against the oracle's restatement of the reference's
CPU lowering, the reference's own known-answer tests, and a float64 evaluation of the definition."""
import numpy as np
import pytest
import torch

import kats

pytestmark = pytest.mark.gpu
_T = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _dev(dt, arr, cuda):
    t = torch.from_numpy(np.ascontiguousarray(arr))
    return (t.view(torch.int16).view(_T[dt]) if dt != 0 else t).to(cuda)


def _host(oracle, dt, t):
    a = t.cpu().view(torch.int16).numpy().view(np.uint16) if dt != 0 else t.cpu().numpy()
    return oracle.to_f32(dt, a)


def _bias_ok(oracle, dt, got, truth, bias, tol):
    """The reference adds the bias as a second op on the rounded convolution (xn-core/src/ops.rs:285-298), the
    kernels here either do the same or add it before the only rounding: accept both, i.e. one element ulp of
    the larger of |conv| and |conv + bias| on top of the usual bar."""
    want = truth + oracle.to_f32(dt, bias).reshape(1, -1, 1)
    ulp = {0: 2.0 ** -23, 1: 2.0 ** -10, 2: 2.0 ** -7}[dt]
    bound = ulp * np.maximum(np.abs(truth), np.abs(want)) + tol * (1e-2 * np.sqrt(np.mean(want * want)) + np.abs(want))
    return bool(np.all(np.abs(got - want) <= bound))


def test_reference_known_answers_through_the_conv_entry_points(xn, cuda):
    """xn-core/tests/tensor_tests.rs:467-613 and the CUDA-only set xn-core/tests/cuda_tests.rs:1483-1680: exact for
    f32, within the reference's own 0.1 for its f16 cases."""
    g = kats.load()
    tdt = {"f32": torch.float32, "f16": torch.float16}

    def check(c, out):
        assert list(out.shape) == c["expected_dims"]
        got = out.float().reshape(-1).cpu().tolist()
        if c.get("tol"):
            assert all(abs(a - b) < c["tol"] for a, b in zip(got, c["expected"])), c["name"]
        else:
            assert got == c["expected"], c["name"]

    for c in g["conv1d"]:
        dt = tdt[c.get("dtype", "f32")]
        x = torch.tensor(c["input"], dtype=dt, device=cuda).reshape(c["input_dims"])
        k = torch.tensor(c["kernel"], dtype=dt, device=cuda).reshape(c["kernel_dims"])
        bias = torch.tensor(c["bias"], dtype=dt, device=cuda) if c["bias"] is not None else None
        check(c, xn.ops.conv1d(x, k, bias, c["stride"], c["padding"], 1, 1))
    for c in g["conv_transpose1d"]:
        dt = tdt[c.get("dtype", "f32")]
        x = torch.tensor(c["input"], dtype=dt, device=cuda).reshape(c["input_dims"])
        k = torch.tensor(c["kernel"], dtype=dt, device=cuda).reshape(c["kernel_dims"])
        bias = torch.tensor(c["bias"], dtype=dt, device=cuda) if c["bias"] is not None else None
        check(c, xn.ops.conv_transpose1d(x, k, bias, c["stride"], 0, 0, 1))
    assert len(g["conv1d"]) + len(g["conv_transpose1d"]) == 15


# batch, c_in, c_out, length, kernel_size, stride, padding, dilation, groups
CONV_CASES = [
    (2, 64, 96, 200, 7, 1, 3, 1, 1),      # SEANet-style k=7, "same" padding
    (1, 128, 64, 333, 3, 1, 2, 2, 1),     # dilated residual unit
    (3, 32, 64, 257, 8, 4, 2, 1, 1),      # strided down-sampling, kernel = 2 * stride
    (2, 40, 24, 100, 16, 8, 0, 1, 1),     # channels not a multiple of the staged chunk, ragged tiles
    (2, 64, 64, 70, 5, 2, 2, 3, 2),       # two groups
    (1, 48, 48, 90, 4, 1, 0, 1, 48),      # depthwise -> direct kernel
    (2, 9, 5, 31, 3, 1, 1, 1, 1),         # thin channels on the tensor-core path
    (1, 16, 8, 6, 6, 1, 0, 1, 1),         # a single output position
    (1, 64, 96, 50, 8, 1, 0, 1, 1),       # one stream, few tiles: the f32 path splits k over the SMs
    (1, 256, 128, 24, 7, 1, 3, 1, 1),     # streaming-codec step: short input, wide channels
]


@pytest.mark.parametrize("dt", [0, 1, 2])
@pytest.mark.parametrize("case", CONV_CASES)
def test_conv1d_matches_oracle_and_definition(xn, oracle, cuda, dt, case):
    b, cin, cout, length, ks, stride, pad, dil, groups = case
    rng = np.random.default_rng(hash(case) % 2**31)
    x = oracle.from_f32(dt, rng.standard_normal((b, cin, length)).astype(np.float32))
    w = oracle.from_f32(dt, (rng.standard_normal((cout, cin // groups, ks)) / np.sqrt(cin // groups * ks)).astype(np.float32))
    bias = oracle.from_f32(dt, rng.standard_normal(cout).astype(np.float32))
    got = _host(oracle, dt, xn.ops.conv1d(_dev(dt, x, cuda), _dev(dt, w, cuda), None, stride, pad, dil, groups))
    truth = kats.conv1d_f64(oracle.to_f32(dt, x), oracle.to_f32(dt, w), stride, pad, dil, groups)
    assert got.shape == truth.shape
    tol = 1e-4 if dt == 0 else 1e-2   # f32 / 16-bit output bars of the matmul path
    assert oracle.rel_err(got, truth) < tol, oracle.rel_err_report(got, truth)
    want = oracle.to_f32(dt, oracle.conv1d(dt, x, w, stride, pad, dil, groups))
    # the reference's grouped CPU loops accumulate in the element type: for 16-bit types the oracle is
    # itself many element ulps away from the definition there, and only the definition is a meaningful bar
    if oracle.rel_err(want, truth) < tol:
        assert oracle.rel_err(got, want) <= 2 * tol
    with_bias = _host(oracle, dt, xn.ops.conv1d(_dev(dt, x, cuda), _dev(dt, w, cuda), _dev(dt, bias, cuda), stride, pad, dil, groups))
    assert _bias_ok(oracle, dt, with_bias, truth, bias, tol)
    # the direct kernel computes the same thing
    import os
    os.environ["XN_CONV_DIRECT"] = "1"
    try:
        direct = _host(oracle, dt, xn.ops.conv1d(_dev(dt, x, cuda), _dev(dt, w, cuda), None, stride, pad, dil, groups))
    finally:
        del os.environ["XN_CONV_DIRECT"]
    assert oracle.rel_err(direct, truth) < tol


# batch, c_in, c_out_per_group, length, kernel_size, stride, padding, output_padding, groups
CONVT_CASES = [
    (2, 64, 32, 50, 8, 4, 0, 0, 1),       # Mimi decoder up-sampling: kernel = 2 * stride (col2im form in the reference)
    (1, 96, 64, 37, 16, 8, 0, 0, 1),
    (2, 32, 48, 41, 5, 3, 1, 1, 1),       # padding + output_padding, kernel not a multiple of stride
    (2, 64, 16, 30, 4, 2, 1, 0, 2),       # groups
    (1, 24, 1, 25, 6, 3, 0, 0, 24),       # depthwise -> direct kernel
    (3, 16, 8, 9, 3, 1, 0, 0, 1),         # stride 1
    (1, 16, 8, 5, 2, 4, 0, 0, 1),         # stride > kernel: phases with no tap write zeros
    (1, 64, 32, 20, 8, 4, 0, 0, 1),       # one stream: split k
    (1, 256, 64, 6, 16, 8, 0, 0, 1),
]


@pytest.mark.parametrize("dt", [0, 1, 2])
@pytest.mark.parametrize("case", CONVT_CASES)
def test_conv_transpose1d_matches_oracle_and_definition(xn, oracle, cuda, dt, case):
    b, cin, cog, length, ks, stride, pad, opad, groups = case
    rng = np.random.default_rng(hash(case) % 2**31)
    x = oracle.from_f32(dt, rng.standard_normal((b, cin, length)).astype(np.float32))
    w = oracle.from_f32(dt, (rng.standard_normal((cin, cog, ks)) / np.sqrt(cin // groups)).astype(np.float32))
    bias = oracle.from_f32(dt, rng.standard_normal(cog * groups).astype(np.float32))
    got = _host(oracle, dt, xn.ops.conv_transpose1d(_dev(dt, x, cuda), _dev(dt, w, cuda), None, stride, pad, opad, groups))
    truth = kats.conv_transpose1d_f64(oracle.to_f32(dt, x), oracle.to_f32(dt, w), stride, pad, opad, groups)
    assert got.shape == truth.shape
    tol = 1e-4 if dt == 0 else 1e-2
    assert oracle.rel_err(got, truth) < tol, oracle.rel_err_report(got, truth)
    want = oracle.to_f32(dt, oracle.conv_transpose1d(dt, x, w, stride, pad, opad, groups))
    if oracle.rel_err(want, truth) < tol:
        assert oracle.rel_err(got, want) <= 2 * tol
    with_bias = _host(oracle, dt, xn.ops.conv_transpose1d(_dev(dt, x, cuda), _dev(dt, w, cuda), _dev(dt, bias, cuda), stride, pad,
                                                      opad, groups))
    assert _bias_ok(oracle, dt, with_bias, truth, bias, tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv_linearity_at_model_size(xn, cuda, dtype):
    """A size the oracle would take minutes on: conv(a*x + y) == a*conv(x) + conv(y), and
    conv_transpose1d is the adjoint of conv1d: <conv(x), z> == <x, convT(z)>."""
    g = torch.Generator(device=cuda).manual_seed(3)
    x = torch.randn(4, 512, 2048, generator=g, device=cuda).to(dtype)
    y = torch.randn(4, 512, 2048, generator=g, device=cuda).to(dtype)
    w = (torch.randn(256, 512, 8, generator=g, device=cuda) / 64).to(dtype)
    tol = 1e-4 if dtype == torch.float32 else 3e-2   # bf16: the inputs of the left side are themselves rounded
    lhs = xn.ops.conv1d(2.5 * x + y, w, None, 4, 2, 1, 1)
    rhs = 2.5 * xn.ops.conv1d(x, w, None, 4, 2, 1, 1) + xn.ops.conv1d(y, w, None, 4, 2, 1, 1)
    assert float((lhs.float() - rhs.float()).abs().max()) < tol * float(rhs.float().abs().max())
    z = torch.randn_like(lhs)
    # conv1d's kernel (c_out, c_in, k) read as conv_transpose1d's (c_in', c_out', k) maps z back to x's shape
    back = xn.ops.conv_transpose1d(z, w, None, 4, 2, 0, 1)
    assert back.shape == x.shape
    a = float((lhs.double() * z.double()).sum())
    b = float(((2.5 * x + y).double() * back.double()).sum())
    assert abs(a - b) < (1e-5 if dtype == torch.float32 else 3e-3) * max(abs(a), abs(b), float(lhs.double().norm() * z.double().norm()))


def test_conv_argument_errors(xn, cuda):
    x = torch.zeros(1, 6, 10, device=cuda)
    with pytest.raises(xn.XnError, match="must be divisible by groups"):
        xn.ops.conv1d(x, torch.zeros(4, 6, 3, device=cuda), None, 1, 0, 1, 4)
    with pytest.raises(xn.XnError, match="kernel in_channels/groups mismatch"):
        xn.ops.conv1d(x, torch.zeros(4, 5, 3, device=cuda), None, 1, 0, 1, 1)
    with pytest.raises(xn.XnError, match="bias shape mismatch"):
        xn.ops.conv1d(x, torch.zeros(4, 6, 3, device=cuda), torch.zeros(3, device=cuda), 1, 0, 1, 1)
    with pytest.raises(xn.XnError, match="kernel in_channels mismatch"):
        xn.ops.conv_transpose1d(x, torch.zeros(5, 4, 3, device=cuda), None, 1, 0, 0, 1)
    s = torch.cuda.current_stream().cuda_stream
    out = torch.zeros(1, 4, 8, device=cuda)
    rc = xn.lib().xn_mm_conv1d(0, out.data_ptr(), x.data_ptr(), torch.zeros(4, 6, 3, device=cuda).data_ptr(), None, 1, 6, 4, 10, 7,
                               3, 1, 0, 1, 1, None, 0, s)
    assert rc == 1 and b"out_length" in xn.lib().xn_mm_last_error()
    # 16-bit calls on the tensor-memory path say how much scratch they need and refuse to run without it
    xb, wb, ob = torch.zeros(1, 8, 10, device=cuda).bfloat16(), torch.zeros(4, 8, 3, device=cuda).bfloat16(), out.bfloat16()
    need = xn.lib().xn_mm_conv1d_workspace_bytes(2, 1, 8, 4, 10, 3, 1, 0, 1, 1)
    assert need > 0 and xn.lib().xn_mm_conv1d_workspace_bytes(2, 1, 8, 4, 10, 3, 1, 0, 2, 1) == 0   # dilated: scratch-free kernel
    rc = xn.lib().xn_mm_conv1d(2, ob.data_ptr(), xb.data_ptr(), wb.data_ptr(), None, 1, 8, 4, 10, 8, 3, 1, 0, 1, 1, None, 0, s)
    assert rc == 4 and b"workspace" in xn.lib().xn_mm_last_error()
    # empty outputs are a no-op
    assert xn.ops.conv1d(torch.zeros(0, 6, 10, device=cuda), torch.zeros(4, 6, 3, device=cuda)).shape == (0, 4, 8)
