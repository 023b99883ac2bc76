"""GPU: the row operations around the matmuls and one reduced-size decoder step against the oracle."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
_T = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16) if t.dtype != torch.float32 else t.cpu().numpy()


def _dev(dt, arr, cuda):
    t = torch.from_numpy(np.ascontiguousarray(arr))
    return (t.view(torch.int16).view(_T[dt]) if dt != 0 else t).to(cuda)


@pytest.mark.parametrize("dt", [0, 1, 2])
def test_row_ops_match_oracle(xn, oracle, cuda, dt):
    rng = np.random.default_rng(dt)
    x = oracle.from_f32(dt, rng.standard_normal((7, 384)).astype(np.float32) * 2)
    a = oracle.from_f32(dt, (1 + 0.1 * rng.standard_normal(384)).astype(np.float32))
    tol = 1e-5 if dt == 0 else 8e-3  # one element-type ulp of slack for expf / division differences
    ulp = {0: 2.0 ** -23, 1: 2.0 ** -10, 2: 2.0 ** -7}[dt]
    got = oracle.to_f32(dt, _bits(xn.ops.rms_norm(_dev(dt, x, cuda), _dev(dt, a, cuda), 1e-5)).reshape(7, 384))
    want = oracle.to_f32(dt, oracle.rms_norm(dt, x, a, 1e-5))
    assert np.max(np.abs(got - want) / (np.abs(want) + 1e-3)) < tol
    got = oracle.to_f32(dt, _bits(xn.ops.softmax(_dev(dt, x, cuda))).reshape(7, 384))
    want = oracle.to_f32(dt, oracle.softmax(dt, x))
    # same roundings as the reference (difference, exponential, quotient each rounded to the element type): the
    # device's expf may differ from the host's in the last f32 bit, which can move a result by one element ulp
    lim = 2e-6 if dt == 0 else 1.001 * ulp  # f32: a few ulps of expf / summation-order difference
    assert np.all(np.abs(got - want) <= lim * np.maximum(np.abs(want), 2.0 ** -14))
    got = oracle.to_f32(dt, _bits(xn.ops.silu_mul(_dev(dt, x, cuda))).reshape(7, 192))
    want = oracle.to_f32(dt, oracle.silu_mul(dt, x))
    assert np.max(np.abs(got - want) / (np.abs(want) + 1e-3)) < tol
    y = oracle.from_f32(dt, rng.standard_normal((7, 384)).astype(np.float32))
    got = oracle.to_f32(dt, _bits(xn.ops.add(_dev(dt, x, cuda), _dev(dt, y, cuda))).reshape(7, 384))
    assert np.array_equal(got, oracle.to_f32(dt, oracle.from_f32(dt, oracle.to_f32(dt, x) + oracle.to_f32(dt, y))))


def test_fused_split_equals_op_then_split(xn, oracle, cuda):
    """rms_norm_split / silu_mul_split == plain op followed by xn_mm_split_rows_e4m3, bit for bit."""
    g = torch.Generator(device=cuda).manual_seed(0)
    lib, chk = xn.lib(), xn._lib.check
    s = torch.cuda.current_stream().cuda_stream
    x = (torch.randn(5, 1024, generator=g, device=cuda) * 3).bfloat16()
    al = (1 + 0.1 * torch.randn(1024, generator=g, device=cuda)).bfloat16()
    hi, lo = torch.empty(5, 1024, dtype=torch.uint8, device=cuda), torch.empty(5, 1024, dtype=torch.uint8, device=cuda)
    xs = torch.empty(5, device=cuda)
    chk(lib.xn_mm_rms_norm_split_e4m3(hi.data_ptr(), lo.data_ptr(), xs.data_ptr(), None, x.data_ptr(), al.data_ptr(), 2, 5,
                                      1024, 1e-5, s))
    h2, l2, s2 = xn.split_rows_e4m3(xn.ops.rms_norm(x, al, 1e-5))
    assert torch.equal(hi, h2) and torch.equal(lo, l2) and torch.equal(xs, s2)
    hh = torch.randn(5, 2048, generator=g, device=cuda).bfloat16()
    chk(lib.xn_mm_silu_mul_split_e4m3(hi.data_ptr(), lo.data_ptr(), xs.data_ptr(), hh.data_ptr(), 2, 5, 1024, s))
    h2, l2, s2 = xn.split_rows_e4m3(xn.ops.silu_mul(hh))
    assert torch.equal(hi, h2) and torch.equal(lo, l2) and torch.equal(xs, s2)


def test_kv_append_is_scatter_set_on_the_context_axis(xn, cuda):
    g = torch.Generator(device=cuda).manual_seed(1)
    B, H, ctx, hd = 3, 4, 10, 128
    cache = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    ref = cache.clone()
    qkv = torch.randn(B, 3 * H * hd, generator=g, device=cuda).bfloat16()
    idx = torch.tensor([9, 0, 4], dtype=torch.int64, device=cuda)
    xn._lib.check(xn.lib().xn_mm_kv_append(2, cache.data_ptr(), qkv.data_ptr() + 2 * H * hd, 3 * H * hd, idx.data_ptr(), B, H,
                                           ctx, hd, torch.cuda.current_stream().cuda_stream))
    src = qkv[:, H * hd:2 * H * hd].reshape(B, H, hd)
    for b in range(B):
        ref[b, :, int(idx[b])] = src[b]
    assert torch.equal(cache, ref)


@pytest.mark.parametrize("ctx", [1, 33, 300, 3000])
def test_decode_attention_vs_float64(xn, oracle, cuda, ctx):
    g = torch.Generator(device=cuda).manual_seed(ctx)
    B, H, hd = 3, 4, 128
    q = torch.randn(B, H * hd, generator=g, device=cuda).bfloat16()
    k = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    v = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    mask = torch.zeros(B, ctx, device=cuda)
    if ctx > 2:
        mask[1, ctx // 2:] = float("-inf")  # stream 1 sees only the first half of its context
    out = torch.empty(B, H * hd, dtype=torch.bfloat16, device=cuda)
    xn._lib.check(xn.lib().xn_mm_decode_attention(out.data_ptr(), q.data_ptr(), H * hd, k.data_ptr(), v.data_ptr(),
                                                  mask.data_ptr(), B, H, ctx, hd, 1 / math.sqrt(hd),
                                                  torch.cuda.current_stream().cuda_stream))
    sc = torch.einsum("bhd,bhcd->bhc", q.double().view(B, H, hd), k.double()) / math.sqrt(hd) + mask.double()[:, None, :]
    ref = torch.einsum("bhc,bhcd->bhd", torch.softmax(sc, -1), v.double()).reshape(B, H * hd).cpu().numpy()
    assert oracle.rel_err(out.float().cpu().numpy(), ref) < 1e-2
    # and the same through Backend::gemm + softmax, the reference's unfused route
    scores = xn.matmul_t(q.view(B, H, 1, hd), k)
    scores = (scores.float() / math.sqrt(hd) + mask[:, None, None, :]).bfloat16()
    p = xn.ops.softmax(scores)
    o2 = xn.matmul(p, v).reshape(B, H * hd)
    # this route rounds scores and probabilities to bf16 between the ops (as the reference does), so
    # it is judged on its rms error rather than element by element
    o2 = o2.float().cpu().numpy()
    assert np.sqrt(np.mean((o2 - ref) ** 2)) < 2e-2 * np.sqrt(np.mean(ref ** 2))


def test_decoder_step_reduced_size(xn, oracle, cuda):
    """2 layers, 4 streams, context 300, full width: the device step against a float64 restatement
    built from the same quantized weights."""
    from xn_b200.decoder import DecoderStack
    st = DecoderStack(2, 4096, 32, 11264, 4, 300, cuda, seed=4)
    g = torch.Generator(device=cuda).manual_seed(9)
    x = torch.randn(4, 4096, generator=g, device=cuda).bfloat16()
    caches = [(l["k"].clone(), l["v"].clone()) for l in st.layers]
    y = st.step(x).float().cpu().numpy()
    torch.cuda.synchronize()
    tab = torch.from_numpy(oracle.e4m3_decode_table()).double().to(cuda)

    def deq(qs):
        q, s = qs
        return tab[q.long()] * s.double()[:, None]

    def rms(t):
        return t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-5)

    cur = x.double()
    for lay, (k0, v0) in zip(st.layers, caches):
        qkv = rms(cur) @ deq(lay["in_proj"]).T
        q, kn, vn = qkv[:, :4096], qkv[:, 4096:8192], qkv[:, 8192:]
        k, v = k0.double(), v0.double()
        k[:, :, 299] = kn.view(4, 32, 128)
        v[:, :, 299] = vn.view(4, 32, 128)
        sc = torch.einsum("bhd,bhcd->bhc", q.view(4, 32, 128), k) / math.sqrt(128)
        att = torch.einsum("bhc,bhcd->bhd", torch.softmax(sc, -1), v).reshape(4, 4096)
        mid = cur + att @ deq(lay["out_proj"]).T
        h = rms(mid) @ deq(lay["linear_in"]).T
        gate = torch.nn.functional.silu(h[:, :11264]) * h[:, 11264:]
        cur = mid + gate @ deq(lay["linear_out"]).T
    ref = cur.cpu().numpy()
    # The device rounds to bf16 at every op boundary (as the reference does) while this restatement
    # keeps float64 throughout, so ~20 roundings of 2^-9 accumulate over the two layers: the step is
    # judged on its rms error and on its largest error relative to the rms of the output.
    rms = np.sqrt(np.mean(ref ** 2))
    err_rms, err_max = np.sqrt(np.mean((y - ref) ** 2)) / rms, np.max(np.abs(y - ref)) / rms
    print("decoder step: rms err", err_rms, "max err / rms", err_max)
    # measured: rms 0.0075, max 0.032 of the output's rms (a wrong head or a skipped residual moves the rms error
    # to order one)
    assert err_rms < 1e-2 and err_max < 4.5e-2
    # the other two ways of launching a layer's append + attention + merge + split give the same bits
    for mode in ("fused", "fused_one_launch"):
        for lay, (k0, v0) in zip(st.layers, caches):
            lay["k"].copy_(k0)
            lay["v"].copy_(v0)
        st.attention = mode
        y2 = st.step(x).float().cpu().numpy()
        assert np.array_equal(y, y2), mode
        assert st.launches_per_step() == 2 * (8 if mode == "fused_one_launch" or st._merge_in_kernel() else 9) + 1


def test_decode_attention_full_width_slice(xn, oracle, cuda):
    """8 streams x 32 heads x 3000 tokens (393 MB of K/V): the per-GPU decode shape at a quarter of the
    streams, against float64 on the device."""
    g = torch.Generator(device=cuda).manual_seed(77)
    B, H, ctx, hd = 8, 32, 3000, 128
    qkv = torch.randn(B, 3 * H * hd, generator=g, device=cuda).bfloat16()
    k = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    v = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    out = torch.empty(B, H * hd, dtype=torch.bfloat16, device=cuda)
    L = xn.lib()
    ws_bytes = int(L.xn_mm_decode_attention_workspace_bytes(B, H, ctx))
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=cuda)
    xn._lib.check(L.xn_mm_decode_attention_split(out.data_ptr(), qkv.data_ptr(), 3 * H * hd, k.data_ptr(), v.data_ptr(), None,
                                                 B, H, ctx, hd, 1 / math.sqrt(hd), ws.data_ptr(), ws_bytes,
                                                 torch.cuda.current_stream().cuda_stream))
    q = qkv[:, : H * hd].double().view(B, H, hd)
    sc = torch.einsum("bhd,bhcd->bhc", q, k.double()) / math.sqrt(hd)
    ref = torch.einsum("bhc,bhcd->bhd", torch.softmax(sc, -1), v.double()).reshape(B, H * hd).cpu().numpy()
    assert oracle.rel_err(out.float().cpu().numpy(), ref) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("B,ctx,masked", [(1, 3000, False), (2, 777, True), (8, 4096, True), (40, 512, False)])
def test_decode_attention_split_context_matches_single_pass(xn, oracle, cuda, B, ctx, masked):
    """The context-split form (slices merged by log-sum-exp) against the one-pass kernel and against f64:
    few streams (several slices), a ragged context, masked slices (a fully masked slice must drop out), and a
    batch large enough for the split to switch itself off."""
    H, hd = 4, 128
    g = torch.Generator().manual_seed(B * 1000 + ctx)
    q = torch.randn(B, H, hd, generator=g).bfloat16().to(cuda)
    k = torch.randn(B, H, ctx, hd, generator=g).bfloat16().to(cuda)
    v = torch.randn(B, H, ctx, hd, generator=g).bfloat16().to(cuda)
    mask = None
    if masked:
        mask = torch.zeros(B, ctx)
        mask[:, ctx // 3: ctx // 3 + ctx // 2] = float("-inf")   # covers whole slices
        mask = mask.to(cuda)
    L = xn.lib()
    ws_bytes = int(L.xn_mm_decode_attention_workspace_bytes(B, H, ctx))
    if B <= 8:
        assert ws_bytes > 0
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=cuda)
    out_s = torch.empty(B, H, hd, dtype=torch.bfloat16, device=cuda)
    out_1 = torch.empty_like(out_s)
    scale = 1.0 / np.sqrt(hd)
    mp = mask.data_ptr() if mask is not None else None
    xn._lib.check(L.xn_mm_decode_attention_split(out_s.data_ptr(), q.data_ptr(), H * hd, k.data_ptr(), v.data_ptr(), mp, B, H,
                                                 ctx, hd, scale, ws.data_ptr(), ws_bytes, None))
    xn._lib.check(L.xn_mm_decode_attention(out_1.data_ptr(), q.data_ptr(), H * hd, k.data_ptr(), v.data_ptr(), mp, B, H, ctx,
                                           hd, scale, None))
    torch.cuda.synchronize()
    a, b = out_s.float().cpu().numpy(), out_1.float().cpu().numpy()
    assert np.max(np.abs(a - b)) <= 2e-2 * max(1e-3, float(np.max(np.abs(b))))  # both round to bf16 once
    # f64 reference
    qd, kd, vd = q.double().cpu(), k.double().cpu(), v.double().cpu()
    s = torch.einsum("bhd,bhcd->bhc", qd, kd) * scale
    if mask is not None:
        s = s + mask.double().cpu()[:, None, :]
    ref = torch.einsum("bhc,bhcd->bhd", torch.softmax(s, dim=-1), vd).numpy()
    assert oracle.rel_err(a.reshape(-1), ref.reshape(-1)) < 1e-2
    # too small a workspace is refused, not overrun
    if ws_bytes:
        rc = L.xn_mm_decode_attention_split(out_s.data_ptr(), q.data_ptr(), H * hd, k.data_ptr(), v.data_ptr(), mp, B, H, ctx,
                                            hd, scale, ws.data_ptr(), ws_bytes - 4, None)
        assert rc == 4


@pytest.mark.parametrize("variant", [0, 1])
def test_add_rms_norm_split_equals_the_two_separate_ops(xn, cuda, variant):
    """The fused residual add + norm + e4m3 split gives bit for bit what xn_mm_add followed by
    xn_mm_rms_norm_split_e4m3 gives (pieces, row scales and the residual sum), also when the sum overwrites
    one of its inputs."""
    L = xn.lib()
    rows, cols = 5, 4096
    g = torch.Generator(device=cuda).manual_seed(3)
    a = torch.randn(rows, cols, generator=g, device=cuda).bfloat16()
    b = (torch.randn(rows, cols, generator=g, device=cuda) * 0.3).bfloat16()
    alpha = (1 + 0.1 * torch.randn(cols, generator=g, device=cuda)).bfloat16()
    u8 = dict(dtype=torch.uint8, device=cuda)
    s0 = torch.empty_like(a)
    hi0, lo0, xs0 = torch.empty(rows, cols, **u8), torch.empty(rows, cols, **u8), torch.empty(rows, device=cuda)
    xn._lib.check(L.xn_mm_add(2, s0.data_ptr(), a.data_ptr(), b.data_ptr(), rows * cols, None))
    xn._lib.check(L.xn_mm_rms_norm_split_e4m3(hi0.data_ptr(), lo0.data_ptr() if variant == 0 else None, xs0.data_ptr(), None,
                                              s0.data_ptr(), alpha.data_ptr(), 2, rows, cols, 1e-5, None))
    hi1, lo1, xs1 = torch.empty(rows, cols, **u8), torch.empty(rows, cols, **u8), torch.empty(rows, device=cuda)
    s1 = a.clone()  # the sum overwrites its first input
    xn._lib.check(L.xn_mm_add_rms_norm_split_e4m3(hi1.data_ptr(), lo1.data_ptr() if variant == 0 else None, xs1.data_ptr(),
                                                  s1.data_ptr(), s1.data_ptr(), b.data_ptr(), alpha.data_ptr(), 2, rows,
                                                  cols, 1e-5, None))
    torch.cuda.synchronize()
    assert torch.equal(s0, s1) and torch.equal(hi0, hi1) and torch.equal(xs0, xs1)
    if variant == 0:
        assert torch.equal(lo0, lo1)


@pytest.mark.parametrize("B,H,ctx,variant", [(4, 32, 3000, 0), (2, 8, 700, 1), (40, 4, 96, 0)])
def test_attention_with_fused_e4m3_split_equals_the_two_calls(xn, cuda, B, H, ctx, variant):
    """xn_mm_decode_attention_split_e4m3 == xn_mm_decode_attention_split followed by xn_mm_split_rows_e4m3, bit for
    bit (attention output, pieces, row scales) -- sliced contexts (fused merge + split kernel) and a context too
    short to slice (fallback to the two kernels)."""
    L = xn.lib()
    hd = 128
    g = torch.Generator(device=cuda).manual_seed(B + ctx)
    qkv = torch.randn(B, 3 * H * hd, generator=g, device=cuda).bfloat16()
    k = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    v = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    ws_bytes = int(L.xn_mm_decode_attention_workspace_bytes(B, H, ctx))
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=cuda)
    u8 = dict(dtype=torch.uint8, device=cuda)
    out0 = torch.empty(B, H * hd, dtype=torch.bfloat16, device=cuda)
    hi0, lo0, xs0 = torch.empty(B, H * hd, **u8), torch.empty(B, H * hd, **u8), torch.empty(B, device=cuda)
    sc = 1.0 / math.sqrt(hd)
    xn._lib.check(L.xn_mm_decode_attention_split(out0.data_ptr(), qkv.data_ptr(), 3 * H * hd, k.data_ptr(), v.data_ptr(), None,
                                                 B, H, ctx, hd, sc, ws.data_ptr(), ws_bytes, None))
    xn._lib.check(L.xn_mm_split_rows_e4m3(hi0.data_ptr(), lo0.data_ptr() if variant == 0 else None, xs0.data_ptr(),
                                          out0.data_ptr(), 2, B, H * hd, None))
    out1 = torch.empty_like(out0)
    hi1, lo1, xs1 = torch.empty(B, H * hd, **u8), torch.empty(B, H * hd, **u8), torch.empty(B, device=cuda)
    xn._lib.check(L.xn_mm_decode_attention_split_e4m3(hi1.data_ptr(), lo1.data_ptr() if variant == 0 else None, xs1.data_ptr(),
                                                      out1.data_ptr(), qkv.data_ptr(), 3 * H * hd, k.data_ptr(), v.data_ptr(),
                                                      None, B, H, ctx, hd, sc, ws.data_ptr(), ws_bytes, None))
    torch.cuda.synchronize()
    assert torch.equal(out0, out1) and torch.equal(hi0, hi1) and torch.equal(xs0, xs1)
    if variant == 0:
        assert torch.equal(lo0, lo1)


@pytest.mark.parametrize("merge", [0, 1, 2])
@pytest.mark.parametrize("B,H,ctx,variant,masked", [(4, 32, 3000, 0, False), (2, 8, 700, 1, True), (40, 4, 96, 0, False),
                                                     (3, 2, 33, 0, True)])
def test_attention_with_fused_append_merge_and_split_equals_the_separate_calls(xn, cuda, B, H, ctx, variant, masked, merge):
    """xn_mm_decode_attention_append_e4m3 == xn_mm_kv_append2, then xn_mm_decode_attention_split_e4m3, bit for bit:
    caches, attention output, pieces and row scales; new rows landing in different slices (first row, last row,
    somewhere inside, outside the cache = nothing appended); called twice in a row (the arrival counters are back at
    zero after a launch); merge inside the attention kernel (1), as a second launch (2), or as the library decides (0)."""
    L = xn.lib()
    hd = 128
    g = torch.Generator(device=cuda).manual_seed(7 * B + ctx)
    sc = 1.0 / math.sqrt(hd)
    u8 = dict(dtype=torch.uint8, device=cuda)
    k0 = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    v0 = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    pos = [ctx - 1, 0, ctx // 2 + 1, ctx + 5, -1, ctx // 3]
    idx = torch.tensor([pos[i % len(pos)] for i in range(B)], dtype=torch.int64, device=cuda)
    mask = None
    if masked:
        mask = torch.zeros(B, ctx, device=cuda)
        mask[:, ::3] = -1e9
        mask[0, :] = 0.0
    mp = mask.data_ptr() if mask is not None else None
    ws_a = int(L.xn_mm_decode_attention_workspace_bytes(B, H, ctx))
    ws_b = int(L.xn_mm_decode_attention_append_workspace_bytes(B, H, ctx))
    assert ws_b >= ws_a and ws_b >= B * H * (hd + 2) * 4
    wsa = torch.empty(max(ws_a, 4), dtype=torch.uint8, device=cuda)
    wsb = torch.empty(ws_b, dtype=torch.uint8, device=cuda)
    k1, v1, k2, v2 = k0.clone(), v0.clone(), k0.clone(), v0.clone()
    for rep in range(2):
        qkv = torch.randn(B, 3 * H * hd, generator=g, device=cuda).bfloat16()
        q, kn, vn = qkv.data_ptr(), qkv.data_ptr() + 2 * H * hd, qkv.data_ptr() + 4 * H * hd
        out1 = torch.empty(B, H * hd, dtype=torch.bfloat16, device=cuda)
        hi1, lo1, xs1 = torch.zeros(B, H * hd, **u8), torch.zeros(B, H * hd, **u8), torch.zeros(B, device=cuda)
        xn._lib.check(L.xn_mm_kv_append2(2, k1.data_ptr(), v1.data_ptr(), kn, vn, 3 * H * hd, idx.data_ptr(), B, H, ctx, hd, None))
        xn._lib.check(L.xn_mm_decode_attention_split_e4m3(hi1.data_ptr(), lo1.data_ptr() if variant == 0 else None, xs1.data_ptr(),
                                                          out1.data_ptr(), q, 3 * H * hd, k1.data_ptr(), v1.data_ptr(), mp,
                                                          B, H, ctx, hd, sc, wsa.data_ptr(), ws_a, None))
        out2 = torch.empty_like(out1)
        hi2, lo2, xs2 = torch.zeros(B, H * hd, **u8), torch.zeros(B, H * hd, **u8), torch.zeros(B, device=cuda)
        xn._lib.check(L.xn_mm_decode_attention_append_e4m3(hi2.data_ptr(), lo2.data_ptr() if variant == 0 else None,
                                                           xs2.data_ptr(), out2.data_ptr(), q, kn, vn, 3 * H * hd,
                                                           k2.data_ptr(), v2.data_ptr(), idx.data_ptr(), mp, B, H, ctx, hd, sc,
                                                           merge, wsb.data_ptr(), ws_b, None))
        torch.cuda.synchronize()
        assert torch.equal(k1, k2) and torch.equal(v1, v2), rep
        assert torch.equal(out1, out2), rep
        assert torch.equal(hi1, hi2) and torch.equal(xs1, xs2), rep
        if variant == 0:
            assert torch.equal(lo1, lo2), rep
    # without pieces: the attention output alone
    out3 = torch.empty_like(out2)
    k3, v3 = k0.clone(), v0.clone()
    xn._lib.check(L.xn_mm_decode_attention_append_e4m3(None, None, None, out3.data_ptr(), q, kn, vn, 3 * H * hd, k3.data_ptr(),
                                                       v3.data_ptr(), idx.data_ptr(), mp, B, H, ctx, hd, sc, merge, wsb.data_ptr(),
                                                       ws_b, None))
    out4 = torch.empty_like(out2)
    k4, v4 = k0.clone(), v0.clone()
    xn._lib.check(L.xn_mm_kv_append2(2, k4.data_ptr(), v4.data_ptr(), kn, vn, 3 * H * hd, idx.data_ptr(), B, H, ctx, hd, None))
    xn._lib.check(L.xn_mm_decode_attention_split(out4.data_ptr(), q, 3 * H * hd, k4.data_ptr(), v4.data_ptr(), mp, B, H, ctx, hd,
                                                 sc, wsa.data_ptr(), ws_a, None))
    torch.cuda.synchronize()
    assert torch.equal(out3, out4) and torch.equal(k3, k4) and torch.equal(v3, v4)
    # a workspace that is too small is refused on the host
    assert L.xn_mm_decode_attention_append_e4m3(None, None, None, out3.data_ptr(), q, kn, vn, 3 * H * hd, k3.data_ptr(),
                                                v3.data_ptr(), idx.data_ptr(), mp, B, H, ctx, hd, sc, merge, wsb.data_ptr(), 8,
                                                None) == 4
    assert L.xn_mm_decode_attention_append_e4m3(None, None, None, out3.data_ptr(), q, kn, vn, 3 * H * hd, k3.data_ptr(),
                                                v3.data_ptr(), idx.data_ptr(), mp, B, H, ctx, hd, sc, 3, wsb.data_ptr(), ws_b,
                                                None) == 1


def test_kv_append2_equals_two_appends(xn, cuda):
    g = torch.Generator(device=cuda).manual_seed(5)
    B, H, ctx, hd = 3, 4, 10, 128
    kc = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    vc = torch.randn(B, H, ctx, hd, generator=g, device=cuda).bfloat16()
    k2, v2 = kc.clone(), vc.clone()
    qkv = torch.randn(B, 3 * H * hd, generator=g, device=cuda).bfloat16()
    idx = torch.tensor([9, 0, 4], dtype=torch.int64, device=cuda)
    L = xn.lib()
    kn, vn = qkv.data_ptr() + 2 * H * hd, qkv.data_ptr() + 4 * H * hd
    xn._lib.check(L.xn_mm_kv_append(2, kc.data_ptr(), kn, 3 * H * hd, idx.data_ptr(), B, H, ctx, hd, None))
    xn._lib.check(L.xn_mm_kv_append(2, vc.data_ptr(), vn, 3 * H * hd, idx.data_ptr(), B, H, ctx, hd, None))
    xn._lib.check(L.xn_mm_kv_append2(2, k2.data_ptr(), v2.data_ptr(), kn, vn, 3 * H * hd, idx.data_ptr(), B, H, ctx, hd, None))
    torch.cuda.synchronize()
    assert torch.equal(kc, k2) and torch.equal(vc, v2)
