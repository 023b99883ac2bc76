"""GPU: stream-order safety of chained gemm calls, the device status word that bounded waits report to,
and the release of library-owned scratch."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
_T = {0: torch.float32, 2: torch.bfloat16}


@pytest.mark.parametrize("dt,m,n,k", [(2, 8, 1024, 1024), (2, 16, 2048, 512), (0, 16, 1024, 1024), (2, 32, 1024, 1024),
                                      (2, 64, 640, 1024), (0, 4, 512, 2048)])
def test_second_gemm_reads_the_first_gemms_output_as_rhs(xn, oracle, cuda, dt, m, n, k):
    """Backend::gemm's rhs can be the tensor the previous call on the stream has just produced.  The
    weight-streaming kernels prefetch a *static* weight ahead of their dependency wait; through xn_mm_gemm they
    must not.  First call: W' [n,k] = A [n,j] * B [k,j]^T (written by a large tiled launch that is still running
    when the second launch starts under programmatic dependent launch); second call: y = x * W'^T on the decode
    kernels.  Repeated so that a stale read of the poisoned W' would show."""
    j = 2048
    g = torch.Generator(device=cuda).manual_seed(m + n)
    a = (torch.randn(n, j, generator=g, device=cuda) * 0.05).to(_T[dt])
    b = (torch.randn(k, j, generator=g, device=cuda) * 0.05).to(_T[dt])
    x = torch.randn(m, k, generator=g, device=cuda).to(_T[dt])
    # the first product on its own, synchronised: the kernels are deterministic, so the chained call below writes
    # the same bits, and the reference of the second product is built from exactly those
    w0 = torch.empty(n, k, dtype=_T[dt], device=cuda)
    xn.matmul_(w0, a, b, True)
    torch.cuda.synchronize()
    ref = (x.double() @ w0.double().T).cpu().numpy()
    tol = 1e-4 if dt == 0 else 1e-2
    for _ in range(5):
        w = torch.full((n, k), float("nan"), dtype=_T[dt], device=cuda)
        y = torch.empty(m, n, dtype=_T[dt], device=cuda)
        xn.matmul_(w, a, b, True)
        xn.matmul_(y, x, w, True)
        torch.cuda.synchronize()
        got = y.float().cpu().numpy()
        assert not np.isnan(got).any()
        assert torch.equal(w, w0)
        assert oracle.rel_err(got, ref) < tol


def test_wait_that_runs_out_is_reported_and_later_launches_are_refused(xn, cuda):
    """A device-side wait that gives up must reach the host: one warp waits 20 us on a barrier nobody arrives on,
    the kernel exits normally (the context stays usable), the status word moves, entry points that launch
    waiting kernels refuse with XN_ERR_DEVICE until the status is cleared."""
    lib = xn.lib()
    n = C.c_uint(7)
    assert lib.xn_mm_device_status(C.byref(n)) == 0 and n.value == 0
    a = torch.randn(256, 128, device=cuda).bfloat16()
    try:
        assert lib.xn_mm_selftest_wait_timeout(20_000, None) == 0
        torch.cuda.synchronize()
        assert lib.xn_mm_device_status(C.byref(n)) == 5 and n.value == 1
        assert b"ran out" in lib.xn_mm_last_error()
        with pytest.raises(xn.XnError) as e:
            xn.matmul_t(a, a)  # the tensor-memory kernel has device-side waits: refused
        assert e.value.code == 5
    finally:
        assert lib.xn_mm_clear_device_status() == 0  # whatever happened above, later tests start clean
    assert lib.xn_mm_device_status(C.byref(n)) == 0 and n.value == 0
    y = xn.matmul_t(a, a)
    torch.cuda.synchronize()
    ref = (a.double() @ a.double().T).cpu().numpy()
    assert np.max(np.abs(y.float().cpu().numpy() - ref)) <= 2.0 ** -7 * np.max(np.abs(ref))
    with pytest.raises(Exception):
        xn._lib.check(lib.xn_mm_selftest_wait_timeout(0, None))


def test_release_scratch_frees_and_the_next_call_reallocates(xn, oracle, cuda):
    """The skinny kernel's hand-over buffer is library-owned; releasing it must leave the library usable."""
    lib = xn.lib()
    g = torch.Generator(device=cuda).manual_seed(2)
    w = (torch.randn(640, 4096, generator=g, device=cuda) * 0.05).bfloat16()
    x = torch.randn(32, 4096, generator=g, device=cuda).bfloat16()
    ref = (x.double() @ w.double().T).cpu().numpy()
    y1 = xn.matmul_t(x, w)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert lib.xn_mm_release_scratch(None, 1) == 0
    assert torch.cuda.mem_get_info()[0] >= free0
    y2 = xn.matmul_t(x, w)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert oracle.rel_err(y2.float().cpu().numpy(), ref) < 1e-2
    # growing on the same stream keeps the replaced block alive (a captured graph may point at it): still correct
    x2 = torch.randn(64, 4096, generator=g, device=cuda).bfloat16()
    y3 = xn.matmul_t(x2, w)
    y4 = xn.matmul_t(x, w)
    torch.cuda.synchronize()
    assert torch.equal(y4, y1)
    assert oracle.rel_err(y3.float().cpu().numpy(), (x2.double() @ w.double().T).cpu().numpy()) < 1e-2
