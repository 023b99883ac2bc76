"""GPU: the allocation-free fp8 linear (xn_mm_linear_fp8_noalloc) against xn_mm_linear_fp8.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  The entry point serves hosts that cannot allocate device memory at call time
(their device budget belongs to another allocator, or they sit in a real-time callback where a
synchronising cudaMalloc is not acceptable); its scratch is a fixed array inside the library, shared
by all calls on a device, so the test makes two calls in a row with different inputs and shapes and
checks each against the workspace-taking entry point -- stale contents of the shared array from the
first call must not leak into the second.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(xn, cuda, m, n, k, variant, seed, check_oracle=False):
    g = torch.Generator(device=cuda).manual_seed(seed)
    x = (torch.randn(m, k, generator=g, device=cuda) * (seed + 1)).bfloat16()
    w = torch.randn(n, k, generator=g, device=cuda) * 0.02
    wq, ws = xn.quantize_weights_fp8(w)
    lib = xn.lib()
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda)
    wsp = torch.empty(lib.xn_mm_linear_fp8_workspace_bytes(m, k), dtype=torch.uint8, device=cuda)
    xn._lib.check(lib.xn_mm_linear_fp8(want.data_ptr(), x.data_ptr(), wq.data_ptr(), ws.data_ptr(), m, n, k, variant,
                                       wsp.data_ptr(), wsp.numel(), stream))
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda)
    xn._lib.check(lib.xn_mm_linear_fp8_noalloc(got.data_ptr(), x.data_ptr(), wq.data_ptr(), ws.data_ptr(), m, n, k,
                                               variant, stream))
    torch.cuda.synchronize()
    if check_oracle:
        # and against the CPU oracle (the sibling entry point is itself oracle-checked elsewhere)
        import oracle as O
        xb = x.cpu().view(torch.int16).numpy().view(np.uint16)
        _, want32 = O.linear_fp8(xb, wq.cpu().numpy(), ws.cpu().numpy(), variant)
        assert O.rel_err(got.float().cpu().numpy(), want32) < 1e-2
    return got, want


def _same(got, want):
    """Same result up to the last bf16 bit: the two entry points may run different kernels (the allocation-free
    one avoids the kernel whose split-tile scratch is library-allocated), i.e. sum in a different order."""
    g, w = got.float(), want.float()
    return bool(not torch.isnan(g).any()) and float((g - w).abs().max()) <= 2.0 ** -7 * float(w.abs().max())


def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row(xn, cuda):
    # first call: a large decode batch that fills most of the built-in scratch
    got, want = _pair(xn, cuda, 16, 512, 8192, 0, seed=0)
    assert _same(got, want)
    # second call right after it: smaller, different data, other variant -- must not see stale pieces
    got, want = _pair(xn, cuda, 3, 328, 1040, 1, seed=1)
    assert torch.equal(got, want)  # same kernel on both sides at 3 rows
    # and a batch that takes the tiled tensor-memory path (m > 32)
    got, want = _pair(xn, cuda, 64, 256, 4096, 0, seed=2, check_oracle=True)
    assert _same(got, want)
    # 33..63 rows: a ragged last 32-row quarter of the tiled path's only row tile
    got, want = _pair(xn, cuda, 40, 264, 2048, 1, seed=3, check_oracle=True)
    assert _same(got, want)


def test_noalloc_rejects_sizes_beyond_its_scratch(xn, cuda):
    lib = xn.lib()
    assert lib.xn_mm_linear_fp8_noalloc_max_elems() == 262144
    # refused on the host before any pointer is touched
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 65, 16, 128, 0, None) == 2
    assert b"built-in scratch" in lib.xn_mm_last_error()
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 32, 16, 16384, 0, None) == 2
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 0, 16, 128, 0, None) == 0


def test_noalloc_checks_every_argument_before_its_first_launch(xn, cuda):
    """A rejected call must not have enqueued the activation split into the shared array: run a good call, then
    calls that fail validation (k not a multiple of 16, null weights, misaligned weights), then check that the
    array still holds the good call's pieces by re-running only the linear on them through the good call's
    result."""
    lib = xn.lib()
    got, want = _pair(xn, cuda, 4, 128, 256, 0, seed=5)
    assert torch.equal(got, want)
    x = torch.randn(4, 256, device=cuda).bfloat16()
    y = torch.empty(4, 128, dtype=torch.bfloat16, device=cuda)
    wq = torch.zeros(128 * 256 + 16, dtype=torch.uint8, device=cuda)
    ws = torch.ones(128, device=cuda)
    assert lib.xn_mm_linear_fp8_noalloc(y.data_ptr(), x.data_ptr(), wq.data_ptr(), ws.data_ptr(), 4, 128, 250, 0, None) == 1
    assert lib.xn_mm_linear_fp8_noalloc(y.data_ptr(), x.data_ptr(), None, ws.data_ptr(), 4, 128, 256, 0, None) == 1
    assert lib.xn_mm_linear_fp8_noalloc(y.data_ptr(), x.data_ptr(), wq.data_ptr() + 8, ws.data_ptr(), 4, 128, 256, 0, None) == 1
    torch.cuda.synchronize()
