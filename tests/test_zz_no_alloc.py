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


def _pair(xn, cuda, m, n, k, variant, seed):
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
    got, want = _pair(xn, cuda, 64, 256, 4096, 0, seed=2)
    assert _same(got, want)


def test_noalloc_rejects_sizes_beyond_its_scratch(xn, cuda):
    lib = xn.lib()
    assert lib.xn_mm_linear_fp8_noalloc_max_elems() == 262144
    # refused on the host before any pointer is touched
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 65, 16, 128, 0, None) == 2
    assert b"built-in scratch" in lib.xn_mm_last_error()
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 32, 16, 16384, 0, None) == 2
    assert lib.xn_mm_linear_fp8_noalloc(None, None, None, None, 0, 16, 128, 0, None) == 0
