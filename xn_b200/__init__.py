"""xn_b200 -- B200 (sm_100a) matmul engine for xn behind a C ABI.

The compute lives in ``libxn_mm.so`` (hand-written CUDA, built by ``python -m xn_b200.build``);
this package is the thin host-side mirror of xn's matmul interface.  Importing it loads the
library and fails if it is absent: there is no CPU or PyTorch fallback.
"""
from ._lib import BF16, F16, F32, LIB_PATH, SIGNATURES, XnError, lib

lib()  # fail loudly at import time when the CUDA library has not been built

from . import ops  # noqa: E402
from .ops import (Linear, LinearFp8, LinearQ4, gemm, linear_fp8, linear_q4, matmul, matmul_, matmul_plan,  # noqa: E402
                  matmul_t, matmul_with_t, quantize_rows_i8, quantize_weights_fp8, quantize_weights_q4, quantize_weights_q8, linear_q8,
                  split_rows_e4m3)
