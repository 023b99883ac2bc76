"""ctypes binding of libxn_mm.so -- the same symbols a Rust `extern "C"` block would bind.

There is no fallback: if the library is missing or a symbol cannot be resolved, importing
fails; if a call returns non-zero, :class:`XnError` carries the library's message.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libxn_mm.so")

F32, F16, BF16 = 0, 1, 2
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE = 0, 1, 2, 3, 4, 5


class XnError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"xn_mm error {code}: {msg}")
        self.code = code


_sz, _p, _i = C.c_size_t, C.c_void_p, C.c_int

# name -> (restype, argtypes); must list every symbol include/xn_mm.h declares.
SIGNATURES = {
    "xn_mm_last_error": (C.c_char_p, []),
    "xn_mm_abi_version": (_i, []),
    "xn_mm_gemm": (_i, [_i, _p, _p, _sz, _p, _sz] + [_sz] * 12 + [_p]),
    "xn_mm_linear": (_i, [_i, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, _p]),
    "xn_mm_device_status": (_i, [_p]),
    "xn_mm_clear_device_status": (_i, []),
    "xn_mm_selftest_wait_timeout": (_i, [C.c_ulonglong, _p]),
    "xn_mm_release_scratch": (_i, [_p, _i]),
    "xn_mm_matmul_plan": (_i, [_sz, _p, _p, _sz, _p, _p, _i, _sz, _p]),
    "xn_mm_q4_packed_bytes": (_sz, [_sz, _sz]),
    "xn_mm_quantize_weights_q4": (_i, [_p, _p, _i, _sz, _sz, _p]),
    "xn_mm_pack_q4_host": (_i, [_p, _p, _p, _sz, _sz]),
    "xn_mm_unpack_q4_host": (_i, [_p, _p, _p, _sz, _sz]),
    "xn_mm_quantize_rows_i8": (_i, [_p, _p, _p, _i, _sz, _sz, _p]),
    "xn_mm_linear_q4": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _p, _p]),
    "xn_mm_linear_q4_host_workspace_bytes": (_sz, [_sz, _sz, _sz]),
    "xn_mm_linear_q4_host": (_i, [_p, _p, _p, _sz, _sz, _sz, _p, _sz, _p]),
    "xn_mm_q8_packed_bytes": (_sz, [_sz, _sz]),
    "xn_mm_quantize_weights_q8": (_i, [_p, _p, _i, _sz, _sz, _p]),
    "xn_mm_pack_q8_host": (_i, [_p, _p, _p, _sz, _sz]),
    "xn_mm_unpack_q8_host": (_i, [_p, _p, _p, _sz, _sz]),
    "xn_mm_linear_q8": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _p, _p]),
    "xn_mm_quantize_weights_fp8": (_i, [_p, _p, _p, _i, _sz, _sz, _p]),
    "xn_mm_split_rows_e4m3": (_i, [_p, _p, _p, _p, _i, _sz, _sz, _p]),
    "xn_mm_linear_fp8_pieces": (_i, [_p, _p, _p, _p, _p, _p, _sz, _sz, _sz, _p]),
    "xn_mm_linear_fp8_pieces_scatter": (_i, [_p, _sz, _sz, _sz, _p, _p, _p, _p, _p, _sz, _sz, _sz, _p]),
    "xn_mm_linear_fp8_pieces_multicast": (_i, [_p, _sz, _sz, _p, _p, _p, _p, _p, _sz, _sz, _sz, _p]),
    "xn_mm_linear_fp8_workspace_bytes": (_sz, [_sz, _sz]),
    "xn_mm_linear_fp8": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _i, _p, _sz, _p]),
    "xn_mm_conv1d_workspace_bytes": (_sz, [_i] + [_sz] * 9),
    "xn_mm_conv1d": (_i, [_i, _p, _p, _p, _p] + [_sz] * 10 + [_p, _sz, _p]),
    "xn_mm_conv_transpose1d_workspace_bytes": (_sz, [_i] + [_sz] * 9),
    "xn_mm_conv_transpose1d": (_i, [_i, _p, _p, _p, _p] + [_sz] * 10 + [_p, _sz, _p]),
    "xn_mm_rms_norm": (_i, [_i, _p, _p, _p, _sz, _sz, C.c_float, _p]),
    "xn_mm_softmax": (_i, [_i, _p, _p, _sz, _sz, _p]),
    "xn_mm_silu_mul": (_i, [_i, _p, _p, _sz, _sz, _p]),
    "xn_mm_add": (_i, [_i, _p, _p, _p, _sz, _p]),
    "xn_mm_add_bias": (_i, [_i, _p, _p, _p, _sz, _sz, _p]),
    "xn_mm_kv_append": (_i, [_i, _p, _p, _sz, _p, _sz, _sz, _sz, _sz, _p]),
    "xn_mm_rms_norm_split_e4m3": (_i, [_p, _p, _p, _p, _p, _p, _i, _sz, _sz, C.c_float, _p]),
    "xn_mm_silu_mul_split_e4m3": (_i, [_p, _p, _p, _p, _i, _sz, _sz, _p]),
    "xn_mm_add_rms_norm_split_e4m3": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _sz, _sz, C.c_float, _p]),
    "xn_mm_decode_attention": (_i, [_p, _p, _sz, _p, _p, _p, _sz, _sz, _sz, _sz, C.c_float, _p]),
    "xn_mm_decode_attention_workspace_bytes": (_sz, [_sz, _sz, _sz]),
    "xn_mm_decode_attention_split": (_i, [_p, _p, _sz, _p, _p, _p, _sz, _sz, _sz, _sz, C.c_float, _p, _sz, _p]),
    "xn_mm_decode_attention_split_e4m3": (_i, [_p, _p, _p, _p, _p, _sz, _p, _p, _p, _sz, _sz, _sz, _sz, C.c_float, _p, _sz, _p]),
    "xn_mm_decode_attention_append_workspace_bytes": (_sz, [_sz, _sz, _sz]),
    "xn_mm_decode_attention_append_e4m3": (_i, [_p, _p, _p, _p, _p, _p, _p, _sz, _p, _p, _p, _p, _sz, _sz, _sz, _sz, C.c_float, _i, _p, _sz, _p]),
    "xn_mm_kv_append2": (_i, [_i, _p, _p, _p, _p, _sz, _p, _sz, _sz, _sz, _sz, _p]),
    "xn_mm_softmax_causal": (_i, [_i, _p, _p, _sz, _sz, _sz, C.c_float, _i, _p]),
    "xn_mm_gemm_causal": (_i, [_i, _sz, _i, _p, _p, _sz, _p, _sz] + [_sz] * 12 + [_p]),
    "xn_mm_attention_prefill": (_i, [_i, _p, _sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, C.c_float, _p]),
    "xn_mm_scatter_columns": (_i, [_p, _sz, _i, _sz, _sz, _p, _sz, _sz, _sz, _p]),
    "xn_mm_linear_fp8_noalloc_max_elems": (_sz, []),
    "xn_mm_linear_fp8_noalloc": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _i, _p]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m xn_b200.build` (nvcc, sm_100a). "
                "There is no CPU or PyTorch fallback.")
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise XnError(code, lib().xn_mm_last_error().decode("utf-8", "replace"))
