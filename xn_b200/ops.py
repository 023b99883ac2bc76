"""Host-side mirror of xn's matmul interface over the C ABI.

Names and argument meaning follow the reference: ``matmul`` / ``matmul_t`` / ``matmul_with_t``
(xn-core/src/ops.rs:631-714), the in-place ``matmul_`` (xn-core/src/inplace_ops.rs:318-436) and
``Linear`` (xn-core/src/nn/linear.rs:4-71).  A ``torch.Tensor`` on a CUDA device plays the role of
xn's ``Tensor`` / ``TensorView``: its storage pointer, ``storage_offset()``, ``stride()`` and
``shape`` are exactly the (storage, start_offset, strides, dims) a TensorView carries
(xn-core/src/tensor_view.rs:103-109), so transposed / narrowed views reach the kernels zero-copy.
torch is used for device memory and streams only; all arithmetic happens in libxn_mm.so.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import BF16, F16, F32, XnError, check, lib

_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        # the reference refuses other element types at the same point (cuda_backend.rs:862)
        raise XnError(_lib.ERR_UNSUPPORTED, f"GEMM not supported for dtype {t.dtype}")
    return _DT[t.dtype]


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda:
            raise XnError(_lib.ERR_INVALID, "xn_b200 runs on CUDA tensors only; there is no CPU path")


def _base_ptr(t: torch.Tensor) -> int:
    return t.untyped_storage().data_ptr()


def _arr(vals):
    return (C.c_size_t * len(vals))(*[int(v) for v in vals])


def matmul_plan(lhs: torch.Tensor, rhs: torch.Tensor, rhs_t: bool, dst_capacity: int):
    """The 12 ``Backend::gemm`` arguments for two views (xn_mm_matmul_plan)."""
    out = (C.c_size_t * 12)()
    check(lib().xn_mm_matmul_plan(lhs.dim(), _arr(lhs.shape), _arr(lhs.stride()), rhs.dim(), _arr(rhs.shape),
                                  _arr(rhs.stride()), int(rhs_t), dst_capacity, out))
    return [int(v) for v in out]


def gemm(dst: torch.Tensor, lhs: torch.Tensor, lhs_off: int, rhs: torch.Tensor, rhs_off: int, m, n, k, lhs_b,
         lhs_b_stride, rhs_b_stride, dst_strides, lhs_strides, rhs_strides) -> None:
    """``Backend::gemm`` on flat storages (xn-core/src/backend.rs:135-148)."""
    _require_cuda(dst, lhs, rhs)
    dt = _dtype_code(dst)
    check(lib().xn_mm_gemm(dt, dst.data_ptr(), lhs.data_ptr(), lhs_off, rhs.data_ptr(), rhs_off, m, n, k, lhs_b,
                           lhs_b_stride, rhs_b_stride, dst_strides[0], dst_strides[1], lhs_strides[0],
                           lhs_strides[1], rhs_strides[0], rhs_strides[1], _stream()))


def matmul_(dst: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor, rhs_t: bool) -> None:
    """``Tensor::matmul_``: dst (a whole contiguous tensor) = lhs @ rhs or lhs @ rhs^T."""
    _require_cuda(dst, lhs, rhs)
    if not (dst.dtype == lhs.dtype == rhs.dtype):
        raise XnError(_lib.ERR_INVALID, f"matmul dtype mismatch: {dst.dtype}, {lhs.dtype}, {rhs.dtype}")
    dt = _dtype_code(dst)
    a = matmul_plan(lhs, rhs, rhs_t, dst.numel())
    check(lib().xn_mm_gemm(dt, dst.data_ptr(), _base_ptr(lhs), lhs.storage_offset(), _base_ptr(rhs),
                           rhs.storage_offset(), *a, _stream()))


def matmul_causal_(dst: torch.Tensor, lhs: torch.Tensor, rhs: torch.Tensor, rhs_t: bool, mode: int, offset: int) -> None:
    """``matmul_`` for the two products of causal attention (xn_mm_gemm_causal): mode 1 = scores ``q @ k^T`` (tiles
    beyond the causal horizon are skipped and left unwritten), mode 2 = values ``p @ v`` (the masked tail of every
    row of p is not read).  Key j is visible to query row i iff j <= i + offset."""
    _require_cuda(dst, lhs, rhs)
    if not (dst.dtype == lhs.dtype == rhs.dtype):
        raise XnError(_lib.ERR_INVALID, f"matmul dtype mismatch: {dst.dtype}, {lhs.dtype}, {rhs.dtype}")
    dt = _dtype_code(dst)
    a = matmul_plan(lhs, rhs, rhs_t, dst.numel())
    check(lib().xn_mm_gemm_causal(mode, offset, dt, dst.data_ptr(), _base_ptr(lhs), lhs.storage_offset(), _base_ptr(rhs),
                                  rhs.storage_offset(), *a, _stream()))


def attention_prefill_(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> None:
    """Causal attention over a block of query rows in one kernel (xn_mm_attention_prefill).  q: [heads, T, 128] view,
    k, v: [heads, context, 128] views with a common row pitch and head stride (e.g. the slices of a fused qkv projection
    viewed per head); out: [T, heads * 128] rows (row pitch out.stride(0)).  Key j is visible to row i iff
    j <= i + (context - T)."""
    _require_cuda(out, q, k, v)
    heads, t_rows, hd = q.shape
    ctx = k.shape[1]
    if not (q.dtype == k.dtype == v.dtype == out.dtype):
        raise XnError(_lib.ERR_INVALID, "attention_prefill: dtype mismatch")
    if not (q.stride(2) == k.stride(2) == v.stride(2) == 1 and q.stride(1) == k.stride(1) == v.stride(1)
            and q.stride(0) == k.stride(0) == v.stride(0) and out.stride(1) == 1):
        raise XnError(_lib.ERR_INVALID, "attention_prefill: q, k, v must share one row pitch and one head stride")
    es = q.element_size()
    check(lib().xn_mm_attention_prefill(_dtype_code(q), out.data_ptr(), out.stride(0),
                                        _base_ptr(q) + q.storage_offset() * es, _base_ptr(k) + k.storage_offset() * es,
                                        _base_ptr(v) + v.storage_offset() * es, q.stride(1), q.stride(0), heads, hd, t_rows, ctx,
                                        float(scale), _stream()))


def matmul_with_t(lhs: torch.Tensor, rhs: torch.Tensor, rhs_t: bool) -> torch.Tensor:
    """``ops::matmul_with_t``: output shape = lhs batch dims + [M, N], allocated uninitialised."""
    if lhs.dim() < 2 or rhs.dim() < 2:
        raise XnError(_lib.ERR_INVALID, "matmul requires at least 2D tensors")
    n = rhs.shape[-2] if rhs_t else rhs.shape[-1]
    out = torch.empty(*lhs.shape[:-2], lhs.shape[-2], n, dtype=lhs.dtype, device=lhs.device)
    matmul_(out, lhs, rhs, rhs_t)
    return out


def matmul(lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    return matmul_with_t(lhs, rhs, False)


def matmul_t(lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    return matmul_with_t(lhs, rhs, True)


class Linear:
    """``nn::Linear``: weight (out_features, in_features), optional bias (out_features)."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        self.weight, self.bias = weight, bias

    def with_bias(self, bias: torch.Tensor) -> "Linear":
        self.bias = bias
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = self.weight, self.bias
        if b is not None:
            _require_cuda(b)
            if b.dtype != x.dtype or list(b.shape) != [w.shape[0]]:
                raise XnError(1, f"bias shape mismatch: expected [{w.shape[0]}] of {x.dtype}, got {list(b.shape)} of {b.dtype}")
        # Contiguous-row activations and weight (what every model layer passes): the Linear entry point, which
        # may prefetch the weight -- a parameter, never the previous kernel's output -- ahead of the stream order.
        if (x.is_cuda and w.is_cuda and x.dtype == w.dtype and x.dim() >= 2 and w.dim() == 2 and x.shape[-1] == w.shape[1]
                and x.stride(-1) == 1 and w.stride(1) == 1 and x.is_contiguous()):
            n, k = w.shape
            m = x.numel() // k if k else 0
            y = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
            check(lib().xn_mm_linear(_dtype_code(x), y.data_ptr(), x.data_ptr(), w.data_ptr(),
                                     b.contiguous().data_ptr() if b is not None else None, m, n, k, k, w.stride(0), n,
                                     _stream()))
            return y
        y = matmul_t(x, w)
        if b is not None:
            # the reference's separate broadcast_add (nn/linear.rs:61-64)
            check(lib().xn_mm_add_bias(_dtype_code(y), y.data_ptr(), y.data_ptr(), b.contiguous().data_ptr(),
                                       y.numel() // y.shape[-1], y.shape[-1], _stream()))
        return y

    __call__ = forward


# ---------------------------------------------------------------------------------------------
# Quantized linears (no counterpart in the reference): same forward(x) signature as Linear.
# ---------------------------------------------------------------------------------------------
def quantize_rows_i8(x: torch.Tensor, out: tuple[torch.Tensor, torch.Tensor] | None = None):
    """Per-row symmetric int8 quantization; `out` = (xq int8 [m,k], x_scale f32 [m]) reuses buffers."""
    _require_cuda(x)
    x = x.contiguous()
    m, k = x.shape
    if out is not None:
        xq, xs = out
        if xq.shape != (m, k) or xq.dtype != torch.int8 or xs.shape != (m,) or xs.dtype != torch.float32:
            raise ValueError("quantize_rows_i8: out must be (int8 [m,k], float32 [m])")
        _require_cuda(xq, xs)
    else:
        xq = torch.empty(m, k, dtype=torch.int8, device=x.device)
        xs = torch.empty(m, dtype=torch.float32, device=x.device)
    check(lib().xn_mm_quantize_rows_i8(xq.data_ptr(), xs.data_ptr(), x.data_ptr(), _dtype_code(x), m, k, _stream()))
    return xq, xs


def quantize_weights_q4(w: torch.Tensor) -> torch.Tensor:
    """W [n,k] -> q4 tiles (uint8 buffer holding nibbles and block scales)."""
    _require_cuda(w)
    w = w.contiguous()
    n, k = w.shape
    packed = torch.empty(lib().xn_mm_q4_packed_bytes(n, k), dtype=torch.uint8, device=w.device)
    check(lib().xn_mm_quantize_weights_q4(packed.data_ptr(), w.data_ptr(), _dtype_code(w), n, k, _stream()))
    return packed


def linear_q4(xq: torch.Tensor, x_scale: torch.Tensor, wq_packed: torch.Tensor, n: int,
              partials: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(xq, wq_packed)
    m, k = xq.shape
    y = out if out is not None else torch.empty(m, n, dtype=torch.float32, device=xq.device)
    check(lib().xn_mm_linear_q4(y.data_ptr(), xq.data_ptr(), x_scale.data_ptr(), wq_packed.data_ptr(), m, n, k,
                                partials.data_ptr() if partials is not None else None, _stream()))
    return y


def quantize_weights_q8(w: torch.Tensor) -> torch.Tensor:
    """W [n,k] -> q8 tiles (int8 block-quantized, scale = max|w|/127 per 32-block)."""
    _require_cuda(w)
    w = w.contiguous()
    n, k = w.shape
    packed = torch.empty(lib().xn_mm_q8_packed_bytes(n, k), dtype=torch.uint8, device=w.device)
    check(lib().xn_mm_quantize_weights_q8(packed.data_ptr(), w.data_ptr(), _dtype_code(w), n, k, _stream()))
    return packed


def linear_q8(xq: torch.Tensor, x_scale: torch.Tensor, wq_packed: torch.Tensor, n: int,
              partials: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(xq, wq_packed)
    m, k = xq.shape
    y = out if out is not None else torch.empty(m, n, dtype=torch.float32, device=xq.device)
    check(lib().xn_mm_linear_q8(y.data_ptr(), xq.data_ptr(), x_scale.data_ptr(), wq_packed.data_ptr(), m, n, k,
                                partials.data_ptr() if partials is not None else None, _stream()))
    return y


class LinearQ4:
    """int4 block-quantized linear: forward(x) quantizes x per row to int8, returns f32."""

    def __init__(self, wq_packed, out_features: int, in_features: int):
        self.wq, self.n, self.k = wq_packed, out_features, in_features

    @classmethod
    def from_weight(cls, w: torch.Tensor) -> "LinearQ4":
        return cls(quantize_weights_q4(w), w.shape[0], w.shape[1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        xq, xs = quantize_rows_i8(x.reshape(-1, self.k))
        return linear_q4(xq, xs, self.wq, self.n).reshape(*lead, self.n)

    __call__ = forward

    def forward_host(self, x_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
        """x_host [m,k] f32 and y_host [m,n] f32 in (pinned) host memory: one library call enqueues the copy in,
        the row quantizer, the linear and the copy out on the current stream (xn_mm_linear_q4_host); the result
        is valid after the stream has been synchronised.  Staging buffers are kept per batch size."""
        m = x_host.shape[0]
        if x_host.is_cuda or y_host.is_cuda or x_host.dtype != torch.float32 or y_host.dtype != torch.float32:
            raise XnError(_lib.ERR_INVALID, "forward_host takes float32 host tensors")
        if list(x_host.shape) != [m, self.k] or list(y_host.shape) != [m, self.n] or not x_host.is_contiguous() \
                or not y_host.is_contiguous():
            raise XnError(_lib.ERR_INVALID, f"forward_host: expected contiguous [{m},{self.k}] and [{m},{self.n}]")
        ws = self._host_ws.get(m) if hasattr(self, "_host_ws") else None
        if ws is None:
            if not hasattr(self, "_host_ws"):
                self._host_ws = {}
            ws = torch.empty(lib().xn_mm_linear_q4_host_workspace_bytes(m, self.n, self.k), dtype=torch.uint8,
                             device=self.wq.device)
            self._host_ws[m] = ws
        check(lib().xn_mm_linear_q4_host(y_host.data_ptr(), x_host.data_ptr(), self.wq.data_ptr(), m, self.n, self.k,
                                         ws.data_ptr(), ws.numel(), _stream()))
        return y_host


def quantize_weights_fp8(w: torch.Tensor):
    _require_cuda(w)
    w = w.contiguous()
    n, k = w.shape
    wq = torch.empty(n, k, dtype=torch.uint8, device=w.device)
    ws = torch.empty(n, dtype=torch.float32, device=w.device)
    check(lib().xn_mm_quantize_weights_fp8(wq.data_ptr(), ws.data_ptr(), w.data_ptr(), _dtype_code(w), n, k, _stream()))
    return wq, ws


def split_rows_e4m3(x: torch.Tensor, want_lo: bool = True):
    _require_cuda(x)
    x = x.contiguous()
    m, k = x.shape
    hi = torch.empty(m, k, dtype=torch.uint8, device=x.device)
    lo = torch.empty(m, k, dtype=torch.uint8, device=x.device) if want_lo else None
    xs = torch.empty(m, dtype=torch.float32, device=x.device)
    check(lib().xn_mm_split_rows_e4m3(hi.data_ptr(), lo.data_ptr() if want_lo else None, xs.data_ptr(), x.data_ptr(),
                                      _dtype_code(x), m, k, _stream()))
    return hi, lo, xs


def linear_fp8(x: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor, variant: int = 0,
               workspace: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """y bf16 [m,n] = fp8 linear of bf16 x [m,k]; variant 0 = W8A16, 1 = W8A8."""
    _require_cuda(x, wq)
    if x.dtype != torch.bfloat16:
        raise XnError(_lib.ERR_INVALID, "linear_fp8 takes bf16 activations")
    x = x.contiguous()
    m, k = x.shape
    n = wq.shape[0]
    need = lib().xn_mm_linear_fp8_workspace_bytes(m, k)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    y = out if out is not None else torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    check(lib().xn_mm_linear_fp8(y.data_ptr(), x.data_ptr(), wq.data_ptr(), w_scale.data_ptr(), m, n, k, variant,
                                 workspace.data_ptr(), workspace.numel(), _stream()))
    return y


class LinearFp8:
    """fp8-e4m3 per-channel linear: forward(x bf16) -> bf16."""

    def __init__(self, wq: torch.Tensor, w_scale: torch.Tensor, variant: int = 0):
        self.wq, self.ws, self.variant = wq, w_scale, variant

    @classmethod
    def from_weight(cls, w: torch.Tensor, variant: int = 0) -> "LinearFp8":
        q, s = quantize_weights_fp8(w)
        return cls(q, s, variant)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        return linear_fp8(x.reshape(-1, x.shape[-1]), self.wq, self.ws, self.variant).reshape(*lead, self.wq.shape[0])

    __call__ = forward


# ---------------------------------------------------------------------------------------------
# Convolutions: Tensor::conv1d / Tensor::conv_transpose1d (xn-core/src/ops.rs:253-300, 305-350),
# same arguments, same shape rules and error texts; one launch each, bias fused.
# ---------------------------------------------------------------------------------------------
_CONV_WS: dict = {}


def _conv_workspace(device, nbytes: int):
    """Scratch of the tensor-memory conv path: one buffer per (device, stream), grown on demand."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _CONV_WS.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _CONV_WS[key] = buf
    return buf


def _check_bias(bias, out_channels):
    if bias is not None and list(bias.shape) != [out_channels]:
        raise XnError(1, f"bias shape mismatch: expected [{out_channels}], got {list(bias.shape)}")


def conv1d(x: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor | None = None, stride: int = 1,
           padding: int = 0, dilation: int = 1, groups: int = 1) -> torch.Tensor:
    _require_cuda(x, kernel)
    if x.dim() != 3 or kernel.dim() != 3:
        raise XnError(1, f"conv1d expects rank-3 input and kernel, got {list(x.shape)} and {list(kernel.shape)}")
    batch, in_channels, length = x.shape
    out_channels, kernel_in_channels, kernel_size = kernel.shape
    if groups < 1 or in_channels % groups:
        raise XnError(1, f"in_channels ({in_channels}) must be divisible by groups ({groups})")
    if out_channels % groups:
        raise XnError(1, f"out_channels ({out_channels}) must be divisible by groups ({groups})")
    if kernel_in_channels != in_channels // groups:
        raise XnError(1, f"kernel in_channels/groups mismatch: expected {in_channels // groups}, got {kernel_in_channels}")
    _check_bias(bias, out_channels)
    span = dilation * (kernel_size - 1) + 1
    if length + 2 * padding < span:
        raise XnError(1, f"kernel span {span} exceeds the padded length {length + 2 * padding}")
    out_length = (length + 2 * padding - span) // stride + 1
    x, kernel = x.contiguous(), kernel.contiguous()
    out = torch.empty(batch, out_channels, out_length, dtype=x.dtype, device=x.device)
    ws_bytes = lib().xn_mm_conv1d_workspace_bytes(_dtype_code(x), batch, in_channels, out_channels, length, kernel_size,
                                                  stride, padding, dilation, groups)
    ws = _conv_workspace(x.device, ws_bytes)
    check(lib().xn_mm_conv1d(_dtype_code(x), out.data_ptr(), x.data_ptr(), kernel.data_ptr(),
                             bias.contiguous().data_ptr() if bias is not None else None, batch, in_channels,
                             out_channels, length, out_length, kernel_size, stride, padding, dilation, groups,
                             ws.data_ptr() if ws is not None else None, ws_bytes, _stream()))
    return out


def conv_transpose1d(x: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor | None = None, stride: int = 1,
                     padding: int = 0, output_padding: int = 0, groups: int = 1) -> torch.Tensor:
    _require_cuda(x, kernel)
    if x.dim() != 3 or kernel.dim() != 3:
        raise XnError(1, f"conv_transpose1d expects rank-3 input and kernel, got {list(x.shape)} and {list(kernel.shape)}")
    batch, in_channels, length = x.shape
    k_in_channels, out_channels_per_group, kernel_size = kernel.shape
    out_channels = out_channels_per_group * groups
    if groups < 1 or in_channels % groups:
        raise XnError(1, f"in_channels ({in_channels}) must be divisible by groups ({groups})")
    if k_in_channels != in_channels:
        raise XnError(1, f"kernel in_channels mismatch: expected {in_channels}, got {k_in_channels}")
    _check_bias(bias, out_channels)
    out_length = (length - 1) * stride + kernel_size + output_padding - 2 * padding
    if out_length < 0:
        raise XnError(1, f"padding {padding} leaves no output")
    x, kernel = x.contiguous(), kernel.contiguous()
    out = torch.empty(batch, out_channels, out_length, dtype=x.dtype, device=x.device)
    ws_bytes = lib().xn_mm_conv_transpose1d_workspace_bytes(_dtype_code(x), batch, in_channels, out_channels, length,
                                                            kernel_size, stride, padding, output_padding, groups)
    ws = _conv_workspace(x.device, ws_bytes)
    check(lib().xn_mm_conv_transpose1d(_dtype_code(x), out.data_ptr(), x.data_ptr(), kernel.data_ptr(),
                                       bias.contiguous().data_ptr() if bias is not None else None, batch, in_channels,
                                       out_channels, length, out_length, kernel_size, stride, padding, output_padding,
                                       groups, ws.data_ptr() if ws is not None else None, ws_bytes, _stream()))
    return out


# ---------------------------------------------------------------------------------------------
# Row operations of a decoder step (xn_mm_rms_norm & co.): thin wrappers used by decoder.py and tests.
# ---------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, alpha: torch.Tensor, eps: float) -> torch.Tensor:
    _require_cuda(x, alpha)
    x = x.contiguous()
    out = torch.empty_like(x)
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    check(lib().xn_mm_rms_norm(_dtype_code(x), out.data_ptr(), x.data_ptr(), alpha.data_ptr(), rows, cols, eps, _stream()))
    return out


def softmax(x: torch.Tensor) -> torch.Tensor:
    _require_cuda(x)
    x = x.contiguous()
    out = torch.empty_like(x)
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    check(lib().xn_mm_softmax(_dtype_code(x), out.data_ptr(), x.data_ptr(), rows, cols, _stream()))
    return out


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    _require_cuda(x)
    x = x.contiguous()
    hidden = x.shape[-1] // 2
    rows = x.numel() // x.shape[-1]
    out = torch.empty(*x.shape[:-1], hidden, dtype=x.dtype, device=x.device)
    check(lib().xn_mm_silu_mul(_dtype_code(x), out.data_ptr(), x.data_ptr(), rows, hidden, _stream()))
    return out


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    _require_cuda(a, b)
    out = torch.empty_like(a)
    check(lib().xn_mm_add(_dtype_code(a), out.data_ptr(), a.contiguous().data_ptr(), b.contiguous().data_ptr(), a.numel(), _stream()))
    return out
