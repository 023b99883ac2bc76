//! FFI binding of `libxn_mm.so`, the sm_100a matmul engine, for xn-core's CUDA backend.
//!
//! UNCOMPILED: this file was written on a machine without a Rust toolchain.  It declares every entry point of
//! `include/xn_mm.h` (a test in the engine's repository diffs the names and argument counts against the header),
//! maps the status codes onto `crate::Error`, and carries the replacement body of `Backend::gemm` for
//! `impl crate::Backend for Device` (xn-core/src/cuda_backend.rs:787-865).  Drop it into `xn-core/src/` as
//! `cuda_mm.rs`, add `mod cuda_mm;` next to `mod cuda_backend;` and call `cuda_mm::gemm` from the trait method.
#![allow(clippy::too_many_arguments)]
use std::ffi::{c_char, c_int, c_uint, c_void, CStr};

use crate::{DType, Result, WithDType};

/// Element types the engine's GEMM accepts: the subset of `DType` the reference's CUDA `gemm` handles
/// (xn-core/src/cuda_backend.rs:803-862).
#[repr(C)]
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum XnDtype {
    F32 = 0,
    F16 = 1,
    BF16 = 2,
}

/// `xn_status` of the C ABI.
pub const XN_OK: c_int = 0;
pub const XN_ERR_INVALID: c_int = 1;
pub const XN_ERR_UNSUPPORTED: c_int = 2;
pub const XN_ERR_CUDA: c_int = 3;
pub const XN_ERR_WORKSPACE: c_int = 4;
pub const XN_ERR_DEVICE: c_int = 5;

#[link(name = "xn_mm")]
extern "C" {
    pub fn xn_mm_last_error() -> *const c_char;
    pub fn xn_mm_abi_version() -> c_int;
    pub fn xn_mm_device_status(timeouts_out: *mut c_uint) -> c_int;
    pub fn xn_mm_clear_device_status() -> c_int;
    pub fn xn_mm_selftest_wait_timeout(limit_ns: u64, stream: *mut c_void) -> c_int;
    pub fn xn_mm_release_scratch(stream: *mut c_void, all_streams: c_int) -> c_int;
    pub fn xn_mm_gemm(dtype: XnDtype, dst: *mut c_void, lhs: *const c_void, lhs_off: usize,
        rhs: *const c_void, rhs_off: usize, m: usize, n: usize, k: usize, lhs_b: usize, lhs_b_stride: usize,
        rhs_b_stride: usize, dst_cs: usize, dst_rs: usize, lhs_cs: usize, lhs_rs: usize, rhs_cs: usize,
        rhs_rs: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_attention_prefill(dtype: XnDtype, out: *mut c_void, ldo: usize, q: *const c_void,
        k: *const c_void, v: *const c_void, ld: usize, head_stride: usize, heads: usize, head_dim: usize,
        t_rows: usize, context: usize, scale: f32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_gemm_causal(mode: c_int, causal_offset: usize, dtype: XnDtype, dst: *mut c_void,
        lhs: *const c_void, lhs_off: usize, rhs: *const c_void, rhs_off: usize, m: usize, n: usize, k: usize,
        lhs_b: usize, lhs_b_stride: usize, rhs_b_stride: usize, dst_cs: usize, dst_rs: usize, lhs_cs: usize,
        lhs_rs: usize, rhs_cs: usize, rhs_rs: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear(dtype: XnDtype, y: *mut c_void, x: *const c_void, weight: *const c_void,
        bias_or_null: *const c_void, m: usize, n: usize, k: usize, ldx: usize, ldw: usize, ldy: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_matmul_plan(lhs_rank: usize, lhs_dims: *const usize, lhs_strides: *const usize,
        rhs_rank: usize, rhs_dims: *const usize, rhs_strides: *const usize, rhs_t: c_int,
        dst_capacity: usize, out12: *mut usize) -> c_int;
    pub fn xn_mm_q4_packed_bytes(n: usize, k: usize) -> usize;
    pub fn xn_mm_quantize_weights_q4(wq_packed: *mut c_void, w: *const c_void, dtype: XnDtype, n: usize,
        k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_pack_q4_host(wq_packed: *mut u8, q: *const i8, scales: *const f32, n: usize,
        k: usize) -> c_int;
    pub fn xn_mm_unpack_q4_host(q: *mut i8, scales: *mut f32, wq_packed: *const u8, n: usize,
        k: usize) -> c_int;
    pub fn xn_mm_quantize_rows_i8(xq: *mut i8, x_scale: *mut f32, x: *const c_void, dtype: XnDtype, m: usize,
        k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_q4(y: *mut f32, xq: *const i8, x_scale: *const f32, wq_packed: *const c_void,
        m: usize, n: usize, k: usize, partials: *mut i32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_q4_host_workspace_bytes(m: usize, n: usize, k: usize) -> usize;
    pub fn xn_mm_linear_q4_host(y_host: *mut f32, x_host: *const f32, wq_packed: *const c_void, m: usize,
        n: usize, k: usize, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_q8_packed_bytes(n: usize, k: usize) -> usize;
    pub fn xn_mm_quantize_weights_q8(wq_packed: *mut c_void, w: *const c_void, dtype: XnDtype, n: usize,
        k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_pack_q8_host(wq_packed: *mut u8, q: *const i8, scales: *const f32, n: usize,
        k: usize) -> c_int;
    pub fn xn_mm_unpack_q8_host(q: *mut i8, scales: *mut f32, wq_packed: *const u8, n: usize,
        k: usize) -> c_int;
    pub fn xn_mm_linear_q8(y: *mut f32, xq: *const i8, x_scale: *const f32, wq_packed: *const c_void,
        m: usize, n: usize, k: usize, partials: *mut i32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_quantize_weights_fp8(wq: *mut u8, w_scale: *mut f32, w: *const c_void, dtype: XnDtype,
        n: usize, k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_split_rows_e4m3(x_hi: *mut u8, x_lo: *mut u8, x_scale: *mut f32, x: *const c_void,
        dtype: XnDtype, m: usize, k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_fp8_pieces(y_bf16: *mut c_void, x_hi: *const u8, x_lo: *const u8,
        x_scale: *const f32, wq: *const u8, w_scale: *const f32, m: usize, n: usize, k: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_fp8_pieces_scatter(y_dsts: *const *mut c_void, num_dst: usize, ldy: usize,
        col_offset: usize, x_hi: *const u8, x_lo: *const u8, x_scale: *const f32, wq: *const u8,
        w_scale: *const f32, m: usize, n: usize, k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_fp8_pieces_multicast(y_multicast: *mut c_void, ldy: usize, col_offset: usize,
        x_hi: *const u8, x_lo: *const u8, x_scale: *const f32, wq: *const u8, w_scale: *const f32, m: usize,
        n: usize, k: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_fp8_workspace_bytes(m: usize, k: usize) -> usize;
    pub fn xn_mm_linear_fp8(y_bf16: *mut c_void, x_bf16: *const c_void, wq: *const u8, w_scale: *const f32,
        m: usize, n: usize, k: usize, variant: c_int, workspace: *mut c_void, workspace_bytes: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_rms_norm(dtype: XnDtype, dst: *mut c_void, src: *const c_void, alpha: *const c_void,
        rows: usize, cols: usize, eps: f32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_softmax(dtype: XnDtype, dst: *mut c_void, src: *const c_void, rows: usize, cols: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_silu_mul(dtype: XnDtype, dst: *mut c_void, src: *const c_void, rows: usize, hidden: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_add(dtype: XnDtype, dst: *mut c_void, a: *const c_void, b: *const c_void, len: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_add_bias(dtype: XnDtype, dst: *mut c_void, src: *const c_void, bias: *const c_void,
        rows: usize, cols: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_kv_append(dtype: XnDtype, cache: *mut c_void, src: *const c_void, src_batch_stride: usize,
        index: *const i64, batch: usize, heads: usize, context: usize, head_dim: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_softmax_causal(dtype: XnDtype, dst: *mut c_void, src: *const c_void, batch: usize,
        t_rows: usize, context: usize, scale: f32, zero_fill_all: c_int, stream: *mut c_void) -> c_int;
    pub fn xn_mm_scatter_columns(dsts: *const *mut c_void, num_dst: usize, multicast: c_int,
        ldy_bytes: usize, col_offset_bytes: usize, src: *const c_void, m: usize, row_bytes: usize,
        groups: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_rms_norm_split_e4m3(x_hi: *mut u8, x_lo: *mut u8, x_scale: *mut f32,
        dst_or_null: *mut c_void, src: *const c_void, alpha: *const c_void, dtype: XnDtype, rows: usize,
        cols: usize, eps: f32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_silu_mul_split_e4m3(x_hi: *mut u8, x_lo: *mut u8, x_scale: *mut f32, src: *const c_void,
        dtype: XnDtype, rows: usize, hidden: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_add_rms_norm_split_e4m3(x_hi: *mut u8, x_lo: *mut u8, x_scale: *mut f32,
        sum_out: *mut c_void, a: *const c_void, b: *const c_void, alpha: *const c_void, dtype: XnDtype,
        rows: usize, cols: usize, eps: f32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_decode_attention(out_bf16: *mut c_void, q_bf16: *const c_void, q_batch_stride: usize,
        k_cache_bf16: *const c_void, v_cache_bf16: *const c_void, mask_or_null: *const f32, batch: usize,
        heads: usize, context: usize, head_dim: usize, scale: f32, stream: *mut c_void) -> c_int;
    pub fn xn_mm_decode_attention_workspace_bytes(batch: usize, heads: usize, context: usize) -> usize;
    pub fn xn_mm_decode_attention_split(out_bf16: *mut c_void, q_bf16: *const c_void, q_batch_stride: usize,
        k_cache_bf16: *const c_void, v_cache_bf16: *const c_void, mask_or_null: *const f32, batch: usize,
        heads: usize, context: usize, head_dim: usize, scale: f32, workspace: *mut c_void,
        workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_decode_attention_split_e4m3(x_hi: *mut u8, x_lo: *mut u8, x_scale: *mut f32,
        out_bf16: *mut c_void, q_bf16: *const c_void, q_batch_stride: usize, k_cache_bf16: *const c_void,
        v_cache_bf16: *const c_void, mask_or_null: *const f32, batch: usize, heads: usize, context: usize,
        head_dim: usize, scale: f32, workspace: *mut c_void, workspace_bytes: usize,
        stream: *mut c_void) -> c_int;
    pub fn xn_mm_decode_attention_append_workspace_bytes(batch: usize, heads: usize, context: usize) -> usize;
    pub fn xn_mm_decode_attention_append_e4m3(x_hi: *mut u8, x_lo: *mut u8, x_scale: *mut f32,
        out_bf16: *mut c_void, q_bf16: *const c_void, k_new_bf16: *const c_void, v_new_bf16: *const c_void,
        qkv_batch_stride: usize, k_cache_bf16: *mut c_void, v_cache_bf16: *mut c_void, index: *const i64,
        mask_or_null: *const f32, batch: usize, heads: usize, context: usize, head_dim: usize, scale: f32,
        merge: c_int, workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_kv_append2(dtype: XnDtype, k_cache: *mut c_void, v_cache: *mut c_void, k_src: *const c_void,
        v_src: *const c_void, src_batch_stride: usize, index: *const i64, batch: usize, heads: usize,
        context: usize, head_dim: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_linear_fp8_noalloc_max_elems() -> usize;
    pub fn xn_mm_linear_fp8_noalloc(y_bf16: *mut c_void, x_bf16: *const c_void, wq: *const u8,
        w_scale: *const f32, m: usize, n: usize, k: usize, variant: c_int, stream: *mut c_void) -> c_int;
    pub fn xn_mm_conv1d_workspace_bytes(dtype: XnDtype, batch: usize, in_channels: usize,
        out_channels: usize, length: usize, kernel_size: usize, stride: usize, padding: usize,
        dilation: usize, groups: usize) -> usize;
    pub fn xn_mm_conv1d(dtype: XnDtype, dst: *mut c_void, src: *const c_void, kernel: *const c_void,
        bias_or_null: *const c_void, batch: usize, in_channels: usize, out_channels: usize, length: usize,
        out_length: usize, kernel_size: usize, stride: usize, padding: usize, dilation: usize, groups: usize,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn xn_mm_conv_transpose1d_workspace_bytes(dtype: XnDtype, batch: usize, in_channels: usize,
        out_channels: usize, length: usize, kernel_size: usize, stride: usize, padding: usize,
        output_padding: usize, groups: usize) -> usize;
    pub fn xn_mm_conv_transpose1d(dtype: XnDtype, dst: *mut c_void, src: *const c_void,
        kernel: *const c_void, bias_or_null: *const c_void, batch: usize, in_channels: usize,
        out_channels: usize, length: usize, out_length: usize, kernel_size: usize, stride: usize,
        padding: usize, output_padding: usize, groups: usize, workspace: *mut c_void, workspace_bytes: usize,
        stream: *mut c_void) -> c_int;
}

/// Turns a status code into the error type `bail!()` produces (xn-core/src/error.rs:127-138), with the
/// library's message for the calling thread.
pub fn check(code: c_int) -> Result<()> {
    if code == XN_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(xn_mm_last_error()) }.to_string_lossy().into_owned();
    Err(crate::Error::Msg(format!("xn_mm error {code}: {msg}")).bt())
}

pub fn dtype_code(dt: DType) -> Result<XnDtype> {
    match dt {
        DType::F32 => Ok(XnDtype::F32),
        DType::F16 => Ok(XnDtype::F16),
        DType::BF16 => Ok(XnDtype::BF16),
        // the reference refuses the same element types at the same point (cuda_backend.rs:862)
        dt => crate::bail!("GEMM not supported for dtype {dt:?}"),
    }
}

/// Body of `Backend::gemm` for the CUDA device (trait method: xn-core/src/backend.rs:135-148).  Same twelve
/// arguments; strides and offsets in elements; `dst` is overwritten; asynchronous on the device's stream.
///
/// `Storage<T>` is `cuda_backend::Storage<T> { data: CudaSlice<T>, device: Device }` and `Device` owns the
/// one stream the backend runs on (cuda_backend.rs:35-60, 168-171).
pub fn gemm<T: WithDType>(
    dst: &mut crate::cuda_backend::Storage<T>,
    (lhs, lhs_o): (&crate::cuda_backend::Storage<T>, usize),
    (rhs, rhs_o): (&crate::cuda_backend::Storage<T>, usize),
    m: usize,
    n: usize,
    k: usize,
    lhs_b: usize,
    lhs_b_stride: usize,
    rhs_b_stride: usize,
    (dst_cs, dst_rs): (usize, usize),
    (lhs_cs, lhs_rs): (usize, usize),
    (rhs_cs, rhs_rs): (usize, usize),
) -> Result<()> {
    use cudarc::driver::{DevicePtr, DevicePtrMut};
    let dt = dtype_code(T::DTYPE)?;
    let stream = dst.device.stream.clone();
    let cu_stream = stream.cu_stream() as *mut c_void;
    // cudarc's event-tracking guards, as the cuBLAS path takes them (cuda_backend.rs:2103-2106)
    let (d, _g0) = dst.data.device_ptr_mut(&stream);
    let (l, _g1) = lhs.data.device_ptr(&stream);
    let (r, _g2) = rhs.data.device_ptr(&stream);
    check(unsafe {
        xn_mm_gemm(
            dt, d as *mut c_void, l as *const c_void, lhs_o, r as *const c_void, rhs_o, m, n, k, lhs_b, lhs_b_stride,
            rhs_b_stride, dst_cs, dst_rs, lhs_cs, lhs_rs, rhs_cs, rhs_rs, cu_stream,
        )
    })
}

/// `Linear::forward` on a static weight (xn-core/src/nn/linear.rs:56-66): the same product through the entry
/// point that may prefetch the weight ahead of the stream order, bias fused.  `x` is `[m, k]` contiguous,
/// `weight` `[n, k]`, `bias` `[n]`.
pub fn linear<T: WithDType>(
    y: &mut crate::cuda_backend::Storage<T>,
    x: &crate::cuda_backend::Storage<T>,
    weight: &crate::cuda_backend::Storage<T>,
    bias: Option<&crate::cuda_backend::Storage<T>>,
    m: usize,
    n: usize,
    k: usize,
) -> Result<()> {
    use cudarc::driver::{DevicePtr, DevicePtrMut};
    let dt = dtype_code(T::DTYPE)?;
    let stream = y.device.stream.clone();
    let (yp, _g0) = y.data.device_ptr_mut(&stream);
    let (xp, _g1) = x.data.device_ptr(&stream);
    let (wp, _g2) = weight.data.device_ptr(&stream);
    let guard = bias.map(|b| b.data.device_ptr(&stream));
    let bp = guard.as_ref().map(|(p, _)| *p as *const c_void).unwrap_or(std::ptr::null());
    check(unsafe {
        xn_mm_linear(dt, yp as *mut c_void, xp as *const c_void, wp as *const c_void, bp, m, n, k, k, k, n,
                     stream.cu_stream() as *mut c_void)
    })
}

/// Polls the current device's status word at a synchronisation point of the caller: `Err` once any device-side
/// wait of this library has run out (see `xn_mm_device_status` in the header).
pub fn device_status() -> Result<()> {
    let mut n: c_uint = 0;
    check(unsafe { xn_mm_device_status(&mut n) })
}
