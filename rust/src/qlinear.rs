//! Quantized payloads behind `nn::Linear` (xn-core/src/nn/linear.rs:4-71).  UNCOMPILED here.
//!
//! `Linear` keeps its `forward(&self, x) -> Result<Tensor<T, B>>` signature; its `weight` field becomes this
//! enum, so xn-moshi and xn-pocket-tts construct and call their projections unchanged.  The quantized arms hold
//! `Tensor<u8, B>` / `Tensor<f32, B>` storages (`u8` already is a `DType`, xn-core/src/dtype.rs:9) in exactly
//! the byte layout the kernels read (include/xn_mm.h: "q4 tiles", "q8 tiles", row-major e4m3 + per-channel
//! scales), which is also the layout of the quantized-weight checkpoints.
use std::ffi::c_void;

use crate::cuda_mm::{self, check};
use crate::{Backend, Result, Tensor, WithDTypeF};

pub enum LinearWeight<T: WithDTypeF, B: Backend> {
    /// (out_features, in_features) in the model's element type: `matmul_t` + optional bias, as today.
    Dense(Tensor<T, B>),
    /// int4 in 32-element blocks with f32 block scales, packed as q4 tiles; activations are quantized per row
    /// to int8 on the fly and the result is f32-accurate before the final rounding to `T`.
    Q4 { packed: Tensor<u8, B>, out_features: usize, in_features: usize },
    /// the same with one byte per weight (q8 tiles)
    Q8 { packed: Tensor<u8, B>, out_features: usize, in_features: usize },
    /// e4m3 bytes (out_features, in_features) + one f32 scale per output channel; `workspace` holds the
    /// activation pieces of the largest batch the layer serves (xn_mm_linear_fp8_workspace_bytes)
    Fp8 { wq: Tensor<u8, B>, scale: Tensor<f32, B>, workspace: Tensor<u8, B>, variant: i32 },
}

/// The CUDA arms.  `ptr` / `ptr_mut` stand for the cudarc guard dance shown in `cuda_mm::gemm`.
impl<T: WithDTypeF> LinearWeight<T, crate::cuda_backend::Device> {
    /// x: (rows, in_features) contiguous; returns (rows, out_features).
    pub fn forward_2d(&self, x: &Tensor<T, crate::cuda_backend::Device>, rows: usize) -> Result<Tensor<T, crate::cuda_backend::Device>> {
        let dev = x.device().clone();
        let stream = dev.cu_stream() as *mut c_void;
        match self {
            LinearWeight::Dense(w) => x.matmul_t(w),
            LinearWeight::Q4 { packed, out_features, in_features } | LinearWeight::Q8 { packed, out_features, in_features } => {
                let (n, k) = (*out_features, *in_features);
                let xq: Tensor<u8, _> = unsafe { Tensor::alloc_uninit((rows, k).into(), &dev) }?; // int8 bytes
                let xs: Tensor<f32, _> = unsafe { Tensor::alloc_uninit((rows,).into(), &dev) }?;
                let y: Tensor<f32, _> = unsafe { Tensor::alloc_uninit((rows, n).into(), &dev) }?;
                check(unsafe {
                    cuda_mm::xn_mm_quantize_rows_i8(xq.ptr_mut() as *mut i8, xs.ptr_mut(), x.ptr() as *const c_void,
                                                    cuda_mm::dtype_code(T::DTYPE)?, rows, k, stream)
                })?;
                let f = if matches!(self, LinearWeight::Q4 { .. }) { cuda_mm::xn_mm_linear_q4 } else { cuda_mm::xn_mm_linear_q8 };
                check(unsafe {
                    f(y.ptr_mut(), xq.ptr() as *const i8, xs.ptr(), packed.ptr() as *const c_void, rows, n, k,
                      std::ptr::null_mut(), stream)
                })?;
                y.to_dtype::<T>()
            }
            LinearWeight::Fp8 { wq, scale, workspace, variant } => {
                // bf16 activations in, bf16 out (other element types convert around the call)
                let (n, k) = (wq.dims()[0], wq.dims()[1]);
                let xb = x.to_dtype::<half::bf16>()?;
                let y: Tensor<half::bf16, _> = unsafe { Tensor::alloc_uninit((rows, n).into(), &dev) }?;
                check(unsafe {
                    cuda_mm::xn_mm_linear_fp8(y.ptr_mut() as *mut c_void, xb.ptr() as *const c_void, wq.ptr(), scale.ptr(),
                                              rows, n, k, *variant, workspace.ptr_mut() as *mut c_void,
                                              workspace.elem_count(), stream)
                })?;
                y.to_dtype::<T>()
            }
        }
    }
}

/// The extra arm of `VarBuilder::load` (xn-core/src/nn/var_builder.rs:53-58 keeps only F32 / F16 / BF16
/// tensors today): U8 tensors whose name ends in `.q4`, `.q8` or `.fp8`, and the F32 `.fp8_scale` that goes
/// with the last, are kept as stored; `xn_mm.<name>` in the file's `__metadata__` carries the logical
/// `[out_features, in_features]` (the writer is xn_b200/checkpoint.py).
pub fn is_quantized_tensor(name: &str, dtype: safetensors::Dtype) -> bool {
    match dtype {
        safetensors::Dtype::U8 => name.ends_with(".q4") || name.ends_with(".q8") || name.ends_with(".fp8"),
        safetensors::Dtype::F32 => name.ends_with(".fp8_scale"),
        _ => false,
    }
}
