// Shared host/device helpers of the sm_100a matmul engine.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <string>

#include "../../include/xn_mm.h"

namespace xn {

// Thread-local message returned by xn_mm_last_error().
std::string &last_error();
int fail(int code, const char *fmt, ...);

#define XN_CHECK_CUDA(expr)                                                                   \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return ::xn::fail(XN_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                    \
                              cudaGetErrorString(_e), __FILE__, __LINE__);                    \
    } while (0)

#define XN_REQUIRE(cond, ...)                                                                 \
    do {                                                                                      \
        if (!(cond)) return ::xn::fail(XN_ERR_INVALID, __VA_ARGS__);                          \
    } while (0)

inline size_t dtype_size(xn_dtype dt) { return dt == XN_F32 ? 4 : 2; }
inline bool valid_dtype(int dt) { return dt == XN_F32 || dt == XN_F16 || dt == XN_BF16; }
inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int sm_count();
// Programmatic dependent launch for the weight-streaming kernels (on unless XN_MM_PDL=0): a kernel
// may begin, and prefetch weights, while its predecessor in the stream is still draining.
bool pdl_enabled();
// Whether the right-hand operand of the matmul being dispatched on this thread is a static weight (a model
// parameter that no work in flight on the stream writes).  Only then may a weight-streaming kernel fetch it
// before its programmatic-dependent-launch wait, i.e. while the previous kernel in the stream is still
// running.  Backend::gemm's rhs can be any tensor -- the previous kernel's output included -- so xn_mm_gemm
// leaves this false; the Linear entry points, whose weight operand is static by contract, set it.
bool rhs_is_static();
struct StaticRhsScope {
    explicit StaticRhsScope(bool on);
    ~StaticRhsScope();
    bool prev;
};

// NVTX range around a C-ABI entry point (host-side marker for timeline tools), off unless XN_MM_NVTX=1 is set
// when the library is first used.  The NVTX v3 header resolves the tool's injection library at run time: no link
// dependency, and a no-op without a tool attached.
struct ApiRange {
    explicit ApiRange(const char *name);
    ~ApiRange();
    bool on;
};
#define XN_API_RANGE(name) ::xn::ApiRange _xn_api_range(name)

// A per-column bias offered to the next matmul launched on this thread (nn::Linear's bias).  The tiled tensor-memory
// kernel adds it in its epilogue and calls take_fused_col_bias(); a route that cannot leaves it, and the caller
// adds the bias with a launch of its own when `taken` is still false at the end of the scope.
struct ColBiasScope {
    explicit ColBiasScope(const void *bias);
    ~ColBiasScope();
    bool taken() const;
};
const void *take_fused_col_bias();  // the offered bias (null if none); marks it taken

// Raises a kernel's dynamic shared-memory limit once per (kernel, device); later calls with a
// size already covered cost one atomic load.  `slot` is a per-kernel table of 64 ints.
int ensure_dynamic_smem(const void *kernel, int *slot, size_t bytes);
#define XN_ENSURE_SMEM(kern, bytes)                                                           \
    do {                                                                                      \
        static int _slot[64];                                                                 \
        int _rc = ::xn::ensure_dynamic_smem((const void *)(kern), _slot, (bytes));            \
        if (_rc) return _rc;                                                                  \
    } while (0)

// Element widening / narrowing (round to nearest even), the same conversions crate `half`
// performs for the reference (xn-core/src/dtype.rs:92-131).
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Streaming 128-bit global load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Dispatch a functor template over the three element types.
#define XN_DISPATCH_DTYPE(dt, T, ...)                                                         \
    do {                                                                                      \
        if ((dt) == XN_F32) { using T = float; __VA_ARGS__; }                                 \
        else if ((dt) == XN_F16) { using T = __half; __VA_ARGS__; }                           \
        else { using T = __nv_bfloat16; __VA_ARGS__; }                                        \
    } while (0)

// ---- kernel launchers implemented in the other translation units ----
int launch_gemm_generic(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n,
                        size_t k, size_t lhs_b, size_t lhs_b_stride, size_t rhs_b_stride,
                        size_t dst_cs, size_t dst_rs, size_t lhs_cs, size_t lhs_rs, size_t rhs_cs,
                        size_t rhs_rs, cudaStream_t st);

bool gemv_h16_single_chunk(size_t m, size_t k);
int launch_gemv_h16(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k, size_t dst_rs,
                    size_t lhs_rs, size_t rhs_cs, cudaStream_t st);
int launch_gemv_f32x3(float *dst, const float *lhs, const float *rhs, size_t m, size_t n, size_t k, size_t dst_rs,
                      size_t lhs_rs, size_t rhs_cs, cudaStream_t st);
int launch_gemv_dense(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k,
                      size_t lhs_b, size_t lhs_b_stride, size_t rhs_b_stride, size_t dst_rs, size_t lhs_rs, size_t rhs_cs,
                      cudaStream_t st);
int launch_gemm_tn_16bit(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k,
                         size_t lda, size_t ldb, size_t ldd, size_t batch, size_t lhs_bs, size_t rhs_bs, cudaStream_t st,
                         int causal = 0, int causal_off = 0);
int launch_gemm_kn_16bit(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k,
                         size_t lda, size_t ldb, size_t ldd, size_t batch, size_t lhs_bs, size_t rhs_bs, cudaStream_t st,
                         int causal = 0, int causal_off = 0);
int launch_gemm_tn_16bit_shared_lhs(xn_dtype dt, void *dst, const void *lhs, const void *rhs, const void *row_bias, size_t m,
                                    size_t n, size_t k, size_t lda, size_t ldb, size_t ldd, size_t batch, size_t rhs_bs,
                                    size_t dst_bs, cudaStream_t st);
int launch_gemm_tn_tf32_shared_lhs(float *dst, const float *lhs, const float *rhs, const float *row_bias, size_t m, size_t n,
                                   size_t k, size_t lda, size_t ldb, size_t ldd, size_t batch, size_t rhs_bs, size_t dst_bs,
                                   cudaStream_t st);
int launch_gemm_tn_tf32_splitk(float *partials, const float *lhs, const float *rhs, size_t m, size_t n, size_t kchunk,
                               size_t splits, size_t lda, size_t ldb, cudaStream_t st);
int launch_gemm_tn_tf32(float *dst, const float *lhs, const float *rhs, size_t m, size_t n, size_t k, size_t ldd,
                        cudaStream_t st);
// int8 x int8 -> int32 block sums on kind::i8 tensor-memory MMAs, scaled per 32-block in f32 (q4 / q8 weights, many rows)
int launch_gemm_q8_block(float *y, size_t ldy, const int8_t *xq, const float *x_scale, const int8_t *w8, const float *w_scale,
                         size_t m, size_t n, size_t n_pad, size_t k, cudaStream_t st);
// fused causal attention over a block of query rows (prefill), head_dim 128, 16-bit elements
int launch_attention_prefill(xn_dtype dt, void *out, size_t ldo, const void *q, const void *k, const void *v, size_t ld,
                             size_t head_stride, size_t heads, size_t t_rows, size_t ctx, float scale, cudaStream_t st);
// runtime.cu: library-owned scratch per (device, stream) and the device status word
struct SkinnyScratch { float *partials = nullptr; size_t partial_bytes = 0; unsigned *counters = nullptr; size_t ncounters = 0; };
int skinny_scratch(cudaStream_t st, size_t partial_bytes, size_t ncounters, SkinnyScratch *out);
int library_scratch(cudaStream_t st, size_t bytes, void **out);
struct WaitCtx;
// Fills the bound and the status-word pointer every kernel with device-side waits takes; fails with
// XN_ERR_DEVICE when an earlier launch on the current device has reported a wait that ran out.
int wait_ctx(WaitCtx *out);
// While alive on this thread, wait_ctx() does not allocate the status word if the device has none yet.
struct NoAllocScope {
    NoAllocScope();
    ~NoAllocScope();
    bool prev;
};
// f32 matmul with many rows on the kind::tf32 tensor-memory kernel (three tf32 pieces per operand); any strides
bool gemm_f32_tc_fits(size_t m, size_t n, size_t k);
int launch_gemm_f32_tc(float *dst, const float *lhs, const float *rhs, size_t m, size_t n, size_t k, size_t dst_rs,
                       size_t lhs_cs, size_t lhs_rs, size_t rhs_cs, size_t rhs_rs, cudaStream_t st);

}  // namespace xn
