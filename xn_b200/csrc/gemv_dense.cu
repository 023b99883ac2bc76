// Dense small-m matmul for the `matmul_t` form (lhs [m,k] and rhs [n,k] both k-contiguous, m <= 16):
// the decode-time Linear::forward of an unquantized model and the f32 linear of the CPU-runnable
// benchmark configuration.  Reference path: cublasGemmStridedBatchedEx (xn-core/src/cuda_backend.rs:
// 2109-2133) with f32 accumulation; this kernel keeps exact f32 products and f32 accumulation for all
// three element types (no TF32), so it is the one that meets the 1e-4 bound for f32.
//
// HBM-bound by the rhs (the weights): each warp streams NR = 4 rhs rows with 128-bit loads while the
// lhs rows sit in shared memory as f32; one shared-memory read of the lhs serves the 4 rhs rows, which
// keeps shared-memory traffic at 4x (not 16x) the global traffic for m = 16.  k is walked in chunks
// of KC elements so that any k fits.  Batched (lhs_b) through blockIdx.y.
#include "common.cuh"

namespace xn {
namespace {

constexpr int KC = 1024;   // lhs elements per row staged at a time
constexpr int NR = 4;      // rhs rows per warp
constexpr int WARPS = 8;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void unpack(const uint4 &v, float (&f)[Vec<T>::N]);
template <> __device__ __forceinline__ void unpack<float>(const uint4 &v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__half>(const uint4 &v, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4 &v, float (&f)[8]) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

template <typename T, int MT>
__global__ void __launch_bounds__(WARPS * 32)
gemv_dense_kernel(T *__restrict__ dst, const T *__restrict__ lhs, const T *__restrict__ rhs, int m, size_t n, size_t k,
                  size_t lhs_b, size_t lhs_b_stride, size_t rhs_b_stride, size_t dst_rs, size_t lhs_rs, size_t rhs_cs) {
    constexpr int V = Vec<T>::N;
    extern __shared__ __align__(16) float sx[];  // [MT][KC]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t j0 = ((size_t)blockIdx.x * WARPS + warp) * NR;

    for (size_t b = blockIdx.y; b < lhs_b; b += gridDim.y) {
        const T *A = lhs + b * lhs_b_stride;
        const T *B = rhs + b * rhs_b_stride;
        float acc[NR][MT];
#pragma unroll
        for (int r = 0; r < NR; ++r)
#pragma unroll
            for (int i = 0; i < MT; ++i) acc[r][i] = 0.0f;
        const T *rows[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) rows[r] = B + min(j0 + r, n - 1) * rhs_cs;  // clamped: results of extra rows are dropped

        for (size_t k0 = 0; k0 < k; k0 += KC) {
            const int kc = (int)min((size_t)KC, k - k0);
            __syncthreads();
            for (int idx = threadIdx.x; idx < MT * (KC / V); idx += WARPS * 32) {
                const int row = idx / (KC / V), c = (idx % (KC / V)) * V;
                float f[V];
#pragma unroll
                for (int e = 0; e < V; ++e) f[e] = 0.0f;
                if (row < m && c < kc) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(A + (size_t)row * lhs_rs + k0 + c));
                    unpack<T>(v, f);
                }
#pragma unroll
                for (int e = 0; e < V; e += 4)
                    *reinterpret_cast<float4 *>(sx + row * KC + c + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
            }
            __syncthreads();
            if (j0 < n) {
                for (int c = lane * V; c < kc; c += 32 * V) {
                    float w[NR][V];
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const uint4 v = ldg_stream(rows[r] + k0 + c);
                        unpack<T>(v, w[r]);
                    }
#pragma unroll
                    for (int i = 0; i < MT; ++i) {
                        float x[V];
#pragma unroll
                        for (int e = 0; e < V; e += 4) {
                            const float4 t = *reinterpret_cast<const float4 *>(sx + i * KC + c + e);
                            x[e] = t.x; x[e + 1] = t.y; x[e + 2] = t.z; x[e + 3] = t.w;
                        }
#pragma unroll
                        for (int r = 0; r < NR; ++r)
#pragma unroll
                            for (int e = 0; e < V; ++e) acc[r][i] = fmaf(x[e], w[r][e], acc[r][i]);
                    }
                }
            }
        }
        if (j0 < n) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    float v = acc[r][i];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0 && j0 + r < n && i < m) dst[b * (size_t)m * n + (size_t)i * dst_rs + j0 + r] = from_f32<T>(v);
                }
        }
    }
}

template <typename T, int MT>
int launch_mt(T *dst, const T *lhs, const T *rhs, int m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
              size_t rhs_b_stride, size_t dst_rs, size_t lhs_rs, size_t rhs_cs, cudaStream_t st) {
    const size_t blocks = (n + WARPS * NR - 1) / (WARPS * NR);
    if (blocks > 0x7fffffffull) return fail(XN_ERR_UNSUPPORTED, "gemv: n=%zu too large", n);
    const size_t smem = (size_t)MT * KC * sizeof(float);
    auto kern = gemv_dense_kernel<T, MT>;
    XN_ENSURE_SMEM(kern, smem);
    dim3 grid((unsigned)blocks, (unsigned)(lhs_b < 65535 ? lhs_b : 65535));
    kern<<<grid, WARPS * 32, smem, st>>>(dst, lhs, rhs, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs);
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

template <typename T>
int launch_t(void *dst, const void *lhs, const void *rhs, int m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
             size_t rhs_b_stride, size_t dst_rs, size_t lhs_rs, size_t rhs_cs, cudaStream_t st) {
    T *d = (T *)dst;
    const T *l = (const T *)lhs, *r = (const T *)rhs;
    if (m <= 1) return launch_mt<T, 1>(d, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
    if (m <= 2) return launch_mt<T, 2>(d, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
    if (m <= 4) return launch_mt<T, 4>(d, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
    if (m <= 8) return launch_mt<T, 8>(d, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
    return launch_mt<T, 16>(d, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
}

}  // namespace

// Caller guarantees: m <= 16, lhs_cs == rhs_rs == dst_cs == 1, k and all pitches / batch strides multiples of
// the 128-bit vector length, 16-byte aligned bases.
int launch_gemv_dense(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k,
                      size_t lhs_b, size_t lhs_b_stride, size_t rhs_b_stride, size_t dst_rs, size_t lhs_rs, size_t rhs_cs,
                      cudaStream_t st) {
    if (dt == XN_F32)
        return launch_t<float>(dst, lhs, rhs, (int)m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
    if (dt == XN_F16)
        return launch_t<__half>(dst, lhs, rhs, (int)m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
    return launch_t<__nv_bfloat16>(dst, lhs, rhs, (int)m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs, st);
}

}  // namespace xn
