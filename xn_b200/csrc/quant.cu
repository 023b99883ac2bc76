// Operand quantizers: int8 rows, int4 block tiles, fp8-e4m3 per channel, e4m3 activation pieces.
// None of these has a counterpart in the reference (its DType is {F16,BF16,F32,I64,U8},
// xn-core/src/dtype.rs:4-10); the arithmetic is the one documented in include/xn_mm.h and every
// result is bit-identical to the CPU restatement used by the tests (IEEE division and
// round-half-even throughout, no fast-math).
#include "common.cuh"

namespace xn {
namespace {

__device__ __forceinline__ float block_max(float v, float *red) {
    v = warp_max(v);
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
    if (w == 0) {
        r = warp_max(r);
        if (lane == 0) red[0] = r;
    }
    __syncthreads();
    r = red[0];
    __syncthreads();
    return r;
}

// One CTA per row.  scale = max|x| / 127, q = clamp(rint(x / scale)).
template <typename T>
__global__ void quantize_rows_i8_kernel(int8_t *__restrict__ xq, float *__restrict__ x_scale,
                                        const T *__restrict__ x, size_t k) {
    __shared__ float red[32];
    const T *row = x + (size_t)blockIdx.x * k;
    float amax = 0.0f;
    for (size_t p = threadIdx.x; p < k; p += blockDim.x) amax = fmaxf(amax, fabsf(to_f32(row[p])));
    amax = block_max(amax, red);
    float scale = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) x_scale[blockIdx.x] = scale;
    for (size_t p = threadIdx.x; p < k; p += blockDim.x) {
        float v = 0.0f;
        if (scale != 0.0f) v = rintf(__fdiv_rn(to_f32(row[p]), scale));
        v = fminf(fmaxf(v, -127.0f), 127.0f);
        xq[(size_t)blockIdx.x * k + p] = (int8_t)v;
    }
}

// One warp per (row, 32-block): lane e owns element e of the block.
// Output layout: see "q4 tiles" in include/xn_mm.h.
template <typename T>
__global__ void quantize_weights_q4_kernel(uint8_t *__restrict__ packed, const T *__restrict__ w, size_t n,
                                           size_t n_pad, size_t k) {
    const size_t nblk = k / 32;
    const size_t warp = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (warp >= n_pad * nblk) return;
    const int e = threadIdx.x & 31;
    const size_t r = warp / nblk, blk = warp % nblk;
    float v = (r < n) ? to_f32(w[r * k + blk * 32 + e]) : 0.0f;
    float amax = warp_max(fabsf(v));
    float scale = __fdiv_rn(amax, 7.0f);
    float qf = 0.0f;
    if (scale != 0.0f) qf = rintf(__fdiv_rn(v, scale));
    qf = fminf(fmaxf(qf, -7.0f), 7.0f);
    unsigned nib = (unsigned)((int)qf) & 0xFu;
    // byte (t,i): low nibble from lane 4t+i, high nibble from lane 16+4t+i
    unsigned hi = __shfl_down_sync(0xffffffffu, nib, 16);
    unsigned byte = nib | (hi << 4);  // meaningful on lanes 0..15
    unsigned b1 = __shfl_down_sync(0xffffffffu, byte, 1);
    unsigned b2 = __shfl_down_sync(0xffffffffu, byte, 2);
    unsigned b3 = __shfl_down_sync(0xffffffffu, byte, 3);
    const size_t kt = k / 128;
    const size_t tile = (r / 16) * kt + blk / 4;
    const size_t rr = r % 16, h = rr / 8, g = rr % 8, j = blk % 4;
    if (e < 16 && (e & 3) == 0) {
        unsigned t = e >> 2;
        unsigned word = byte | (b1 << 8) | (b2 << 16) | (b3 << 24);
        *reinterpret_cast<unsigned *>(packed + tile * 1280 + (32 * h + 4 * g + t) * 16 + j * 4) = word;
    }
    if (e == 0) reinterpret_cast<float *>(packed + tile * 1280 + 1024)[(4 * g + j) * 2 + h] = scale;
}

// int8 block tiles ("q8 tiles", include/xn_mm.h): one warp per (row, 32-block), lane e owns element e.
template <typename T>
__global__ void quantize_weights_q8_kernel(uint8_t *__restrict__ packed, const T *__restrict__ w, size_t n,
                                           size_t n_pad, size_t k) {
    const size_t nblk = k / 32;
    const size_t warp = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (warp >= n_pad * nblk) return;
    const int e = threadIdx.x & 31;
    const size_t r = warp / nblk, blk = warp % nblk;
    float v = (r < n) ? to_f32(w[r * k + blk * 32 + e]) : 0.0f;
    float amax = warp_max(fabsf(v));
    float scale = __fdiv_rn(amax, 127.0f);
    float qf = 0.0f;
    if (scale != 0.0f) qf = rintf(__fdiv_rn(v, scale));
    qf = fminf(fmaxf(qf, -127.0f), 127.0f);
    const size_t tile = (r / 16) * (k / 128) + blk / 4;
    const size_t rr = r % 16, h = rr / 8, g = rr % 8, j = blk % 4;
    const size_t t = (e % 16) / 4, i = e % 4, hi = e / 16;
    packed[tile * 2304 + j * 512 + (4 * g + t) * 16 + (h + 2 * hi) * 4 + i] = (uint8_t)(int8_t)qf;
    if (e == 0) reinterpret_cast<float *>(packed + tile * 2304 + 2048)[(4 * g + j) * 2 + h] = scale;
}

// One CTA per output channel.  scale = max|w| / 448, q = e4m3(w / scale).
template <typename T>
__global__ void quantize_weights_fp8_kernel(uint8_t *__restrict__ wq, float *__restrict__ w_scale,
                                            const T *__restrict__ w, size_t k) {
    __shared__ float red[32];
    const T *row = w + (size_t)blockIdx.x * k;
    float amax = 0.0f;
    for (size_t p = threadIdx.x; p < k; p += blockDim.x) amax = fmaxf(amax, fabsf(to_f32(row[p])));
    amax = block_max(amax, red);
    float scale = __fdiv_rn(amax, 448.0f);
    if (threadIdx.x == 0) w_scale[blockIdx.x] = scale;
    for (size_t p = threadIdx.x; p < k; p += blockDim.x) {
        uint8_t q = 0;
        if (scale != 0.0f)
            q = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(to_f32(row[p]), scale), __NV_SATFINITE, __NV_E4M3);
        wq[(size_t)blockIdx.x * k + p] = q;
    }
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}

// One CTA per activation row.  s = the power of two with max|x|/s in (224, 448];
// hi = e4m3(x/s), lo = e4m3(x/s - hi).  x_lo may be null (hi only).
template <typename T>
__global__ void split_rows_e4m3_kernel(uint8_t *__restrict__ x_hi, uint8_t *__restrict__ x_lo,
                                       float *__restrict__ x_scale, const T *__restrict__ x, size_t k) {
    __shared__ float red[32];
    const T *row = x + (size_t)blockIdx.x * k;
    float amax = 0.0f;
    for (size_t p = threadIdx.x; p < k; p += blockDim.x) amax = fmaxf(amax, fabsf(to_f32(row[p])));
    amax = block_max(amax, red);
    float s = 1.0f;
    if (amax != 0.0f && isfinite(amax)) {
        int e;
        float f = frexpf(amax, &e);
        s = ldexpf(1.0f, f <= 0.875f ? e - 9 : e - 8);
    }
    if (threadIdx.x == 0) x_scale[blockIdx.x] = s;
    for (size_t p = threadIdx.x; p < k; p += blockDim.x) {
        float v = __fdiv_rn(to_f32(row[p]), s);
        uint8_t h = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
        x_hi[(size_t)blockIdx.x * k + p] = h;
        if (x_lo) {
            float r = v - e4m3_to_f32(h);
            x_lo[(size_t)blockIdx.x * k + p] = (uint8_t)__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
        }
    }
}

// Fast path of the split for 16-bit rows: 256 threads per row, each holds up to VPT 8-element vectors of
// the row in registers between the maximum and the rounding pass (one read of x), 8-byte stores.
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
split_rows_e4m3_vec_kernel(uint8_t *__restrict__ x_hi, uint8_t *__restrict__ x_lo, float *__restrict__ x_scale,
                           const T *__restrict__ x, size_t k) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + row * k);
    const int nvec = (int)(k / 8);
    uint4 v[VPT];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = i * 256 + threadIdx.x;
        v[i] = idx < nvec ? __ldg(src + idx) : make_uint4(0, 0, 0, 0);
        const T *e = reinterpret_cast<const T *>(&v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(to_f32(e[j])));
    }
    amax = block_max(amax, red);
    float s = 1.0f;
    if (amax != 0.0f && isfinite(amax)) {
        int ex;
        float f = frexpf(amax, &ex);
        s = ldexpf(1.0f, f <= 0.875f ? ex - 9 : ex - 8);
    }
    if (threadIdx.x == 0) x_scale[row] = s;
    const float inv = 1.0f / s;  // exact: s is a power of two
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = i * 256 + threadIdx.x;
        if (idx >= nvec) continue;
        const T *e = reinterpret_cast<const T *>(&v[i]);
        uint8_t h[8], l[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float val = to_f32(e[j]) * inv;
            h[j] = (uint8_t)__nv_cvt_float_to_fp8(val, __NV_SATFINITE, __NV_E4M3);
            l[j] = (uint8_t)__nv_cvt_float_to_fp8(val - e4m3_to_f32(h[j]), __NV_SATFINITE, __NV_E4M3);
        }
        reinterpret_cast<uint2 *>(x_hi + row * k)[idx] = *reinterpret_cast<const uint2 *>(h);
        if (x_lo) reinterpret_cast<uint2 *>(x_lo + row * k)[idx] = *reinterpret_cast<const uint2 *>(l);
    }
}

}  // namespace
}  // namespace xn

using namespace xn;

extern "C" int xn_mm_quantize_rows_i8(int8_t *xq, float *x_scale, const void *x, xn_dtype dtype,
                                      size_t m, size_t k, void *stream) {
    XN_API_RANGE("xn_mm_quantize_rows_i8");
    XN_REQUIRE(valid_dtype(dtype), "quantize_rows_i8: unknown dtype %d", (int)dtype);
    if (m == 0 || k == 0) return XN_OK;
    XN_REQUIRE(xq && x_scale && x, "quantize_rows_i8: null pointer");
    XN_REQUIRE(m <= 0x7fffffffull, "quantize_rows_i8: m too large");
    cudaStream_t st = (cudaStream_t)stream;
    XN_DISPATCH_DTYPE(dtype, T,
        quantize_rows_i8_kernel<T><<<(unsigned)m, 256, 0, st>>>(xq, x_scale, (const T *)x, k));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" size_t xn_mm_q4_packed_bytes(size_t n, size_t k) { return ((n + 15) / 16) * (k / 128) * 1280; }

extern "C" int xn_mm_quantize_weights_q4(void *wq_packed, const void *w, xn_dtype dtype, size_t n, size_t k,
                                         void *stream) {
    XN_API_RANGE("xn_mm_quantize_weights_q4");
    XN_REQUIRE(valid_dtype(dtype), "quantize_weights_q4: unknown dtype %d", (int)dtype);
    XN_REQUIRE(k % 128 == 0 && k > 0, "quantize_weights_q4: k=%zu must be a positive multiple of 128", k);
    if (n == 0) return XN_OK;
    XN_REQUIRE(wq_packed && w, "quantize_weights_q4: null pointer");
    XN_REQUIRE(aligned(wq_packed, 16), "quantize_weights_q4: packed buffer must be 16-byte aligned");
    size_t n_pad = (n + 15) / 16 * 16;
    size_t warps = n_pad * (k / 32);
    size_t blocks = (warps + 7) / 8;
    XN_REQUIRE(blocks <= 0x7fffffffull, "quantize_weights_q4: matrix too large");
    cudaStream_t st = (cudaStream_t)stream;
    XN_DISPATCH_DTYPE(dtype, T,
        quantize_weights_q4_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
            (uint8_t *)wq_packed, (const T *)w, n, n_pad, k));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" size_t xn_mm_q8_packed_bytes(size_t n, size_t k) { return ((n + 15) / 16) * (k / 128) * 2304; }

extern "C" int xn_mm_quantize_weights_q8(void *wq_packed, const void *w, xn_dtype dtype, size_t n, size_t k,
                                         void *stream) {
    XN_API_RANGE("xn_mm_quantize_weights_q8");
    XN_REQUIRE(valid_dtype(dtype), "quantize_weights_q8: unknown dtype %d", (int)dtype);
    XN_REQUIRE(k % 128 == 0 && k > 0, "quantize_weights_q8: k=%zu must be a positive multiple of 128", k);
    if (n == 0) return XN_OK;
    XN_REQUIRE(wq_packed && w, "quantize_weights_q8: null pointer");
    XN_REQUIRE(aligned(wq_packed, 16), "quantize_weights_q8: packed buffer must be 16-byte aligned");
    size_t n_pad = (n + 15) / 16 * 16;
    size_t warps = n_pad * (k / 32);
    size_t blocks = (warps + 7) / 8;
    XN_REQUIRE(blocks <= 0x7fffffffull, "quantize_weights_q8: matrix too large");
    cudaStream_t st = (cudaStream_t)stream;
    XN_DISPATCH_DTYPE(dtype, T,
        quantize_weights_q8_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((uint8_t *)wq_packed, (const T *)w, n, n_pad, k));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_quantize_weights_fp8(uint8_t *wq, float *w_scale, const void *w, xn_dtype dtype,
                                          size_t n, size_t k, void *stream) {
    XN_API_RANGE("xn_mm_quantize_weights_fp8");
    XN_REQUIRE(valid_dtype(dtype), "quantize_weights_fp8: unknown dtype %d", (int)dtype);
    if (n == 0 || k == 0) return XN_OK;
    XN_REQUIRE(wq && w_scale && w, "quantize_weights_fp8: null pointer");
    XN_REQUIRE(n <= 0x7fffffffull, "quantize_weights_fp8: n too large");
    cudaStream_t st = (cudaStream_t)stream;
    XN_DISPATCH_DTYPE(dtype, T,
        quantize_weights_fp8_kernel<T><<<(unsigned)n, 256, 0, st>>>(wq, w_scale, (const T *)w, k));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_split_rows_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, const void *x,
                                     xn_dtype dtype, size_t m, size_t k, void *stream) {
    XN_API_RANGE("xn_mm_split_rows_e4m3");
    XN_REQUIRE(valid_dtype(dtype), "split_rows_e4m3: unknown dtype %d", (int)dtype);
    if (m == 0 || k == 0) return XN_OK;
    XN_REQUIRE(x_hi && x_scale && x, "split_rows_e4m3: null pointer");
    XN_REQUIRE(m <= 0x7fffffffull, "split_rows_e4m3: m too large");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != XN_F32 && k % 8 == 0 && k <= 8 * 256 * 8 && aligned(x, 16) && aligned(x_hi, 8) &&
        (!x_lo || aligned(x_lo, 8))) {
        const bool small = k <= 8 * 256 * 2;
        if (dtype == XN_BF16) {
            if (small) split_rows_e4m3_vec_kernel<__nv_bfloat16, 2><<<(unsigned)m, 256, 0, st>>>(x_hi, x_lo, x_scale, (const __nv_bfloat16 *)x, k);
            else split_rows_e4m3_vec_kernel<__nv_bfloat16, 8><<<(unsigned)m, 256, 0, st>>>(x_hi, x_lo, x_scale, (const __nv_bfloat16 *)x, k);
        } else {
            if (small) split_rows_e4m3_vec_kernel<__half, 2><<<(unsigned)m, 256, 0, st>>>(x_hi, x_lo, x_scale, (const __half *)x, k);
            else split_rows_e4m3_vec_kernel<__half, 8><<<(unsigned)m, 256, 0, st>>>(x_hi, x_lo, x_scale, (const __half *)x, k);
        }
        XN_CHECK_CUDA(cudaGetLastError());
        return XN_OK;
    }
    XN_DISPATCH_DTYPE(dtype, T,
        split_rows_e4m3_kernel<T><<<(unsigned)m, 256, 0, st>>>(x_hi, x_lo, x_scale, (const T *)x, k));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}
