// Row operations a decoder step needs around its matmuls, with the reference's semantics (f32
// math on widened elements, one rounding to the element type where the reference rounds):
//   rms_norm   xn-core/src/cpu_backend.rs:766-784 (CUDA: cuda-kernels/reduce.cu:139-181)
//   softmax    xn-core/src/cpu_backend.rs:742-764 (reduce.cu:185-225)
//   silu * mul the gating of Mlp::Gating, xn-moshi/src/transformer.rs:239-245 (silu: cpu_backend.rs:216-218)
//   add        the residual adds, xn-moshi/src/batched_transformer.rs:259,266
//   kv_append  ScatteredKvCache::append's scatter_set along the context axis,
//              xn-core/src/models/kv_cache.rs:352-366, xn-core/src/cpu_backend.rs:673-697
// plus two fusions that have no counterpart in the reference:
//   *_split_e4m3      the norm / gating writes the fp8 activation pieces of the next linear directly
//   decode_attention  q.k^T -> scale -> +mask -> softmax -> .v (batched_transformer.rs:174-190) in
//                     one pass over the (batch, heads, context, head_dim) cache
// All of them are bandwidth-bound; one CTA per row (or per (stream, head)), 128-bit accesses.
#include "common.cuh"

namespace xn {
namespace {

constexpr int NT = 1024;  // one CTA per row: decode has few rows, so each gets a full SM

__device__ __forceinline__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
    if (w == 0) {
        r = warp_sum(r);
        if (lane == 0) red[0] = r;
    }
    __syncthreads();
    r = red[0];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max2(float v, float *red) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
    if (w == 0) {
        r = warp_max(r);
        if (lane == 0) red[0] = r;
    }
    __syncthreads();
    r = red[0];
    __syncthreads();
    return r;
}

__device__ __forceinline__ float e4m3_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}

// Writes the e4m3 pieces of one row held as f32 values v[i] at columns c(i) (already rounded to
// bf16): s = power of two with max|v|/s in (224, 448]; hi = e4m3(v/s), lo = e4m3(v/s - hi).
__device__ __forceinline__ float pow2_scale(float amax) {
    if (amax == 0.0f || !isfinite(amax)) return 1.0f;
    int ex;
    const float f = frexpf(amax, &ex);
    return ldexpf(1.0f, f <= 0.875f ? ex - 9 : ex - 8);
}

// y = x / sqrt(mean(x^2) + eps) * alpha, rounded to T.  Optionally also the e4m3 pieces of y.
// With `res` the input is the residual sum x = T(src + res), which is also written to `sum_out` (the row then
// comes from sum_out in the later passes: every thread re-reads only what it wrote itself).
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(NT)
rms_norm_kernel(T *__restrict__ dst, uint8_t *__restrict__ hi, uint8_t *__restrict__ lo, float *__restrict__ scale,
                const T *__restrict__ src, const T *__restrict__ alpha, size_t cols, float eps,
                const T *__restrict__ res = nullptr, T *sum_out = nullptr) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const T *x = res ? sum_out + row * cols : src + row * cols;
    float s2 = 0.0f;
    for (size_t c = threadIdx.x; c < cols; c += NT) {
        float v;
        if (res) {
            const T sum = from_f32<T>(to_f32(src[row * cols + c]) + to_f32(res[row * cols + c]));
            sum_out[row * cols + c] = sum;
            v = to_f32(sum);
        } else {
            v = to_f32(x[c]);
        }
        s2 += v * v;
    }
    s2 = block_sum(s2, red);
    const float denom = sqrtf(s2 / (float)cols + eps);
    float amax = 0.0f;
    for (size_t c = threadIdx.x; c < cols; c += NT) {
        const T y = from_f32<T>(to_f32(x[c]) / denom * to_f32(alpha[c]));
        if (dst) dst[row * cols + c] = y;
        if (SPLIT) amax = fmaxf(amax, fabsf(to_f32(y)));
    }
    if (SPLIT) {
        amax = block_max2(amax, red);
        const float s = pow2_scale(amax), inv = 1.0f / s;
        if (threadIdx.x == 0) scale[row] = s;
        for (size_t c = threadIdx.x; c < cols; c += NT) {
            const float y = to_f32(from_f32<T>(to_f32(x[c]) / denom * to_f32(alpha[c]))) * inv;
            const uint8_t h = (uint8_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
            hi[row * cols + c] = h;
            if (lo) lo[row * cols + c] = (uint8_t)__nv_cvt_float_to_fp8(y - e4m3_f32(h), __NV_SATFINITE, __NV_E4M3);
        }
    }
}

// 16-bit fast paths of the two kernels above: 128-bit loads, the row held in registers between the passes (one
// read of the inputs, no recomputation), 8-byte piece stores.  Element arithmetic and roundings are those of the
// scalar kernels; only the order of the f32 sum of squares differs.
constexpr int NTV = 512;

template <typename T> __device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = to_f32(e[j]);
}
template <typename T> __device__ __forceinline__ uint4 pack8(const T (&y)[8]) {
    uint4 r;
    T *e = reinterpret_cast<T *>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = y[j];
    return r;
}
// two 16-bit elements in one 32-bit word: widen, round a pair with one conversion, packed maximum
template <typename T> __device__ __forceinline__ float2 unpack2(unsigned w);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(unsigned w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(unsigned w) { return __half22float2(*reinterpret_cast<const __half2 *>(&w)); }
template <typename T> __device__ __forceinline__ unsigned pack2(float a, float b);
template <> __device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float a, float b) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&r);
}
template <> __device__ __forceinline__ unsigned pack2<__half>(float a, float b) {
    const __half2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<const unsigned *>(&r);
}
template <typename T> __device__ __forceinline__ unsigned max2(unsigned a, unsigned b);
template <> __device__ __forceinline__ unsigned max2<__nv_bfloat16>(unsigned a, unsigned b) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&a), *reinterpret_cast<const __nv_bfloat162 *>(&b));
    return *reinterpret_cast<const unsigned *>(&r);
}
template <> __device__ __forceinline__ unsigned max2<__half>(unsigned a, unsigned b) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
    return *reinterpret_cast<const unsigned *>(&r);
}
// the e4m3 pieces of eight values already divided by the row scale
__device__ __forceinline__ void store_pieces8(uint8_t *hi, uint8_t *lo, size_t off, const float (&yv)[8]) {
    uint8_t h[8], l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        h[j] = (uint8_t)__nv_cvt_float_to_fp8(yv[j], __NV_SATFINITE, __NV_E4M3);
        l[j] = (uint8_t)__nv_cvt_float_to_fp8(yv[j] - e4m3_f32(h[j]), __NV_SATFINITE, __NV_E4M3);
    }
    *reinterpret_cast<uint2 *>(hi + off) = *reinterpret_cast<const uint2 *>(h);
    if (lo) *reinterpret_cast<uint2 *>(lo + off) = *reinterpret_cast<const uint2 *>(l);
}

template <typename T, int VPT, bool SPLIT>
__global__ void __launch_bounds__(NTV)
rms_norm_vec_kernel(T *__restrict__ dst, uint8_t *__restrict__ hi, uint8_t *__restrict__ lo, float *__restrict__ scale,
                    const T *__restrict__ src, const T *__restrict__ alpha, int cols, float eps, const T *__restrict__ res,
                    T *sum_out) {
    __shared__ float red[32];
    const size_t row = blockIdx.x, base = row * (size_t)cols;
    const int nvec = cols / 8;
    uint4 v[VPT];
    float s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = i * NTV + threadIdx.x;
        if (idx >= nvec) { v[i] = make_uint4(0, 0, 0, 0); continue; }
        v[i] = __ldg(reinterpret_cast<const uint4 *>(src + base) + idx);
        float f[8];
        unpack8<T>(v[i], f);
        if (res) {
            float r[8];
            unpack8<T>(__ldg(reinterpret_cast<const uint4 *>(res + base) + idx), r);
            T sum[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { sum[j] = from_f32<T>(f[j] + r[j]); f[j] = to_f32(sum[j]); }
            v[i] = pack8<T>(sum);
            reinterpret_cast<uint4 *>(sum_out + base)[idx] = v[i];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s2 += f[j] * f[j];
    }
    s2 = block_sum(s2, red);
    const float denom = sqrtf(s2 / (float)cols + eps);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = i * NTV + threadIdx.x;
        if (idx >= nvec) continue;
        float f[8], al[8];
        unpack8<T>(v[i], f);
        unpack8<T>(__ldg(reinterpret_cast<const uint4 *>(alpha) + idx), al);
        T y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            y[j] = from_f32<T>(f[j] / denom * al[j]);
            if (SPLIT) amax = fmaxf(amax, fabsf(to_f32(y[j])));
        }
        v[i] = pack8<T>(y);
        if (dst) reinterpret_cast<uint4 *>(dst + base)[idx] = v[i];
    }
    if (SPLIT) {
        amax = block_max2(amax, red);
        const float sc = pow2_scale(amax), inv = 1.0f / sc;
        if (threadIdx.x == 0) scale[row] = sc;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = i * NTV + threadIdx.x;
            if (idx >= nvec) continue;
            float f[8];
            unpack8<T>(v[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] *= inv;
            store_pieces8(hi, lo, base + (size_t)idx * 8, f);
        }
    }
}

template <typename T, int VPT, bool SPLIT>
__global__ void __launch_bounds__(NTV)
silu_mul_vec_kernel(T *__restrict__ dst, uint8_t *__restrict__ hi, uint8_t *__restrict__ lo, float *__restrict__ scale,
                    const T *__restrict__ src, int hidden) {
    __shared__ float red[32];
    const size_t row = blockIdx.x, obase = row * (size_t)hidden;
    const uint4 *a = reinterpret_cast<const uint4 *>(src + row * 2 * (size_t)hidden);
    const uint4 *b = reinterpret_cast<const uint4 *>(src + row * 2 * (size_t)hidden + hidden);
    const int nvec = hidden / 8;
    uint4 v[VPT];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = i * NTV + threadIdx.x;
        if (idx >= nvec) { v[i] = make_uint4(0, 0, 0, 0); continue; }
        float av[8], bv[8];
        unpack8<T>(__ldg(a + idx), av);
        unpack8<T>(__ldg(b + idx), bv);
        T y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sl = to_f32(from_f32<T>(av[j] / (1.0f + expf(-av[j]))));
            y[j] = from_f32<T>(sl * bv[j]);
            if (SPLIT) amax = fmaxf(amax, fabsf(to_f32(y[j])));
        }
        v[i] = pack8<T>(y);
        if (dst) reinterpret_cast<uint4 *>(dst + obase)[idx] = v[i];
    }
    if (SPLIT) {
        amax = block_max2(amax, red);
        const float sc = pow2_scale(amax), inv = 1.0f / sc;
        if (threadIdx.x == 0) scale[row] = sc;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = i * NTV + threadIdx.x;
            if (idx >= nvec) continue;
            float f[8];
            unpack8<T>(v[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] *= inv;
            store_pieces8(hi, lo, obase + (size_t)idx * 8, f);
        }
    }
}

// Picks the vector kernels for 16-bit rows that fit (8-element vectors, 16-byte aligned rows); returns false when the
// scalar kernel has to run.
template <typename T, bool SPLIT>
bool launch_rms_norm_vec(T *dst, uint8_t *hi, uint8_t *lo, float *scale, const T *src, const T *alpha, size_t rows, size_t cols,
                         float eps, const T *res, T *sum_out, cudaStream_t st) {
    if (sizeof(T) != 2 || cols % 8 != 0 || cols > (size_t)NTV * 8 * 4 || !aligned(src, 16) || !aligned(alpha, 16) ||
        (dst && !aligned(dst, 16)) || (res && (!aligned(res, 16) || !aligned(sum_out, 16))) || (hi && !aligned(hi, 8)) ||
        (lo && !aligned(lo, 8)))
        return false;
    if (cols <= (size_t)NTV * 8)
        rms_norm_vec_kernel<T, 1, SPLIT><<<(unsigned)rows, NTV, 0, st>>>(dst, hi, lo, scale, src, alpha, (int)cols, eps, res, sum_out);
    else
        rms_norm_vec_kernel<T, 4, SPLIT><<<(unsigned)rows, NTV, 0, st>>>(dst, hi, lo, scale, src, alpha, (int)cols, eps, res, sum_out);
    return true;
}
template <typename T, bool SPLIT>
bool launch_silu_mul_vec(T *dst, uint8_t *hi, uint8_t *lo, float *scale, const T *src, size_t rows, size_t hidden, cudaStream_t st) {
    if (sizeof(T) != 2 || hidden % 8 != 0 || hidden > (size_t)NTV * 8 * 8 || !aligned(src, 16) || (dst && !aligned(dst, 16)) ||
        (hi && !aligned(hi, 8)) || (lo && !aligned(lo, 8)))
        return false;
    if (hidden <= (size_t)NTV * 8)
        silu_mul_vec_kernel<T, 1, SPLIT><<<(unsigned)rows, NTV, 0, st>>>(dst, hi, lo, scale, src, (int)hidden);
    else if (hidden <= (size_t)NTV * 8 * 3)
        silu_mul_vec_kernel<T, 3, SPLIT><<<(unsigned)rows, NTV, 0, st>>>(dst, hi, lo, scale, src, (int)hidden);
    else
        silu_mul_vec_kernel<T, 8, SPLIT><<<(unsigned)rows, NTV, 0, st>>>(dst, hi, lo, scale, src, (int)hidden);
    return true;
}

// One warp per row: max-subtract, exp rounded to T, f32 sum of the rounded values, divide.
template <typename T>
__global__ void softmax_kernel(T *__restrict__ dst, const T *__restrict__ src, size_t rows, size_t cols) {
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const T *x = src + row * cols;
    T *y = dst + row * cols;
    float mx = -INFINITY;
    for (size_t c = lane; c < cols; c += 32) mx = fmaxf(mx, to_f32(x[c]));
    mx = warp_max(mx);
    float sum = 0.0f;
    for (size_t c = lane; c < cols; c += 32) {
        // the reference subtracts in the element type: (x - max) is rounded before the exponential
        const T e = from_f32<T>(expf(to_f32(from_f32<T>(to_f32(x[c]) - mx))));
        y[c] = e;
        sum += to_f32(e);
    }
    sum = warp_sum(sum);
    for (size_t c = lane; c < cols; c += 32) y[c] = from_f32<T>(to_f32(y[c]) / sum);
}

// out[r, c] = T(silu(a)) * b with a = src[r, c], b = src[r, hidden + c]; optionally the e4m3 pieces.
template <typename T, bool SPLIT>
__global__ void __launch_bounds__(NT)
silu_mul_kernel(T *__restrict__ dst, uint8_t *__restrict__ hi, uint8_t *__restrict__ lo, float *__restrict__ scale,
                const T *__restrict__ src, size_t hidden) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const T *a = src + row * 2 * hidden, *b = a + hidden;
    auto f = [&](size_t c) {
        const float av = to_f32(a[c]);
        const float s = to_f32(from_f32<T>(av / (1.0f + expf(-av))));
        return from_f32<T>(s * to_f32(b[c]));
    };
    float amax = 0.0f;
    for (size_t c = threadIdx.x; c < hidden; c += NT) {
        const T y = f(c);
        if (dst) dst[row * hidden + c] = y;
        if (SPLIT) amax = fmaxf(amax, fabsf(to_f32(y)));
    }
    if (SPLIT) {
        amax = block_max2(amax, red);
        const float s = pow2_scale(amax), inv = 1.0f / s;
        if (threadIdx.x == 0) scale[row] = s;
        for (size_t c = threadIdx.x; c < hidden; c += NT) {
            const float y = to_f32(f(c)) * inv;
            const uint8_t h = (uint8_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
            hi[row * hidden + c] = h;
            if (lo) lo[row * hidden + c] = (uint8_t)__nv_cvt_float_to_fp8(y - e4m3_f32(h), __NV_SATFINITE, __NV_E4M3);
        }
    }
}

template <typename T>
__global__ void add_kernel(T *__restrict__ dst, const T *__restrict__ a, const T *__restrict__ b, size_t len) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < len) dst[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
}

// cache [batch, heads, context, hd] <- src [batch, heads, 1, hd] at context index idx[batch].
template <typename T>
__global__ void kv_append_kernel(T *__restrict__ cache, const T *__restrict__ src, const int64_t *__restrict__ idx,
                                 size_t heads, size_t context, size_t hd, size_t src_batch_stride, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t d = i % hd, h = (i / hd) % heads, b = i / (hd * heads);
    const int64_t p = idx[b];
    if (p < 0 || (size_t)p >= context) return;  // out-of-range index: nothing is written
    cache[((b * heads + h) * context + (size_t)p) * hd + d] = src[b * src_batch_stride + h * hd + d];
}

// Fused single-token attention over a (batch, heads, context, 128) bf16 cache.  One CTA of 4 warps per
// (stream, head); a half-warp owns a key/value row (16 lanes x 16 bytes = 128 bf16), so a warp
// handles two rows per step; online softmax per half-warp, merged at the end.  f32 throughout.
constexpr int HD = 128;
// SLICED = false is the one-pass form (whole context, result straight to `out`); it is a separate
// instantiation because the sliced form's extra bounds cost the one-pass case 6 % when they are run-time values.
template <bool SLICED>
__global__ void __launch_bounds__(128)
decode_attention_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ q,
                        const __nv_bfloat16 *__restrict__ kc, const __nv_bfloat16 *__restrict__ vc,
                        const float *__restrict__ mask, size_t heads, size_t context, size_t q_batch_stride,
                        float scale, size_t rows_per_split, float *__restrict__ partial) {
    // blockIdx.y = slice of the context (rows [row_lo, row_hi)); with one slice the result goes straight to `out`,
    // otherwise the slice's running maximum, sum and unnormalised output go to `partial` for the combine kernel
    const size_t bh = blockIdx.x, b = bh / heads;
    const size_t row_lo = SLICED ? (size_t)blockIdx.y * rows_per_split : 0;
    const size_t row_hi = SLICED ? (row_lo + rows_per_split < context ? row_lo + rows_per_split : context) : context;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4, l16 = lane & 15;
    const int group = warp * 2 + half;  // 8 half-warps stride over the rows
    float qv[8];
    {
        const uint4 t = *reinterpret_cast<const uint4 *>(q + b * q_batch_stride + (bh % heads) * HD + l16 * 8);
        const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&t);
#pragma unroll
        for (int j = 0; j < 8; ++j) qv[j] = __bfloat162float(e[j]) * scale;
    }
    const __nv_bfloat16 *kb = kc + bh * context * HD, *vb = vc + bh * context * HD;
    const float *mrow = mask ? mask + b * context : nullptr;
    float m_run = -INFINITY, l_run = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    constexpr int U = 4;
    // Software pipeline: the loads of the next 8 * U rows are in flight while this group's scores and products are
    // computed, so the memory system always has a full set of requests from every warp (without it a warp's
    // requests drain during its shuffle / exp chain and the kernel sat at 83 % of the copy bandwidth).
    uint4 kn[U], vn[U];
    auto fetch = [&](size_t base) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t r = base + group + 8 * u;
            if (r < row_hi) {
                kn[u] = ldg_stream(kb + r * HD + l16 * 8);
                vn[u] = ldg_stream(vb + r * HD + l16 * 8);
            } else {
                kn[u] = make_uint4(0, 0, 0, 0);
                vn[u] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    fetch(row_lo);
    for (size_t base = row_lo; base < row_hi; base += 8 * U) {  // uniform trip count across the CTA
        const size_t r0 = base + group;
        uint4 kr[U], vr[U];
        float s[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { kr[u] = kn[u]; vr[u] = vn[u]; }
        if (base + 8 * U < row_hi) fetch(base + 8 * U);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&kr[u]);
            float d = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) d = fmaf(qv[j], __bfloat162float(e[j]), d);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);  // within the half-warp
            const size_t r = r0 + 8 * u;
            if (r >= row_hi) d = -INFINITY;
            else if (mrow) d += mrow[r];
            s[u] = d;
        }
        float m_new = m_run;
#pragma unroll
        for (int u = 0; u < U; ++u) m_new = fmaxf(m_new, s[u]);
        if (m_new == -INFINITY) continue;  // everything masked so far
        const float corr = __expf(m_run - m_new);
        l_run *= corr;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= corr;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float p = __expf(s[u] - m_new);
            l_run += p;
            const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&vr[u]);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(p, __bfloat162float(e[j]), acc[j]);
        }
        m_run = m_new;
    }
    // merge the 8 half-warp states
    __shared__ float sm_m[8], sm_l[8], sm_acc[8][HD];
    if (l16 == 0) { sm_m[group] = m_run; sm_l[group] = l_run; }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm_acc[group][l16 * 8 + j] = acc[j];
    __syncthreads();
    if (threadIdx.x < HD) {
        float mx = -INFINITY;
#pragma unroll
        for (int gI = 0; gI < 8; ++gI) mx = fmaxf(mx, sm_m[gI]);
        float l = 0.0f, o = 0.0f;
#pragma unroll
        for (int gI = 0; gI < 8; ++gI) {
            const float w = sm_m[gI] == -INFINITY ? 0.0f : __expf(sm_m[gI] - mx);
            l += w * sm_l[gI];
            o += w * sm_acc[gI][threadIdx.x];
        }
        if (!SLICED) {
            out[bh * HD + threadIdx.x] = __float2bfloat16_rn(o / l);
        } else {
            float *p = partial + (bh * gridDim.y + blockIdx.y) * (HD + 2);
            p[2 + threadIdx.x] = o;
            if (threadIdx.x == 0) { p[0] = mx; p[1] = l; }
        }
    }
}

// Log-sum-exp merge of the context slices of one (stream, head): out = sum_s w_s o_s / sum_s w_s l_s,
// w_s = exp(m_s - max_s m_s).  One CTA of 128 threads per (stream, head).
__global__ void __launch_bounds__(HD)
decode_attention_combine_kernel(__nv_bfloat16 *__restrict__ out, const float *__restrict__ partial, int splits) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t bh = blockIdx.x;
    const float *p = partial + bh * splits * (HD + 2);
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, p[(size_t)s * (HD + 2)]);
    float l = 0.0f, o = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float m = p[(size_t)s * (HD + 2)];
        const float w = m == -INFINITY ? 0.0f : __expf(m - mx);
        l += w * p[(size_t)s * (HD + 2) + 1];
        o += w * p[(size_t)s * (HD + 2) + 2 + threadIdx.x];
    }
    out[bh * HD + threadIdx.x] = __float2bfloat16_rn(o / l);
}

constexpr int AHD = 128;  // head dimension of the attention kernels
// The same merge for a whole stream row (all heads), followed by the e4m3 split of that row: the attention output is
// the activation of the output projection, whose fp8 pieces need the row's maximum over all heads.  One CTA of
// 1024 threads per stream; a thread owns 4 consecutive dimensions of up to two heads (heads <= 64).
__global__ void __launch_bounds__(1024)
decode_attention_combine_split_kernel(__nv_bfloat16 *__restrict__ out, uint8_t *__restrict__ hi, uint8_t *__restrict__ lo,
                                      float *__restrict__ xs, const float *__restrict__ partial, int splits, int heads) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float red[32];
    const size_t b = blockIdx.x;
    const int items = heads * (AHD / 4);
    float val[2][4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int it = i * 1024 + (int)threadIdx.x;
        if (it >= items) continue;
        const int h = it / (AHD / 4), d0 = (it % (AHD / 4)) * 4;
        const float *p = partial + (b * heads + h) * (size_t)splits * (AHD + 2);
        float mx = -INFINITY;
        for (int s = 0; s < splits; ++s) mx = fmaxf(mx, p[(size_t)s * (AHD + 2)]);
        float l = 0.0f, o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int s = 0; s < splits; ++s) {
            const float m = p[(size_t)s * (AHD + 2)];
            const float w = m == -INFINITY ? 0.0f : __expf(m - mx);
            l += w * p[(size_t)s * (AHD + 2) + 1];
            // a slice's record is 130 floats: its output vector is 8-byte, not 16-byte, aligned
            const float2 o01 = *reinterpret_cast<const float2 *>(p + (size_t)s * (AHD + 2) + 2 + d0);
            const float2 o23 = *reinterpret_cast<const float2 *>(p + (size_t)s * (AHD + 2) + 4 + d0);
            o[0] += w * o01.x; o[1] += w * o01.y; o[2] += w * o23.x; o[3] += w * o23.y;
        }
        __nv_bfloat16 y[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            y[j] = __float2bfloat16_rn(o[j] / l);
            val[i][j] = __bfloat162float(y[j]);
            amax = fmaxf(amax, fabsf(val[i][j]));
        }
        *reinterpret_cast<uint2 *>(out + (b * heads + h) * AHD + d0) = *reinterpret_cast<const uint2 *>(y);
    }
    amax = block_max2(amax, red);
    const float sc = pow2_scale(amax), inv = 1.0f / sc;
    if (threadIdx.x == 0) xs[b] = sc;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int it = i * 1024 + (int)threadIdx.x;
        if (it >= items) continue;
        uint8_t hh[4], ll[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float yv = val[i][j] * inv;
            hh[j] = (uint8_t)__nv_cvt_float_to_fp8(yv, __NV_SATFINITE, __NV_E4M3);
            ll[j] = (uint8_t)__nv_cvt_float_to_fp8(yv - e4m3_f32(hh[j]), __NV_SATFINITE, __NV_E4M3);
        }
        const size_t off = b * (size_t)heads * AHD + (size_t)it * 4;
        *reinterpret_cast<uint32_t *>(hi + off) = *reinterpret_cast<const uint32_t *>(hh);
        if (lo) *reinterpret_cast<uint32_t *>(lo + off) = *reinterpret_cast<const uint32_t *>(ll);
    }
}


// The row loop of the single-token attention for one half-warp: rows row_lo + group, + 8, ... below row_hi of a
// (stream, head) cache, online softmax in f32, the loads of the next 8 * U rows in flight while this group's scores
// and products are computed.  kl / vl point at this lane's 16 bytes of row 0; with NEW, row r_new is read from
// knl / vnl (the key / value being appended) instead of the cache.
template <bool NEW>
__device__ __forceinline__ void attend_rows(const float (&qv)[8], const __nv_bfloat16 *kl, const __nv_bfloat16 *vl,
                                            const __nv_bfloat16 *knl, const __nv_bfloat16 *vnl, int r_new,
                                            const float *mrow, int row_lo, int row_hi, int group, float &m_run, float &l_run,
                                            float (&acc)[8]) {
    constexpr int U = 4;
    uint4 kn[U], vn[U];
    auto fetch = [&](int base) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int r = base + group + 8 * u;
            if (r < row_hi) {
                const bool is_new = NEW && r == r_new;
                kn[u] = ldg_stream(is_new ? knl : kl + (size_t)r * HD);
                vn[u] = ldg_stream(is_new ? vnl : vl + (size_t)r * HD);
            } else {
                kn[u] = make_uint4(0, 0, 0, 0);
                vn[u] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    fetch(row_lo);
    for (int base = row_lo; base < row_hi; base += 8 * U) {  // uniform trip count across the CTA
        const int r0 = base + group;
        uint4 kr[U], vr[U];
        float sc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { kr[u] = kn[u]; vr[u] = vn[u]; }
        if (base + 8 * U < row_hi) fetch(base + 8 * U);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&kr[u]);
            float d = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) d = fmaf(qv[j], __bfloat162float(e[j]), d);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);  // within the half-warp
            const int r = r0 + 8 * u;
            if (r >= row_hi) d = -INFINITY;
            else if (mrow) d += mrow[r];
            sc[u] = d;
        }
        float m_new = m_run;
#pragma unroll
        for (int u = 0; u < U; ++u) m_new = fmaxf(m_new, sc[u]);
        if (m_new == -INFINITY) continue;  // everything masked so far
        const float corr = __expf(m_run - m_new);
        l_run *= corr;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= corr;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float p = __expf(sc[u] - m_new);
            l_run += p;
            const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&vr[u]);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(p, __bfloat162float(e[j]), acc[j]);
        }
        m_run = m_new;
    }
}

// One launch for what a decode layer does between its input and output projections: append the new key / value row
// of every (stream, head) to the caches at index[stream], attend over the cache, merge the context slices, and split
// the [streams, heads * 128] output row into e4m3 pieces -- xn_mm_kv_append2, xn_mm_decode_attention_split and the
// merge + split kernel in one grid, with identical results.
//   * The slice that holds row index[stream] takes that row from the new key / value instead of the cache and writes
//     it to the cache on the way (no other CTA of the grid touches the row).
//   * Every slice stores its (maximum, sum, output) record; the CTA that arrives last at a (stream, head) merges
//     the records in slice order, and the CTA that finishes the last head of a stream splits the stream's row.  Both
//     "last" decisions are arrival counters in library scratch, zero between launches; the merges run in a fixed
//     order, so the result does not depend on which CTA happens to be last.
template <bool MERGE>
__global__ void __launch_bounds__(128, 5)   // five CTAs per SM, like the kernel it extends
decode_attention_append_kernel(__nv_bfloat16 *__restrict__ out, uint8_t *__restrict__ hi, uint8_t *__restrict__ lo,
                               float *__restrict__ xs, const __nv_bfloat16 *__restrict__ q,
                               const __nv_bfloat16 *__restrict__ k_new, const __nv_bfloat16 *__restrict__ v_new,
                               __nv_bfloat16 *__restrict__ kc, __nv_bfloat16 *__restrict__ vc,
                               const int64_t *__restrict__ index, const float *__restrict__ mask, size_t heads, size_t context,
                               size_t qkv_batch_stride, float scale, size_t rows_per_split, float *__restrict__ partial,
                               unsigned *__restrict__ cnt_head, unsigned *__restrict__ cnt_stream) {
    const size_t bh = blockIdx.x, b = bh / heads, h = bh % heads;
    // 32-bit row indices (context < 2^31): the loop's live state must fit 96 registers with the new-row pointers
    const int row_lo = (int)(blockIdx.y * rows_per_split);
    const int row_hi = (int)(row_lo + rows_per_split < context ? row_lo + rows_per_split : context);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4, l16 = lane & 15;
    const int group = warp * 2 + half;  // 8 half-warps stride over the rows
    float qv[8];
    {
        const uint4 t = *reinterpret_cast<const uint4 *>(q + b * qkv_batch_stride + h * HD + l16 * 8);
        const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&t);
#pragma unroll
        for (int j = 0; j < 8; ++j) qv[j] = __bfloat162float(e[j]) * scale;
    }
    const int64_t pidx = index[b];
    const int r_new = (pidx >= 0 && (size_t)pidx < context) ? (int)pidx : -1;  // out of range: nothing appended
    const float *mrow = mask ? mask + b * context : nullptr;
    float m_run = -INFINITY, l_run = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // Only the slice that holds the appended row pays for it: there the row's source is selected per load (no
    // branch inside the software pipeline), everywhere else the loop is the plain one.
    if (r_new >= row_lo && r_new < row_hi) {
        const __nv_bfloat16 *knl = k_new + b * qkv_batch_stride + h * HD + l16 * 8;
        const __nv_bfloat16 *vnl = v_new + b * qkv_batch_stride + h * HD + l16 * 8;
        attend_rows<true>(qv, kc + bh * context * HD + l16 * 8, vc + bh * context * HD + l16 * 8, knl, vnl, r_new, mrow, row_lo,
                          row_hi, group, m_run, l_run, acc);
        if (group == ((r_new - row_lo) & 7)) {  // the half-warp that read the row also writes it to the caches
            const size_t off = (bh * context + (size_t)r_new) * HD + l16 * 8, noff = b * qkv_batch_stride + h * HD + l16 * 8;
            *reinterpret_cast<uint4 *>(kc + off) = *reinterpret_cast<const uint4 *>(k_new + noff);
            *reinterpret_cast<uint4 *>(vc + off) = *reinterpret_cast<const uint4 *>(v_new + noff);
        }
    } else {
        attend_rows<false>(qv, kc + bh * context * HD + l16 * 8, vc + bh * context * HD + l16 * 8, nullptr, nullptr, -1, mrow,
                           row_lo, row_hi, group, m_run, l_run, acc);
    }
    // merge the 8 half-warp states into the slice's record
    __shared__ float sm_m[8], sm_l[8], sm_acc[8][HD];
    __shared__ float red[32];
    __shared__ int s_last;
    if (l16 == 0) { sm_m[group] = m_run; sm_l[group] = l_run; }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm_acc[group][l16 * 8 + j] = acc[j];
    __syncthreads();
    const int splits = (int)gridDim.y;
    {
        float mx = -INFINITY;
#pragma unroll
        for (int gI = 0; gI < 8; ++gI) mx = fmaxf(mx, sm_m[gI]);
        float l = 0.0f, o = 0.0f;
#pragma unroll
        for (int gI = 0; gI < 8; ++gI) {
            const float w = sm_m[gI] == -INFINITY ? 0.0f : __expf(sm_m[gI] - mx);
            l += w * sm_l[gI];
            o += w * sm_acc[gI][threadIdx.x];
        }
        float *p = partial + (bh * splits + blockIdx.y) * (HD + 2);
        p[2 + threadIdx.x] = o;
        if (threadIdx.x == 0) { p[0] = mx; p[1] = l; }
    }
    if (!MERGE) return;  // the merge + split kernel follows as its own launch
    // last slice of this (stream, head)?
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(cnt_head + bh, 1u) == (unsigned)splits - 1 ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    {
        const float *p = partial + bh * splits * (HD + 2);
        float mx = -INFINITY;
        for (int s2 = 0; s2 < splits; ++s2) mx = fmaxf(mx, __ldcg(p + (size_t)s2 * (HD + 2)));
        float l = 0.0f, o = 0.0f;
        for (int s2 = 0; s2 < splits; ++s2) {
            const float m = __ldcg(p + (size_t)s2 * (HD + 2));
            const float w = m == -INFINITY ? 0.0f : __expf(m - mx);
            l += w * __ldcg(p + (size_t)s2 * (HD + 2) + 1);
            o += w * __ldcg(p + (size_t)s2 * (HD + 2) + 2 + threadIdx.x);
        }
        out[bh * HD + threadIdx.x] = __float2bfloat16_rn(o / l);
    }
    // last head of this stream?
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        cnt_head[bh] = 0;  // ready for the next launch
        s_last = atomicAdd(cnt_stream + b, 1u) == (unsigned)heads - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last || !hi) {
        if (s_last && threadIdx.x == 0) cnt_stream[b] = 0;
        return;
    }
    __threadfence();
    if (threadIdx.x == 0) cnt_stream[b] = 0;
    // e4m3 pieces of the stream's row: a thread owns 4 consecutive dimensions of every fourth head
    const int items = (int)heads * (HD / 4);
    const __nv_bfloat16 *row = out + b * heads * HD;
    float amax = 0.0f;
    for (int it = threadIdx.x; it < items; it += 128) {
        const uint2 t = __ldcg(reinterpret_cast<const uint2 *>(row + (size_t)it * 4));
        const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&t);
#pragma unroll
        for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fabsf(__bfloat162float(e[j])));
    }
    amax = block_max2(amax, red);
    const float scl = pow2_scale(amax), inv = 1.0f / scl;
    if (threadIdx.x == 0) xs[b] = scl;
    for (int it = threadIdx.x; it < items; it += 128) {
        const uint2 t = __ldcg(reinterpret_cast<const uint2 *>(row + (size_t)it * 4));
        const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&t);
        uint8_t hh[4], ll[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float yv = __bfloat162float(e[j]) * inv;
            hh[j] = (uint8_t)__nv_cvt_float_to_fp8(yv, __NV_SATFINITE, __NV_E4M3);
            ll[j] = (uint8_t)__nv_cvt_float_to_fp8(yv - e4m3_f32(hh[j]), __NV_SATFINITE, __NV_E4M3);
        }
        const size_t off = b * heads * HD + (size_t)it * 4;
        *reinterpret_cast<uint32_t *>(hi + off) = *reinterpret_cast<const uint32_t *>(hh);
        if (lo) *reinterpret_cast<uint32_t *>(lo + off) = *reinterpret_cast<const uint32_t *>(ll);
    }
}


// Causal attention probabilities for a block of T query rows against ctx keys (the last T keys are the block's
// own): row i sees keys j <= i + (ctx - T).  y = softmax(T(s * scale)) over the visible keys with the roundings of
// the unfused route (scores scaled and rounded to the element type, exp and quotient rounded as in softmax_kernel),
// zeros elsewhere -- the scale -> +mask -> softmax sequence of xn-moshi/src/batched_transformer.rs:176-189 in one
// pass.  One CTA of 256 threads per row.
template <typename T>
__global__ void __launch_bounds__(256)
softmax_causal_kernel(T *dst, const T *src, size_t t_rows, size_t ctx, float scale, int fill_all) {  // dst may be src
    __shared__ float red[32];
    const size_t row = blockIdx.x, i = row % t_rows;
    const size_t vis = i + (ctx - t_rows) + 1;  // visible keys
    const T *x = src + row * ctx;
    T *y = dst + row * ctx;
    float mx = -INFINITY;
    for (size_t c = threadIdx.x; c < vis; c += 256) mx = fmaxf(mx, to_f32(from_f32<T>(to_f32(x[c]) * scale)));
    mx = block_max2(mx, red);
    float sum = 0.0f;
    for (size_t c = threadIdx.x; c < vis; c += 256) {
        const float sv = to_f32(from_f32<T>(to_f32(x[c]) * scale));
        const T e = from_f32<T>(expf(to_f32(from_f32<T>(sv - mx))));
        y[c] = e;
        sum += to_f32(e);
    }
    sum = block_sum(sum, red);
    // the values matmul reads whole 64-element k stages up to the horizon of the row's 128-row tile
    const size_t zend = fill_all ? ctx : min(ctx, ((i / 128 + 1) * 128 + (ctx - t_rows) + 63) / 64 * 64);
    for (size_t c = threadIdx.x; c < zend; c += 256) y[c] = c < vis ? from_f32<T>(to_f32(y[c]) / sum) : from_f32<T>(0.0f);
}

// 16-bit fast path: the row in registers (128-bit loads of the visible part only, one read, one write).
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
softmax_causal_vec_kernel(T *dst, const T *src, size_t t_rows, size_t ctx, float scale, int fill_all) {
    __shared__ float red[32];
    const size_t row = blockIdx.x, i = row % t_rows;
    const int vis = (int)(i + (ctx - t_rows) + 1), nvec = (int)(ctx / 8);
    const uint4 *x = reinterpret_cast<const uint4 *>(src + row * ctx);
    uint4 *y = reinterpret_cast<uint4 *>(dst + row * ctx);
    float v[VPT][8];
    float mx = -INFINITY;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = u * 256 + (int)threadIdx.x, c0 = idx * 8;
        if (idx < nvec && c0 < vis) {
            unpack8<T>(x[idx], v[u]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[u][j] = c0 + j < vis ? to_f32(from_f32<T>(v[u][j] * scale)) : -INFINITY;
                mx = fmaxf(mx, v[u][j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[u][j] = -INFINITY;
        }
    }
    mx = block_max2(mx, red);
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < VPT; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // masked positions (-inf) give exp = 0 and stay 0 after the division
            v[u][j] = v[u][j] == -INFINITY ? 0.0f : to_f32(from_f32<T>(expf(to_f32(from_f32<T>(v[u][j] - mx)))));
            sum += v[u][j];
        }
    sum = block_sum(sum, red);
#pragma unroll
    const int zend = fill_all ? (int)ctx : (int)min(ctx, ((i / 128 + 1) * 128 + (ctx - t_rows) + 63) / 64 * 64);
    for (int u = 0; u < VPT; ++u) {
        const int idx = u * 256 + (int)threadIdx.x;
        if (idx >= nvec || idx * 8 >= zend) continue;
        T o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = from_f32<T>(v[u][j] / sum);
        y[idx] = pack8<T>(o);
    }
}

// One warp per row, the row packed in registers in the element type (every intermediate of the computation is
// rounded to it anyway): no CTA-wide barriers, VPT 128-bit loads per lane in flight -- a CTA per row is bound by
// its own latency when there are 10^5 rows of a few KB (prefill attention: heads x tokens rows).
template <typename T, int VPT>
__global__ void __launch_bounds__(256, 2)
softmax_causal_warp_kernel(T *dst, const T *src, size_t rows, size_t t_rows, size_t ctx, float scale, int fill_all) {
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const size_t i = row % t_rows;
    const int vis = (int)(i + (ctx - t_rows) + 1), nvec = (int)(ctx / 8);
    const int zend = fill_all ? (int)ctx : (int)min(ctx, ((i / 128 + 1) * 128 + (ctx - t_rows) + 63) / 64 * 64);
    const uint4 *x = reinterpret_cast<const uint4 *>(src + row * ctx);
    uint4 *y = reinterpret_cast<uint4 *>(dst + row * ctx);
    // groups of 256 columns (one vector per lane) that lie entirely beyond the row's horizon are skipped by the whole
    // warp in every pass; they only receive zeros
    uint4 v[VPT];
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = u * 32 + lane;
        v[u] = (u * 256 < vis && idx * 8 < vis) ? x[idx] : make_uint4(0, 0, 0, 0);
    }
    // the three passes work on 32-bit words of two elements: one conversion instruction rounds a pair, the running
    // maximum is a packed maximum, and only the vector that straddles the horizon tests its columns one by one
    unsigned m2 = pack2<T>(-INFINITY, -INFINITY);
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        if (u * 256 >= vis) continue;
        const int c0 = (u * 32 + lane) * 8;
        unsigned w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        const bool edge = c0 + 8 > vis;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float2 f = unpack2<T>(w[p]);
            f.x *= scale;
            f.y *= scale;
            if (edge) {
                if (c0 + 2 * p >= vis) f.x = -INFINITY;
                if (c0 + 2 * p + 1 >= vis) f.y = -INFINITY;
            }
            w[p] = pack2<T>(f.x, f.y);
            m2 = max2<T>(m2, w[p]);
        }
        v[u] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    const float2 mm = unpack2<T>(m2);
    const float mx = warp_max(fmaxf(mm.x, mm.y));
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        if (u * 256 >= vis) continue;
        unsigned w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float2 f = unpack2<T>(w[p]);
            const float2 d = unpack2<T>(pack2<T>(f.x - mx, f.y - mx));
            // the exponential is rounded to a 16-bit type right away: the fast form (2^-21 relative) rounds to the same
            // value; a masked column holds -inf and comes out as zero
            w[p] = pack2<T>(__expf(d.x), __expf(d.y));
            const float2 e = unpack2<T>(w[p]);
            sum += e.x;
            sum += e.y;
        }
        v[u] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    sum = warp_sum(sum);
    const float inv = __fdividef(1.0f, sum);
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const int idx = u * 32 + lane;
        if (idx >= nvec || idx * 8 >= zend) continue;
        unsigned w[4] = {0u, 0u, 0u, 0u};
        if (u * 256 < vis) {
            const unsigned s[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float2 e = unpack2<T>(s[p]);
                w[p] = pack2<T>(e.x * inv, e.y * inv);
            }
        }
        y[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// dst_p[row][col_offset + c] = src element (row, c) for every destination p: the all-gather of a locally computed
// [m, n] slice into the [m, ldy] result of every rank (destinations are the rank's own buffer and its peers', mapped
// into this process; plain 16-byte stores over NVLink, or ONE multimem.st per piece when `mc` is set and dsts[0]
// is an NVLink multicast address).  The source is [groups][m][n / groups] (groups = 1: plain row-major [m, n]).
struct ScatterArgs {
    void *dst[8];
    int ndst, mc;
};
__global__ void __launch_bounds__(256)
scatter_columns_kernel(ScatterArgs a, const unsigned char *__restrict__ src, size_t m, size_t row_bytes, size_t group_row_bytes,
                       size_t ldy_bytes, size_t col_offset_bytes) {
    const size_t chunks_per_row = row_bytes / 16, total = m * chunks_per_row;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / chunks_per_row, cb = (i - row * chunks_per_row) * 16;
        const size_t g = cb / group_row_bytes, within = cb - g * group_row_bytes;
        const uint4 v = *reinterpret_cast<const uint4 *>(src + (g * m + row) * group_row_bytes + within);
        const size_t off = row * ldy_bytes + col_offset_bytes + cb;
        if (a.mc) {
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                             static_cast<unsigned char *>(a.dst[0]) + off),
                         "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                         : "memory");
        } else {
            for (int p = 0; p < a.ndst; ++p) *reinterpret_cast<uint4 *>(static_cast<unsigned char *>(a.dst[p]) + off) = v;
        }
    }
}
}  // namespace
}  // namespace xn

using namespace xn;

extern "C" int xn_mm_rms_norm(xn_dtype dtype, void *dst, const void *src, const void *alpha, size_t rows, size_t cols,
                              float eps, void *stream) {
    XN_API_RANGE("xn_mm_rms_norm");
    XN_REQUIRE(valid_dtype(dtype), "rms_norm: unknown dtype %d", (int)dtype);
    if (rows == 0 || cols == 0) return XN_OK;
    XN_REQUIRE(dst && src && alpha, "rms_norm: null pointer");
    XN_REQUIRE(rows <= 0x7fffffffull, "rms_norm: too many rows");
    XN_DISPATCH_DTYPE(dtype, T,
        if (!launch_rms_norm_vec<T, false>((T *)dst, nullptr, nullptr, nullptr, (const T *)src, (const T *)alpha, rows, cols, eps,
                                           nullptr, nullptr, (cudaStream_t)stream))
            rms_norm_kernel<T, false><<<(unsigned)rows, NT, 0, (cudaStream_t)stream>>>(
                (T *)dst, nullptr, nullptr, nullptr, (const T *)src, (const T *)alpha, cols, eps));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_rms_norm_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *dst_or_null,
                                         const void *src, const void *alpha, xn_dtype dtype, size_t rows, size_t cols,
                                         float eps, void *stream) {
    XN_API_RANGE("xn_mm_rms_norm_split_e4m3");
    XN_REQUIRE(valid_dtype(dtype), "rms_norm_split: unknown dtype %d", (int)dtype);
    if (rows == 0 || cols == 0) return XN_OK;
    XN_REQUIRE(x_hi && x_scale && src && alpha, "rms_norm_split: null pointer");
    XN_REQUIRE(rows <= 0x7fffffffull, "rms_norm_split: too many rows");
    XN_DISPATCH_DTYPE(dtype, T,
        if (!launch_rms_norm_vec<T, true>((T *)dst_or_null, x_hi, x_lo, x_scale, (const T *)src, (const T *)alpha, rows, cols, eps,
                                          nullptr, nullptr, (cudaStream_t)stream))
            rms_norm_kernel<T, true><<<(unsigned)rows, NT, 0, (cudaStream_t)stream>>>(
                (T *)dst_or_null, x_hi, x_lo, x_scale, (const T *)src, (const T *)alpha, cols, eps));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_add_rms_norm_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *sum_out, const void *a,
                                             const void *b, const void *alpha, xn_dtype dtype, size_t rows, size_t cols,
                                             float eps, void *stream) {
    XN_API_RANGE("xn_mm_add_rms_norm_split_e4m3");
    XN_REQUIRE(valid_dtype(dtype), "add_rms_norm_split: unknown dtype %d", (int)dtype);
    if (rows == 0 || cols == 0) return XN_OK;
    XN_REQUIRE(x_hi && x_scale && sum_out && a && b && alpha, "add_rms_norm_split: null pointer");
    XN_REQUIRE(rows <= 0x7fffffffull, "add_rms_norm_split: too many rows");
    XN_DISPATCH_DTYPE(dtype, T,
        if (!launch_rms_norm_vec<T, true>((T *)nullptr, x_hi, x_lo, x_scale, (const T *)a, (const T *)alpha, rows, cols, eps,
                                          (const T *)b, (T *)sum_out, (cudaStream_t)stream))
            rms_norm_kernel<T, true><<<(unsigned)rows, NT, 0, (cudaStream_t)stream>>>(
                (T *)nullptr, x_hi, x_lo, x_scale, (const T *)a, (const T *)alpha, cols, eps, (const T *)b, (T *)sum_out));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_softmax(xn_dtype dtype, void *dst, const void *src, size_t rows, size_t cols, void *stream) {
    XN_API_RANGE("xn_mm_softmax");
    XN_REQUIRE(valid_dtype(dtype), "softmax: unknown dtype %d", (int)dtype);
    if (rows == 0 || cols == 0) return XN_OK;
    XN_REQUIRE(dst && src, "softmax: null pointer");
    const size_t blocks = (rows + 7) / 8;
    XN_REQUIRE(blocks <= 0x7fffffffull, "softmax: too many rows");
    XN_DISPATCH_DTYPE(dtype, T, softmax_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
                                    (T *)dst, (const T *)src, rows, cols));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_silu_mul(xn_dtype dtype, void *dst, const void *src, size_t rows, size_t hidden, void *stream) {
    XN_API_RANGE("xn_mm_silu_mul");
    XN_REQUIRE(valid_dtype(dtype), "silu_mul: unknown dtype %d", (int)dtype);
    if (rows == 0 || hidden == 0) return XN_OK;
    XN_REQUIRE(dst && src, "silu_mul: null pointer");
    XN_REQUIRE(rows <= 0x7fffffffull, "silu_mul: too many rows");
    XN_DISPATCH_DTYPE(dtype, T,
        if (!launch_silu_mul_vec<T, false>((T *)dst, nullptr, nullptr, nullptr, (const T *)src, rows, hidden, (cudaStream_t)stream))
            silu_mul_kernel<T, false><<<(unsigned)rows, NT, 0, (cudaStream_t)stream>>>(
                (T *)dst, nullptr, nullptr, nullptr, (const T *)src, hidden));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_silu_mul_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, const void *src,
                                         xn_dtype dtype, size_t rows, size_t hidden, void *stream) {
    XN_API_RANGE("xn_mm_silu_mul_split_e4m3");
    XN_REQUIRE(valid_dtype(dtype), "silu_mul_split: unknown dtype %d", (int)dtype);
    if (rows == 0 || hidden == 0) return XN_OK;
    XN_REQUIRE(x_hi && x_scale && src, "silu_mul_split: null pointer");
    XN_REQUIRE(rows <= 0x7fffffffull, "silu_mul_split: too many rows");
    XN_DISPATCH_DTYPE(dtype, T,
        if (!launch_silu_mul_vec<T, true>((T *)nullptr, x_hi, x_lo, x_scale, (const T *)src, rows, hidden, (cudaStream_t)stream))
            silu_mul_kernel<T, true><<<(unsigned)rows, NT, 0, (cudaStream_t)stream>>>(
                (T *)nullptr, x_hi, x_lo, x_scale, (const T *)src, hidden));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_add(xn_dtype dtype, void *dst, const void *a, const void *b, size_t len, void *stream) {
    XN_API_RANGE("xn_mm_add");
    XN_REQUIRE(valid_dtype(dtype), "add: unknown dtype %d", (int)dtype);
    if (len == 0) return XN_OK;
    XN_REQUIRE(dst && a && b, "add: null pointer");
    const size_t blocks = (len + 255) / 256;
    XN_REQUIRE(blocks <= 0x7fffffffull, "add: too many elements");
    XN_DISPATCH_DTYPE(dtype, T, add_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
                                    (T *)dst, (const T *)a, (const T *)b, len));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

// dst[r][c] = src[r][c] + bias[c]: the broadcast_add that follows Linear::forward's matmul
// (xn-core/src/nn/linear.rs:61-64); the sum is formed in f32 and rounded once to the element type, as the
// reference's binary Add does for f16 / bf16.  dst may alias src.
// Both caches in one launch: blockIdx.y = 0 appends to the key cache, 1 to the value cache.
template <typename T>
__global__ void kv_append2_kernel(T *__restrict__ k_cache, T *__restrict__ v_cache, const T *__restrict__ k_src,
                                  const T *__restrict__ v_src, const int64_t *__restrict__ idx, size_t heads, size_t context,
                                  size_t hd, size_t src_batch_stride, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    T *cache = blockIdx.y ? v_cache : k_cache;
    const T *src = blockIdx.y ? v_src : k_src;
    const size_t d = i % hd, h = (i / hd) % heads, b = i / (hd * heads);
    const int64_t p = idx[b];
    if (p < 0 || (size_t)p >= context) return;  // out-of-range index: nothing is written
    cache[((b * heads + h) * context + (size_t)p) * hd + d] = src[b * src_batch_stride + h * hd + d];
}

template <typename T>
__global__ void __launch_bounds__(256) add_bias_kernel(T *dst, const T *src, const T *__restrict__ bias, size_t cols, size_t len) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < len; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = from_f32<T>(to_f32(src[i]) + to_f32(bias[i % cols]));
}

extern "C" int xn_mm_add_bias(xn_dtype dtype, void *dst, const void *src, const void *bias, size_t rows, size_t cols,
                              void *stream) {
    XN_API_RANGE("xn_mm_add_bias");
    XN_REQUIRE(valid_dtype(dtype), "add_bias: unknown dtype %d", (int)dtype);
    const size_t len = rows * cols;
    if (len == 0) return XN_OK;
    XN_REQUIRE(dst && src && bias, "add_bias: null pointer");
    const size_t blocks = (len + 255) / 256;
    const unsigned grid = (unsigned)(blocks < (size_t)sm_count() * 32 ? blocks : (size_t)sm_count() * 32);
    XN_DISPATCH_DTYPE(dtype, T, add_bias_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((T *)dst, (const T *)src,
                                                                                          (const T *)bias, cols, len));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_kv_append(xn_dtype dtype, void *cache, const void *src, size_t src_batch_stride,
                               const int64_t *index, size_t batch, size_t heads, size_t context, size_t head_dim,
                               void *stream) {
    XN_API_RANGE("xn_mm_kv_append");
    XN_REQUIRE(valid_dtype(dtype), "kv_append: unknown dtype %d", (int)dtype);
    const size_t total = batch * heads * head_dim;
    if (total == 0) return XN_OK;
    XN_REQUIRE(cache && src && index, "kv_append: null pointer");
    const size_t blocks = (total + 255) / 256;
    XN_REQUIRE(blocks <= 0x7fffffffull, "kv_append: too many elements");
    XN_DISPATCH_DTYPE(dtype, T, kv_append_kernel<T><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
                                    (T *)cache, (const T *)src, index, heads, context, head_dim, src_batch_stride, total));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

namespace {
// Slices of the context per (stream, head).  The kernel keeps two sets of loads per warp in flight (96 registers:
// five CTAs per SM), so 32 streams x 32 heads as one slice each would be 1024 CTAs on 740 slots -- a full wave and
// a 38 % one.  The context is therefore cut until there are six to seven CTAs per slot (the hardware hands the next
// slice to whichever slot frees up first, so the tail is a fraction of one short slice), each slice at least 128
// rows; the log-sum-exp combine of the slices moves a few MB.  Measured on the 32-layer decode step (32 streams x
// 32 heads x 3000 rows): 3 / 4 / 5 / 6 / 7 / 9 slices per head = 10.51 / 10.41 / 10.20-10.27 / 10.41 / 10.41 / 10.36 ms.
int attention_splits(size_t batch, size_t heads, size_t context) {
    const size_t slots = (size_t)sm_count() * 5, bh = batch * heads;
    static const size_t per_slot = [] { const char *e = getenv("XN_ATTN_CTAS_PER_SLOT"); return (size_t)(e ? atoi(e) : 6); }();
    size_t s = (slots * per_slot + bh - 1) / bh;
    if (s > context / 128) s = context / 128;
    if (s > 32) s = 32;
    return s < 1 ? 1 : (int)s;
}

int decode_attention_impl(void *out_bf16, const void *q_bf16, size_t q_batch_stride, const void *k_cache_bf16,
                          const void *v_cache_bf16, const float *mask_or_null, size_t batch, size_t heads, size_t context,
                          size_t head_dim, float scale, void *workspace, size_t workspace_bytes, bool use_ws, void *stream,
                          uint8_t *x_hi = nullptr, uint8_t *x_lo = nullptr, float *x_scale = nullptr) {
    XN_REQUIRE(head_dim == 128, "decode_attention: head_dim %zu is not supported (128 only)", head_dim);
    if (batch == 0 || heads == 0) return XN_OK;
    XN_REQUIRE(context > 0, "decode_attention: empty context");
    XN_REQUIRE(out_bf16 && q_bf16 && k_cache_bf16 && v_cache_bf16, "decode_attention: null pointer");
    XN_REQUIRE(aligned(q_bf16, 16) && aligned(k_cache_bf16, 16) && aligned(v_cache_bf16, 16) && q_batch_stride % 8 == 0,
               "decode_attention: q and the caches must be 16-byte aligned (q_batch_stride a multiple of 8)");
    XN_REQUIRE(batch * heads <= 0x7fffffffull, "decode_attention: too many (stream, head) pairs");
    int splits = use_ws ? attention_splits(batch, heads, context) : 1;
    if (splits > 1) {
        const size_t need = batch * heads * splits * (HD + 2) * sizeof(float);
        if (workspace_bytes < need || !workspace)
            return fail(XN_ERR_WORKSPACE, "decode_attention_split: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        XN_REQUIRE(aligned(workspace, 4), "decode_attention_split: workspace must be 4-byte aligned");
    }
    const size_t rows_per_split = ((context + splits - 1) / splits + 31) / 32 * 32;
    splits = (int)((context + rows_per_split - 1) / rows_per_split);
    cudaStream_t st = (cudaStream_t)stream;
    if (splits > 1)
        decode_attention_kernel<true><<<dim3((unsigned)(batch * heads), (unsigned)splits), 128, 0, st>>>(
            (__nv_bfloat16 *)out_bf16, (const __nv_bfloat16 *)q_bf16, (const __nv_bfloat16 *)k_cache_bf16,
            (const __nv_bfloat16 *)v_cache_bf16, mask_or_null, heads, context, q_batch_stride, scale, rows_per_split,
            (float *)workspace);
    else
        decode_attention_kernel<false><<<(unsigned)(batch * heads), 128, 0, st>>>(
            (__nv_bfloat16 *)out_bf16, (const __nv_bfloat16 *)q_bf16, (const __nv_bfloat16 *)k_cache_bf16,
            (const __nv_bfloat16 *)v_cache_bf16, mask_or_null, heads, context, q_batch_stride, scale, context, nullptr);
    XN_CHECK_CUDA(cudaGetLastError());
    if (splits > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(batch * heads));
        cfg.blockDim = dim3(HD);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;
        if (x_hi && heads <= 64) {  // merge + e4m3 split of the whole row in one launch
            cfg.gridDim = dim3((unsigned)batch);
            cfg.blockDim = dim3(1024);
            XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, xn::decode_attention_combine_split_kernel, (__nv_bfloat16 *)out_bf16, x_hi, x_lo,
                                             x_scale, (const float *)workspace, splits, (int)heads));
            return XN_OK;
        }
        XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, decode_attention_combine_kernel, (__nv_bfloat16 *)out_bf16,
                                         (const float *)workspace, splits));
    }
    if (x_hi) return xn_mm_split_rows_e4m3(x_hi, x_lo, x_scale, out_bf16, XN_BF16, batch, heads * head_dim, stream);
    return XN_OK;
}
}  // namespace

extern "C" size_t xn_mm_decode_attention_workspace_bytes(size_t batch, size_t heads, size_t context) {
    if (batch == 0 || heads == 0 || context == 0) return 0;
    const int splits = attention_splits(batch, heads, context);
    return splits > 1 ? batch * heads * splits * (HD + 2) * sizeof(float) : 0;
}

extern "C" int xn_mm_decode_attention_split(void *out_bf16, const void *q_bf16, size_t q_batch_stride,
                                            const void *k_cache_bf16, const void *v_cache_bf16, const float *mask_or_null,
                                            size_t batch, size_t heads, size_t context, size_t head_dim, float scale,
                                            void *workspace, size_t workspace_bytes, void *stream) {
    XN_API_RANGE("xn_mm_decode_attention_split");
    return decode_attention_impl(out_bf16, q_bf16, q_batch_stride, k_cache_bf16, v_cache_bf16, mask_or_null, batch, heads,
                                 context, head_dim, scale, workspace, workspace_bytes, true, stream);
}

extern "C" int xn_mm_decode_attention_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *out_bf16,
                                                 const void *q_bf16, size_t q_batch_stride, const void *k_cache_bf16,
                                                 const void *v_cache_bf16, const float *mask_or_null, size_t batch,
                                                 size_t heads, size_t context, size_t head_dim, float scale, void *workspace,
                                                 size_t workspace_bytes, void *stream) {
    XN_API_RANGE("xn_mm_decode_attention_split_e4m3");
    XN_REQUIRE(x_hi && x_scale, "decode_attention_split_e4m3: null pointer");
    XN_REQUIRE(aligned(x_hi, 4) && (!x_lo || aligned(x_lo, 4)), "decode_attention_split_e4m3: pieces must be 4-byte aligned");
    return decode_attention_impl(out_bf16, q_bf16, q_batch_stride, k_cache_bf16, v_cache_bf16, mask_or_null, batch, heads,
                                 context, head_dim, scale, workspace, workspace_bytes, true, stream, x_hi, x_lo, x_scale);
}

extern "C" int xn_mm_kv_append2(xn_dtype dtype, void *k_cache, void *v_cache, const void *k_src, const void *v_src,
                                size_t src_batch_stride, const int64_t *index, size_t batch, size_t heads, size_t context,
                                size_t head_dim, void *stream) {
    XN_API_RANGE("xn_mm_kv_append2");
    XN_REQUIRE(valid_dtype(dtype), "kv_append2: unknown dtype %d", (int)dtype);
    const size_t total = batch * heads * head_dim;
    if (total == 0) return XN_OK;
    XN_REQUIRE(k_cache && v_cache && k_src && v_src && index, "kv_append2: null pointer");
    const size_t blocks = (total + 255) / 256;
    XN_REQUIRE(blocks <= 0x7fffffffull, "kv_append2: too many elements");
    XN_DISPATCH_DTYPE(dtype, T, kv_append2_kernel<T><<<dim3((unsigned)blocks, 2), 256, 0, (cudaStream_t)stream>>>(
                                    (T *)k_cache, (T *)v_cache, (const T *)k_src, (const T *)v_src, index, heads, context, head_dim,
                                    src_batch_stride, total));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" size_t xn_mm_decode_attention_append_workspace_bytes(size_t batch, size_t heads, size_t context) {
    if (batch == 0 || heads == 0 || context == 0) return 0;
    return batch * heads * (size_t)attention_splits(batch, heads, context) * (HD + 2) * sizeof(float);
}

extern "C" int xn_mm_decode_attention_append_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *out_bf16,
                                                  const void *q_bf16, const void *k_new_bf16, const void *v_new_bf16,
                                                  size_t qkv_batch_stride, void *k_cache_bf16, void *v_cache_bf16,
                                                  const int64_t *index, const float *mask_or_null, size_t batch, size_t heads,
                                                  size_t context, size_t head_dim, float scale, int merge, void *workspace,
                                                  size_t workspace_bytes, void *stream) {
    XN_API_RANGE("xn_mm_decode_attention_append_e4m3");
    XN_REQUIRE(merge >= 0 && merge <= 2, "decode_attention_append: merge=%d (0 = library decides, 1 = in the kernel, 2 = own launch)", merge);
    XN_REQUIRE(head_dim == 128, "decode_attention_append: head_dim %zu is not supported (128 only)", head_dim);
    if (batch == 0 || heads == 0) return XN_OK;
    XN_REQUIRE(context > 0, "decode_attention_append: empty context");
    XN_REQUIRE(out_bf16 && q_bf16 && k_new_bf16 && v_new_bf16 && k_cache_bf16 && v_cache_bf16 && index,
               "decode_attention_append: null pointer");
    XN_REQUIRE((x_hi != nullptr) == (x_scale != nullptr) && (x_hi || !x_lo), "decode_attention_append: pieces and scales go together");
    XN_REQUIRE(aligned(q_bf16, 16) && aligned(k_new_bf16, 16) && aligned(v_new_bf16, 16) && aligned(k_cache_bf16, 16) &&
                   aligned(v_cache_bf16, 16) && qkv_batch_stride % 8 == 0,
               "decode_attention_append: q, the new rows and the caches must be 16-byte aligned (batch stride a multiple of 8)");
    XN_REQUIRE(aligned(out_bf16, 8) && (!x_hi || aligned(x_hi, 4)) && (!x_lo || aligned(x_lo, 4)),
               "decode_attention_append: output row must be 8-byte, pieces 4-byte aligned");
    XN_REQUIRE(batch * heads <= 0x7fffffffull, "decode_attention_append: too many (stream, head) pairs");
    XN_REQUIRE(context <= 0x7fffffffull, "decode_attention_append: context %zu too long", context);
    int splits = attention_splits(batch, heads, context);
    const size_t need = batch * heads * (size_t)splits * (HD + 2) * sizeof(float);
    if (workspace_bytes < need || !workspace)
        return fail(XN_ERR_WORKSPACE, "decode_attention_append: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    XN_REQUIRE(aligned(workspace, 4), "decode_attention_append: workspace must be 4-byte aligned");
    const size_t rows_per_split = ((context + splits - 1) / splits + 31) / 32 * 32;
    splits = (int)((context + rows_per_split - 1) / rows_per_split);
    cudaStream_t st = (cudaStream_t)stream;
    // Where the merge runs.  Inside the attention kernel every CTA ends with a fence and an arrival (about 1.4 us
    // during which its slot streams nothing); with many short slices per slot that costs more than the merge kernel's
    // launch saves (32 streams x 32 heads x 3000 rows, 4864 CTAs: decode step 10.83 ms merged in the kernel against
    // 10.5 ms with the merge as its own launch), so the library fuses the merge only when a slot sees at most two CTAs.
    bool in_kernel = batch * heads * (size_t)splits <= (size_t)sm_count() * 5 * 2;
    if (merge) in_kernel = merge == 1;
    if (in_kernel) {
        SkinnyScratch sc;  // arrival counters: one per (stream, head), one per stream; zero between launches
        if (int rc = skinny_scratch(st, 0, batch * heads + batch, &sc)) return rc;
        decode_attention_append_kernel<true><<<dim3((unsigned)(batch * heads), (unsigned)splits), 128, 0, st>>>(
            (__nv_bfloat16 *)out_bf16, x_hi, x_lo, x_scale, (const __nv_bfloat16 *)q_bf16, (const __nv_bfloat16 *)k_new_bf16,
            (const __nv_bfloat16 *)v_new_bf16, (__nv_bfloat16 *)k_cache_bf16, (__nv_bfloat16 *)v_cache_bf16, index, mask_or_null,
            heads, context, qkv_batch_stride, scale, rows_per_split, (float *)workspace, sc.counters, sc.counters + batch * heads);
        XN_CHECK_CUDA(cudaGetLastError());
        return XN_OK;
    }
    decode_attention_append_kernel<false><<<dim3((unsigned)(batch * heads), (unsigned)splits), 128, 0, st>>>(
        (__nv_bfloat16 *)out_bf16, x_hi, x_lo, x_scale, (const __nv_bfloat16 *)q_bf16, (const __nv_bfloat16 *)k_new_bf16,
        (const __nv_bfloat16 *)v_new_bf16, (__nv_bfloat16 *)k_cache_bf16, (__nv_bfloat16 *)v_cache_bf16, index, mask_or_null,
        heads, context, qkv_batch_stride, scale, rows_per_split, (float *)workspace, nullptr, nullptr);
    XN_CHECK_CUDA(cudaGetLastError());
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    if (x_hi && heads <= 64) {  // merge + e4m3 split of the whole row in one launch
        cfg.gridDim = dim3((unsigned)batch);
        cfg.blockDim = dim3(1024);
        XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, xn::decode_attention_combine_split_kernel, (__nv_bfloat16 *)out_bf16, x_hi, x_lo,
                                         x_scale, (const float *)workspace, splits, (int)heads));
        return XN_OK;
    }
    cfg.gridDim = dim3((unsigned)(batch * heads));
    cfg.blockDim = dim3(HD);
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, decode_attention_combine_kernel, (__nv_bfloat16 *)out_bf16, (const float *)workspace,
                                     splits));
    if (x_hi) return xn_mm_split_rows_e4m3(x_hi, x_lo, x_scale, out_bf16, XN_BF16, batch, heads * head_dim, stream);
    return XN_OK;
}

extern "C" int xn_mm_decode_attention(void *out_bf16, const void *q_bf16, size_t q_batch_stride,
                                      const void *k_cache_bf16, const void *v_cache_bf16, const float *mask_or_null,
                                      size_t batch, size_t heads, size_t context, size_t head_dim, float scale,
                                      void *stream) {
    XN_API_RANGE("xn_mm_decode_attention");
    return decode_attention_impl(out_bf16, q_bf16, q_batch_stride, k_cache_bf16, v_cache_bf16, mask_or_null, batch, heads,
                                 context, head_dim, scale, nullptr, 0, false, stream);
}

extern "C" int xn_mm_softmax_causal(xn_dtype dtype, void *dst, const void *src, size_t batch, size_t t_rows, size_t context,
                                    float scale, int zero_fill_all, void *stream) {
    XN_API_RANGE("xn_mm_softmax_causal");
    XN_REQUIRE(valid_dtype(dtype), "softmax_causal: unknown dtype %d", (int)dtype);
    if (batch == 0 || t_rows == 0 || context == 0) return XN_OK;
    XN_REQUIRE(dst && src, "softmax_causal: null pointer");
    XN_REQUIRE(t_rows <= context, "softmax_causal: %zu query rows but only %zu keys", t_rows, context);
    XN_REQUIRE(batch * t_rows <= 0x7fffffffull, "softmax_causal: too many rows");
    if (dtype != XN_F32 && context % 8 == 0 && context <= 8 * 32 * 16 && aligned(src, 16) && aligned(dst, 16)) {
        const size_t rows = batch * t_rows;
        const unsigned grid = (unsigned)((rows + 7) / 8);
        cudaStream_t st = (cudaStream_t)stream;
        const int vpt = context <= 1024 ? 4 : (context <= 2048 ? 8 : 16);
#define XN_SMW(T, V) xn::softmax_causal_warp_kernel<T, V><<<grid, 256, 0, st>>>((T *)dst, (const T *)src, rows, t_rows, context, scale, zero_fill_all)
        if (dtype == XN_BF16) { if (vpt == 4) XN_SMW(__nv_bfloat16, 4); else if (vpt == 8) XN_SMW(__nv_bfloat16, 8); else XN_SMW(__nv_bfloat16, 16); }
        else { if (vpt == 4) XN_SMW(__half, 4); else if (vpt == 8) XN_SMW(__half, 8); else XN_SMW(__half, 16); }
#undef XN_SMW
        XN_CHECK_CUDA(cudaGetLastError());
        return XN_OK;
    }
    if (dtype != XN_F32 && context % 8 == 0 && context <= 8 * 256 * 4 && aligned(src, 16) && aligned(dst, 16)) {
        const unsigned grid = (unsigned)(batch * t_rows);
        cudaStream_t st = (cudaStream_t)stream;
        const int vpt = context <= 2048 ? 1 : (context <= 4096 ? 2 : 4);
#define XN_SMC(T, V) xn::softmax_causal_vec_kernel<T, V><<<grid, 256, 0, st>>>((T *)dst, (const T *)src, t_rows, context, scale, zero_fill_all)
        if (dtype == XN_BF16) { if (vpt == 1) XN_SMC(__nv_bfloat16, 1); else if (vpt == 2) XN_SMC(__nv_bfloat16, 2); else XN_SMC(__nv_bfloat16, 4); }
        else { if (vpt == 1) XN_SMC(__half, 1); else if (vpt == 2) XN_SMC(__half, 2); else XN_SMC(__half, 4); }
#undef XN_SMC
        XN_CHECK_CUDA(cudaGetLastError());
        return XN_OK;
    }
    XN_DISPATCH_DTYPE(dtype, T, xn::softmax_causal_kernel<T><<<(unsigned)(batch * t_rows), 256, 0, (cudaStream_t)stream>>>(
                                    (T *)dst, (const T *)src, t_rows, context, scale, zero_fill_all));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

extern "C" int xn_mm_scatter_columns(void *const *dsts, size_t num_dst, int multicast, size_t ldy_bytes, size_t col_offset_bytes,
                                     const void *src, size_t m, size_t row_bytes, size_t groups, void *stream) {
    XN_API_RANGE("xn_mm_scatter_columns");
    XN_REQUIRE(num_dst >= 1 && num_dst <= 8, "scatter_columns: %zu destinations (1..8 supported)", num_dst);
    XN_REQUIRE(!multicast || num_dst == 1, "scatter_columns: a multicast address is one destination");
    if (m == 0 || row_bytes == 0) return XN_OK;
    XN_REQUIRE(dsts && src, "scatter_columns: null pointer");
    XN_REQUIRE(groups >= 1 && row_bytes % groups == 0 && (row_bytes / groups) % 16 == 0 && ldy_bytes % 16 == 0 &&
                   col_offset_bytes % 16 == 0 && aligned(src, 16),
               "scatter_columns: rows, groups, pitch and offset must be multiples of 16 bytes");
    XN_REQUIRE(col_offset_bytes + row_bytes <= ldy_bytes, "scatter_columns: slice does not fit the destination row");
    xn::ScatterArgs a{};
    for (size_t p = 0; p < num_dst; ++p) {
        XN_REQUIRE(dsts[p] && aligned(dsts[p], 16), "scatter_columns: destination %zu is null or not 16-byte aligned", p);
        a.dst[p] = dsts[p];
    }
    a.ndst = (int)num_dst;
    a.mc = multicast ? 1 : 0;
    const size_t total = m * (row_bytes / 16);
    const size_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < (size_t)sm_count() * 8 ? blocks : (size_t)sm_count() * 8);
    xn::scatter_columns_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a, (const unsigned char *)src, m, row_bytes, row_bytes / groups,
                                                                       ldy_bytes, col_offset_bytes);
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}
