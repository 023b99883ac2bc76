// f32 matmul with many rows on the tensor-memory kernel.
//
// The reference sends an f32 Backend::gemm to cublasGemmStridedBatchedEx with CUBLAS_COMPUTE_32F
// (xn-core/src/cuda_backend.rs:2085-2150): full-precision products on the FFMA pipe, ~50 TFLOP/s on this
// part.  tcgen05 has no f32 MMA, but kind::tf32 multiplies 11-bit mantissas exactly into an f32 accumulator,
// so an f32 product is recovered from three of them: with x = x_hi + x_lo and w = w_hi + w_lo (both pieces
// on the tf32 grid), x*w = x_hi*w_hi + x_hi*w_lo + x_lo*w_hi up to 2^-21 relative.  Laid out along k --
// a row of the activations becomes (x_hi | x_hi | x_lo), a row of the weights (w_hi | w_lo | w_hi) -- the
// three products are one ordinary dot product of length 3k, and the unmodified tf32 GEMM kernel computes
// the f32 result.  The repack is one pass over each operand (any element strides: it also normalises the
// layout to k-contiguous rows); it costs 4x the operand bytes in traffic and pays for itself once the GEMM
// is compute-bound, which is why calls with up to 96 rows in matmul_t form go to the weight-streaming 3xTF32 kernel first (passes
// of 16 rows, no repacked weight); other stride patterns come here from 17 rows on.  Few output tiles with a
// long k are split along k (partials summed in a fixed order).
// The packed copies live in the library's per-(device, stream) scratch.
#include "common.cuh"

namespace xn {
namespace {

__device__ __forceinline__ float tf32_rn(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }

// out[r][0:k | k:2k | 2k:3k] from element (r, p) at in[r * rs + p * cs].  32 x 32 tiles through shared memory:
// reads run along whichever axis is contiguous in the source, writes along p.
template <bool IS_W>
__global__ void __launch_bounds__(256)
pack_tf32x3_kernel(float *__restrict__ out, const float *__restrict__ in, size_t rows, size_t k, size_t rs, size_t cs) {
    __shared__ float tile[32][33];
    const size_t r0 = (size_t)blockIdx.y * 32, p0 = (size_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const bool along_p = cs <= rs;   // source contiguous (or closer to it) along p
    for (int i = ty; i < 32; i += 8) {
        const size_t r = along_p ? r0 + i : r0 + tx, p = along_p ? p0 + tx : p0 + i;
        float v = 0.f;
        if (r < rows && p < k) v = in[r * rs + p * cs];
        if (along_p) tile[i][tx] = v; else tile[tx][i] = v;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const size_t r = r0 + i, p = p0 + tx;
        if (r < rows && p < k) {
            const float v = tile[i][tx], hi = tf32_rn(v), lo = tf32_rn(v - hi);
            float *o = out + r * 3 * k;
            o[p] = hi;
            o[k + p] = IS_W ? lo : hi;
            o[2 * k + p] = IS_W ? hi : lo;
        }
    }
}

constexpr size_t F32_TC_MAX_SCRATCH = (size_t)2 << 30;

// out[i] = sum over splits of part[s][i], in split order
__global__ void __launch_bounds__(256)
sum_partials_kernel(float *__restrict__ out, const float *__restrict__ part, int splits, size_t n, size_t ldd, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += part[(size_t)k * total + i];
        out[(i / n) * ldd + i % n] = s;
    }
}

// Few output tiles and a long k: cut k (in units of the 32-word k stage) into equal chunks so that about one
// CTA per SM has work; 1 = no split.
int k_splits(size_t m, size_t n, size_t k3) {
    if (k3 % 32) return 1;
    const size_t tiles = ((m + 127) / 128) * ((n + 127) / 128), sms = (size_t)sm_count(), units = k3 / 32;
    if (tiles == 0 || tiles * 2 > sms || units < 8) return 1;
    size_t want = sms / tiles;
    if (want > units / 4) want = units / 4;
    if (want > 32) want = 32;
    for (size_t s = want; s > 1; --s)
        if (units % s == 0) return (int)s;
    return 1;
}

}  // namespace

bool gemm_f32_tc_fits(size_t m, size_t n, size_t k) {
    static const bool off = [] { const char *e = getenv("XN_MM_F32_TC"); return e && atoi(e) == 0; }();
    static const size_t min_m = [] { const char *e = getenv("XN_MM_F32_TC_MIN_M"); return e ? (size_t)atoi(e) : (size_t)17; }();
    return !off && m >= min_m && n >= 64 && k >= 32 && k % 4 == 0 && m <= 65535 * 32 && n <= 65535 * 32 && 3 * k <= 0x7fffffff &&
           (m + n) * k * 12 + (k_splits(m, n, 3 * k) > 1 ? (size_t)k_splits(m, n, 3 * k) * m * n * 4 : 0) <= F32_TC_MAX_SCRATCH;
}

int launch_gemm_f32_tc(float *dst, const float *lhs, const float *rhs, size_t m, size_t n, size_t k, size_t dst_rs,
                       size_t lhs_cs, size_t lhs_rs, size_t rhs_cs, size_t rhs_rs, cudaStream_t st) {
    void *ws = nullptr;
    const size_t xbytes = (m * k * 12 + 255) / 256 * 256, wbytes = (n * k * 12 + 255) / 256 * 256;
    const int splits = k_splits(m, n, 3 * k);
    const size_t pbytes = splits > 1 ? (size_t)splits * m * n * 4 : 0;
    if (int rc = library_scratch(st, xbytes + wbytes + pbytes, &ws)) return rc;
    float *xp = static_cast<float *>(ws), *wp = reinterpret_cast<float *>(static_cast<unsigned char *>(ws) + xbytes);
    // lhs element (i, p) at i * lhs_rs + p * lhs_cs; rhs element (p, j) at p * rhs_rs + j * rhs_cs: row j of the
    // packed weights runs over p
    dim3 gx((unsigned)((k + 31) / 32), (unsigned)((m + 31) / 32)), gw((unsigned)((k + 31) / 32), (unsigned)((n + 31) / 32));
    pack_tf32x3_kernel<false><<<gx, 256, 0, st>>>(xp, lhs, m, k, lhs_rs, lhs_cs);
    pack_tf32x3_kernel<true><<<gw, 256, 0, st>>>(wp, rhs, n, k, rhs_cs, rhs_rs);
    XN_CHECK_CUDA(cudaGetLastError());
    if (splits > 1) {
        float *part = reinterpret_cast<float *>(static_cast<unsigned char *>(ws) + xbytes + wbytes);
        if (int rc = launch_gemm_tn_tf32_splitk(part, xp, wp, m, n, 3 * k / splits, splits, 3 * k, 3 * k, st)) return rc;
        const size_t total = m * n;
        const unsigned grid = (unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        sum_partials_kernel<<<grid, 256, 0, st>>>(dst, part, splits, n, dst_rs, total);
        XN_CHECK_CUDA(cudaGetLastError());
        return XN_OK;
    }
    return launch_gemm_tn_tf32(dst, xp, wp, m, n, 3 * k, dst_rs, st);
}

}  // namespace xn
