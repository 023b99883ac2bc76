// fp8-e4m3 weight linear for decode-sized batches (M <= 16 per pass): weight streaming with the
// weights used as stored -- no dequantization instructions at all.  No counterpart in the
// reference; contract in include/xn_mm.h.
//
// The activation row x (bf16) is represented as s * (hi + lo) with hi, lo in e4m3 and s a power of
// two, so x . w = s * (hi . w + lo . w) and both dot products are e4m3 x e4m3 tensor-core MMAs
// (m16n8k32, f32 accumulate) whose products are exact in f32.  A 128-bit load of 16 weight bytes
// per lane feeds two MMAs directly: the MMA's k positions are a fixed permutation of memory order,
// applied identically to the activation fragment, which shared memory serves as one 128-bit read
// of 16 contiguous bytes of the activation row.  Output rows ride the MMA's 16-row dimension; the
// activation rows its 8 columns (two column groups for M = 9..16).
//
// Work split as in the int4 path: `tpc` consecutive 16-row tiles per CTA, `ksplit` warps per tile
// reduced in a fixed order.  When the activation pieces do not fit in shared memory at once, k is
// walked in chunks.
#include "common.cuh"

namespace xn {
namespace {

constexpr int MAX_WARPS = 20;
constexpr int SMEM_BUDGET = 200 * 1024;

__device__ __forceinline__ void mma_e4m3(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool pred) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    int sz = pred ? 16 : 0;  // size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz));
}

// row stride of the staged activation pieces: k chunk rounded to 128, plus 64, so that the eight
// rows a quarter-warp reads fall in distinct 16-byte bank groups
__host__ __device__ inline int x_row_stride(int kc) { return (kc + 127) / 128 * 128 + 64; }

template <int MT, bool LO>
__global__ void __launch_bounds__(MAX_WARPS * 32)
linear_fp8_gemv_kernel(__nv_bfloat16 *__restrict__ y, const uint8_t *__restrict__ x_hi,
                       const uint8_t *__restrict__ x_lo, const float *__restrict__ x_scale,
                       const uint8_t *__restrict__ wq, const float *__restrict__ w_scale, int m, size_t n,
                       int k, int kchunk, int tiles, int tpc, int slots, int ksplit) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = x_row_stride(kchunk);
    unsigned char *sHi = smem;
    unsigned char *sLo = smem + (size_t)MT * 8 * RS;
    float *red = reinterpret_cast<float *>(smem + (size_t)(LO ? 2 : 1) * MT * 8 * RS);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int slot = warp / ksplit, ks = warp % ksplit;
    constexpr int MAX_ITERS = 1;  // launch() gives every tile of the CTA its own warp slot
    const int iters = 1;
    float acc[MAX_ITERS][MT][4];
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[it][mt][i] = 0.0f;

    for (int kc0 = 0; kc0 < k; kc0 += kchunk) {
        const int kc = min(kchunk, k - kc0);
        if (kc0 > 0) __syncthreads();
        // stage rows [0, 8*MT) x bytes [kc0, kc0 + round64(kc)) of both pieces, zero-filled outside
        const int cols16 = (kc + 63) / 64 * 4;
        for (int idx = tid; idx < MT * 8 * cols16; idx += blockDim.x) {
            const int row = idx / cols16, c = idx % cols16;
            const bool ok = row < m && c * 16 < kc;
            const size_t src = ok ? (size_t)row * k + kc0 + c * 16 : 0;
            cp_async16(sHi + (size_t)row * RS + c * 16, x_hi + src, ok);
            if (LO) cp_async16(sLo + (size_t)row * RS + c * 16, x_lo + src, ok);
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        const int nst = (kc + 63) / 64;  // 64-k steps in this chunk
        const int st0 = (int)((long long)nst * ks / ksplit), st1 = (int)((long long)nst * (ks + 1) / ksplit);
#pragma unroll
        for (int it = 0; it < MAX_ITERS; ++it) {
            if (it >= iters) break;
            const int tl = it * slots + slot;
            const int tile = blockIdx.x * tpc + tl;
            if (tl >= tpc || tile >= tiles) continue;
            const size_t r0 = min((size_t)tile * 16 + g, n - 1), r1 = min((size_t)tile * 16 + g + 8, n - 1);
            const uint8_t *wp0 = wq + r0 * k + kc0 + 16 * t;
            const uint8_t *wp1 = wq + r1 * k + kc0 + 16 * t;
            constexpr int U = 4;
            for (int st = st0; st < st1; st += U) {
                uint4 w0[U], w1[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int s = min(st + u, st1 - 1);
                    if (s * 64 + 16 * t < kc) {
                        w0[u] = ldg_stream(wp0 + (size_t)s * 64);
                        w1[u] = ldg_stream(wp1 + (size_t)s * 64);
                    } else {
                        w0[u] = make_uint4(0, 0, 0, 0);
                        w1[u] = make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (st + u >= st1) break;
                    const int off = (st + u) * 64 + 16 * t;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint4 bh = *reinterpret_cast<const uint4 *>(sHi + (size_t)(8 * mt + g) * RS + off);
                        mma_e4m3(acc[it][mt], w0[u].x, w1[u].x, w0[u].y, w1[u].y, bh.x, bh.y);
                        mma_e4m3(acc[it][mt], w0[u].z, w1[u].z, w0[u].w, w1[u].w, bh.z, bh.w);
                        if (LO) {
                            const uint4 bl = *reinterpret_cast<const uint4 *>(sLo + (size_t)(8 * mt + g) * RS + off);
                            mma_e4m3(acc[it][mt], w0[u].x, w1[u].x, w0[u].y, w1[u].y, bl.x, bl.y);
                            mma_e4m3(acc[it][mt], w0[u].z, w1[u].z, w0[u].w, w1[u].w, bl.z, bl.w);
                        }
                    }
                }
            }
        }
    }

    // fixed-order reduction over the ksplit warps of each slot, then the scaled bf16 store
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it) {
        if (it >= iters) break;
        if (ksplit > 1) {
            __syncthreads();
            if (ks > 0)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) red[((size_t)warp * MT * 4 + mt * 4 + i) * 32 + lane] = acc[it][mt][i];
            __syncthreads();
            if (ks == 0)
                for (int o = 1; o < ksplit; ++o)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            acc[it][mt][i] += red[((size_t)(warp + o) * MT * 4 + mt * 4 + i) * 32 + lane];
        }
        const int tl = it * slots + slot;
        const int tile = blockIdx.x * tpc + tl;
        if (ks == 0 && tl < tpc && tile < tiles) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const size_t row_n = (size_t)tile * 16 + g + 8 * (i >> 1);
                    const int row_m = 8 * mt + 2 * t + (i & 1);
                    if (row_n < n && row_m < m)
                        y[(size_t)row_m * n + row_n] =
                            __float2bfloat16_rn(w_scale[row_n] * (x_scale[row_m] * acc[it][mt][i]));
                }
        }
    }
}

template <int MT, bool LO>
int launch(__nv_bfloat16 *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale, const uint8_t *wq,
           const float *w_scale, int m, size_t n, int k, cudaStream_t st) {
    const int tiles = (int)((n + 15) / 16);
    const int sms = sm_count();
    int tpc = (tiles + sms - 1) / sms;
    if (tpc > MAX_WARPS) tpc = MAX_WARPS;  // very tall weights: more CTAs than SMs
    const int slots = tpc;
    int ksplit = MAX_WARPS / slots;
    // largest k chunk (multiple of 128) whose staged pieces fit the shared-memory budget
    const int pieces = LO ? 2 : 1;
    int kchunk = (k + 127) / 128 * 128;
    while ((size_t)pieces * MT * 8 * x_row_stride(kchunk) > (size_t)SMEM_BUDGET - MAX_WARPS * MT * 4 * 32 * 4)
        kchunk = ((kchunk / 128 + 1) / 2) * 128;
    const int nst = (kchunk < k ? kchunk : k) / 64;
    if (ksplit > nst / 4) ksplit = nst / 4;
    if (ksplit < 1) ksplit = 1;
    const int warps = slots * ksplit;
    const int grid = (tiles + tpc - 1) / tpc;
    const size_t smem = (size_t)pieces * MT * 8 * x_row_stride(kchunk) + (size_t)warps * MT * 4 * 32 * sizeof(float);
    auto kern = linear_fp8_gemv_kernel<MT, LO>;
    XN_ENSURE_SMEM(kern, smem);
    kern<<<grid, warps * 32, smem, st>>>(y, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, kchunk, tiles, tpc,
                                         slots, ksplit);
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

}  // namespace

// y [m,n] bf16 from row-major e4m3 pieces; m <= 16.
int launch_linear_fp8_gemv(void *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale,
                           const uint8_t *wq, const float *w_scale, int m, size_t n, int k, cudaStream_t st) {
    __nv_bfloat16 *yy = (__nv_bfloat16 *)y;
    if (m <= 8)
        return x_lo ? launch<1, true>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st)
                    : launch<1, false>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
    return x_lo ? launch<2, true>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st)
                : launch<2, false>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
}

}  // namespace xn
