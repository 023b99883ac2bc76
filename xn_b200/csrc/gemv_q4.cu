// int4 block-quantized decode linear (M <= 16 per pass): the memory-bound weight-streaming path.
// No counterpart in the reference (it has no quantized matmul); the contract is in
// include/xn_mm.h.  Exact integer arithmetic: every 32-element block product is an int32.
//
// Data movement.  The packed weights are stored as 1 KB tiles of 16 output rows x 128 k so that
// one warp-wide 128-bit load is 512 contiguous bytes and lands directly in the A-fragment
// registers of an integer tensor-core MMA (m16n8k32, s8 x s8 -> s32) -- the output rows ride
// the MMA's 16-row dimension, the (at most 16) activation rows its 8-column dimension, so an
// M = 1..8 pass needs one MMA per 16 rows x 32 k and M = 9..16 two.  A 32-bit word of eight
// nibbles becomes two int8x4 operands with two logic ops: (w << 4) & 0xF0F0F0F0 and
// w & 0xF0F0F0F0 are the low / high nibbles times 16 as signed bytes; the factor 16 is
// removed exactly at the end (power of two).  The int8 activations are staged once per CTA in
// shared memory, already in B-fragment order.
//
// Work split.  A CTA owns `tpc` consecutive 16-row tiles (chosen so that the grid is about one
// CTA per SM); `ksplit` warps share a tile's k range and reduce through shared memory in a fixed
// order, so results do not depend on scheduling.
#include "common.cuh"

namespace xn {
namespace {

constexpr int MAX_WARPS = 20;

__device__ __forceinline__ void mma_s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <int MT, bool DUMP>
__global__ void __launch_bounds__(MAX_WARPS * 32)
linear_q4_kernel(float *__restrict__ y, const int8_t *__restrict__ xq, const float *__restrict__ x_scale,
                 const uint4 *__restrict__ wq, const float4 *__restrict__ ws, int m, size_t n, int k,
                 int tiles, int tpc, int slots, int ksplit, int32_t *__restrict__ partials) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int nblk = k / 32, nsb = k / 128;
    // B fragments: [nblk][32 lanes][MT] x uint2
    uint2 *sB = reinterpret_cast<uint2 *>(smem);
    float *red = reinterpret_cast<float *>(smem + (size_t)nblk * 32 * MT * sizeof(uint2));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int slot = warp / ksplit, ks = warp % ksplit;
    const int sb0 = (int)((long long)nsb * ks / ksplit), sb1 = (int)((long long)nsb * (ks + 1) / ksplit);

    // Stage the activations in fragment order: entry (kb, lane, mt) = the two words
    // xq[8*mt + g][32*kb + 4*t ..], xq[8*mt + g][32*kb + 16 + 4*t ..]; rows >= m read as zero.
    for (int idx = tid; idx < nblk * 32; idx += blockDim.x) {
        const int kb = idx >> 5, l = idx & 31, gg = l >> 2, tt = l & 3;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int row = 8 * mt + gg;
            uint2 v = make_uint2(0u, 0u);
            if (row < m) {
                const int8_t *src = xq + (size_t)row * k + 32 * kb + 4 * tt;
                v.x = *reinterpret_cast<const unsigned *>(src);
                v.y = *reinterpret_cast<const unsigned *>(src + 16);
            }
            sB[(size_t)idx * MT + mt] = v;
        }
    }
    __syncthreads();

    const int iters = (tpc + slots - 1) / slots;
    for (int it = 0; it < iters; ++it) {
        const int tl = it * slots + slot;
        const int tile = blockIdx.x * tpc + tl;
        const bool valid = (tl < tpc) && (tile < tiles);
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;

        if (valid) {
            const uint4 *wp = wq + ((size_t)tile * nsb) * 64 + lane;
            const float4 *sp = ws + ((size_t)tile * nsb) * 16 + g;
            constexpr int U = 4;
            for (int sb = sb0; sb < sb1; sb += U) {
                uint4 w0[U], w1[U];
                float4 s0[U], s1[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int s = min(sb + u, sb1 - 1);  // clamp: a repeated load, never out of range
                    w0[u] = ldg_stream(wp + (size_t)s * 64);
                    w1[u] = ldg_stream(wp + (size_t)s * 64 + 32);
                    s0[u] = __ldg(sp + (size_t)s * 16);
                    s1[u] = __ldg(sp + (size_t)s * 16 + 8);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (sb + u >= sb1) break;
                    const unsigned wa[4] = {w0[u].x, w0[u].y, w0[u].z, w0[u].w};
                    const unsigned wb[4] = {w1[u].x, w1[u].y, w1[u].z, w1[u].w};
                    const float sa[4] = {s0[u].x, s0[u].y, s0[u].z, s0[u].w};
                    const float sc[4] = {s1[u].x, s1[u].y, s1[u].z, s1[u].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const unsigned a0 = (wa[j] << 4) & 0xF0F0F0F0u, a2 = wa[j] & 0xF0F0F0F0u;
                        const unsigned a1 = (wb[j] << 4) & 0xF0F0F0F0u, a3 = wb[j] & 0xF0F0F0F0u;
                        const int kb = (sb + u) * 4 + j;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint2 b = sB[((size_t)kb * 32 + lane) * MT + mt];
                            int d[4];
                            mma_s8(d, a0, a1, a2, a3, b.x, b.y);
                            acc[mt][0] = fmaf((float)d[0], sa[j], acc[mt][0]);
                            acc[mt][1] = fmaf((float)d[1], sa[j], acc[mt][1]);
                            acc[mt][2] = fmaf((float)d[2], sc[j], acc[mt][2]);
                            acc[mt][3] = fmaf((float)d[3], sc[j], acc[mt][3]);
                            if (DUMP) {
                                // d[0],d[1]: weight row g, activation rows 8mt+2t, +1; d[2],d[3]: row g+8
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const size_t row_n = (size_t)tile * 16 + g + 8 * (i >> 1);
                                    const int row_m = 8 * mt + 2 * t + (i & 1);
                                    if (row_n < n && row_m < m)
                                        partials[((size_t)row_m * n + row_n) * nblk + kb] = d[i] >> 4;
                                }
                            }
                        }
                    }
                }
            }
        }

        // Fixed-order reduction over the ksplit warps of a slot.
        if (ksplit > 1) {
            if (ks > 0) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) red[((size_t)warp * MT * 4 + mt * 4 + i) * 32 + lane] = acc[mt][i];
            }
            __syncthreads();
            if (ks == 0) {
                for (int o = 1; o < ksplit; ++o)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            acc[mt][i] += red[((size_t)(warp + o) * MT * 4 + mt * 4 + i) * 32 + lane];
            }
            __syncthreads();
        }
        if (valid && ks == 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const size_t row_n = (size_t)tile * 16 + g + 8 * (i >> 1);
                    const int row_m = 8 * mt + 2 * t + (i & 1);
                    if (row_n < n && row_m < m)
                        y[(size_t)row_m * n + row_n] = x_scale[row_m] * (acc[mt][i] * 0.0625f);
                }
        }
    }
}

template <int MT, bool DUMP>
int launch(float *y, const int8_t *xq, const float *x_scale, const void *wq, const float *ws, int m,
           size_t n, int k, int32_t *partials, cudaStream_t st) {
    const int tiles = (int)((n + 15) / 16);
    const int nsb = k / 128;
    const int sms = sm_count();
    int tpc = (tiles + sms - 1) / sms;
    int slots = tpc < MAX_WARPS ? tpc : MAX_WARPS;
    int ksplit = MAX_WARPS / slots;
    if (ksplit > nsb / 4) ksplit = nsb / 4;
    if (ksplit < 1) ksplit = 1;
    const int warps = slots * ksplit;
    const int grid = (tiles + tpc - 1) / tpc;
    const size_t smem = (size_t)(k / 32) * 32 * MT * sizeof(uint2) + (size_t)warps * MT * 4 * 32 * sizeof(float);
    if (smem > 227 * 1024)
        return fail(XN_ERR_UNSUPPORTED, "linear_q4: k=%d needs %zu bytes of shared memory (max 232448)", k, smem);
    auto kern = linear_q4_kernel<MT, DUMP>;
    XN_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, warps * 32, smem, st>>>(y, xq, x_scale, (const uint4 *)wq, (const float4 *)ws, m, n, k,
                                         tiles, tpc, slots, ksplit, partials);
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

}  // namespace
}  // namespace xn

using namespace xn;

extern "C" int xn_mm_linear_q4(float *y, const int8_t *xq, const float *x_scale, const void *wq_packed,
                               const float *w_scale_tiled, size_t m, size_t n, size_t k,
                               int32_t *partials, void *stream) {
    XN_REQUIRE(k > 0 && k % 128 == 0, "linear_q4: k=%zu must be a positive multiple of 128", k);
    XN_REQUIRE(k <= 0x7fffffffull && n <= 0x7ffffff0ull, "linear_q4: dimension too large");
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y && xq && x_scale && wq_packed && w_scale_tiled, "linear_q4: null pointer");
    XN_REQUIRE(aligned(wq_packed, 16) && aligned(w_scale_tiled, 16),
               "linear_q4: packed weights and scales must be 16-byte aligned");
    XN_REQUIRE(aligned(xq, 4), "linear_q4: xq must be 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    for (size_t i0 = 0; i0 < m; i0 += 16) {
        const int mc = (int)((m - i0) < 16 ? (m - i0) : 16);
        int32_t *pp = partials ? partials + i0 * n * (k / 32) : nullptr;
        int rc;
        if (mc <= 8)
            rc = pp ? launch<1, true>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, w_scale_tiled, mc, n, (int)k, pp, st)
                    : launch<1, false>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, w_scale_tiled, mc, n, (int)k, pp, st);
        else
            rc = pp ? launch<2, true>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, w_scale_tiled, mc, n, (int)k, pp, st)
                    : launch<2, false>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, w_scale_tiled, mc, n, (int)k, pp, st);
        if (rc) return rc;
    }
    return XN_OK;
}
