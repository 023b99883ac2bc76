// int4 block-quantized decode linear (M <= 16 per pass): the memory-bound weight-streaming path.
// No counterpart in the reference (it has no quantized matmul); the contract is in
// include/xn_mm.h.  Exact integer arithmetic: every 32-element block product is an int32.
//
// Arithmetic.  The packed weights are stored as 1 KB tiles of 16 output rows x 128 k laid out in
// the A-fragment order of an integer tensor-core MMA (m16n8k32, s8 x s8 -> s32): the output rows
// ride the MMA's 16-row dimension, the (at most 16) activation rows its 8-column dimension, so
// an M = 1..8 pass needs one MMA per 16 rows x 32 k and M = 9..16 two.  A 32-bit word of eight
// nibbles becomes two int8x4 operands with two logic ops: (w << 4) & 0xF0F0F0F0 and
// w & 0xF0F0F0F0 are the low / high nibbles times 16 as signed bytes; the factor 16 is removed
// exactly at the end (power of two).  The MMA's accumulator input is the bit pattern of
// 1.5 * 2^23, so the int32 result read as a float is exactly 12582912 + sum and one full-rate
// FADD replaces the slow int-to-float conversion before the block scale is applied.
//
// Data movement.  The kernel lasts a few microseconds, so it is organised like a copy engine:
// one CTA per SM; a "unit" is one 1280-byte q4 tile (1 KB of nibbles + its 256 bytes of scales);
// every warp owns a run of consecutive units of one 16-row tile band and a private ring of slots
// in shared memory which lane 0 fills with bulk asynchronous copies (cp.async.bulk + mbarrier), re-arming a slot as soon as the
// warp has read it.  The first ring-full of copies is issued before anything else -- before the
// dependency wait of a programmatic dependent launch and before the activations are staged -- so
// about 150 KB per SM are in flight without holding a single register.  The int8 activations are
// staged once per CTA in shared memory in B-fragment order.  Warps that share a tile (k split)
// combine their partial sums through shared memory in a fixed order: results are run-to-run
// identical.
#include "common.cuh"

namespace xn {
namespace {

constexpr int MAX_WARPS = 20;
template <int BITS> struct Tile { static constexpr int W = BITS == 4 ? 1024 : 2048, UNIT = W + 256; };  // bytes
constexpr int MAGIC_I = 0x4B400000;
constexpr float MAGIC_F = 12582912.0f;
constexpr unsigned WAIT_LIMIT = 1u << 24;  // polls of one mbarrier before the warp gives up

__device__ unsigned g_q4_wait_timeouts;  // counts abandoned waits (never expected to move)

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *b, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *b, unsigned parity) {
    for (unsigned i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(b, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mma_s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(MAGIC_I));
}

template <int MT, bool DUMP, int BITS>
__global__ void __launch_bounds__(MAX_WARPS * 32, 1)
linear_q4_kernel(float *__restrict__ y, const int8_t *__restrict__ xq, const float *__restrict__ x_scale,
                 const unsigned char *__restrict__ wq, int m, size_t n, int k, int tiles, int tpc, int ksplit,
                 int depth, int upc, int32_t *__restrict__ partials) {
    constexpr int UNIT_BYTES = Tile<BITS>::UNIT, W_BYTES = Tile<BITS>::W;
    extern __shared__ __align__(128) unsigned char smem[];
    const int nblk = k / 32, nsb = k / 128;
    const int nwarps = blockDim.x >> 5;
    // [rings: nwarps * depth slots of upc units, reused as red: nwarps * MT*4*32 f32][B fragments: nblk * 32 * MT uint2][mbarriers]
    unsigned char *rings = smem;
    const int slot_bytes = upc * UNIT_BYTES;
    uint2 *sB = reinterpret_cast<uint2 *>(smem + (size_t)nwarps * depth * slot_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(sB) + (size_t)nblk * 32 * MT * sizeof(uint2));
    float *red = reinterpret_cast<float *>(rings);  // the rings are dead once every warp has left its unit loop

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tl = warp / ksplit, ks = warp % ksplit;
    const int tile = blockIdx.x * tpc + tl;
    const bool valid = tile < tiles;
    const int sb0 = (int)((long long)nsb * ks / ksplit), sb1 = (int)((long long)nsb * (ks + 1) / ksplit);
    const int nu = valid ? sb1 - sb0 : 0;

    unsigned char *ring = rings + (size_t)warp * depth * slot_bytes;
    uint64_t *bar = bars + (size_t)warp * depth;
    const unsigned char *wsrc = wq + ((size_t)tile * nsb + sb0) * UNIT_BYTES;
    const int nchunk = (nu + upc - 1) / upc;
    auto issue = [&](int c) {  // lane 0 only: fetch chunk c (upc consecutive units) into slot c % depth
        const int slot = c % depth;
        const unsigned bytes = (unsigned)min(upc, nu - c * upc) * UNIT_BYTES;
        mbar_expect_tx(&bar[slot], bytes);
        bulk_load(ring + (size_t)slot * slot_bytes, wsrc + (size_t)c * slot_bytes, bytes, &bar[slot]);
    };
    if (lane == 0) {
        for (int s = 0; s < depth; ++s) mbar_init(&bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (nchunk > 0) issue(0);
    }
    __syncwarp();

    // Everything above read only the weights; the activations may come from the previous kernel.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Activation loads go out next, ahead of the bulk of the weight traffic, so that they are not
    // queued behind ~150 KB of copies per SM; rows >= m read as zero.
    // One work item = one (row group g, 32-block): 2*MT 128-bit loads (rows g and, for MT = 2,
    // g + 8), then 32*MT contiguous bytes of fragments: entry (kb, lane = 4*g + t, mt) =
    // {xq[8mt+g][32kb+4t..], xq[8mt+g][32kb+16+4t..]}.
    constexpr int STAGE_ITEMS = 2;  // items per thread and pass
    const int items = nblk * 8;
    float xs_reg[MT][2];            // x_scale of the activation rows this lane stores at the end
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int row_m = 8 * mt + 2 * t + e;
            xs_reg[mt][e] = row_m < m ? __ldg(x_scale + row_m) : 0.0f;
        }
    for (int base = 0; base < items; base += STAGE_ITEMS * (int)blockDim.x) {
        uint4 lo[STAGE_ITEMS][MT], hi[STAGE_ITEMS][MT];
#pragma unroll
        for (int q = 0; q < STAGE_ITEMS; ++q) {
            const int idx = base + q * (int)blockDim.x + tid;
            const int gg = idx & 7, kb = idx >> 3;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                lo[q][mt] = make_uint4(0u, 0u, 0u, 0u);
                hi[q][mt] = lo[q][mt];
                const int row = 8 * mt + gg;
                if (idx < items && row < m) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(xq + (size_t)row * k + 32 * kb);
                    lo[q][mt] = __ldg(src);
                    hi[q][mt] = __ldg(src + 1);
                }
            }
        }
        if (base == 0 && lane == 0) {
            for (int c = 1; c < depth && c < nchunk; ++c) issue(c);  // the rest of the first ring-full
            // What does not fit in the ring yet is pulled into L2 now, so that the refills of the
            // ring are L2 hits instead of a second round trip to HBM.
            if (nchunk > depth) {
                const unsigned rest = (unsigned)(nu - depth * upc) * UNIT_BYTES;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wsrc + (size_t)depth * slot_bytes), "r"(rest)
                             : "memory");
            }
        }
#pragma unroll
        for (int q = 0; q < STAGE_ITEMS; ++q) {
            const int idx = base + q * (int)blockDim.x + tid;
            if (idx >= items) continue;
            const int gg = idx & 7, kb = idx >> 3;
            uint2 *dst = sB + ((size_t)kb * 32 + 4 * gg) * MT;
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
                const int t2 = (tt + gg) & 3;  // rotate the order per lane: fewer bank conflicts
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const unsigned a = t2 == 0 ? lo[q][mt].x : t2 == 1 ? lo[q][mt].y : t2 == 2 ? lo[q][mt].z : lo[q][mt].w;
                    const unsigned bq = t2 == 0 ? hi[q][mt].x : t2 == 1 ? hi[q][mt].y : t2 == 2 ? hi[q][mt].z : hi[q][mt].w;
                    dst[t2 * MT + mt] = make_uint2(a, bq);
                }
            }
        }
    }
    __syncthreads();

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    bool timed_out = false;

    for (int i = 0; i < nu; ++i) {
        const int c = i / upc, slot = c % depth;
        if (i % upc == 0 && !mbar_wait(&bar[slot], (unsigned)(c / depth) & 1u)) {
            timed_out = true;
            break;
        }
        const unsigned char *u = ring + (size_t)slot * slot_bytes + (size_t)(i % upc) * UNIT_BYTES;
        uint4 wv[4];  // int4: wv[0] = row g, wv[1] = row g+8 (four 32-blocks each); int8: wv[j] = block j's {a0,a1,a2,a3}
        if (BITS == 4) {
            wv[0] = *reinterpret_cast<const uint4 *>(u + lane * 16);
            wv[1] = *reinterpret_cast<const uint4 *>(u + 512 + lane * 16);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const uint4 *>(u + j * 512 + lane * 16);
        }
        float2 sc[4];  // {scale[g][j], scale[g+8][j]}
#pragma unroll
        for (int j = 0; j < 4; ++j) sc[j] = *reinterpret_cast<const float2 *>(u + W_BYTES + (4 * g + j) * 8);
        if (i % upc == upc - 1 || i == nu - 1) {
            __syncwarp();  // every lane holds its part of the slot: it can be refilled
            if (lane == 0 && c + depth < nchunk) issue(c + depth);
        }

        const unsigned wa[4] = {wv[0].x, wv[0].y, wv[0].z, wv[0].w};
        const unsigned wb[4] = {wv[1].x, wv[1].y, wv[1].z, wv[1].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unsigned a0, a1, a2, a3;
            if (BITS == 4) {
                a0 = (wa[j] << 4) & 0xF0F0F0F0u; a2 = wa[j] & 0xF0F0F0F0u;
                a1 = (wb[j] << 4) & 0xF0F0F0F0u; a3 = wb[j] & 0xF0F0F0F0u;
            } else {
                a0 = wv[j].x; a1 = wv[j].y; a2 = wv[j].z; a3 = wv[j].w;
            }
            const int kb = (sb0 + i) * 4 + j;
            // both column groups' fragments sit side by side: one 128-bit shared-memory read for MT = 2
            uint2 bfrag[MT];
            if (MT == 2) {
                const uint4 t4 = *reinterpret_cast<const uint4 *>(sB + ((size_t)kb * 32 + lane) * 2);
                bfrag[0] = make_uint2(t4.x, t4.y);
                bfrag[MT - 1] = make_uint2(t4.z, t4.w);
            } else {
                bfrag[0] = sB[(size_t)kb * 32 + lane];
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint2 bb = bfrag[mt];
                int d[4];
                mma_s8(d, a0, a1, a2, a3, bb.x, bb.y);
                acc[mt][0] = fmaf(__int_as_float(d[0]) - MAGIC_F, sc[j].x, acc[mt][0]);
                acc[mt][1] = fmaf(__int_as_float(d[1]) - MAGIC_F, sc[j].x, acc[mt][1]);
                acc[mt][2] = fmaf(__int_as_float(d[2]) - MAGIC_F, sc[j].y, acc[mt][2]);
                acc[mt][3] = fmaf(__int_as_float(d[3]) - MAGIC_F, sc[j].y, acc[mt][3]);
                if (DUMP) {
                    // d[0],d[1]: weight row g, activation rows 8mt+2t, +1; d[2],d[3]: weight row g+8
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const size_t row_n = (size_t)tile * 16 + g + 8 * (e >> 1);
                        const int row_m = 8 * mt + 2 * t + (e & 1);
                        if (row_n < n && row_m < m)
                            partials[((size_t)row_m * n + row_n) * nblk + kb] = (d[e] - MAGIC_I) >> (BITS == 4 ? 4 : 0);
                    }
                }
            }
        }
    }
    if (timed_out) {
        // A bulk copy never completed (not expected).  Record it, poison this warp's result so the
        // failure is visible, and fall through to the barriers below: nothing spins for ever.
        if (lane == 0) atomicAdd(&g_q4_wait_timeouts, 1u);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][e] = __int_as_float(0x7fc00000);
    }

    // Fixed-order reduction over the ksplit warps of a tile.
    if (ksplit > 1) {
        __syncthreads();  // all unit loops are over: the ring area becomes the reduction buffer
        if (ks > 0) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[((size_t)warp * MT * 4 + mt * 4 + e) * 32 + lane] = acc[mt][e];
        }
        __syncthreads();
        if (ks == 0) {
            for (int o = 1; o < ksplit; ++o)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        acc[mt][e] += red[((size_t)(warp + o) * MT * 4 + mt * 4 + e) * 32 + lane];
        }
    }
    if (valid && ks == 0) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const size_t row_n = (size_t)tile * 16 + g + 8 * (e >> 1);
                const int row_m = 8 * mt + 2 * t + (e & 1);
                if (row_n < n && row_m < m) y[(size_t)row_m * n + row_n] = xs_reg[mt][e & 1] * (acc[mt][e] * (BITS == 4 ? 0.0625f : 1.0f));
            }
    }
}

template <int MT, bool DUMP, int BITS>
int launch(float *y, const int8_t *xq, const float *x_scale, const void *wq, int m, size_t n, int k,
           int32_t *partials, cudaStream_t st) {
    constexpr int UNIT_BYTES = Tile<BITS>::UNIT;
    const int tiles = (int)((n + 15) / 16);
    const int nsb = k / 128;
    const int sms = sm_count();
    int tpc = (tiles + sms - 1) / sms;
    static const int maxw = [] { const char *e = getenv("XN_Q4_MAXW"); int v = e ? atoi(e) : MAX_WARPS; return v < 1 ? 1 : (v > MAX_WARPS ? MAX_WARPS : v); }();
    static const size_t smem_cap = [] { const char *e = getenv("XN_Q4_SMEM_KB"); return (size_t)(e ? atoi(e) : 227) * 1024; }();
    if (tpc > maxw) tpc = maxw;  // very tall weights: more CTAs than SMs
    int ksplit = maxw / tpc;
    if (ksplit > nsb) ksplit = nsb;
    const int warps = tpc * ksplit;
    const int grid = (tiles + tpc - 1) / tpc;
    const size_t fixed = (size_t)(k / 32) * 32 * MT * sizeof(uint2) + (size_t)warps * 8 * sizeof(uint64_t);
    if (fixed + (size_t)warps * UNIT_BYTES > 227 * 1024)  // hard limit of the part
        return fail(XN_ERR_UNSUPPORTED, "linear_q4: k=%d needs more than 232448 bytes of shared memory", k);
    const int per_warp = (nsb + ksplit - 1) / ksplit;
    static const int upc_env = [] { const char *e = getenv("XN_Q4_UPC"); return e ? atoi(e) : 0; }();
    int upc = upc_env > 0 ? upc_env : 2;  // units per bulk copy
    if (upc > per_warp) upc = per_warp;
    const size_t cap = smem_cap > fixed + (size_t)warps * UNIT_BYTES ? smem_cap : fixed + (size_t)warps * UNIT_BYTES;
    while (upc > 1 && fixed + (size_t)warps * 2 * upc * UNIT_BYTES > cap) --upc;
    int depth = (int)((cap - fixed) / ((size_t)warps * upc * UNIT_BYTES));
    if (depth < 1) depth = 1;
    if (depth > (per_warp + upc - 1) / upc) depth = (per_warp + upc - 1) / upc;
    if (depth > 8) depth = 8;
    const size_t smem = fixed + (size_t)warps * depth * upc * UNIT_BYTES;
    auto kern = linear_q4_kernel<MT, DUMP, BITS>;
    XN_ENSURE_SMEM(kern, smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, y, xq, x_scale, (const unsigned char *)wq, m, n, k, tiles, tpc,
                                     ksplit, depth, upc, partials));
    return XN_OK;
}

}  // namespace
}  // namespace xn

using namespace xn;

template <int BITS>
static int linear_q(const char *name, float *y, const int8_t *xq, const float *x_scale, const void *wq_packed, size_t m,
                    size_t n, size_t k, int32_t *partials, void *stream) {
    XN_REQUIRE(k > 0 && k % 128 == 0, "%s: k=%zu must be a positive multiple of 128", name, k);
    XN_REQUIRE(k <= 0x7fffffffull && n <= 0x7ffffff0ull, "%s: dimension too large", name);
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y && xq && x_scale && wq_packed, "%s: null pointer", name);
    XN_REQUIRE(aligned(wq_packed, 16), "%s: packed weights must be 16-byte aligned", name);
    XN_REQUIRE(aligned(xq, 16), "%s: xq must be 16-byte aligned", name);
    cudaStream_t st = (cudaStream_t)stream;
    for (size_t i0 = 0; i0 < m; i0 += 16) {
        const int mc = (int)((m - i0) < 16 ? (m - i0) : 16);
        int32_t *pp = partials ? partials + i0 * n * (k / 32) : nullptr;
        int rc;
        if (mc <= 8)
            rc = pp ? launch<1, true, BITS>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, mc, n, (int)k, pp, st)
                    : launch<1, false, BITS>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, mc, n, (int)k, pp, st);
        else
            rc = pp ? launch<2, true, BITS>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, mc, n, (int)k, pp, st)
                    : launch<2, false, BITS>(y + i0 * n, xq + i0 * k, x_scale + i0, wq_packed, mc, n, (int)k, pp, st);
        if (rc) return rc;
    }
    return XN_OK;
}

extern "C" int xn_mm_linear_q4(float *y, const int8_t *xq, const float *x_scale, const void *wq_packed, size_t m,
                               size_t n, size_t k, int32_t *partials, void *stream) {
    return linear_q<4>("linear_q4", y, xq, x_scale, wq_packed, m, n, k, partials, stream);
}

extern "C" int xn_mm_linear_q8(float *y, const int8_t *xq, const float *x_scale, const void *wq_packed, size_t m,
                               size_t n, size_t k, int32_t *partials, void *stream) {
    return linear_q<8>("linear_q8", y, xq, x_scale, wq_packed, m, n, k, partials, stream);
}
