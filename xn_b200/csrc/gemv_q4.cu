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
// 1.5 * 2^23, so the int32 result read as a float is exactly 12582912 + sum and one packed
// full-rate add (add.f32x2, two elements per instruction) replaces the slow int-to-float
// conversion before the block scale is applied.
//
// Data movement.  The kernel lasts a few microseconds and issues about as many instructions as the
// SM can retire in that time, so it is organised like a copy engine with a lean inner loop:
// one CTA per SM; a "unit" is one 1280-byte q4 tile (1 KB of nibbles + its 256 bytes of scales);
// every warp owns a run of consecutive units of one 16-row tile band and a private ring of slots
// in shared memory which lane 0 fills with bulk asynchronous copies (cp.async.bulk + mbarrier),
// re-arming a slot as soon as the warp is done with it.  The first copy of every warp is issued
// before anything else -- before the dependency wait of a programmatic dependent launch -- and the
// rest of the ring right after the activation copies, so about 150 KB per SM are in flight
// without holding a single register.  The int8 activations arrive by bulk copies too, row-major
// at a pitch of k + 16 bytes, and are read in B-fragment order with ldmatrix (the pitch spreads the
// 8 rows of a fragment over distinct banks): no staging code, no CTA-wide barrier before the math.
// The unit loop has no divisions and no per-unit address arithmetic beyond two adds.  Warps that
// share a tile (k split) combine their partial sums through shared memory in a fixed order:
// results are run-to-run identical.
//
// When k is so long that the activations leave no room for the rings, a second kernel with one small
// CTA per 16-row band takes over: it reads the activation fragments straight from global memory
// and has no limit on k.
#include "common.cuh"
#include "wait.cuh"

namespace xn {
namespace {

constexpr int MAX_WARPS = 20;
template <int BITS> struct Tile { static constexpr int W = BITS == 4 ? 1024 : 2048, UNIT = W + 256; };  // bytes
constexpr int MAGIC_I = 0x4B400000;
constexpr float MAGIC_F = 12582912.0f;
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t *b, unsigned parity, const WaitCtx &w) {
    return mbar_wait_bounded(smem_u32(b), parity, w);
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

__device__ __forceinline__ unsigned long long pack_f2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// (int bits read as float) - 1.5 * 2^23 for two accumulator elements in one packed instruction
__device__ __forceinline__ void unmagic2(int d0, int d1, float &f0, float &f1) {
    unsigned long long v, r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(d0), "r"(d1));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(v), "l"(pack_f2(-MAGIC_F, -MAGIC_F)));
    unpack_f2(r, f0, f1);
}

// One unit (16 weight rows x 128 k, at u in shared memory) against the activation words of its four
// 32-blocks: b[mt][2j] = {x[8mt+g][32j+4t..+3]}, b[mt][2j+1] = {x[8mt+g][32j+16+4t..+3]} of the unit's k range.
// acc[mt][e]: e = 0,1 -> weight row g, activation rows 8mt+2t, +1; e = 2,3 -> weight row g+8.
template <int MT, bool DUMP, int BITS>
__device__ __forceinline__ void unit_mma(const unsigned char *u, const unsigned (&b)[MT][8], float (&acc)[MT][4], int lane,
                                         int tile, int kb0, int m, size_t n, int nblk, int32_t *__restrict__ partials) {
    constexpr int W_BYTES = Tile<BITS>::W;
    const int g = lane >> 2, t = lane & 3;
    uint4 wv[4];  // int4: wv[0] = row g, wv[1] = row g+8 (four blocks each); int8: wv[j] = block j's {a0,a1,a2,a3}
    if (BITS == 4) {
        wv[0] = *reinterpret_cast<const uint4 *>(u + lane * 16);
        wv[1] = *reinterpret_cast<const uint4 *>(u + 512 + lane * 16);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const uint4 *>(u + j * 512 + lane * 16);
    }
    // {scale[g][j], scale[g+8][j]} for j = 0..3: 32 contiguous bytes
    const float4 s01 = *reinterpret_cast<const float4 *>(u + W_BYTES + g * 32);
    const float4 s23 = *reinterpret_cast<const float4 *>(u + W_BYTES + g * 32 + 16);
    const float sx[4] = {s01.x, s01.z, s23.x, s23.z}, sy[4] = {s01.y, s01.w, s23.y, s23.w};
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
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            int d[4];
            mma_s8(d, a0, a1, a2, a3, b[mt][2 * j], b[mt][2 * j + 1]);
            float f0, f1, f2, f3;
            unmagic2(d[0], d[1], f0, f1);
            unmagic2(d[2], d[3], f2, f3);
            acc[mt][0] = fmaf(f0, sx[j], acc[mt][0]);
            acc[mt][1] = fmaf(f1, sx[j], acc[mt][1]);
            acc[mt][2] = fmaf(f2, sy[j], acc[mt][2]);
            acc[mt][3] = fmaf(f3, sy[j], acc[mt][3]);
            if (DUMP) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const size_t row_n = (size_t)tile * 16 + g + 8 * (e >> 1);
                    const int row_m = 8 * mt + 2 * t + (e & 1);
                    if (row_n < n && row_m < m)
                        partials[((size_t)row_m * n + row_n) * nblk + kb0 + j] = (d[e] - MAGIC_I) >> (BITS == 4 ? 4 : 0);
                }
            }
        }
    }
}

template <int MT, bool DUMP, int BITS>
__global__ void __launch_bounds__(MAX_WARPS * 32, 1)
linear_q4_kernel(float *__restrict__ y, const int8_t *__restrict__ xq, const float *__restrict__ x_scale,
                 const unsigned char *__restrict__ wq, int m, size_t n, int k, int tiles, int tpc, int ksplit,
                 int usplit, int urem, int depth, int32_t *__restrict__ partials, const WaitCtx wctx) {
    constexpr int UNIT_BYTES = Tile<BITS>::UNIT;
    constexpr int UPC = 2;  // units per bulk copy and ring slot
    extern __shared__ __align__(128) unsigned char smem[];
    const int nblk = k / 32, nsb = k / 128;
    const int nwarps = blockDim.x >> 5;
    // [rings: nwarps * depth slots of UPC units, reused as red: nwarps * MT*4*32 f32]
    // [activations: 8*MT rows of k int8 at a pitch of k+16 bytes][mbarriers: nwarps * depth, then one per k slice for the activations]
    unsigned char *rings = smem;
    constexpr int slot_bytes = UPC * UNIT_BYTES;
    unsigned char *sX = smem + (size_t)nwarps * depth * slot_bytes;
    const int pitch = k + 16;  // rows 16 bytes apart modulo 128: the 8 rows of an ldmatrix tile hit distinct banks
    uint64_t *bars = reinterpret_cast<uint64_t *>(sX + (size_t)8 * MT * pitch);
    uint64_t *xbars = bars + (size_t)nwarps * depth;
    float *red = reinterpret_cast<float *>(rings);  // the rings are dead once every warp has left its unit loop

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // warp -> (tile of this CTA, k slice): slice ks covers usplit units, the first urem slices one more
    const int tl = (int)((unsigned)warp / (unsigned)ksplit), ks = warp - tl * ksplit;
    const int tile = blockIdx.x * tpc + tl;
    const bool valid = tile < tiles;
    const int sb0 = ks * usplit + min(ks, urem);
    const int nu = valid ? usplit + (ks < urem ? 1 : 0) : 0;

    unsigned char *ring = rings + (size_t)warp * depth * slot_bytes;
    uint64_t *bar = bars + (size_t)warp * depth;
    const unsigned char *wsrc = wq + ((size_t)tile * nsb + sb0) * UNIT_BYTES;
    const int nchunk = (nu + UPC - 1) / UPC;
    auto issue = [&](int c, int slot) {  // lane 0 only: fetch chunk c (UPC consecutive units) into its slot (c % depth)
        const unsigned bytes = (unsigned)min(UPC, nu - c * UPC) * UNIT_BYTES;
        mbar_expect_tx(&bar[slot], bytes);
        bulk_load(ring + (size_t)slot * slot_bytes, wsrc + (size_t)c * slot_bytes, bytes, &bar[slot]);
    };
    if (lane == 0) {
        for (int s = 0; s < depth; ++s) mbar_init(&bar[s], 1);
        if (tl == 0) mbar_init(&xbars[ks], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (nchunk > 0) issue(0, 0);
    }
    __syncthreads();  // the activation barrier is initialised before any warp can wait on it

    // Everything above read only the weights; the activations may come from the previous kernel.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // The activations come in row-major by bulk copies; rows >= m stay unwritten: their columns of the
    // product are computed from whatever the shared memory holds and never stored.  Up to 8 rows: one
    // copy per row and one barrier (few large copies are the cheapest).  16 rows are 64 KB at k = 4096,
    // wanted by every SM at once: one copy per row and k slice, tracked per slice, lets a slice's warps
    // start on their part while the rest is still arriving.
    constexpr bool SLICED = MT == 2;
    if (!SLICED && tid == 0) {
        mbar_expect_tx(&xbars[0], (unsigned)min(m, 8) * (unsigned)k);
        for (int r = 0; r < min(m, 8); ++r) bulk_load(sX + (size_t)r * pitch, xq + (size_t)r * k, (unsigned)k, &xbars[0]);
    }
    if (SLICED && tl == 0 && lane == 0) {
        const int rows = min(m, 16);
        const unsigned bytes = (unsigned)nu * 128u;
        mbar_expect_tx(&xbars[ks], (unsigned)rows * bytes);
        for (int r = 0; r < rows; ++r)
            bulk_load(sX + (size_t)r * pitch + (size_t)sb0 * 128, xq + (size_t)r * k + (size_t)sb0 * 128, bytes, &xbars[ks]);
    }
    float xs_reg[MT][2];  // x_scale of the activation rows this lane stores at the end
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int row_m = 8 * mt + 2 * t + e;
            xs_reg[mt][e] = row_m < m ? __ldg(x_scale + row_m) : 0.0f;
        }
    // The rest of the first ring-full.  With few activation rows it goes out at once.  From 6 rows on the
    // activation copies (24+ KB per SM, wanted before any MMA can start) would share the SM's copy
    // bandwidth with 100 KB of weights that are not needed yet: there the ring is filled only after the
    // activations have landed (measured: 8.6 -> 7.8 us at 16 rows, 7.5 -> 6.8 us at 8; slower below 6).
    // What is not in the ring yet is pulled into L2 right away either way, so that later copies into the
    // ring are L2 hits instead of a second round trip to HBM.
    const bool defer_ring = m >= 6;
    if (lane == 0) {
        const int c1 = defer_ring ? 1 : depth;
        if (!defer_ring)
            for (int c = 1; c < depth && c < nchunk; ++c) issue(c, c);
        if (nchunk > c1) {
            const unsigned rest = (unsigned)(nu - c1 * UPC) * UNIT_BYTES;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wsrc + (size_t)c1 * slot_bytes), "r"(rest)
                         : "memory");
        }
    }
    // ldmatrix row address of this lane: matrix lane/8 = {block lo, block hi, next block lo, next block hi}, row lane%8
    unsigned xaddr[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xaddr[mt] = smem_u32(sX) + (unsigned)(8 * mt + (lane & 7)) * (unsigned)pitch + 16u * (lane >> 3);

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    bool timed_out = nu > 0 && !mbar_wait(&xbars[SLICED ? ks : 0], 0, wctx);
    if (defer_ring && lane == 0)
        for (int c = 1; c < depth && c < nchunk; ++c) issue(c, c);

    // Chunks of UPC units walk the ring; slot and phase advance without divisions.
    int slot = 0;
    unsigned phase = 0;
    for (int c = 0; c < nchunk && !timed_out; ++c) {
        const int cu = min(UPC, nu - c * UPC);
        if (!mbar_wait(&bar[slot], phase, wctx)) {
            timed_out = true;
            break;
        }
        const unsigned char *base = ring + (size_t)slot * slot_bytes;
#pragma unroll
        for (int iu = 0; iu < UPC; ++iu) {
            if (iu >= cu) break;
            const int kb0 = (sb0 + c * UPC + iu) * 4;
            unsigned b[MT][8];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(b[mt][4 * h]), "=r"(b[mt][4 * h + 1]), "=r"(b[mt][4 * h + 2]), "=r"(b[mt][4 * h + 3])
                                 : "r"(xaddr[mt] + (unsigned)kb0 * 32u + 64u * h));
            unit_mma<MT, DUMP, BITS>(base + iu * UNIT_BYTES, b, acc, lane, tile, kb0, m, n, nblk, partials);
        }
        __syncwarp();  // every lane is done with the slot: it can be refilled
        if (lane == 0 && c + depth < nchunk) issue(c + depth, slot);
        if (++slot == depth) {
            slot = 0;
            phase ^= 1u;
        }
    }
    if (timed_out) {
        // A bulk copy never completed (not expected; the wait has reported it to the host).  Poison this
        // warp's result so the failure is visible in the output too, and fall through to the barriers
        // below: nothing spins for ever.
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

// ---------------------------------------------------------------------------------------------
// One small CTA per 16-row tile band ("tile kernel").  KS warps split the band's k range; each warp
// pulls its run of units into a private two-slot ring with bulk copies (for k = 4096 the whole run is
// in flight from the first instruction), reads the activation fragments straight from global memory
// (L1-resident: 8 or 16 rows of int8) and the KS partial sums meet in shared memory in a fixed order.
// No CTA-wide staging and 40-odd KB of shared memory per CTA: about five CTAs share an SM, they start
// and finish independently, and the CTAs of the next launch in the stream (programmatic dependent
// launch) move in as soon as individual CTAs of this one retire -- the hand-over between consecutive
// launches is staggered like that of a plain copy kernel instead of a full-SM barrier.
// ---------------------------------------------------------------------------------------------
constexpr int TK_WARPS = 4;    // k split inside a CTA

template <int MT, bool DUMP, int BITS>
__global__ void __launch_bounds__(TK_WARPS * 32, 5)
linear_q_tile_kernel(float *__restrict__ y, const int8_t *__restrict__ xq, const float *__restrict__ x_scale,
                     const unsigned char *__restrict__ wq, int m, size_t n, int k, int32_t *__restrict__ partials, const WaitCtx wctx) {
    constexpr int UNIT_BYTES = Tile<BITS>::UNIT;
    constexpr int SU = BITS == 4 ? 4 : 2;  // units per ring slot: 5 KB either way (static shared memory < 48 KB)
    constexpr int SLOT_BYTES = SU * UNIT_BYTES;
    constexpr int G = MT == 1 ? SU : SU / 2;  // units whose activation words are in registers at a time
    __shared__ __align__(128) unsigned char rings[TK_WARPS][2][SLOT_BYTES];
    __shared__ __align__(8) uint64_t bars[TK_WARPS][2];
    __shared__ float red[TK_WARPS][MT * 4][32];

    const int nblk = k / 32, nsb = k / 128;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x;
    const int sb0 = (int)((long long)nsb * warp / TK_WARPS), sb1 = (int)((long long)nsb * (warp + 1) / TK_WARPS);
    const int nu = sb1 - sb0;
    const int nchunk = (nu + SU - 1) / SU;
    const unsigned char *wsrc = wq + ((size_t)tile * nsb + sb0) * UNIT_BYTES;
    auto issue = [&](int c) {  // lane 0 only
        const int slot = c & 1;
        const unsigned bytes = (unsigned)min(SU, nu - c * SU) * UNIT_BYTES;
        mbar_expect_tx(&bars[warp][slot], bytes);
        bulk_load(&rings[warp][slot][0], wsrc + (size_t)c * SLOT_BYTES, bytes, &bars[warp][slot]);
    };
    if (lane == 0) {
        mbar_init(&bars[warp][0], 1);
        mbar_init(&bars[warp][1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (nchunk > 0) issue(0);
        if (nchunk > 1) issue(1);
    }
    __syncwarp();
    // Only weights were touched so far; the activations may be produced by the previous kernel.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Activation words of block kb for column group mt: {xq[8mt+g][32kb+4t..], xq[8mt+g][32kb+16+4t..]}.
    // Rows past m are clamped to row m-1: their columns of the product are computed and dropped.
    const int8_t *xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xrow[mt] = xq + (size_t)min(8 * mt + g, m - 1) * k + (size_t)sb0 * 128 + 4 * t;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    bool timed_out = false;

    auto unit_math = [&](const unsigned char *u, const unsigned (&b)[MT][8], int kb0) {
        unit_mma<MT, DUMP, BITS>(u, b, acc, lane, tile, kb0, m, n, nblk, partials);
    };
    auto fetch_unit = [&](unsigned (&b)[MT][8], int i) {  // unit i of this warp's run
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const unsigned *src = reinterpret_cast<const unsigned *>(xrow[mt] + (size_t)i * 128);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[mt][2 * j] = __ldg(src + 8 * j);
                b[mt][2 * j + 1] = __ldg(src + 8 * j + 4);
            }
        }
    };

    for (int c = 0; c < nchunk && !timed_out; ++c) {
        const int slot = c & 1;
        const int cu = min(SU, nu - c * SU);  // units in this chunk
        const unsigned char *base = &rings[warp][slot][0];
        if (cu == SU) {
            // full chunk: the activation loads of G units go out together, ahead of the wait for the weights
#pragma unroll
            for (int h = 0; h < SU / G; ++h) {
                unsigned b[G][MT][8];
#pragma unroll
                for (int ug = 0; ug < G; ++ug) fetch_unit(b[ug], c * SU + h * G + ug);
                if (h == 0 && !mbar_wait(&bars[warp][slot], (unsigned)(c >> 1) & 1u, wctx)) {
                    timed_out = true;
                    break;
                }
#pragma unroll
                for (int ug = 0; ug < G; ++ug)
                    unit_math(base + (h * G + ug) * UNIT_BYTES, b[ug], (sb0 + c * SU + h * G + ug) * 4);
            }
        } else {
            if (!mbar_wait(&bars[warp][slot], (unsigned)(c >> 1) & 1u, wctx)) {
                timed_out = true;
                break;
            }
            for (int iu = 0; iu < cu; ++iu) {
                unsigned b[MT][8];
                fetch_unit(b, c * SU + iu);
                unit_math(base + iu * UNIT_BYTES, b, (sb0 + c * SU + iu) * 4);
            }
        }
        __syncwarp();  // every lane is done with the slot: it can be refilled
        if (lane == 0 && c + 2 < nchunk) issue(c + 2);
    }
    if (timed_out) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][e] = __int_as_float(0x7fc00000);
    }
    if (warp > 0) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[warp][mt * 4 + e][lane] = acc[mt][e];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int o = 1; o < TK_WARPS; ++o)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[mt][e] += red[o][mt * 4 + e][lane];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const size_t row_n = (size_t)tile * 16 + g + 8 * (e >> 1);
                const int row_m = 8 * mt + 2 * t + (e & 1);
                if (row_n < n && row_m < m)
                    y[(size_t)row_m * n + row_n] = __ldg(x_scale + row_m) * (acc[mt][e] * (BITS == 4 ? 0.0625f : 1.0f));
            }
    }
}

template <int MT, bool DUMP, int BITS>
int launch_tile(float *y, const int8_t *xq, const float *x_scale, const void *wq, int m, size_t n, int k,
                int32_t *partials, cudaStream_t st) {
    const int tiles = (int)((n + 15) / 16);
    auto kern = linear_q_tile_kernel<MT, DUMP, BITS>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles);
    cfg.blockDim = dim3(TK_WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    WaitCtx wctx;
    if (int rcw = wait_ctx(&wctx)) return rcw;
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, y, xq, x_scale, (const unsigned char *)wq, m, n, k, partials, wctx));
    return XN_OK;
}

template <int MT, bool DUMP, int BITS>
int launch(float *y, const int8_t *xq, const float *x_scale, const void *wq, int m, size_t n, int k,
           int32_t *partials, cudaStream_t st) {
    constexpr int UNIT_BYTES = Tile<BITS>::UNIT;
    static const int tile_max_m = [] { const char *e = getenv("XN_Q4_TILE_MAX_M"); return e ? atoi(e) : 0; }();
    if (m <= tile_max_m) return launch_tile<MT, DUMP, BITS>(y, xq, x_scale, wq, m, n, k, partials, st);
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
    const size_t fixed = (size_t)8 * MT * (k + 16) + ((size_t)warps * 8 + MAX_WARPS) * sizeof(uint64_t);
    if (fixed + (size_t)warps * 2 * UNIT_BYTES > smem_cap)  // activations of a very long k leave no room for the rings
        return launch_tile<MT, DUMP, BITS>(y, xq, x_scale, wq, m, n, k, partials, st);
    const int per_warp = (nsb + ksplit - 1) / ksplit;
    constexpr int upc = 2;  // units per bulk copy and ring slot (the kernel's UPC)
    int depth = (int)((smem_cap - fixed) / ((size_t)warps * upc * UNIT_BYTES));
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
    WaitCtx wctx;
    if (int rcw = wait_ctx(&wctx)) return rcw;
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, y, xq, x_scale, (const unsigned char *)wq, m, n, k, tiles, tpc,
                                     ksplit, nsb / ksplit, nsb % ksplit, depth, partials, wctx));
    return XN_OK;
}

// q4 / q8 tiles -> row-major int8 weights [n_pad, k] and row-major block scales [n_pad, k / 32]: the operand
// images of the tensor-memory kernel that serves many activation rows.  One warp per 16-row x 128-k tile; the
// tile is rebuilt in shared memory (row pitch 144 bytes: the 4-byte scatter is free of bank conflicts) and leaves
// as whole 128-byte row segments.
template <int BITS>
__global__ void __launch_bounds__(256)
unpack_q_tiles_kernel(int8_t *__restrict__ w8, float *__restrict__ scales, const unsigned char *__restrict__ wq, size_t tiles,
                      int nsb, size_t k) {
    constexpr int UNIT = Tile<BITS>::UNIT, W = Tile<BITS>::W, PITCH = 144;
    __shared__ __align__(16) unsigned char stage[8][16 * PITCH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *sm = stage[warp];
    const int nblk = nsb * 4;
    for (size_t tile = (size_t)blockIdx.x * 8 + warp; tile < tiles; tile += (size_t)gridDim.x * 8) {
        const size_t band = tile / nsb;
        const int kt = (int)(tile - band * nsb);
        const unsigned char *u = wq + tile * UNIT;
        if (BITS == 4) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int g = lane >> 2, t = lane & 3;
                const uint4 c = *reinterpret_cast<const uint4 *>(u + (32 * h + lane) * 16);
                const unsigned w[4] = {c.x, c.y, c.z, c.w};
                unsigned char *row = sm + (8 * h + g) * PITCH;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned lo = w[j] & 0x0F0F0F0Fu, hi = (w[j] >> 4) & 0x0F0F0F0Fu;
                    *reinterpret_cast<unsigned *>(row + 32 * j + 4 * t) = __vsub4(lo ^ 0x08080808u, 0x08080808u);
                    *reinterpret_cast<unsigned *>(row + 32 * j + 16 + 4 * t) = __vsub4(hi ^ 0x08080808u, 0x08080808u);
                }
            }
        } else {
            const int g = lane >> 2, t = lane & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 c = *reinterpret_cast<const uint4 *>(u + j * 512 + lane * 16);
                *reinterpret_cast<unsigned *>(sm + g * PITCH + 32 * j + 4 * t) = c.x;
                *reinterpret_cast<unsigned *>(sm + (g + 8) * PITCH + 32 * j + 4 * t) = c.y;
                *reinterpret_cast<unsigned *>(sm + g * PITCH + 32 * j + 16 + 4 * t) = c.z;
                *reinterpret_cast<unsigned *>(sm + (g + 8) * PITCH + 32 * j + 16 + 4 * t) = c.w;
            }
        }
#pragma unroll
        for (int e0 = 0; e0 < 64; e0 += 32) {
            const int e = e0 + lane, h = e & 1, g = (e >> 1) >> 2, j = (e >> 1) & 3;
            scales[(band * 16 + 8 * h + g) * nblk + kt * 4 + j] = *reinterpret_cast<const float *>(u + W + e * 4);
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = it * 32 + lane, r = idx >> 3, piece = idx & 7;
            *reinterpret_cast<uint4 *>(w8 + (band * 16 + r) * k + (size_t)kt * 128 + piece * 16) =
                *reinterpret_cast<const uint4 *>(sm + r * PITCH + piece * 16);
        }
        __syncwarp();
    }
}

// Many activation rows: unpack once, then the kind::i8 tensor-memory kernel (exact block sums, the same f32
// arithmetic per block as the decode kernel).  The unpacked image lives in the stream's library scratch.
template <int BITS>
int linear_q_tensor(float *y, const int8_t *xq, const float *x_scale, const void *wq, size_t m, size_t n, size_t k, cudaStream_t st) {
    const size_t n_pad = (n + 15) / 16 * 16, nblk = k / 32;
    const size_t w_bytes = (n_pad * k + 255) / 256 * 256;
    void *ws = nullptr;
    if (int rc = library_scratch(st, w_bytes + n_pad * nblk * sizeof(float), &ws)) return rc;
    int8_t *w8 = static_cast<int8_t *>(ws);
    float *scales = reinterpret_cast<float *>(static_cast<unsigned char *>(ws) + w_bytes);
    const size_t tiles = (n_pad / 16) * (k / 128);
    const size_t blocks = (tiles + 7) / 8;
    const unsigned grid = (unsigned)(blocks < (size_t)sm_count() * 16 ? blocks : (size_t)sm_count() * 16);
    unpack_q_tiles_kernel<BITS><<<grid, 256, 0, st>>>(w8, scales, (const unsigned char *)wq, tiles, (int)(k / 128), k);
    XN_CHECK_CUDA(cudaGetLastError());
    return launch_gemm_q8_block(y, n, xq, x_scale, w8, scales, m, n, n_pad, k, st);
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
    // from this many rows on (and when the caller does not ask for the block sums), the weights are unpacked once
    // and the tensor-memory kernel takes all rows in one launch instead of one weight pass per 16 rows (measured
    // break-even on [4096, 4096] and [11264, 4096]: 128 to 160 rows)
    static const size_t tensor_min_m = [] { const char *e = getenv("XN_Q_TENSOR_MIN_M"); return e ? (size_t)atoi(e) : (size_t)160; }();
    if (!partials && m >= tensor_min_m && m <= 0x7fffffffull) return linear_q_tensor<BITS>(y, xq, x_scale, wq_packed, m, n, k, st);
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
    XN_API_RANGE("xn_mm_linear_q4");
    return linear_q<4>("linear_q4", y, xq, x_scale, wq_packed, m, n, k, partials, stream);
}

extern "C" int xn_mm_linear_q8(float *y, const int8_t *xq, const float *x_scale, const void *wq_packed, size_t m,
                               size_t n, size_t k, int32_t *partials, void *stream) {
    XN_API_RANGE("xn_mm_linear_q8");
    return linear_q<8>("linear_q8", y, xq, x_scale, wq_packed, m, n, k, partials, stream);
}

// Host-buffer form: the decode call of a host that keeps its activations and results in (pinned) host memory.
// One C call enqueues the host->device copy, the row quantizer, the linear and the device->host copy on
// `stream`; the staging buffers live in a caller-owned device workspace.
extern "C" size_t xn_mm_linear_q4_host_workspace_bytes(size_t m, size_t n, size_t k) {
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    return up(m * k * 4) + up(m * k) + up(m * 4) + up(m * n * 4);
}

extern "C" int xn_mm_linear_q4_host(float *y_host, const float *x_host, const void *wq_packed, size_t m, size_t n, size_t k,
                                    void *workspace, size_t workspace_bytes, void *stream) {
    XN_API_RANGE("xn_mm_linear_q4_host");
    XN_REQUIRE(k > 0 && k % 128 == 0, "linear_q4_host: k=%zu must be a positive multiple of 128", k);
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y_host && x_host && wq_packed && workspace, "linear_q4_host: null pointer");
    XN_REQUIRE(aligned(workspace, 256), "linear_q4_host: workspace must be 256-byte aligned");
    if (workspace_bytes < xn_mm_linear_q4_host_workspace_bytes(m, n, k))
        return fail(XN_ERR_WORKSPACE, "linear_q4_host: workspace of %zu bytes, %zu needed", workspace_bytes,
                    xn_mm_linear_q4_host_workspace_bytes(m, n, k));
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    unsigned char *p = static_cast<unsigned char *>(workspace);
    float *x_dev = reinterpret_cast<float *>(p);
    int8_t *xq = reinterpret_cast<int8_t *>(p + up(m * k * 4));
    float *xs = reinterpret_cast<float *>(p + up(m * k * 4) + up(m * k));
    float *y_dev = reinterpret_cast<float *>(p + up(m * k * 4) + up(m * k) + up(m * 4));
    cudaStream_t st = (cudaStream_t)stream;
    XN_CHECK_CUDA(cudaMemcpyAsync(x_dev, x_host, m * k * 4, cudaMemcpyHostToDevice, st));
    if (int rc = xn_mm_quantize_rows_i8(xq, xs, x_dev, XN_F32, m, k, stream)) return rc;
    if (int rc = linear_q<4>("linear_q4_host", y_dev, xq, xs, wq_packed, m, n, k, nullptr, stream)) return rc;
    XN_CHECK_CUDA(cudaMemcpyAsync(y_host, y_dev, m * n * 4, cudaMemcpyDeviceToHost, st));
    return XN_OK;
}
