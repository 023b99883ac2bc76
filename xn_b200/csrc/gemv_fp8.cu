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
// Schedule.  `tpc` consecutive 16-row tiles per CTA (about one CTA per SM), `ksplit` warps per tile
// reduced in a fixed order.  Every warp keeps DEPTH 64-byte k steps (two 128-bit loads each) in
// flight in registers, refilling a step's registers right after consuming them; the first DEPTH
// steps are requested before the dependency wait of a programmatic dependent launch and before the
// activation pieces are staged (cp.async), so the weight stream never waits for the prologue.
// When the activation pieces do not fit in shared memory at once, k is walked in chunks.
#include "common.cuh"

namespace xn {
namespace {

constexpr int MAX_WARPS = 24;
constexpr int DEPTH = 4;
constexpr int SMEM_BUDGET = 200 * 1024;

__device__ __forceinline__ void mma_e4m3(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
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
__global__ void __launch_bounds__(MAX_WARPS * 32, 1)
linear_fp8_gemv_kernel(__nv_bfloat16 *__restrict__ y, const uint8_t *__restrict__ x_hi,
                       const uint8_t *__restrict__ x_lo, const float *__restrict__ x_scale,
                       const uint8_t *__restrict__ wq, const float *__restrict__ w_scale, int m, size_t n,
                       int k, int kchunk, int tiles, int tpc, int ksplit) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = x_row_stride(kchunk);
    unsigned char *sHi = smem;
    unsigned char *sLo = smem + (size_t)MT * 8 * RS;
    float *red = reinterpret_cast<float *>(smem + (size_t)(LO ? 2 : 1) * MT * 8 * RS);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tl = warp / ksplit, ks = warp % ksplit;
    const int tile = blockIdx.x * tpc + tl;
    const bool valid = tile < tiles;
    const size_t r0 = valid ? min((size_t)tile * 16 + g, n - 1) : 0, r1 = valid ? min((size_t)tile * 16 + g + 8, n - 1) : 0;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    // scales of the rows this lane stores at the end, requested early
    float xs_reg[MT][2], ws_reg[2];

    for (int kc0 = 0; kc0 < k; kc0 += kchunk) {
        const int kc = min(kchunk, k - kc0);
        const int nst = (kc + 63) / 64;  // 64-byte k steps in this chunk
        const int st0 = (int)((long long)nst * ks / ksplit), st1 = valid ? (int)((long long)nst * (ks + 1) / ksplit) : st0;
        const uint8_t *wp0 = wq + r0 * k + kc0 + 16 * t;
        const uint8_t *wp1 = wq + r1 * k + kc0 + 16 * t;
        uint4 w0[DEPTH], w1[DEPTH];
        auto load = [&](int i, int st) {  // step st -> register slot i
            if (st < st1 && st * 64 + 16 * t < kc) {
                w0[i] = ldg_stream(wp0 + (size_t)st * 64);
                w1[i] = ldg_stream(wp1 + (size_t)st * 64);
            } else {
                w0[i] = make_uint4(0, 0, 0, 0);
                w1[i] = make_uint4(0, 0, 0, 0);
            }
        };
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) load(i, st0 + i);

        if (kc0 == 0) {
            // Everything so far read only the weights; the activations may come from the previous kernel.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int row_m = 8 * mt + 2 * t + e;
                    xs_reg[mt][e] = row_m < m ? __ldg(x_scale + row_m) : 0.0f;
                }
            ws_reg[0] = valid ? __ldg(w_scale + r0) : 0.0f;
            ws_reg[1] = valid ? __ldg(w_scale + r1) : 0.0f;
        } else {
            __syncthreads();  // every warp is done with the previous chunk's pieces
        }
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

        for (int st = st0; st < st1; st += DEPTH) {
#pragma unroll
            for (int i = 0; i < DEPTH; ++i) {
                if (st + i < st1) {
                    const int off = (st + i) * 64 + 16 * t;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint4 bh = *reinterpret_cast<const uint4 *>(sHi + (size_t)(8 * mt + g) * RS + off);
                        mma_e4m3(acc[mt], w0[i].x, w1[i].x, w0[i].y, w1[i].y, bh.x, bh.y);
                        mma_e4m3(acc[mt], w0[i].z, w1[i].z, w0[i].w, w1[i].w, bh.z, bh.w);
                        if (LO) {
                            const uint4 bl = *reinterpret_cast<const uint4 *>(sLo + (size_t)(8 * mt + g) * RS + off);
                            mma_e4m3(acc[mt], w0[i].x, w1[i].x, w0[i].y, w1[i].y, bl.x, bl.y);
                            mma_e4m3(acc[mt], w0[i].z, w1[i].z, w0[i].w, w1[i].w, bl.z, bl.w);
                        }
                    }
                }
                load(i, st + i + DEPTH);
            }
        }
    }

    // fixed-order reduction over the ksplit warps of a tile, then the scaled bf16 store
    if (ksplit > 1) {
        __syncthreads();
        if (ks > 0)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) red[((size_t)warp * MT * 4 + mt * 4 + i) * 32 + lane] = acc[mt][i];
        __syncthreads();
        if (ks == 0)
            for (int o = 1; o < ksplit; ++o)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][i] += red[((size_t)(warp + o) * MT * 4 + mt * 4 + i) * 32 + lane];
    }
    if (ks == 0 && valid) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const size_t row_n = (size_t)tile * 16 + g + 8 * (i >> 1);
                const int row_m = 8 * mt + 2 * t + (i & 1);
                if (row_n < n && row_m < m)
                    y[(size_t)row_m * n + row_n] = __float2bfloat16_rn(ws_reg[i >> 1] * (xs_reg[mt][i & 1] * acc[mt][i]));
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
    int ksplit = MAX_WARPS / tpc;
    // largest k chunk (multiple of 128) whose staged pieces fit the shared-memory budget
    const int pieces = LO ? 2 : 1;
    int kchunk = (k + 127) / 128 * 128;
    while ((size_t)pieces * MT * 8 * x_row_stride(kchunk) > (size_t)SMEM_BUDGET - MAX_WARPS * MT * 4 * 32 * 4)
        kchunk = ((kchunk / 128 + 1) / 2) * 128;
    const int nst = ((kchunk < k ? kchunk : k) + 63) / 64;
    if (ksplit > nst / DEPTH) ksplit = nst / DEPTH;
    if (ksplit < 1) ksplit = 1;
    const int warps = tpc * ksplit;
    const int grid = (tiles + tpc - 1) / tpc;
    const size_t smem = (size_t)pieces * MT * 8 * x_row_stride(kchunk) + (size_t)warps * MT * 4 * 32 * sizeof(float);
    auto kern = linear_fp8_gemv_kernel<MT, LO>;
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
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, y, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, kchunk, tiles, tpc, ksplit));
    return XN_OK;
}

}  // namespace

// y [m,n] bf16 from row-major e4m3 pieces; m <= 32.
int launch_linear_fp8_gemv(void *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale,
                           const uint8_t *wq, const float *w_scale, int m, size_t n, int k, cudaStream_t st) {
    __nv_bfloat16 *yy = (__nv_bfloat16 *)y;
    if (m <= 8)
        return x_lo ? launch<1, true>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st)
                    : launch<1, false>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
    if (m <= 16)
        return x_lo ? launch<2, true>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st)
                    : launch<2, false>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
    return x_lo ? launch<4, true>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st)
                : launch<4, false>(yy, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
}

}  // namespace xn
