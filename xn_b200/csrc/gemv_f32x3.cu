// f32 decode-sized matmul_t (lhs [m,k], rhs [n,k] both k-contiguous, m <= 16) on the tensor cores:
// the "3xTF32" split.  This is the benchmark's CPU-runnable configuration (x [16,4096], W [11264,4096]
// f32) and the decode-time Linear::forward of an f32 model.  Reference path:
// cublasGemmStridedBatchedEx with CUBLAS_COMPUTE_32F (xn-core/src/cuda_backend.rs:2109-2133).
//
// Arithmetic.  Every f32 operand is cut into hi + lo on the tf32 grid (10 mantissa bits): hi = the nearest
// tf32 number, lo = the exact remainder x - hi (12 significant bits) rounded to tf32 as well, so hi + lo
// carries x to 2^-23.  x * w = xh*wh + xh*wl + xl*wh + xl*wl; the first three are tf32 MMAs
// (mma.sync.m16n8k8, a native tensor instruction on sm_100a), the last (<= 2^-22 |x w|) is dropped.
// A plain FFMA kernel is bound by the FP32 pipe here (16 x 11264 x 4096 FMAs are 20 us of a fully busy
// B200; it measured 82 us).
// Accumulation.  The parity bound for f32 is 1e-4 relative with a floor of 1e-2 of the output's rms in the
// denominator, i.e. an absolute error below 1e-6 of the rms at the maximum over 180 000 outputs -- tighter
// than a sequential f32 sum over k = 4096 delivers, and the tensor core adds into its accumulator with
// truncation, which is worse.  So nothing of full size is accumulated inside the MMA: every hi x hi MMA
// starts from a zero accumulator (one rounding of an 8-term sum), the small cross terms of a 32-k step share
// one accumulator, the five values are added with ordinary roundings, and the step's sum goes into the
// running total with a compensated (Kahan) add.
//
// Data movement: like the fp8 GEMV.  Output rows ride the MMA's 16-row dimension, the activation rows
// its 8 columns (two column groups for m = 9..16); a lane's two 128-bit loads of a row (8 consecutive
// k) feed four MMAs through a fixed k permutation that the activation fragment follows; DEPTH steps
// of 32 k per warp are in flight in registers; the activations are staged in shared memory per k chunk.
#include "common.cuh"

namespace xn {
namespace {

constexpr int X_WARPS = 20;
constexpr int X_DEPTH = 2;   // 32-k steps in flight per warp (4 x 128-bit loads each)
constexpr int X_SMEM = 200 * 1024;

__device__ __forceinline__ void mma_tf32(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split(unsigned x, unsigned &hi, unsigned &lo) {
    // nearest tf32 (ties away from zero) with two integer ops: add half an ulp of the 10-bit mantissa to the
    // sign-magnitude bit pattern, clear the 13 low bits; a carry into the exponent is the correct rounding
    hi = (x + 0x00001000u) & 0xFFFFE000u;  // |x - hi| <= 2^-11 |x|
    // the remainder is exact in f32 (12 significant bits); the MMA would cut it to its upper 11, so it is
    // rounded to the tf32 grid here instead: half the error, and no bias towards zero
    lo = (__float_as_uint(__uint_as_float(x) - __uint_as_float(hi)) + 0x00001000u) & 0xFFFFE000u;
}
// total += v with the rounding error of the addition carried in comp (Kahan): the sum of the per-step MMA
// accumulators is then as good as one rounding, however long k is
__device__ __forceinline__ void fold(float &total, float &comp, float v) {
    const float yv = v - comp;
    const float tv = total + yv;
    comp = (tv - total) - yv;
    total = tv;
}
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool pred) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    int sz = pred ? 16 : 0;  // size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz));
}

// staged row pitch in bytes for a chunk of kc elements: 16 bytes past a multiple of 128, so that the
// eight lanes of a 128-bit access phase (two rows x four 32-byte segments) fall in distinct bank groups
__host__ __device__ inline int x_pitch(int kc) { return (kc + 31) / 32 * 128 + 16; }

template <int MT>
__global__ void __launch_bounds__(X_WARPS * 32, 1)
gemv_f32x3_kernel(float *__restrict__ y, const float *__restrict__ x, const float *__restrict__ w, int m, size_t n, int k,
                  size_t ldy, size_t ldx, size_t ldw, int kchunk, int tiles, int tpc, int ksplit, int w_static) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = x_pitch(kchunk);
    unsigned char *sX = smem;  // MT*8 rows of f32
    float *red = reinterpret_cast<float *>(smem + (size_t)MT * 8 * RS);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tl = (int)((unsigned)warp / (unsigned)ksplit), ks = warp - tl * ksplit;
    const int tile = blockIdx.x * tpc + tl;
    const bool valid = tile < tiles;
    const size_t r0 = valid ? min((size_t)tile * 16 + g, n - 1) : 0, r1 = valid ? min((size_t)tile * 16 + g + 8, n - 1) : 0;

    float total[MT][4], comp[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[mt][i] = comp[mt][i] = 0.0f;

    // A weight operand that the previous kernel in the stream may have written is read only after that kernel
    // has completed; a static weight is prefetched ahead of the wait below.
    if (!w_static) asm volatile("griddepcontrol.wait;" ::: "memory");

    for (int kc0 = 0; kc0 < k; kc0 += kchunk) {
        const int kc = min(kchunk, k - kc0);
        const int nst = kc / 32;  // 32-k steps in this chunk (k is a multiple of 32)
        const int sq = nst / ksplit, sr = nst - sq * ksplit;
        const int st0 = ks * sq + min(ks, sr);
        const int st1 = valid ? st0 + sq + (ks < sr ? 1 : 0) : st0;
        const float *wp0 = w + r0 * ldw + kc0 + 8 * t;
        const float *wp1 = w + r1 * ldw + kc0 + 8 * t;
        uint4 wa[X_DEPTH][2], wb[X_DEPTH][2];  // rows g and g+8: 8 consecutive k each
        auto load = [&](int i, int st) {
            if (st < st1) {
                wa[i][0] = ldg_stream(wp0 + (size_t)st * 32);
                wa[i][1] = ldg_stream(wp0 + (size_t)st * 32 + 4);
                wb[i][0] = ldg_stream(wp1 + (size_t)st * 32);
                wb[i][1] = ldg_stream(wp1 + (size_t)st * 32 + 4);
            } else {
                wa[i][0] = wa[i][1] = wb[i][0] = wb[i][1] = make_uint4(0, 0, 0, 0);
            }
        };
#pragma unroll
        for (int i = 0; i < X_DEPTH; ++i) load(i, st0 + i);

        if (kc0 == 0) {
            // Everything so far read only the (static) weights; the activations may come from the previous kernel.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        } else {
            __syncthreads();  // every warp is done with the previous chunk
        }
        const int cols16 = kc / 4;  // 16-byte pieces per row
        for (int idx = tid; idx < MT * 8 * cols16; idx += blockDim.x) {
            const int row = (int)((unsigned)idx / (unsigned)cols16), c = idx - row * cols16;
            const bool ok = row < m;
            cp_async16(sX + (size_t)row * RS + (size_t)c * 16, x + (ok ? (size_t)row * ldx + kc0 + (size_t)c * 4 : 0), ok);
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        for (int st = st0; st < st1; st += X_DEPTH) {
#pragma unroll
            for (int i = 0; i < X_DEPTH; ++i) {
                if (st + i < st1) {
                    const unsigned wg[8] = {wa[i][0].x, wa[i][0].y, wa[i][0].z, wa[i][0].w, wa[i][1].x, wa[i][1].y, wa[i][1].z, wa[i][1].w};
                    const unsigned wh[8] = {wb[i][0].x, wb[i][0].y, wb[i][0].z, wb[i][0].w, wb[i][1].x, wb[i][1].y, wb[i][1].z, wb[i][1].w};
                    unsigned ah[8], al[8], bh[8], bl[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        split(wg[e], ah[e], al[e]);
                        split(wh[e], bh[e], bl[e]);
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const unsigned char *xr = sX + (size_t)(8 * mt + g) * RS + (size_t)(st + i) * 128 + 32 * t;
                        const uint4 x0 = *reinterpret_cast<const uint4 *>(xr);
                        const uint4 x1 = *reinterpret_cast<const uint4 *>(xr + 16);
                        const unsigned xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        // The tensor core adds into its accumulator with truncation, so nothing of full size is
                        // ever accumulated there: each hi x hi MMA (8 k) starts from zero, the 2^-11 smaller cross
                        // terms of the whole step share one accumulator, and the results are added with ordinary
                        // roundings before the compensated fold into the running total.
                        float sum[4], small[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            unsigned xh0, xl0, xh1, xl1;
                            split(xv[2 * q], xh0, xl0);
                            split(xv[2 * q + 1], xh1, xl1);
                            mma_tf32(small, al[2 * q], bl[2 * q], al[2 * q + 1], bl[2 * q + 1], xh0, xh1);
                            mma_tf32(small, ah[2 * q], bh[2 * q], ah[2 * q + 1], bh[2 * q + 1], xl0, xl1);
                            float big[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            mma_tf32(big, ah[2 * q], bh[2 * q], ah[2 * q + 1], bh[2 * q + 1], xh0, xh1);
#pragma unroll
                            for (int e = 0; e < 4; ++e) sum[e] = q == 0 ? big[e] : sum[e] + big[e];
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) fold(total[mt][e], comp[mt][e], sum[e] + small[e]);
                    }
                }
                load(i, st + i + X_DEPTH);
            }
        }
    }

    // fixed-order reduction over the ksplit warps of a tile, then the store
    if (ksplit > 1) {
        if (ks > 0)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) red[((size_t)warp * MT * 4 + mt * 4 + i) * 32 + lane] = total[mt][i];
        __syncthreads();
        if (ks == 0)
            for (int o = 1; o < ksplit; ++o)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) total[mt][i] += red[((size_t)(warp + o) * MT * 4 + mt * 4 + i) * 32 + lane];
    }
    if (ks == 0 && valid) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const size_t row_n = (size_t)tile * 16 + g + 8 * (i >> 1);
                const int row_m = 8 * mt + 2 * t + (i & 1);
                if (row_n < n && row_m < m) y[(size_t)row_m * ldy + row_n] = total[mt][i];
            }
    }
}

template <int MT>
int launch(float *y, const float *x, const float *w, int m, size_t n, int k, size_t ldy, size_t ldx, size_t ldw,
           cudaStream_t st) {
    const int tiles = (int)((n + 15) / 16);
    const int sms = sm_count();
    int tpc = (tiles + sms - 1) / sms;
    if (tpc > X_WARPS) tpc = X_WARPS;  // very tall weights: more CTAs than SMs
    int ksplit = X_WARPS / tpc;
    // largest k chunk (multiple of 256) whose staged rows fit the shared-memory budget
    int kchunk = (k + 255) / 256 * 256;
    while ((size_t)MT * 8 * x_pitch(kchunk) > (size_t)X_SMEM - X_WARPS * MT * 4 * 32 * 4) kchunk = ((kchunk / 256 + 1) / 2) * 256;
    const int nst = (kchunk < k ? kchunk : k) / 32;
    if (ksplit > nst / X_DEPTH) ksplit = nst / X_DEPTH;
    if (ksplit < 1) ksplit = 1;
    const int warps = tpc * ksplit;
    const int grid = (tiles + tpc - 1) / tpc;
    const size_t smem = (size_t)MT * 8 * x_pitch(kchunk) + (size_t)warps * MT * 4 * 32 * sizeof(float);
    auto kern = gemv_f32x3_kernel<MT>;
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
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, y, x, w, m, n, k, ldy, ldx, ldw, kchunk, tiles, tpc, ksplit, rhs_is_static() ? 1 : 0));
    return XN_OK;
}

}  // namespace

// Caller guarantees: f32, m <= 16, one batch, k a multiple of 32, lhs/rhs k-contiguous with pitches that are
// multiples of 4 elements, 16-byte aligned bases, dst rows contiguous.
int launch_gemv_f32x3(float *dst, const float *lhs, const float *rhs, size_t m, size_t n, size_t k, size_t dst_rs,
                      size_t lhs_rs, size_t rhs_cs, cudaStream_t st) {
    if (m <= 8) return launch<1>(dst, lhs, rhs, (int)m, n, (int)k, dst_rs, lhs_rs, rhs_cs, st);
    return launch<2>(dst, lhs, rhs, (int)m, n, (int)k, dst_rs, lhs_rs, rhs_cs, st);
}

}  // namespace xn
