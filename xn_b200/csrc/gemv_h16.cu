// 16-bit (bf16 / f16) decode-sized matmul_t (lhs [m,k], rhs [n,k] both k-contiguous, m <= 16) on the
// tensor cores: the decode-time Linear::forward of an unquantized model, which the reference sends to
// cublasGemmStridedBatchedEx with f32 accumulation (xn-core/src/cuda_backend.rs:2151-2257).
//
// HBM-bound by the weights.  Output rows ride the 16-row dimension of mma.sync.m16n8k16 (a native
// tensor instruction on sm_100a for both 16-bit types), the activation rows its 8 columns (1 or 2 column
// groups; the instruction issues at about one per 32 cycles per SM sub-partition here, so with 4 groups the
// kernel would be bound by it: 35 us at m = 32 on [12288, 4096] against 18 us at m <= 8).  A lane's 128-bit load of a weight row (8 consecutive k) feeds two MMAs through a
// fixed k permutation that the activation fragment follows, so a 64-byte k step costs two loads and,
// per column group, one 128-bit shared-memory read and two MMAs: about a dozen instructions per KB of
// weights (the FFMA kernel this replaces for these shapes needed one FMA per weight element and
// activation row and measured 96 us on [12288, 4096] at m = 16 where cuBLAS takes 20 us).
// DEPTH steps per warp are in flight in registers, the first ones before the dependency wait of a
// programmatic dependent launch; the activations are staged in shared memory, per k chunk when they
// do not fit at once.  Accumulation is f32, k-split partial sums meet in a fixed order.
#include "common.cuh"

namespace xn {
namespace {

constexpr int H_WARPS = 20;
constexpr int H_DEPTH = 6;   // 64-byte k steps in flight per warp (two 128-bit loads each)
constexpr int H_SMEM = 200 * 1024;

template <typename T> struct Mma;
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool pred) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    int sz = pred ? 16 : 0;  // size 0: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz));
}

// staged row pitch in bytes for a chunk of kc elements: 64 bytes past a multiple of 128, so that the
// eight lanes of a 128-bit access phase (two rows x four 16-byte segments) fall in distinct bank groups
__host__ __device__ inline int h_pitch(int kc) { return (kc + 63) / 64 * 128 + 64; }

template <typename T, int MT>
__global__ void __launch_bounds__(H_WARPS * 32, 1)
gemv_h16_kernel(T *__restrict__ y, const T *__restrict__ x, const T *__restrict__ w, int m, size_t n, int k, size_t ldy,
                size_t ldx, size_t ldw, int kchunk, int tiles, int tpc, int ksplit, int w_static) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int RS = h_pitch(kchunk);
    unsigned char *sX = smem;  // MT*8 rows of 16-bit elements
    float *red = reinterpret_cast<float *>(smem + (size_t)MT * 8 * RS);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tl = (int)((unsigned)warp / (unsigned)ksplit), ks = warp - tl * ksplit;
    const int tile = blockIdx.x * tpc + tl;
    const bool valid = tile < tiles;
    const size_t r0 = valid ? min((size_t)tile * 16 + g, n - 1) : 0, r1 = valid ? min((size_t)tile * 16 + g + 8, n - 1) : 0;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    // A weight operand that the previous kernel in the stream may have written is read only after that kernel
    // has completed; a static weight is prefetched ahead of the wait below.
    if (!w_static) asm volatile("griddepcontrol.wait;" ::: "memory");

    for (int kc0 = 0; kc0 < k; kc0 += kchunk) {
        const int kc = min(kchunk, k - kc0);
        const int nst = (kc + 31) / 32;  // 32-k (64-byte) steps in this chunk
        const int sq = nst / ksplit, sr = nst - sq * ksplit;
        const int st0 = ks * sq + min(ks, sr);
        const int st1 = valid ? st0 + sq + (ks < sr ? 1 : 0) : st0;
        const T *wp0 = w + r0 * ldw + kc0 + 8 * t;
        const T *wp1 = w + r1 * ldw + kc0 + 8 * t;
        uint4 wa[H_DEPTH], wb[H_DEPTH];  // rows g and g+8: 8 consecutive k each
        auto load = [&](int i, int st) {
            if (st < st1 && st * 32 + 8 * t < kc) {
                wa[i] = ldg_stream(wp0 + (size_t)st * 32);
                wb[i] = ldg_stream(wp1 + (size_t)st * 32);
            } else {
                wa[i] = wb[i] = make_uint4(0, 0, 0, 0);
            }
        };
#pragma unroll
        for (int i = 0; i < H_DEPTH; ++i) load(i, st0 + i);

        if (kc0 == 0) {
            // Everything so far read only the (static) weights; the activations may come from the previous kernel.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        } else {
            __syncthreads();  // every warp is done with the previous chunk
        }
        // stage rows [0, 8*MT) x elements [kc0, kc0 + round32(kc)), zero-filled outside [0, m) x [0, kc)
        const int cols16 = nst * 4;  // 16-byte pieces per staged row
        for (int idx = tid; idx < MT * 8 * cols16; idx += blockDim.x) {
            const int row = (int)((unsigned)idx / (unsigned)cols16), c = idx - row * cols16;
            const bool ok = row < m && c * 8 < kc;
            cp_async16(sX + (size_t)row * RS + (size_t)c * 16, x + (ok ? (size_t)row * ldx + kc0 + (size_t)c * 8 : 0), ok);
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        for (int st = st0; st < st1; st += H_DEPTH) {
#pragma unroll
            for (int i = 0; i < H_DEPTH; ++i) {
                if (st + i < st1) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint4 xv = *reinterpret_cast<const uint4 *>(sX + (size_t)(8 * mt + g) * RS + (size_t)(st + i) * 64 + 16 * t);
                        Mma<T>::run(acc[mt], wa[i].x, wb[i].x, wa[i].y, wb[i].y, xv.x, xv.y);
                        Mma<T>::run(acc[mt], wa[i].z, wb[i].z, wa[i].w, wb[i].w, xv.z, xv.w);
                    }
                }
                load(i, st + i + H_DEPTH);
            }
        }
    }

    // fixed-order reduction over the ksplit warps of a tile, then the store
    if (ksplit > 1) {
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
                if (row_n < n && row_m < m) y[(size_t)row_m * ldy + row_n] = from_f32<T>(acc[mt][i]);
            }
    }
}

template <typename T, int MT>
int launch(T *y, const T *x, const T *w, int m, size_t n, int k, size_t ldy, size_t ldx, size_t ldw, cudaStream_t st) {
    const int tiles = (int)((n + 15) / 16);
    const int sms = sm_count();
    int tpc = (tiles + sms - 1) / sms;
    if (tpc > H_WARPS) tpc = H_WARPS;  // very tall weights: more CTAs than SMs
    int ksplit = H_WARPS / tpc;
    // largest k chunk (multiple of 256) whose staged rows fit the shared-memory budget
    int kchunk = (k + 255) / 256 * 256;
    while ((size_t)MT * 8 * h_pitch(kchunk) > (size_t)H_SMEM - H_WARPS * MT * 4 * 32 * 4) kchunk = ((kchunk / 256 + 1) / 2) * 256;
    const int nst = ((kchunk < k ? kchunk : k) + 31) / 32;
    if (ksplit > nst / H_DEPTH) ksplit = nst / H_DEPTH;
    if (ksplit < 1) ksplit = 1;
    const int warps = tpc * ksplit;
    const int grid = (tiles + tpc - 1) / tpc;
    const size_t smem = (size_t)MT * 8 * h_pitch(kchunk) + (size_t)warps * MT * 4 * 32 * sizeof(float);
    auto kern = gemv_h16_kernel<T, MT>;
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

template <typename T>
int launch_t(void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k, size_t dst_rs, size_t lhs_rs,
             size_t rhs_cs, cudaStream_t st) {
    T *y = (T *)dst;
    const T *x = (const T *)lhs, *w = (const T *)rhs;
    if (m <= 8) return launch<T, 1>(y, x, w, (int)m, n, (int)k, dst_rs, lhs_rs, rhs_cs, st);
    return launch<T, 2>(y, x, w, (int)m, n, (int)k, dst_rs, lhs_rs, rhs_cs, st);
}

}  // namespace

// True when the staged activations of an m x k problem fit in shared memory at once (no k chunking): the
// case this kernel is good at.  Chunked, it loses to the tcgen05 skinny kernel.
bool gemv_h16_single_chunk(size_t m, size_t k) {
    const size_t mt = m <= 8 ? 1 : 2;
    return mt * 8 * (size_t)h_pitch((int)((k + 255) / 256 * 256)) <= (size_t)H_SMEM - H_WARPS * mt * 4 * 32 * 4;
}

// Caller guarantees: f16 or bf16, m <= 16, one batch, k a multiple of 8, lhs/rhs k-contiguous with pitches that
// are multiples of 8 elements, 16-byte aligned bases, dst rows contiguous.
int launch_gemv_h16(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k, size_t dst_rs,
                    size_t lhs_rs, size_t rhs_cs, cudaStream_t st) {
    if (dt == XN_F16) return launch_t<__half>(dst, lhs, rhs, m, n, k, dst_rs, lhs_rs, rhs_cs, st);
    return launch_t<__nv_bfloat16>(dst, lhs, rhs, m, n, k, dst_rs, lhs_rs, rhs_cs, st);
}

}  // namespace xn
