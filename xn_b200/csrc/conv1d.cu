// conv1d and conv_transpose1d as implicit GEMMs on the tensor cores, with the argument lists of
// Backend::conv1d / Backend::conv_transpose1d (xn-core/src/backend.rs:275-316).
//
// The reference lowers both to a GEMM through memory: conv1d is im2col -> cuBLAS -> transpose
// (xn-core/src/cuda_backend.rs:1490-1561), conv_transpose1d is transpose -> cuBLAS -> col2im
// (xn-core/src/cuda_backend.rs:1783-1856); grouped or padded forms fall back to one thread per output
// element.  Here nothing but the input, the kernel and the output touches HBM:
//
//   * a CTA owns a 64 (output channels) x 64 (output positions) tile of one batch entry and one group;
//   * per chunk of input channels it stages, once, the window of input positions its 64 outputs can
//     reach as sX[position][channel] and the kernel taps as sW[tap][out channel][channel];
//   * every tap is then a row-shifted view of that one window: the B fragment of output position j and
//     tap t is the row  j*step + t*tap_step + origin  of sX, which ldmatrix fetches from any row, so
//     stride, dilation and padding cost nothing and the im2col matrix never exists;
//   * conv_transpose1d is split by output phase r = (position + padding) mod stride: outputs of one
//     phase see only the taps r, r+stride, ... and are a stride-1 correlation over the input, so no
//     product with a structural zero is formed and no col2im scatter is needed.
//
// f16 / bf16 use mma.sync.m16n8k16 with f32 accumulation; f32 uses three mma.sync.m16n8k8.tf32 per
// product on a hi/lo split of both operands (products to ~1e-6, exact on small integers).  Groups with
// fewer than 8 channels per group (depthwise) and windows that do not fit shared memory take the direct
// kernel at the end of the file: one thread per output element, f32 accumulation.
#include "common.cuh"

namespace xn {
namespace {

constexpr int C_TM = 64, C_TN = 64, C_THREADS = 128;
constexpr int C_ROW = 64;             // bytes of channels per staged row (32 x 16-bit or 16 x f32)
constexpr int C_PITCH = C_ROW + 16;   // 80-byte rows: the 8 rows of an ldmatrix phase hit 8 distinct 16-byte bank groups

struct ConvArgs {
    int batch, cin_g, cout_g, groups;   // channels per group
    int length, out_length, ksize;
    int stride, padding, dilation;
    int taps;        // taps staged per pass (ksize, or the most one phase of the transposed form sees)
    int rows;        // staged window rows
    int ntile;       // tiles along the position axis
    int wvec;        // conv1d taps can be staged with 128-bit loads
};

__device__ __forceinline__ unsigned smem_addr(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1, __half) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1, __nv_bfloat16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo with both pieces on the tf32 grid (round to nearest by integer arithmetic): the remainder x - hi is
// exact in f32 and would be cut, not rounded, by the MMA
__device__ __forceinline__ void split_tf32(float x, unsigned &hi, unsigned &lo) {
    hi = (__float_as_uint(x) + 0x1000u) & 0xFFFFE000u;
    lo = (__float_as_uint(x - __uint_as_float(hi)) + 0x1000u) & 0xFFFFE000u;
}
__device__ __forceinline__ void mma_tf32_zero(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// One CTA: 64 output channels x 64 output positions of one (batch entry, group[, phase]).
// TR = false: conv1d, kernel [cout, cin_g, ksize].  TR = true: conv_transpose1d, kernel [cin, cout_g, ksize].
template <typename T, bool TR>
__global__ void __launch_bounds__(C_THREADS)
conv_igemm_kernel(T *__restrict__ dst, const T *__restrict__ src, const T *__restrict__ kernel, const T *__restrict__ bias,
                  ConvArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int ES = (int)sizeof(T);
    constexpr int CK = C_ROW / ES;          // channels per staged chunk
    unsigned char *sX = smem;               // [rows][CK]
    unsigned char *sW = smem + (size_t)a.rows * C_PITCH;  // [taps][64][CK]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int wm = warp >> 1, wn = warp & 1;

    const int cotiles = (a.cout_g + C_TM - 1) / C_TM;
    const int grp = blockIdx.y / cotiles, co0 = (blockIdx.y - grp * cotiles) * C_TM;
    const int phases = TR ? a.stride : 1;
    const int b = blockIdx.z / phases, r = blockIdx.z - b * phases;
    const int j0 = blockIdx.x * C_TN;

    // taps this CTA uses, the input position of window row 0, and the row of (position j, tap t)
    const int ntap = TR ? (a.ksize > r ? (a.ksize - r + a.stride - 1) / a.stride : 0) : a.ksize;
    const int win0 = TR ? j0 - (a.taps - 1) : j0 * a.stride - a.padding;
    const int sj = TR ? 1 : a.stride, st = TR ? -1 : a.dilation, off = TR ? a.taps - 1 : 0;

    const int cin = a.cin_g * a.groups, cout = a.cout_g * a.groups;
    const T *srcb = src + ((size_t)b * cin + (size_t)grp * a.cin_g) * a.length;

    // f32 only: the tensor core adds into its accumulator with truncation, so the full-size hi x hi products are
    // never accumulated there -- each such MMA starts from zero and is added to `acc` with a compensated (Kahan)
    // add (`comp`), while the 2^-11 smaller cross terms share the chained accumulator `small`
    constexpr int NC = ES == 4 ? 4 : 1;
    float acc[2][4][4], comp[2][4][NC], small[2][4][NC];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[i][j][e] = 0.f;
                if (e < NC) comp[i][j][e] = small[i][j][e] = 0.f;
            }

    // per-lane fragment addresses (tap 0, k step 0)
    unsigned abase[2], bbase[4];
    if constexpr (ES == 2) {
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
            abase[mi] = smem_addr(sW) + (32 * wm + 16 * mi + (lane & 15)) * C_PITCH + (lane >> 4) * 16;
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            const int j = 32 * wn + 8 * (2 * pr + (lane >> 4)) + (lane & 7);
            bbase[pr] = smem_addr(sX) + (j * sj + off) * C_PITCH + ((lane >> 3) & 1) * 16;
        }
    } else {
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) abase[mi] = smem_addr(sW) + (32 * wm + 16 * mi + g) * C_PITCH + tq * 4;
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) bbase[ni] = smem_addr(sX) + ((32 * wn + 8 * ni + g) * sj + off) * C_PITCH + tq * 4;
    }

    for (int c0 = 0; c0 < a.cin_g; c0 += CK) {
        __syncthreads();
        // the input window, transposed on the way in: global reads run along positions, rows hold channels
        for (int ci = warp; ci < CK; ci += C_THREADS / 32) {
            const bool cok = c0 + ci < a.cin_g;
            const T *row = srcb + (size_t)(c0 + ci) * a.length;
            for (int p = lane; p < a.rows; p += 32) {
                const int li = win0 + p;
                T v = from_f32<T>(0.f);
                if (cok && li >= 0 && li < a.length) v = row[li];
                *reinterpret_cast<T *>(sX + p * C_PITCH + ci * ES) = v;
            }
        }
        // the taps: sW[tap][out channel][channel]
        if constexpr (!TR) {
            const int run = CK * a.ksize;   // one output channel's (channel, tap) pairs of this chunk are contiguous
            for (int co = warp; co < C_TM; co += C_THREADS / 32) {
                const bool ook = co0 + co < a.cout_g;
                const T *wrow = kernel + (((size_t)grp * a.cout_g + co0 + co) * a.cin_g + c0) * a.ksize;
                if (a.wvec) {
                    // whole chunks and 16-byte aligned runs: 128-bit loads, one division per load
                    constexpr int V = 16 / ES;
#pragma unroll 2
                    for (int v = lane; v < run / V; v += 32) {
                        uint4 q = make_uint4(0u, 0u, 0u, 0u);
                        if (ook) q = __ldg(reinterpret_cast<const uint4 *>(wrow) + v);
                        const T *el = reinterpret_cast<const T *>(&q);
                        int ci = (v * V) / a.ksize, kk = v * V - ci * a.ksize;
#pragma unroll
                        for (int j = 0; j < V; ++j) {
                            *reinterpret_cast<T *>(sW + (kk * C_TM + co) * C_PITCH + ci * ES) = el[j];
                            if (++kk == a.ksize) { kk = 0; ++ci; }
                        }
                    }
                    continue;
                }
                for (int e = lane; e < run; e += 32) {
                    const int ci = e / a.ksize, kk = e - ci * a.ksize;
                    T v = from_f32<T>(0.f);
                    if (ook && c0 + ci < a.cin_g) v = wrow[e];
                    *reinterpret_cast<T *>(sW + (kk * C_TM + co) * C_PITCH + ci * ES) = v;
                }
            }
        } else {
            const int run = C_TM * a.ksize; // one input channel's (out channel, tap) pairs of this tile are contiguous
            for (int ci = warp; ci < CK; ci += C_THREADS / 32) {
                const bool cok = c0 + ci < a.cin_g;
                const T *wrow = kernel + (((size_t)grp * a.cin_g + c0 + ci) * a.cout_g + co0) * a.ksize;
                for (int e = lane; e < run; e += 32) {
                    const int co = e / a.ksize, kk = e - co * a.ksize;
                    const int t = kk / a.stride;
                    if (kk - t * a.stride != r) continue;
                    T v = from_f32<T>(0.f);
                    if (cok && co0 + co < a.cout_g) v = wrow[e];
                    *reinterpret_cast<T *>(sW + (t * C_TM + co) * C_PITCH + ci * ES) = v;
                }
            }
        }
        __syncthreads();

        for (int t = 0; t < ntap; ++t) {
            const unsigned aoff = t * C_TM * C_PITCH;
            const int boff = t * st * C_PITCH;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                if constexpr (ES == 2) {
                    unsigned af[2][4], bf[2][4];
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) ldmatrix_x4(af[mi], abase[mi] + aoff + ks * 32);
#pragma unroll
                    for (int pr = 0; pr < 2; ++pr) ldmatrix_x4(bf[pr], bbase[pr] + boff + ks * 32);
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                        for (int ni = 0; ni < 4; ++ni)
                            mma16(acc[mi][ni], af[mi], bf[ni >> 1][(ni & 1) * 2], bf[ni >> 1][(ni & 1) * 2 + 1], T());
                } else {
                    unsigned ah[2][4], al[2][4], bh[4][2], bl[4][2];
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        const unsigned ad = abase[mi] + aoff + ks * 32;
                        float v0, v1, v2, v3;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v0) : "r"(ad));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v1) : "r"(ad + 8 * C_PITCH));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v2) : "r"(ad + 16));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v3) : "r"(ad + 8 * C_PITCH + 16));
                        split_tf32(v0, ah[mi][0], al[mi][0]);
                        split_tf32(v1, ah[mi][1], al[mi][1]);
                        split_tf32(v2, ah[mi][2], al[mi][2]);
                        split_tf32(v3, ah[mi][3], al[mi][3]);
                    }
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni) {
                        const unsigned bd = bbase[ni] + boff + ks * 32;
                        float v0, v1;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v0) : "r"(bd));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v1) : "r"(bd + 16));
                        split_tf32(v0, bh[ni][0], bl[ni][0]);
                        split_tf32(v1, bh[ni][1], bl[ni][1]);
                    }
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                        for (int ni = 0; ni < 4; ++ni) {
                            float (&sm)[4] = reinterpret_cast<float (&)[4]>(small[mi][ni]);
                            mma_tf32(sm, al[mi], bh[ni][0], bh[ni][1]);
                            mma_tf32(sm, ah[mi], bl[ni][0], bl[ni][1]);
                            float big[4];
                            mma_tf32_zero(big, ah[mi], bh[ni][0], bh[ni][1]);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float yv = big[e] - comp[mi][ni][e % NC];
                                const float tv = acc[mi][ni][e] + yv;
                                comp[mi][ni][e % NC] = (tv - acc[mi][ni][e]) - yv;
                                acc[mi][ni][e] = tv;
                            }
                        }
                }
            }
        }
    }

    if constexpr (ES == 4) {
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[mi][ni][e] += small[mi][ni][e % NC];
    }
    // epilogue: bias, one rounding to T, rows of the output are position-contiguous
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int co = co0 + 32 * wm + 16 * mi + g + 8 * hf;
            if (co >= a.cout_g) continue;
            const int cog = grp * a.cout_g + co;
            const float bv = bias ? to_f32(bias[cog]) : 0.f;
            T *drow = dst + ((size_t)b * cout + cog) * a.out_length;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + 32 * wn + 8 * ni + 2 * tq + e;
                    const int lo = TR ? j * a.stride + r - a.padding : j;
                    if (lo >= 0 && lo < a.out_length) drow[lo] = from_f32<T>(acc[mi][ni][hf * 2 + e] + bv);
                }
        }
}

// One thread per output element, f32 accumulation: depthwise and other thin groups, and windows too
// large to stage.  The loops are those of conv1d_direct / conv_transpose1d_direct
// (xn-core/src/cpu_backend.rs:1233-1310, 1354-1430) read per output element.
template <typename T, bool TR>
__global__ void __launch_bounds__(256)
conv_direct_kernel(T *__restrict__ dst, const T *__restrict__ src, const T *__restrict__ kernel, const T *__restrict__ bias,
                   ConvArgs a, size_t total) {
    const int cin = a.cin_g * a.groups, cout = a.cout_g * a.groups;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int lo = (int)(i % a.out_length);
        const size_t bc = i / a.out_length;
        const int co = (int)(bc % cout), b = (int)(bc / cout);
        const int grp = co / a.cout_g, cog = co - grp * a.cout_g;
        const T *srcb = src + ((size_t)b * cin + (size_t)grp * a.cin_g) * a.length;
        // f32 products summed in runs of 16 channels; the runs go into the total with a compensated (Kahan) add, so
        // that a long cin * ksize sum stays within the f32 parity bound (1e-6 of the output's rms)
        float s = 0.f, comp = 0.f;
        auto fold = [&](float part) {
            const float yv = part - comp, tv = s + yv;
            comp = (tv - s) - yv;
            s = tv;
        };
        if (!TR) {
            const T *w = kernel + (size_t)co * a.cin_g * a.ksize;
            for (int kk = 0; kk < a.ksize; ++kk) {
                const int li = lo * a.stride + kk * a.dilation - a.padding;
                if (li < 0 || li >= a.length) continue;
                for (int c0 = 0; c0 < a.cin_g; c0 += 16) {
                    float part = 0.f;
                    for (int ci = c0; ci < min(c0 + 16, a.cin_g); ++ci)
                        part += to_f32(srcb[(size_t)ci * a.length + li]) * to_f32(w[(size_t)ci * a.ksize + kk]);
                    fold(part);
                }
            }
        } else {
            const int raw = lo + a.padding, r = raw % a.stride;
            for (int kk = r; kk < a.ksize; kk += a.stride) {
                const int li = (raw - kk) / a.stride;
                if (raw < kk || li >= a.length) continue;
                for (int c0 = 0; c0 < a.cin_g; c0 += 16) {
                    float part = 0.f;
                    for (int ci = c0; ci < min(c0 + 16, a.cin_g); ++ci)
                        part += to_f32(srcb[(size_t)ci * a.length + li]) *
                                to_f32(kernel[(((size_t)grp * a.cin_g + ci) * a.cout_g + cog) * a.ksize + kk]);
                    fold(part);
                }
            }
        }
        if (bias) s += to_f32(bias[co]);
        dst[i] = from_f32<T>(s);
    }
}

// ---------------------------------------------------------------------------------------------------
// 16-bit types, groups == 1, dilation == 1, channels a multiple of 8: the tensor-memory GEMM kernel does
// the work.  With the input repacked channels-last and zero-padded, xt[b][position][channel], the im2col
// row of output position l is the contiguous run of kernel_size * in_channels elements that starts at
// xt[b][l * stride][0]: the im2col matrix is a view of xt whose rows overlap (row pitch stride *
// in_channels), which a TMA tensor map describes as it stands.  The kernel taps are repacked once per
// call to [out channel][tap][channel]; dst[b] = taps * view^T lands directly in (out_channels,
// out_length) layout, bias added in the GEMM epilogue.  conv_transpose1d runs every output phase as
// extra rows of the same GEMM (rows = (phase, out channel), columns = position / stride) and a last pass
// interleaves the phases into the output.
// ---------------------------------------------------------------------------------------------------
// Packed rows.  16-bit types: `cin` channels.  f32: three pieces of `cin` words on the tf32 grid each, the input
// as (hi | hi | lo) and the taps as (hi | lo | hi), so that one kind::tf32 dot product over the tripled row is
// x_hi*w_hi + x_hi*w_lo + x_lo*w_hi: f32 products to ~2^-21 relative on MMAs that read 11-bit mantissas.
template <typename T> __host__ __device__ constexpr int pack_mult() { return sizeof(T) == 4 ? 3 : 1; }
__device__ __forceinline__ float tf32_round(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }
template <typename T, bool IS_TAP>
__device__ __forceinline__ void pack_store(T *row, int cin, int c, T v) {
    if constexpr (sizeof(T) == 4) {
        const float hi = tf32_round(v), lo = tf32_round(v - hi);
        row[c] = hi;
        row[cin + c] = IS_TAP ? lo : hi;
        row[2 * cin + c] = IS_TAP ? hi : lo;
    } else {
        row[c] = v;
    }
}

// xt[b][lead + l][c] = x[b][c][l]; rows outside [lead, lead + length) are zero.  32 x 32 tiles through
// shared memory so that both the reads (along l) and the writes (along c) are coalesced.
constexpr int PI_C = 128;   // channels per block of the input repack
template <typename T>
__global__ void __launch_bounds__(256)
conv_pack_input_kernel(T *__restrict__ xt, const T *__restrict__ x, int cin, int length, int lead, int rows) {
    // 32 positions x 128 channels per block: 16 independent loads per thread in flight, output rows written in
    // runs of 128 channels
    __shared__ T tile[PI_C][33];
    const int b = blockIdx.z, r0 = blockIdx.x * 32, c0 = blockIdx.y * PI_C;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const T *xb = x + (size_t)b * cin * length;
    T *xtb = xt + (size_t)b * rows * cin * pack_mult<T>();
    const int l = r0 + tx - lead;
    const bool lok = l >= 0 && l < length;
#pragma unroll 8
    for (int i = ty; i < PI_C; i += 8) {
        const int c = c0 + i;
        T v = from_f32<T>(0.f);
        if (lok && c < cin) v = xb[(size_t)c * length + l];
        tile[i][tx] = v;
    }
    __syncthreads();
    const int c = threadIdx.x & (PI_C - 1);
    if (c0 + c < cin) {
#pragma unroll 4
        for (int i = threadIdx.x / PI_C; i < 32; i += 256 / PI_C) {
            const int r = r0 + i;
            if (r < rows) pack_store<T, false>(xtb + (size_t)r * cin * pack_mult<T>(), cin, c0 + c, tile[c][i]);
        }
    }
}

// conv1d: wp[co][kk][ci] = w[co][ci][kk]
template <typename T>
__global__ void __launch_bounds__(256)
conv_pack_taps_kernel(T *__restrict__ wp, const T *__restrict__ w, int cin, int ksize, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ci = (int)(i % cin);
        const size_t t = i / cin;
        const int kk = (int)(t % ksize);
        const size_t co = t / ksize;
        pack_store<T, true>(wp + t * cin * pack_mult<T>(), cin, ci, w[(co * cin + ci) * ksize + kk]);
    }
}

// conv_transpose1d: wp[r][co][j][ci] = w[ci][co][r + stride * (taps - 1 - j)] (zero where that tap does not
// exist): row (r, co) of the GEMM, whose k axis runs over (window position j, channel).
template <typename T>
__global__ void __launch_bounds__(256)
conv_pack_taps_tr_kernel(T *__restrict__ wp, const T *__restrict__ w, int cin, int cout, int ksize, int stride, int taps,
                         size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ci = (int)(i % cin);
        const size_t row = i / cin;
        size_t t = row;
        const int j = (int)(t % taps);
        t /= taps;
        const int co = (int)(t % cout), r = (int)(t / cout);
        const int kk = r + stride * (taps - 1 - j);
        pack_store<T, true>(wp + row * cin * pack_mult<T>(), cin, ci,
                            kk < ksize ? w[((size_t)ci * cout + co) * ksize + kk] : from_f32<T>(0.f));
    }
}

// The same two repackings through shared memory, one block per (out channel, 64 input channels): the taps are
// read in runs of kernel_size contiguous elements and written in runs of 64 contiguous channels, so every
// sector moves once (the per-element kernels above touch a sector per element on one side and are kept for
// kernel sizes whose tile does not fit).  TR = false: source (ci, kk) at w[(co * cin + ci) * ksize + kk],
// destination rows co * ksize + kk.  TR = true: source at w[(ci * cout + co) * ksize + kk], destination rows
// ((r * cout + co) * taps + j) holding tap kk = r + stride * (taps - 1 - j) or zeros.
constexpr int PK_CC = 64;
template <typename T, bool TR>
__global__ void __launch_bounds__(256)
conv_pack_taps_tiled_kernel(T *__restrict__ wp, const T *__restrict__ w, int cin, int cout, int ksize, int stride, int taps) {
    extern __shared__ __align__(16) unsigned char pk_smem[];
    T *tile = reinterpret_cast<T *>(pk_smem);   // [PK_CC][ksize + 1]
    const int co = blockIdx.x, c0 = blockIdx.y * PK_CC, pitch = ksize + 1;
    const size_t ci_stride = TR ? (size_t)cout * ksize : (size_t)ksize;
    const T *base = TR ? w + (size_t)co * ksize : w + (size_t)co * cin * ksize;
    for (int e = threadIdx.x; e < PK_CC * ksize; e += 256) {
        const int ci = e / ksize, kk = e - ci * ksize;
        T v = from_f32<T>(0.f);
        if (c0 + ci < cin) v = base[(size_t)(c0 + ci) * ci_stride + kk];
        tile[ci * pitch + kk] = v;
    }
    __syncthreads();
    const int nslots = TR ? stride * taps : ksize;
    const int ci = threadIdx.x & (PK_CC - 1);
    if (c0 + ci >= cin) return;
    for (int sl = threadIdx.x / PK_CC; sl < nslots; sl += 256 / PK_CC) {
        size_t row;
        int kk;
        if (TR) {
            const int r = sl / taps, j = sl - r * taps;
            row = ((size_t)r * cout + co) * taps + j;
            kk = r + stride * (taps - 1 - j);
        } else {
            row = (size_t)co * ksize + sl;
            kk = sl;
        }
        pack_store<T, true>(wp + row * cin * pack_mult<T>(), cin, c0 + ci, kk < ksize ? tile[ci * pitch + kk] : from_f32<T>(0.f));
    }
}

// Phase interleave through shared memory: one block per (batch entry, out channel, 512 values of q); rows of d
// are read contiguously, the output run of 512 * stride positions is written contiguously.
constexpr int IL_QT = 512;
template <typename T>
__global__ void __launch_bounds__(256)
conv_interleave_tiled_kernel(T *__restrict__ out, const T *__restrict__ d, const T *__restrict__ bias, int cout, int out_length,
                             int stride, int padding, int nq) {
    extern __shared__ __align__(16) unsigned char il_smem[];
    T *tile = reinterpret_cast<T *>(il_smem);
    constexpr int PITCH = IL_QT + 4 / (int)sizeof(T);   // an odd number of 32-bit words: phases fall in distinct banks
    const int q0 = blockIdx.x * IL_QT, co = blockIdx.y, b = blockIdx.z;
    const T *db = d + ((size_t)b * stride * cout + co) * nq;
    const size_t row_pitch = (size_t)cout * nq;
#pragma unroll 4
    for (int i = threadIdx.x; i < stride * IL_QT; i += 256) {
        const int r = i / IL_QT, q = i - r * IL_QT;
        if (q0 + q < nq) tile[r * PITCH + q] = db[r * row_pitch + q0 + q];
    }
    __syncthreads();
    const float bv = bias ? to_f32(bias[co]) : 0.f;
    T *ob = out + ((size_t)b * cout + co) * out_length;
    // output position q0 * stride + i - padding holds (q, r) = (i / stride, i % stride); i advances by 256 per
    // iteration, so (q, r) advance by (256 / stride, 256 % stride) with a carry: one division per thread
    const int lo0 = q0 * stride - padding, dq = 256 / stride, dr = 256 - dq * stride;
    int q = threadIdx.x / stride, r = threadIdx.x - q * stride;
#pragma unroll 4
    for (int i = threadIdx.x; i < stride * IL_QT; i += 256) {
        const int lo = lo0 + i;
        if (q0 + q < nq && lo >= 0 && lo < out_length) ob[lo] = from_f32<T>(to_f32(tile[r * PITCH + q]) + bv);
        q += dq;
        r += dr;
        if (r >= stride) { r -= stride; ++q; }
    }
}

// out[b][co][q * stride + r - padding] = d[b][r * cout + co][q] + bias[co]; positions no phase row covers
// (beyond the last tap: output_padding) are bias alone.  One thread per output element, reads gathered.
template <typename T>
__global__ void __launch_bounds__(256)
conv_interleave_kernel(T *__restrict__ out, const T *__restrict__ d, const T *__restrict__ bias, int cout, int out_length,
                       int stride, int padding, int nq, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int lo = (int)(i % out_length);
        const size_t bc = i / out_length;
        const int co = (int)(bc % cout);
        const size_t b = bc / cout;
        const int raw = lo + padding, q = raw / stride, r = raw - q * stride;
        float v = to_f32(d[((b * stride + r) * cout + co) * (size_t)nq + q]);
        if (bias) v += to_f32(bias[co]);
        out[i] = from_f32<T>(v);
    }
}

// out[row][col] = sum over splits of part[s][row][col] (+ bias[row]), summed in split order
__global__ void __launch_bounds__(256)
conv_sum_partials_kernel(float *__restrict__ out, const float *__restrict__ part, const float *__restrict__ bias, int splits,
                         size_t n, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += part[(size_t)k * total + i];
        if (bias) s += bias[i / n];
        out[i] = s;
    }
}

inline size_t round256(size_t v) { return (v + 255) / 256 * 256; }

// Scratch of the tensor-memory path in bytes (0: the call uses the scratch-free kernels).
struct ConvPlan { bool gemm; size_t xt_bytes, wp_bytes, d_bytes, part_bytes; int rows, taps, nq, splits; };

// f32, one batch entry, few output tiles, long k: cut k into equal chunks (multiples of the 32-word k stage)
// so that about one CTA per SM has work; 1 = no split.
inline int conv_splits(size_t m, size_t n, size_t k) {
    if (k % 32) return 1;
    const size_t tiles = ((m + 127) / 128) * ((n + 255) / 256), sms = (size_t)sm_count();
    const size_t units = k / 32;
    if (tiles == 0 || tiles * 2 > sms || units < 8) return 1;
    size_t want = sms / tiles;
    if (want > units / 4) want = units / 4;   // at least 4 k stages per chunk
    if (want > 64) want = 64;
    for (size_t s = want; s > 1; --s)
        if (units % s == 0) return (int)s;
    return 1;
}
template <bool TR>
ConvPlan conv_plan(int dtype, const ConvArgs &a) {
    ConvPlan p{};
    static const bool off = [] { const char *e = getenv("XN_CONV_GEMM"); return e && atoi(e) == 0; }();
    const size_t cin = (size_t)a.cin_g, cout = (size_t)a.cout_g;
    const size_t es = dtype == XN_F32 ? 4 : 2, mult = dtype == XN_F32 ? 3 : 1;
    p.gemm = !off && a.groups == 1 && a.dilation == 1 && (cin * mult * es) % 16 == 0 && a.batch <= 65535;
    if (!p.gemm) return p;
    if (!TR) {
        p.rows = a.length + 2 * a.padding;
        p.taps = a.ksize;
        p.wp_bytes = round256(cout * a.ksize * cin * mult * es);
    } else {
        p.taps = (a.ksize + a.stride - 1) / a.stride;
        p.nq = (a.out_length - 1 + a.padding) / a.stride + 1;
        p.rows = p.nq + p.taps - 1;      // window of position q starts at input position q - (taps - 1)
        p.wp_bytes = round256((size_t)a.stride * cout * p.taps * cin * mult * es);
        p.d_bytes = round256((size_t)a.batch * a.stride * cout * p.nq * es);
    }
    p.xt_bytes = round256((size_t)a.batch * p.rows * cin * mult * es);
    // the GEMM kernel indexes rows, columns and k with 32-bit integers
    if ((size_t)p.taps * cin * mult > 0x7fffffff || (size_t)a.stride * cin * mult > 0x7fffffff ||
        (size_t)a.stride * cout > 0x7fffffff || (size_t)p.rows * cin * mult > ((size_t)1 << 40)) {
        p = ConvPlan{};
        return p;
    }
    p.splits = 1;
    if (dtype == XN_F32 && a.batch == 1) {
        const size_t m = TR ? (size_t)a.stride * cout : cout, n = TR ? (size_t)p.nq : (size_t)a.out_length;
        p.splits = conv_splits(m, n, (size_t)p.taps * cin * mult);
        if (p.splits > 1) {
            p.part_bytes = round256((size_t)p.splits * m * n * 4);
            if (!TR) p.d_bytes = 0;
        }
    }
    return p;
}

template <typename T, bool TR>
int launch_conv_gemm(xn_dtype dt, T *dst, const T *src, const T *kernel, const T *bias, const ConvArgs &a, const ConvPlan &p,
                     unsigned char *ws, cudaStream_t st) {
    const int cin = a.cin_g, cout = a.cout_g;
    T *xt = reinterpret_cast<T *>(ws);
    T *wp = reinterpret_cast<T *>(ws + p.xt_bytes);
    T *d = reinterpret_cast<T *>(ws + p.xt_bytes + p.wp_bytes);
    const int lead = TR ? p.taps - 1 : a.padding;
    dim3 pg((unsigned)((p.rows + 31) / 32), (unsigned)((cin + PI_C - 1) / PI_C), (unsigned)a.batch);
    conv_pack_input_kernel<T><<<pg, 256, 0, st>>>(xt, src, cin, a.length, lead, p.rows);
    const size_t wtotal = TR ? (size_t)a.stride * cout * p.taps * cin : (size_t)cout * a.ksize * cin;
    const unsigned wgrid = (unsigned)((wtotal + 255) / 256 < 4096 ? (wtotal + 255) / 256 : 4096);
    const size_t pk_smem = (size_t)PK_CC * (a.ksize + 1) * sizeof(T);
    if (pk_smem <= 40 * 1024 && cout <= 0x7fffffff / 2 && (cin + PK_CC - 1) / PK_CC <= 65535) {
        dim3 wg((unsigned)cout, (unsigned)((cin + PK_CC - 1) / PK_CC));
        conv_pack_taps_tiled_kernel<T, TR><<<wg, 256, pk_smem, st>>>(wp, kernel, cin, cout, a.ksize, a.stride, p.taps);
    } else if (!TR) {
        conv_pack_taps_kernel<T><<<wgrid, 256, 0, st>>>(wp, kernel, cin, a.ksize, wtotal);
    } else {
        conv_pack_taps_tr_kernel<T><<<wgrid, 256, 0, st>>>(wp, kernel, cin, cout, a.ksize, a.stride, p.taps, wtotal);
    }
    XN_CHECK_CUDA(cudaGetLastError());
    const size_t cpr = (size_t)cin * pack_mult<T>();   // packed row length
    const size_t k = (size_t)p.taps * cpr;
    auto gemm = [&](T *out, const T *row_bias, size_t m, size_t n, size_t ldb, size_t out_bs) -> int {
        if constexpr (sizeof(T) == 4) {
            if (p.splits > 1) {
                float *part = reinterpret_cast<float *>(ws + p.xt_bytes + p.wp_bytes + p.d_bytes);
                if (int rc = launch_gemm_tn_tf32_splitk(part, wp, xt, m, n, k / p.splits, p.splits, k, ldb, st)) return rc;
                const size_t total = m * n;
                const unsigned grid = (unsigned)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
                conv_sum_partials_kernel<<<grid, 256, 0, st>>>(out, part, row_bias, p.splits, n, total);
                XN_CHECK_CUDA(cudaGetLastError());
                return XN_OK;
            }
            return launch_gemm_tn_tf32_shared_lhs(out, wp, xt, row_bias, m, n, k, k, ldb, n, a.batch, (size_t)p.rows * cpr, out_bs, st);
        } else
            return launch_gemm_tn_16bit_shared_lhs(dt, out, wp, xt, row_bias, m, n, k, k, ldb, n, a.batch, (size_t)p.rows * cpr,
                                                   out_bs, st);
    };
    if (!TR) return gemm(dst, bias, cout, a.out_length, (size_t)a.stride * cpr, (size_t)cout * a.out_length);
    const size_t m = (size_t)a.stride * cout;
    if (int rc = gemm(d, nullptr, m, p.nq, cpr, m * p.nq)) return rc;
    const size_t total = (size_t)a.batch * cout * a.out_length;
    const size_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks < (size_t)sm_count() * 32 ? blocks : (size_t)sm_count() * 32);
    const size_t il_smem = (size_t)a.stride * (IL_QT + 4 / sizeof(T)) * sizeof(T);
    if (il_smem <= 40 * 1024 && cout <= 65535) {
        dim3 ig((unsigned)((p.nq + IL_QT - 1) / IL_QT), (unsigned)cout, (unsigned)a.batch);
        conv_interleave_tiled_kernel<T><<<ig, 256, il_smem, st>>>(dst, d, bias, cout, a.out_length, a.stride, a.padding, p.nq);
    } else {
        conv_interleave_kernel<T><<<grid, 256, 0, st>>>(dst, d, bias, cout, a.out_length, a.stride, a.padding, p.nq, total);
    }
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

constexpr size_t C_SMEM_CAP = 200 * 1024;

template <typename T, bool TR>
int launch_conv(xn_dtype dt, T *dst, const T *src, const T *kernel, const T *bias, ConvArgs a, void *ws, size_t ws_bytes,
                cudaStream_t st) {
    const size_t total = (size_t)a.batch * a.cout_g * a.groups * a.out_length;
    if (total == 0) return XN_OK;
    {
        const ConvPlan p = conv_plan<TR>(dt, a);
        if (p.gemm) {
            const size_t need = p.xt_bytes + p.wp_bytes + p.d_bytes + p.part_bytes;
            if (!ws || ws_bytes < need)
                return fail(XN_ERR_WORKSPACE, "conv: workspace of %zu bytes, %zu needed (ask the _workspace_bytes function)",
                            ws ? ws_bytes : (size_t)0, need);
            XN_REQUIRE(aligned(ws, 256) && aligned(src, 2) && aligned(dst, 2), "conv: workspace must be 256-byte aligned");
            return launch_conv_gemm<T, TR>(dt, dst, src, kernel, bias, a, p, static_cast<unsigned char *>(ws), st);
        }
    }
    if (TR) {
        a.taps = (a.ksize + a.stride - 1) / a.stride;
        a.rows = C_TN + a.taps - 1;
        a.ntile = (a.out_length - 1 + a.padding) / a.stride / C_TN + 1;
    } else {
        a.taps = a.ksize;
        a.rows = (C_TN - 1) * a.stride + (a.ksize - 1) * a.dilation + 1;
        a.ntile = (a.out_length + C_TN - 1) / C_TN;
    }
    const size_t smem = ((size_t)a.rows + (size_t)a.taps * C_TM) * C_PITCH;
    const size_t gy = (size_t)a.groups * ((a.cout_g + C_TM - 1) / C_TM), gz = (size_t)a.batch * (TR ? a.stride : 1);
    const char *force = getenv("XN_CONV_DIRECT");
    const bool direct = a.cin_g < 8 || smem > C_SMEM_CAP || gy > 65535 || gz > 65535 || (force && atoi(force));
    if (direct) {
        const size_t blocks = (total + 255) / 256;
        const unsigned grid = (unsigned)(blocks < (size_t)sm_count() * 16 ? blocks : (size_t)sm_count() * 16);
        conv_direct_kernel<T, TR><<<grid, 256, 0, st>>>(dst, src, kernel, bias, a, total);
    } else {
        constexpr int CK = C_ROW / (int)sizeof(T);
        a.wvec = !TR && a.cin_g % CK == 0 && ((size_t)a.cin_g * a.ksize * sizeof(T)) % 16 == 0 && aligned(kernel, 16);
        XN_ENSURE_SMEM((conv_igemm_kernel<T, TR>), smem);
        dim3 grid((unsigned)a.ntile, (unsigned)gy, (unsigned)gz);
        conv_igemm_kernel<T, TR><<<grid, C_THREADS, smem, st>>>(dst, src, kernel, bias, a);
    }
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

int check_common(const void *dst, const void *src, const void *kernel, int dtype, size_t batch, size_t in_channels,
                 size_t out_channels, size_t length, size_t out_length, size_t kernel_size, size_t stride, size_t groups) {
    XN_REQUIRE(valid_dtype(dtype), "conv: dtype %d is not f32/f16/bf16", dtype);
    XN_REQUIRE(groups >= 1 && stride >= 1 && kernel_size >= 1, "conv: groups, stride and kernel_size must be at least 1");
    XN_REQUIRE(in_channels % groups == 0, "in_channels (%zu) must be divisible by groups (%zu)", in_channels, groups);
    XN_REQUIRE(out_channels % groups == 0, "out_channels (%zu) must be divisible by groups (%zu)", out_channels, groups);
    const size_t lim = (size_t)1 << 30;
    XN_REQUIRE(batch < lim && in_channels < lim && out_channels < lim && length < lim && out_length < lim &&
                   kernel_size < (1 << 16) && stride < (1 << 16),
               "conv: a dimension exceeds the 32-bit index range of the kernels");
    if (batch * out_channels * out_length == 0) return XN_OK;
    XN_REQUIRE(dst && src && kernel, "conv: null pointer");
    XN_REQUIRE(in_channels > 0 && length > 0, "conv: empty input for a non-empty output");
    return XN_OK;
}

}  // namespace
}  // namespace xn

using namespace xn;

extern "C" int xn_mm_conv1d(xn_dtype dtype, void *dst, const void *src, const void *kernel, const void *bias, size_t batch,
                            size_t in_channels, size_t out_channels, size_t length, size_t out_length, size_t kernel_size,
                            size_t stride, size_t padding, size_t dilation, size_t groups, void *workspace,
                            size_t workspace_bytes, void *stream) {
    XN_API_RANGE("xn_mm_conv1d");
    if (int rc = check_common(dst, src, kernel, dtype, batch, in_channels, out_channels, length, out_length, kernel_size,
                              stride, groups))
        return rc;
    if (batch * out_channels * out_length == 0) return XN_OK;
    XN_REQUIRE(dilation >= 1 && dilation < (1 << 16) && padding < ((size_t)1 << 30), "conv1d: dilation / padding out of range");
    const size_t span = dilation * (kernel_size - 1) + 1;
    XN_REQUIRE(length + 2 * padding >= span, "conv1d: kernel span %zu exceeds the padded length %zu", span, length + 2 * padding);
    const size_t expect = (length + 2 * padding - span) / stride + 1;
    XN_REQUIRE(out_length == expect, "conv1d: out_length %zu, expected %zu", out_length, expect);
    ConvArgs a{};
    a.batch = (int)batch, a.groups = (int)groups, a.cin_g = (int)(in_channels / groups), a.cout_g = (int)(out_channels / groups);
    a.length = (int)length, a.out_length = (int)out_length, a.ksize = (int)kernel_size;
    a.stride = (int)stride, a.padding = (int)padding, a.dilation = (int)dilation;
    cudaStream_t st = (cudaStream_t)stream;
    XN_DISPATCH_DTYPE(dtype, T, return (launch_conv<T, false>(dtype, (T *)dst, (const T *)src, (const T *)kernel, (const T *)bias, a,
                                                              workspace, workspace_bytes, st)));
    return XN_OK;
}

extern "C" int xn_mm_conv_transpose1d(xn_dtype dtype, void *dst, const void *src, const void *kernel, const void *bias,
                                      size_t batch, size_t in_channels, size_t out_channels, size_t length,
                                      size_t out_length, size_t kernel_size, size_t stride, size_t padding,
                                      size_t output_padding, size_t groups, void *workspace, size_t workspace_bytes,
                                      void *stream) {
    XN_API_RANGE("xn_mm_conv_transpose1d");
    if (int rc = check_common(dst, src, kernel, dtype, batch, in_channels, out_channels, length, out_length, kernel_size,
                              stride, groups))
        return rc;
    if (batch * out_channels * out_length == 0) return XN_OK;
    const size_t full = (length - 1) * stride + kernel_size + output_padding;
    XN_REQUIRE(padding < ((size_t)1 << 30) && full >= 2 * padding && out_length == full - 2 * padding,
               "conv_transpose1d: out_length %zu does not match (length-1)*stride + kernel_size + output_padding - 2*padding",
               out_length);
    ConvArgs a{};
    a.batch = (int)batch, a.groups = (int)groups, a.cin_g = (int)(in_channels / groups), a.cout_g = (int)(out_channels / groups);
    a.length = (int)length, a.out_length = (int)out_length, a.ksize = (int)kernel_size;
    a.stride = (int)stride, a.padding = (int)padding, a.dilation = 1;
    cudaStream_t st = (cudaStream_t)stream;
    XN_DISPATCH_DTYPE(dtype, T, return (launch_conv<T, true>(dtype, (T *)dst, (const T *)src, (const T *)kernel, (const T *)bias, a,
                                                             workspace, workspace_bytes, st)));
    return XN_OK;
}

// Bytes of device scratch the call with these arguments needs (0 when it runs the scratch-free kernels).
extern "C" size_t xn_mm_conv1d_workspace_bytes(xn_dtype dtype, size_t batch, size_t in_channels, size_t out_channels,
                                               size_t length, size_t kernel_size, size_t stride, size_t padding,
                                               size_t dilation, size_t groups) {
    if (!valid_dtype(dtype) || groups != 1 || stride < 1 || kernel_size < 1 || length + 2 * padding >= ((size_t)1 << 30)) return 0;
    ConvArgs a{};
    a.batch = (int)batch, a.groups = 1, a.cin_g = (int)in_channels, a.cout_g = (int)out_channels;
    a.length = (int)length, a.ksize = (int)kernel_size, a.stride = (int)stride, a.padding = (int)padding, a.dilation = (int)dilation;
    const size_t span = dilation * (kernel_size - 1) + 1;
    if (dilation < 1 || length + 2 * padding < span) return 0;
    a.out_length = (int)((length + 2 * padding - span) / stride + 1);
    const ConvPlan p = conv_plan<false>(dtype, a);
    return p.gemm ? p.xt_bytes + p.wp_bytes + p.d_bytes + p.part_bytes : 0;
}

extern "C" size_t xn_mm_conv_transpose1d_workspace_bytes(xn_dtype dtype, size_t batch, size_t in_channels,
                                                         size_t out_channels, size_t length, size_t kernel_size,
                                                         size_t stride, size_t padding, size_t output_padding,
                                                         size_t groups) {
    if (!valid_dtype(dtype) || groups != 1 || stride < 1 || kernel_size < 1 || length < 1) return 0;
    const size_t full = (length - 1) * stride + kernel_size + output_padding;
    if (full <= 2 * padding || full >= ((size_t)1 << 30)) return 0;
    ConvArgs a{};
    a.batch = (int)batch, a.groups = 1, a.cin_g = (int)in_channels, a.cout_g = (int)out_channels;
    a.length = (int)length, a.out_length = (int)(full - 2 * padding), a.ksize = (int)kernel_size, a.stride = (int)stride;
    a.padding = (int)padding, a.dilation = 1;
    const ConvPlan p = conv_plan<true>(dtype, a);
    return p.gemm ? p.xt_bytes + p.wp_bytes + p.d_bytes + p.part_bytes : 0;
}
