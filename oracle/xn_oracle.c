/*
 * CPU oracle for the xn matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, what xn computes on its CPU backend for
 * `matmul` -> `Backend::gemm`, plus the quantized-operand arithmetic the
 * B200 engine adds.  It exists so the CUDA kernels can be checked against an
 * independent implementation on identical inputs.  Nothing in the shipped
 * library links, imports or calls it: only the tests, the smoke check and the
 * benchmark's CPU-baseline / reference legs do.
 *
 * Parity status
 *   - f32 / f16 / bf16 gemm: pinned by the reference's own known-answer tests
 *     (xn-core/tests/cuda_tests.rs:214-287, xn-core/tests/tensor_tests.rs:467-613,
 *     954-980), which tests/test_oracle_golden.py replays against this file.
 *     The reference's inner product lives in the un-vendored crate `gemm` 0.19.0
 *     (xn-core/Cargo.toml:13); its published contract, dst = lhs * rhs with
 *     arbitrary element strides, is what xo_gemm restates.
 *   - int4 / int8 block-quantized and fp8-e4m3 linears: PARITY UNPINNED.  The
 *     reference has no such code; the arithmetic below follows the operand
 *     specification of the benchmark configurations only.
 *
 * All strides, offsets and sizes are in ELEMENTS, as in the reference
 * (xn-core/src/backend.rs:135-148).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define XO_F32 0
#define XO_F16 1
#define XO_BF16 2

/* ------------------------------------------------------------------------- */
/* 16-bit float conversions: round-to-nearest-even, as crate `half` does      */
/* (xn-core/src/dtype.rs:92-131 go through f32 for every 16-bit element).     */
/* ------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float xo_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

uint16_t xo_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

float xo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: man * 2^-24 */
        float v = (float)man * (1.0f / 16777216.0f);
        return (sign ? -v : v);
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

uint16_t xo_f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a < 0x33000001u) return sign; /* < 2^-25 (or exactly 2^-25, ties to even 0) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    return (uint16_t)(sign | (base + q));
}

static inline float load_elem(int dtype, const void *p, size_t i) {
    switch (dtype) {
    case XO_F32: return ((const float *)p)[i];
    case XO_F16: return xo_f16_to_f32(((const uint16_t *)p)[i]);
    default: return xo_bf16_to_f32(((const uint16_t *)p)[i]);
    }
}

static inline void store_elem(int dtype, void *p, size_t i, float v) {
    switch (dtype) {
    case XO_F32: ((float *)p)[i] = v; break;
    case XO_F16: ((uint16_t *)p)[i] = xo_f32_to_f16(v); break;
    default: ((uint16_t *)p)[i] = xo_f32_to_bf16(v); break;
    }
}

/* ------------------------------------------------------------------------- */
/* gemm: xn-core/src/cpu_backend.rs:48-93 (`gemm_`).  For every batch b the   */
/* reference slices dst at b*m*n, lhs at lhs_off + b*lhs_b_stride, rhs at     */
/* rhs_off + b*rhs_b_stride and computes dst = lhs * rhs (alpha = 0 on the    */
/* old dst, i.e. dst is overwritten; xn-core/src/cpu_backend.rs:69-89).       */
/* accum == 0: f32 accumulation (what the reference's element type gives for  */
/* f32; 16-bit types are widened to f32 first).  accum == 1: f64 accumulation,*/
/* used to bound this oracle's own rounding noise.                            */
/* ------------------------------------------------------------------------- */
void xo_gemm(int dtype, void *dst, const void *lhs, size_t lhs_off, const void *rhs,
             size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
             size_t rhs_b_stride, size_t dst_cs, size_t dst_rs, size_t lhs_cs, size_t lhs_rs,
             size_t rhs_cs, size_t rhs_rs, int accum) {
    for (size_t b = 0; b < lhs_b; ++b) {
        size_t d0 = b * m * n;
        size_t l0 = lhs_off + b * lhs_b_stride;
        size_t r0 = rhs_off + b * rhs_b_stride;
#pragma omp parallel for schedule(static) if (m * n * k > (1u << 20))
        for (long long ij = 0; ij < (long long)(m * n); ++ij) {
            size_t i = (size_t)ij / n, j = (size_t)ij % n;
            if (accum == 0) {
                float acc = 0.0f;
                for (size_t p = 0; p < k; ++p)
                    acc += load_elem(dtype, lhs, l0 + i * lhs_rs + p * lhs_cs) *
                           load_elem(dtype, rhs, r0 + p * rhs_rs + j * rhs_cs);
                store_elem(dtype, dst, d0 + i * dst_rs + j * dst_cs, acc);
            } else {
                double acc = 0.0;
                for (size_t p = 0; p < k; ++p)
                    acc += (double)load_elem(dtype, lhs, l0 + i * lhs_rs + p * lhs_cs) *
                           (double)load_elem(dtype, rhs, r0 + p * rhs_rs + j * rhs_cs);
                store_elem(dtype, dst, d0 + i * dst_rs + j * dst_cs, (float)acc);
            }
        }
    }
}

/* f64-accumulated result kept in f64 (no final rounding), contiguous [lhs_b,m,n]. */
void xo_gemm_f64out(int dtype, double *dst, const void *lhs, size_t lhs_off, const void *rhs,
                    size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b,
                    size_t lhs_b_stride, size_t rhs_b_stride, size_t lhs_cs, size_t lhs_rs,
                    size_t rhs_cs, size_t rhs_rs) {
    for (size_t b = 0; b < lhs_b; ++b) {
        size_t l0 = lhs_off + b * lhs_b_stride, r0 = rhs_off + b * rhs_b_stride;
#pragma omp parallel for schedule(static) if (m * n * k > (1u << 20))
        for (long long ij = 0; ij < (long long)(m * n); ++ij) {
            size_t i = (size_t)ij / n, j = (size_t)ij % n;
            double acc = 0.0;
            for (size_t p = 0; p < k; ++p)
                acc += (double)load_elem(dtype, lhs, l0 + i * lhs_rs + p * lhs_cs) *
                       (double)load_elem(dtype, rhs, r0 + p * rhs_rs + j * rhs_cs);
            dst[b * m * n + i * n + j] = acc;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* matmul front-end: xn-core/src/ops.rs:640-700 (shape rules) and             */
/* xn-core/src/inplace_ops.rs:318-436 (strides -> the gemm arguments,         */
/* including the batch-flattening branch at :414-419).                        */
/* out[0..11] = m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_cs, dst_rs,   */
/*              lhs_cs, lhs_rs, rhs_cs, rhs_rs.                               */
/* Returns 0, or 1 rank<2, 2 inner-dim mismatch, 3 batch mismatch.            */
/* ------------------------------------------------------------------------- */
int xo_matmul_plan(size_t lhs_rank, const size_t *lhs_dims, const size_t *lhs_strides,
                   size_t rhs_rank, const size_t *rhs_dims, const size_t *rhs_strides, int rhs_t,
                   size_t *out) {
    if (lhs_rank < 2 || rhs_rank < 2) return 1;
    size_t lhs_m = lhs_dims[lhs_rank - 2], lhs_k = lhs_dims[lhs_rank - 1];
    size_t rhs_k = rhs_t ? rhs_dims[rhs_rank - 1] : rhs_dims[rhs_rank - 2];
    size_t rhs_n = rhs_t ? rhs_dims[rhs_rank - 2] : rhs_dims[rhs_rank - 1];
    if (lhs_k != rhs_k) return 2;
    /* ops.rs:682: rhs batch dims must be empty or equal to the lhs batch dims */
    if (rhs_rank > 2) {
        if (rhs_rank != lhs_rank) return 3;
        for (size_t i = 0; i + 2 < rhs_rank; ++i)
            if (rhs_dims[i] != lhs_dims[i]) return 3;
    }
    size_t lhs_batch = 1, rhs_batch = 1;
    for (size_t i = 0; i + 2 < lhs_rank; ++i) lhs_batch *= lhs_dims[i];
    for (size_t i = 0; i + 2 < rhs_rank; ++i) rhs_batch *= rhs_dims[i];
    if (lhs_batch < 1) lhs_batch = 1;
    if (rhs_batch < 1) rhs_batch = 1;
    if (rhs_batch != 1 && rhs_batch != lhs_batch) return 3;
    size_t m = lhs_m, n = rhs_n, k = lhs_k;
    size_t lhs_cs = lhs_strides[lhs_rank - 1], lhs_rs = lhs_strides[lhs_rank - 2];
    size_t rhs_cs, rhs_rs;
    if (rhs_t) { rhs_cs = rhs_strides[rhs_rank - 2]; rhs_rs = rhs_strides[rhs_rank - 1]; }
    else { rhs_cs = rhs_strides[rhs_rank - 1]; rhs_rs = rhs_strides[rhs_rank - 2]; }
    size_t lhs_b_stride = lhs_rank >= 3 ? lhs_strides[lhs_rank - 3] : m * k;
    size_t rhs_b_stride;
    if (rhs_batch == 1) rhs_b_stride = 0;
    else if (rhs_rank >= 3) rhs_b_stride = rhs_strides[rhs_rank - 3];
    else rhs_b_stride = rhs_dims[rhs_rank - 2] * rhs_dims[rhs_rank - 1];
    size_t lhs_b = lhs_batch;
    if (lhs_b_stride == m * lhs_rs && rhs_batch == 1) {
        lhs_b = 1; rhs_b_stride = 1; m = lhs_batch * lhs_m;
    }
    out[0] = m; out[1] = n; out[2] = k; out[3] = lhs_b; out[4] = lhs_b_stride;
    out[5] = rhs_b_stride; out[6] = 1; out[7] = n; out[8] = lhs_cs; out[9] = lhs_rs;
    out[10] = rhs_cs; out[11] = rhs_rs;
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Block-quantized integer weights (no counterpart in the reference).         */
/* W [n,k] f32, k split in `block`-element groups, one f32 scale per group:   */
/*   scale = max|w| / qmax   (qmax = 7 for int4, 127 for int8)                */
/*   q     = clamp(round_half_even(w / scale), -qmax, qmax); scale 0 -> q = 0 */
/* q is returned one value per int8 (logical form).                           */
/* ------------------------------------------------------------------------- */
void xo_quantize_blocks(const float *w, size_t n, size_t k, size_t block, int qmax, int8_t *q,
                        float *scales) {
    size_t nblk = k / block;
    for (size_t r = 0; r < n; ++r)
        for (size_t b = 0; b < nblk; ++b) {
            const float *src = w + r * k + b * block;
            float amax = 0.0f;
            for (size_t i = 0; i < block; ++i) amax = fmaxf(amax, fabsf(src[i]));
            float scale = amax / (float)qmax;
            scales[r * nblk + b] = scale;
            for (size_t i = 0; i < block; ++i) {
                float v = 0.0f;
                if (scale != 0.0f) v = nearbyintf(src[i] / scale);
                if (v > (float)qmax) v = (float)qmax;
                if (v < -(float)qmax) v = -(float)qmax;
                q[r * k + b * block + i] = (int8_t)v;
            }
        }
}

/* Dynamic per-row int8 activation quantization: scale = max|x|/127. */
void xo_quantize_rows_i8(const float *x, size_t m, size_t k, int8_t *q, float *scale) {
    xo_quantize_blocks(x, m, k, k, 127, q, scale);
}

/* Physical int4 layout used by the engine ("q4 tiles", documented in include/xn_mm.h):
 * rows padded to a multiple of 16, k a multiple of 128.  Tile (r/16, kk/128) = 1280 bytes.
 * Bytes 0..1023 = 64 chunks of 16 bytes; chunk 32*h + 4*g + t belongs to row 16*(r/16) + 8*h + g
 * and holds four u32 words, word j for 32-block j of the 128-k group.  In word j, byte i carries
 * element 4*t+i (low nibble) and element 16+4*t+i (high nibble) of that block, each as 4-bit
 * two's complement.  Bytes 1024..1279 = 64 f32 scales; entry (4*g + j)*2 + h is the scale of row
 * 8*h + g, block j.  `packed` must hold ceil(n/16)*(k/128)*1280 bytes and is fully written. */
static size_t q4_pos(size_t r, size_t kk, size_t k, int *hi) {
    size_t tile = (r / 16) * (k / 128) + kk / 128;
    size_t rr = r % 16, h = rr / 8, g = rr % 8, j = (kk % 128) / 32, e = kk % 32;
    size_t t = (e % 16) / 4, i = e % 4;
    *hi = (int)(e / 16);
    return tile * 1280 + (32 * h + 4 * g + t) * 16 + j * 4 + i;
}
static size_t q4_scale_pos(size_t r, size_t blk, size_t k) {
    size_t tile = (r / 16) * (k / 128) + blk / 4;
    return tile * 1280 + 1024 + 4 * ((4 * (r % 8) + blk % 4) * 2 + (r % 16) / 8);
}

void xo_pack_q4(const int8_t *q, const float *scales, size_t n, size_t k, uint8_t *packed) {
    memset(packed, 0, ((n + 15) / 16) * (k / 128) * 1280);
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) {
            int hi;
            size_t byte = q4_pos(r, kk, k, &hi);
            uint8_t nib = (uint8_t)q[r * k + kk] & 0xF;
            packed[byte] |= hi ? (uint8_t)(nib << 4) : nib;
        }
        for (size_t b = 0; b < k / 32; ++b) memcpy(packed + q4_scale_pos(r, b, k), &scales[r * (k / 32) + b], 4);
    }
}

void xo_unpack_q4(const uint8_t *packed, size_t n, size_t k, int8_t *q, float *scales) {
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) {
            int hi;
            uint8_t b = packed[q4_pos(r, kk, k, &hi)];
            int v = hi ? (b >> 4) : (b & 0xF);
            if (v >= 8) v -= 16;
            q[r * k + kk] = (int8_t)v;
        }
        for (size_t b = 0; b < k / 32; ++b) memcpy(&scales[r * (k / 32) + b], packed + q4_scale_pos(r, b, k), 4);
    }
}

/* int8 block tiles ("q8 tiles"): tile (r/16, kk/128) = 2304 bytes; for 32-block j and lane 4*g + t the 16
 * bytes at j*512 + (4*g+t)*16 are the words {row g, k 4t..}, {row g+8, k 4t..}, {row g, k 16+4t..},
 * {row g+8, k 16+4t..}; scales at +2048 as in the q4 tiles. */
static size_t q8_pos(size_t r, size_t kk, size_t k) {
    size_t tile = (r / 16) * (k / 128) + kk / 128;
    size_t rr = r % 16, h = rr / 8, g = rr % 8, j = (kk % 128) / 32, e = kk % 32;
    size_t t = (e % 16) / 4, i = e % 4, hi = e / 16;
    return tile * 2304 + j * 512 + (4 * g + t) * 16 + (h + 2 * hi) * 4 + i;
}
void xo_pack_q8(const int8_t *q, const float *scales, size_t n, size_t k, uint8_t *packed) {
    memset(packed, 0, ((n + 15) / 16) * (k / 128) * 2304);
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) packed[q8_pos(r, kk, k)] = (uint8_t)q[r * k + kk];
        for (size_t b = 0; b < k / 32; ++b) {
            size_t tile = (r / 16) * (k / 128) + b / 4;
            memcpy(packed + tile * 2304 + 2048 + 4 * ((4 * (r % 8) + b % 4) * 2 + (r % 16) / 8), &scales[r * (k / 32) + b], 4);
        }
    }
}

/* Quantized linear: P[i,j,blk] = sum over the block of xq*wq as int32,
 * y[i,j] = x_scale[i] * sum_blk (float)P * w_scale[j,blk]  (f32, blocks in order).
 * partials may be NULL. wq is the logical (one value per int8) form. */
/* The 32-element block (the only block size the engine uses) gets its own loop with a constant trip count so
 * that the compiler turns the int8 x int8 -> int32 dot product into SIMD widening multiplies; the function is
 * cloned per instruction set and dispatched at load time, so one binary runs at full width on whatever host
 * it lands on (this is also the timed CPU baseline of the int4 configuration). */
__attribute__((target_clones("arch=skylake-avx512", "avx2", "default")))
void xo_linear_q(const int8_t *xq, const float *x_scale, const int8_t *wq, const float *w_scale,
                 size_t m, size_t n, size_t k, size_t block, int32_t *partials, float *y) {
    size_t nblk = k / block;
#pragma omp parallel for schedule(static)
    for (long long jj = 0; jj < (long long)n; ++jj) {
        size_t j = (size_t)jj;
        for (size_t i = 0; i < m; ++i) {
            float acc = 0.0f;
            for (size_t b = 0; b < nblk; ++b) {
                int32_t p = 0;
                const int8_t *xa = xq + i * k + b * block, *wa = wq + j * k + b * block;
                if (block == 32) {
                    for (int e = 0; e < 32; ++e) p += (int32_t)xa[e] * (int32_t)wa[e];
                } else {
                    for (size_t e = 0; e < block; ++e) p += (int32_t)xa[e] * (int32_t)wa[e];
                }
                if (partials) partials[(i * n + j) * nblk + b] = p;
                acc += (float)p * w_scale[j * nblk + b];
            }
            y[i * n + j] = x_scale[i] * acc;
        }
    }
}

/* Timed CPU baseline of the int4 configuration: the same linear as xo_linear_q, y only, written for the host's
 * widest integer dot product (AVX-512 VNNI: vpdpbusd, u8 x s8 -> s32 over 64 bytes).  The activations are
 * offset to unsigned (x + 128) and the surplus 128 * sum(w) is taken out per output channel; every 64-byte step
 * of a weight row is loaded once and multiplied with all activation rows; the int32 lanes are scaled and
 * accumulated as floats without a per-block horizontal sum.  The integer arithmetic is exact, the float sum
 * runs in another order than the definition (xo_linear_q), against which tests check it to 1e-5.  Hosts without
 * VNNI run xo_linear_q. */
#if defined(__x86_64__)
#include <immintrin.h>
#define XO_VNNI __attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni")))
/* one weight row against MI activation rows (MI a compile-time constant so the accumulators stay in registers) */
XO_VNNI static inline __attribute__((always_inline)) void q32_row_vnni(const uint8_t *xu, const float *x_scale,
                                                                       const int8_t *wr, const float *sr, size_t k,
                                                                       size_t n, size_t j, float *y, const int MI) {
    const __m512i lane_blk = _mm512_set_epi32(1, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0, 0);
    const __m512i off = _mm512_set1_epi8((char)0x80);
    __m512 acc[16];
    for (int i = 0; i < MI; ++i) acc[i] = _mm512_setzero_ps();
    for (size_t c = 0; c < k / 64; ++c) {
        const __m512i wv = _mm512_loadu_si512((const void *)(wr + c * 64));
        /* the activations are offset by +128 to fit the unsigned operand: take 128 * w back out per lane */
        const __m512i corr = _mm512_dpbusd_epi32(_mm512_setzero_si512(), off, wv);
        const __m512 pair = _mm512_castpd_ps(_mm512_set1_pd(*(const double *)(const void *)(sr + 2 * c)));
        const __m512 sc = _mm512_permutexvar_ps(lane_blk, pair);
        for (int i = 0; i < MI; ++i) {
            const __m512i xv = _mm512_loadu_si512((const void *)(xu + (size_t)i * k + c * 64));
            const __m512i dp = _mm512_sub_epi32(_mm512_dpbusd_epi32(_mm512_setzero_si512(), xv, wv), corr);
            acc[i] = _mm512_fmadd_ps(_mm512_cvtepi32_ps(dp), sc, acc[i]);
        }
    }
    for (int i = 0; i < MI; ++i) y[(size_t)i * n + j] = x_scale[i] * _mm512_reduce_add_ps(acc[i]);
}

XO_VNNI static void linear_q32_vnni(const int8_t *xq, const float *x_scale, const int8_t *wq, const float *w_scale,
                                    size_t m, size_t n, size_t k, float *y) {
    const size_t nblk = k / 32;
    uint8_t *xu = (uint8_t *)malloc(m * k);
    for (size_t i = 0; i < m * k; ++i) xu[i] = (uint8_t)((int)xq[i] + 128);
#pragma omp parallel for schedule(static)
    for (long long jj = 0; jj < (long long)n; ++jj) {
        const size_t j = (size_t)jj;
        const int8_t *wr = wq + j * k;
        const float *sr = w_scale + j * nblk;
        size_t i0 = 0;
        for (; i0 + 16 <= m; i0 += 16) q32_row_vnni(xu + i0 * k, x_scale + i0, wr, sr, k, n, j, y + i0 * n, 16);
        for (; i0 + 4 <= m; i0 += 4) q32_row_vnni(xu + i0 * k, x_scale + i0, wr, sr, k, n, j, y + i0 * n, 4);
        for (; i0 < m; ++i0) q32_row_vnni(xu + i0 * k, x_scale + i0, wr, sr, k, n, j, y + i0 * n, 1);
    }
    free(xu);
}
#endif

void xo_linear_q_fast(const int8_t *xq, const float *x_scale, const int8_t *wq, const float *w_scale,
                      size_t m, size_t n, size_t k, size_t block, float *y) {
#if defined(__x86_64__)
    if (block == 32 && k % 64 == 0 && __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bw")) {
        linear_q32_vnni(xq, x_scale, wq, w_scale, m, n, k, y);
        return;
    }
#endif
    xo_linear_q(xq, x_scale, wq, w_scale, m, n, k, block, NULL, y);
}

int xo_linear_q_fast_is_vnni(void) {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bw");
#else
    return 0;
#endif
}

/* ------------------------------------------------------------------------- */
/* fp8 e4m3 (OCP "e4m3fn": bias 7, max 448, no infinity, NaN = 0x7f/0xff).    */
/* Encode: round to nearest even, saturate finite values to +-448, NaN -> 0x7f */
/* with sign; the device twin is __nv_cvt_float_to_fp8(.., __NV_SATFINITE,    */
/* __NV_E4M3).                                                                */
/* ------------------------------------------------------------------------- */
float xo_e4m3_to_f32(uint8_t b) {
    int s = b >> 7, e = (b >> 3) & 0xF, mnt = b & 7;
    float v;
    if (e == 0) v = ldexpf((float)mnt, -9);
    else if (e == 15 && mnt == 7) v = NAN;
    else v = ldexpf((float)(8 + mnt), e - 10);
    return s ? -v : v;
}

uint8_t xo_f32_to_e4m3(float f) {
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7f);
    float af = bits_f32(a);
    if (af >= 448.0f) return (uint8_t)(sign | 0x7e); /* also covers values that would round above 448: saturate */
    /* scale so that the e4m3 grid becomes the integers, round to nearest even */
    int e;
    (void)frexpf(af, &e); /* af = f * 2^e, f in [0.5,1) -> exponent of leading bit is e-1 */
    int lead = e - 1;
    if (af == 0.0f) return sign;
    if (lead < -6) lead = -6; /* subnormal grid: spacing 2^-9 */
    /* spacing = 2^(lead-3) */
    float q = nearbyintf(ldexpf(af, 3 - lead)); /* in [0,16] */
    int qi = (int)q;
    if (qi == 16) { qi = 8; lead += 1; }
    if (lead > 8 || (lead == 8 && qi > 14)) return (uint8_t)(sign | 0x7e);
    if (qi < 8) return (uint8_t)(sign | qi); /* subnormal (lead == -6) or zero */
    return (uint8_t)(sign | ((lead + 7) << 3) | (qi - 8));
}

void xo_f32_to_e4m3_vec(const float *x, size_t len, uint8_t *out) {
    for (size_t i = 0; i < len; ++i) out[i] = xo_f32_to_e4m3(x[i]);
}

/* Per-output-channel fp8 weights: scale[n] = max_k|w| / 448, q = e4m3(w / scale). */
void xo_quantize_fp8_channel(const float *w, size_t n, size_t k, uint8_t *q, float *scale) {
    for (size_t r = 0; r < n; ++r) {
        float amax = 0.0f;
        for (size_t i = 0; i < k; ++i) amax = fmaxf(amax, fabsf(w[r * k + i]));
        float s = amax / 448.0f;
        scale[r] = s;
        for (size_t i = 0; i < k; ++i)
            q[r * k + i] = (s != 0.0f) ? xo_f32_to_e4m3(w[r * k + i] / s) : 0;
    }
}

/* Row scale used when activations are turned into e4m3 pieces: the power of two
 * s with max|x| / s in (224, 448] (s = 1 for an all-zero row). */
float xo_pow2_row_scale(const float *x, size_t k) {
    float amax = 0.0f;
    for (size_t i = 0; i < k; ++i) amax = fmaxf(amax, fabsf(x[i]));
    if (amax == 0.0f || !isfinite(amax)) return 1.0f;
    int e;
    float f = frexpf(amax, &e);
    return ldexpf(1.0f, f <= 0.875f ? e - 9 : e - 8);
}

/* x [m,k] (f32 values; callers widen bf16 first) -> hi = e4m3(x/s), lo = e4m3(x/s - hi). */
void xo_split_rows_e4m3(const float *x, size_t m, size_t k, uint8_t *hi, uint8_t *lo,
                        float *scale) {
    for (size_t i = 0; i < m; ++i) {
        float s = xo_pow2_row_scale(x + i * k, k);
        scale[i] = s;
        for (size_t p = 0; p < k; ++p) {
            float v = x[i * k + p] / s;
            uint8_t h = xo_f32_to_e4m3(v);
            float r = v - xo_e4m3_to_f32(h);
            hi[i * k + p] = h;
            lo[i * k + p] = xo_f32_to_e4m3(r);
        }
    }
}

/* fp8 linear: y[i,j] = bf16( w_scale[j] * sum_p x[i,p] * e4m3(wq[j,p]) ), f32 accumulate.
 * variant 0 ("W8A16"): x is the bf16 activation itself.
 * variant 1 ("W8A8"):  x is replaced by s_i * e4m3(x / s_i) with the power-of-two row scale.
 * y_f32 (optional) receives the unrounded f32 value. */
void xo_linear_fp8(const uint16_t *x_bf16, const uint8_t *wq, const float *w_scale, size_t m,
                   size_t n, size_t k, int variant, uint16_t *y_bf16, float *y_f32) {
    float *xf = (float *)malloc(sizeof(float) * m * k);
    float *wf = (float *)malloc(sizeof(float) * n * k);
    for (size_t i = 0; i < m * k; ++i) xf[i] = xo_bf16_to_f32(x_bf16[i]);
    for (size_t i = 0; i < n * k; ++i) wf[i] = xo_e4m3_to_f32(wq[i]);
    if (variant == 1)
        for (size_t i = 0; i < m; ++i) {
            float s = xo_pow2_row_scale(xf + i * k, k);
            for (size_t p = 0; p < k; ++p)
                xf[i * k + p] = s * xo_e4m3_to_f32(xo_f32_to_e4m3(xf[i * k + p] / s));
        }
#pragma omp parallel for schedule(static)
    for (long long jj = 0; jj < (long long)n; ++jj) {
        size_t j = (size_t)jj;
        for (size_t i = 0; i < m; ++i) {
            double acc = 0.0; /* f64 here: the true value, so kernels are judged against truth */
            for (size_t p = 0; p < k; ++p) acc += (double)xf[i * k + p] * (double)wf[j * k + p];
            float v = w_scale[j] * (float)acc;
            if (y_f32) y_f32[i * n + j] = v;
            if (y_bf16) y_bf16[i * n + j] = xo_f32_to_bf16(v);
        }
    }
    free(xf);
    free(wf);
}

/* ------------------------------------------------------------------------- */
/* Row ops a decoder step needs around its matmuls (f32 math, as the CPU      */
/* backend does after widening): rms_norm xn-core/src/cpu_backend.rs:766-784, */
/* softmax :742-764, silu :216-218.                                           */
/* ------------------------------------------------------------------------- */
void xo_rms_norm(int dtype, void *dst, const void *src, const void *alpha, size_t rows,
                 size_t cols, float eps) {
    for (size_t r = 0; r < rows; ++r) {
        float sum2 = 0.0f;
        for (size_t c = 0; c < cols; ++c) {
            float v = load_elem(dtype, src, r * cols + c);
            sum2 += v * v;
        }
        float mden = sqrtf(sum2 / (float)cols + eps);
        for (size_t c = 0; c < cols; ++c)
            store_elem(dtype, dst, r * cols + c,
                       load_elem(dtype, src, r * cols + c) / mden * load_elem(dtype, alpha, c));
    }
}

void xo_softmax(int dtype, void *dst, const void *src, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r) {
        float mx = -INFINITY;
        for (size_t c = 0; c < cols; ++c) mx = fmaxf(mx, load_elem(dtype, src, r * cols + c));
        float sum = 0.0f;
        for (size_t c = 0; c < cols; ++c) {
            /* `*d = (*s - max).exp()` on the element type (xn-core/src/cpu_backend.rs:756): the difference
             * is rounded to the element type, then the exponential is, before the f32 sum */
            store_elem(dtype, dst, r * cols + c, load_elem(dtype, src, r * cols + c) - mx);
            store_elem(dtype, dst, r * cols + c, expf(load_elem(dtype, dst, r * cols + c)));
            sum += load_elem(dtype, dst, r * cols + c);
        }
        for (size_t c = 0; c < cols; ++c)
            store_elem(dtype, dst, r * cols + c, load_elem(dtype, dst, r * cols + c) / sum);
    }
}

/* gated activation of the FFN: out[r,c] = silu(a[r,c]) * b[r,c] where a = first `hidden`
 * channels of src row, b = the second `hidden` (xn-moshi/src/transformer.rs:239-245). */
void xo_silu_mul(int dtype, void *dst, const void *src, size_t rows, size_t hidden) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < hidden; ++c) {
            float a = load_elem(dtype, src, r * 2 * hidden + c);
            float b = load_elem(dtype, src, r * 2 * hidden + hidden + c);
            /* the reference rounds silu(a) to the element type before the multiply */
            float s = a / (1.0f + expf(-a));
            if (dtype != XO_F32) { uint16_t t; store_elem(dtype, &t, 0, s); s = load_elem(dtype, &t, 0); }
            store_elem(dtype, dst, r * hidden + c, s * b);
        }
}

/* ------------------------------------------------------------------------- */
/* Timed CPU baseline: the same f32 x * W^T product as xo_gemm for the        */
/* `matmul_t` form (lhs [m,k] row-major, rhs [n,k] row-major), written so the */
/* compiler can vectorise it, threaded over n with OpenMP -- the stand-in for */
/* crate gemm + rayon (xn-core/src/cpu_backend.rs:88, 1519-1526).             */
/* ------------------------------------------------------------------------- */
#if defined(__x86_64__)
/* AVX-512 form: one 16-float piece of a weight row is loaded once and multiplied into MI register accumulators. */
__attribute__((target("avx512f"))) static inline __attribute__((always_inline)) void f32_row_avx512(
    const float *x, const float *wr, float *y, size_t n, size_t k, size_t j, const int MI) {
    __m512 acc[16];
    for (int i = 0; i < MI; ++i) acc[i] = _mm512_setzero_ps();
    size_t p = 0;
    for (; p + 16 <= k; p += 16) {
        const __m512 wv = _mm512_loadu_ps(wr + p);
        for (int i = 0; i < MI; ++i) acc[i] = _mm512_fmadd_ps(_mm512_loadu_ps(x + (size_t)i * k + p), wv, acc[i]);
    }
    for (int i = 0; i < MI; ++i) {
        float s = _mm512_reduce_add_ps(acc[i]);
        for (size_t q = p; q < k; ++q) s += x[(size_t)i * k + q] * wr[q];
        y[(size_t)i * n + j] = s;
    }
}
__attribute__((target("avx512f"))) static void linear_f32_avx512(const float *x, const float *w, float *y, size_t m,
                                                                 size_t n, size_t k) {
#pragma omp parallel for schedule(static)
    for (long long jj = 0; jj < (long long)n; ++jj) {
        const float *wr = w + (size_t)jj * k;
        size_t i0 = 0;
        for (; i0 + 16 <= m; i0 += 16) f32_row_avx512(x + i0 * k, wr, y + i0 * n, n, k, (size_t)jj, 16);
        for (; i0 + 4 <= m; i0 += 4) f32_row_avx512(x + i0 * k, wr, y + i0 * n, n, k, (size_t)jj, 4);
        for (; i0 < m; ++i0) f32_row_avx512(x + i0 * k, wr, y + i0 * n, n, k, (size_t)jj, 1);
    }
}
#endif

static void linear_f32_portable(const float *x, const float *w, float *y, size_t m, size_t n, size_t k);
void xo_linear_f32_fast(const float *x, const float *w, float *y, size_t m, size_t n, size_t k) {
#if defined(__x86_64__)
    if (__builtin_cpu_supports("avx512f")) {
        linear_f32_avx512(x, w, y, m, n, k);
        return;
    }
#endif
    linear_f32_portable(x, w, y, m, n, k);
}

__attribute__((target_clones("avx2,fma", "default")))
static void linear_f32_portable(const float *x, const float *w, float *y, size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
    for (long long jj = 0; jj < (long long)n; ++jj) {
        const float *wr = w + (size_t)jj * k;
        size_t i0 = 0;
        /* eight activation rows per pass over the weight row: each 16-float piece of the row is loaded once
         * and multiplied into eight vector accumulators */
        for (; i0 + 8 <= m; i0 += 8) {
            float acc[8][16] = {{0}};
            size_t p = 0;
            for (; p + 16 <= k; p += 16)
                for (int i = 0; i < 8; ++i)
                    for (int l = 0; l < 16; ++l) acc[i][l] += x[(i0 + i) * k + p + l] * wr[p + l];
            for (int i = 0; i < 8; ++i) {
                float s = 0.0f;
                for (int l = 0; l < 16; ++l) s += acc[i][l];
                for (size_t q = p; q < k; ++q) s += x[(i0 + i) * k + q] * wr[q];
                y[(i0 + i) * n + (size_t)jj] = s;
            }
        }
        for (size_t i = i0; i < m; ++i) {
            const float *xr = x + i * k;
            float acc[16] = {0};
            size_t p = 0;
            for (; p + 16 <= k; p += 16)
                for (int l = 0; l < 16; ++l) acc[l] += xr[p + l] * wr[p + l];
            float s = 0.0f;
            for (int l = 0; l < 16; ++l) s += acc[l];
            for (; p < k; ++p) s += xr[p] * wr[p];
            y[i * n + (size_t)jj] = s;
        }
    }
}

/* The launcher of multi-process runs pins OpenMP to one thread per process; the timed CPU legs set the
 * count back to the cores this process may run on. */
void xo_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int xo_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* Convolutions, as Backend::conv1d / conv_transpose1d of the CPU backend      */
/* run them (xn-core/src/cpu_backend.rs:959-1136): groups == 1 goes through    */
/* im2col + gemm + transpose (:959-1030), respectively transpose + gemm +      */
/* col2im when padding and output_padding are 0 (:1072-1115, col2im :1319-     */
/* 1350); everything else takes the direct loops (:1233-1310, :1354-1430),     */
/* which accumulate in the ELEMENT type: every product and every sum is        */
/* rounded to f16 / bf16 there.                                                */
/* ------------------------------------------------------------------------- */
static inline float round_elem(int dtype, float v) {
    if (dtype == XO_F32) return v;
    uint16_t t;
    store_elem(dtype, &t, 0, v);
    return load_elem(dtype, &t, 0);
}
static inline size_t elem_size(int dtype) { return dtype == XO_F32 ? 4 : 2; }

void xo_conv1d(int dtype, void *dst, const void *src, const void *kernel, size_t batch,
               size_t in_channels, size_t out_channels, size_t length, size_t out_length,
               size_t kernel_size, size_t stride, size_t padding, size_t dilation, size_t groups) {
    size_t es = elem_size(dtype);
    if (groups == 1) {
        size_t k = in_channels * kernel_size;
        void *col = calloc(batch * out_length * k + 1, es);
        void *res = calloc(batch * out_length * out_channels + 1, es);
        for (size_t b = 0; b < batch; ++b)
            for (size_t l = 0; l < out_length; ++l)
                for (size_t c = 0; c < in_channels; ++c)
                    for (size_t kk = 0; kk < kernel_size; ++kk) {
                        size_t sl = l * stride + kk * dilation;
                        if (sl < padding || sl >= length + padding) continue;
                        store_elem(dtype, col, (b * out_length + l) * k + c * kernel_size + kk,
                                   load_elem(dtype, src, (b * in_channels + c) * length + sl - padding));
                    }
        xo_gemm(dtype, res, col, 0, kernel, 0, out_length, out_channels, k, batch, out_length * k, 0,
                1, out_channels, 1, k, k, 1, 0);
        for (size_t b = 0; b < batch; ++b)
            for (size_t l = 0; l < out_length; ++l)
                for (size_t c = 0; c < out_channels; ++c)
                    store_elem(dtype, dst, (b * out_channels + c) * out_length + l,
                               load_elem(dtype, res, (b * out_length + l) * out_channels + c));
        free(col);
        free(res);
        return;
    }
    size_t cig = in_channels / groups, cog = out_channels / groups;
    for (size_t i = 0; i < batch * out_channels * out_length; ++i) store_elem(dtype, dst, i, 0.0f);
    for (size_t kk = 0; kk < kernel_size; ++kk)
        for (size_t oc = 0; oc < out_channels; ++oc) {
            size_t c0 = (oc / cog) * cig;
            for (size_t b = 0; b < batch; ++b)
                for (size_t ol = 0; ol < out_length; ++ol) {
                    size_t sl = ol * stride + kk * dilation;
                    if (sl < padding || sl >= padding + length) continue;
                    sl -= padding;
                    float d = 0.0f;
                    for (size_t ic = 0; ic < cig; ++ic) {
                        float p = round_elem(dtype, load_elem(dtype, src, (b * in_channels + c0 + ic) * length + sl) *
                                                        load_elem(dtype, kernel, (oc * cig + ic) * kernel_size + kk));
                        d = round_elem(dtype, d + p);
                    }
                    size_t di = (b * out_channels + oc) * out_length + ol;
                    store_elem(dtype, dst, di, load_elem(dtype, dst, di) + d);
                }
        }
}

void xo_conv_transpose1d(int dtype, void *dst, const void *src, const void *kernel, size_t batch,
                         size_t in_channels, size_t out_channels, size_t length, size_t out_length,
                         size_t kernel_size, size_t stride, size_t padding, size_t output_padding,
                         size_t groups) {
    size_t es = elem_size(dtype);
    for (size_t i = 0; i < batch * out_channels * out_length; ++i) store_elem(dtype, dst, i, 0.0f);
    if (groups == 1 && padding == 0 && output_padding == 0) {
        size_t n = out_channels * kernel_size;
        void *srct = calloc(batch * length * in_channels + 1, es);
        void *col = calloc(batch * length * n + 1, es);
        for (size_t b = 0; b < batch; ++b)
            for (size_t l = 0; l < length; ++l)
                for (size_t c = 0; c < in_channels; ++c)
                    store_elem(dtype, srct, (b * length + l) * in_channels + c,
                               load_elem(dtype, src, (b * in_channels + c) * length + l));
        xo_gemm(dtype, col, srct, 0, kernel, 0, length, n, in_channels, batch, length * in_channels, 0,
                1, n, 1, in_channels, 1, n, 0);
        for (size_t l = 0; l < length; ++l)
            for (size_t kk = 0; kk < kernel_size; ++kk)
                for (size_t b = 0; b < batch; ++b)
                    for (size_t c = 0; c < out_channels; ++c) {
                        size_t di = (b * out_channels + c) * out_length + l * stride + kk;
                        store_elem(dtype, dst, di, load_elem(dtype, dst, di) +
                                   load_elem(dtype, col, ((b * length + l) * out_channels + c) * kernel_size + kk));
                    }
        free(srct);
        free(col);
        return;
    }
    size_t cig = in_channels / groups, cog = out_channels / groups;
    for (size_t kk = 0; kk < kernel_size; ++kk)
        for (size_t oc = 0; oc < out_channels; ++oc) {
            size_t g = oc / cog, ocg = oc % cog, c0 = g * cig;
            for (size_t b = 0; b < batch; ++b)
                for (size_t il = 0; il < length; ++il) {
                    size_t raw = il * stride + kk;
                    if (raw < padding || raw >= out_length + padding) continue;
                    float d = 0.0f;
                    for (size_t ic = 0; ic < cig; ++ic) {
                        float p = round_elem(dtype, load_elem(dtype, src, (b * in_channels + c0 + ic) * length + il) *
                                                        load_elem(dtype, kernel, ((c0 + ic) * cog + ocg) * kernel_size + kk));
                        d = round_elem(dtype, d + p);
                    }
                    size_t di = (b * out_channels + oc) * out_length + raw - padding;
                    store_elem(dtype, dst, di, load_elem(dtype, dst, di) + d);
                }
        }
}
