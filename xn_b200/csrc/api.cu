// Host side of the C ABI: error reporting, argument validation, kernel selection for
// Backend::gemm, and the host-only restatement of Tensor::matmul_'s stride lowering.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace xn {

std::string &last_error() {
    static thread_local std::string msg;
    return msg;
}

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

int sm_count() {
    // Cached per device; devices are few and the table is written once per entry.
    static int cache[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cache[dev] = v;
    }
    return cache[dev];
}

bool pdl_enabled() {
    static const bool on = [] {
        const char *e = getenv("XN_MM_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

static thread_local bool tl_rhs_static = false;
bool rhs_is_static() { return tl_rhs_static; }
StaticRhsScope::StaticRhsScope(bool on) : prev(tl_rhs_static) { tl_rhs_static = on; }
StaticRhsScope::~StaticRhsScope() { tl_rhs_static = prev; }

static thread_local const void *tl_col_bias = nullptr;
static thread_local bool tl_col_bias_taken = false;
ColBiasScope::ColBiasScope(const void *bias) { tl_col_bias = bias; tl_col_bias_taken = false; }
ColBiasScope::~ColBiasScope() { tl_col_bias = nullptr; tl_col_bias_taken = false; }
bool ColBiasScope::taken() const { return tl_col_bias_taken; }
const void *take_fused_col_bias() {
    if (tl_col_bias) tl_col_bias_taken = true;
    return tl_col_bias;
}

int ensure_dynamic_smem(const void *kernel, int *slot, size_t bytes) {
    int dev = 0;
    XN_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) dev = 0;
    if (bytes <= 32 * 1024) return XN_OK;  // leaves room for static shared memory under the 48 KB default
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if ((size_t)slot[dev] >= bytes) return XN_OK;
    XN_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    slot[dev] = (int)bytes;
    return XN_OK;
}

}  // namespace xn

using namespace xn;

extern "C" const char *xn_mm_last_error(void) { return last_error().c_str(); }
extern "C" int xn_mm_abi_version(void) { return 1; }

static int gemm_dispatch(xn_dtype dtype, void *dst, const void *lhs, size_t lhs_off, const void *rhs,
                         size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b,
                         size_t lhs_b_stride, size_t rhs_b_stride, size_t dst_cs, size_t dst_rs,
                         size_t lhs_cs, size_t lhs_rs, size_t rhs_cs, size_t rhs_rs, void *stream, int causal = 0,
                         int causal_off = 0) {
    // Same refusal as the reference for element types it has no GEMM for
    // (xn-core/src/cuda_backend.rs:862).
    if (!valid_dtype(dtype)) return fail(XN_ERR_UNSUPPORTED, "GEMM not supported for dtype %d", (int)dtype);
    if (lhs_b == 0 || m == 0 || n == 0) return XN_OK;  // nothing to write
    XN_REQUIRE(dst && lhs && rhs, "gemm: null pointer (dst=%p lhs=%p rhs=%p)", dst, lhs, rhs);
    const size_t es = dtype_size(dtype);
    XN_REQUIRE(aligned(dst, es) && aligned(lhs, es) && aligned(rhs, es), "gemm: operand not aligned to its element size");
    // Distinct (i,j) must map to distinct dst elements inside one batch slab of m*n elements.
    XN_REQUIRE((dst_cs == 1 && dst_rs >= n) || (dst_rs == 1 && dst_cs >= m) || m == 1 || n == 1,
               "gemm: unsupported dst strides (%zu, %zu) for m:%zu n:%zu", dst_cs, dst_rs, m, n);
    const char *l = static_cast<const char *>(lhs) + lhs_off * es;
    const char *r = static_cast<const char *>(rhs) + rhs_off * es;
    // Decode-sized matmul_t with 16-bit elements (m <= 16, one batch, both operands k-contiguous, a weight worth
    // streaming): the tensor-core weight-streaming kernel.  (Its mma.sync instructions issue at about one per 32
    // cycles per SM sub-partition on this architecture -- 1/16 of the tcgen05 rate -- so beyond two column groups
    // it is bound by them and the tcgen05 kernel below is faster.)
    const bool h16_fits = dtype != XN_F32 && m <= 16 && k <= 0x7fffffff && gemv_h16_single_chunk(m, k);
    // what the tcgen05 kernels need: both operands k-contiguous, dst rows contiguous, 16-byte pitches and bases
    const bool tn16_ok = dtype != XN_F32 && lhs_cs == 1 && rhs_rs == 1 && dst_cs == 1 && k % 8 == 0 && lhs_rs % 8 == 0 &&
                         rhs_cs % 8 == 0 && aligned(l, 16) && aligned(r, 16) && m <= 0x7fffffff && n <= 0x7fffffff &&
                         k <= 0x7fffffff && dst_rs <= 0x7fffffff;
    // up to 16 rows with k too long for the weight-streaming kernel's staged activations: tensor-memory skinny form
    const bool long_k_skinny = tn16_ok && m <= 16 && !h16_fits && n >= 256 && lhs_b == 1;
    if (h16_fits && lhs_b == 1 && n >= 64 && lhs_cs == 1 && rhs_rs == 1 && dst_cs == 1 && k % 8 == 0 &&
        lhs_rs % 8 == 0 && rhs_cs % 8 == 0 && aligned(l, 16) && aligned(r, 16) && k <= 0x7fffffff)
        return launch_gemv_h16(dtype, dst, l, r, m, n, k, dst_rs, lhs_rs, rhs_cs, (cudaStream_t)stream);
    // Decode-sized matmul_t (m <= 16, both operands k-contiguous): the weight-streaming kernel with exact f32
    // products, for all three element types and any batch count.
    {
        const size_t v = 16 / es;
        if (m <= 16 && !long_k_skinny && lhs_cs == 1 && rhs_rs == 1 && dst_cs == 1 && k % v == 0 && lhs_rs % v == 0 && rhs_cs % v == 0 &&
            (lhs_b == 1 || (lhs_b_stride % v == 0 && rhs_b_stride % v == 0)) && aligned(l, 16) && aligned(r, 16)) {
            // f32, one batch, k a multiple of 32, a weight worth streaming: the tensor-core 3xTF32 form
            // (products to ~1e-6 relative; XN_MM_F32_EXACT=1 keeps the exact-product FFMA kernel)
            static const bool exact = [] { const char *e = getenv("XN_MM_F32_EXACT"); return e && atoi(e) != 0; }();
            if (dtype == XN_F32 && !exact && lhs_b == 1 && k % 32 == 0 && n >= 256)
                return launch_gemv_f32x3((float *)dst, (const float *)l, (const float *)r, m, n, k, dst_rs, lhs_rs, rhs_cs,
                                         (cudaStream_t)stream);
            return launch_gemv_dense(dtype, dst, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_rs, lhs_rs, rhs_cs,
                                     (cudaStream_t)stream);
        }
    }
    // f32 matmul_t with 17..96 rows on a weight worth streaming: the same 3xTF32 weight-streaming kernel, 16 rows
    // per pass (one pass per 16 rows re-reads the weight, but never writes a repacked copy of it, which the
    // tensor-memory form below would; at ~45 us per pass on a [11264, 4096] weight the two meet near 100 rows).
    {
        static const bool exact = [] { const char *e = getenv("XN_MM_F32_EXACT"); return e && atoi(e) != 0; }();
        static const size_t pass_max = [] { const char *e = getenv("XN_MM_F32_PASS_MAX_M"); return e ? (size_t)atoi(e) : (size_t)96; }();
        if (dtype == XN_F32 && !exact && m > 16 && m <= pass_max && lhs_b == 1 && lhs_cs == 1 && rhs_rs == 1 && dst_cs == 1 &&
            k % 32 == 0 && n >= 256 && lhs_rs % 4 == 0 && rhs_cs % 4 == 0 && dst_rs >= n && aligned(l, 16) && aligned(r, 16)) {
            for (size_t i0 = 0; i0 < m; i0 += 16) {
                const size_t rows = m - i0 < 16 ? m - i0 : 16;
                if (int rc = launch_gemv_f32x3((float *)dst + i0 * dst_rs, (const float *)l + i0 * lhs_rs, (const float *)r, rows, n, k,
                                               dst_rs, lhs_rs, rhs_cs, (cudaStream_t)stream))
                    return rc;
            }
            return XN_OK;
        }
    }
    // Linear::forward's form with 16-bit elements -- both operands k-contiguous, rows of dst
    // contiguous -- goes to the tcgen05 kernel when TMA can address it (16-byte pitches and bases).
    // The strided-batched / grouped form (lhs_b > 1 with per-batch weights) is one launch as well.
    if (tn16_ok && (m > 16 || long_k_skinny) &&
        (lhs_b == 1 || (lhs_b <= 0x7fffffff && lhs_b_stride % 8 == 0 && rhs_b_stride % 8 == 0 && rhs_b_stride != 0 &&
                        lhs_b_stride != 0)))
        return launch_gemm_tn_16bit(dtype, dst, l, r, m, n, k, lhs_rs, rhs_cs, dst_rs, lhs_b, lhs_b_stride, rhs_b_stride,
                                    (cudaStream_t)stream, causal == 1 ? 1 : 0, causal_off);
    // 16-bit `matmul` with a row-major [k, n] right-hand side (n contiguous; cuBLAS's OP_N in the reference): the
    // tcgen05 kernel reads it as an MN-major operand.  Worth it from a few thousand MACs per output row on; tiny
    // products (decode attention's p.v with one query row) stay on the generic kernel.
    {
        static const bool kn_off = [] { const char *e = getenv("XN_MM_KN_TC"); return e && atoi(e) == 0; }();
        const bool kn16_ok = !kn_off && dtype != XN_F32 && lhs_cs == 1 && rhs_cs == 1 && dst_cs == 1 && n >= 2 && k % 8 == 0 &&
                             lhs_rs % 8 == 0 && rhs_rs % 8 == 0 && rhs_rs >= n && aligned(l, 16) && aligned(r, 16) &&
                             m <= 0x7fffffff && n <= 0x7fffffff && k <= 0x7fffffff && dst_rs <= 0x7fffffff &&
                             (m >= 8 || n * k >= (size_t)1 << 20);
        // batched: one matrix after the other, or interleaved row by row (per-head slices of a wider row)
        if (kn16_ok && (lhs_b == 1 || (lhs_b <= 0x7fffffff && lhs_b_stride % 8 == 0 && rhs_b_stride % 8 == 0 && lhs_b_stride != 0 &&
                                       (rhs_b_stride >= k * rhs_rs || (rhs_b_stride >= n && lhs_b * rhs_b_stride <= rhs_rs)))))
            return launch_gemm_kn_16bit(dtype, dst, l, r, m, n, k, lhs_rs, rhs_rs, dst_rs, lhs_b, lhs_b_stride, rhs_b_stride,
                                        (cudaStream_t)stream, causal == 2 ? 2 : 0, causal_off);
    }
    if (causal == 2)
        return fail(XN_ERR_UNSUPPORTED, "gemm_causal (values): needs 16-bit elements, an n-contiguous right-hand side and "
                                        "16-byte aligned pitches (the masked probabilities are not read, so no other kernel may run it)");
    // f32 with many rows, one batch, row-major dst: three tf32 pieces per operand on the tensor-memory kernel
    // (any operand strides; the repack normalises them).
    if (dtype == XN_F32 && lhs_b == 1 && dst_cs == 1 && dst_rs <= 0x7fffffff && gemm_f32_tc_fits(m, n, k))
        return launch_gemm_f32_tc(static_cast<float *>(dst), reinterpret_cast<const float *>(l), reinterpret_cast<const float *>(r),
                                  m, n, k, dst_rs, lhs_cs, lhs_rs, rhs_cs, rhs_rs, (cudaStream_t)stream);
    return launch_gemm_generic(dtype, dst, l, r, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_cs, dst_rs,
                               lhs_cs, lhs_rs, rhs_cs, rhs_rs, (cudaStream_t)stream);
}

extern "C" int xn_mm_gemm(xn_dtype dtype, void *dst, const void *lhs, size_t lhs_off, const void *rhs,
                          size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b,
                          size_t lhs_b_stride, size_t rhs_b_stride, size_t dst_cs, size_t dst_rs,
                          size_t lhs_cs, size_t lhs_rs, size_t rhs_cs, size_t rhs_rs, void *stream) {
    XN_API_RANGE("xn_mm_gemm");
    // Backend::gemm's rhs is any tensor, possibly the output of the kernel just enqueued on this stream: no
    // kernel may read it ahead of its dependency wait.
    StaticRhsScope scope(false);
    return gemm_dispatch(dtype, dst, lhs, lhs_off, rhs, rhs_off, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_cs, dst_rs,
                         lhs_cs, lhs_rs, rhs_cs, rhs_rs, stream);
}

extern "C" int xn_mm_gemm_causal(int mode, size_t causal_offset, xn_dtype dtype, void *dst, const void *lhs, size_t lhs_off,
                                 const void *rhs, size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
                                 size_t rhs_b_stride, size_t dst_cs, size_t dst_rs, size_t lhs_cs, size_t lhs_rs, size_t rhs_cs,
                                 size_t rhs_rs, void *stream) {
    XN_API_RANGE("xn_mm_gemm_causal");
    XN_REQUIRE(mode == 1 || mode == 2, "gemm_causal: mode %d (1 = scores q.k^T, 2 = values p.v)", mode);
    XN_REQUIRE(causal_offset <= 0x3fffffffull, "gemm_causal: offset too large");
    StaticRhsScope scope(false);
    return gemm_dispatch(dtype, dst, lhs, lhs_off, rhs, rhs_off, m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_cs, dst_rs,
                         lhs_cs, lhs_rs, rhs_cs, rhs_rs, stream, mode, (int)causal_offset);
}

extern "C" int xn_mm_linear(xn_dtype dtype, void *y, const void *x, const void *weight, const void *bias_or_null, size_t m,
                            size_t n, size_t k, size_t ldx, size_t ldw, size_t ldy, void *stream) {
    XN_API_RANGE("xn_mm_linear");
    if (!valid_dtype(dtype)) return fail(XN_ERR_UNSUPPORTED, "linear: GEMM not supported for dtype %d", (int)dtype);
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y && x && weight, "linear: null pointer (y=%p x=%p weight=%p)", y, x, weight);
    XN_REQUIRE(ldx >= k && ldw >= k && ldy >= n, "linear: row pitch smaller than the row (ldx=%zu ldw=%zu k=%zu ldy=%zu n=%zu)",
               ldx, ldw, k, ldy, n);
    int rc;
    {
        StaticRhsScope scope(true);  // the weight is a parameter: weight-streaming kernels may prefetch it
        ColBiasScope bias_scope(bias_or_null);  // the tiled tensor-memory kernel adds it in its epilogue
        rc = gemm_dispatch(dtype, y, x, 0, weight, 0, m, n, k, 1, m * ldx, 1, 1, ldy, 1, ldx, ldw, 1, stream);
        if (bias_scope.taken()) return rc;
    }
    if (rc || !bias_or_null) return rc;
    if (ldy == n) return xn_mm_add_bias(dtype, y, y, bias_or_null, m, n, stream);
    const size_t es = dtype_size(dtype);
    for (size_t i = 0; i < m; ++i) {  // pitched rows: one row at a time (rare; a view of a wider output)
        char *row = static_cast<char *>(y) + i * ldy * es;
        if (int r2 = xn_mm_add_bias(dtype, row, row, bias_or_null, 1, n, stream)) return r2;
    }
    return XN_OK;
}

extern "C" int xn_mm_matmul_plan(size_t lhs_rank, const size_t *lhs_dims, const size_t *lhs_strides,
                                 size_t rhs_rank, const size_t *rhs_dims, const size_t *rhs_strides,
                                 int rhs_t, size_t dst_capacity, size_t *out) {
    XN_API_RANGE("xn_mm_matmul_plan");
    XN_REQUIRE(lhs_dims && lhs_strides && rhs_dims && rhs_strides && out, "matmul: null pointer");
    XN_REQUIRE(lhs_rank >= 2 && rhs_rank >= 2, "matmul requires at least 2D tensors, got lhs rank %zu, rhs rank %zu",
               lhs_rank, rhs_rank);
    const size_t *ld = lhs_dims + lhs_rank - 2, *rd = rhs_dims + rhs_rank - 2;
    const size_t m = ld[0], k = ld[1];
    const size_t rk = rhs_t ? rd[1] : rd[0], n = rhs_t ? rd[0] : rd[1];
    XN_REQUIRE(k == rk, "matmul inner dimension mismatch: lhs k=%zu, rhs k=%zu, rhs_t=%d", k, rk, rhs_t);
    size_t lb = 1, rb = 1;
    for (size_t i = 0; i + 2 < lhs_rank; ++i) lb *= lhs_dims[i];
    for (size_t i = 0; i + 2 < rhs_rank; ++i) rb *= rhs_dims[i];
    if (rhs_rank > 2) {
        bool same = rhs_rank == lhs_rank;
        for (size_t i = 0; same && i + 2 < rhs_rank; ++i) same = rhs_dims[i] == lhs_dims[i];
        XN_REQUIRE(same, "batch dimensions do not match in matmul");
    }
    if (lb < 1) lb = 1;
    if (rb < 1) rb = 1;
    XN_REQUIRE(lb * m * n <= dst_capacity, "matmul dst is too small, dst %zu < %zu", dst_capacity, lb * m * n);
    const size_t *ls = lhs_strides + lhs_rank, *rs = rhs_strides + rhs_rank;
    size_t lhs_b_stride = lhs_rank >= 3 ? ls[-3] : m * k;
    size_t rhs_b_stride = rb == 1 ? 0 : (rhs_rank >= 3 ? rs[-3] : rd[0] * rd[1]);
    size_t mm = m, batch = lb;
    if (lhs_b_stride == m * ls[-2] && rb == 1) {  // one flat GEMM over all lhs rows
        batch = 1;
        rhs_b_stride = 1;
        mm = lb * m;
    }
    out[0] = mm; out[1] = n; out[2] = k; out[3] = batch; out[4] = lhs_b_stride; out[5] = rhs_b_stride;
    out[6] = 1; out[7] = n; out[8] = ls[-1]; out[9] = ls[-2];
    out[10] = rhs_t ? rs[-2] : rs[-1];
    out[11] = rhs_t ? rs[-1] : rs[-2];
    return XN_OK;
}

// ---- host-side q4 tile packing (layout documented in include/xn_mm.h) ----
static inline size_t q4_byte_index(size_t r, size_t kk, size_t k) {
    const size_t tile = (r / 16) * (k / 128) + kk / 128;
    const size_t rr = r % 16, h = rr / 8, g = rr % 8, j = (kk % 128) / 32, e = kk % 32;
    const size_t t = (e % 16) / 4, i = e % 4;
    return tile * 1280 + (32 * h + 4 * g + t) * 16 + j * 4 + i;
}
static inline size_t q4_scale_offset(size_t r, size_t blk, size_t k) {  // byte offset of a block scale
    const size_t tile = (r / 16) * (k / 128) + blk / 4;
    return tile * 1280 + 1024 + ((4 * (r % 8) + blk % 4) * 2 + (r % 16) / 8) * 4;
}

extern "C" int xn_mm_pack_q4_host(uint8_t *packed, const int8_t *q, const float *scales, size_t n, size_t k) {
    XN_API_RANGE("xn_mm_pack_q4_host");
    XN_REQUIRE(k % 128 == 0, "pack_q4: k=%zu must be a multiple of 128", k);
    if (n == 0 || k == 0) return XN_OK;
    XN_REQUIRE(packed && q && scales, "pack_q4: null pointer");
    memset(packed, 0, xn_mm_q4_packed_bytes(n, k));
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) {
            const int v = q[r * k + kk];
            XN_REQUIRE(v >= -8 && v <= 7, "pack_q4: value %d at (%zu,%zu) does not fit in 4 bits", v, r, kk);
            const uint8_t nib = (uint8_t)v & 0xF;
            uint8_t &b = packed[q4_byte_index(r, kk, k)];
            b = (kk % 32) / 16 ? (uint8_t)(b | (nib << 4)) : (uint8_t)(b | nib);
        }
        for (size_t blk = 0; blk < k / 32; ++blk)
            memcpy(packed + q4_scale_offset(r, blk, k), &scales[r * (k / 32) + blk], 4);
    }
    return XN_OK;
}

extern "C" int xn_mm_unpack_q4_host(int8_t *q, float *scales, const uint8_t *packed, size_t n, size_t k) {
    XN_API_RANGE("xn_mm_unpack_q4_host");
    XN_REQUIRE(k % 128 == 0, "unpack_q4: k=%zu must be a multiple of 128", k);
    if (n == 0 || k == 0) return XN_OK;
    XN_REQUIRE(packed && q && scales, "unpack_q4: null pointer");
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) {
            const uint8_t b = packed[q4_byte_index(r, kk, k)];
            int v = (kk % 32) / 16 ? (b >> 4) : (b & 0xF);
            q[r * k + kk] = (int8_t)(v >= 8 ? v - 16 : v);
        }
        for (size_t blk = 0; blk < k / 32; ++blk)
            memcpy(&scales[r * (k / 32) + blk], packed + q4_scale_offset(r, blk, k), 4);
    }
    return XN_OK;
}

// ---- host-side q8 tile packing ----
static inline size_t q8_byte_index(size_t r, size_t kk, size_t k) {
    const size_t tile = (r / 16) * (k / 128) + kk / 128;
    const size_t rr = r % 16, h = rr / 8, g = rr % 8, j = (kk % 128) / 32, e = kk % 32;
    const size_t t = (e % 16) / 4, i = e % 4, hi = e / 16;
    return tile * 2304 + j * 512 + (4 * g + t) * 16 + (h + 2 * hi) * 4 + i;
}
static inline size_t q8_scale_offset(size_t r, size_t blk, size_t k) {
    const size_t tile = (r / 16) * (k / 128) + blk / 4;
    return tile * 2304 + 2048 + ((4 * (r % 8) + blk % 4) * 2 + (r % 16) / 8) * 4;
}

extern "C" int xn_mm_pack_q8_host(uint8_t *packed, const int8_t *q, const float *scales, size_t n, size_t k) {
    XN_API_RANGE("xn_mm_pack_q8_host");
    XN_REQUIRE(k % 128 == 0, "pack_q8: k=%zu must be a multiple of 128", k);
    if (n == 0 || k == 0) return XN_OK;
    XN_REQUIRE(packed && q && scales, "pack_q8: null pointer");
    memset(packed, 0, xn_mm_q8_packed_bytes(n, k));
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) packed[q8_byte_index(r, kk, k)] = (uint8_t)q[r * k + kk];
        for (size_t blk = 0; blk < k / 32; ++blk)
            memcpy(packed + q8_scale_offset(r, blk, k), &scales[r * (k / 32) + blk], 4);
    }
    return XN_OK;
}

extern "C" int xn_mm_unpack_q8_host(int8_t *q, float *scales, const uint8_t *packed, size_t n, size_t k) {
    XN_API_RANGE("xn_mm_unpack_q8_host");
    XN_REQUIRE(k % 128 == 0, "unpack_q8: k=%zu must be a multiple of 128", k);
    if (n == 0 || k == 0) return XN_OK;
    XN_REQUIRE(packed && q && scales, "unpack_q8: null pointer");
    for (size_t r = 0; r < n; ++r) {
        for (size_t kk = 0; kk < k; ++kk) q[r * k + kk] = (int8_t)packed[q8_byte_index(r, kk, k)];
        for (size_t blk = 0; blk < k / 32; ++blk)
            memcpy(&scales[r * (k / 32) + blk], packed + q8_scale_offset(r, blk, k), 4);
    }
    return XN_OK;
}

extern "C" int xn_mm_attention_prefill(xn_dtype dtype, void *out, size_t ldo, const void *q, const void *k, const void *v,
                                       size_t ld, size_t head_stride, size_t heads, size_t head_dim, size_t t_rows,
                                       size_t context, float scale, void *stream) {
    XN_API_RANGE("xn_mm_attention_prefill");
    XN_REQUIRE(dtype == XN_BF16 || dtype == XN_F16, "attention_prefill: 16-bit element types only (dtype %d)", (int)dtype);
    XN_REQUIRE(head_dim == 128, "attention_prefill: head_dim %zu (128 supported)", head_dim);
    if (heads == 0 || t_rows == 0) return XN_OK;
    XN_REQUIRE(out && q && k && v, "attention_prefill: null pointer");
    XN_REQUIRE(context >= t_rows && context <= 0x3fffffffull && heads <= 65535,
               "attention_prefill: context %zu must be at least the %zu query rows", context, t_rows);
    XN_REQUIRE(ld % 8 == 0 && head_stride % 8 == 0 && ldo % 8 == 0 && ldo >= heads * 128 && aligned(out, 16) && aligned(q, 16) &&
                   aligned(k, 16) && aligned(v, 16),
               "attention_prefill: pointers, row pitches and the head stride must be multiples of 16 bytes");
    XN_REQUIRE(head_stride >= 128 || heads == 1, "attention_prefill: heads overlap (head stride %zu)", head_stride);
    return launch_attention_prefill(dtype, out, ldo, q, k, v, ld, head_stride, heads, t_rows, context, scale, (cudaStream_t)stream);
}
