// Entry points of the fp8-e4m3 weight linear: validation, workspace carving, regime selection
// (decode-sized batches -> weight-streaming kernel; larger batches -> tensor-core GEMM).
#include <mutex>

#include "common.cuh"

namespace xn {
int launch_linear_fp8_gemv(void *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale,
                           const uint8_t *wq, const float *w_scale, int m, size_t n, int k, cudaStream_t st);

int launch_linear_fp8_gemm(void *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale, const uint8_t *wq,
                           const float *w_scale, size_t m, size_t n, size_t k, cudaStream_t st);

int launch_linear_fp8_gemm_scatter(void *const *y_dsts, int ndst, size_t ldy, size_t col_offset, const uint8_t *x_hi,
                                   const uint8_t *x_lo, const float *x_scale, const uint8_t *wq, const float *w_scale,
                                   size_t m, size_t n, size_t k, cudaStream_t st);

int launch_linear_fp8_gemm_multicast(void *y_mc, size_t ldy, size_t col_offset, const uint8_t *x_hi, const uint8_t *x_lo,
                                     const float *x_scale, const uint8_t *wq, const float *w_scale, size_t m, size_t n,
                                     size_t k, cudaStream_t st);

static inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace xn

using namespace xn;

extern "C" int xn_mm_linear_fp8_pieces(void *y_bf16, const uint8_t *x_hi, const uint8_t *x_lo,
                                       const float *x_scale, const uint8_t *wq, const float *w_scale,
                                       size_t m, size_t n, size_t k, void *stream) {
    XN_API_RANGE("xn_mm_linear_fp8_pieces");
    XN_REQUIRE(k > 0 && k % 16 == 0, "linear_fp8: k=%zu must be a positive multiple of 16", k);
    XN_REQUIRE(k <= 0x7ffffff0ull && n <= 0x7ffffff0ull, "linear_fp8: dimension too large");
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y_bf16 && x_hi && x_scale && wq && w_scale, "linear_fp8: null pointer");
    XN_REQUIRE(aligned(wq, 16) && aligned(x_hi, 16) && (!x_lo || aligned(x_lo, 16)),
               "linear_fp8: weights and activation pieces must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    // Up to 8 rows (one MMA column group) stream the weights once through the GEMV kernel; anything larger
    // goes to the tensor-memory kernels (skinny form up to 64 rows, tiled GEMM beyond), which were measured
    // faster from 9 rows on for every transformer shape.
    static const size_t gemv_max_m = [] { const char *e = getenv("XN_FP8_GEMV_MAX_M"); return e ? (size_t)atoi(e) : (size_t)8; }();
    if (m > gemv_max_m) return launch_linear_fp8_gemm(y_bf16, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
    for (size_t i0 = 0; i0 < m; i0 += 32) {
        const int mc = (int)((m - i0) < 32 ? (m - i0) : 32);
        int rc = launch_linear_fp8_gemv((char *)y_bf16 + i0 * n * 2, x_hi + i0 * k, x_lo ? x_lo + i0 * k : nullptr,
                                        x_scale + i0, wq, w_scale, mc, n, (int)k, st);
        if (rc) return rc;
    }
    return XN_OK;
}

extern "C" int xn_mm_linear_fp8_pieces_scatter(void *const *y_dsts, size_t num_dst, size_t ldy, size_t col_offset,
                                               const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale,
                                               const uint8_t *wq, const float *w_scale, size_t m, size_t n, size_t k,
                                               void *stream) {
    XN_API_RANGE("xn_mm_linear_fp8_pieces_scatter");
    XN_REQUIRE(k > 0 && k % 16 == 0, "linear_fp8_scatter: k=%zu must be a positive multiple of 16", k);
    XN_REQUIRE(num_dst >= 1 && num_dst <= 8, "linear_fp8_scatter: %zu destinations (1..8 supported)", num_dst);
    XN_REQUIRE(k <= 0x7ffffff0ull && n <= 0x7ffffff0ull && ldy <= 0x7ffffff0ull, "linear_fp8_scatter: dimension too large");
    XN_REQUIRE(col_offset + n <= ldy, "linear_fp8_scatter: columns [%zu, %zu) do not fit a row of %zu", col_offset,
               col_offset + n, ldy);
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y_dsts && x_hi && x_scale && wq && w_scale, "linear_fp8_scatter: null pointer");
    for (size_t p = 0; p < num_dst; ++p) XN_REQUIRE(y_dsts[p], "linear_fp8_scatter: destination %zu is null", p);
    XN_REQUIRE(aligned(wq, 16) && aligned(x_hi, 16) && (!x_lo || aligned(x_lo, 16)),
               "linear_fp8_scatter: weights and activation pieces must be 16-byte aligned");
    return launch_linear_fp8_gemm_scatter(y_dsts, (int)num_dst, ldy, col_offset, x_hi, x_lo, x_scale, wq, w_scale, m, n, k,
                                          (cudaStream_t)stream);
}

extern "C" int xn_mm_linear_fp8_pieces_multicast(void *y_multicast, size_t ldy, size_t col_offset, const uint8_t *x_hi,
                                                 const uint8_t *x_lo, const float *x_scale, const uint8_t *wq,
                                                 const float *w_scale, size_t m, size_t n, size_t k, void *stream) {
    XN_API_RANGE("xn_mm_linear_fp8_pieces_multicast");
    XN_REQUIRE(k > 0 && k % 16 == 0, "linear_fp8_multicast: k=%zu must be a positive multiple of 16", k);
    XN_REQUIRE(k <= 0x7ffffff0ull && n <= 0x7ffffff0ull && ldy <= 0x7ffffff0ull, "linear_fp8_multicast: dimension too large");
    XN_REQUIRE(col_offset + n <= ldy, "linear_fp8_multicast: columns [%zu, %zu) do not fit a row of %zu", col_offset,
               col_offset + n, ldy);
    XN_REQUIRE(n % 8 == 0 && col_offset % 8 == 0 && ldy % 8 == 0,
               "linear_fp8_multicast: n=%zu, col_offset=%zu and ldy=%zu must be multiples of 8 (16-byte multicast stores)", n,
               col_offset, ldy);
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y_multicast && x_hi && x_scale && wq && w_scale, "linear_fp8_multicast: null pointer");
    XN_REQUIRE(aligned(y_multicast, 16) && aligned(wq, 16) && aligned(x_hi, 16) && (!x_lo || aligned(x_lo, 16)),
               "linear_fp8_multicast: output, weights and activation pieces must be 16-byte aligned");
    return launch_linear_fp8_gemm_multicast(y_multicast, ldy, col_offset, x_hi, x_lo, x_scale, wq, w_scale, m, n, k,
                                            (cudaStream_t)stream);
}

extern "C" size_t xn_mm_linear_fp8_workspace_bytes(size_t m, size_t k) {
    return 2 * round_up(m * k, 256) + round_up(m * sizeof(float), 256);
}

extern "C" int xn_mm_linear_fp8(void *y_bf16, const void *x_bf16, const uint8_t *wq, const float *w_scale,
                                size_t m, size_t n, size_t k, int variant, void *workspace,
                                size_t workspace_bytes, void *stream) {
    XN_API_RANGE("xn_mm_linear_fp8");
    XN_REQUIRE(variant == 0 || variant == 1, "linear_fp8: variant must be 0 (W8A16) or 1 (W8A8), got %d", variant);
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(workspace && aligned(workspace, 256), "linear_fp8: workspace must be a 256-byte aligned device buffer");
    if (workspace_bytes < xn_mm_linear_fp8_workspace_bytes(m, k))
        return fail(XN_ERR_WORKSPACE, "linear_fp8: workspace of %zu bytes is smaller than the %zu needed",
                    workspace_bytes, xn_mm_linear_fp8_workspace_bytes(m, k));
    uint8_t *hi = (uint8_t *)workspace;
    uint8_t *lo = hi + round_up(m * k, 256);
    float *xs = (float *)(lo + round_up(m * k, 256));
    int rc = xn_mm_split_rows_e4m3(hi, variant == 0 ? lo : nullptr, xs, x_bf16, XN_BF16, m, k, stream);
    if (rc) return rc;
    return xn_mm_linear_fp8_pieces(y_bf16, hi, variant == 0 ? lo : nullptr, xs, wq, w_scale, m, n, k, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of xn_mm_linear_fp8.
//
// Some hosts of this library cannot obtain device memory at call time: a serving loop whose whole
// device budget was handed to another allocator at start-up, a real-time audio callback where a
// cudaMalloc (which may synchronise the device) is not acceptable, or an embedder that is simply not
// allowed to call the CUDA allocator.  xn_mm_linear_fp8 needs scratch for the e4m3 activation pieces
// and their row scales; here that scratch is a fixed array that is part of the library image, so the
// call allocates nothing -- no cudaMalloc, cudaFree or allocating library routine is reached.
//
// Cost and limits: every GPU that loads the library holds XN_NOALLOC_SCRATCH_BYTES (513 KiB) until
// the process exits.  Sizes are limited to m <= 64 and m * k <= 262144 (decode-sized batches, e.g.
// 16 x 16384 or 64 x 4096); anything larger is refused with XN_ERR_UNSUPPORTED.
//
// The array is shared by every call on a device.  It keeps the previous call's contents; nothing in
// it has to start at zero, because each call rewrites the m * k piece bytes and m scales it then
// reads.  Two calls that overlap on the GPU (different streams, or different host threads on
// different streams) race on it: keep all calls on one device in one stream order.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that
// first call outside any stream capture.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t NOALLOC_MAX_ELEMS = 262144;  // m * k
constexpr size_t NOALLOC_MAX_ROWS = 64;
constexpr size_t NOALLOC_SCALE_OFFSET = 2 * NOALLOC_MAX_ELEMS;
constexpr size_t NOALLOC_BYTES = NOALLOC_SCALE_OFFSET + 1024;

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) unsigned char g_fp8_noalloc_scratch[NOALLOC_BYTES];

int noalloc_scratch(unsigned char **out) {
    static unsigned char *table[64];
    static std::mutex mu;
    int dev = 0;
    XN_CHECK_CUDA(cudaGetDevice(&dev));
    XN_REQUIRE(dev >= 0 && dev < 64, "linear_fp8_noalloc: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!table[dev]) {
        void *p = nullptr;
        XN_CHECK_CUDA(cudaGetSymbolAddress(&p, g_fp8_noalloc_scratch));  // address on the current device
        table[dev] = static_cast<unsigned char *>(p);
    }
    *out = table[dev];
    return XN_OK;
}
}  // namespace

extern "C" size_t xn_mm_linear_fp8_noalloc_max_elems(void) { return NOALLOC_MAX_ELEMS; }

extern "C" int xn_mm_linear_fp8_noalloc(void *y_bf16, const void *x_bf16, const uint8_t *wq, const float *w_scale,
                                        size_t m, size_t n, size_t k, int variant, void *stream) {
    XN_API_RANGE("xn_mm_linear_fp8_noalloc");
    XN_REQUIRE(variant == 0 || variant == 1, "linear_fp8_noalloc: variant must be 0 (W8A16) or 1 (W8A8), got %d",
               variant);
    if (m > NOALLOC_MAX_ROWS || (k != 0 && m > NOALLOC_MAX_ELEMS / k))
        return fail(XN_ERR_UNSUPPORTED,
                    "linear_fp8_noalloc: m=%zu k=%zu exceeds the built-in scratch (m <= %zu and m*k <= %zu); "
                    "use xn_mm_linear_fp8 with a caller workspace",
                    m, k, NOALLOC_MAX_ROWS, NOALLOC_MAX_ELEMS);
    XN_REQUIRE(k > 0 && k % 16 == 0, "linear_fp8_noalloc: k=%zu must be a positive multiple of 16", k);
    XN_REQUIRE(k <= 0x7ffffff0ull && n <= 0x7ffffff0ull, "linear_fp8_noalloc: dimension too large");
    if (m == 0 || n == 0) return XN_OK;
    XN_REQUIRE(y_bf16 && x_bf16 && wq && w_scale, "linear_fp8_noalloc: null pointer");
    XN_REQUIRE(aligned(wq, 16), "linear_fp8_noalloc: weights must be 16-byte aligned");
    // Every argument check is above this line: nothing has been enqueued, and the shared scratch has not been
    // touched, when a call is rejected.
    NoAllocScope no_alloc;  // the kernels' wait-status word is not allocated on behalf of this entry point
    unsigned char *base = nullptr;
    int rc = noalloc_scratch(&base);
    if (rc) return rc;
    uint8_t *hi = base;
    uint8_t *lo = base + NOALLOC_MAX_ELEMS;
    float *xs = reinterpret_cast<float *>(base + NOALLOC_SCALE_OFFSET);
    rc = xn_mm_split_rows_e4m3(hi, variant == 0 ? lo : nullptr, xs, x_bf16, XN_BF16, m, k, stream);
    if (rc) return rc;
    // Only kernels that need no scratch of their own: the weight-streaming GEMV up to 32 rows, the tiled
    // tensor-memory kernel beyond.  (xn_mm_linear_fp8_pieces would pick the skinny kernel from 9 rows on, whose
    // split-tile hand-over lives in a library-owned buffer that is allocated on first use.)
    const uint8_t *lo_or_null = variant == 0 ? lo : nullptr;
    if (m <= 32) return launch_linear_fp8_gemv(y_bf16, hi, lo_or_null, xs, wq, w_scale, (int)m, n, (int)k, (cudaStream_t)stream);
    void *dst[1] = {y_bf16};
    return launch_linear_fp8_gemm_scatter(dst, 1, n, 0, hi, lo_or_null, xs, wq, w_scale, m, n, k, (cudaStream_t)stream);
}
