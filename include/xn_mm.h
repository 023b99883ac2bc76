/*
 * xn_mm.h -- C ABI of the B200 (sm_100a) matmul engine for xn.
 *
 * Every entry point takes plain pointers and sizes.  Device pointers are CUDA
 * device addresses on the current device; `stream` is a cudaStream_t passed as
 * void* (NULL = the default stream, which is what xn-core's Device uses,
 * xn-core/src/cuda_backend.rs:52).  All work is enqueued asynchronously; the
 * caller synchronises (xn-core/src/cuda_backend.rs:427-430).  Sizes, strides
 * and offsets are in ELEMENTS unless a name ends in _bytes.
 *
 * Return value: 0 on success, otherwise an xn_status code; a human-readable
 * message for the calling thread's last failure is returned by
 * xn_mm_last_error().  Arguments are validated on the host before any launch;
 * no entry point traps on the device.  Entry points may be called from many
 * host threads at once (the reference's Backend is Send + Sync,
 * xn-core/src/backend.rs:4).
 *
 * Library-owned device memory: one kernel (the skinny tensor-memory form, used by xn_mm_gemm for
 * 16-bit operands with 17..64 rows, or fewer rows and a very long k, and by the fp8 linears for 9..64
 * rows) hands split tiles over through a buffer per (device, stream) that the library allocates when a
 * stream first needs it and grows when a larger problem arrives (a few MB; cudaMalloc, i.e. not allowed
 * during stream capture: run each shape once before capturing it, as a decode loop does anyway; a stream
 * under capture borrows the buffer of the stream that ran those shapes, so keep the graph's replays ordered
 * with that stream's own calls).  Calls on different streams use different buffers and may overlap.
 * The same buffer holds the repacked operands of an f32 xn_mm_gemm with 17 or more rows (three tf32
 * pieces per element: 12 bytes per operand element, refused above 2 GiB in favour of the plain f32
 * kernel; XN_MM_F32_TC=0 in the environment keeps every f32 call on the plain kernel).
 * Nothing else allocates;
 * xn_mm_linear_fp8_noalloc avoids that kernel altogether.
 */
#ifndef XN_MM_H
#define XN_MM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types Backend::gemm accepts on CUDA (xn-core/src/cuda_backend.rs:803-862);
 * numbering is this library's own. */
typedef enum { XN_F32 = 0, XN_F16 = 1, XN_BF16 = 2 } xn_dtype;

typedef enum {
    XN_OK = 0,
    XN_ERR_INVALID = 1,     /* shape / stride / null / alignment problem: the Rust side's bail!() */
    XN_ERR_UNSUPPORTED = 2, /* dtype or size outside what the engine implements */
    XN_ERR_CUDA = 3,        /* a CUDA runtime call failed (Error::CudaDriver in the reference) */
    XN_ERR_WORKSPACE = 4,   /* caller-provided workspace too small */
    XN_ERR_DEVICE = 5       /* a device-side wait ran out in an earlier launch (see xn_mm_device_status) */
} xn_status;

const char *xn_mm_last_error(void);
/* Library version, bumped when the ABI changes. */
int xn_mm_abi_version(void);

/* ------------------------------------------------------------------------------------------
 * Device-side failures.  The reference turns every CUDA failure into an Err at the call that hit it
 * (xn-core/src/error.rs:71-92).  The kernels here wait on hardware barriers (copy completions, MMA
 * completions); each such wait is bounded to 2 s, after which the kernel gives up, leaves through its
 * normal exit and increments a status word in pinned host memory (one per device, allocated at the first
 * launch that needs it -- make that launch outside stream capture).  From then on every entry point that
 * would launch such a kernel on that device returns XN_ERR_DEVICE instead, because outputs written since
 * are undefined.
 *   xn_mm_device_status        non-blocking read of the current device's word: XN_OK when zero, XN_ERR_DEVICE
 *                              otherwise; *timeouts_out (optional) receives the count.  Call it at your own
 *                              synchronisation points to learn about a failure in work already completed.
 *   xn_mm_clear_device_status  synchronises the device, zeroes the word and the library's scratch counters.
 *   xn_mm_selftest_wait_timeout  launches one warp that waits, with the given limit, on a barrier nobody
 *                              arrives on: the wait runs out, the kernel exits normally and the status word
 *                              moves.  For tests of the reporting path; nothing faults or hangs.
 * Library-owned scratch (see the top of this file) is kept per (device, stream) for the life of the process;
 * a replaced block is kept too, since a captured graph may still point at it.  xn_mm_release_scratch
 * synchronises the current device and frees the blocks of `stream` (or of every stream when all_streams != 0)
 * together with all replaced blocks of the device; graphs captured earlier that ran the skinny kernel or the
 * f32 repack must not be replayed afterwards.
 * ------------------------------------------------------------------------------------------ */
int xn_mm_device_status(unsigned *timeouts_out);
int xn_mm_clear_device_status(void);
int xn_mm_selftest_wait_timeout(unsigned long long limit_ns, void *stream);
int xn_mm_release_scratch(void *stream, int all_streams);

/* ------------------------------------------------------------------------------------------
 * Backend::gemm -- replaces the body of CudaDevice's `gemm` (xn-core/src/cuda_backend.rs:787-865,
 * which calls cublasGemmStridedBatchedEx at :2109/:2170/:2231); signature mirrors the trait
 * method xn-core/src/backend.rs:135-148 argument for argument, plus dtype and stream.
 *
 *   for b < lhs_b, i < m, j < n:
 *     dst[b*m*n + i*dst_rs + j*dst_cs] =
 *        sum_{p<k} lhs[lhs_off + b*lhs_b_stride + i*lhs_rs + p*lhs_cs]
 *                * rhs[rhs_off + b*rhs_b_stride + p*rhs_rs + j*rhs_cs]
 *
 * f32 accumulation, dst overwritten (it arrives uninitialised, xn-core/src/ops.rs:697).
 * rhs_b_stride == 0 shares rhs across the batch.  This is also the grouped / per-codebook
 * form: one call, lhs_b groups.  Every stride pattern is accepted (the reference's CUDA path
 * rejects patterns cuBLAS cannot express, xn-core/src/cuda_backend.rs:208-223; its CPU path
 * accepts all of them).  dst must not overlap lhs or rhs.
 * ------------------------------------------------------------------------------------------ */
int xn_mm_gemm(xn_dtype dtype, void *dst, const void *lhs, size_t lhs_off, const void *rhs,
               size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
               size_t rhs_b_stride, size_t dst_cs, size_t dst_rs, size_t lhs_cs, size_t lhs_rs,
               size_t rhs_cs, size_t rhs_rs, void *stream);

/* Causal attention over a block of query rows as one kernel (prefill): for every head h < heads and query row i < t_rows,
 *   out[i][128 h .. 128 h + 127] = softmax_j(scale * q[i,h,:] . k[j,h,:]) v[j,h,:]   over the keys j <= i + (context - t_rows),
 * the block of xn-moshi/src/batched_transformer.rs:174-190 (matmul_t, scale, mask, softmax, matmul) for t_rows > 1.
 * q is [t_rows][heads][128], k and v are [context][heads][128]: row pitch `ld` elements, heads `head_stride` elements
 * apart (the three slices of a fused qkv projection, or separate tensors); out row pitch ldo.  bf16 / f16, head_dim
 * 128.  Scores and probabilities stay on the SM (tensor memory and shared memory): f32 scores, exact row maximum,
 * probabilities rounded to the element type before the product with v, f32 row sums, one division at the end. */
int xn_mm_attention_prefill(xn_dtype dtype, void *out, size_t ldo, const void *q, const void *k, const void *v,
                            size_t ld, size_t head_stride, size_t heads, size_t head_dim, size_t t_rows, size_t context,
                            float scale, void *stream);

/* The two batched matmuls of causal attention over a block of query rows (xn-moshi/src/batched_transformer.rs:175,
 * 190, with the mask IndicesAndMask builds): key j is visible to query row i iff j <= i + causal_offset
 * (causal_offset = context - rows).  Same arguments and arithmetic as xn_mm_gemm; what differs is the work skipped:
 *   mode 1 (scores, q.k^T: m = query rows, n = keys)  output tiles that lie entirely beyond the horizon of their
 *          last row are neither computed nor written: dst is defined for j <= i + causal_offset (and, tile-wise,
 *          a little beyond); the rest keeps whatever it held.  xn_mm_softmax_causal reads only the visible part.
 *   mode 2 (values, p.v: m = query rows, k = keys)     the k loop of a 128-row tile stops at the horizon of its
 *          last row; lhs entries beyond it are never read (xn_mm_softmax_causal writes zeros up to that bound
 *          and nothing beyond).  16-bit elements with an n-contiguous rhs only (XN_ERR_UNSUPPORTED otherwise).
 * No counterpart in the reference, which multiplies the full squares. */
int xn_mm_gemm_causal(int mode, size_t causal_offset, xn_dtype dtype, void *dst, const void *lhs, size_t lhs_off,
                      const void *rhs, size_t rhs_off, size_t m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
                      size_t rhs_b_stride, size_t dst_cs, size_t dst_rs, size_t lhs_cs, size_t lhs_rs, size_t rhs_cs,
                      size_t rhs_rs, void *stream);

/* Linear::forward (xn-core/src/nn/linear.rs:56-66): y [m,n] = x [m,k] * weight [n,k]^T (+ bias [n]), rows
 * ldx / ldw / ldy elements apart.  Same arithmetic and kernels as xn_mm_gemm with
 * (lhs_cs,lhs_rs) = (1,ldx), (rhs_cs,rhs_rs) = (ldw,1); the difference is a promise: `weight` is a model
 * parameter that no work in flight on `stream` writes, so the weight-streaming kernels may start fetching it
 * while the previous kernel on the stream is still running (programmatic dependent launch).  xn_mm_gemm
 * makes no such assumption about rhs -- it may be the previous call's dst -- and reads it only after the
 * stream order allows.  The same promise holds for the weight operand (wq / wq_packed and scales) of every
 * quantized linear below.  x, bias and y follow the stream order as usual. */
int xn_mm_linear(xn_dtype dtype, void *y, const void *x, const void *weight, const void *bias_or_null, size_t m,
                 size_t n, size_t k, size_t ldx, size_t ldw, size_t ldy, void *stream);

/* Host-only: Tensor::matmul_'s lowering of two views to the gemm arguments
 * (xn-core/src/inplace_ops.rs:318-436, shape rules of xn-core/src/ops.rs:640-700).
 * out12 = {m, n, k, lhs_b, lhs_b_stride, rhs_b_stride, dst_cs, dst_rs, lhs_cs, lhs_rs,
 * rhs_cs, rhs_rs}.  dst_capacity is the element count of the destination storage
 * (inplace_ops.rs:371-383).  XN_ERR_INVALID on rank < 2, inner-dimension mismatch, batch
 * mismatch or a destination that is too small. */
int xn_mm_matmul_plan(size_t lhs_rank, const size_t *lhs_dims, const size_t *lhs_strides,
                      size_t rhs_rank, const size_t *rhs_dims, const size_t *rhs_strides,
                      int rhs_t, size_t dst_capacity, size_t *out12);

/* ------------------------------------------------------------------------------------------
 * Block-quantized integer weights.  No counterpart in the reference (its DType has no
 * quantized member, xn-core/src/dtype.rs:4-10); these follow the operand specification of the
 * int4 decode configuration.
 *
 * Weights W [n,k], k in 32-element blocks, scale = max|w|/7 (int4) or /127 (int8) per block,
 * q = clamp(round_half_even(w/scale)).  Activations: int8 per row, scale = max|x|/127.
 *   P[i,j,blk] = sum_32 xq*wq   (int32, exact)
 *   y[i,j]     = x_scale[i] * sum_blk (float)P[i,j,blk] * w_scale[j,blk]
 *
 * Packed int4 storage ("q4 tiles"): rows padded to a multiple of 16, k a multiple of 128.
 * Tile (r/16, kk/128) is 1280 bytes; tiles are ordered [r/16][kk/128].
 *   bytes 0..1023: 64 chunks of 16 bytes; chunk 32*h + 4*g + t holds, for row 16*(r/16) + 8*h + g,
 *     four u32 words, word j for 32-block j of the 128-k group; in a word, byte i = element 4*t+i
 *     of the block in its low nibble and element 16+4*t+i in its high nibble, 4-bit two's
 *     complement.
 *   bytes 1024..1279: 64 f32 scales; entry (4*g + j)*2 + h is the scale of row 16*(r/16) + 8*h + g,
 *     32-block j of the 128-k group.
 * xn_mm_q4_packed_bytes gives the buffer size (pad rows are zero).
 * ------------------------------------------------------------------------------------------ */
size_t xn_mm_q4_packed_bytes(size_t n, size_t k);

/* Device: quantize + pack W (dtype f32/f16/bf16, row-major [n,k]) into q4 tiles. */
int xn_mm_quantize_weights_q4(void *wq_packed, const void *w, xn_dtype dtype, size_t n, size_t k,
                              void *stream);
/* Host: logical int8 values in [-7,7] and f32 block scales, both row-major ([n,k], [n,k/32])
 * <-> q4 tiles. */
int xn_mm_pack_q4_host(uint8_t *wq_packed, const int8_t *q, const float *scales, size_t n, size_t k);
int xn_mm_unpack_q4_host(int8_t *q, float *scales, const uint8_t *wq_packed, size_t n, size_t k);

/* Device: dynamic per-row int8 activation quantization of x [m,k] (dtype f32/f16/bf16). */
int xn_mm_quantize_rows_i8(int8_t *xq, float *x_scale, const void *x, xn_dtype dtype, size_t m,
                           size_t k, void *stream);

/* Device: y [m,n] f32 = int4 linear as specified above.  partials (optional, may be NULL)
 * receives the int32 block sums as [m][n][k/32].  Any m >= 1.  Up to 159 rows (and whenever partials is
 * given) the rows are processed 16 at a time with the weights streamed once per 16 rows; from 160 rows on the
 * tiles are unpacked once into library scratch (row-major int8 + block scales) and one launch of a
 * tensor-memory kernel (tcgen05.mma kind::i8, one exact int32 block sum per MMA, scaled in f32 per block)
 * serves all rows.  Same arithmetic on both routes; the f32 sum over the blocks may differ in order.
 * xn_mm_linear_q8 below does the same. */
int xn_mm_linear_q4(float *y, const int8_t *xq, const float *x_scale, const void *wq_packed, size_t m,
                    size_t n, size_t k, int32_t *partials, void *stream);

/* The same linear for a caller whose activations and results live in host memory (pinned, for the copies to
 * be asynchronous): one call enqueues x_host [m,k] f32 -> device, the per-row int8 quantizer, the linear and
 * y [m,n] f32 -> y_host on `stream`.  `workspace` is caller-owned device memory of
 * xn_mm_linear_q4_host_workspace_bytes(m,n,k) bytes (256-byte aligned, reusable by every call on the stream);
 * y_host is valid once the stream has been synchronised.  No counterpart in the reference. */
size_t xn_mm_linear_q4_host_workspace_bytes(size_t m, size_t n, size_t k);
int xn_mm_linear_q4_host(float *y_host, const float *x_host, const void *wq_packed, size_t m, size_t n, size_t k,
                         void *workspace, size_t workspace_bytes, void *stream);

/* int8 block-quantized weights: the same scheme with scale = max|w|/127 and one byte per weight.
 * "q8 tiles": tile (r/16, kk/128) is 2304 bytes, ordered [r/16][kk/128]; bytes 0..2047 = for each
 * 32-block j (512 bytes) and each lane 4*g + t (16 bytes) the four MMA A-operand words
 * {row g, k 4t..4t+3}, {row g+8, k 4t..}, {row g, k 16+4t..}, {row g+8, k 16+4t..}; bytes
 * 2048..2303 = 64 f32 scales laid out as in the q4 tiles. */
size_t xn_mm_q8_packed_bytes(size_t n, size_t k);
int xn_mm_quantize_weights_q8(void *wq_packed, const void *w, xn_dtype dtype, size_t n, size_t k,
                              void *stream);
int xn_mm_pack_q8_host(uint8_t *wq_packed, const int8_t *q, const float *scales, size_t n, size_t k);
int xn_mm_unpack_q8_host(int8_t *q, float *scales, const uint8_t *wq_packed, size_t n, size_t k);
int xn_mm_linear_q8(float *y, const int8_t *xq, const float *x_scale, const void *wq_packed, size_t m,
                    size_t n, size_t k, int32_t *partials, void *stream);

/* ------------------------------------------------------------------------------------------
 * fp8-e4m3 weights with one f32 scale per output channel.  No counterpart in the reference.
 *   scale[j] = max_p |w[j,p]| / 448 ; wq = e4m3_rn_satfinite(w / scale)   (row-major [n,k] bytes)
 *   y[i,j]   = bf16( scale[j] * sum_p x[i,p] * wq[j,p] ),  f32 accumulation
 * Activations reach the fp8 tensor-core path as e4m3 pieces of x / s_i, s_i a power of two
 * with max|x_i| / s_i in (224, 448]:  hi = e4m3(x/s), lo = e4m3(x/s - hi).
 *   variant 0 ("W8A16"): hi and lo are both used; x = s*(hi+lo) holds exactly for every
 *                        bf16 x within 2^-11 of the row maximum and to 2^-10 * s otherwise.
 *   variant 1 ("W8A8"):  hi only.
 * ------------------------------------------------------------------------------------------ */
int xn_mm_quantize_weights_fp8(uint8_t *wq, float *w_scale, const void *w, xn_dtype dtype,
                               size_t n, size_t k, void *stream);
int xn_mm_split_rows_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, const void *x,
                          xn_dtype dtype, size_t m, size_t k, void *stream);
/* x_lo == NULL selects variant 1. y is bf16 [m,n]. */
int xn_mm_linear_fp8_pieces(void *y_bf16, const uint8_t *x_hi, const uint8_t *x_lo,
                            const float *x_scale, const uint8_t *wq, const float *w_scale,
                            size_t m, size_t n, size_t k, void *stream);
/* Column-parallel prefill (no counterpart in the reference, which has no multi-GPU path): this rank
 * owns output channels [col_offset, col_offset + n) of an [m, ldy] result and writes its slice into
 * every one of the num_dst (<= 8) destination buffers -- its own and its peers', mapped into this
 * process (CUDA IPC / symmetric memory) -- with plain stores from the GEMM epilogue, so the
 * "all-gather" travels over NVLink tile by tile while the tensor cores work on the next tile.
 * The caller synchronises the ranks before the result is read. */
int xn_mm_linear_fp8_pieces_scatter(void *const *y_dsts, size_t num_dst, size_t ldy, size_t col_offset,
                                    const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale,
                                    const uint8_t *wq, const float *w_scale, size_t m, size_t n, size_t k,
                                    void *stream);
/* The same slice written through ONE address: y_multicast is an NVLink multicast (NVLS) mapping of the ranks'
 * [m, ldy] buffers (cuMulticast* / a symmetric-memory allocation's multicast pointer); the epilogue issues
 * multimem.st, NVSwitch replicates each 16-byte store into every GPU bound to the object, and the rank sends its
 * slice once instead of once per peer.  n, col_offset and ldy must be multiples of 8.  Stores only: nothing is
 * loaded through the multicast address.  The caller synchronises the ranks before the result is read. */
int xn_mm_linear_fp8_pieces_multicast(void *y_multicast, size_t ldy, size_t col_offset, const uint8_t *x_hi,
                                      const uint8_t *x_lo, const float *x_scale, const uint8_t *wq,
                                      const float *w_scale, size_t m, size_t n, size_t k, void *stream);
/* Convenience: split + linear.  workspace must hold xn_mm_linear_fp8_workspace_bytes(m,k). */
size_t xn_mm_linear_fp8_workspace_bytes(size_t m, size_t k);
int xn_mm_linear_fp8(void *y_bf16, const void *x_bf16, const uint8_t *wq, const float *w_scale,
                     size_t m, size_t n, size_t k, int variant, void *workspace,
                     size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * Row operations around the matmuls of a decoder step, with the reference's semantics (f32 math on
 * widened elements, rounded to the element type where the reference rounds).  Contiguous rows.
 *   rms_norm   Backend::rms_norm, xn-core/src/cpu_backend.rs:766-784 (cuda-kernels/reduce.cu:139-181)
 *   softmax    Backend::softmax,  xn-core/src/cpu_backend.rs:742-764 (reduce.cu:185-225)
 *   silu_mul   Mlp::Gating's silu(x1) * x2 over the two halves of a [rows, 2*hidden] tensor,
 *              xn-moshi/src/transformer.rs:239-245 (silu: xn-core/src/cpu_backend.rs:216-218)
 *   add        the residual add (binary Add), xn-moshi/src/batched_transformer.rs:259,266
 *   kv_append  ScatteredKvCache::append = scatter_set along the context axis of a
 *              (batch, heads, context, head_dim) cache, xn-core/src/models/kv_cache.rs:352-366;
 *              src is (batch, heads, 1, head_dim) with a batch stride of src_batch_stride elements
 *              (a narrow()-ed view of the fused qkv projection), index[b] the context slot of stream b
 * ------------------------------------------------------------------------------------------ */
int xn_mm_rms_norm(xn_dtype dtype, void *dst, const void *src, const void *alpha, size_t rows, size_t cols,
                   float eps, void *stream);
int xn_mm_softmax(xn_dtype dtype, void *dst, const void *src, size_t rows, size_t cols, void *stream);
int xn_mm_silu_mul(xn_dtype dtype, void *dst, const void *src, size_t rows, size_t hidden, void *stream);
int xn_mm_add(xn_dtype dtype, void *dst, const void *a, const void *b, size_t len, void *stream);
/* dst[r][c] = src[r][c] + bias[c] (dst may alias src): the broadcast_add of Linear::forward's bias,
 * xn-core/src/nn/linear.rs:61-64. */
int xn_mm_add_bias(xn_dtype dtype, void *dst, const void *src, const void *bias, size_t rows, size_t cols, void *stream);
int xn_mm_kv_append(xn_dtype dtype, void *cache, const void *src, size_t src_batch_stride, const int64_t *index,
                    size_t batch, size_t heads, size_t context, size_t head_dim, void *stream);

/* Causal attention probabilities for a block of t_rows query rows per batch entry against `context` keys, the last
 * t_rows of which are the block's own: dst[b][i][j] = softmax_j(T(src[b][i][j] * scale)) over j <= i + (context -
 * t_rows), 0 beyond -- the scale -> +mask -> softmax sequence of the unfused attention
 * (xn-moshi/src/batched_transformer.rs:176-189, mask as IndicesAndMask builds it) in one pass, with the same
 * roundings to the element type.  src / dst: [batch, t_rows, context] contiguous (batch = streams x heads); dst may
 * be src.  Only the visible part of src is read.  The zeros are written up to the end of the row's 128-row tile
 * horizon, ((i / 128) + 1) * 128 + (context - t_rows) -- what xn_mm_gemm_causal mode 2 reads -- when
 * zero_fill_all == 0, over the whole row otherwise. */
int xn_mm_softmax_causal(xn_dtype dtype, void *dst, const void *src, size_t batch, size_t t_rows, size_t context,
                         float scale, int zero_fill_all, void *stream);
/* All-gather of a locally computed slice (no counterpart in the reference): copies src, [m] rows of row_bytes bytes
 * laid out [groups][m][row_bytes / groups] (groups = 1: plain row-major; groups = heads: the (heads, tokens, head_dim)
 * output of a batched attention matmul), into bytes [col_offset_bytes, col_offset_bytes + row_bytes) of every row of
 * each of the num_dst destination buffers (row pitch ldy_bytes) -- the rank's own and its peers', mapped into this
 * process.  multicast != 0: dsts[0] is an NVLink multicast address and every 16-byte piece is one multimem.st.
 * Everything in multiples of 16 bytes.  The caller synchronises the ranks before the result is read. */
int xn_mm_scatter_columns(void *const *dsts, size_t num_dst, int multicast, size_t ldy_bytes, size_t col_offset_bytes,
                          const void *src, size_t m, size_t row_bytes, size_t groups, void *stream);

/* Fusions with no counterpart in the reference (it runs every op as its own kernel):
 * the norm / the gating write the e4m3 activation pieces (and power-of-two row scale) of the next
 * fp8 linear directly -- identical to running the plain op and then xn_mm_split_rows_e4m3;
 * x_lo may be NULL (W8A8), dst_or_null additionally receives the rounded row. */
int xn_mm_rms_norm_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *dst_or_null, const void *src,
                              const void *alpha, xn_dtype dtype, size_t rows, size_t cols, float eps, void *stream);
int xn_mm_silu_mul_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, const void *src, xn_dtype dtype,
                              size_t rows, size_t hidden, void *stream);
/* Residual add fused into the next norm: sum_out = a + b (rounded like xn_mm_add; sum_out may alias a or b),
 * then the pieces of rms_norm(sum_out) as above -- identical to xn_mm_add followed by
 * xn_mm_rms_norm_split_e4m3, in one launch and one pass less over the row. */
int xn_mm_add_rms_norm_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *sum_out, const void *a,
                                  const void *b, const void *alpha, xn_dtype dtype, size_t rows, size_t cols, float eps,
                                  void *stream);
/* Single-token attention in one pass over the cache: replaces q.matmul_t(k) -> scale -> +mask ->
 * softmax -> matmul(v) (xn-moshi/src/batched_transformer.rs:174-190) for T = 1.  q: (batch, heads,
 * 128) bf16 with a batch stride of q_batch_stride elements; out: contiguous (batch, heads, 128) bf16;
 * caches (batch, heads, context, 128) bf16; mask (optional) f32
 * [batch, context], added to the scaled scores (0 / -inf as IndicesAndMask builds it).  f32 math. */
int xn_mm_decode_attention(void *out_bf16, const void *q_bf16, size_t q_batch_stride, const void *k_cache_bf16,
                           const void *v_cache_bf16, const float *mask_or_null, size_t batch, size_t heads,
                           size_t context, size_t head_dim, float scale, void *stream);
/* The same attention with the context cut into slices handled by different CTAs and merged by a
 * log-sum-exp combine: with few streams one CTA per (stream, head) leaves most of the GPU idle (8 streams
 * x 32 heads = 256 CTAs of 128 threads on 148 SMs).  The number of slices is chosen inside (1 when
 * batch * heads already fills the machine: then this is xn_mm_decode_attention).  `workspace` holds the
 * slices' partial results: xn_mm_decode_attention_workspace_bytes(batch, heads, context) bytes of device
 * memory (may be 0), owned by the caller and reusable by every call on the same stream. */
size_t xn_mm_decode_attention_workspace_bytes(size_t batch, size_t heads, size_t context);
int xn_mm_decode_attention_split(void *out_bf16, const void *q_bf16, size_t q_batch_stride, const void *k_cache_bf16,
                                 const void *v_cache_bf16, const float *mask_or_null, size_t batch, size_t heads,
                                 size_t context, size_t head_dim, float scale, void *workspace, size_t workspace_bytes,
                                 void *stream);

/* xn_mm_decode_attention_split followed by xn_mm_split_rows_e4m3 of its [batch, heads * 128] output, with the merge of
 * the context slices and the e4m3 split of the row fused into one launch (the attention output is the activation
 * of the output projection): identical results, one launch and one pass over the row less.  out_bf16 still
 * receives the attention output. */
int xn_mm_decode_attention_split_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *out_bf16, const void *q_bf16,
                                      size_t q_batch_stride, const void *k_cache_bf16, const void *v_cache_bf16,
                                      const float *mask_or_null, size_t batch, size_t heads, size_t context,
                                      size_t head_dim, float scale, void *workspace, size_t workspace_bytes,
                                      void *stream);

/* One launch for what a decode layer does between its input and output projections
 * (xn-moshi/src/batched_transformer.rs:136-160 with xn-core/src/models/kv_cache.rs:352-366): xn_mm_kv_append2 of the
 * new key / value rows (k_new, v_new: [batch, heads * 128] bf16 rows qkv_batch_stride elements apart, appended at
 * context index index[batch]; an index outside [0, context) appends nothing), xn_mm_decode_attention_split over the
 * caches with q taken at the same batch stride, the merge of the context slices and the e4m3 split of the output row,
 * with results identical to the three separate calls.  x_hi / x_lo / x_scale may all be null (no pieces wanted).
 * merge: where the merge of the slices and the split run -- 1 = inside the attention kernel (one launch: the CTA that
 * arrives last at a (stream, head) merges, the one that finishes a stream's last head splits the row), 2 = as a second
 * launch, 0 = the library decides (inside when every resident slot sees at most two CTAs; with many short slices the
 * fence and arrival at the end of every CTA cost more than the second launch).
 * workspace: xn_mm_decode_attention_append_workspace_bytes(batch, heads, context) bytes of device memory owned by the
 * caller; the arrival counters of the merge live in the library's per-stream scratch, so calls on one device must be
 * stream-ordered with the other calls that use that scratch. */
size_t xn_mm_decode_attention_append_workspace_bytes(size_t batch, size_t heads, size_t context);
int xn_mm_decode_attention_append_e4m3(uint8_t *x_hi, uint8_t *x_lo, float *x_scale, void *out_bf16, const void *q_bf16,
                                       const void *k_new_bf16, const void *v_new_bf16, size_t qkv_batch_stride,
                                       void *k_cache_bf16, void *v_cache_bf16, const int64_t *index,
                                       const float *mask_or_null, size_t batch, size_t heads, size_t context,
                                       size_t head_dim, float scale, int merge, void *workspace, size_t workspace_bytes,
                                       void *stream);
/* xn_mm_kv_append for the key and the value cache in one launch (same index, same source layout). */
int xn_mm_kv_append2(xn_dtype dtype, void *k_cache, void *v_cache, const void *k_src, const void *v_src,
                     size_t src_batch_stride, const int64_t *index, size_t batch, size_t heads, size_t context,
                     size_t head_dim, void *stream);

/* Allocation-free form of xn_mm_linear_fp8.  It has no counterpart in the reference.  For hosts
 * that must not (or cannot) allocate device memory at call time -- a serving loop whose device
 * budget belongs to another allocator, a real-time audio callback that cannot afford a
 * synchronising cudaMalloc, an embedder barred from the CUDA allocator.  The scratch for the
 * activation pieces is a fixed 513 KiB array inside the library image (held by every GPU that loads
 * the library until the process exits), so sizes are limited to m <= 64 and
 * m*k <= xn_mm_linear_fp8_noalloc_max_elems() (262144); larger calls return XN_ERR_UNSUPPORTED.
 * All calls on a device share that array: calls that overlap on the GPU race, so keep them in one
 * stream order.  The first call on a device resolves the array's device address and should be made
 * outside any stream capture; `stream` must belong to the device that is current at the call (the array
 * is looked up for the current device).  Every argument is checked before anything is enqueued, so a
 * rejected call leaves the shared array untouched.  A device-side wait that runs out inside this call is
 * still bounded, but it is reported to xn_mm_device_status only if some other entry point has already
 * set up the device's status word (this one must not allocate it).  It runs only kernels that need no scratch of their own (the
 * weight-streaming kernel up to 32 rows, the tiled tensor-memory kernel beyond), so from 9 rows on its
 * results can differ from xn_mm_linear_fp8 in the last bf16 bit (another summation order). */
size_t xn_mm_linear_fp8_noalloc_max_elems(void);
int xn_mm_linear_fp8_noalloc(void *y_bf16, const void *x_bf16, const uint8_t *wq, const float *w_scale,
                             size_t m, size_t n, size_t k, int variant, void *stream);

/* --------------------------------------------------------------------------------------------
 * Convolutions as implicit GEMMs.  Argument lists of Backend::conv1d / Backend::conv_transpose1d
 * (xn-core/src/backend.rs:275-316) plus an optional bias the reference adds as a separate
 * broadcast_add (xn-core/src/ops.rs:253-300, 305-350); replaces the im2col -> gemm -> transpose and
 * transpose -> gemm -> col2im lowerings of xn-core/src/cuda_backend.rs:1376-1488, 1490-1561,
 * 1783-1856 and their direct fallbacks, for every groups / padding / dilation value.
 *   src    (batch, in_channels, length), contiguous
 *   kernel conv1d: (out_channels, in_channels/groups, kernel_size)
 *          conv_transpose1d: (in_channels, out_channels/groups, kernel_size)
 *   bias   (out_channels) or NULL
 *   dst    (batch, out_channels, out_length), contiguous; out_length must be
 *          (length + 2*padding - dilation*(kernel_size-1) - 1)/stride + 1, respectively
 *          (length-1)*stride + kernel_size + output_padding - 2*padding, as the reference computes it
 * Accumulation is f32 with one rounding to dtype (f32 operands: products to about 1e-6 relative,
 * exact on small integers).
 * workspace: calls with groups == 1, dilation == 1 and in_channels a multiple of 8 (f16 / bf16) or 4 (f32,
 * computed as three tf32 pieces per operand) run on the
 * tensor-memory GEMM kernel over a channels-last copy of the input and repacked taps, which live in
 * caller-owned device scratch of xn_mm_conv*_workspace_bytes(...) bytes (256-byte aligned, reusable by
 * every call on the same stream; XN_ERR_WORKSPACE when absent or too small).  Every other call needs no
 * scratch: the size function returns 0 and workspace may be NULL.
 * ------------------------------------------------------------------------------------------ */
size_t xn_mm_conv1d_workspace_bytes(xn_dtype dtype, size_t batch, size_t in_channels, size_t out_channels, size_t length,
                                    size_t kernel_size, size_t stride, size_t padding, size_t dilation, size_t groups);
int xn_mm_conv1d(xn_dtype dtype, void *dst, const void *src, const void *kernel, const void *bias_or_null,
                 size_t batch, size_t in_channels, size_t out_channels, size_t length, size_t out_length,
                 size_t kernel_size, size_t stride, size_t padding, size_t dilation, size_t groups, void *workspace,
                 size_t workspace_bytes, void *stream);
size_t xn_mm_conv_transpose1d_workspace_bytes(xn_dtype dtype, size_t batch, size_t in_channels, size_t out_channels,
                                              size_t length, size_t kernel_size, size_t stride, size_t padding,
                                              size_t output_padding, size_t groups);
int xn_mm_conv_transpose1d(xn_dtype dtype, void *dst, const void *src, const void *kernel, const void *bias_or_null,
                           size_t batch, size_t in_channels, size_t out_channels, size_t length, size_t out_length,
                           size_t kernel_size, size_t stride, size_t padding, size_t output_padding, size_t groups,
                           void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* XN_MM_H */
