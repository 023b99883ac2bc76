// Dense tensor-core GEMM for the `matmul_t` form, D[M,N] = A[M,K] * B[N,K]^T with both operands
// K-contiguous -- the shape every Linear::forward produces (xn-core/src/nn/linear.rs:56-66), which
// the reference sends to cublasGemmStridedBatchedEx (xn-core/src/cuda_backend.rs:2109-2133).
// Written for sm_100a: TMA (cp.async.bulk.tensor, no multicast) stages 128-byte-swizzled tiles in
// shared memory, one elected thread issues tcgen05.mma with the accumulators in tensor memory, and
// the epilogue warps read them back with tcgen05.ld.
//
//   warp 0      producer: TMA loads into a ring of NSTAGE stages, mbarrier full/empty pairs
//   warp 1      tensor-memory allocation; MMA issue; tcgen05.commit releases stages / publishes tiles
//   warps 2..9  epilogue: TMEM -> registers -> scale/convert -> shared-memory transpose -> global (each warp owns
//               the 32 TMEM lanes of its warp-id-mod-4 quarter and half of the tile's columns; the tf32 kind,
//               whose epilogue keeps a row of the tile in registers, runs with warps 2..5 only)
//
// The kernel is persistent (grid = #SMs, tiles round-robin) and keeps two accumulator buffers in
// TMEM so the epilogue of one tile overlaps the MMAs of the next.
//
// Operand kinds
//   FP8 pieces: A is one (W8A8) or two (W8A16: hi + lo) e4m3 matrices, B the e4m3 weights;
//               kind::f8f6f4, the two pieces accumulate into the same TMEM tile, the epilogue
//               applies x_scale[m] * w_scale[n] and rounds to bf16.
//   BF16 / F16: kind::f16, the epilogue rounds the f32 accumulator to the element type.
//   TF32 pieces: kind::tf32 on f32 words already on the tf32 grid, f32 out.  Callers carry f32 precision by
//               laying three such pieces per operand along k (gemm_f32_tc.cu, conv1d.cu).  The accumulator is
//               handed to the epilogue every 2 k stages and summed in registers, because tcgen05
//               accumulates with truncation (see KCH in the kernel); tiles are at most 128 columns wide.
// Batches: a third tensor-map dimension (strided-batched and grouped calls, split-k chunks), optionally with
// one A matrix shared by every batch entry (the convolutions' packed taps) and a per-row bias.
//
// Every mbarrier wait is bounded in time (wait.cuh); a wait that gives up reports it through the device's
// host-visible status word and the CTA drains through its common exit (tensor memory is always released).
#include <cuda.h>

#include "common.cuh"
#include "wait.cuh"

namespace xn {
namespace {

constexpr int BM = 128;        // rows of A per tile = TMEM lanes
constexpr int BKB = 128;       // bytes of K per stage = one 128-byte swizzle atom
constexpr int UMMA_KB = 32;    // bytes of K per tcgen05.mma (32 x 8-bit or 16 x 16-bit)
constexpr int NTHREADS = 192;
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
// Pull a tensor map (a kernel parameter) into the TMA unit's descriptor cache: the first copy that names it then
// does not start with a fetch of the descriptor.
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_only(uint64_t *b, unsigned bytes) {  // no arrival
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t *b, unsigned parity, const WaitCtx &w) {
    return mbar_wait_bounded(smem_u32(b), parity, w);
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(const void *tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)0 << 16;                             // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                             // descriptor version
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}

// The same for an MN-major operand (the [K, N] right-hand side of a plain `matmul`, n contiguous): the tile is a
// row of 64-column blocks, each block = BK k-rows of 128 bytes as TMA writes them with the 128-byte swizzle.
// Within a block the 8-row groups along k are 1024 bytes apart (stride byte offset), the blocks along n
// `block_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_mn(const void *tile, unsigned block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFFu) >> 4);
    d |= (uint64_t)(block_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: D = f32, A/B formats, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int a_fmt, int b_fmt, int n) {
    return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

template <bool F8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    if (F8)
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
            : "memory");
    else
        asm volatile(
            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
            : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// issue only: the caller waits once for all its loads
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31,%32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Tile order within one batch entry.  Tiles that run at the same time (148 consecutive indices) should share as
// many operand panels as possible, or every wave re-reads both operands from HBM (at 8192^3 the plain m-fastest
// order reads 4 GB for 0.4 GB of operands and the kernel becomes bandwidth-bound).  The m blocks are cut into
// groups of group_m; inside a group m runs fastest and every n block is visited before the next group starts, so
// a wave covers about group_m x (148 / group_m) tiles and the group's A panels stay in L2 while B streams once.
__device__ __forceinline__ void tile_coords(int tin, int num_m, int num_n, int group_m, int &m_blk, int &n_blk) {
    const int per_group = group_m * num_n;
    const int grp = tin / per_group, first_m = grp * group_m;
    const int gm = min(num_m - first_m, group_m);
    const int r = tin - grp * per_group;
    n_blk = r / gm;
    m_blk = first_m + (r - n_blk * gm);
}

constexpr int MAX_DST = 8;
struct GemmArgs {
    void *y[MAX_DST];     // ndst destinations for the [M, N] result (own buffer and, in the column-parallel
                          // prefill, the peers' buffers mapped into this process); row stride ldy elements
    int ndst;
    int col_offset;       // first output column inside each destination row
    const float *x_scale; // FP8 only: per activation row
    const float *w_scale; // FP8 only: per output channel
    int M, N, K;          // K in elements
    int ldy;
    int batch;            // strided-batched / grouped form: `batch` independent problems in one launch
    long long y_batch_stride;  // elements between consecutive outputs (m * n in Backend::gemm)
    int a_batch_inner, b_batch_inner;  // the tensor map's dimension order is (k, batch, rows) instead of (k, rows, batch)
    int a_bcast;          // every batch entry multiplies the same A matrix (the A map then holds one matrix)
    const void *row_bias; // optional, not for fp8: added to every element of output row i (element type of y)
    const void *col_bias; // optional, 16-bit kinds: bias[j] (element type of y) added to the ROUNDED product of column j and
                          // rounded again -- nn::Linear's matmul followed by broadcast_add, bit for bit
    WaitCtx wait;         // bound and status word of the kernel's mbarrier waits
    int group_m;          // m blocks per rasterisation group (see tile_coords)
    int causal, causal_off;  // causal attention (16-bit kinds): 1 = q.k^T, tiles whose keys all lie beyond the last query row's
                          // horizon (key j visible to row i iff j <= i + causal_off) are skipped and left unwritten; 2 = p.v, the k
                          // loop of a row tile stops at that horizon (the probabilities beyond it are zero and never read)
    int mc;               // y[0] is an NVLink multicast address: one multimem.st per 16 bytes reaches every GPU's copy
    int b_mn;             // 16-bit kinds: B is [K, N] with n contiguous (MN-major); its map is (n, k, batch), box 64 x BK
    int rows2;            // NA = 2 instantiations: the two A tiles are rows [256 i, +128) and [256 i + 128, +128) of ONE matrix
                          // (a 256 x BN tile: both accumulator buffers belong to one tile, the B stage is read by two MMAs)
    int fast_store;       // one destination, no multicast, and every 16-byte output chunk of an interior tile is aligned
    float *split_out;     // split-k launch: the batch index is a k chunk of ONE product and every tile leaves as an f32
                          // record [chunk][tile][column group of 4][128 rows][4] for splitk_reduce_kernel
};

__device__ __forceinline__ bool tile_masked(const GemmArgs &a, int m_blk, int n_blk, int bn) {
    return a.causal == 1 && n_blk * bn > m_blk * BM + BM - 1 + a.causal_off;
}
__device__ __forceinline__ int tile_kb(const GemmArgs &a, int m_blk, int num_kb, int bk) {
    if (a.causal != 2) return num_kb;
    const int lim = min(a.K, (m_blk + 1) * BM + a.causal_off);
    const int kb = (lim + bk - 1) / bk;
    return kb < 1 ? 1 : min(kb, num_kb);
}

// Epilogue of one output tile for the fp8 / bf16 / f16 kinds.  Eight warps share a tile: warp (q, half) owns the
// 32 accumulator rows of tensor-memory lane quarter q (output rows m_row0 + 32 q ..) and the 32-column chunks
// [c_begin, c_end) of buffer `acc`.  Two chunks at a time are loaded together, scaled / biased, rounded to the
// output type, transposed through the warp's 4 KB shared-memory slab (16-byte pieces XOR-swizzled by row) and
// stored as 128-byte row segments into every destination.  With one warp per scheduler the epilogue of a
// 128 x 256 tile took 4.7 us -- a chain of dependent instructions with nothing to overlap it -- which bounded every
// product with few k stages per tile (attention's q.k^T: two stages); two warps per scheduler and both
// tensor-memory loads of a group in flight bring it under the time of four k stages.
constexpr int EPI_WARPS_16 = 8;  // epilogue warps of the fp8 / 16-bit kinds (the tf32 kind keeps four)
template <int KIND, int BN>
__device__ __forceinline__ void epilogue_tile(const GemmArgs &args, uint32_t tmem_base, int acc, int q, int lane, int m_row0,
                                              int n_blk, int g, unsigned char *slab, int c_begin, int c_end) {
    constexpr bool F8 = KIND == 0;
    if (args.split_out) {
        // raw f32 accumulators, a lane's row of every 4-column group next to its neighbours' rows: 512 contiguous
        // bytes per warp store; scales, bias and rounding belong to the reduction over the chunks
        const int num_n = (args.N + BN - 1) / BN, num_m = (args.M + BM - 1) / BM;
        const size_t t = (size_t)g * num_m * num_n + (size_t)(m_row0 / BM) * num_n + n_blk;
        float *rec = args.split_out + t * (size_t)(BN * BM) + (size_t)(q * 32 + lane) * 4;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
            uint32_t v[32];
            tmem_ld32(taddr + c * 32, v);
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4)
                *reinterpret_cast<float4 *>(rec + (size_t)(c * 8 + j4) * (BM * 4)) =
                    make_float4(__uint_as_float(v[4 * j4]), __uint_as_float(v[4 * j4 + 1]), __uint_as_float(v[4 * j4 + 2]),
                                __uint_as_float(v[4 * j4 + 3]));
        }
        return;
    }
    const int row = m_row0 + q * 32 + lane;
    float xs = 1.0f;
    if (F8 && row < args.M) xs = __ldg(args.x_scale + row);
    float rb = 0.0f;
    if (!F8 && args.row_bias && row < args.M)
        rb = KIND == 2 ? __half2float(reinterpret_cast<const __half *>(args.row_bias)[row])
                       : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(args.row_bias)[row]);
    // Interior tiles of a plain single-destination launch (the host has checked the 16-byte alignment of every
    // row segment) take a lean store loop: one address per warp and tile, no per-store bounds or alignment tests.
    const bool fast = args.fast_store && m_row0 + BM <= args.M && (n_blk + 1) * BN <= args.N;
    uint16_t *warp_out = reinterpret_cast<uint16_t *>(args.y[0]) + (size_t)g * args.y_batch_stride +
                         (size_t)(m_row0 + q * 32) * args.ldy + args.col_offset + n_blk * BN;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end; c0 += 2) {
        const int nch = c_end - c0 < 2 ? 1 : 2;   // 32-column chunks in this group
        const int cpr = nch * 4;                  // 16-byte pieces per slab row
        const int row_bytes = nch * 64;
        uint32_t v[2][32];
        tmem_ld32_nowait(lane_addr + c0 * 32, v[0]);
        if (nch == 2) tmem_ld32_nowait(lane_addr + c0 * 32 + 32, v[1]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (h >= nch) break;
            const int col0 = n_blk * BN + (c0 + h) * 32;
            uint32_t packed[16];
            if (F8 && fast) {
                const float4 *ws4 = reinterpret_cast<const float4 *>(args.w_scale + col0);
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 w = __ldg(ws4 + j4);
                    const float f0 = w.x * (xs * __uint_as_float(v[h][4 * j4])), f1 = w.y * (xs * __uint_as_float(v[h][4 * j4 + 1]));
                    const float f2 = w.z * (xs * __uint_as_float(v[h][4 * j4 + 2])), f3 = w.w * (xs * __uint_as_float(v[h][4 * j4 + 3]));
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(f0, f1), h1 = __floats2bfloat162_rn(f2, f3);
                    packed[2 * j4] = *reinterpret_cast<uint32_t *>(&h0);
                    packed[2 * j4 + 1] = *reinterpret_cast<uint32_t *>(&h1);
                }
            } else if (F8) {  // edge tile or unaligned scales: one guarded scale load per column
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int i0 = min(col0 + 2 * j, args.N - 1), i1 = min(col0 + 2 * j + 1, args.N - 1);
                    const float f0 = __ldg(args.w_scale + i0) * (xs * __uint_as_float(v[h][2 * j]));
                    const float f1 = __ldg(args.w_scale + i1) * (xs * __uint_as_float(v[h][2 * j + 1]));
                    __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
                    packed[j] = *reinterpret_cast<uint32_t *>(&hh);
                }
            } else if (!args.col_bias) {  // plain product (rb is zero without a row bias): one conversion per pair
                // (the branches on the kind of epilogue are taken once per chunk, outside the unrolled loops: tested
                // per element they cost more than the conversions themselves)
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float f0 = __uint_as_float(v[h][2 * j]) + rb, f1 = __uint_as_float(v[h][2 * j + 1]) + rb;
                    if (KIND == 2) {
                        __half2 hh = __floats2half2_rn(f0, f1);
                        packed[j] = *reinterpret_cast<uint32_t *>(&hh);
                    } else {
                        __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
                        packed[j] = *reinterpret_cast<uint32_t *>(&hh);
                    }
                }
            } else {  // nn::Linear's bias: added to the rounded product, rounded again
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float f0 = __uint_as_float(v[h][2 * j]) + rb, f1 = __uint_as_float(v[h][2 * j + 1]) + rb;
                    const int i0 = min(col0 + 2 * j, args.N - 1), i1 = min(col0 + 2 * j + 1, args.N - 1);
                    if (KIND == 2) {
                        const __half *cb = reinterpret_cast<const __half *>(args.col_bias);
                        const float2 r = __half22float2(__floats2half2_rn(f0, f1));
                        __half2 hh = __floats2half2_rn(r.x + __half2float(cb[i0]), r.y + __half2float(cb[i1]));
                        packed[j] = *reinterpret_cast<uint32_t *>(&hh);
                    } else {
                        const __nv_bfloat16 *cb = reinterpret_cast<const __nv_bfloat16 *>(args.col_bias);
                        const float2 r = __bfloat1622float2(__floats2bfloat162_rn(f0, f1));
                        __nv_bfloat162 hh = __floats2bfloat162_rn(r.x + __bfloat162float(cb[i0]), r.y + __bfloat162float(cb[i1]));
                        packed[j] = *reinterpret_cast<uint32_t *>(&hh);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int piece = (h * 4 + j) ^ (lane & (cpr - 1));
                *reinterpret_cast<uint4 *>(slab + lane * row_bytes + piece * 16) =
                    make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
            }
        }
        __syncwarp();
        const int sub = lane / cpr, pc = lane % cpr;  // this lane's row within a store instruction, 16-byte piece
        const int rpi = 32 / cpr;                     // rows written per store instruction
        if (fast) {
            uint16_t *p = warp_out + (size_t)sub * args.ldy + c0 * 32 + pc * 8;
            const size_t step = (size_t)rpi * args.ldy;
#pragma unroll 4
            for (int r = sub; r < 32; r += rpi) {
                *reinterpret_cast<uint4 *>(p) = *reinterpret_cast<const uint4 *>(slab + r * row_bytes + ((pc ^ (r & (cpr - 1))) * 16));
                p += step;
            }
        } else {
#pragma unroll 1
            for (int r = sub; r < 32; r += rpi) {
                const uint4 val = *reinterpret_cast<const uint4 *>(slab + r * row_bytes + ((pc ^ (r & (cpr - 1))) * 16));
                const int grow = m_row0 + q * 32 + r;
                const int gcol = n_blk * BN + c0 * 32 + pc * 8;
                if (grow < args.M && gcol < args.N) {
                    for (int p = 0; p < args.ndst; ++p) {
                        uint16_t *dst = reinterpret_cast<uint16_t *>(args.y[p]) + (size_t)g * args.y_batch_stride +
                                        (size_t)grow * args.ldy + args.col_offset + gcol;
                        if (args.mc) {
                            // the switch replicates the store into every GPU bound to the multicast object (the host
                            // checked that n is a multiple of 8 and the rows are 16-byte aligned)
                            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                                         "f"(__uint_as_float(val.x)), "f"(__uint_as_float(val.y)), "f"(__uint_as_float(val.z)),
                                         "f"(__uint_as_float(val.w))
                                         : "memory");
                        } else if (gcol + 8 <= args.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                            *reinterpret_cast<uint4 *>(dst) = val;
                        } else {
                            const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
                            for (int j = 0; j < 8 && gcol + j < args.N; ++j)
                                dst[j] = (uint16_t)(w4[j >> 1] >> ((j & 1) * 16));
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
}

// KIND: 0 = fp8 pieces -> bf16 out, 1 = bf16 -> bf16, 2 = f16 -> f16, 3 = tf32 operands (f32 words already on
// the tf32 grid) -> f32 out
template <int KIND, int BN, int NA, int NSTAGE>
__global__ void __launch_bounds__(KIND == 3 ? NTHREADS : 64 + 32 * EPI_WARPS_16, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                    const __grid_constant__ CUtensorMap map_b, const GemmArgs args) {
    constexpr bool F8 = KIND == 0;
    constexpr int ELEM = F8 ? 1 : (KIND == 3 ? 4 : 2);
    constexpr int BK = BKB / ELEM;  // K elements per stage
    constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB;
    constexpr int STAGE_BYTES = NA * A_BYTES + B_BYTES;
    // tcgen05 adds into its f32 accumulator with truncation: over n MMAs the result drifts by about n * 3e-8
    // of the running sum (4e-5 at 1536 MMAs, measured).  The tf32 kind, whose callers expect f32 accuracy (an
    // absolute error below 1e-6 of the output's rms at k = 4096), therefore hands the accumulator to the
    // epilogue every KCH k stages (8 MMAs).  The epilogue warps sum the hand-overs in registers in
    // round-to-nearest f32, and every L2_EVERY hand-overs move that block sum into a second-level total kept in
    // tensor memory (columns [2 BN, 3 BN), read and written with tcgen05.ld / tcgen05.st by the warp that owns
    // the lanes), so that no sum ever runs over more than L2_EVERY terms at either level.
    constexpr int KCH = KIND == 3 ? 2 : (1 << 30);
    constexpr int L2_EVERY = 16;
    static_assert(KIND != 3 || BN <= 128, "the tf32 kind keeps BN accumulator registers per epilogue thread");
    constexpr uint32_t IDESC = F8 ? instr_desc(0, 0, BN)
                               : (KIND == 1 ? instr_desc(1, 1, BN) : (KIND == 3 ? instr_desc(2, 2, BN) : instr_desc(0, 0, BN)));
    constexpr int ACC_COLS = (KIND == 3 ? 3 : 2) * BN;  // two accumulator buffers (+ the tf32 kind's second-level total)
    constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : (ACC_COLS <= 256 ? 256 : 512)));

    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *epi_smem = smem + (size_t)NSTAGE * STAGE_BYTES;  // epilogue slabs: 8 x 4 KB (fp8 / 16-bit kinds) or 4 x 8 KB (tf32 kind)
    __shared__ __align__(8) uint64_t full[NSTAGE], empty[NSTAGE], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BMT = (NA == 2 && args.rows2) ? 2 * BM : BM;  // rows of A per tile
    const int num_m = (args.M + BMT - 1) / BMT, num_n = (args.N + BN - 1) / BN;
    const int tiles_per_batch = num_m * num_n;
    const int num_tiles = tiles_per_batch * args.batch;
    const int num_kb = (args.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        prefetch_tmap(&map_a0);
        if (NA == 2) prefetch_tmap(&map_a1);
        prefetch_tmap(&map_b);
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], KIND == 3 ? 4 : EPI_WARPS_16); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    // Programmatic dependent launch: barrier set-up and the tensor-memory allocation above overlap the
    // tail of the previous kernel in the stream; operands and outputs are touched only after this wait.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int it = 0;  // running k-block count across tiles: stage = it % NSTAGE
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int g = tile / tiles_per_batch, tin = tile % tiles_per_batch;
                int m_blk, n_blk;
                tile_coords(tin, num_m, num_n, args.group_m, m_blk, n_blk);
                if (KIND != 3 && tile_masked(args, m_blk, n_blk, BN)) continue;
                const int nkb = KIND != 3 ? tile_kb(args, m_blk, num_kb, BK) : num_kb;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % NSTAGE;
                    const unsigned ph = (unsigned)(it / NSTAGE) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, args.wait)) { ok = false; break; }
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    const int ga = args.a_bcast ? 0 : g;
                    const int ay = args.a_batch_inner ? ga : m_blk * BMT, az = args.a_batch_inner ? m_blk * BMT : ga;
                    const int by = args.b_batch_inner ? g : n_blk * BN, bz = args.b_batch_inner ? n_blk * BN : g;
                    tma_load_3d(st, &map_a0, kb * BK, ay, az, &full[s]);
                    if (NA == 2) {
                        const int second = args.rows2 ? BM : 0;  // the second A tile: the next 128 rows, or the second piece
                        tma_load_3d(st + A_BYTES, &map_a1, kb * BK, args.a_batch_inner ? ay : ay + second,
                                    args.a_batch_inner ? az + second : az, &full[s]);
                    }
                    if (args.b_mn) {
                        // one 64-column block (64 n x BK k, 8 KB) per copy
                        for (int i = 0; i < BN / 64; ++i)
                            tma_load_3d(st + NA * A_BYTES + i * (64 * BKB), &map_b, n_blk * BN + 64 * i,
                                        args.b_batch_inner ? g : kb * BK, args.b_batch_inner ? kb * BK : g, &full[s]);
                    } else {
                        tma_load_3d(st + NA * A_BYTES, &map_b, kb * BK, by, bz, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int it = 0, vt = 0;   // vt: accumulator hand-overs to the epilogue so far (one per tile, or per k chunk)
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int nkb = num_kb;
            if (KIND != 3 && args.causal) {
                int m_blk, n_blk;
                tile_coords(tile % tiles_per_batch, num_m, num_n, args.group_m, m_blk, n_blk);
                if (tile_masked(args, m_blk, n_blk, BN)) continue;
                nkb = tile_kb(args, m_blk, num_kb, BK);
            }
            for (int kb0 = 0; (kb0 < nkb || kb0 == 0) && ok; kb0 += KCH, ++vt) {
                const bool rows2 = NA == 2 && args.rows2;  // both buffers belong to this tile: one barrier pair, phase per tile
                const int acc = rows2 ? 0 : (vt & 1);
                const unsigned acc_ph = rows2 ? ((unsigned)vt & 1u) : ((unsigned)(vt >> 1) & 1u);
                if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u, args.wait)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                const int kend = nkb - kb0 < KCH ? nkb : kb0 + KCH;
                for (int kb = kb0; kb < kend; ++kb, ++it) {
                    const int s = it % NSTAGE;
                    const unsigned ph = (unsigned)(it / NSTAGE) & 1u;
                    if (!mbar_wait(&full[s], ph, args.wait)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    const uint64_t da0 = smem_desc(st), da1 = smem_desc(st + A_BYTES);
                    const bool bmn = ELEM == 2 && args.b_mn;
                    const uint64_t db = bmn ? smem_desc_mn(st + NA * A_BYTES, 64 * BKB) : smem_desc(st + NA * A_BYTES);
                    const uint32_t idesc = bmn ? (IDESC | (1u << 16)) : IDESC;   // bit 16: B is MN-major
                    // k advance per MMA: 32 bytes inside the swizzled row (K-major), 16 k-rows of 128 bytes (MN-major)
                    const uint64_t badv = bmn ? (uint64_t)((UMMA_KB / ELEM) * 128 >> 4) : (uint64_t)(UMMA_KB >> 4);
#pragma unroll
                    for (int ks = 0; ks < BKB / UMMA_KB; ++ks) {
                        const uint64_t adv = (uint64_t)(ks * UMMA_KB >> 4);
                        if constexpr (KIND == 3) {
                            umma_tf32(d_tmem, da0 + adv, db + adv, IDESC, kb > kb0 || ks != 0);
                        } else {
                            umma<F8>(d_tmem, da0 + adv, db + ks * badv, idesc, (kb | ks) != 0);
                            if (NA == 2) umma<F8>(rows2 ? d_tmem + BN : d_tmem, da1 + adv, db + ks * badv, idesc, rows2 ? (uint32_t)((kb | ks) != 0) : 1u);
                        }
                    }
                    umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(&tmem_full[acc]);
            }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int t_local = 0;
        bool ok = true;
        if constexpr (KIND == 3) {
            constexpr int GC = BN % 64 == 0 ? 64 : 32, CPR = GC / 4, RPI = 32 / CPR;
            unsigned char *slab = epi_smem + (size_t)(warp - 2) * 32 * 256;
            int vt = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int g = tile / tiles_per_batch, tin = tile % tiles_per_batch;
                int m_blk, n_blk;
                tile_coords(tin, num_m, num_n, args.group_m, m_blk, n_blk);
                float racc[BN];  // sum of the hand-overs since the last move into the second-level total
#pragma unroll
                for (int i = 0; i < BN; ++i) racc[i] = 0.f;
                const uint32_t l2_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(2 * BN);
                bool l2_live = false;  // the second-level total of this tile has been written
                int since = 0;
                for (int kb0 = 0; (kb0 < num_kb || kb0 == 0) && ok; kb0 += KCH, ++vt) {
                    const int acc = vt & 1;
                    if (!mbar_wait(&tmem_full[acc], (unsigned)(vt >> 1) & 1u, args.wait)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < BN / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 32), v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) racc[c * 32 + i] += __uint_as_float(v[i]);
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[acc]);
                    if (++since == L2_EVERY && kb0 + KCH < num_kb) {
                        since = 0;
#pragma unroll
                        for (int c = 0; c < BN / 32; ++c) {
                            uint32_t v[32];
                            if (l2_live) {
                                tmem_ld32(l2_addr + (uint32_t)(c * 32), v);
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + racc[c * 32 + i]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(racc[c * 32 + i]);
                            }
                            tmem_st32(l2_addr + (uint32_t)(c * 32), v);
#pragma unroll
                            for (int i = 0; i < 32; ++i) racc[c * 32 + i] = 0.f;
                        }
                        l2_live = true;
                    }
                }
                if (!ok) break;
                if (l2_live) {
#pragma unroll
                    for (int c = 0; c < BN / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(l2_addr + (uint32_t)(c * 32), v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) racc[c * 32 + i] += __uint_as_float(v[i]);
                    }
                }
                const int row = m_blk * BM + q * 32 + lane;
                const float rb = (args.row_bias && row < args.M) ? reinterpret_cast<const float *>(args.row_bias)[row] : 0.f;
#pragma unroll
                for (int g0 = 0; g0 < BN; g0 += GC) {
#pragma unroll
                    for (int j = 0; j < GC / 4; ++j) {
                        const int chunk = j ^ (lane & (CPR - 1));
                        *reinterpret_cast<float4 *>(slab + lane * (GC * 4) + chunk * 16) =
                            make_float4(racc[g0 + 4 * j] + rb, racc[g0 + 4 * j + 1] + rb, racc[g0 + 4 * j + 2] + rb,
                                        racc[g0 + 4 * j + 3] + rb);
                    }
                    __syncwarp();
                    const int sub = lane / CPR, ch = lane % CPR;
#pragma unroll 1
                    for (int r0 = 0; r0 < 32; r0 += RPI) {
                        const int r = r0 + sub;
                        const uint4 val = *reinterpret_cast<const uint4 *>(slab + r * (GC * 4) + ((ch ^ (r & (CPR - 1))) * 16));
                        const int grow = m_blk * BM + q * 32 + r;
                        const int gcol = n_blk * BN + g0 + ch * 4;
                        if (grow < args.M && gcol < args.N) {
                            uint32_t *dst = reinterpret_cast<uint32_t *>(args.y[0]) + (size_t)g * args.y_batch_stride +
                                            (size_t)grow * args.ldy + args.col_offset + gcol;
                            if (gcol + 4 <= args.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                                *reinterpret_cast<uint4 *>(dst) = val;
                            } else {
                                const uint32_t w4[4] = {val.x, val.y, val.z, val.w};
                                for (int j = 0; j < 4 && gcol + j < args.N; ++j) dst[j] = w4[j];
                            }
                        }
                    }
                    __syncwarp();
                }
            }
        } else
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int g = tile / tiles_per_batch, tin = tile % tiles_per_batch;
            int m_blk, n_blk;
            tile_coords(tin, num_m, num_n, args.group_m, m_blk, n_blk);
            if (tile_masked(args, m_blk, n_blk, BN)) continue;
            const bool rows2 = NA == 2 && args.rows2;
            const int acc = rows2 ? 0 : (t_local & 1);
            const unsigned acc_ph = rows2 ? ((unsigned)t_local & 1u) : ((unsigned)(t_local >> 1) & 1u);
            if (!mbar_wait(&tmem_full[acc], acc_ph, args.wait)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // warps 2-5 take the first half of the tile's 32-column chunks, warps 6-9 the second (odd counts: one more first)
            constexpr int NCHUNK = BN / 32, FIRST = (NCHUNK + 1) / 2;
            const int half = (warp - 2) >> 2;
            epilogue_tile<KIND, BN>(args, tmem_base, acc, q, lane, m_blk * BMT, n_blk, g, epi_smem + (size_t)(warp - 2) * 4096,
                                    half ? FIRST : 0, half ? NCHUNK : FIRST);
            if (rows2)  // rows 128..255 of the tile sit in the second buffer
                epilogue_tile<KIND, BN>(args, tmem_base, 1, q, lane, m_blk * BMT + BM, n_blk, g, epi_smem + (size_t)(warp - 2) * 4096,
                                        half ? FIRST : 0, half ? NCHUNK : FIRST);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
            ++t_local;
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Skinny form for 8 < M <= 64 (weights >> activations, HBM-bound): the operands swap roles.  The
// 128 TMEM lanes carry 128 output channels (a 16 KB weight tile per 128-byte k stage) and the MMA's N
// dimension carries the M activation rows (one or two e4m3 pieces of MB rows each), so almost all
// bytes in flight are weight bytes and a deep ring (up to 8 stages) keeps ~100 KB of them in flight
// per SM.  D[n, m] is written transposed: lane = output channel, column = activation row.
// ---------------------------------------------------------------------------------------------
struct SkinnyArgs {
    void *y;     // [M, ldy] bf16 (fp8 and bf16 operands) or f16
    int ldy;
    const float *x_scale, *w_scale;  // fp8 operands only
    float *partials;     // scratch: [2 * grid][MB][128] f32 partial accumulators of split tiles
    unsigned *counters;  // scratch: [tiles] arrival counts; zero between launches
    int M, N, K;
    int MB;      // MMA N dimension: M rounded up to 16
    int nstage;
    int np;      // pieces (1 or 2)
    int uq, ur;  // stage units per CTA: total / grid and total % grid
    int w_static;  // the weights are a model parameter: they may be fetched before the dependency wait
    WaitCtx wait;  // bound and status word of the kernel's mbarrier waits
};

// Work is cut at k-stage granularity ("stream-K"): total = tiles * num_kb stage units, CTA c owns the
// contiguous unit range [c*total/G, (c+1)*total/G), i.e. a run of segments (tile, kb0..kb1).  A tile
// that is covered by several CTAs is finished by whichever of them arrives last:
// every contributor stores its f32 partial to scratch, and the finisher adds all partials in k order
// -- a fixed order, so the result does not depend on which CTA happens to be last.
// (32-bit arithmetic only: a 64-bit division is ~100 dependent instructions, and the epilogue warps sit on
// the critical path at the end of the kernel.)  uq = total / G, ur = total % G come from the host: the first ur
// CTAs own uq + 1 units, the others uq.
__device__ __forceinline__ int unit_begin(int c, int uq, int ur) { return c * uq + min(c, ur); }
__device__ __forceinline__ int unit_owner(int u, int uq, int ur) {  // the CTA whose range holds unit u
    const int big = ur * (uq + 1);
    return u < big ? (int)((unsigned)u / (unsigned)(uq + 1)) : ur + (int)((unsigned)(u - big) / (unsigned)uq);
}

// The finisher's sum over a split tile's contributors.  The four epilogue warps of the CTA that arrived last share
// the tile's rows (warp w takes rows w, w + 4, ...); a lane owns four consecutive channels, so one 128-bit load per
// (row, contributor) and one 8-byte store per row replace four scalar ones -- the reduction is the tail of the
// kernel and was bound by its own instruction count on one warp per scheduler.  RB rows x NC contributors are in
// flight per round; the additions run in contributor (= k) order whatever the arrival order was.
template <int KIND, int RB, int NC>
__device__ __forceinline__ void skinny_reduce(const SkinnyArgs &args, const float *s_xs, int tile, int w, int lane, int c_first,
                                              int c_last, int t0, int uq, int ur, size_t slot_elems) {
    constexpr bool F8 = KIND == 0;
    const int ch0 = tile * BM + 4 * lane;  // first of this lane's four channels
    float ws[4] = {1.0f, 1.0f, 1.0f, 1.0f};
    if (F8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) ws[i] = ch0 + i < args.N ? __ldg(args.w_scale + ch0 + i) : 0.0f;
    }
    const bool vec_store = ch0 + 4 <= args.N && (args.ldy & 3) == 0 && (reinterpret_cast<uintptr_t>(args.y) & 7) == 0;
    for (int m0 = w; m0 < args.M; m0 += 4 * RB) {
        float4 sum[RB];
#pragma unroll
        for (int j = 0; j < RB; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int cc0 = c_first; cc0 <= c_last; cc0 += NC) {
            float4 tv[NC][RB];
#pragma unroll
            for (int d = 0; d < NC; ++d) {
                const int cc = cc0 + d;
                const bool on = cc <= c_last;
                const int slot = on ? 2 * cc + (unit_begin(cc, uq, ur) >= t0 ? 0 : 1) : 0;
                const float *src = args.partials + (size_t)slot * slot_elems + 4 * lane;
#pragma unroll
                for (int j = 0; j < RB; ++j) {
                    const int row = m0 + 4 * j;
                    tv[d][j] = (on && row < args.M) ? __ldcg(reinterpret_cast<const float4 *>(src + (size_t)row * BM))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int d = 0; d < NC; ++d)
#pragma unroll
                for (int j = 0; j < RB; ++j) {
                    sum[j].x += tv[d][j].x; sum[j].y += tv[d][j].y; sum[j].z += tv[d][j].z; sum[j].w += tv[d][j].w;
                }
        }
#pragma unroll
        for (int j = 0; j < RB; ++j) {
            const int row = m0 + 4 * j;
            if (row >= args.M) continue;
            const float xs = F8 ? s_xs[row] : 1.0f;
            const float val[4] = {F8 ? ws[0] * (xs * sum[j].x) : sum[j].x, F8 ? ws[1] * (xs * sum[j].y) : sum[j].y,
                                  F8 ? ws[2] * (xs * sum[j].z) : sum[j].z, F8 ? ws[3] * (xs * sum[j].w) : sum[j].w};
            if (KIND == 2) {
                __half *dst = reinterpret_cast<__half *>(args.y) + (size_t)row * args.ldy + ch0;
                if (vec_store) {
                    const __half2 lo = __floats2half2_rn(val[0], val[1]), hi = __floats2half2_rn(val[2], val[3]);
                    *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
                } else {
                    for (int i = 0; i < 4; ++i)
                        if (ch0 + i < args.N) dst[i] = __float2half_rn(val[i]);
                }
            } else {
                __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(args.y) + (size_t)row * args.ldy + ch0;
                if (vec_store) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(val[0], val[1]), hi = __floats2bfloat162_rn(val[2], val[3]);
                    *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
                } else {
                    for (int i = 0; i < 4; ++i)
                        if (ch0 + i < args.N) dst[i] = __float2bfloat16_rn(val[i]);
                }
            }
        }
    }
}

// KIND: 0 = fp8 pieces -> bf16 out (scaled), 1 = bf16 -> bf16, 2 = f16 -> f16 (one piece, no scales)
template <int KIND>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tcgen05_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x0,
                           const __grid_constant__ CUtensorMap map_x1, const SkinnyArgs args) {
    constexpr int W_BYTES = BM * BKB;
    const int X_BYTES = args.MB * BKB;
    const int STAGE_BYTES = W_BYTES + args.np * X_BYTES;
    const int NSTAGE = args.nstage;
    // One MMA per k step covers both pieces: they sit back to back in the stage, so they form one
    // K-major operand of np * MB rows; D columns [0, MB) are the hi products, [MB, 2 MB) the lo products
    // (an MMA instruction costs about 130 cycles here however small N is: fewer, wider MMAs).
    const int NB = args.np * args.MB;  // MMA N dimension = TMEM columns of one accumulator buffer
    constexpr bool F8 = KIND == 0;
    const uint32_t IDESC = KIND == 1 ? instr_desc(1, 1, NB) : instr_desc(0, 0, NB);
    const int TMEM_COLS = 2 * NB <= 32 ? 32 : (2 * NB <= 64 ? 64 : (2 * NB <= 128 ? 128 : (2 * NB <= 256 ? 256 : 512)));

    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full[8], empty[8], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ float s_xs[64];  // x_scale of the (at most 64) activation rows
    __shared__ int s_ok[2][4];  // per segment parity: has each epilogue warp seen its accumulator?
    __shared__ int s_last;      // this CTA arrived last at the split tile of the current segment

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (args.K + (KIND == 0 ? BKB : BKB / 2) - 1) / (KIND == 0 ? BKB : BKB / 2);
    const int uq = args.uq, ur = args.ur;
    const int u0 = unit_begin(blockIdx.x, uq, ur), u1 = unit_begin(blockIdx.x + 1, uq, ur);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        prefetch_tmap(&map_w);
        prefetch_tmap(&map_x0);
        if (args.np == 2) prefetch_tmap(&map_x1);
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    // Programmatic dependent launch.  The kernel is small enough (shared memory, registers, tensor-memory
    // columns) for two of them to share an SM, so the next launch's CTAs set up, allocate and -- since
    // weights do not depend on the previous kernel -- fetch the weight halves of their first ring-full while
    // this one is still running.  Activations, scales, the output and the split-tile scratch belong to the
    // stream order: the producer waits before its first activation load, the epilogue warps before their
    // first global access; the MMA warp only reads shared memory.
    if (warp == 0) {
        if (lane == 0) {
            constexpr int BK = F8 ? BKB : BKB / 2;  // k elements per stage
            const int pre = min(NSTAGE, u1 - u0);
            if (!args.w_static) asm volatile("griddepcontrol.wait;" ::: "memory");  // the previous kernel may have written w
            for (int it = 0; it < pre; ++it) {
                const int u = u0 + it;
                const int tile = (int)((unsigned)u / (unsigned)num_kb), kb = u - tile * num_kb;
                mbar_expect_tx_only(&full[it], (unsigned)W_BYTES);
                tma_load_2d(smem + (size_t)it * STAGE_BYTES, &map_w, kb * BK, tile * BM, &full[it]);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int it = 0;
            bool ok = true;
            for (int u = u0; u < u1 && ok;) {
                const int tile = (int)((unsigned)u / (unsigned)num_kb), kb0 = u - tile * num_kb;
                const int kb1 = min(num_kb, kb0 + (u1 - u));
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % NSTAGE;
                    const unsigned ph = (unsigned)(it / NSTAGE) & 1u;
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    if (it < pre) {  // the weights of this stage are already on their way
                        mbar_expect_tx(&full[s], (unsigned)(args.np * X_BYTES));
                    } else {
                        if (!mbar_wait(&empty[s], ph ^ 1u, args.wait)) { ok = false; break; }
                        mbar_expect_tx(&full[s], STAGE_BYTES);
                        tma_load_2d(st, &map_w, kb * BK, tile * BM, &full[s]);
                    }
                    tma_load_2d(st + W_BYTES, &map_x0, kb * BK, 0, &full[s]);
                    if (args.np == 2) tma_load_2d(st + W_BYTES + X_BYTES, &map_x1, kb * BK, 0, &full[s]);
                }
                u += kb1 - kb0;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, t_local = 0;
            bool ok = true;
            for (int u = u0; u < u1 && ok; ++t_local) {
                const int kb0 = u - (int)((unsigned)u / (unsigned)num_kb) * num_kb;
                const int kb1 = min(num_kb, kb0 + (u1 - u));
                const int acc = t_local & 1;
                const unsigned acc_ph = (unsigned)(t_local >> 1) & 1u;
                if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u, args.wait)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * NB);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % NSTAGE;
                    const unsigned ph = (unsigned)(it / NSTAGE) & 1u;
                    if (!mbar_wait(&full[s], ph, args.wait)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    const uint64_t dw = smem_desc(st), dx = smem_desc(st + W_BYTES);
#pragma unroll
                    for (int ks = 0; ks < BKB / UMMA_KB; ++ks) {
                        const uint64_t adv = (uint64_t)(ks * UMMA_KB >> 4);
                        umma<F8>(d_tmem, dw + adv, dx + adv, IDESC, (kb > kb0) || ks != 0);
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&tmem_full[acc]);
                u += kb1 - kb0;
            }
        }
    } else {
        const int q = warp & 3;
        int t_local = 0;
        bool ok = true;
        const size_t slot_elems = (size_t)args.MB * BM;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (F8 && warp == 2) {
            s_xs[lane] = lane < args.M ? __ldg(args.x_scale + lane) : 0.0f;
            s_xs[lane + 32] = lane + 32 < args.M ? __ldg(args.x_scale + lane + 32) : 0.0f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        for (int u = u0; u < u1 && ok; ++t_local) {
            const int tile = (int)((unsigned)u / (unsigned)num_kb), kb0 = u - tile * num_kb;
            const int kb1 = min(num_kb, kb0 + (u1 - u));
            const bool whole = kb0 == 0 && kb1 == num_kb;
            const int acc = t_local & 1;
            const unsigned acc_ph = (unsigned)(t_local >> 1) & 1u;
            // The four warps act together below (named barrier 1): a warp whose wait ran out still takes part in this
            // segment's barrier, and all four leave the loop together.
            const bool got = mbar_wait(&tmem_full[acc], acc_ph, args.wait);
            if (lane == 0) s_ok[t_local & 1][q] = got ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!(s_ok[t_local & 1][0] && s_ok[t_local & 1][1] && s_ok[t_local & 1][2] && s_ok[t_local & 1][3])) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int ch = tile * BM + q * 32 + lane;  // output channel of this lane
            const float ws = !F8 ? 1.0f : (ch < args.N ? __ldg(args.w_scale + ch) : 0.0f);
            // a split tile's segment is this CTA's first one iff its range starts inside that tile
            const int my_slot = 2 * blockIdx.x + ((u == u0) ? 0 : 1);
            float *mine = args.partials + (size_t)my_slot * slot_elems + q * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < args.MB; c += 16) {
                uint32_t v[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * NB + c)));
                if (args.np == 2) {
                    uint32_t w[16];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]),
                          "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15])
                        : "r"(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * NB + args.MB + c)));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
                if (whole) {
                    if (ch < args.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int mrow = c + j;
                            if (mrow < args.M) {  // 32 lanes = 32 consecutive channels of one activation row
                                const float val = F8 ? ws * (s_xs[mrow] * __uint_as_float(v[j])) : __uint_as_float(v[j]);
                                if (KIND == 2) reinterpret_cast<__half *>(args.y)[(size_t)mrow * args.ldy + ch] = __float2half_rn(val);
                                else reinterpret_cast<__nv_bfloat16 *>(args.y)[(size_t)mrow * args.ldy + ch] = __float2bfloat16_rn(val);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[(size_t)(c + j) * BM] = __uint_as_float(v[j]);
                }
            }
            // the accumulator buffer can be reused as soon as it has been read
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);

            if (!whole) {
                // contributors of this tile: the CTAs whose unit ranges intersect [tile*num_kb, (tile+1)*num_kb)
                const int t0 = tile * num_kb, t1 = t0 + num_kb;
                const int c_first = unit_owner(t0, uq, ur), c_last = unit_owner(t1 - 1, uq, ur);
                const unsigned ncontrib = (unsigned)(c_last - c_first + 1);
                __threadfence();  // this warp's quarter of the partial is visible before the CTA is counted
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) s_last = atomicAdd(args.counters + tile, 1u) == ncontrib - 1 ? 1 : 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (s_last) {  // last arriver: reduce in k order and store
                    __threadfence();
                    if (warp == 2 && lane == 0) args.counters[tile] = 0;  // ready for the next launch
                    // Every round of loads is an L2 round trip on the critical path at the end of the kernel: 16
                    // 128-bit loads per lane are in flight per round (8 rows x 2 contributors when a tile has at most
                    // two, 4 rows x 4 otherwise).
                    if (c_last - c_first < 2)
                        skinny_reduce<KIND, 8, 2>(args, s_xs, tile, warp - 2, lane, c_first, c_last, t0, uq, ur, slot_elems);
                    else
                        skinny_reduce<KIND, 4, 4>(args, s_xs, tile, warp - 2, lane, c_first, c_last, t0, uq, ur, slot_elems);
                }
            }
            u += kb1 - kb0;
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Block-quantized integer weights with many activation rows: kind::i8 MMAs (s8 x s8 -> s32, exact) with one
// hand-over per 32-element block.  The operands swap roles as in the skinny form: the 128 TMEM lanes carry 128
// output channels (row-major int8 weights, unpacked from the q4 / q8 tiles by a pre-pass), the MMA's N dimension
// BN activation rows.  Every MMA covers exactly one quantization block (32 bytes of k), starts from a zero
// accumulator and is handed to the epilogue warps through a ring of 512 / BN tensor-memory buffers; each epilogue
// thread owns one output channel and half of the tile's activation rows, turns the int32 block sums into floats
// without the conversion unit and adds scale[channel, block] * sum to its f32 accumulators in block order -- the
// arithmetic of the specification (exact int32 block sums, f32 sum over the blocks), so the result matches the
// decode kernel's.  The tensor pipe idles most of the time by design: the kernel is bound by the CUDA-core work
// per (channel, row, block), i.e. per 32 multiply-adds.
// ---------------------------------------------------------------------------------------------
struct QGemmArgs {
    float *y;              // [MA, ldy] f32
    int ldy;
    const float *x_scale;  // [MA]
    const float *w_scale;  // [n_pad, K / 32] row-major
    int NW, NPAD;          // output channels, and the row count of the unpacked weights (multiple of 16)
    int MA, K;
    WaitCtx wait;
};

__host__ __device__ constexpr uint32_t instr_desc_i8(int n) {  // D = s32, A and B signed 8-bit, both K-major
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {  // D = A * B
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
}
// An int32 block sum plus 0x4B400000, read as a float, is 1.5 * 2^23 + sum exactly (|sum| <= 32 * 127 * 127 < 2^22):
// one integer add per element and one packed subtraction per pair replace the integer-to-float conversion.
constexpr uint32_t Q_MAGIC_I = 0x4B400000u;
constexpr float Q_MAGIC_F = 12582912.0f;
constexpr int Q_NTHREADS = 64 + 256;  // producer, MMA issuer, eight epilogue warps (two per tensor-memory lane quarter)

template <int BN>
__global__ void __launch_bounds__(Q_NTHREADS, 1)
gemm_q8_block_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const QGemmArgs args) {
    constexpr int NACC = 512 / BN > 4 ? 4 : 512 / BN;   // accumulator buffers in flight
    constexpr int W_BYTES = BM * BKB, X_BYTES = BN * BKB, STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int NSTAGE = 4;
    constexpr uint32_t IDESC = instr_desc_i8(BN);
    constexpr int BPS = BKB / UMMA_KB;  // quantization blocks (= MMAs) per stage
    constexpr int HALF = BN / 2;        // columns per epilogue warp

    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full[NSTAGE], empty[NSTAGE], acc_full[NACC], acc_empty[NACC];
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_w = (args.NPAD + BM - 1) / BM, num_x = (args.MA + BN - 1) / BN;
    const int num_tiles = num_w * num_x;
    const int num_kb = args.K / BKB;
    const int nblk = args.K / 32;

    if (threadIdx.x == 0) {
        prefetch_tmap(&map_w);
        prefetch_tmap(&map_x);
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < NACC; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int x_blk = tile / num_w, w_blk = tile - x_blk * num_w;  // consecutive CTAs share the activation tile
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % NSTAGE;
                    if (!mbar_wait(&empty[s], ((unsigned)(it / NSTAGE) & 1u) ^ 1u, args.wait)) { ok = false; break; }
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(st, &map_w, kb * BKB, w_blk * BM, &full[s]);
                    tma_load_2d(st + W_BYTES, &map_x, kb * BKB, x_blk * BN, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0;
            unsigned vt = 0;  // hand-overs so far
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
                    const int s = it % NSTAGE;
                    if (!mbar_wait(&full[s], (unsigned)(it / NSTAGE) & 1u, args.wait)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    const uint64_t dw = smem_desc(st), dx = smem_desc(st + W_BYTES);
                    for (int ks = 0; ks < BPS; ++ks, ++vt) {
                        const unsigned a = vt % NACC;
                        if (!mbar_wait(&acc_empty[a], ((vt / NACC) & 1u) ^ 1u, args.wait)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t adv = (uint64_t)(ks * UMMA_KB >> 4);
                        umma_i8(tmem_base + a * BN, dw + adv, dx + adv, IDESC);
                        umma_commit(&acc_full[a]);
                    }
                    if (ok) umma_commit(&empty[s]);
                }
            }
        }
    } else {
        const int q = warp & 3, half = warp >= 6 ? 1 : 0;  // tensor-memory lane quarter, column half
        unsigned vt = 0;
        bool ok = true;
        unsigned long long neg2;
        asm("mov.b64 %0, {%1, %2};" : "=l"(neg2) : "f"(-Q_MAGIC_F), "f"(-Q_MAGIC_F));
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * HALF);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int x_blk = tile / num_w, w_blk = tile - x_blk * num_w;
            const int ch = w_blk * BM + q * 32 + lane;  // this thread's output channel
            const float4 *srow = reinterpret_cast<const float4 *>(args.w_scale + (size_t)(ch < args.NPAD ? ch : 0) * nblk);
            unsigned long long acc2[HALF / 2];  // f32 pairs
#pragma unroll
            for (int i = 0; i < HALF / 2; ++i) acc2[i] = 0ull;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const float4 s4 = ch < args.NPAD ? __ldg(srow + kb) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float sc[BPS] = {s4.x, s4.y, s4.z, s4.w};
                // The stage's BPS blocks x CPB 32-column chunks form one software pipeline: the tensor-memory load of
                // chunk j + 1 is in flight while chunk j is scaled and added.
                constexpr int CPB = HALF / 32, NCH = BPS * CPB;
                uint32_t v[2][32];
                if (!mbar_wait(&acc_full[vt % NACC], (vt / NACC) & 1u, args.wait)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                tmem_ld32_nowait(lane_addr + (vt % NACC) * BN, v[0]);
#pragma unroll
                for (int j = 0; j < NCH; ++j) {
                    const int ks = j / CPB, c = j % CPB;
                    const unsigned a = (vt + ks) % NACC;
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c == CPB - 1) {  // the block has been read: its buffer goes back to the MMA issuer
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[a]);
                    }
                    if (j + 1 < NCH) {
                        const int ks1 = (j + 1) / CPB, c1 = (j + 1) % CPB;
                        const unsigned vt1 = vt + ks1, a1 = vt1 % NACC;
                        if (c1 == 0) {
                            if (!mbar_wait(&acc_full[a1], (vt1 / NACC) & 1u, args.wait)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        tmem_ld32_nowait(lane_addr + a1 * BN + c1 * 32, v[(j + 1) & 1]);
                    }
                    unsigned long long s2;
                    asm("mov.b64 %0, {%1, %2};" : "=l"(s2) : "f"(sc[ks]), "f"(sc[ks]));
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        unsigned long long p;
                        asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(v[j & 1][i] + Q_MAGIC_I), "r"(v[j & 1][i + 1] + Q_MAGIC_I));
                        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(p) : "l"(p), "l"(neg2));
                        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(acc2[c * 16 + i / 2]) : "l"(s2), "l"(p), "l"(acc2[c * 16 + i / 2]));
                    }
                }
                vt += BPS;
            }
            if (!ok) break;
            if (ch < args.NW) {
#pragma unroll
                for (int i = 0; i < HALF; i += 2) {
                    float a0, a1;
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc2[i / 2]));
                    const int row = x_blk * BN + half * HALF + i;  // 32 lanes = 32 consecutive channels of one activation row
                    if (row < args.MA) args.y[(size_t)row * args.ldy + ch] = __ldg(args.x_scale + row) * a0;
                    if (row + 1 < args.MA) args.y[(size_t)(row + 1) * args.ldy + ch] = __ldg(args.x_scale + row + 1) * a1;
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Causal attention over a block of query rows as ONE kernel (prefill): scores never leave the SM.
// A work item is a (head, 128-query block) pair; one pass over its visible 128-key blocks:
//   S = Q K^T into tensor memory (two buffers); the softmax warps read it back, p = 2^((s - m) c) with
//   c = scale * log2(e) and m the stream's reference point, row sums in f32, P rounded to the element type and written
//   BACK into tensor memory over the scores it came from (a thread's row is its lane; two elements per column):
//   O += P V takes its A operand from tensor memory and V from shared memory as it lies in memory (keys x head_dim,
//   an MN-major B operand), accumulating in tensor memory; at the end O / l, rounded, stored.  Nothing but K, V and
//   Q tiles ever touches shared memory.
// Thread layout: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..9 = softmax, two per tensor-memory lane
// quarter.  A softmax thread owns one query row and ONE HALF of every key block (keys 0..63 or 64..127 of the block),
// and the two halves are two independent online-softmax streams: each has its own running maximum, its own row sum
// and its own accumulator in tensor memory (O_0 += P[:, :64] V[:64], O_1 += P[:, 64:] V[64:]; S0 S1 O_0 O_1 fill the
// 512 columns), so the warps never exchange anything per block; the streams are merged once at the end with the
// usual log-sum-exp weights.  When a block raises a stream's maximum, the thread rescales its row of that stream's
// accumulator in place (tcgen05.ld / st, after the previous block's P V has completed); the reference point of a
// stream's exponentials moves only when a block exceeds it by 2^8, so this is rare.  Key j is visible to query row i iff j <= i + off and j < ctx.
// head_dim = 128, 16-bit elements.  The kernel is bound by its tensor-memory MMAs (16 per key block, each costing
// about the same for N = 128 as for N = 256) and by the exponentials, in that order.
// ---------------------------------------------------------------------------------------------
struct AttnArgs {
    void *out;         // [T][ldo] elements; head h at columns [128 h, 128 h + 128)
    long long ldo;
    int T, ctx, off, heads;
    int nqb;           // query blocks per head
    float c;           // scale * log2(e)
    int q_inner, k_inner, v_inner;  // dimension order of the three tensor maps (see make_map3 / make_map_mn)
    WaitCtx wait;
};
constexpr int ATT_THREADS = 64 + 256;
constexpr int ATT_TILE = 128 * BKB;  // one 128-row x 128-byte tile: 16 KB
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D += A * B with the A operand in tensor memory (lane = row, two 16-bit elements per column, 8 columns per MMA)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}

template <int KIND>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const AttnArgs args) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *sQ = smem;                       // 2 tiles (head_dim halves)
    unsigned char *sK = sQ + 2 * ATT_TILE;          // 2 stages x 2 tiles
    unsigned char *sV = sK + 4 * ATT_TILE;          // 2 stages x 2 key halves x (2 blocks of 64 head_dim columns)
    __shared__ __align__(8) uint64_t q_full, q_empty, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2],
        p_full[2], pv_done[2], o_full, o_empty;
    __shared__ uint32_t tmem_slot;
    __shared__ float red_m[2][128], red_l[2][128];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The kernel is persistent: CTA c works on items c, c + grid, ... of the list of (query block, head) pairs ordered
    // by falling work (the last query block of every head first), so that every CTA gets the same share within a block
    // or two, and the set-up, the first loads and the first scores of an item overlap the tail of the previous one.
    // Every barrier is used once per key block or once per item; the roles keep running counts for the phases.
    const int nitems = args.nqb * args.heads;
    constexpr uint32_t IDESC = KIND == 1 ? instr_desc(1, 1, 128) : instr_desc(0, 0, 128);
    // Item k of this CTA: the list is dealt out in rounds of `grid` items, forwards in even rounds and backwards in odd
    // ones, so a CTA that got the heaviest item of one round gets the lightest of the next.
    auto first_item = [&](unsigned k) -> int {
        return (int)(k * gridDim.x + ((k & 1u) ? gridDim.x - 1 - blockIdx.x : blockIdx.x));
    };
    auto item_geom = [&](int item, int &head, int &q0, int &nkb) {
        head = (int)((unsigned)item % (unsigned)args.heads);
        q0 = (args.nqb - 1 - (int)((unsigned)item / (unsigned)args.heads)) * 128;
        nkb = (min(args.ctx - 1, q0 + 127 + args.off) >> 7) + 1;  // visible 128-key blocks
        if (nkb < 1) nkb = 1;
    };

    if (threadIdx.x == 0) {
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_k);
        prefetch_tmap(&map_v);
        mbar_init(&q_full, 1); mbar_init(&q_empty, 1);
        mbar_init(&o_full, 1); mbar_init(&o_empty, 8);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 1);
            mbar_init(&p_full[i], 8);
            mbar_init(&pv_done[i], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;  // O_0 at columns [256, 384), O_1 at [384, 512)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            unsigned g = 0, n_item = 0;  // key blocks and items so far
            for (int item = first_item(0); item < nitems && ok; item = first_item(++n_item)) {
                int head, q0, nkb;
                item_geom(item, head, q0, nkb);
                if (!mbar_wait(&q_empty, (n_item & 1u) ^ 1u, args.wait)) { ok = false; break; }  // the previous item's scores are done
                mbar_expect_tx(&q_full, 2 * ATT_TILE);
                for (int h = 0; h < 2; ++h)
                    tma_load_3d(sQ + h * ATT_TILE, &map_q, h * 64, args.q_inner ? head : q0, args.q_inner ? q0 : head, &q_full);
                for (int j = 0; j < nkb && ok; ++j, ++g) {
                    const int s = (int)(g & 1u);
                    const unsigned ph = ((g >> 1) & 1u) ^ 1u;
                    if (!mbar_wait(&k_empty[s], ph, args.wait)) { ok = false; break; }
                    mbar_expect_tx(&k_full[s], 2 * ATT_TILE);
                    for (int h = 0; h < 2; ++h)
                        tma_load_3d(sK + (2 * s + h) * ATT_TILE, &map_k, h * 64, args.k_inner ? head : j * 128,
                                    args.k_inner ? j * 128 : head, &k_full[s]);
                    if (!mbar_wait(&v_empty[s], ph, args.wait)) { ok = false; break; }
                    mbar_expect_tx(&v_full[s], 2 * ATT_TILE);
                    for (int kh = 0; kh < 2; ++kh)      // 64 keys each
                        for (int nb = 0; nb < 2; ++nb)  // 64 head_dim columns each
                            tma_load_3d(sV + (2 * s + kh) * ATT_TILE + nb * (64 * BKB), &map_v, nb * 64,
                                        args.v_inner ? head : j * 128 + kh * 64, args.v_inner ? j * 128 + kh * 64 : head,
                                        &v_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            unsigned gs = 0, gp = 0, n_item = 0;  // scores issued, products issued, items so far
            // S[gs & 1] = Q K^T for the next key block of the K ring
            auto issue_s = [&]() -> bool {
                const unsigned b = gs & 1u, ph = (gs >> 1) & 1u;
                if (!mbar_wait(&k_full[b], ph, args.wait)) return false;
                if (!mbar_wait(&s_empty[b], ph ^ 1u, args.wait)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint64_t da = smem_desc(sQ + h * ATT_TILE), db = smem_desc(sK + (2 * b + h) * ATT_TILE);
#pragma unroll
                    for (int ks = 0; ks < BKB / UMMA_KB; ++ks) {
                        const uint64_t adv = (uint64_t)(ks * UMMA_KB >> 4);
                        umma<false>(tmem_base + b * 128, da + adv, db + adv, IDESC, (h | ks) != 0);
                    }
                }
                umma_commit(&k_empty[b]);
                umma_commit(&s_full[b]);
                ++gs;
                return true;
            };
            for (int item = first_item(0); item < nitems && ok; item = first_item(++n_item)) {
                int head, q0, nkb;
                item_geom(item, head, q0, nkb);
                if (!mbar_wait(&q_full, n_item & 1u, args.wait)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                ok = issue_s();
                if (ok && nkb == 1) umma_commit(&q_empty);
                for (int j = 0; j < nkb && ok; ++j, ++gp) {
                    if (j + 1 < nkb) {
                        ok = issue_s();
                        if (ok && j + 2 == nkb) umma_commit(&q_empty);  // the last scores of the item: Q may be replaced
                    }
                    if (!ok) break;
                    const unsigned b = gp & 1u, ph = (gp >> 1) & 1u;
                    if (!mbar_wait(&p_full[b], ph, args.wait) || !mbar_wait(&v_full[b], ph, args.wait)) { ok = false; break; }
                    // the first product of an item overwrites the accumulators: the previous item's rows must have been read
                    if (j == 0 && !mbar_wait(&o_empty, (n_item & 1u) ^ 1u, args.wait)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int kh = 0; kh < 2; ++kh) {  // stream kh: O_kh += P[:, keys of half kh] V[keys of half kh]
                        const uint64_t db = smem_desc_mn(sV + (2 * b + kh) * ATT_TILE, 64 * BKB);
#pragma unroll
                        for (int ks = 0; ks < BKB / UMMA_KB; ++ks) {
                            const uint64_t badv = (uint64_t)((UMMA_KB / 2) * 128 >> 4);  // 16 key rows of 128 bytes per MMA
                            // P of stream kh sits in the first 32 columns of the stream's half of S[b]: 8 columns per MMA
                            umma_ts(tmem_o + kh * 128, tmem_base + b * 128 + kh * 64 + ks * 8, db + ks * badv, IDESC | (1u << 16),
                                    (j | ks) != 0);
                        }
                    }
                    umma_commit(&v_empty[b]);
                    umma_commit(&pv_done[b]);
                    umma_commit(&s_empty[b]);  // S[b] (and the P inside it) is free once these products have read it
                }
                if (ok) umma_commit(&o_full);
            }
        }
    } else {
        const int q = warp & 3, half = (warp - 2) >> 2;
        const int row_local = q * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t s_addr = lane_base + (uint32_t)(half * 64);
        const uint32_t o_mine = lane_base + 256 + (uint32_t)(half * 128);  // this stream's accumulator row
        bool ok = true;
        unsigned g = 0, n_item = 0;
        for (int item = first_item(0); item < nitems; item = first_item(++n_item)) {
            int head, q0, nkb;
            item_geom(item, head, q0, nkb);
            const int row = q0 + row_local;
            const int horizon = min(args.ctx - 1, row + args.off);  // last visible key of this row
            float m = -INFINITY, l = 0.0f;
            for (int j = 0; j < nkb && ok; ++j, ++g) {
                const unsigned b = g & 1u, ph = (g >> 1) & 1u;
                if (!mbar_wait(&s_full[b], ph, args.wait)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t v[2][32];
                tmem_ld32_nowait(s_addr + b * 128, v[0]);
                tmem_ld32_nowait(s_addr + b * 128 + 32, v[1]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col0 = j * 128 + half * 64;
                const bool full = col0 + 63 <= horizon;
                if (!full) {  // a block that straddles the row's horizon: hidden scores become -inf (probability 0)
#pragma unroll
                    for (int i = 0; i < 64; ++i)
                        if (col0 + i > horizon) v[i >> 5][i & 31] = 0xff800000u;
                }
                float bm4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains: the maximum is on the critical path
#pragma unroll
                for (int i = 0; i < 64; ++i) bm4[i & 3] = fmaxf(bm4[i & 3], __uint_as_float(v[i >> 5][i & 31]));
                const float bm = fmaxf(fmaxf(bm4[0], bm4[1]), fmaxf(bm4[2], bm4[3]));
                // The reference point m of the stream's exponentials moves only when a block exceeds it by more than 2^8:
                // any reference gives the same quotient at the end, probabilities up to 256 are harmless in f32 and in the
                // 16-bit types, and the rescaling below (a round trip through tensor memory that has to wait for the previous
                // product) becomes rare instead of happening whenever one of a warp's 32 rows sees a new maximum.
                const float m_new = (bm - m) * args.c > 8.0f ? bm : m;  // m = -inf: the first visible block sets it
                const float alpha = m_new != m ? ex2_approx((m - m_new) * args.c) : 1.0f;  // m = -inf: 0
                if (j > 0 && __any_sync(0xffffffffu, m_new != m)) {
                    // this stream's accumulator holds the sum up to block j - 1 relative to the old reference: wait for that
                    // product to be complete, then scale the row in place
                    if (!mbar_wait(&pv_done[b ^ 1u], ((g - 1) >> 1) & 1u, args.wait)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                    for (int cq = 0; cq < 4; ++cq) {
                        uint32_t o[32];
                        tmem_ld32(o_mine + cq * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(o_mine + cq * 32, o);
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                }
                l *= alpha;
                m = m_new;
                const float mc = m == -INFINITY ? 0.0f : m * args.c;  // a stream that has seen no key yet: its scores are all -inf
                uint32_t packed[32];
                float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i = 0; i < 64; i += 2) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(v[i >> 5][i & 31]), args.c, -mc));
                    const float p1 = ex2_approx(fmaf(__uint_as_float(v[(i + 1) >> 5][(i + 1) & 31]), args.c, -mc));
                    l4[i & 2] += p0;
                    l4[(i & 2) + 1] += p1;
                    if (KIND == 2) {
                        __half2 hh = __floats2half2_rn(p0, p1);
                        packed[i >> 1] = *reinterpret_cast<uint32_t *>(&hh);
                    } else {
                        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                        packed[i >> 1] = *reinterpret_cast<uint32_t *>(&hh);
                    }
                }
                l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
                // P goes back into tensor memory, over the first 32 columns of the scores this thread has just consumed
                // (its row = its lane, two elements per column): the A operand of the P V product is read from there
                tmem_st32(s_addr + b * 128, packed);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[b]);
            }
            // merge the two streams of a row: weights 2^((m_h - M) c), M = max(m_0, m_1).  (Every softmax warp passes the
            // two barriers of every item, also after a wait has run out: nobody is left waiting at them.)
            red_m[half][row_local] = m;
            red_l[half][row_local] = l;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float m0 = red_m[0][row_local], m1 = red_m[1][row_local];
            const float mm = fmaxf(m0, m1);
            const float w0 = m0 == -INFINITY ? 0.0f : ex2_approx((m0 - mm) * args.c);
            const float w1 = m1 == -INFINITY ? 0.0f : ex2_approx((m1 - mm) * args.c);
            const float lsum = w0 * red_l[0][row_local] + w1 * red_l[1][row_local];
            asm volatile("bar.sync 1, 256;" ::: "memory");  // the exchange arrays may be rewritten for the next item
            if (ok && !mbar_wait(&o_full, n_item & 1u, args.wait)) ok = false;
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float i0 = w0 / lsum, i1 = w1 / lsum;
                uint16_t *dst = reinterpret_cast<uint16_t *>(args.out) + (size_t)row * args.ldo + (size_t)head * 128 + half * 64;
#pragma unroll 1
                for (int cq = 0; cq < 2; ++cq) {  // 32 output columns at a time
                    uint32_t a[32], bb[32];
                    tmem_ld32_nowait(lane_base + 256 + half * 64 + cq * 32, a);
                    tmem_ld32_nowait(lane_base + 384 + half * 64 + cq * 32, bb);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (cq == 1) {  // both accumulators of this item are in registers: the next item may overwrite them
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&o_empty);
                    }
                    if (row < args.T) {
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int i = 8 * ch + 2 * e;
                                const float f0 = __uint_as_float(a[i]) * i0 + __uint_as_float(bb[i]) * i1;
                                const float f1 = __uint_as_float(a[i + 1]) * i0 + __uint_as_float(bb[i + 1]) * i1;
                                if (KIND == 2) {
                                    __half2 hh = __floats2half2_rn(f0, f1);
                                    w[e] = *reinterpret_cast<uint32_t *>(&hh);
                                } else {
                                    __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
                                    w[e] = *reinterpret_cast<uint32_t *>(&hh);
                                }
                            }
                            *reinterpret_cast<uint4 *>(dst + cq * 32 + 8 * ch) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 2-D row-major [rows, k] tensor with `elem` bytes per element and a row pitch of ld elements;
// box = 128 bytes of k by box_rows rows, 128-byte swizzle, out-of-range reads give zeros.
// 3-D form of the same map: `batch` matrices `batch_stride` elements apart (box covers one of them).
// Dimensions are ordered by increasing stride: when the batch stride is smaller than the row pitch (a
// transposed view such as [groups, rows, k] over storage [rows, groups, k]) the map is (k, batch, rows) and
// *batch_inner is set; the shared-memory image of a box is the same either way.
int make_map3(CUtensorMap *map, const void *base, int elem, size_t rows, size_t k, size_t ld, int box_rows,
              size_t batch, size_t batch_stride, int *batch_inner) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(XN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (batch <= 1) { batch = 1; batch_stride = rows * ld; }
    const bool inner = batch_stride < ld;
    *batch_inner = inner ? 1 : 0;
    cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)(inner ? batch : rows), (cuuint64_t)(inner ? rows : batch)};
    cuuint64_t strides[2] = {(cuuint64_t)(inner ? batch_stride : ld) * elem, (cuuint64_t)(inner ? ld : batch_stride) * elem};
    cuuint32_t box[3] = {(cuuint32_t)(BKB / elem), (cuuint32_t)(inner ? 1 : box_rows), (cuuint32_t)(inner ? box_rows : 1)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapDataType dt = elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                       : (elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16);
    CUresult r = fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(XN_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with code %d", (int)r);
    return XN_OK;
}

int make_map(CUtensorMap *map, const void *base, int elem, size_t rows, size_t k, size_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(XN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem};
    cuuint32_t box[2] = {(cuuint32_t)(BKB / elem), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(XN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return XN_OK;
}

// [K, N] operand with n contiguous, k-rows `ld` elements apart, `batch` matrices batch_stride elements apart:
// dimensions (n, k, batch), box 64 n x 64 k (128-byte rows, 128-byte swizzle).  16-bit elements only.
// As in make_map3 the dimensions are ordered by increasing stride: when the matrices interleave (batch stride
// smaller than the k-row pitch, e.g. the per-head value slices of a fused qkv projection) the map is (n, batch, k)
// and *batch_inner is set.
int make_map_mn(CUtensorMap *map, const void *base, size_t n, size_t k, size_t ld, size_t batch, size_t batch_stride,
                int *batch_inner) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(XN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (batch <= 1) { batch = 1; batch_stride = k * ld; }
    const bool inner = batch_stride < ld;
    *batch_inner = inner ? 1 : 0;
    cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)(inner ? batch : k), (cuuint64_t)(inner ? k : batch)};
    cuuint64_t strides[2] = {(cuuint64_t)(inner ? batch_stride : ld) * 2, (cuuint64_t)(inner ? ld : batch_stride) * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)(inner ? 1 : BKB / 2), (cuuint32_t)(inner ? BKB / 2 : 1)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(XN_ERR_CUDA, "cuTensorMapEncodeTiled (n-contiguous operand) failed with code %d", (int)r);
    return XN_OK;
}

// Second half of a split-k product: y = epilogue(sum over the k chunks of the f32 tile records the tiled kernel left
// in `rec`), the chunks added in k order.  A thread owns one row of a tile and one group of 4 columns; a CTA of 256
// threads covers the tile's 128 rows x 2 column groups, so every record read is 512 contiguous bytes per warp.
// Epilogue as in the tiled kernel: fp8 scales, or nn::Linear's bias added to the rounded product and rounded again.
template <int KIND>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(void *__restrict__ y, int ldy, const float *__restrict__ rec, int chunks, int M, int N, int bn,
                     const float *__restrict__ x_scale, const float *__restrict__ w_scale, const void *__restrict__ col_bias) {
    constexpr bool F8 = KIND == 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int per_tile = bn / 8;  // CTAs per tile
    const int t = blockIdx.x / per_tile, cg = (blockIdx.x - t * per_tile) * 2 + (threadIdx.x >> 7), r = threadIdx.x & 127;
    const int num_n = (N + bn - 1) / bn, num_m = (M + BM - 1) / BM;
    const int m_blk = t / num_n, n_blk = t - m_blk * num_n;
    const int row = m_blk * BM + r, col = n_blk * bn + cg * 4;
    if (row >= M || col >= N) return;
    const size_t tile_elems = (size_t)bn * BM, chunk_elems = tile_elems * num_m * num_n;
    const float *p = rec + (size_t)t * tile_elems + ((size_t)cg * BM + r) * 4;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < chunks; c0 += 4) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            v[j] = c0 + j < chunks ? __ldcg(reinterpret_cast<const float4 *>(p + (size_t)(c0 + j) * chunk_elems))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
    }
    float val[4] = {sum.x, sum.y, sum.z, sum.w};
    if (F8) {
        const float xs = __ldg(x_scale + row);
#pragma unroll
        for (int e = 0; e < 4; ++e) val[e] = (col + e < N ? __ldg(w_scale + col + e) : 0.0f) * (xs * val[e]);
    }
    uint16_t out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (KIND == 2) {
            __half h = __float2half_rn(val[e]);
            if (col_bias && col + e < N) h = __float2half_rn(__half2float(h) + __half2float(reinterpret_cast<const __half *>(col_bias)[col + e]));
            out[e] = *reinterpret_cast<const uint16_t *>(&h);
        } else {
            __nv_bfloat16 h = __float2bfloat16_rn(val[e]);
            if (col_bias && col + e < N)
                h = __float2bfloat16_rn(__bfloat162float(h) + __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(col_bias)[col + e]));
            out[e] = *reinterpret_cast<const uint16_t *>(&h);
        }
    }
    uint16_t *dst = reinterpret_cast<uint16_t *>(y) + (size_t)row * ldy + col;
    if (col + 4 <= N && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
        *reinterpret_cast<uint2 *>(dst) = make_uint2((uint32_t)out[0] | ((uint32_t)out[1] << 16), (uint32_t)out[2] | ((uint32_t)out[3] << 16));
    } else {
        for (int e = 0; e < 4 && col + e < N; ++e) dst[e] = out[e];
    }
}

struct BatchGeom { size_t batch = 1, a_stride = 0, b_stride = 0; };

template <int KIND, int BN, int NA>
int launch_cfg(const void *a0, const void *a1, const void *b, size_t lda, size_t ldb, const GemmArgs &args,
               cudaStream_t st, const BatchGeom &bg = BatchGeom()) {
    constexpr int ELEM = KIND == 0 ? 1 : (KIND == 3 ? 4 : 2);
    constexpr int STAGE_BYTES = NA * BM * BKB + BN * BKB;
    constexpr int NSTAGE = (192 * 1024) / STAGE_BYTES > 8 ? 8 : (192 * 1024) / STAGE_BYTES;
    CUtensorMap ma0, ma1, mb;
    GemmArgs args2 = args;
    if (int rcw = wait_ctx(&args2.wait)) return rcw;
    {
        // group_m ~ sqrt(SMs x B-panel rows / A-panel rows): the wave's footprint gm x A + (SMs / gm) x B is smallest
        // there.  Operands that fit in L2 together (about half of its 126 MB, leaving room for the output) keep the
        // plain m-fastest order, which measured 2-4 % faster on them (4096^3: 104.5 vs 108.5 us).
        static const int force_gm = [] { const char *e = getenv("XN_GEMM_GROUP_M"); return e ? atoi(e) : 0; }();
        const int bmt = (NA == 2 && args.rows2) ? 2 * BM : BM;
        const int num_m = (args.M + bmt - 1) / bmt;
        int gm = 1;
        while ((gm + 1) * (gm + 1) * bmt <= sm_count() * BN) ++gm;
        const double operand_bytes = ((double)args.M * ((NA == 2 && !args.rows2) ? 2 : 1) + (double)args.N) * (double)args.K * ELEM;
        if (operand_bytes <= 64.0 * 1024 * 1024) gm = num_m;
        if (force_gm > 0) gm = force_gm;
        args2.group_m = gm < num_m ? gm : num_m;
        if (args2.group_m < 1) args2.group_m = 1;
    }
    args2.fast_store = (args.ndst == 1 && !args.mc && args.ldy % 8 == 0 && args.col_offset % 8 == 0 &&
                        args.y_batch_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(args.y[0]) & 15) == 0 &&
                        (KIND != 0 || (reinterpret_cast<uintptr_t>(args.w_scale) & 15) == 0))
                           ? 1 : 0;
    const size_t a_batch = args.a_bcast ? 1 : bg.batch;
    int rc = make_map3(&ma0, a0, ELEM, args.M, args.K, lda, BM, a_batch, bg.a_stride, &args2.a_batch_inner);
    if (rc) return rc;
    rc = make_map3(&ma1, NA == 2 ? a1 : a0, ELEM, args.M, args.K, lda, BM, a_batch, bg.a_stride, &args2.a_batch_inner);
    if (rc) return rc;
    if (args.b_mn) {
        if constexpr (ELEM == 2 && BN % 64 == 0) rc = make_map_mn(&mb, b, args.N, args.K, ldb, bg.batch, bg.b_stride, &args2.b_batch_inner);
        else rc = fail(XN_ERR_UNSUPPORTED, "n-contiguous right-hand side: tile width %d / element size %d not supported", BN, ELEM);
    } else {
        rc = make_map3(&mb, b, ELEM, args.N, args.K, ldb, BN, bg.batch, bg.b_stride, &args2.b_batch_inner);
    }
    if (rc) return rc;
    auto kern = gemm_tcgen05_kernel<KIND, BN, NA, NSTAGE>;
    const size_t smem = (size_t)NSTAGE * STAGE_BYTES + 4 * 32 * 256 + 1024;
    XN_ENSURE_SMEM(kern, smem);
    const int bmt_rows = (NA == 2 && args.rows2) ? 2 * BM : BM;
    const long long tiles = (long long)((args.M + bmt_rows - 1) / bmt_rows) * ((args.N + BN - 1) / BN) * args.batch;
    const int sms = sm_count();
    const int grid = (int)(tiles < sms ? tiles : sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(KIND == 3 ? NTHREADS : 64 + 32 * EPI_WARPS_16);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, ma0, ma1, mb, args2));
    return XN_OK;
}

// Split-k for a product with too few 128 x 256 tiles to occupy the machine (a hundred-odd rows against a narrow
// weight): `chunks` equal k ranges ride the tiled kernel's batch dimension (the operands' batch stride is the chunk
// length along k), every (chunk, tile) leaves as an f32 record in library scratch, and splitk_reduce_kernel adds the
// chunks in k order and applies the epilogue.  Narrow tiles would fill the SMs too, but every one of them re-reads the
// whole A tile: 256 x 4096 x 4096 as 128 tiles of 128 x 64 pulls 196 MB through L2 for 36 MB of operands.
template <int KIND, int NA>
int launch_split_k(const void *a0, const void *a1, const void *b, size_t lda, size_t ldb, const GemmArgs &args, int chunks,
                   cudaStream_t st) {
    constexpr int bn = 256;
    const long long num_m = (args.M + BM - 1) / BM, num_n = (args.N + bn - 1) / bn;
    void *scratch = nullptr;
    if (int rc = library_scratch(st, (size_t)chunks * num_m * num_n * bn * BM * sizeof(float), &scratch)) return rc;
    GemmArgs a2 = args;
    a2.K = args.K / chunks;
    a2.batch = chunks;
    a2.split_out = static_cast<float *>(scratch);
    a2.col_bias = nullptr;
    BatchGeom bg;
    bg.batch = (size_t)chunks; bg.a_stride = (size_t)a2.K; bg.b_stride = (size_t)a2.K;
    if (int rc = launch_cfg<KIND, bn, NA>(a0, a1, b, lda, ldb, a2, st, bg)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(num_m * num_n * (bn / 8)));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<KIND>, args.y[0], args.ldy, (const float *)scratch, chunks, args.M,
                                     args.N, bn, args.x_scale, args.w_scale, args.col_bias));
    return XN_OK;
}

template <int KIND, int NA>
int launch_kind(const void *a0, const void *a1, const void *b, size_t lda, size_t ldb, const GemmArgs &args,
                cudaStream_t st, const BatchGeom &bg = BatchGeom()) {
    // Tile width.  A CTA's time per k stage follows the bytes it pulls through L2 (NA activation tiles of 128
    // rows + BN weight rows; an MMA costs the same ~130 cycles for any BN <= 256), and the launch lasts as many
    // stages as the busiest SM gets: waves x bytes per stage, minimised over the widths the kernel is
    // instantiated for.  Ties go to the wider tile (fewer re-reads of the activation tile).
    const int sms = sm_count();
    static const int force_bn = [] { const char *e = getenv("XN_GEMM_BN"); return e ? atoi(e) : 0; }();
    const long long m_tiles = (long long)((args.M + BM - 1) / BM) * args.batch;
    if constexpr (KIND != 3) {
        // split-k when 128 x 256 tiles would leave three quarters of the SMs idle and every chunk keeps >= 16 k stages
        // (measured: two chunks gain nothing -- 512 x 4096 x 4096 bf16 25.2 us either way -- and chunks of 8 stages lose:
        // fp8 W8A8 256 x 4096 x 4096 13.6 -> 15.0 us)
        static const int force_split = [] { const char *e = getenv("XN_GEMM_SPLITK"); return e ? atoi(e) : -1; }();
        constexpr int BKE = BKB / (KIND == 0 ? 1 : 2);
        const long long t256 = m_tiles * ((args.N + 255) / 256);
        if (force_split != 0 && args.batch == 1 && !args.causal && !args.a_bcast && args.ndst == 1 && !args.mc && !args.b_mn &&
            !args.row_bias && !args.rows2 && args.col_offset == 0 && t256 * 4 <= sms && args.N >= 256) {
            int chunks = 0;
            for (int c = 8; c >= 4; c >>= 1)
                if (c * t256 <= sms && args.K % (c * BKE) == 0 && args.K / (c * BKE) >= 16) { chunks = c; break; }
            if (force_split > 1 && args.K % (force_split * BKE) == 0) chunks = force_split;
            if (chunks >= 2) return launch_split_k<KIND, NA>(a0, a1, b, lda, ldb, args, chunks, st);
        }
    }
    int best = 256;
    long long best_cost = -1;
    const int bn_step = args.b_mn ? 64 : 32;  // an n-contiguous B arrives in 64-column blocks
    for (int bn = 256; bn >= 64; bn -= bn_step) {
        const long long tiles = m_tiles * ((args.N + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        const long long cost = waves * (NA * BM + bn);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    if (force_bn >= 64 && force_bn <= 256 && force_bn % bn_step == 0) best = force_bn;
    if constexpr ((KIND == 1 || KIND == 2) && NA == 1) {
        // 256 x 256 tiles (two row blocks share every B stage; both accumulator buffers belong to one tile) when the
        // problem is large enough to fill the machine with them.  A k stage of a 128 x 256 tile moves 96 KB through
        // shared memory for 512 tensor cycles (the SM moves 128 B per clock: 0.67 of the tensor rate); the 256-row tile
        // moves 160 KB for 1024 cycles (0.8) at the price of an epilogue that is no longer hidden behind the next tile.
        // Measured: bf16 4096^3 105.2 -> 97.0 us, 8192^3 794 -> 712 us (cuBLAS 93 / 690 us); a 256-row tile costs 1.84 x
        // a 128-row one, which is what the wave count below is weighed with.  The fp8 kinds stay on 128-row tiles: W8A8
        // runs under the power cap and measured slower with the exposed epilogue (qkv at 4096 rows 152 -> 168 us).
        static const int force_rows2 = [] { const char *e = getenv("XN_GEMM_ROWS2"); return e ? atoi(e) : -1; }();
        if (best == 256 && !args.causal && !args.a_bcast && args.ndst == 1 && !args.mc) {
            const long long n_tiles = (args.N + 255) / 256;
            const long long t1 = m_tiles * n_tiles, t2 = (long long)((args.M + 2 * BM - 1) / (2 * BM)) * args.batch * n_tiles;
            const double c1 = (double)((t1 + sms - 1) / sms) * 1.0, c2 = (double)((t2 + sms - 1) / sms) * 1.84;
            bool rows2 = t2 >= sms && args.K >= 1024 && c2 < 0.97 * c1;
            if (force_rows2 >= 0) rows2 = force_rows2 != 0;
            if (rows2) {
                GemmArgs a2 = args;
                a2.rows2 = 1;
                return launch_cfg<KIND, 256, 2>(a0, a0, b, lda, ldb, a2, st, bg);
            }
        }
    }
    if constexpr (KIND == 3) {
        // the tf32 kind is instantiated up to 128 columns (its epilogue holds a row of the tile in registers)
        best = 128;
        best_cost = -1;
        for (int bn = 128; bn >= 64; bn -= 32) {
            const long long tiles = m_tiles * ((args.N + bn - 1) / bn);
            const long long cost = ((tiles + sms - 1) / sms) * (NA * BM + bn);
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
        }
        switch (best) {
            case 128: return launch_cfg<KIND, 128, NA>(a0, a1, b, lda, ldb, args, st, bg);
            case 96: return launch_cfg<KIND, 96, NA>(a0, a1, b, lda, ldb, args, st, bg);
            default: return launch_cfg<KIND, 64, NA>(a0, a1, b, lda, ldb, args, st, bg);
        }
    } else
    switch (best) {
        case 256: return launch_cfg<KIND, 256, NA>(a0, a1, b, lda, ldb, args, st, bg);
        case 224: return launch_cfg<KIND, 224, NA>(a0, a1, b, lda, ldb, args, st, bg);
        case 192: return launch_cfg<KIND, 192, NA>(a0, a1, b, lda, ldb, args, st, bg);
        case 160: return launch_cfg<KIND, 160, NA>(a0, a1, b, lda, ldb, args, st, bg);
        case 128: return launch_cfg<KIND, 128, NA>(a0, a1, b, lda, ldb, args, st, bg);
        case 96: return launch_cfg<KIND, 96, NA>(a0, a1, b, lda, ldb, args, st, bg);
        default: return launch_cfg<KIND, 64, NA>(a0, a1, b, lda, ldb, args, st, bg);
    }
}

}  // namespace

// Skinny path, m <= 64.  KIND 0: e4m3 pieces x0 (hi) and optional x1 (lo) with scales; KIND 1 / 2: bf16 / f16
// operands (x1, scales unused).  Strides in elements.
template <int KIND>
int launch_skinny(void *y, size_t ldy, const void *x0, const void *x1, size_t ldx, const float *x_scale, const void *w,
                  size_t ldw, const float *w_scale, size_t m, size_t n, size_t k, cudaStream_t st) {
    constexpr int ELEM = KIND == 0 ? 1 : 2;
    constexpr int BK = BKB / ELEM;  // k elements per stage
    SkinnyArgs a{};
    a.y = y; a.ldy = (int)ldy; a.x_scale = x_scale; a.w_scale = w_scale;
    a.M = (int)m; a.N = (int)n; a.K = (int)k;
    a.MB = (int)((m + 15) / 16 * 16);
    a.np = x1 ? 2 : 1;
    const int stage = BM * BKB + a.np * a.MB * BKB;
    // a ring of about 100 KB: two CTAs (this launch's and the next one's, see the kernel) fit an SM, and the
    // kernel is not bound by bytes in flight (3 to 8 stages measured the same)
    static const int ring_kb = [] { const char *e = getenv("XN_SKINNY_RING_KB"); return e ? atoi(e) : 100; }();
    a.nstage = (ring_kb * 1024) / stage > 8 ? 8 : (ring_kb * 1024) / stage;
    if (a.nstage < 2) a.nstage = 2;
    const int tiles = (int)((n + BM - 1) / BM);
    const int num_kb = (int)((k + BK - 1) / BK);
    const int sms = sm_count();
    const long long total = (long long)tiles * num_kb;
    // at least 4 k stages per CTA, so that a split never degenerates into single-stage crumbs
    long long grid = total / 4 < 1 ? 1 : total / 4;
    if (grid > sms) grid = sms;
    // Whole tiles (no fix-up pass) only when they fill at least 90 % of the machine; otherwise split at
    // k-stage granularity so that every SM streams its share of the weights and issues its share of the MMAs
    // (an MMA costs ~130 cycles whatever its N, so the MMA count per CTA is what bounds a skinny problem).
    if (tiles <= sms && tiles * 100 >= sms * 90) grid = tiles;
    // Fewer tiles than SMs: S = SMs / tiles CTAs per tile, cut at the same k positions in every tile, when that
    // still occupies 60 % of the machine.  Every tile then has exactly S contributors (S = 1: none) instead of the
    // S + 1 or S + 2 ragged ones of the even split over all SMs, and the last arriver's reduction -- the tail of
    // the kernel -- gets shorter by more than the k loop gets longer.  Measured (fp8, 32 / 64 rows): N = 4096,
    // k = 4096 on 128 CTAs 12.6 -> 11.2 / 18.1 -> 15.4 us; k = 11264 17.7 -> 17.0 / 23.6 -> 22.0 us; N = 12288 as 96
    // whole tiles 16.9 -> 17.1 / 22.3 -> 19.7 us.
    if (tiles < sms && grid == sms) {
        const long long s_per_tile = sms / tiles;
        const long long aligned = tiles * (s_per_tile < num_kb ? s_per_tile : num_kb);
        // S = 1 (whole tiles on 60-90 % of the SMs) trades a longer k loop for no reduction at all: that pays from
        // 33 rows on (N = 12288: 20.0 us either way at 64 rows, 17.6 us whole against 16.2 us split at 32).
        const bool whole_tiles = aligned == tiles;
        if (aligned * 100 >= (long long)sms * 60 && total / aligned >= 4 && (!whole_tiles || a.MB > 32)) grid = aligned;
    }
    static const int force_grid = [] { const char *e = getenv("XN_SKINNY_GRID"); return e ? atoi(e) : 0; }();
    if (force_grid > 0 && force_grid <= sms && force_grid <= total) grid = force_grid;
    XN_REQUIRE(total < (1ll << 30), "skinny matmul: problem too large for the kernel's 32-bit unit index");
    a.uq = (int)(total / grid);
    a.ur = (int)(total % grid);
    if (int rcw = wait_ctx(&a.wait)) return rcw;
    a.w_static = (KIND == 0 || rhs_is_static()) ? 1 : 0;  // the fp8 entry points take a static weight by contract
    SkinnyScratch sc;
    int rc = skinny_scratch(st, (size_t)2 * grid * a.MB * BM * sizeof(float), (size_t)tiles * 4, &sc);
    if (rc) return rc;
    a.partials = sc.partials;
    a.counters = sc.counters;
    CUtensorMap mw, mx0, mx1;
    rc = make_map(&mw, w, ELEM, n, k, ldw, BM);
    if (rc) return rc;
    rc = make_map(&mx0, x0, ELEM, m, k, ldx, a.MB);
    if (rc) return rc;
    rc = make_map(&mx1, x1 ? x1 : x0, ELEM, m, k, ldx, a.MB);
    if (rc) return rc;
    const size_t smem = (size_t)a.nstage * stage + 1024;
    auto kern = gemm_tcgen05_skinny_kernel<KIND>;
    XN_ENSURE_SMEM(kern, smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, mw, mx0, mx1, a));
    return XN_OK;
}

// y f32 [m, ldy] = x_scale[i] * sum over 32-blocks of scale[j, blk] * (int32 block sum of xq[i] . w8[j]); w8 is the
// row-major int8 image [n_pad, k] of a q4 / q8 weight, w_scale its [n_pad, k / 32] block scales.
int launch_gemm_q8_block(float *y, size_t ldy, const int8_t *xq, const float *x_scale, const int8_t *w8, const float *w_scale,
                         size_t m, size_t n, size_t n_pad, size_t k, cudaStream_t st) {
    QGemmArgs a{};
    a.y = y; a.ldy = (int)ldy; a.x_scale = x_scale; a.w_scale = w_scale;
    a.NW = (int)n; a.NPAD = (int)n_pad; a.MA = (int)m; a.K = (int)k;
    if (int rcw = wait_ctx(&a.wait)) return rcw;
    constexpr int bn = 128;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w8, 1, n_pad, k, k, BM);
    if (rc) return rc;
    rc = make_map(&mx, xq, 1, m, k, k, bn);
    if (rc) return rc;
    const size_t smem = (size_t)4 * (BM * BKB + bn * BKB) + 1024;
    const long long tiles = (long long)((n_pad + BM - 1) / BM) * ((m + bn - 1) / bn);
    const int sms = sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles < sms ? tiles : sms));
    cfg.blockDim = dim3(Q_NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    auto kern = gemm_q8_block_kernel<bn>;
    XN_ENSURE_SMEM(kern, smem);
    XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, mw, mx, a));
    return XN_OK;
}

// out [T][ldo] = causal softmax(scale * q k^T) v per head; q, k, v are [rows][head][128] views (row pitch ld elements,
// heads head_stride elements apart: the slices of a fused qkv projection, or separate contiguous tensors).
int launch_attention_prefill(xn_dtype dt, void *out, size_t ldo, const void *q, const void *k, const void *v, size_t ld,
                             size_t head_stride, size_t heads, size_t t_rows, size_t ctx, float scale, cudaStream_t st) {
    AttnArgs a{};
    a.out = out; a.ldo = (long long)ldo; a.T = (int)t_rows; a.ctx = (int)ctx; a.off = (int)(ctx - t_rows); a.heads = (int)heads;
    a.nqb = (int)((t_rows + 127) / 128);
    a.c = scale * 1.4426950408889634f;
    if (int rcw = wait_ctx(&a.wait)) return rcw;
    CUtensorMap mq, mk, mv;
    int rc = make_map3(&mq, q, 2, t_rows, 128, ld, 128, heads, head_stride, &a.q_inner);
    if (rc) return rc;
    rc = make_map3(&mk, k, 2, ctx, 128, ld, 128, heads, head_stride, &a.k_inner);
    if (rc) return rc;
    rc = make_map_mn(&mv, v, 128, ctx, ld, heads, head_stride, &a.v_inner);
    if (rc) return rc;
    const size_t smem = (size_t)10 * ATT_TILE + 1024;
    cudaLaunchConfig_t cfg = {};
    const size_t items = heads * (size_t)a.nqb;
    cfg.gridDim = dim3((unsigned)(items < (size_t)sm_count() ? items : (size_t)sm_count()));
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    if (dt == XN_BF16) {
        auto kern = attention_prefill_kernel<1>;
        XN_ENSURE_SMEM(kern, smem);
        XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, a));
    } else {
        auto kern = attention_prefill_kernel<2>;
        XN_ENSURE_SMEM(kern, smem);
        XN_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, a));
    }
    return XN_OK;
}

int launch_linear_fp8_skinny(void *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale, const uint8_t *wq,
                             const float *w_scale, size_t m, size_t n, size_t k, cudaStream_t st) {
    return launch_skinny<0>(y, n, x_hi, x_lo, k, x_scale, wq, k, w_scale, m, n, k, st);
}

// y bf16 [m,n] = x_scale[m] * w_scale[n] * (x_hi (+ x_lo)) * wq^T, all operands row-major e4m3.
int launch_linear_fp8_gemm(void *y, const uint8_t *x_hi, const uint8_t *x_lo, const float *x_scale, const uint8_t *wq,
                           const float *w_scale, size_t m, size_t n, size_t k, cudaStream_t st) {
    static const size_t skinny_max = [] { const char *e = getenv("XN_FP8_SKINNY_MAX_M"); return e ? (size_t)atoi(e) : (size_t)64; }();
    if (m <= skinny_max) return launch_linear_fp8_skinny(y, x_hi, x_lo, x_scale, wq, w_scale, m, n, k, st);
    GemmArgs a{};
    a.y[0] = y; a.ndst = 1; a.col_offset = 0; a.batch = 1; a.y_batch_stride = 0;
    a.x_scale = x_scale; a.w_scale = w_scale; a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)n;
    return x_lo ? launch_kind<0, 2>(x_hi, x_lo, wq, k, k, a, st) : launch_kind<0, 1>(x_hi, nullptr, wq, k, k, a, st);
}

// Column-parallel form: this rank's [m, n] slice is written at column col_offset of every destination
// (row stride ldy).  Destinations may live on peer GPUs (plain stores over NVLink).
int launch_linear_fp8_gemm_scatter(void *const *y_dsts, int ndst, size_t ldy, size_t col_offset, const uint8_t *x_hi,
                                   const uint8_t *x_lo, const float *x_scale, const uint8_t *wq, const float *w_scale,
                                   size_t m, size_t n, size_t k, cudaStream_t st) {
    GemmArgs a{};
    for (int p = 0; p < ndst; ++p) a.y[p] = y_dsts[p];
    a.ndst = ndst; a.col_offset = (int)col_offset; a.batch = 1; a.y_batch_stride = 0;
    a.x_scale = x_scale; a.w_scale = w_scale; a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldy;
    return x_lo ? launch_kind<0, 2>(x_hi, x_lo, wq, k, k, a, st) : launch_kind<0, 1>(x_hi, nullptr, wq, k, k, a, st);
}

// The same slice written once through an NVLink multicast address (NVSwitch replicates every store into all the
// GPUs bound to it): the rank's egress is its slice once, not once per peer.
int launch_linear_fp8_gemm_multicast(void *y_mc, size_t ldy, size_t col_offset, const uint8_t *x_hi, const uint8_t *x_lo,
                                     const float *x_scale, const uint8_t *wq, const float *w_scale, size_t m, size_t n,
                                     size_t k, cudaStream_t st) {
    GemmArgs a{};
    a.y[0] = y_mc; a.ndst = 1; a.mc = 1; a.col_offset = (int)col_offset; a.batch = 1; a.y_batch_stride = 0;
    a.x_scale = x_scale; a.w_scale = w_scale; a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldy;
    return x_lo ? launch_kind<0, 2>(x_hi, x_lo, wq, k, k, a, st) : launch_kind<0, 1>(x_hi, nullptr, wq, k, k, a, st);
}

// dst [b][m,n] (row stride ldd, batch stride m*n) = lhs [b][m,k] (row stride lda, batch stride lhs_bs) *
// rhs [b][n,k]^T (row stride ldb, batch stride rhs_bs); dt BF16 or F16; one launch for all batches.
int launch_gemm_tn_16bit(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k,
                         size_t lda, size_t ldb, size_t ldd, size_t batch, size_t lhs_bs, size_t rhs_bs, cudaStream_t st,
                         int causal, int causal_off) {
    // Up to 64 rows, one batch: the skinny form (weights on the tensor-memory lanes, work split at k-stage
    // granularity over all SMs) -- a tiled launch would have too few tiles and too many MMAs per CTA.
    static const size_t skinny_max = [] { const char *e = getenv("XN_MM_SKINNY16_MAX_M"); return e ? (size_t)atoi(e) : (size_t)64; }();
    // (measured on the transformer shapes: always better up to 32 rows; from 33 to 64 only when the tiled kernel
    // would have fewer 64-column tiles than there are SMs)
    if (!causal && batch == 1 && m <= skinny_max && (m <= 32 || (m <= 64 && (n + 63) / 64 < (size_t)sm_count())))
        return dt == XN_BF16 ? launch_skinny<1>(dst, ldd, lhs, nullptr, lda, nullptr, rhs, ldb, nullptr, m, n, k, st)
                             : launch_skinny<2>(dst, ldd, lhs, nullptr, lda, nullptr, rhs, ldb, nullptr, m, n, k, st);
    GemmArgs a{};
    a.y[0] = dst; a.ndst = 1; a.col_offset = 0; a.batch = (int)batch; a.y_batch_stride = (long long)(m * n);
    a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldd;
    a.causal = causal; a.causal_off = causal_off;
    if (batch == 1 && !causal) a.col_bias = take_fused_col_bias();
    BatchGeom bg;
    bg.batch = batch; bg.a_stride = lhs_bs; bg.b_stride = rhs_bs;
    return dt == XN_BF16 ? launch_kind<1, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg)
                         : launch_kind<2, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg);
}

// `matmul` with a row-major [k, n] right-hand side (rhs rows ldb elements apart, n contiguous) -- cuBLAS's OP_N
// form of the reference (xn-core/src/cuda_backend.rs:208-223), e.g. attn.matmul(&v)
// (xn-moshi/src/batched_transformer.rs:190) and the reference's bf16 benchmark
// (xn-core/examples/basic_cuda.rs:35-56).  The tiled kernel reads B as an MN-major operand; any row count.
int launch_gemm_kn_16bit(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n, size_t k,
                         size_t lda, size_t ldb, size_t ldd, size_t batch, size_t lhs_bs, size_t rhs_bs, cudaStream_t st,
                         int causal, int causal_off) {
    GemmArgs a{};
    a.y[0] = dst; a.ndst = 1; a.col_offset = 0; a.batch = (int)batch; a.y_batch_stride = (long long)(m * n);
    a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldd;
    a.causal = causal; a.causal_off = causal_off;
    a.b_mn = 1;
    BatchGeom bg;
    bg.batch = batch; bg.a_stride = lhs_bs; bg.b_stride = rhs_bs;
    return dt == XN_BF16 ? launch_kind<1, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg)
                         : launch_kind<2, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg);
}

// The same product with one lhs shared by every batch entry and an optional per-row bias: the form the
// convolutions use (lhs = packed kernel taps, rhs = overlapping rows of the channels-last input, dst rows =
// output channels).  Always the tiled kernel.  dst batch stride dst_bs elements.
int launch_gemm_tn_16bit_shared_lhs(xn_dtype dt, void *dst, const void *lhs, const void *rhs, const void *row_bias, size_t m,
                                    size_t n, size_t k, size_t lda, size_t ldb, size_t ldd, size_t batch, size_t rhs_bs,
                                    size_t dst_bs, cudaStream_t st) {
    GemmArgs a{};
    a.y[0] = dst; a.ndst = 1; a.col_offset = 0; a.batch = (int)batch; a.y_batch_stride = (long long)dst_bs;
    a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldd;
    a.a_bcast = 1; a.row_bias = row_bias;
    BatchGeom bg;
    bg.batch = batch; bg.a_stride = 0; bg.b_stride = rhs_bs;
    return dt == XN_BF16 ? launch_kind<1, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg)
                         : launch_kind<2, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg);
}

// f32 form of the same call on kind::tf32 MMAs.  Both operands must already be f32 words on the tf32 grid
// (low 13 mantissa bits zero): the caller carries full f32 precision by splitting each operand into such
// pieces along k (see conv1d.cu).  dst and row_bias are f32.
int launch_gemm_tn_tf32_shared_lhs(float *dst, const float *lhs, const float *rhs, const float *row_bias, size_t m, size_t n,
                                   size_t k, size_t lda, size_t ldb, size_t ldd, size_t batch, size_t rhs_bs, size_t dst_bs,
                                   cudaStream_t st) {
    GemmArgs a{};
    a.y[0] = dst; a.ndst = 1; a.col_offset = 0; a.batch = (int)batch; a.y_batch_stride = (long long)dst_bs;
    a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldd;
    a.a_bcast = 1; a.row_bias = row_bias;
    BatchGeom bg;
    bg.batch = batch; bg.a_stride = 0; bg.b_stride = rhs_bs;
    return launch_kind<3, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg);
}

// Split-k form for problems with too few output tiles to fill the GPU: the k axis is cut into `splits` equal
// chunks of kchunk elements that ride the kernel's batch dimension (both tensor maps get a batch stride of
// kchunk inside the rows), each writing its own [m, n] f32 partial; the caller sums them in a fixed order.
// dst [m, n] f32 (row stride ldd) = lhs [m, k] * rhs [n, k]^T, both operands packed tf32 pieces (row stride = k).
int launch_gemm_tn_tf32(float *dst, const float *lhs, const float *rhs, size_t m, size_t n, size_t k, size_t ldd,
                        cudaStream_t st) {
    GemmArgs a{};
    a.y[0] = dst; a.ndst = 1; a.col_offset = 0; a.batch = 1; a.y_batch_stride = 0;
    a.M = (int)m; a.N = (int)n; a.K = (int)k; a.ldy = (int)ldd;
    return launch_kind<3, 1>(lhs, nullptr, rhs, k, k, a, st);
}

int launch_gemm_tn_tf32_splitk(float *partials, const float *lhs, const float *rhs, size_t m, size_t n, size_t kchunk,
                               size_t splits, size_t lda, size_t ldb, cudaStream_t st) {
    GemmArgs a{};
    a.y[0] = partials; a.ndst = 1; a.col_offset = 0; a.batch = (int)splits; a.y_batch_stride = (long long)(m * n);
    a.M = (int)m; a.N = (int)n; a.K = (int)kchunk; a.ldy = (int)n;
    BatchGeom bg;
    bg.batch = splits; bg.a_stride = kchunk; bg.b_stride = kchunk;
    return launch_kind<3, 1>(lhs, nullptr, rhs, lda, ldb, a, st, bg);
}

}  // namespace xn
