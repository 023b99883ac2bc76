// Any-stride strided-batched GEMM on CUDA cores: the path every Backend::gemm argument tuple
// can take (xn-core/src/backend.rs:135-148), including stride patterns the reference's cuBLAS
// lowering rejects (xn-core/src/cuda_backend.rs:208-223) but its CPU backend accepts
// (xn-core/src/cpu_backend.rs:48-93).  f32 accumulation, dst overwritten.
//
// 64x64 output tile per CTA, 16-deep k slices staged through shared memory, 4x4 register
// micro-tile per thread.  Loads walk whichever of the two operand strides is 1 so that global
// reads coalesce for both the `matmul` ([k,n] row-major rhs) and `matmul_t` ([n,k] rhs) forms.
#include "common.cuh"

namespace xn {

namespace {
constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

template <typename T>
__global__ void __launch_bounds__(NT)
gemm_generic_kernel(T *__restrict__ dst, const T *__restrict__ lhs, const T *__restrict__ rhs,
                    size_t m, size_t n, size_t k, size_t lhs_b, size_t lhs_b_stride,
                    size_t rhs_b_stride, size_t dst_cs, size_t dst_rs, size_t lhs_cs,
                    size_t lhs_rs, size_t rhs_cs, size_t rhs_rs, unsigned tiles_n) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const unsigned tile = blockIdx.x;
    const size_t i0 = (size_t)(tile / tiles_n) * BM, j0 = (size_t)(tile % tiles_n) * BN;
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;  // 16x16 threads, each a 4x4 micro tile
    const bool lhs_k_fast = (lhs_cs == 1);   // consecutive threads along k, else along m
    const bool rhs_k_fast = (rhs_rs == 1);

    for (size_t b = blockIdx.y; b < lhs_b; b += gridDim.y) {
        const T *A = lhs + b * lhs_b_stride;
        const T *B = rhs + b * rhs_b_stride;
        // Two-level accumulation: each 16-deep slice is summed on its own and then added to the running
        // total -- for f32 outputs with a compensated (Kahan) add, so that the total carries one rounding
        // however long k is (the f32 parity bound allows 1e-6 of the output's rms; k / 16 plain additions
        // already exceed it at k = 4096).
        float acc[4][4] = {}, comp[4][4] = {};
        for (size_t p0 = 0; p0 < k; p0 += BK) {
            float part[4][4] = {};
#pragma unroll
            for (int e = tid; e < BM * BK; e += NT) {
                int ii, pp;
                if (lhs_k_fast) { pp = e % BK; ii = e / BK; } else { ii = e % BM; pp = e / BM; }
                size_t i = i0 + ii, p = p0 + pp;
                As[pp][ii] = (i < m && p < k) ? to_f32(A[i * lhs_rs + p * lhs_cs]) : 0.0f;
            }
#pragma unroll
            for (int e = tid; e < BN * BK; e += NT) {
                int jj, pp;
                if (rhs_k_fast) { pp = e % BK; jj = e / BK; } else { jj = e % BN; pp = e / BN; }
                size_t j = j0 + jj, p = p0 + pp;
                Bs[pp][jj] = (j < n && p < k) ? to_f32(B[p * rhs_rs + j * rhs_cs]) : 0.0f;
            }
            __syncthreads();
#pragma unroll
            for (int pp = 0; pp < BK; ++pp) {
                float a[4], bb[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) a[r] = As[pp][ty * 4 + r];
#pragma unroll
                for (int c = 0; c < 4; ++c) bb[c] = Bs[pp][tx * 4 + c];
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) part[r][c] = fmaf(a[r], bb[c], part[r][c]);
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if constexpr (sizeof(T) == 4) {
                        const float yv = part[r][c] - comp[r][c];
                        const float tv = acc[r][c] + yv;
                        comp[r][c] = (tv - acc[r][c]) - yv;
                        acc[r][c] = tv;
                    } else {
                        acc[r][c] += part[r][c];
                    }
                }
            __syncthreads();
        }
        T *D = dst + b * m * n;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                size_t i = i0 + ty * 4 + r, j = j0 + tx * 4 + c;
                if (i < m && j < n) D[i * dst_rs + j * dst_cs] = from_f32<T>(acc[r][c]);
            }
    }
}
}  // namespace

int launch_gemm_generic(xn_dtype dt, void *dst, const void *lhs, const void *rhs, size_t m, size_t n,
                        size_t k, size_t lhs_b, size_t lhs_b_stride, size_t rhs_b_stride,
                        size_t dst_cs, size_t dst_rs, size_t lhs_cs, size_t lhs_rs, size_t rhs_cs,
                        size_t rhs_rs, cudaStream_t st) {
    size_t tiles_m = (m + BM - 1) / BM, tiles_n = (n + BN - 1) / BN;
    if (tiles_m * tiles_n > 0x7fffffffull)
        return fail(XN_ERR_UNSUPPORTED, "gemm: %zu x %zu output tiles exceed the grid limit", tiles_m, tiles_n);
    dim3 grid((unsigned)(tiles_m * tiles_n), (unsigned)(lhs_b < 65535 ? lhs_b : 65535));
    XN_DISPATCH_DTYPE(dt, T,
        gemm_generic_kernel<T><<<grid, NT, 0, st>>>((T *)dst, (const T *)lhs, (const T *)rhs, m, n, k,
                                                    lhs_b, lhs_b_stride, rhs_b_stride, dst_cs, dst_rs,
                                                    lhs_cs, lhs_rs, rhs_cs, rhs_rs, (unsigned)tiles_n));
    XN_CHECK_CUDA(cudaGetLastError());
    return XN_OK;
}

}  // namespace xn
