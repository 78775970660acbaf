// True 32-bit matrix product for the float32 path:  C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]).
//
// IEEE fp32 multiply-add on the CUDA cores, no tensor-core or TF32 mode anywhere.  W has
// the layout of a linear layer's weight ([out, in], in-dim contiguous, pyre/model.py:84-87
// via nn.Linear).  Every output element is summed in two levels: a chain
// part = fma(a[k], w[k], part) over each run of 32 consecutive k (from k = 0, ascending),
// and the runs' sums added in ascending order.  The rounding error then grows with
// K / 32 + 32 terms instead of K.  The grouping depends on k alone, whatever tile shape
// computes it: a row's result is bit-identical for any M and any batch composition.
//
// Two tile shapes (same arithmetic): 128x128 with 8x8 per thread for many rows,
// 32x128 with 2x8 per thread for few (decode).
#include "common.cuh"

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_nt_kernel(const float* __restrict__ A, long long lda, const float* __restrict__ W, long long ldw,
                float* __restrict__ C, long long ldc, const float* __restrict__ bias, int M, int N, int K) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);  // column group
    const int ty = tid / (BN / TN);  // row group
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    constexpr int RUN = 32;  // k per first-level sum; a multiple of both tile depths
    static_assert(RUN % BK == 0, "a run of the first level must end at a tile's end");
    float acc[TM][TN], part[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = part[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // tile loads: consecutive threads read consecutive k of one row
        for (int e = tid; e < BM * BK; e += THREADS) {
            const int r = e / BK, kk = e % BK;
            const int gm = m0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
        }
        for (int e = tid; e < BN * BK; e += THREADS) {
            const int r = e / BK, kk = e % BK;
            const int gn = n0 + r, gk = k0 + kk;
            Ws[kk][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
        }
        if ((k0 + BK) % RUN == 0 || k0 + BK >= K) {
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] += part[i][j];
                    part[i][j] = 0.f;
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = bias ? acc[i][j] + bias[gn] : acc[i][j];
        }
    }
}

PYRE_API int pyre_sgemm_nt(const float* A, long long lda, const float* W, long long ldw, float* C, long long ldc,
                           const float* bias, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K < 0) return PYRE_ERR_BAD_ARG;
    if (M > 32) {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 128));
        pyre_launch(sgemm_nt_kernel<128, 128, 8, 8, 8>, dim3(grid), dim3(256), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    } else {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 32));
        pyre_launch(sgemm_nt_kernel<32, 128, 16, 2, 8>, dim3(grid), dim3(256), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    }
    PYRE_LAUNCH_CHECK();
    return 0;
}
