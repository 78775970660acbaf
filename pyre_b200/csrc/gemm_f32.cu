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
// Three kernels, the same arithmetic in each:
//   * many rows, rows of both operands 16-byte aligned and K a multiple of 4: 128 x 128 tiles, 8 x 8 per thread,
//     16 k per step fetched as float4 into registers one step ahead and stored transposed into the other half of a
//     double-buffered shared-memory tile (one barrier per step);
//   * up to 32 rows (decode), same alignment: a CTA of 128 threads owns 16 output features and streams their
//     weight rows in runs of 32 k through a four-stage cp.async ring (a weight stream: many small CTAs keep the
//     memory system busy, where one 128-wide tile per CTA left most SMs without work);
//   * anything else: the plain tile kernel with scalar loads.
#include "common.cuh"

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_nt_kernel(const float* A, long long lda, const float* W, long long ldw,
                float* C, long long ldc, const float* bias, int M, int N, int K) {
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

// ---------------------------------------------------------------------------
// Many rows: float4 loads along k, register prefetch, double-buffered shared memory.
// A thread's 8 rows (columns) are two groups of 4, 64 apart, so that the float4 reads of eight neighbouring threads
// cover 128 consecutive bytes of shared memory.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
sgemm_nt_tiles_kernel(const float* A, long long lda, const float* W, long long ldw,
                      float* C, long long ldc, const float* bias, int M, int N, int K) {
    constexpr int BM = 128, BN = 128, BK = 16, RUN = 32;
    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Ws[2][BK][BN + 4];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // loads: 128 rows x 4 float4 per operand and step; a thread fetches rows lr and lr + 64, k quad lq
    const int lr = tid >> 2, lq = tid & 3;
    float acc[8][8], part[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = part[i][j] = 0.f;
    float4 ra[2], rw[2];
    auto fetch = [&](int k0) {
        const int gk = k0 + 4 * lq;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int gm = m0 + lr + 64 * h, gn = n0 + lr + 64 * h;
            ra[h] = (gm < M && gk < K) ? *reinterpret_cast<const float4*>(A + (size_t)gm * lda + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
            rw[h] = (gn < N && gk < K) ? *reinterpret_cast<const float4*>(W + (size_t)gn * ldw + gk) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = lr + 64 * h;
            As[buf][4 * lq + 0][r] = ra[h].x; As[buf][4 * lq + 1][r] = ra[h].y;
            As[buf][4 * lq + 2][r] = ra[h].z; As[buf][4 * lq + 3][r] = ra[h].w;
            Ws[buf][4 * lq + 0][r] = rw[h].x; Ws[buf][4 * lq + 1][r] = rw[h].y;
            Ws[buf][4 * lq + 2][r] = rw[h].z; Ws[buf][4 * lq + 3][r] = rw[h].w;
        }
    };
    const int n_steps = (K + BK - 1) / BK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int t = 0; t < n_steps; ++t) {
        const int buf = t & 1;
        if (t + 1 < n_steps) fetch((t + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][4 * ty]), a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + 4 * ty]);
            const float4 w0 = *reinterpret_cast<const float4*>(&Ws[buf][kk][4 * tx]), w1 = *reinterpret_cast<const float4*>(&Ws[buf][kk][64 + 4 * tx]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
        }
        if (((t + 1) * BK) % RUN == 0 || t + 1 == n_steps) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[i][j] += part[i][j];
                    part[i][j] = 0.f;
                }
        }
        if (t + 1 < n_steps) stash(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gm = m0 + (i < 4 ? 4 * ty + i : 64 + 4 * ty + i - 4);
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int gn = n0 + (j < 4 ? 4 * tx + j : 64 + 4 * tx + j - 4);
            if (gn < N) C[(size_t)gm * ldc + gn] = bias ? acc[i][j] + bias[gn] : acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------
// Few rows (MT = 8 or 32 of them per CTA): 16 output features per CTA, their weight rows and the rows of A in runs of
// 32 k through a four-stage cp.async ring.  Thread (feature tn, row group tg) owns MT / 8 outputs; one stage is one
// run of the first level, so a stage ends with acc += part.
// ---------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(128)
sgemm_nt_stream_kernel(const float* A, long long lda, const float* W, long long ldw,
                       float* C, long long ldc, const float* bias, int M, int N, int K) {
    constexpr int FN = 16, RUN = 32, STAGES = 4, PITCH = RUN + 4, PER = MT / 8;
    __shared__ __align__(16) float Ws[STAGES][FN][PITCH];
    __shared__ __align__(16) float As[STAGES][MT][PITCH];
    pdl_trigger();
    const int tid = threadIdx.x, tn = tid & 15, tg = tid >> 4;
    const int n0 = blockIdx.x * FN, m0 = blockIdx.y * MT;
    const int n_runs = (K + RUN - 1) / RUN;
    // a 16-byte copy, or 16 bytes of zeros where the source lies outside the matrix
    auto copy16 = [](float* dst, const float* src, bool live) {
        const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
        const int bytes = live ? 16 : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
    };
    auto load_w = [&](int run, int st) {      // 16 rows x 8 quads: one per thread
        const int r = tid >> 3, q = tid & 7, gk = run * RUN + 4 * q, gn = n0 + r;
        const bool live = run < n_runs && gn < N && gk < K;
        copy16(&Ws[st][r][4 * q], live ? W + (size_t)gn * ldw + gk : W, live);
    };
    auto load_a = [&](int run, int st) {      // MT rows x 8 quads
        for (int e = tid; e < MT * 8; e += 128) {
            const int r = e >> 3, q = e & 7, gk = run * RUN + 4 * q, gm = m0 + r;
            const bool live = run < n_runs && gm < M && gk < K;
            copy16(&As[st][r][4 * q], live ? A + (size_t)gm * lda + gk : A, live);
        }
    };
    // the weights depend on no earlier kernel: their first stages are on their way before the wait
    for (int s = 0; s < STAGES - 1; ++s) load_w(s, s);
    pdl_wait();
    for (int s = 0; s < STAGES - 1; ++s) {
        load_a(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[PER], part[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = part[i] = 0.f;
    for (int run = 0; run < n_runs; ++run) {
        const int st = run % STAGES;
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();      // this run's stage has landed for every thread; the stage refilled below was read a run ago
        load_w(run + STAGES - 1, (run + STAGES - 1) % STAGES);
        load_a(run + STAGES - 1, (run + STAGES - 1) % STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
        for (int q = 0; q < RUN / 4; ++q) {
            const float4 w = *reinterpret_cast<const float4*>(&Ws[st][tn][4 * q]);
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const float4 a = *reinterpret_cast<const float4*>(&As[st][tg * PER + i][4 * q]);
                part[i] = fmaf(a.x, w.x, part[i]);
                part[i] = fmaf(a.y, w.y, part[i]);
                part[i] = fmaf(a.z, w.z, part[i]);
                part[i] = fmaf(a.w, w.w, part[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            acc[i] += part[i];
            part[i] = 0.f;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const int gn = n0 + tn;
    if (gn < N) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int gm = m0 + tg * PER + i;
            if (gm < M) C[(size_t)gm * ldc + gn] = bias ? acc[i] + bias[gn] : acc[i];
        }
    }
}

PYRE_API int pyre_sgemm_nt(const float* A, long long lda, const float* W, long long ldw, float* C, long long ldc,
                           const float* bias, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K < 0) return PYRE_ERR_BAD_ARG;
    // float4 loads and 16-byte copies need aligned rows in both operands
    const bool vec = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && !((uintptr_t)A & 15) && !((uintptr_t)W & 15);
    if (vec && M <= 8) {
        dim3 grid(ceil_div(N, 16), 1);
        pyre_launch(sgemm_nt_stream_kernel<8>, dim3(grid), dim3(128), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    } else if (vec && M <= 32) {
        dim3 grid(ceil_div(N, 16), 1);
        pyre_launch(sgemm_nt_stream_kernel<32>, dim3(grid), dim3(128), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    } else if (vec) {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 128));
        pyre_launch(sgemm_nt_tiles_kernel, dim3(grid), dim3(256), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    } else if (M > 32) {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 128));
        pyre_launch(sgemm_nt_kernel<128, 128, 8, 8, 8>, dim3(grid), dim3(256), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    } else {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 32));
        pyre_launch(sgemm_nt_kernel<32, 128, 16, 2, 8>, dim3(grid), dim3(256), 0, stream, A, lda, W, ldw, C, ldc, bias, M, N, K);
    }
    PYRE_LAUNCH_CHECK();
    return 0;
}
