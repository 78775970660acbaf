// Sampling over fp32 logits, one block per row.
//
// The reference samples greedily only: `int(logits[i, -1].argmax())` on the host
// after a device-to-host copy per request (pyre/scheduler.py:80,94).  Here both
// rules run on the device and one int per row comes back:
//   temperature == 0 : argmax, the lowest index winning a tie
//   temperature  > 0 : Gumbel-max, argmax_v(logit[v] / temperature + g(seed, index, v))
// The noise g depends only on the request's seed, the index of the token being
// generated and the vocabulary entry, never on the batch: a request draws the same
// tokens alone or beside others.  u = (23 random bits + 0.5) / 2^23 is exact in fp32
// and lies strictly inside (0, 1), so g = -log(-log(u)) is finite.
#include "common.cuh"

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float gumbel(unsigned long long seed, unsigned int token_index, unsigned int v) {
    const unsigned long long h = mix64(seed ^ mix64(((unsigned long long)token_index << 32) | v));
    const float u = ((float)(h >> 41) + 0.5f) * (1.0f / 8388608.0f);
    return -logf(-logf(u));
}

struct Best {
    float score;
    int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    // larger score wins; equal scores: lower index; an empty slot has index INT_MAX
    if (b.score > a.score || (b.score == a.score && b.index < a.index)) return b;
    return a;
}

__global__ void sample_kernel(const float* logits, long long ld, const float* temperature,
                              const unsigned long long* seeds, const int* token_index,
                              int* out, int V) {
    __shared__ Best warp_best[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.0f / temp;
    const unsigned long long seed = seeds ? seeds[r] : 0ull;
    const unsigned int tix = token_index ? (unsigned int)token_index[r] : 0u;

    Best best{-INFINITY, 0x7fffffff};
    for (int v = threadIdx.x; v < V; v += blockDim.x) {
        float s = row[v];
        if (!greedy) s = __fadd_rn(__fmul_rn(s, inv_t), gumbel(seed, tix, (unsigned int)v));
        if (s > best.score || best.index == 0x7fffffff) best = Best{s, v};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.score, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_best[warp] = best;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        best = lane < n_warps ? warp_best[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.score, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            best = better(best, other);
        }
        if (lane == 0) out[r] = best.index == 0x7fffffff ? 0 : best.index;
    }
}

// Large vocabularies: stage 1 scans a slice of the row per block and leaves its best
// (score, index) in scratch; stage 2 picks the best slice.  The winner is the same as
// in the one-block kernel: largest score, lowest index on a tie.
__global__ void sample_slices_kernel(const float* logits, long long ld, const float* temperature,
                                     const unsigned long long* seeds, const int* token_index,
                                     float* slice_score, int* slice_index, int V, int slice) {
    __shared__ Best warp_best[32];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, sl = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.0f / temp;
    const unsigned long long seed = seeds ? seeds[r] : 0ull;
    const unsigned int tix = token_index ? (unsigned int)token_index[r] : 0u;
    const int begin = sl * slice, end = min(begin + slice, V);
    Best best{-INFINITY, 0x7fffffff};
    for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
        float s = row[v];
        if (!greedy) s = __fadd_rn(__fmul_rn(s, inv_t), gumbel(seed, tix, (unsigned int)v));
        if (s > best.score || best.index == 0x7fffffff) best = Best{s, v};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.score, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_best[warp] = best;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        best = lane < n_warps ? warp_best[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.score, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            best = better(best, other);
        }
        if (lane == 0) {
            slice_score[(size_t)r * gridDim.x + sl] = best.score;
            slice_index[(size_t)r * gridDim.x + sl] = best.index;
        }
    }
}

__global__ void sample_pick_kernel(const float* slice_score, const int* slice_index,
                                   int* out, int n_slices) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    Best best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < n_slices; i += 32)
        best = better(best, Best{slice_score[(size_t)r * n_slices + i], slice_index[(size_t)r * n_slices + i]});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.score, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
        best = better(best, other);
    }
    if (threadIdx.x == 0) out[r] = best.index == 0x7fffffff ? 0 : best.index;
}

// Slices the two-stage path cuts a row of V entries into (0: use the one-block kernel).
PYRE_API int pyre_sample_slices(int V) { return V >= 16384 ? (V + 4095) / 4096 : 0; }

// logits [R, V] fp32 with row stride ld; temperature [R] fp32 (null = all greedy);
// seeds [R] uint64 and token_index [R] int32 (may be null when all rows are greedy);
// out [R] int32.  scratch: R * pyre_sample_slices(V) * 2 words, needed when that is not 0.
PYRE_API int pyre_sample(const float* logits, long long ld, const float* temperature,
                         const unsigned long long* seeds, const int* token_index, int* out, int n_rows, int V,
                         void* scratch, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0) return PYRE_ERR_BAD_ARG;
    const int n_slices = pyre_sample_slices(V);
    if (n_slices > 0) {
        if (!scratch) return PYRE_ERR_BAD_ARG;
        float* sc = (float*)scratch;
        int* ix = (int*)scratch + (size_t)n_rows * n_slices;
        pyre_launch(sample_slices_kernel, dim3(dim3(n_slices, n_rows)), dim3(256), 0, stream, logits, ld, temperature, seeds, token_index, sc, ix, V, 4096);
        PYRE_LAUNCH_CHECK();
        pyre_launch(sample_pick_kernel, dim3(n_rows), dim3(32), 0, stream, sc, ix, out, n_slices);
        PYRE_LAUNCH_CHECK();
        return 0;
    }
    const int threads = V >= 8192 ? 1024 : (V >= 1024 ? 256 : 64);
    pyre_launch(sample_kernel, dim3(n_rows), dim3(threads), 0, stream, logits, ld, temperature, seeds, token_index, out, V);
    PYRE_LAUNCH_CHECK();
    return 0;
}
