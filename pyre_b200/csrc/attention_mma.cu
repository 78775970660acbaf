// Paged attention on the tensor cores for bfloat16: decode tokens and short prompt
// portions, with the query heads that share a key/value head stacked into the 16 rows
// of one MMA tile, and the keys of a sequence split over warps and CTAs (split-KV).
//
// Work unit ("row group"): up to 16 rows = tpg consecutive tokens of one sequence x the
// hpg query heads of one key/value head (hpg = min(n_rep, 16), tpg = 16 / hpg).  A decode
// token is a group with one token.  CTA (group, kv head [x head block], split) walks its
// share of the group's keys in tiles of 16; its 4 warps take tiles round-robin, each
// with its own online softmax, and merge through shared memory.  With more than one
// split the CTA writes an unnormalised partial (max, sum, accumulator) to scratch and
// `combine` merges the splits; with one split it writes the output directly.  When the
// caller gives no scratch, the splits of a group form a thread-block cluster (up to 16 CTAs)
// and merge through distributed shared memory instead: no scratch, no second kernel.
//
// Keys and values go from global memory straight into MMA fragments, no shared memory:
//  * S = Q K^T contracts over head dims.  A permutation of the contraction index applied
//    to both operands changes nothing, so lane (g, t) of the m16n8k16 fragment owns the
//    CONTIGUOUS dims [t*HD/4, (t+1)*HD/4) of key g: one or more 16-byte loads, and four
//    lanes cover a whole row.
//  * O = P V contracts over keys, and a B fragment register holds two adjacent KEYS of
//    one dim, while memory is contiguous along dims.  Lane (g, t) loads the contiguous
//    dims [g*HD/8, (g+1)*HD/8) of keys 2t, 2t+1, 2t+8, 2t+9 and pairs the keys with
//    byte permutes; the permutation of the output dims this implies is undone at the store.
// Masked keys (beyond a row's position, before its window, outside the sequence) are
// never loaded: their fragments are zero and their scores -inf, so stale or non-finite
// memory in unowned slots cannot reach the result.
//
// Formula: pyre/model.py:104-124, pyre/kernels/paged_attn.py:43-71 (online softmax, fp32
// scores; probabilities rounded to the activation dtype before the product with V, as
// pyre/model.py:122 does).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int WARPS = 4;
constexpr int TILE = 16;  // keys per tile

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Load N 32-bit words from p (aligned to the widest vector that divides N words).
template <int N>
__device__ __forceinline__ void load_words(uint32_t (&dst)[N], const void* p) {
    if constexpr (N % 4 == 0) {
        const uint4* s = reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            uint4 v = __ldg(s + i);
            dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
        }
    } else if constexpr (N % 2 == 0) {
        const uint2* s = reinterpret_cast<const uint2*>(p);
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            uint2 v = __ldg(s + i);
            dst[2 * i] = v.x; dst[2 * i + 1] = v.y;
        }
    } else {
        const uint32_t* s = reinterpret_cast<const uint32_t*>(p);
#pragma unroll
        for (int i = 0; i < N; ++i) dst[i] = __ldg(s + i);
    }
}

template <int N>
__device__ __forceinline__ void zero_words(uint32_t (&dst)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) dst[i] = 0u;
}

struct AttnParams {
    const __nv_bfloat16* q;      // [T, nh, HD]
    const __nv_bfloat16* cache;  // layer: [page][2][nkv][page_size][HD]
    __nv_bfloat16* out;          // [T, nh * HD]
    float* part_acc;             // [T, nh, n_splits, HD]   (n_splits > 1)
    float* part_ml;              // [T, nh, n_splits, 2]
    const int* block_table;      // [B, bt_stride]
    const int* cu_seqlens;       // [B + 1]
    const int* positions;        // [T]
    int bt_stride, n_seqs, nh, nkv, page_size, window, n_splits, tpg, hpg, head_blocks;
    int max_len;                 // > 0: only entries with at most this many tokens (longer ones go to the prefill kernel)
    float scale;
};

// CLUSTER: the n_splits CTAs of a (group, kv head) form one thread-block cluster and merge their
// partial results through distributed shared memory; no scratch, no second kernel.
template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_mma_kernel(const AttnParams p) {
    constexpr int KW = HD / 8;    // 32-bit words of K per lane per key   (HD/4 dims)
    constexpr int VW = HD / 16;   // 32-bit words of V per lane per key   (HD/8 dims)
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;  // output n-tiles
    __shared__ float sm_o[WARPS][16][HD + 1];
    __shared__ float sm_m[WARPS][16];
    __shared__ float sm_l[WARPS][16];
    __shared__ float sm_cm[16], sm_cl[16];   // this CTA's merged (max, sum) per row, read by its cluster peers

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    pdl_trigger();
    pdl_wait();   // queries, the pages of this step and the step's index arrays come from earlier kernels

    // ---- which group is this CTA's?  groups are counted entry by entry
    int grp = blockIdx.x, seq = -1, tok0 = 0, n_tok = 0;
    for (int b = 0; b < p.n_seqs; ++b) {
        const int begin = p.cu_seqlens[b], len = p.cu_seqlens[b + 1] - begin;
        if (p.max_len > 0 && len > p.max_len) continue;
        const int ng = (len + p.tpg - 1) / p.tpg;
        if (grp < ng) {
            seq = b;
            tok0 = begin + grp * p.tpg;
            n_tok = min(p.tpg, len - grp * p.tpg);
            break;
        }
        grp -= ng;
    }
    if (seq < 0) return;  // the grid is an upper bound
    const int kvh = blockIdx.y / p.head_blocks, hb = blockIdx.y % p.head_blocks;
    const int n_rep = p.nh / p.nkv;
    const int split = blockIdx.z;

    // ---- rows g and g + 8 of this lane: (token, head), causal limit, window start
    int row_tok[2], row_head[2], row_pos[2], row_lo[2];
    bool row_ok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        const int ti = row / p.hpg, hi = row % p.hpg;
        const int h_in_kv = hb * p.hpg + hi;
        row_ok[r] = ti < n_tok && ti < p.tpg && h_in_kv < n_rep;
        row_tok[r] = tok0 + (row_ok[r] ? ti : 0);
        row_head[r] = kvh * n_rep + (row_ok[r] ? h_in_kv : 0);
        row_pos[r] = p.positions[row_tok[r]];
        row_lo[r] = (p.window > 0 && row_pos[r] - p.window + 1 > 0) ? row_pos[r] - p.window + 1 : 0;
    }
    const int pos_first = p.positions[tok0], pos_last = p.positions[tok0 + n_tok - 1];
    const int lo_g = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int tile_lo = lo_g / TILE, tile_hi = pos_last / TILE;
    const int tiles_total = tile_hi - tile_lo + 1;
    const int tps = (tiles_total + p.n_splits - 1) / p.n_splits;
    const int tile_begin = tile_lo + split * tps;
    const int tile_end = min(tile_begin + tps, tile_hi + 1);

    // ---- Q fragments: lane (g, t) holds dims [t*HD/4, (t+1)*HD/4) of rows g and g + 8
    uint32_t qw[2][KW];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (row_ok[r]) load_words<KW>(qw[r], p.q + ((size_t)row_tok[r] * p.nh + row_head[r]) * HD + t * (HD / 4));
        else zero_words<KW>(qw[r]);
    }

    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int* table = p.block_table + (size_t)seq * p.bt_stride;
    const size_t kv_stride = (size_t)p.nkv * p.page_size * HD;  // K block -> V block of a page

    // Page numbers of a tile's six rows (two for K, four for V) are read one tile ahead, so
    // that the dependent loads of keys and values never wait for the block table.
    auto tile_pages = [&](int kt, int (&pk)[2], int (&pv)[4]) {
        const int key0 = kt * TILE;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int key = key0 + 8 * i + g;
            pk[i] = (kt < tile_end && key >= lo_g && key <= pos_last) ? table[key / p.page_size] : -1;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = key0 + 2 * t + (i & 1) + 8 * (i >> 1);
            pv[i] = (kt < tile_end && key >= lo_g && key <= pos_last) ? table[key / p.page_size] : -1;
        }
    };
    int pk_next[2], pv_next[4];
    tile_pages(tile_begin + warp, pk_next, pv_next);

    for (int kt = tile_begin + warp; kt < tile_end; kt += WARPS) {
        const int key0 = kt * TILE;
        int pk[2], pv[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) pk[i] = pk_next[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) pv[i] = pv_next[i];
        // ---- K: keys key0 + 8 i + g, i = 0, 1
        uint32_t kw[2][KW];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int key = key0 + 8 * i + g;
            if (pk[i] >= 0) {
                const size_t row = ((size_t)(pk[i] * 2) * p.nkv + kvh) * p.page_size + key % p.page_size;
                load_words<KW>(kw[i], p.cache + row * HD + t * (HD / 4));
            } else {
                zero_words<KW>(kw[i]);
            }
        }
        // ---- V: keys key0 + 2t + {0, 1, 8, 9}, dims [g*HD/8, (g+1)*HD/8)
        uint32_t vw[4][VW];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = key0 + 2 * t + (i & 1) + 8 * (i >> 1);
            if (pv[i] >= 0) {
                const size_t row = ((size_t)(pv[i] * 2) * p.nkv + kvh) * p.page_size + key % p.page_size;
                load_words<VW>(vw[i], p.cache + kv_stride + row * HD + g * (HD / 8));
            } else {
                zero_words<VW>(vw[i]);
            }
        }
        tile_pages(kt + WARPS, pk_next, pv_next);
        // ---- S = Q K^T
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int j = 0; j < KSTEPS; ++j) {
                const uint32_t a[4] = {qw[0][2 * j], qw[1][2 * j], qw[0][2 * j + 1], qw[1][2 * j + 1]};
                mma_bf16_16816(s[i], a, kw[i][2 * j], kw[i][2 * j + 1]);
            }
        }
        // ---- mask, scale, online softmax (rows g: c = 0, 1; rows g + 8: c = 2, 3)
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int r = c >> 1;
                const int key = key0 + 8 * i + 2 * t + (c & 1);
                const bool ok = row_ok[r] && key <= row_pos[r] && key >= row_lo[r];
                s[i][c] = ok ? s[i][c] * p.scale : -INFINITY;
                tile_max[r] = fmaxf(tile_max[r], s[i][c]);
            }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
            tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
            const float m_new = fmaxf(m_run[r], tile_max[r]);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[r] = expf(m_run[r] - m_use);
            m_run[r] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[i][2 * r] = expf(s[i][2 * r] - m_use);
                s[i][2 * r + 1] = expf(s[i][2 * r + 1] - m_use);
                sum += s[i][2 * r] + s[i][2 * r + 1];
            }
            l_run[r] = l_run[r] * alpha[r] + sum;  // this lane's share; the quad is summed at the end
        }
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        // ---- O += P V
        const uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                                pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            const int c = i >> 1;
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;  // high or low halves of two words
            const uint32_t b0 = __byte_perm(vw[0][c], vw[1][c], sel);
            const uint32_t b1 = __byte_perm(vw[2][c], vw[3][c], sel);
            mma_bf16_16816(o[i], pa, b0, b1);
        }
    }

    // ---- merge the warps of the CTA
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        if (t == 0) {
            sm_m[warp][g + 8 * r] = m_run[r];
            sm_l[warp][g + 8 * r] = l_run[r];
        }
    }
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int dim = (2 * t + (c & 1)) * (HD / 8) + i;  // undo the dim permutation of the V fragments
            sm_o[warp][g + 8 * (c >> 1)][dim] = o[i][c];
        }
    __syncthreads();

    for (int e = threadIdx.x; e < 16 * HD; e += WARPS * 32) {
        const int row = e / HD, d = e % HD;
        const int ti = row / p.hpg, hi = row % p.hpg;
        const int h_in_kv = hb * p.hpg + hi;
        if (!(ti < n_tok && ti < p.tpg && h_in_kv < n_rep)) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w][row]);
        const float m_use = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = expf(sm_m[w][row] - m_use);
            L += sm_l[w][row] * f;
            O += sm_o[w][row][d] * f;
        }
        const size_t th = (size_t)(tok0 + ti) * p.nh + (kvh * n_rep + h_in_kv);
        if (p.n_splits == 1) {
            p.out[th * HD + d] = __float2bfloat16_rn(O / L);
        } else if constexpr (CLUSTER) {
            // keep this CTA's merged partial in its own shared memory: element (row, d) of warp
            // slot 1 is read by this thread only, so it can be overwritten now; the row's max
            // and sum are read by many threads and get arrays of their own
            sm_o[1][row][d] = O;
            if (d == 0) { sm_cm[row] = M; sm_cl[row] = L; }
        } else {
            p.part_acc[(th * p.n_splits + split) * HD + d] = O;
            if (d == 0) {
                p.part_ml[(th * p.n_splits + split) * 2] = M;
                p.part_ml[(th * p.n_splits + split) * 2 + 1] = L;
            }
        }
    }
    if constexpr (CLUSTER) {
        if (p.n_splits > 1) {
            cg::cluster_group cluster = cg::this_cluster();
            cluster.sync();
            const int n = p.n_splits, rank = (int)cluster.block_rank();
            for (int e = threadIdx.x * n + rank; e < 16 * HD; e += WARPS * 32 * n) {
                const int row = e / HD, d = e % HD;
                const int ti = row / p.hpg, hi = row % p.hpg;
                const int h_in_kv = hb * p.hpg + hi;
                if (!(ti < n_tok && ti < p.tpg && h_in_kv < n_rep)) continue;
                float M = -INFINITY;
                for (int c = 0; c < n; ++c) M = fmaxf(M, *cluster.map_shared_rank(&sm_cm[row], c));
                const float m_use = (M == -INFINITY) ? 0.f : M;
                float L = 0.f, O = 0.f;
                for (int c = 0; c < n; ++c) {
                    const float f = expf(*cluster.map_shared_rank(&sm_cm[row], c) - m_use);
                    L += *cluster.map_shared_rank(&sm_cl[row], c) * f;
                    O += *cluster.map_shared_rank(&sm_o[1][row][d], c) * f;
                }
                const size_t th = (size_t)(tok0 + ti) * p.nh + (kvh * n_rep + h_in_kv);
                p.out[th * HD + d] = __float2bfloat16_rn(O / L);
            }
            cluster.sync();   // nobody leaves while a peer may still read its shared memory
        }
    }
}

// out[t, h, :] = sum_s acc_s exp(m_s - M) / sum_s l_s exp(m_s - M)
__global__ void combine_splits_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                      __nv_bfloat16* __restrict__ out, int n_splits, int hd, int nh,
                                      const int* __restrict__ cu_seqlens, int n_seqs, int max_len) {
    pdl_trigger();
    pdl_wait();
    const size_t th = blockIdx.x;
    if (max_len > 0) {
        // rows of entries longer than max_len belong to the prefill kernel: no partials, nothing to do
        const int tok = (int)(th / nh);
        for (int b = 0; b < n_seqs; ++b)
            if (tok < cu_seqlens[b + 1]) {
                if (cu_seqlens[b + 1] - cu_seqlens[b] > max_len) return;
                break;
            }
    }
    const float* ml = part_ml + th * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
    const float m_use = (M == -INFINITY) ? 0.f : M;
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) L += ml[2 * s + 1] * expf(ml[2 * s] - m_use);
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float O = 0.f;
        for (int s = 0; s < n_splits; ++s) O += part_acc[(th * n_splits + s) * hd + d] * expf(ml[2 * s] - m_use);
        out[th * hd + d] = __float2bfloat16_rn(O / L);
    }
}

template <int HD>
int launch(const AttnParams& p, int n_groups_bound, bool use_cluster, cudaStream_t stream) {
    dim3 grid(n_groups_bound, p.nkv * p.head_blocks, p.n_splits);
    if (!use_cluster) {
        pyre_launch(paged_attention_mma_kernel<HD, false>, dim3(grid), dim3(WARPS * 32), 0, stream, p);
        return (int)cudaGetLastError();
    }
    static bool configured = false;
    if (!configured) {   // clusters of more than 8 CTAs are an opt-in
        cudaError_t e = cudaFuncSetAttribute(paged_attention_mma_kernel<HD, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = p.n_splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pyre_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, paged_attention_mma_kernel<HD, true>, p);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

}  // namespace

// Scratch floats needed for `n_splits` > 1: acc [T, nh, n_splits, hd] then ml [T, nh, n_splits, 2].
PYRE_API long long pyre_attention_mma_scratch_floats(int n_tokens, int nh, int hd, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * nh * n_splits * (hd + 2);
}

PYRE_API int pyre_paged_attention_mma(const void* q, const void* cache, void* out, float* scratch,
                                      const int* block_table, int bt_stride, const int* cu_seqlens,
                                      const int* positions, int n_tokens, int n_seqs, int nh, int nkv, int hd,
                                      int page_size, int window, float scale, int n_splits, int max_len,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 16 || hd < 16 || hd > 128 || nkv <= 0 || nh % nkv || page_size <= 0 || n_splits < 1) return PYRE_ERR_UNSUPPORTED;
    // without scratch the splits merge through a thread-block cluster (at most 16 CTAs)
    const bool use_cluster = n_splits > 1 && !scratch;
    if (use_cluster && n_splits > 16) return PYRE_ERR_BAD_ARG;
    AttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.cache = (const __nv_bfloat16*)cache;
    p.out = (__nv_bfloat16*)out;
    p.part_acc = scratch;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * nh * n_splits * hd : nullptr;
    p.block_table = block_table;
    p.cu_seqlens = cu_seqlens;
    p.positions = positions;
    p.bt_stride = bt_stride; p.n_seqs = n_seqs; p.nh = nh; p.nkv = nkv; p.page_size = page_size;
    p.window = window; p.n_splits = n_splits; p.scale = scale; p.max_len = max_len;
    const int n_rep = nh / nkv;
    p.hpg = n_rep < 16 ? n_rep : 16;
    p.tpg = 16 / p.hpg;
    p.head_blocks = (n_rep + p.hpg - 1) / p.hpg;
    const int groups_bound = n_tokens / p.tpg + n_seqs;  // sum over entries of ceil(len / tpg) is at most this
    int rc;
    switch (hd) {
        case 16: rc = launch<16>(p, groups_bound, use_cluster, stream); break;
        case 32: rc = launch<32>(p, groups_bound, use_cluster, stream); break;
        case 48: rc = launch<48>(p, groups_bound, use_cluster, stream); break;
        case 64: rc = launch<64>(p, groups_bound, use_cluster, stream); break;
        case 80: rc = launch<80>(p, groups_bound, use_cluster, stream); break;
        case 96: rc = launch<96>(p, groups_bound, use_cluster, stream); break;
        case 112: rc = launch<112>(p, groups_bound, use_cluster, stream); break;
        case 128: rc = launch<128>(p, groups_bound, use_cluster, stream); break;
        default: return PYRE_ERR_UNSUPPORTED;
    }
    if (rc) return rc;
    if (n_splits > 1 && !use_cluster) {
        pyre_launch(combine_splits_kernel, dim3(n_tokens * nh), dim3(hd >= 64 ? 64 : 32), 0, stream, p.part_acc, p.part_ml, p.out, n_splits, hd, nh, cu_seqlens, n_seqs, max_len);
        PYRE_LAUNCH_CHECK();
    }
    return 0;
}
