// Paged attention for prompt portions in bfloat16: 64 queries of one head per CTA, keys and
// values staged in shared memory by cp.async (double-buffered, 64 keys per tile), tensor-core
// products with ldmatrix-fed fragments, online softmax in fp32.
//
// A CTA owns 64 consecutive tokens of one portion (entry of the step) and one query head;
// its 4 warps own 16 query rows each and walk the same key tiles, from the tile that holds
// the start of the first row's window to the tile that holds the last row's position.  A
// tile is read from the paged cache row by row through the block table; rows beyond the
// portion's last position are zero-filled, so unowned cache slots never enter the math.
// Only entries with at least `min_len` tokens are handled here; shorter ones (decoded
// tokens, tiny portions) go to the split-KV kernel of attention_mma.cu, which the host
// launches with the complementary filter.
//
// Shared-memory tiles are [row][HD] with the 16-byte chunks of a row XOR-swizzled by
// (row & 7), which makes both the cp.async stores and the ldmatrix reads conflict-free.
//
// Formula: pyre/model.py:104-124 (scores = (q k^T) * scale, causal mask from the query's
// absolute position, fp32 softmax, probabilities rounded to the activation dtype, times v).
#include "common.cuh"

namespace {

constexpr int BM = 64;      // queries per CTA
constexpr int BN = 64;      // keys per tile
constexpr int WARPS = 4;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct PrefillParams {
    const __nv_bfloat16* q;      // [T, nh, HD]
    const __nv_bfloat16* cache;  // layer: [page][2][nkv][page_size][HD]
    __nv_bfloat16* out;          // [T, nh * HD]
    const int* block_table;      // [B, bt_stride]
    const int* cu_seqlens;       // [B + 1]
    const int* positions;        // [T]
    int bt_stride, n_seqs, nh, nkv, page_size, window, min_len;
    float scale;
    long long n_pages;           // pages of the pool (0 = not known) and the device's error word: for the debug checks
    int* err_flag;
};

template <int HD>
__global__ void __launch_bounds__(WARPS * 32, 3) attention_prefill_kernel(const PrefillParams p) {
    constexpr int CH = HD / 8;                 // 16-byte chunks per row
    constexpr int TILE_BYTES = BN * HD * 2;
    extern __shared__ __align__(128) uint8_t smem[];   // [2 stages][K tile, V tile]
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    pdl_trigger();
    pdl_wait();   // queries, pages and index arrays come from earlier kernels of the step

    // ---- which 64-token tile of which entry is this CTA's?  (entries shorter than min_len are skipped)
    // CTAs start in the order of blockIdx.x; the last tile of a portion sees the most keys, so
    // tiles are numbered from the end of each portion (longest work first, short tail last).
    int tile = blockIdx.x, seq = -1, tok0 = 0, n_tok = 0;
    for (int b = 0; b < p.n_seqs; ++b) {
        const int begin = p.cu_seqlens[b], len = p.cu_seqlens[b + 1] - begin;
        if (len < p.min_len) continue;
        const int nt = (len + BM - 1) / BM;
        if (tile < nt) {
            const int qt = nt - 1 - tile;
            seq = b;
            tok0 = begin + qt * BM;
            n_tok = min(BM, len - qt * BM);
            break;
        }
        tile -= nt;
    }
    if (seq < 0) return;
    const int head = blockIdx.y;
    const int kvh = head / (p.nh / p.nkv);
    const int* table = p.block_table + (size_t)seq * p.bt_stride;

    // ---- this lane's two query rows
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const bool ok0 = r0 < n_tok, ok1 = r1 < n_tok;
    const int pos0 = p.positions[tok0 + (ok0 ? r0 : 0)], pos1 = p.positions[tok0 + (ok1 ? r1 : 0)];
    const int lo0 = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int lo1 = (p.window > 0 && pos1 - p.window + 1 > 0) ? pos1 - p.window + 1 : 0;
    const int pos_first = p.positions[tok0], pos_last = p.positions[tok0 + n_tok - 1];
    const int lo_cta = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int tile_lo = lo_cta / BN, tile_hi = pos_last / BN;
    // rows of this warp: positions pos_first + 16 warp .. + 15 (consecutive tokens of one entry)
    const int warp_pos_lo = pos_first + warp * 16, warp_pos_hi = min(pos_first + warp * 16 + 15, pos_last);
    const int warp_key_lo = (p.window > 0 && warp_pos_lo - p.window + 1 > 0) ? warp_pos_lo - p.window + 1 : 0;

    // ---- Q fragments straight from global memory (once)
    uint32_t qa[HD / 16][4];
    {
        const __nv_bfloat16* q0 = p.q + ((size_t)(tok0 + (ok0 ? r0 : 0)) * p.nh + head) * HD;
        const __nv_bfloat16* q1 = p.q + ((size_t)(tok0 + (ok1 ? r1 : 0)) * p.nh + head) * HD;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
            qa[k][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * k + 2 * t) : 0u;
            qa[k][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * k + 2 * t) : 0u;
            qa[k][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * k + 8 + 2 * t) : 0u;
            qa[k][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * k + 8 + 2 * t) : 0u;
        }
    }

    // ---- tile loader: 64 rows x CH chunks for K and for V; thread i copies chunk (i % CH) of rows i / CH + j * (128 / CH)
    auto load_tile = [&](int kt, int stage) {
        const uint32_t k_dst = smem_base + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
        constexpr int ROWS_PER_PASS = WARPS * 32 / CH;
        const int c = threadIdx.x % CH, rr = threadIdx.x / CH;
#pragma unroll
        for (int j = 0; j < BN / ROWS_PER_PASS; ++j) {
            const int row = rr + j * ROWS_PER_PASS;
            const int key = kt * BN + row;
            const bool live = key >= lo_cta && key <= pos_last;
            const int page = live ? pyre_checked_page(table[key / p.page_size], p.n_pages, p.err_flag) : 0;
            const size_t krow = ((size_t)(page * 2) * p.nkv + kvh) * p.page_size + (live ? key % p.page_size : 0);
            const __nv_bfloat16* ksrc = p.cache + krow * HD + c * 8;
            const __nv_bfloat16* vsrc = ksrc + (size_t)p.nkv * p.page_size * HD;
            const uint32_t off = row * (HD * 2) + ((c ^ (row & 7)) * 16);
            cp_async_16(k_dst + off, ksrc, live ? 16 : 0);
            cp_async_16(v_dst + off, vsrc, live ? 16 : 0);
        }
    };

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sl2 = p.scale * 1.44269504088896341f;   // scores are kept in units of log2(e)

    load_tile(tile_lo, 0);
    cp_async_commit();
    for (int kt = tile_lo; kt <= tile_hi; ++kt) {
        const int stage = (kt - tile_lo) & 1;
        if (kt < tile_hi) load_tile(kt + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const int key0 = kt * BN;
        // this warp needs the tile only if it holds a key that one of its rows may see
        if (key0 <= warp_pos_hi && key0 + BN - 1 >= warp_key_lo && warp * 16 < n_tok) {
            const uint32_t k_tile = smem_base + stage * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
            // ---- S = Q K^T : 8 key n-tiles
            float s[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
                // the four fragment loads of a k-step go out together, then its eight products
                uint32_t b[BN / 16][4];
#pragma unroll
                for (int n = 0; n < BN / 16; ++n) {
                    // matrices: (keys n*16 + 0..7 | 8..15) x (dims 16k + 0..7 | 8..15)
                    const int mi = lane >> 3;
                    const int row = n * 16 + (mi >> 1) * 8 + (lane & 7);
                    const int ch = 2 * k + (mi & 1);
                    ldmatrix_x4(b[n], k_tile + row * (HD * 2) + ((ch ^ (row & 7)) * 16));
                }
#pragma unroll
                for (int n = 0; n < BN / 16; ++n) {
                    mma_bf16_16816(s[2 * n], qa[k], b[n][0], b[n][1]);
                    mma_bf16_16816(s[2 * n + 1], qa[k], b[n][2], b[n][3]);
                }
            }
            // ---- mask (only tiles that touch a row's limits), online softmax.  The maximum is taken
            // on the raw scores (the scale is positive) in four independent chains; the scale and
            // the maximum enter the exponent through one fused multiply-add; the accumulator is
            // rescaled only when some row's maximum moved.
            const bool need_mask = key0 + BN - 1 > warp_pos_lo || (p.window > 0 && key0 < warp_key_lo + 15) || !ok0 || !ok1;
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < BN / 8; ++i)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int key = key0 + 8 * i + 2 * t + (c & 1);
                        const bool okk = (c < 2) ? (ok0 && key <= pos0 && key >= lo0) : (ok1 && key <= pos1 && key >= lo1);
                        s[i][c] = okk ? s[i][c] : -INFINITY;
                    }
            }
            float tm[2][4];
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int q = 0; q < 4; ++q) tm[r][q] = fmaxf(s[q][2 * r], s[q][2 * r + 1]);
#pragma unroll
            for (int i = 4; i < BN / 8; ++i)
#pragma unroll
                for (int r = 0; r < 2; ++r) tm[r][i & 3] = fmaxf(tm[r][i & 3], fmaxf(s[i][2 * r], s[i][2 * r + 1]));
            float alpha[2] = {1.f, 1.f};
            bool moved = false;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float tmax = fmaxf(fmaxf(tm[r][0], tm[r][1]), fmaxf(tm[r][2], tm[r][3])) * sl2;   // base-2 units
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run[r], tmax);
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                if (m_new != m_run[r]) {
                    alpha[r] = exp2f(m_run[r] - m_use);
                    moved = true;
                }
                m_run[r] = m_new;
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < BN / 8; ++i) {
                    s[i][2 * r] = exp2f(fmaf(s[i][2 * r], sl2, -m_use));
                    s[i][2 * r + 1] = exp2f(fmaf(s[i][2 * r + 1], sl2, -m_use));
                    sum[i & 3] += s[i][2 * r] + s[i][2 * r + 1];
                }
                l_run[r] = l_run[r] * alpha[r] + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
            }
            if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                    o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
            // ---- O += P V : 4 key k-steps x HD/8 dim n-tiles
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                const uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                        pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int d0 = 0; d0 < HD / 16; d0 += 4) {
                    uint32_t b[4][4];
#pragma unroll
                    for (int dd = 0; dd < 4; ++dd) {
                        // matrices (stored [key][dim], read transposed): (keys 16kk + 0..7 | 8..15) x (dims 16d + 0..7 | 8..15)
                        const int d = d0 + dd;
                        const int mi = lane >> 3;
                        const int row = kk * 16 + (mi & 1) * 8 + (lane & 7);
                        const int ch = 2 * d + (mi >> 1);
                        ldmatrix_x4_trans(b[dd], v_tile + row * (HD * 2) + ((ch ^ (row & 7)) * 16));
                    }
#pragma unroll
                    for (int dd = 0; dd < 4; ++dd) {
                        mma_bf16_16816(o[2 * (d0 + dd)], pa, b[dd][0], b[dd][1]);
                        mma_bf16_16816(o[2 * (d0 + dd) + 1], pa, b[dd][2], b[dd][3]);
                    }
                }
            }
        }
        __syncthreads();   // the stage is overwritten by the load issued in the next iteration
    }

    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = ok0 ? 1.0f / l_run[0] : 0.f, inv1 = ok1 ? 1.0f / l_run[1] : 0.f;
    __nv_bfloat16* out0 = p.out + ((size_t)(tok0 + (ok0 ? r0 : 0)) * p.nh + head) * HD;
    __nv_bfloat16* out1 = p.out + ((size_t)(tok0 + (ok1 ? r1 : 0)) * p.nh + head) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        if (ok0) *reinterpret_cast<uint32_t*>(out0 + 8 * i + 2 * t) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (ok1) *reinterpret_cast<uint32_t*>(out1 + 8 * i + 2 * t) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

template <int HD>
int launch(const PrefillParams& p, int tiles_bound, cudaStream_t stream) {
    constexpr int SMEM = 2 * 2 * BN * HD * 2;
    static bool configured_on[PYRE_MAX_DEVICES] = {};      // the attributes are per device
    bool& configured = configured_on[pyre_current_device()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = pyre_launch(attention_prefill_kernel<HD>, dim3(tiles_bound, p.nh), dim3(WARPS * 32), (size_t)SMEM, stream, p);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

}  // namespace

// Attention of every entry with at least min_len tokens (others are left untouched).  bfloat16,
// head sizes 64 and 128.  n_long_tokens: total tokens of those entries (bounds the grid).
PYRE_API int pyre_attention_prefill(const void* q, const void* cache, void* out, const int* block_table, int bt_stride,
                                    const int* cu_seqlens, const int* positions, int n_long_tokens, int n_seqs, int nh,
                                    int nkv, int hd, int page_size, int window, float scale, int min_len,
                                    long long n_pages, int* err_flag, cudaStream_t stream) {
    if (n_long_tokens <= 0) return 0;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || page_size <= 0 || min_len < 1) return PYRE_ERR_UNSUPPORTED;
    PrefillParams p;
    p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.bt_stride = bt_stride; p.n_seqs = n_seqs; p.nh = nh; p.nkv = nkv; p.page_size = page_size;
    p.window = window; p.min_len = min_len; p.scale = scale; p.n_pages = n_pages; p.err_flag = err_flag;
    const int tiles_bound = n_long_tokens / BM + n_seqs;
    return hd == 128 ? launch<128>(p, tiles_bound, stream) : launch<64>(p, tiles_bound, stream);
}
