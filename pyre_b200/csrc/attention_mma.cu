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
// and merge through distributed shared memory instead: every CTA pushes its partial to the
// CTA that owns the output dims (remote stores, nobody waits for a remote load), one cluster
// barrier makes them visible, and each CTA reduces and writes its dims.  No scratch, no
// second kernel.
//
// Each warp owns a three-stage ring in shared memory, so two tiles are in flight while it
// computes on a third.  With power-of-two pages and head sizes that are multiples of 64 the
// tiles come by TMA; with pages of 16 tokens or more one 5-d tensor copy brings a whole tile
// ([K, V] x [column boxes] x [16 rows] x [64 columns], 128-byte swizzle), and the page numbers
// of a warp's tiles are read 32 at a time, one per lane.  Other sizes use cp.async copies
// (16 keys and 16 values, row by row through the block table in 16-byte chunks) with rows
// XOR-swizzled by chunk, so that the copies and the ldmatrix reads (plain for K, transposed
// for V) do not collide on banks.  Masked keys (beyond a row's position, before its window,
// outside the sequence) get a score of -inf and their value rows are zero (zero-filled by
// cp.async, zeroed in shared memory after a TMA copy), so stale or non-finite memory in
// unowned slots cannot reach the result.
//
// Formula: pyre/model.py:104-124, pyre/kernels/paged_attn.py:43-71 (online softmax, fp32
// scores; probabilities rounded to the activation dtype before the product with V, as
// pyre/model.py:122 does).
#include <cooperative_groups.h>
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int WARPS = 4;
constexpr int TILE = 16;  // keys per tile
constexpr int STAGES = 3; // tiles in flight per warp

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

// ---- TMA pieces (tiles of power-of-two pages, head sizes that are multiples of 64)
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// 2^x on the special-function unit (results below 2^-126 become 0; 2^-inf = 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr int ERR_ATTN_TIMEOUT = 3;

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
    int page_shift;              // log2(page_size) if it is a power of two, else -1
    int use_tma;                 // tiles come by TMA through `map` (power-of-two pages, HD % 64 == 0): 1 = one copy per
                                 // 128-byte column box, page piece and K/V (pages under 16 tokens), 2 = one 5-d copy per tile
    int box_rows;                // rows per TMA box: min(16, page_size)
    int* err_flag;
    long long n_pages;           // pages of the pool (0 = not known); read by the debug checks only
    int uniform_len;             // > 0: every entry has exactly this many tokens (a decode step): no scan for the group
    int max_len;                 // > 0: only entries with at most this many tokens (longer ones go to the prefill kernel)
    float scale;
};

// CLUSTER: the n_splits CTAs of a (group, kv head) form one thread-block cluster and merge their
// partial results through distributed shared memory; no scratch, no second kernel.
template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32) paged_attention_mma_kernel(const __grid_constant__ CUtensorMap map, const AttnParams p) {
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;  // output n-tiles
    constexpr int CH = HD / 8;    // 16-byte chunks per row
    constexpr int SWZ = (CH % 8 == 0) ? 7 : (CH % 4 == 0) ? 3 : (CH % 2 == 0) ? 1 : 0;   // XOR mask that stays inside a row
    constexpr int TILE_BYTES = TILE * HD * 2;          // one K (or V) tile
    constexpr int WARP_BYTES = STAGES * 2 * TILE_BYTES;   // the stages of K + V
    static_assert(16 * (HD + 1) * 4 <= WARP_BYTES, "the merge buffer of a warp must fit into its ring");
    // a warp's ring is dead once its key loop is over; its merge buffer sm_o[warp] reuses the space
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 128B-swizzled boxes must start on 1024-byte boundaries
    uint8_t* smem_dyn = smem_raw + ((1024u - ((uint32_t)__cvta_generic_to_shared(smem_raw) & 1023u)) & 1023u);
    __shared__ float sm_m[WARPS][16];
    __shared__ float sm_l[WARPS][16];
    // cluster merge: partials pushed by the peers, [rank][row][dims owned by this CTA] and [rank][row][max, sum];
    // n * ceil(HD / n) <= HD + 15 dims in all
    __shared__ __align__(16) float rx_o[CLUSTER ? 16 * (HD + 16) : 4];
    __shared__ __align__(16) float rx_ml[CLUSTER ? 16 * 16 * 2 : 4];
    __shared__ int sm_th[16];                // per row: token * nh + head of its output row, or -1
    __shared__ __align__(8) uint64_t tma_bar[WARPS][STAGES];   // per warp and stage: "the tile has landed"
    auto sm_o = [&](int w, int row, int d) -> float& {
        return reinterpret_cast<float*>(smem_dyn + (size_t)w * WARP_BYTES)[row * (HD + 1) + d];
    };

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    if constexpr (CLUSTER) (void)cg::this_cluster().barrier_arrive();   // phase 1 ("this CTA runs"), awaited before the merge
    pdl_trigger();
    // What follows until pdl_wait() reads only what no kernel of this step writes: the step's index arrays
    // (copied from the host before the step's first kernel) and keys and values of EARLIER steps.  The
    // queries, and the keys and values of this step's own tokens, are touched after the wait.

    // ---- which group is this CTA's?  groups are counted entry by entry
    int grp = blockIdx.x, seq = -1, tok0 = 0, n_tok = 0, seq_begin = 0;
    if (p.uniform_len > 0) {
        const int ng = (p.uniform_len + p.tpg - 1) / p.tpg;
        const int b = grp / ng, gi = grp % ng;
        if (b < p.n_seqs) {
            seq = b;
            seq_begin = b * p.uniform_len;
            tok0 = seq_begin + gi * p.tpg;
            n_tok = min(p.tpg, p.uniform_len - gi * p.tpg);
        }
    } else
    for (int b = 0; b < p.n_seqs; ++b) {
        const int begin = p.cu_seqlens[b], len = p.cu_seqlens[b + 1] - begin;
        if (p.max_len > 0 && len > p.max_len) continue;
        const int ng = (len + p.tpg - 1) / p.tpg;
        if (grp < ng) {
            seq = b;
            seq_begin = begin;
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
    const int new_from = p.positions[seq_begin];   // the sequence's keys from here on are written by this step
    const int lo_g = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int tile_lo = lo_g / TILE, tile_hi = pos_last / TILE;
    const int tiles_total = tile_hi - tile_lo + 1;
    const int tps = (tiles_total + p.n_splits - 1) / p.n_splits;
    const int tile_begin = tile_lo + split * tps;
    const int tile_end = min(tile_begin + tps, tile_hi + 1);

    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int* table = p.block_table + (size_t)seq * p.bt_stride;
    const size_t kv_stride = (size_t)p.nkv * p.page_size * HD;  // K block -> V block of a page
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem_dyn) + warp * WARP_BYTES;

    // copy tile kt (16 keys, 16 values) into a stage of this warp's ring; chunk i of the
    // 16 * CH chunks of a tile belongs to row i / CH
    auto load_tile = [&](int kt, int stage) {
        const uint32_t k_dst = ring + stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
#pragma unroll
        for (int i = lane; i < TILE * CH; i += 32) {
            const int row = i / CH, c = i % CH;
            const int key = kt * TILE + row;
            const bool live = key >= lo_g && key <= pos_last;
            const int lp = p.page_shift >= 0 ? key >> p.page_shift : key / p.page_size;
            const int slot = p.page_shift >= 0 ? key & (p.page_size - 1) : key % p.page_size;
            const int page = live ? pyre_checked_page(table[lp], p.n_pages, p.err_flag) : 0;
            const size_t krow = ((size_t)(page * 2) * p.nkv + kvh) * p.page_size + (live ? slot : 0);
            const __nv_bfloat16* ksrc = p.cache + krow * HD + c * 8;
            const uint32_t off = row * (HD * 2) + ((c ^ (row & SWZ)) * 16);
            cp_async_16(k_dst + off, ksrc, live ? 16 : 0);
            cp_async_16(v_dst + off, ksrc + kv_stride, live ? 16 : 0);
        }
    };

    // TMA variant: one lane brings a tile with a few bulk tensor copies.  A tile is HD / 64
    // column boxes of 128 bytes (the swizzle span) for K and for V, each 16 / box_rows row
    // pieces (one piece per page the tile touches).  Stage layout: [K col 0][K col 1]..[V col 0]..,
    // every box 16 rows x 128 B = 2 KB, 128B-swizzled by the copy engine.
    const bool tma = p.use_tma != 0;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&tma_bar[warp][0]);
    if (tma && lane == 0) {
#pragma unroll
        for (int st = 0; st < STAGES; ++st) mbar_init(bar0 + 8 * st, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // This warp's tiles are tile_begin + warp + WARPS * j, j = 0, 1, ...  With pages of 16 tokens or
    // more a tile lies in one page; lane l then holds the page number of tile j_base + l, read 32
    // tiles at a time (one coalesced look-up instead of one dependent load per tile).
    int pg = 0, j_base = 0;
    auto read_pages = [&](int jb) {
        j_base = jb;
        const int kt2 = tile_begin + warp + WARPS * (jb + lane);
        const int key = kt2 * TILE;
        const bool live = kt2 < tile_end && key + TILE - 1 >= lo_g && key <= pos_last;
        pg = live ? pyre_checked_page(table[key >> p.page_shift], p.n_pages, p.err_flag) : 0;   // a tile wholly outside [lo_g, pos_last] reads page 0 (masked)
    };
    if (p.use_tma == 2) read_pages(0);
    // bring tile number j of this warp into `stage` (the whole warp calls; lane 0 issues)
    auto tma_tile = [&](int j, int stage) {
        const int kt2 = tile_begin + warp + WARPS * j;
        const uint32_t dst = ring + stage * 2 * TILE_BYTES;
        const uint32_t bar = bar0 + 8 * stage;
        if (p.use_tma == 2) {
            // one 5-d copy: [K, V] x [column boxes] x [16 rows] x [64 columns], the layout of a stage
            if (j - j_base >= 32) read_pages(j_base + 32);
            const int page = __shfl_sync(0xffffffffu, pg, j - j_base);
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier generic accesses to the stage come first
                mbar_expect_tx(bar, 2 * TILE_BYTES);
                tma_load_5d(dst, &map, bar, 0, kvh * p.page_size + ((kt2 * TILE) & (p.page_size - 1)), 0, 0, page);
            }
            return;
        }
        if (lane != 0) return;
        // pages under 16 tokens: a tile is HD / 64 column boxes of 128 bytes (the swizzle span) for K
        // and for V, each 16 / box_rows row pieces (one piece per page the tile touches).  Stage layout:
        // [K col 0][K col 1]..[V col 0].., every box 16 rows x 128 B = 2 KB, 128B-swizzled by the copy engine.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar, 2 * TILE_BYTES);
        const int pieces = TILE / p.box_rows;
        for (int pc = 0; pc < pieces; ++pc) {
            const int key = kt2 * TILE + pc * p.box_rows;
            // a piece wholly outside [lo_g, pos_last] still has to be filled: read page 0 (its scores are masked)
            const int lp = key >> p.page_shift;
            const bool live = key + p.box_rows - 1 >= lo_g && key <= pos_last;
            const int page = live ? pyre_checked_page(table[lp], p.n_pages, p.err_flag) : 0;
            const int krow = ((page * 2) * p.nkv + kvh) * p.page_size + (key & (p.page_size - 1));
            const int vrow = krow + p.nkv * p.page_size;
#pragma unroll
            for (int cb = 0; cb < HD / 64; ++cb) {
                tma_load_2d(dst + cb * 2048 + pc * p.box_rows * 128, &map, bar, cb * 64, krow);
                tma_load_2d(dst + TILE_BYTES + cb * 2048 + pc * p.box_rows * 128, &map, bar, cb * 64, vrow);
            }
        }
    };
    // shared-memory address of 16-byte chunk `ch` of row `row` of a tile
    auto chunk_addr = [&](uint32_t tile, int row, int ch) -> uint32_t {
        if (tma) return tile + (ch >> 3) * 2048 + row * 128 + (((ch & 7) ^ (row & 7)) * 16);
        return tile + row * (HD * 2) + ((ch ^ (row & SWZ)) * 16);
    };
    bool timed_out = false;

    const bool upper = __any_sync(0xffffffffu, row_ok[1]);   // does any lane own a valid row among rows 8..15?
    const float sl2 = p.scale * 1.44269504088896341f;        // log2(e): maxima and scores live in base 2

    // ---- the first STAGES - 1 tiles go out before anything else is read: those that hold only keys of
    // earlier steps even before this kernel waits for the kernels before it (their latency, and all of the
    // set-up above, then hide behind the kernel that writes this step's keys)
    const int n_mine = tile_begin + warp < tile_end ? (tile_end - tile_begin - warp + WARPS - 1) / WARPS : 0;
    auto is_old = [&](int j) { return (tile_begin + warp + WARPS * j) * TILE + TILE - 1 < new_from; };
#pragma unroll
    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < n_mine && is_old(j)) {
            if (!tma) load_tile(tile_begin + warp + WARPS * j, j);
            else tma_tile(j, j);
        }
    }
    pdl_wait();
#pragma unroll
    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < n_mine && !is_old(j)) {
            if (!tma) load_tile(tile_begin + warp + WARPS * j, j);
            else tma_tile(j, j);
        }
        cp_async_commit();
    }

    // ---- Q fragments (A operand, natural layout) straight from global memory
    uint32_t qa[KSTEPS][4];
    {
        const __nv_bfloat16* q0 = p.q + ((size_t)row_tok[0] * p.nh + row_head[0]) * HD;
        const __nv_bfloat16* q1 = p.q + ((size_t)row_tok[1] * p.nh + row_head[1]) * HD;
#pragma unroll
        for (int k = 0; k < KSTEPS; ++k) {
            qa[k][0] = row_ok[0] ? *reinterpret_cast<const uint32_t*>(q0 + 16 * k + 2 * t) : 0u;
            qa[k][1] = row_ok[1] ? *reinterpret_cast<const uint32_t*>(q1 + 16 * k + 2 * t) : 0u;
            qa[k][2] = row_ok[0] ? *reinterpret_cast<const uint32_t*>(q0 + 16 * k + 8 + 2 * t) : 0u;
            qa[k][3] = row_ok[1] ? *reinterpret_cast<const uint32_t*>(q1 + 16 * k + 8 + 2 * t) : 0u;
        }
    }

    if constexpr (CLUSTER) {
        // phase 1 of the cluster barrier (every CTA of the cluster runs, so its shared memory may be written
        // by the merge below); waited for here, where the first tiles are still on their way
        if (p.n_splits > 1) cg::this_cluster().barrier_wait();
    }
    for (int it = 0; it < n_mine; ++it) {
        const int kt = tile_begin + warp + WARPS * it;
        const int stage = it % STAGES;
        if (it + STAGES - 1 < n_mine) {   // the stage that was read in the last iteration
            if (!tma) load_tile(kt + WARPS * (STAGES - 1), (it + STAGES - 1) % STAGES);
            else tma_tile(it + STAGES - 1, (it + STAGES - 1) % STAGES);
        }
        cp_async_commit();
        const int key0 = kt * TILE;
        const uint32_t k_tile = ring + stage * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
        if (!tma) {
            cp_async_wait<STAGES - 1>();
        } else {
            const uint32_t parity = (it / STAGES) & 1;
            if (!mbar_try_wait(bar0 + 8 * stage, parity)) {
                const unsigned long long t0 = pyre_now_ns();
                uint32_t spins = 0;
                while (!mbar_try_wait(bar0 + 8 * stage, parity)) {
                    if ((++spins & 255) == 0 && pyre_now_ns() - t0 > PYRE_WAIT_NS) { timed_out = true; break; }
                }
            }
            timed_out = __any_sync(0xffffffffu, timed_out);   // the whole warp gives up together
            if (timed_out) break;
            // the copy engine brought whole rows of the page: rows outside [lo_g, pos_last] may hold
            // anything, so their values are zeroed here (their scores are masked below)
            if (key0 + TILE - 1 > pos_last || key0 < lo_g) {
                for (int i = lane; i < TILE * CH; i += 32) {
                    const int row = i / CH, c = i % CH;
                    const int key = key0 + row;
                    if (key > pos_last || key < lo_g)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(chunk_addr(v_tile, row, c)), "r"(0u) : "memory");
                }
            }
        }
        __syncwarp();       // every lane sees the whole tile
        const int mi = lane >> 3, lr = lane & 7;
        // ---- S = Q K^T: matrices (keys 0..7 | 8..15) x (dims 16k + 0..7 | 8..15)
        // two sets of accumulators (even and odd k-steps) halve the chain of dependent products
        float s[2][4], s2[2][4];
#pragma unroll
        for (int c = 0; c < 4; ++c) { s[0][c] = s[1][c] = s2[0][c] = s2[1][c] = 0.f; }
#pragma unroll
        for (int k = 0; k < KSTEPS; ++k) {
            const int row = (mi >> 1) * 8 + lr;
            const int ch = 2 * k + (mi & 1);
            uint32_t b[4];
            ldmatrix_x4(b, chunk_addr(k_tile, row, ch));
            if (k & 1) {
                mma_bf16_16816(s2[0], qa[k], b[0], b[1]);
                mma_bf16_16816(s2[1], qa[k], b[2], b[3]);
            } else {
                mma_bf16_16816(s[0], qa[k], b[0], b[1]);
                mma_bf16_16816(s[1], qa[k], b[2], b[3]);
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) { s[0][c] += s2[0][c]; s[1][c] += s2[1][c]; }
        // ---- mask, scale, online softmax (rows g: c = 0, 1; rows g + 8: c = 2, 3).  Scores are kept
        // in units of log2(e) so that ex2 serves; when no lane has a valid row among the upper
        // eight (a decode token of a model with at most 8 query heads per key/value head) that
        // half is skipped, and the accumulator is rescaled only when some row's maximum moved.
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int r = c >> 1;
                if (r == 1 && !upper) { s[i][c] = 0.f; continue; }
                const int key = key0 + 8 * i + 2 * t + (c & 1);
                const bool ok = row_ok[r] && key <= row_pos[r] && key >= row_lo[r];
                s[i][c] = ok ? s[i][c] * sl2 : -INFINITY;
                tile_max[r] = fmaxf(tile_max[r], s[i][c]);
            }
        float alpha[2] = {1.f, 1.f};
        bool moved = false;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (r == 1 && !upper) continue;
            tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
            tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
            const float m_new = fmaxf(m_run[r], tile_max[r]);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            if (m_new != m_run[r]) {
                alpha[r] = ex2(m_run[r] - m_use);
                moved = true;
            }
            m_run[r] = m_new;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[i][2 * r] = ex2(s[i][2 * r] - m_use);
                s[i][2 * r + 1] = ex2(s[i][2 * r + 1] - m_use);
                sum += s[i][2 * r] + s[i][2 * r + 1];
            }
            l_run[r] = l_run[r] * alpha[r] + sum;  // this lane's share; the quad is summed at the end
        }
        if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
            for (int i = 0; i < NT_O; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
        }
        // ---- O += P V: matrices read transposed, (keys 0..7 | 8..15) x (dims 16d + 0..7 | 8..15)
        const uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                                pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
        for (int d = 0; d < HD / 16; ++d) {
            const int row = (mi & 1) * 8 + lr;
            const int ch = 2 * d + (mi >> 1);
            uint32_t b[4];
            ldmatrix_x4_trans(b, chunk_addr(v_tile, row, ch));
            mma_bf16_16816(o[2 * d], pa, b[0], b[1]);
            mma_bf16_16816(o[2 * d + 1], pa, b[2], b[3]);
        }
        __syncwarp();       // the stage is refilled by the copies issued in the next iteration
    }
    cp_async_wait<0>();
    if (timed_out && p.err_flag) atomicExch(p.err_flag, ERR_ATTN_TIMEOUT);   // the result of this group is wrong; the host reads the flag
    __syncwarp();

    // ---- merge the warps of the CTA: (max, sum) per warp and row, the accumulators of the valid
    // row halves, then one pass over the valid (row, dim) elements
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
            if (c >= 2 && !upper) continue;   // rows 8..15 are all invalid
            sm_o(warp, g + 8 * (c >> 1), 8 * i + 2 * t + (c & 1)) = o[i][c];
        }
    // which of the 16 rows are real (token, head) pairs, and where their output rows start
    if (threadIdx.x < 16) {
        const int row = threadIdx.x, ti = row / p.hpg, hi = row % p.hpg;
        const bool v = ti < n_tok && ti < p.tpg && hb * p.hpg + hi < n_rep;
        sm_th[row] = v ? (tok0 + ti) * p.nh + (kvh * n_rep + hb * p.hpg + hi) : -1;
    }
    __syncthreads();

    int n_cl = 1, rank = 0, cp = HD;   // cluster size, this CTA's rank, output dims owned per rank
    if constexpr (CLUSTER) {
        if (p.n_splits > 1) {
            n_cl = p.n_splits;
            rank = (int)cg::this_cluster().block_rank();
            cp = (HD + n_cl - 1) / n_cl;
        }
    }
    // four consecutive output dims of a row per thread
    for (int e = threadIdx.x; e < 16 * (HD / 4); e += WARPS * 32) {
        const int row = e / (HD / 4), d4 = e % (HD / 4), d = 4 * d4;
        const int th_row = sm_th[row];
        if (th_row < 0) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w][row]);
        const float m_use = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, O[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = ex2(sm_m[w][row] - m_use);
            L += sm_l[w][row] * f;
#pragma unroll
            for (int k = 0; k < 4; ++k) O[k] += sm_o(w, row, d + k) * f;
        }
        const size_t th = (size_t)th_row;
        if (p.n_splits == 1) {
            const float inv = 1.0f / L;
            *reinterpret_cast<uint2*>(p.out + th * HD + d) = make_uint2(pack_bf16(O[0] * inv, O[1] * inv), pack_bf16(O[2] * inv, O[3] * inv));
        } else if constexpr (CLUSTER) {
            // push this CTA's partial to the CTA that owns the output dims: slot [this rank][row][d - owner * cp]
            // of its receive buffer; the row's (max, sum) go to every CTA
            cg::cluster_group cluster = cg::this_cluster();
            if ((cp & 3) == 0) {
                const int owner = d / cp;
                *reinterpret_cast<float4*>(cluster.map_shared_rank(&rx_o[(rank * 16 + row) * cp + (d - owner * cp)], owner)) =
                    make_float4(O[0], O[1], O[2], O[3]);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int owner = (d + k) / cp;
                    *cluster.map_shared_rank(&rx_o[(rank * 16 + row) * cp + (d + k - owner * cp)], owner) = O[k];
                }
            }
            for (int c = d4; c < n_cl; c += HD / 4)
                *reinterpret_cast<float2*>(cluster.map_shared_rank(&rx_ml[(rank * 16 + row) * 2], c)) = make_float2(M, L);
        } else {
            *reinterpret_cast<float4*>(p.part_acc + (th * p.n_splits + split) * HD + d) = make_float4(O[0], O[1], O[2], O[3]);
            if (d == 0) {
                p.part_ml[(th * p.n_splits + split) * 2] = M;
                p.part_ml[(th * p.n_splits + split) * 2 + 1] = L;
            }
        }
    }
    if constexpr (CLUSTER) {
        if (p.n_splits > 1) {
            // phase 2: all partials have arrived (release / acquire); nobody touches remote memory afterwards,
            // so a CTA may leave as soon as it has written its share of the output
            cg::cluster_group cluster = cg::this_cluster();
            (void)cluster.barrier_arrive();
            cluster.barrier_wait();
            const int d0 = rank * cp, n_own = min(cp, HD - d0);   // may be <= 0 for the last ranks
            for (int e = threadIdx.x; e < 16 * n_own; e += WARPS * 32) {
                const int row = e / n_own, dl = e - row * n_own;
                const int th_row = sm_th[row];
                if (th_row < 0) continue;
                float M = -INFINITY;
                for (int c = 0; c < n_cl; ++c) M = fmaxf(M, rx_ml[(c * 16 + row) * 2]);
                const float m_use = (M == -INFINITY) ? 0.f : M;
                float L = 0.f, O = 0.f;
                for (int c = 0; c < n_cl; ++c) {
                    const float2 ml = *reinterpret_cast<const float2*>(&rx_ml[(c * 16 + row) * 2]);
                    const float f = ex2(ml.x - m_use);
                    L += ml.y * f;
                    O += rx_o[(c * 16 + row) * cp + dl] * f;
                }
                p.out[(size_t)th_row * HD + d0 + dl] = __float2bfloat16_rn(O / L);
            }
        }
    }
}

// out[t, h, :] = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)   (maxima are kept in base 2)
// One block of COMBINE_WARPS warps per (token, head).  Warp w takes splits w, w + COMBINE_WARPS, ...; a lane holds
// four output dims, so a split's partial row is one 16-byte load per lane, and the loads of a warp's splits are
// independent (four splits in flight).  Each warp keeps a running (max, sum, accumulator) of its own; the warps
// merge through shared memory in warp order.
constexpr int COMBINE_WARPS = 8;
__global__ void __launch_bounds__(COMBINE_WARPS * 32)
combine_splits_kernel(const float* part_acc, const float* part_ml,
                      __nv_bfloat16* out, int n_splits, int hd, int nh,
                      const int* cu_seqlens, int n_seqs, int max_len) {
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
    __shared__ float sm_m[COMBINE_WARPS], sm_l[COMBINE_WARPS];
    __shared__ __align__(16) float sm_o[COMBINE_WARPS][128];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* ml = part_ml + th * n_splits * 2;
    const float* acc = part_acc + th * n_splits * hd;
    const bool has_dims = 4 * lane < hd;       // hd is a multiple of 16, at most 128
    float M = -INFINITY, L = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = warp; s0 < n_splits; s0 += 4 * COMBINE_WARPS) {
        float m_s[4], l_s[4];
        float4 a[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int sp = s0 + k * COMBINE_WARPS;
            const bool live = sp < n_splits;
            m_s[k] = live ? ml[2 * sp] : -INFINITY;
            l_s[k] = live ? ml[2 * sp + 1] : 0.f;
            a[k] = (live && has_dims) ? *reinterpret_cast<const float4*>(acc + (size_t)sp * hd + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float M_new = fmaxf(M, m_s[k]);
            const float m_use = (M_new == -INFINITY) ? 0.f : M_new;
            const float f_old = exp2f(M - m_use), f = exp2f(m_s[k] - m_use);      // 0 for an empty side
            L = L * f_old + l_s[k] * f;
            O.x = O.x * f_old + a[k].x * f; O.y = O.y * f_old + a[k].y * f;
            O.z = O.z * f_old + a[k].z * f; O.w = O.w * f_old + a[k].w * f;
            M = M_new;
        }
    }
    if (lane == 0) { sm_m[warp] = M; sm_l[warp] = L; }
    if (has_dims) *reinterpret_cast<float4*>(&sm_o[warp][4 * lane]) = O;
    __syncthreads();
    if (warp == 0 && has_dims) {
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < COMBINE_WARPS; ++w) Mx = fmaxf(Mx, sm_m[w]);
        const float m_use = (Mx == -INFINITY) ? 0.f : Mx;
        float Ls = 0.f;
        float4 Os = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < COMBINE_WARPS; ++w) {
            const float f = exp2f(sm_m[w] - m_use);
            const float4 o = *reinterpret_cast<const float4*>(&sm_o[w][4 * lane]);
            Ls += sm_l[w] * f;
            Os.x += o.x * f; Os.y += o.y * f; Os.z += o.z * f; Os.w += o.w * f;
        }
        const float inv = 1.0f / Ls;
        *reinterpret_cast<uint2*>(out + th * hd + 4 * lane) = make_uint2(pack_bf16(Os.x * inv, Os.y * inv), pack_bf16(Os.z * inv, Os.w * inv));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// The cache layer seen as a matrix [rows = pages * 2 * nkv * page_size, hd]; boxes of box_rows x 64.
bool make_cache_map(CUtensorMap* map, const void* cache, long long rows, int hd, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The cache layer as a 5-d tensor for whole-tile copies (pages of 16 tokens or more):
// [page][K, V][column box of 64][row = kv head * page_size + slot][64 columns]; a box is one tile:
// 1 page x 2 x (hd / 64) x 16 rows x 64 columns, which lands as [K col 0][K col 1]..[V col 0].. .
bool make_cache_map_5d(CUtensorMap* map, const void* cache, long long n_pages, int nkv, int page_size, int hd) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t row_bytes = (cuuint64_t)hd * 2, kv_bytes = (cuuint64_t)nkv * page_size * row_bytes;
    cuuint64_t dims[5] = {64, (cuuint64_t)nkv * page_size, (cuuint64_t)(hd / 64), 2, (cuuint64_t)n_pages};
    cuuint64_t strides[4] = {row_bytes, 128, kv_bytes, 2 * kv_bytes};
    cuuint32_t box[5] = {64, (cuuint32_t)TILE, (cuuint32_t)(hd / 64), 2, 1};
    cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
int launch(const CUtensorMap& map, const AttnParams& p, int n_groups_bound, bool use_cluster, cudaStream_t stream) {
    dim3 grid(n_groups_bound, p.nkv * p.head_blocks, p.n_splits);
    constexpr int SMEM = WARPS * STAGES * 2 * TILE * HD * 2 + 1024;   // per warp: the stages of a K and a V tile; alignment slack
    static bool configured_on[PYRE_MAX_DEVICES] = {};      // the attributes are per device
    bool& configured = configured_on[pyre_current_device()];
    if (!configured) {   // more than 48 KB of dynamic shared memory and clusters of more than 8 CTAs are opt-ins
        cudaError_t e = cudaFuncSetAttribute(paged_attention_mma_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(paged_attention_mma_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(paged_attention_mma_kernel<HD, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (!use_cluster) {
        cudaError_t e = pyre_launch(paged_attention_mma_kernel<HD, false>, dim3(grid), dim3(WARPS * 32), (size_t)SMEM, stream, map, p);
        if (e != cudaSuccess) return (int)e;
        return (int)cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = SMEM;
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, paged_attention_mma_kernel<HD, true>, map, p);
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
                                      long long n_pages, int uniform_len, int* err_flag, cudaStream_t stream) {
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
    p.page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) { p.page_shift = 0; while ((1 << p.page_shift) < page_size) ++p.page_shift; }
    // TMA tiles: power-of-two pages, head size a multiple of 64 (the 128-byte swizzle span), aligned base
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    p.err_flag = err_flag;
    p.n_pages = n_pages;
    p.uniform_len = (uniform_len > 0 && (long long)uniform_len * n_seqs == n_tokens) ? uniform_len : 0;
    p.box_rows = page_size < TILE ? page_size : TILE;
    p.use_tma = 0;
    if (p.page_shift >= 0 && hd % 64 == 0 && n_pages > 0 && ((uintptr_t)cache & 127) == 0 &&
        n_pages * 2 * nkv * page_size < (1ll << 31))
    {
        // whole-tile copies when a tile lies in one page; if the driver refuses the 5-d map, the 2-d one serves
        if (page_size >= TILE && make_cache_map_5d(&map, cache, n_pages, nkv, page_size, hd)) p.use_tma = 2;
        else p.use_tma = make_cache_map(&map, cache, n_pages * 2 * nkv * page_size, hd, p.box_rows) ? 1 : 0;
    }
    const int n_rep = nh / nkv;
    p.hpg = n_rep < 16 ? n_rep : 16;
    p.tpg = 16 / p.hpg;
    p.head_blocks = (n_rep + p.hpg - 1) / p.hpg;
    const int groups_bound = n_tokens / p.tpg + n_seqs;  // sum over entries of ceil(len / tpg) is at most this
    int rc;
    switch (hd) {
        case 16: rc = launch<16>(map, p, groups_bound, use_cluster, stream); break;
        case 32: rc = launch<32>(map, p, groups_bound, use_cluster, stream); break;
        case 48: rc = launch<48>(map, p, groups_bound, use_cluster, stream); break;
        case 64: rc = launch<64>(map, p, groups_bound, use_cluster, stream); break;
        case 80: rc = launch<80>(map, p, groups_bound, use_cluster, stream); break;
        case 96: rc = launch<96>(map, p, groups_bound, use_cluster, stream); break;
        case 112: rc = launch<112>(map, p, groups_bound, use_cluster, stream); break;
        case 128: rc = launch<128>(map, p, groups_bound, use_cluster, stream); break;
        default: return PYRE_ERR_UNSUPPORTED;
    }
    if (rc) return rc;
    if (n_splits > 1 && !use_cluster) {
        pyre_launch(combine_splits_kernel, dim3(n_tokens * nh), dim3(COMBINE_WARPS * 32), 0, stream, p.part_acc, p.part_ml, p.out, n_splits, hd, nh, cu_seqlens, n_seqs, max_len);
        PYRE_LAUNCH_CHECK();
    }
    return 0;
}
