// Paged attention for prompt portions on the 5th-generation tensor cores (bfloat16, head
// sizes 64 and 128): both products, S = Q K^T and O = P V, are tcgen05.mma instructions with
// their accumulators in tensor memory; queries, keys and values arrive by TMA.
//
// A CTA (224 threads) owns 128 consecutive tokens of one portion and one query head and walks
// the keys in tiles of 64, from the tile holding the start of the first row's window to the
// tile holding the last row's position:
//   warps 0 and 6      : TMA producers (lane 0 issues).  Warp 0 copies the Q tile once (128 rows
//                        of this head out of the [T, nh * hd] activation matrix) and then the K
//                        tiles, warp 6 the V tiles: per key tile the rows of 64 / box_rows pages
//                        through a tensor map over the cache layer viewed as [rows, hd]
//                        (128-byte swizzle).  K and V have two-stage rings of their own: a K stage
//                        is free as soon as its scores exist, a V stage after its P V.  Issuing a
//                        copy costs about a hundred cycles, so the two rings have a warp each.
//   warp 1, one thread : issues the MMAs.  S (128 x 64, fp32, one of two TMEM buffers) = Q K^T with
//                        both operands K-major; then, once the softmax threads have put P
//                        (bf16, 128 x 64) into shared memory, O (128 x hd, TMEM columns
//                        128..) += P V with V as an MN-major operand straight from the page rows.
//   warps 2..5         : one thread per query row.  Reads its row of S with tcgen05.ld, masks
//                        by position (causal limit, window), keeps the running maximum and sum
//                        in fp32, writes P.  No shuffles: a row lives in one thread.
// The accumulator O is rescaled only when a row's maximum grows by more than 2^8 beyond the
// value it was scaled with (probabilities then stay below 256, exact in the final O / l);
// the rescale is a tcgen05.ld / multiply / tcgen05.st pass over the row.
// S is double-buffered in tensor memory: the scores of tile i + 1 are computed while the row
// threads work on tile i.  Two CTAs fit on an SM (112 KB of shared memory, 256 TMEM columns
// each), so the tensor core also alternates between two CTAs.  The grid runs the heads fastest
// and the tiles of a portion from its end, so the tiles with the most keys start first.
// The softmax arithmetic uses the packed fp32 pairs of sm_100 (fma.rn.f32x2, add.rn.f32x2), the
// three-input max and ex2.approx: about four instructions per score.
//
// Few query tiles after a long context (a short portion of a long prompt) would leave most SMs idle: then
// grid.z CTAs share the key tiles of every (query tile, head), each leaves its unnormalised O with the rows'
// maxima and sums in scratch memory, and combine_shares_kernel puts them together (the host decides how many:
// only while there are fewer items than SMs, see ops.prefill_key_splits).
//
// Whole page rows arrive, so rows of a V tile outside [first row's window start, last row's
// position] may hold anything; the row threads zero them in shared memory before the P V
// product (their probabilities are exactly 0, but 0 x NaN is not).
//
// Every mbarrier wait is bounded; on a time-out the kernel raises the error flag, stops
// waiting everywhere, skips its stores, frees its tensor memory and returns.
//
// Formula: pyre/model.py:104-124 (scores = (q k^T) * scale, causal mask from the query's
// absolute position, fp32 softmax, probabilities rounded to the activation dtype, times v).
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace {

constexpr int BM = 128;       // queries per CTA = TMEM lanes
constexpr int BN = 64;        // keys per tile
constexpr int THREADS = 224;   // warp 0: K producer, 1: MMA issuer, 2-5: one thread per query row, 6: V producer
constexpr int ERR_TIMEOUT = 4;
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = pyre_now_ns();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 0) {
            if (*abort_flag) return false;
            if (pyre_now_ns() - t0 > PYRE_WAIT_NS) break;
        }
    }
    *abort_flag = 1;
    if (err_flag) atomicExch(err_flag, ERR_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major operand, 128-byte rows, 128B swizzle: LBO unused (1), SBO = 1024 B (eight rows).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand: each K row (a key) holds 64 MN elements (128 B, swizzled); eight rows form
// an atom (SBO = 1024 B); the next 64 MN elements start `lbo` bytes further.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 bytes per thread in one request (sm_100: 256-bit global stores; the address is 32-byte aligned): whole sectors
__device__ __forceinline__ void st_global_32B(void* ptr, const uint32_t* w) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :: "l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// Two fp32 lanes in one 64-bit register for the packed fma/add of sm_100 (each lane is the same
// IEEE operation as its scalar form).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 2^x on the special-function unit; results below 2^-126 are flushed to zero (a weight that
// small adds nothing to a sum whose largest term is at least 2^-8).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct TcParams {
    __nv_bfloat16* out;          // [T, nh * HD]
    const int* block_table;      // [B, bt_stride]
    const int* cu_seqlens;       // [B + 1]
    const int* positions;        // [T]
    int bt_stride, n_seqs, nh, nkv, page_size, page_shift, box_rows, window, min_len;
    float scale;
    int* err_flag;
    long long n_pages;           // pages of the pool; read by the debug checks only
    // key_splits > 1: grid.z CTAs share the key tiles of one (query tile, head); each leaves its unnormalised O
    // (fp32 [T, nh, key_splits, HD]) and the row's (maximum in log2 units, sum) ([T, nh, key_splits, 2]) for the
    // combining kernel
    int key_splits;
    float* part_o;
    float* part_ml;
};

template <int HD>
struct Smem {
    static constexpr int HALVES = HD / 64;                 // 128-byte column boxes per row
    static constexpr int Q_BYTES = HALVES * BM * 128;
    static constexpr int KV_TILE = HALVES * BN * 128;      // one K (or V) tile
    static constexpr int P_BYTES = BM * 128;               // 128 rows x 64 bf16
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = Q_BYTES;                  // [2 stages]
    static constexpr int OFF_V = OFF_K + 2 * KV_TILE;      // [2 stages]
    static constexpr int OFF_P = OFF_V + 2 * KV_TILE;
    static constexpr int OFF_BAR = OFF_P + P_BYTES;        // q_full, k_full[2], v_full[2], s_full[2], o_ready[2], p_full
    static constexpr int N_BARS = 10;
    static constexpr int TOTAL = OFF_BAR + N_BARS * 8 + 16;   // the dynamic window must start 1024-byte aligned (checked)
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const TcParams p) {
    using L = Smem<HD>;
    constexpr int HALVES = L::HALVES;
    constexpr uint32_t TMEM_COLS = 256;                     // two S buffers of 64 columns, O: HD columns
    constexpr uint32_t S_COL = 0, O_COL = 128;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    uint8_t* gen = smem_raw;
    if (base & 1023u) {   // swizzled boxes need 1024-byte alignment; two CTAs per SM leave no room for slack
        if (threadIdx.x == 0 && p.err_flag) atomicExch(p.err_flag, ERR_TIMEOUT + 1);
        return;
    }
    // s_full[t & 1] also tells the producer that the K stage of tile t is free, o_ready[t & 1] that its V stage is
    const uint32_t bar_q = base + L::OFF_BAR, bar_k_full = bar_q + 8, bar_v_full = bar_q + 24;
    const uint32_t bar_s = bar_q + 40 /* [2] */, bar_o = bar_q + 56 /* [2] */, bar_p = bar_q + 72;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::OFF_BAR + L::N_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::OFF_BAR + L::N_BARS * 8 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();

    // ---- which 128-token tile of which entry?  tiles are numbered from the end of each portion
    // (the last tile sees the most keys and starts first)
    int tile = blockIdx.y, seq = -1, tok0 = 0, n_tok = 0;
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
    if (seq < 0) return;   // the grid is an upper bound (whole CTA leaves: nothing was set up yet)
    const int head = blockIdx.x;   // heads are the fast grid dimension: the longest tiles of all heads start first
    const int kvh = head / (p.nh / p.nkv);
    const int* table = p.block_table + (size_t)seq * p.bt_stride;
    const int pos_first = p.positions[tok0], pos_last = pos_first + n_tok - 1;   // consecutive positions
    const int lo_cta = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    int tile_lo = lo_cta / BN, tile_hi = pos_last / BN;
    if (p.key_splits > 1) {
        // this CTA's share of the key tiles; a share may be empty (few tiles): it says so and leaves
        const int per = (tile_hi - tile_lo + p.key_splits) / p.key_splits;
        tile_lo += (int)blockIdx.z * per;
        tile_hi = min(tile_hi, tile_lo + per - 1);
        if (tile_lo > tile_hi) {
            pdl_wait();      // the scratch may still be read by the combining kernel of the layer before
            if ((int)threadIdx.x < n_tok) {
                float* ml = p.part_ml + (((size_t)(tok0 + threadIdx.x) * p.nh + blockIdx.x) * p.key_splits + blockIdx.z) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.f;
            }
            return;
        }
    }
    const int n_tiles = tile_hi - tile_lo + 1;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_q, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_k_full + 8 * s, 1); mbar_init(bar_v_full + 8 * s, 1);
            mbar_init(bar_s + 8 * s, 1); mbar_init(bar_o + 8 * s, 1);
        }
        mbar_init(bar_p, 4);      // one arrival per row warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || warp == 6) {
        // ---------------- producers: warp 0 copies Q and the K tiles, warp 6 the V tiles.  The whole
        // warp runs the loop (no divergent region) and lane 0 issues the copies.
        const int which = warp == 0 ? 0 : 1;
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
        }
        pdl_wait();   // queries and pages of this step come from earlier kernels
        if (which == 0 && lane == 0) {
            mbar_expect_tx(bar_q, L::Q_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) tma_load_2d(base + L::OFF_Q + h * (BM * 128), &map_q, bar_q, head * HD + h * 64, tok0);
        }
        // K and V have rings of their own (two stages each).  A K stage is free again as soon
        // as its scores are computed (s_full), a V stage after its P V (o_ready).
        // A tile is copied in pieces of one page (or of the whole tile, for pages of 64 tokens and
        // more); lane pc holds the page number of piece pc, read two tiles ahead of its use.
        const int pieces = BN / p.box_rows;   // at most 16 (pages of 4 tokens or more)
        auto read_pages = [&](int i) -> int {
            const int key = (tile_lo + i) * BN + lane * p.box_rows;
            const bool live = lane < pieces && i < n_tiles && key + p.box_rows - 1 >= lo_cta && key <= pos_last;
            return live ? pyre_checked_page(table[key >> p.page_shift], p.n_pages, p.err_flag) : 0;   // pieces outside the range read page 0 (masked)
        };
        const uint32_t bar_empty = which ? bar_o : bar_s, bar_full = which ? bar_v_full : bar_k_full;
        const uint32_t ring = base + (which ? L::OFF_V : L::OFF_K);
        const int row_base = (which * p.nkv + kvh) * p.page_size, page_rows = 2 * p.nkv * p.page_size;
        int pg0 = read_pages(0), pg1 = read_pages(1), pg2 = read_pages(2);   // tiles i, i + 1, i + 2
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i & 1;
            const bool ok = mbar_wait(bar_empty + 8 * s, ((i >> 1) & 1) ^ 1, abort_flag, p.err_flag);
            if (!__all_sync(0xffffffffu, ok)) break;
            const uint32_t full = bar_full + 8 * s, dst = ring + s * L::KV_TILE;
            if (lane == 0) mbar_expect_tx(full, L::KV_TILE);
            __syncwarp();
            // one box (a page's rows x one 128-byte column box) per lane: the copies of a tile go out as one
            // instruction of up to 32 lanes instead of a loop in one thread (about a hundred cycles per copy there,
            // which set the pace of the ring with pages of 16 tokens: eight boxes per tile)
            for (int b0 = 0; b0 < pieces * HALVES; b0 += 32) {
                const int box = b0 + lane, pc = box / HALVES, h = box - pc * HALVES;
                const int page = __shfl_sync(0xffffffffu, pg0, pc & 31);
                if (box < pieces * HALVES) {
                    const int key = (tile_lo + i) * BN + pc * p.box_rows;
                    const int row = page * page_rows + row_base + (key & (p.page_size - 1));
                    tma_load_2d(dst + h * (BN * 128) + pc * p.box_rows * 128, &map_kv, full, h * 64, row);
                }
            }
            __syncwarp();
            pg0 = pg1;
            pg1 = pg2;
            pg2 = read_pages(i + 3);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer
            // instruction descriptors: D fp32 (bit 4), A and B bf16 (bits 7, 10), N >> 3 at bit 17, M >> 4 at bit 24;
            // bit 16: B is MN-major (V: the head dims are contiguous, the keys are the K index)
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // S of tile i goes to S buffer i & 1; it is issued one tile ahead, so the tensor core
            // works on the next scores while the row threads are busy with this tile's softmax
            auto issue_s = [&](int i) -> bool {
                const int st = i & 1;
                if (!mbar_wait(bar_k_full + 8 * st, (i >> 1) & 1, abort_flag, p.err_flag)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t kd = base + L::OFF_K + st * L::KV_TILE;
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
#pragma unroll
                    for (int j = 0; j < 4; ++j)   // HD / 16 steps of 16 dims; 4 steps per 128-byte column box
                        umma_bf16(tmem_base + S_COL + st * BN, desc_k_major(base + L::OFF_Q + h * (BM * 128)) + 2 * j,
                                  desc_k_major(kd + h * (BN * 128)) + 2 * j, idesc_s, (h > 0 || j > 0) ? 1u : 0u);
                umma_commit(bar_s + 8 * st);
                return true;
            };
            bool ok = mbar_wait(bar_q, 0, abort_flag, p.err_flag);
            if (ok) ok = issue_s(0);
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int st = i & 1;
                if (i + 1 < n_tiles) {
                    ok = issue_s(i + 1);
                    if (!ok) break;
                }
                ok = mbar_wait(bar_p, i & 1, abort_flag, p.err_flag);   // P is in shared memory, O has been rescaled
                if (ok) ok = mbar_wait(bar_v_full + 8 * st, (i >> 1) & 1, abort_flag, p.err_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t vd = base + L::OFF_V + st * L::KV_TILE;
                // O += P V: 4 steps of 16 keys; V rows are 128 B per column box, the second box lies BN * 128 B further
#pragma unroll
                for (int j = 0; j < BN / 16; ++j)
                    umma_bf16(tmem_base + O_COL, desc_k_major(base + L::OFF_P) + 2 * j,
                              desc_mn_major(vd + j * (16 * 128), BN * 128), idesc_pv, (i > 0 || j > 0) ? 1u : 0u);
                umma_commit(bar_o + 8 * st);   // O holds this tile; P may be overwritten, the V stage refilled
            }
        }
    } else {
        // ---------------- row threads: TMEM lane = query row
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool row_ok = row < n_tok;
        const int pos = pos_first + row;
        const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const float sl2 = p.scale * 1.44269504088896341f;
        float m_ref = -INFINITY, l_sum = 0.f;
        bool alive = true;
        for (int i = 0; i < n_tiles && alive; ++i) {
            const int s = i & 1;
            const int key0 = (tile_lo + i) * BN;
            bool ok = mbar_wait(bar_s + 8 * s, (i >> 1) & 1, abort_flag, p.err_flag);
            alive = __all_sync(0xffffffffu, ok);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc[BN];
            {
                uint32_t r0[16], r1[16], r2[16], r3[16];   // all four loads go out before the one wait
                tmem_ld16(lane_addr + S_COL + s * BN, r0);
                tmem_ld16(lane_addr + S_COL + s * BN + 16, r1);
                tmem_ld16(lane_addr + S_COL + s * BN + 32, r2);
                tmem_ld16(lane_addr + S_COL + s * BN + 48, r3);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    sc[q] = __uint_as_float(r0[q]); sc[16 + q] = __uint_as_float(r1[q]);
                    sc[32 + q] = __uint_as_float(r2[q]); sc[48 + q] = __uint_as_float(r3[q]);
                }
            }
            // mask by position (only tiles that some row's causal limit or window edge cuts; rows
            // beyond the portion's end are never stored, so they need no mask); the raw maximum in four chains
            const bool need_mask = key0 + BN - 1 > pos_first || (p.window > 0 && key0 < pos_last - p.window + 1);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int key = key0 + c;
                    const bool okk = row_ok && key <= pos && key >= lo;
                    sc[c] = okk ? sc[c] : -INFINITY;
                }
            }
            float tm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < BN; c += 8) {
                tm[0] = max3(tm[0], sc[c], sc[c + 1]);
                tm[1] = max3(tm[1], sc[c + 2], sc[c + 3]);
                tm[2] = max3(tm[2], sc[c + 4], sc[c + 5]);
                tm[3] = max3(tm[3], sc[c + 6], sc[c + 7]);
            }
            const float tmax = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3])) * sl2;
            // the accumulator keeps its scaling unless the maximum grew by more than 2^8
            const bool grow = tmax > m_ref + RESCALE_THRESHOLD;   // also the first finite maximum (m_ref = -inf)
            const float m_new = grow ? tmax : m_ref;
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = grow ? ex2(m_ref - m_use) : 1.f;   // 2^(-inf) = 0 the first time
            m_ref = m_new;
            // p = 2^(s * scale * log2 e - m): packed fma, one special-function op per element, packed sums
            const uint64_t sl2_2 = pack2(sl2, sl2), neg_m2 = pack2(-m_use, -m_use);
            uint64_t sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                float a, b;
                unpack2(fma2(pack2(sc[c], sc[c + 1]), sl2_2, neg_m2), a, b);
                sc[c] = ex2(a);
                sc[c + 1] = ex2(b);
                sum2[(c >> 1) & 1] = add2(sum2[(c >> 1) & 1], pack2(sc[c], sc[c + 1]));
            }
            float sum[4];
            unpack2(sum2[0], sum[0], sum[1]);
            unpack2(sum2[1], sum[2], sum[3]);
            l_sum = l_sum * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));

            // the previous tile's P V must be complete before P is overwritten or O is touched
            if (i > 0) {
                ok = mbar_wait(bar_o + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, p.err_flag);
                alive = __all_sync(0xffffffffu, ok);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 16) {
                        uint32_t r[16];
                        tmem_ld16(lane_addr + O_COL + c, r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int q = 0; q < 16; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * alpha);
                        tmem_st16(lane_addr + O_COL + c, r);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            // rows of the V tile outside [lo_cta, pos_last] hold whatever the page holds: zero them
            if (key0 + BN - 1 > pos_last || key0 < lo_cta) {
                ok = mbar_wait(bar_v_full + 8 * s, (i >> 1) & 1, abort_flag, p.err_flag);   // the tile has landed
                alive = __all_sync(0xffffffffu, ok);
                if (!alive) break;
                const uint32_t vd = base + L::OFF_V + s * L::KV_TILE;
                for (int idx = threadIdx.x - 64; idx < BN * HALVES * 8; idx += 128) {
                    const int k = idx / (HALVES * 8), rem = idx % (HALVES * 8);
                    const int key = key0 + k;
                    if (key > pos_last || key < lo_cta)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vd + (rem >> 3) * (BN * 128) + k * 128 + (rem & 7) * 16), "r"(0u) : "memory");
                }
            }
            // P (bf16) into shared memory, K-major with the 128-byte swizzle: chunk c of row r at c ^ (r & 7)
            {
                const uint32_t prow = base + L::OFF_P + row * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t w0 = pack_bf16(sc[8 * c], sc[8 * c + 1]), w1 = pack_bf16(sc[8 * c + 2], sc[8 * c + 3]);
                    const uint32_t w2 = pack_bf16(sc[8 * c + 4], sc[8 * c + 5]), w3 = pack_bf16(sc[8 * c + 6], sc[8 * c + 7]);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(prow + ((c ^ (row & 7)) * 16)), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes before the tensor core reads them
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p);
        }
        // ---- the last P V, then out = O / l
        if (alive) {
            bool ok = mbar_wait(bar_o + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag, p.err_flag);
            alive = __all_sync(0xffffffffu, ok);
        }
        if (alive) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = (row_ok && l_sum > 0.f) ? 1.0f / l_sum : 0.f;
            __nv_bfloat16* orow = p.out + ((size_t)(tok0 + (row_ok ? row : 0)) * p.nh + head) * HD;
            const size_t piece_at = ((size_t)(tok0 + (row_ok ? row : 0)) * p.nh + head) * p.key_splits + blockIdx.z;
            if (p.key_splits > 1 && row_ok) {
                p.part_ml[piece_at * 2] = m_ref;
                p.part_ml[piece_at * 2 + 1] = l_sum;
            }
#pragma unroll 1
            for (int c = 0; c < HD; c += 16) {
                uint32_t r[16];
                __syncwarp();
                tmem_ld16(lane_addr + O_COL + c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.key_splits > 1) {
                    if (row_ok) {
                        st_global_32B(p.part_o + piece_at * HD + c, r);
                        st_global_32B(p.part_o + piece_at * HD + c + 8, r + 8);
                    }
                } else if (row_ok) {
                    uint32_t w[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) w[q] = pack_bf16(__uint_as_float(r[2 * q]) * inv, __uint_as_float(r[2 * q + 1]) * inv);
                    st_global_32B(orow + c, w);
                }
            }
        }
    }

    // ---------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// The shares of a (query tile, head) put together: out = sum_i O_i 2^(m_i - M) / sum_i l_i 2^(m_i - M) over the
// shares that saw a key (l_i > 0).  One CTA per query tile and head as in the main kernel, a warp per row, a lane per
// four head dimensions.
template <int HD>
__global__ void __launch_bounds__(128)
combine_shares_kernel(const TcParams p) {
    pdl_trigger();
    pdl_wait();
    int tile = blockIdx.y, seq = -1, tok0 = 0, n_tok = 0;
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
    const int head = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, S = p.key_splits;
    for (int row = warp; row < n_tok; row += 4) {
        const size_t at = ((size_t)(tok0 + row) * p.nh + head) * S;
        float m = -INFINITY, l = 0.f;
        if (lane < S) {
            m = p.part_ml[(at + lane) * 2];
            l = p.part_ml[(at + lane) * 2 + 1];
            if (!(l > 0.f)) { m = -INFINITY; l = 0.f; }
        }
        float top = m;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
        const float w = l > 0.f ? ex2(m - top) : 0.f;
        float denom = l * w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < S; ++i) {
            const float wi = __shfl_sync(0xffffffffu, w, i);
            if (wi > 0.f && lane < HD / 4) {
                const float4 o = *reinterpret_cast<const float4*>(p.part_o + (at + i) * HD + 4 * lane);
                acc.x = fmaf(wi, o.x, acc.x); acc.y = fmaf(wi, o.y, acc.y); acc.z = fmaf(wi, o.z, acc.z); acc.w = fmaf(wi, o.w, acc.w);
            }
        }
        if (lane < HD / 4) {
            const float inv = denom > 0.f ? 1.0f / denom : 0.f;
            uint2 packed;
            packed.x = pack_bf16(acc.x * inv, acc.y * inv);
            packed.y = pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(p.out + ((size_t)(tok0 + row) * p.nh + head) * HD + 4 * lane) = packed;
        }
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

// A bf16 matrix [rows, cols] with row pitch `pitch` elements; boxes of box_rows x 64 columns, 128B swizzle.
bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long pitch, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const TcParams& p, int tiles_bound, cudaStream_t stream) {
    using L = Smem<HD>;
    static bool configured_on[PYRE_MAX_DEVICES] = {};      // the attributes are per device
    bool& configured = configured_on[pyre_current_device()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = pyre_launch(attention_tc_kernel<HD>, dim3(p.nh, tiles_bound, p.key_splits), dim3(THREADS), (size_t)L::TOTAL, stream, mq, mkv, p);
    if (e != cudaSuccess) return (int)e;
    if (p.key_splits > 1) {
        e = pyre_launch(combine_shares_kernel<HD>, dim3(p.nh, tiles_bound), dim3(128), 0, stream, p);
        if (e != cudaSuccess) return (int)e;
    }
    return (int)cudaGetLastError();
}

}  // namespace

// Attention of every entry with at least min_len tokens (other entries' rows are left untouched).
// bfloat16, head sizes 64 and 128, pages of a power-of-two number of tokens (4 or more).  n_long_tokens: total
// tokens of those entries (bounds the grid); n_tokens: rows of q; n_pages: pages of the cache layer.
// key_splits > 1: that many CTAs share the key tiles of every (query tile, head) and a second kernel puts their
// results together; part_o: fp32 [n_tokens, nh, key_splits, hd], part_ml: fp32 [n_tokens, nh, key_splits, 2].
PYRE_API int pyre_attention_prefill_tc(const void* q, const void* cache, void* out, const int* block_table,
                                       int bt_stride, const int* cu_seqlens, const int* positions, int n_tokens,
                                       int n_long_tokens, int n_seqs, int nh, int nkv, int hd, int page_size,
                                       long long n_pages, int window, float scale, int min_len, int key_splits,
                                       float* part_o, float* part_ml, int* err_flag, cudaStream_t stream) {
    if (n_long_tokens <= 0) return 0;
    if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || page_size < 4 || (page_size & (page_size - 1)) || min_len < 1)
        return PYRE_ERR_UNSUPPORTED;
    const long long kv_rows = n_pages * 2 * nkv * page_size;
    if (((uintptr_t)q & 15) || ((uintptr_t)cache & 15) || ((uintptr_t)out & 31) || kv_rows >= (1ll << 31) || n_pages <= 0)
        return PYRE_ERR_UNSUPPORTED;
    TcParams p;
    p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.cu_seqlens = cu_seqlens; p.positions = positions;
    p.bt_stride = bt_stride; p.n_seqs = n_seqs; p.nh = nh; p.nkv = nkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.box_rows = page_size < BN ? page_size : BN;
    p.window = window; p.min_len = min_len; p.scale = scale; p.err_flag = err_flag; p.n_pages = n_pages;
    if (key_splits < 1 || key_splits > 32 || (key_splits > 1 && (!part_o || !part_ml || ((uintptr_t)part_o & 31)))) return PYRE_ERR_BAD_ARG;
    p.key_splits = key_splits; p.part_o = part_o; p.part_ml = part_ml;
    CUtensorMap mq, mkv;
    memset(&mq, 0, sizeof(mq));
    memset(&mkv, 0, sizeof(mkv));
    if (!make_map(&mq, q, n_tokens, (long long)nh * hd, (long long)nh * hd, BM)) return PYRE_ERR_UNSUPPORTED;
    if (!make_map(&mkv, cache, kv_rows, hd, hd, p.box_rows)) return PYRE_ERR_UNSUPPORTED;
    const int tiles_bound = n_long_tokens / BM + n_seqs;
    if (tiles_bound > 65535) return PYRE_ERR_BAD_ARG;   // grid.y
    return hd == 128 ? launch<128>(mq, mkv, p, tiles_bound, stream) : launch<64>(mq, mkv, p, tiles_bound, stream);
}
