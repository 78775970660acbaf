// bfloat16 matrix product on the 5th-generation tensor cores:  D[x, y] = sum_k X[x, k] * Y[y, k]
// with X [x_rows, K] and Y [y_rows, K] both row-major (K contiguous), fp32 accumulation in
// tensor memory, output in fp32 or bfloat16 with arbitrary strides.
//
// One kernel serves both orientations of a linear layer y = a W^T (pyre/model.py:84-87):
//   few tokens (decode)  : X = W (the out-features fill the 128 rows of the MMA), Y = a
//                          (8..128 tokens are the narrow N side), output stored transposed;
//                          K may be split over CTAs (blockIdx.z) into fp32 partial sums
//                          that the consumer kernel adds up, so that shapes with few
//                          128-row tiles still put a CTA on every SM;
//   many tokens (prefill): X = a (128 tokens per tile), Y = W (up to 256 features per tile); by default
//                          as pairs of CTAs on 256-token tiles (tcgen05 cta_group::2, see the kernel).
//
// Structure of a CTA (192 threads), one 128 x BN output tile, K in blocks of 64:
//   warp 0, one thread : TMA producer.  cp.async.bulk.tensor.2d loads an X box (128 x 64)
//                        and a Y box (BN x 64) per K block into a ring of shared-memory
//                        stages, 128-byte swizzled, completion counted on a "full" mbarrier.
//   warp 1, one thread : issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN,
//                        K = 16, four per K block) from shared-memory descriptors into a
//                        TMEM accumulator; tcgen05.commit frees each stage ("empty"
//                        mbarrier) and finally signals the accumulator.  Warp 1 also
//                        allocates and frees the TMEM columns.
//   warps 2..5         : epilogue.  tcgen05.ld (32 lanes x 32 bit, 16 columns at a time)
//                        reads the warp's quarter of the 128 accumulator rows and stores
//                        it, converted if asked.
// The CTA is persistent (one per SM, walking tiles c, c + gridDim.x, ...) and holds TWO
// accumulators in tensor memory: while the epilogue warps drain tile i, the MMA thread is
// already multiplying tile i + 1 into the other one, and the TMA ring never stops.
// Rows or K beyond the matrices are zero-filled by TMA, so any x_rows, y_rows and K work
// (K and the leading dimensions must be multiples of 8 elements: TMA strides are 16-byte
// multiples).  No load uses cluster multicast (a CTA of a pair fetches its own boxes).
//
// Every wait on an mbarrier is bounded.  If one runs out, the kernel raises the error
// flag, stops waiting everywhere, skips its stores, frees its tensor memory and returns;
// the host reads the flag.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;           // rows of X per tile = TMEM lanes
constexpr int BK = 64;            // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int THREADS = 192;
constexpr int ERR_TIMEOUT = 2;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

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
// Bounded wait.  Returns false if the limit ran out or another thread already gave up.
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
// The same for a CTA of a pair: the destination is this CTA's shared memory, the mbarrier may be the peer's
// (a shared::cluster address).  No multicast: each CTA fetches its own boxes.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// shared::cluster address of the same shared-memory offset in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128B swizzle:
// start address >> 4, leading byte offset 1 (unused with swizzle), stride byte offset
// 1024 >> 4 (eight rows), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
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
// A pair of CTAs on one tile (cta_group::2): M = 256, each CTA holds 128 rows of A, half the rows of B and, in its
// tensor memory, its 128 rows of D.  Issued by one thread of the pair's first CTA; the descriptors name the same
// shared-memory offsets in both.  The commit arrives on the barrier of that offset in both CTAs.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
// 32 bytes per thread in one request (sm_100: 256-bit global accesses; the address is 32-byte aligned).  A plain load,
// not the read-only path (see common.cuh on programmatic dependent launch).
__device__ __forceinline__ void ld_global_32B(const float* ptr, float* v) {
    asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(ptr) : "memory");
}
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

// The four epilogue warps agree on a predicate (barrier 1 with an AND reduction).  The gated epilogue of the
// transposed store synchronises those warps inside its loops; whether a tile is processed at all must
// therefore be one decision for the four of them, also when a bounded wait ran out for some and not for others.
__device__ __forceinline__ bool epilogue_warps_all(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "bar.red.and.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r) : "r"((uint32_t)pred) : "memory");
    return r != 0;
}

struct GemmParams {
    int x_rows, y_rows, K;
    int k_blocks_per_split;       // K blocks (of 64) per blockIdx.z
    int tiles_x, tiles_y;         // output tiles; CTA c works on tiles c, c + gridDim.x, ... (x fastest)
    long long stride_x, stride_y, split_stride;  // output element strides
    void* out;
    int out_f32;
    int x_is_constant;            // 1: X holds weights (may be loaded before the kernels before this one finish); 0: Y does
    int gated;                    // 1: the weight rows are gate/up rows interleaved in blocks of 64 (gate rows, then the up
                                  // rows of the same features); the epilogue writes silu(gate) * up, half as many features
    int* err_flag;
    // ---- work folded into the product so that no small kernel runs around it.  With the transposed store (few
    // tokens, the weights on the MMA's rows) as described below; with the row store (many tokens in one split, an
    // epilogue thread owns a token row) the same three without a fix-up: (a) the thread scales its own row, fix == 1
    // and fix == 2 happen in the epilogue itself (resid, bias, tables and outputs are then indexed [x_rows, y_rows]).
    // (a) rows scaled: out[token] *= 1 / sqrt(sum_i scale_ssq[i][token] / scale_n + scale_eps), the 1/rms of an
    //     RMSNorm whose weight the producer of the activations has already applied (see fix == 1)
    const float* scale_ssq;       // [scale_tiles][y_rows] partial sums of squares per token, or null
    int scale_tiles;
    float scale_n, scale_eps;
    // (b) fix-up: the CTA that finishes a tile last (an arrival counter per tile) turns the tile's fp32 partial
    //     sums, which every split has stored to `out`, into their final form:
    //     fix == 1  residual add + norm preparation:  v = resid + sum of partials;  resid = v;
    //               h_out = bf16(v * norm_w);  ssq_out[tile][token] = sum over the tile's features of v^2
    //     fix == 2  bias + rotary (half-split pairs over the whole head) + paged K/V write:  the tile's features are
    //               whole heads of the stacked q/k/v projection; q heads go to q_out, k and v heads to the cache
    int fix;
    int* tile_counters;           // [tiles] zero before the launch and after it
    float* resid;                 // fp32 [y_rows, x_rows]
    const float* norm_w;          // fp32 [x_rows]
    __nv_bfloat16* h_out;         // [y_rows, x_rows]
    float* ssq_out;               // [tiles_x][y_rows]
    const float* bias;            // fp32 [x_rows] or null
    const float* cos_t;           // fp32 [y_rows, rot / 2]
    const float* sin_t;
    __nv_bfloat16* q_out;         // [y_rows, nh * hd]
    __nv_bfloat16* kv_cache;      // one layer: [page][2][nkv][page_size][hd], or null (store nothing)
    const int* slot_mapping;      // [y_rows]
    int nh, nkv, hd, rot, page_size;
    long long n_pages;
};

template <int BN, int STAGES, bool XC, int CTAS = 1>
struct SmemLayout {
    static constexpr int X_BYTES = BM * BK * 2;
    static constexpr int Y_BYTES = (BN / CTAS) * BK * 2;      // a CTA of a pair holds half of the tile's Y rows
    static constexpr int STAGE_BYTES = X_BYTES + Y_BYTES;
    static constexpr int TILES = STAGES * STAGE_BYTES;
    static constexpr int N_BARS = 2 * STAGES + 4;     // full, empty per stage; accumulator full, empty per TMEM buffer
    static constexpr int EPI_OFF = TILES + N_BARS * 8 + 16;
    // transposed store: the gated epilogue's exchange of 64 up rows x BN tokens (fp32) between epilogue warps;
    // row store: per epilogue warp 32 rows x GW bf16 (pitch 2 GW + 16 bytes) for stores of whole lines, GW = 64
    // (128-byte lines) if the ring leaves room, else 32, else 0 (every thread stores its own 32 bytes)
    static constexpr int ROOM = 232448 - 1024 - EPI_OFF;
    static constexpr int GW = XC ? 0 : (ROOM >= 4 * 32 * 144 ? 64 : ROOM >= 4 * 32 * 80 ? 32 : 0);
    static constexpr int OUT_PITCH = 2 * GW + 16;
    static constexpr int EPI_BYTES = XC ? (BN <= 128 ? 64 * BN * 4 : 0) : 4 * 32 * OUT_PITCH * (GW > 0 ? 1 : 0);
    // transposed store: 1/rms of the tile's tokens (128 floats) and the "this CTA finished the tile last" flag
    static constexpr int SCALE_OFF = EPI_OFF + EPI_BYTES;
    static constexpr int SCALE_BYTES = XC ? 512 + 16 : 0;
    static constexpr int TOTAL = SCALE_OFF + SCALE_BYTES + 1024;  // bars, tmem slot and abort flag, epilogue buffers, alignment slack
};

// A CTA is persistent: it walks output tiles c, c + gridDim.x, ...  Two TMEM accumulators
// alternate, so the epilogue warps drain tile i while the MMA thread already works on tile
// i + 1; the shared-memory ring runs on across tiles.
//
// CTAS == 2 (row store only): two CTAs of a cluster, on the two SMs of a TPC, share a 256 x BN tile.  Each loads its
// own 128 rows of X and half of the tile's Y rows, so a K block costs an SM 128 (128 + BN / 2) bytes of loads
// instead of 128 (128 + BN) for the same MMA work; the first CTA's thread issues the MMAs for both, every CTA
// drains its own 128 accumulator rows.  Barriers: the first CTA's "full" barriers count the bytes of both CTAs'
// loads; the MMA commits arrive on the "empty" and "accumulator full" barriers of both; the epilogue warps of
// both arrive on the first CTA's "accumulator empty" barriers.
template <int BN, int STAGES, bool X_CONTIGUOUS_OUT, int CTAS = 1, int FOLD = 1>
__global__ void __launch_bounds__(THREADS, (X_CONTIGUOUS_OUT && FOLD != 0) ? 5 : (!X_CONTIGUOUS_OUT && FOLD == 0) ? 3 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, const GemmParams p) {
    static_assert(CTAS == 1 || (CTAS == 2 && !X_CONTIGUOUS_OUT && BN % 16 == 0), "pairs serve the row store");
    using L = SmemLayout<BN, STAGES, X_CONTIGUOUS_OUT, CTAS>;
    uint32_t rank = 0;                       // of this CTA in its pair
    if constexpr (CTAS == 2) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int worker = blockIdx.x / CTAS, n_workers = gridDim.x / CTAS;   // a worker (CTA or pair) walks tiles worker, worker + n_workers, ...
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles want 1024-byte alignment
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_full = base + L::TILES;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;     // [2]
    const uint32_t bar_acc_empty = bar_acc_full + 16;         // [2]
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::TILES + L::N_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::TILES + L::N_BARS * 8 + 8);

    // the folded work (row scales, fix-ups, the residual fold) is compiled into the FOLD != 0 variants only: the plain
    // weight stream keeps its small register count, so that the next kernel's CTAs find room beside it
    const int fix = FOLD != 0 ? p.fix : 0;
    const float* const scale_ssq = FOLD != 0 ? p.scale_ssq : nullptr;
    // the row store's residual fold, and its rotary epilogue (FOLD == 2), live in variants of their own: each keeps
    // its registers (compiled into one kernel, the 32-byte accesses of the one cost the other 8 % of its time)
    [[maybe_unused]] const bool fix1_rows = !X_CONTIGUOUS_OUT && FOLD == 1 && fix == 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (p.K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * p.k_blocks_per_split;
    const int kb_end = min(kb_begin + p.k_blocks_per_split, total_kb);
    const int n_kb = max(kb_end - kb_begin, 0);
    const int n_tiles = p.tiles_x * p.tiles_y;
    constexpr uint32_t ACC_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;   // columns of one accumulator (a power of two)
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;        // power of two >= 32, at most 512

    pdl_trigger();
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4 * CTAS);      // one arrival per epilogue warp (of both CTAs of a pair)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (CTAS == 2) {      // the same warp of both CTAs allocates the same columns in both
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (CTAS == 2) cluster_sync_all();     // the peer's barriers exist before anything arrives on them
    else __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_y)) : "memory");
            int it = 0;   // K blocks issued so far, over all tiles of this CTA
            bool waited = false;
            // loads of a pair's second CTA complete on the first CTA's barriers, which expect the bytes of both
            const uint32_t full_to = CTAS == 2 ? mapa_u32(bar_full, 0) : bar_full;
            auto load = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
                if constexpr (CTAS == 2) tma_load_2d_pair(dst, map, bar, c0, c1);
                else tma_load_2d(dst, map, bar, c0, c1);
            };
            for (int tile = worker; tile < n_tiles && !*abort_flag; tile += n_workers) {
                const int x0 = (tile % p.tiles_x) * (BM * CTAS) + rank * BM;
                const int y0 = (tile / p.tiles_x) * BN + rank * (BN / CTAS);
                int i = 0;
                if (!waited) {
                    // The weights do not depend on the kernels before this one: fill the ring with
                    // their tiles first, then wait for those kernels, then fetch the activations.
                    const int pre = n_kb < STAGES ? n_kb : STAGES;
                    for (int j = 0; j < pre; ++j) {
                        if (rank == 0) mbar_expect_tx(bar_full + 8 * j, CTAS * L::STAGE_BYTES);
                        const uint32_t xs = base + j * L::STAGE_BYTES, ys = xs + L::X_BYTES;
                        const int k = (kb_begin + j) * BK;
                        if (p.x_is_constant) load(xs, &map_x, full_to + 8 * j, k, x0);
                        else load(ys, &map_y, full_to + 8 * j, k, y0);
                    }
                    pdl_wait();
                    waited = true;
                    for (int j = 0; j < pre; ++j) {
                        const uint32_t xs = base + j * L::STAGE_BYTES, ys = xs + L::X_BYTES;
                        const int k = (kb_begin + j) * BK;
                        if (p.x_is_constant) load(ys, &map_y, full_to + 8 * j, k, y0);
                        else load(xs, &map_x, full_to + 8 * j, k, x0);
                    }
                    i = pre;
                    it = pre;
                }
                bool ok = true;
                for (; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    ok = mbar_wait(bar_empty + 8 * s, phase ^ 1, abort_flag, p.err_flag);
                    if (!ok) break;
                    if (rank == 0) mbar_expect_tx(bar_full + 8 * s, CTAS * L::STAGE_BYTES);
                    const uint32_t xs = base + s * L::STAGE_BYTES, ys = xs + L::X_BYTES;
                    const int k = (kb_begin + i) * BK;
                    load(xs, &map_x, full_to + 8 * s, k, x0);
                    load(ys, &map_y, full_to + 8 * s, k, y0);
                }
                if (!ok) break;
            }
            if (!waited) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---------------- MMA issuer (of a pair: the first CTA's, for both)
            // instruction descriptor: D fp32 (bit 4), A and B bf16 (bits 7, 10), both K-major,
            // N >> 3 at bit 17, M >> 4 at bit 24
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((BM * CTAS) >> 4) << 24);
            auto mma = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t accumulate) {
                if constexpr (CTAS == 2) umma_bf16_pair(d, a, b, idesc, accumulate);
                else umma_bf16(d, a, b, idesc, accumulate);
            };
            auto commit = [&](uint32_t bar) {
                if constexpr (CTAS == 2) umma_commit_pair(bar);
                else umma_commit(bar);
            };
            int it = 0, j = 0;
            bool ok = true;
            for (int tile = worker; tile < n_tiles && ok; tile += n_workers, ++j) {
                const int buf = j & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                ok = mbar_wait(bar_acc_empty + 8 * buf, ((j >> 1) & 1) ^ 1, abort_flag, p.err_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * ACC_COLS;
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    ok = mbar_wait(bar_full + 8 * s, phase, abort_flag, p.err_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t xs = base + s * L::STAGE_BYTES, ys = xs + L::X_BYTES;
                    const uint64_t da = umma_desc(xs), db = umma_desc(ys);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)   // 16 bf16 = 32 bytes = 2 descriptor units along K
                        mma(acc, da + 2 * k, db + 2 * k, (i > 0 || k > 0) ? 1u : 0u);
                    commit(bar_empty + 8 * s);     // the stage is free once these MMAs have read it
                }
                commit(bar_acc_full + 8 * buf);    // this tile's accumulator is complete (also signalled on abort)
            }
        }
    } else {
        // ---------------- epilogue: warp w reads TMEM lanes 32 (w % 4) .. + 31
        const int quarter = warp & 3;
        int j = 0;
        bool alive = true;
        if (n_kb == 0) pdl_wait();   // nothing orders the zero stores after the earlier kernels otherwise
        // the accumulator goes back to the MMA thread, which for a pair sits in the first CTA
        const uint32_t acc_empty_to = CTAS == 2 ? mapa_u32(bar_acc_empty, 0) : bar_acc_empty;
        auto hand_back = [&](int buf) {
            if constexpr (CTAS == 2) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(acc_empty_to + 8 * buf) : "memory");
            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty_to + 8 * buf) : "memory");
        };
        [[maybe_unused]] float* rstd_s = reinterpret_cast<float*>(gen + L::SCALE_OFF);
        [[maybe_unused]] volatile int* last_s = reinterpret_cast<volatile int*>(gen + L::SCALE_OFF + 512);
        [[maybe_unused]] const int epi_tid = quarter * 32 + lane;
        [[maybe_unused]] int scaled_y0 = -1;
        [[maybe_unused]] bool in_step = false;     // the epilogue warps synchronise among themselves in this launch
        if constexpr (X_CONTIGUOUS_OUT) in_step = p.gated || scale_ssq != nullptr || fix != 0;
        if (scale_ssq != nullptr || fix != 0) pdl_wait();     // these warps read what earlier kernels wrote
        for (int tile = worker; tile < n_tiles && alive; tile += n_workers, ++j) {
            const int buf = j & 1;
            const int x0 = (tile % p.tiles_x) * (BM * CTAS) + rank * BM, y0 = (tile / p.tiles_x) * BN;
            const int xr = x0 + quarter * 32 + lane;
            if constexpr (X_CONTIGUOUS_OUT) {
                if (scale_ssq != nullptr && y0 != scaled_y0) {
                    // 1/rms of this tile's tokens, from the per-tile sums of squares that the producer of the
                    // activations left (added in tile order: the same sum whatever else the launch holds);
                    // computed while the main loop of the tile still runs
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const int y = y0 + epi_tid;
                    float rs = 0.f;
                    if (epi_tid < BN && y < p.y_rows) {
                        float ssq = 0.f;
                        for (int i = 0; i < p.scale_tiles; ++i) ssq += scale_ssq[(size_t)i * p.y_rows + y];
                        rs = 1.0f / sqrtf(ssq / p.scale_n + p.scale_eps);
                    }
                    rstd_s[epi_tid] = rs;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    scaled_y0 = y0;
                }
            }
            // row store: a thread owns a token row, so the row's 1/rms is the thread's own (sums of squares added in
            // tile order), looked up while the tile's main loop still runs
            [[maybe_unused]] float row_scale = 1.f;
            [[maybe_unused]] float row_ssq = 0.f;        // fix == 1: this row's sum of squares over the tile's columns
            if constexpr (!X_CONTIGUOUS_OUT) {
                if (scale_ssq != nullptr && xr < p.x_rows) {
                    float ssq = 0.f;
                    for (int i = 0; i < p.scale_tiles; ++i) ssq += scale_ssq[(size_t)i * p.x_rows + xr];
                    row_scale = 1.0f / sqrtf(ssq / p.scale_n + p.scale_eps);
                }
            }
            bool ok = true;
            if (n_kb > 0) ok = mbar_wait(bar_acc_full + 8 * buf, (j >> 1) & 1, abort_flag, p.err_flag);
            ok = ok && !*abort_flag;   // the issuer signals the accumulator even when it gave up
            if constexpr (CTAS == 2) ok = ok && (p.err_flag == nullptr || *(volatile int*)p.err_flag == 0);   // ... and it may sit in the peer CTA
            alive = __all_sync(0xffffffffu, ok);
            if constexpr (X_CONTIGUOUS_OUT) {
                if (in_step) alive = epilogue_warps_all(alive);     // the warps meet at barriers below: all of them or none
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const long long out_base = (long long)blockIdx.z * p.split_stride + (long long)xr * p.stride_x;
            const uint32_t acc = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            // Row store of bf16: a thread owns a row, but 32 threads writing 32 bytes each of 32 different rows waste
            // the memory system's lines.  64 columns of the warp's 32 rows go through shared memory instead and leave
            // as whole 128-byte lines (eight lanes per row, four rows per instruction).
            constexpr int GW = L::GW;     // columns per staged group (0: no staging)
            [[maybe_unused]] const uint32_t out_stage = base + L::EPI_OFF + (X_CONTIGUOUS_OUT ? 0 : quarter * 32 * L::OUT_PITCH);
            [[maybe_unused]] auto store_lines = [&](const uint32_t (&w)[GW > 0 ? GW / 2 : 1], long long col0, long long row_stride) {
                // w: GW bf16 of this thread's row, columns col0 .. col0 + GW - 1 of the output
                if constexpr (GW > 0) {
                    constexpr int LPR = GW / 8;            // lanes (16-byte pieces) per row
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < LPR; ++q)
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(out_stage + lane * L::OUT_PITCH + q * 16),
                                     "r"(w[4 * q]), "r"(w[4 * q + 1]), "r"(w[4 * q + 2]), "r"(w[4 * q + 3]) : "memory");
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < LPR; ++i) {
                        const int rr = i * (32 / LPR) + lane / LPR, piece = lane % LPR;
                        uint32_t v0, v1, v2, v3;
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                     : "r"(out_stage + rr * L::OUT_PITCH + piece * 16) : "memory");
                        const int grow = x0 + quarter * 32 + rr;
                        if (alive && grow < p.x_rows)
                            *reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + (long long)blockIdx.z * p.split_stride + grow * row_stride + col0 + piece * 8) =
                                make_uint4(v0, v1, v2, v3);
                    }
                }
            };
            // Row store with the residual add folded in (fix == 1, one split): the 16 accumulator values of columns
            // yc .. yc + 15 of this thread's row become v = resid + product (written back to the fp32 stream), the
            // value that goes on to the store is v * norm_w (the next norm's activations without their 1/rms), and
            // the row's sum of squares grows by v^2
            // (`pre`: the row's residual values of these columns, fetched ahead by the caller, or null)
            [[maybe_unused]] auto fold16 = [&](uint32_t (&r)[16], int yc, const float4* pre) {
                if constexpr (!X_CONTIGUOUS_OUT) {
                    if (!alive || xr >= p.x_rows) return;
                    float* xp = p.resid + (size_t)xr * p.y_rows + yc;
                    const float* wp = p.norm_w + yc;
                    if (yc + 16 <= p.y_rows) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            float4 v = pre ? pre[q4] : *reinterpret_cast<const float4*>(xp + 4 * q4);
                            const float4 w4 = *reinterpret_cast<const float4*>(wp + 4 * q4);
                            v.x += __uint_as_float(r[4 * q4]); v.y += __uint_as_float(r[4 * q4 + 1]);
                            v.z += __uint_as_float(r[4 * q4 + 2]); v.w += __uint_as_float(r[4 * q4 + 3]);
                            *reinterpret_cast<float4*>(xp + 4 * q4) = v;
                            row_ssq = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, fmaf(v.x, v.x, row_ssq))));
                            r[4 * q4] = __float_as_uint(__fmul_rn(v.x, w4.x)); r[4 * q4 + 1] = __float_as_uint(__fmul_rn(v.y, w4.y));
                            r[4 * q4 + 2] = __float_as_uint(__fmul_rn(v.z, w4.z)); r[4 * q4 + 3] = __float_as_uint(__fmul_rn(v.w, w4.w));
                        }
                    } else {
                        for (int q = 0; q < 16 && yc + q < p.y_rows; ++q) {
                            const float v = xp[q] + __uint_as_float(r[q]);
                            xp[q] = v;
                            row_ssq = fmaf(v, v, row_ssq);
                            r[q] = __float_as_uint(__fmul_rn(v, wp[q]));
                        }
                    }
                }
            };
            if constexpr (!X_CONTIGUOUS_OUT && BN == 256) {
                if (p.gated) {
                    // the tile's columns are two blocks of 64 gate features followed by the 64 up features of the
                    // same indices: out[x, y0 / 2 + c] = silu(gate) * up, with the products rounded to bfloat16
                    // first (as a separate activation kernel would read them) and the rest in fp32
#pragma unroll 1
                    for (int blk = 0; blk < 2; ++blk) {      // 64 output features per block of 64 gates + 64 ups
                        static_assert(BN != 256 || L::GW == 64, "the gated epilogue stages 64 columns");
                        uint32_t w[32];
#pragma unroll
                        for (int cc = 0; cc < 64; cc += 16) {
                            uint32_t g[16], u[16];
                            __syncwarp();
                            tmem_ld16(acc + blk * 128 + cc, g);
                            tmem_ld16(acc + blk * 128 + 64 + cc, u);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                float o[2];
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const float z = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[2 * q + e]) * row_scale));
                                    const float v = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[2 * q + e]) * row_scale));
                                    o[e] = __fmul_rn(z / (1.0f + expf(-z)), v);
                                }
                                __nv_bfloat162 pr = __floats2bfloat162_rn(o[0], o[1]);
                                w[cc / 2 + q] = *reinterpret_cast<uint32_t*>(&pr);
                            }
                        }
                        store_lines(w, (y0 >> 1) + blk * 64, p.stride_x);
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) hand_back(buf);
                    continue;
                }
            }
            if constexpr (X_CONTIGUOUS_OUT && BN <= 128) {
                if (p.gated) {
                    // weights on the rows: this tile's 128 rows are 64 gate features (warps of rows 0..63) and the
                    // up features of the same indices (rows 64..127), its columns are tokens.  The up warps hand
                    // their values over through shared memory; the gate warps compute silu(gate) * up as above and
                    // store out[token, x0 / 2 + row] (for a token 32 consecutive features per warp).
                    float* exch = reinterpret_cast<float*>(gen + L::EPI_OFF);
                    const bool up_warp = quarter >= 2;
                    const int frow = (quarter & 1) * 32 + lane;        // feature within the block of 64
#pragma unroll 1
                    for (int c = 0; c < BN; c += 16) {
                        uint32_t r[16];
                        __syncwarp();
                        tmem_ld16(acc + c, r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (up_warp) {
                            float4* dst = reinterpret_cast<float4*>(exch + frow * 16);
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                dst[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                     __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");     // the four epilogue warps
                        if (!up_warp && alive) {
                            const float4* src = reinterpret_cast<const float4*>(exch + frow * 16);
                            const int feature = (x0 >> 1) + frow;
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                const float4 u4 = src[q4];
                                const float uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int y = y0 + c + 4 * q4 + e;
                                    if (y < p.y_rows && x0 + (quarter & 1) * 32 + lane < p.x_rows) {
                                        const float rs = scale_ssq ? rstd_s[c + 4 * q4 + e] : 1.f;
                                        const float z = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[4 * q4 + e]) * rs));
                                        const float v = __bfloat162float(__float2bfloat16_rn(uu[e] * rs));
                                        ((__nv_bfloat16*)p.out)[(long long)y * p.stride_y + feature] =
                                            __float2bfloat16_rn(__fmul_rn(z / (1.0f + expf(-z)), v));
                                    }
                                }
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");     // the buffer is free for the next chunk
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) hand_back(buf);
                    continue;
                }
            }
            if constexpr (!X_CONTIGUOUS_OUT && FOLD == 2) {
                if (fix == 2) {
                    // Row store with bias, rotary and the paged K/V write folded in (one split; the tile's columns are
                    // whole heads): this thread's token row holds, per head, the pairs (d, d + hd / 2) that the half-split
                    // rotation mixes.  q heads go to q_out, k and v heads to the token's slot of the cache; the
                    // arithmetic is that of the rotary kernel (separate products and sum, one rounding to bf16).
                    const bool live = alive && xr < p.x_rows;
                    const int hd = p.hd, half = hd >> 1;
                    int page = 0, off = 0;
                    bool kv_ok = false;
                    if (live && p.kv_cache && p.slot_mapping) {
                        const int slot = pyre_checked_slot(p.slot_mapping[xr], p.n_pages, p.page_size, p.err_flag);
                        if (slot >= 0) { page = slot / p.page_size; off = slot - page * p.page_size; kv_ok = true; }
                    }
                    const float* ct = p.cos_t + (size_t)(live ? xr : 0) * half;
                    const float* st = p.sin_t + (size_t)(live ? xr : 0) * half;
#pragma unroll 1
                    for (int hc = 0; hc < BN && y0 + hc < p.y_rows; hc += hd) {
                        const int gh = (y0 + hc) / hd;
                        const bool is_v = gh >= p.nh + p.nkv, is_k = !is_v && gh >= p.nh;
                        __nv_bfloat16* dst = nullptr;
                        if (live) {
                            if (!is_k && !is_v) dst = (__nv_bfloat16*)p.q_out + ((size_t)xr * p.nh + gh) * hd;
                            else if (kv_ok) dst = (__nv_bfloat16*)p.kv_cache +
                                (((size_t)(page * 2 + (is_v ? 1 : 0)) * p.nkv + (is_k ? gh - p.nh : gh - p.nh - p.nkv)) * p.page_size + off) * hd;
                        }
                        const bool rotate = !is_v && p.rot != 0;
#pragma unroll 1
                        for (int c = 0; c < half; c += 16) {
                            // the tables' 16 values of this token (32 bytes per request, asked for before the
                            // accumulator is read), then 32 bytes per store: whole sectors
                            float cs[16], sn[16];
                            if (rotate && dst != nullptr) {
                                ld_global_32B(ct + c, cs); ld_global_32B(ct + c + 8, cs + 8);
                                ld_global_32B(st + c, sn); ld_global_32B(st + c + 8, sn + 8);
                            }
                            uint32_t lo[16], hi[16];
                            __syncwarp();
                            tmem_ld16(acc + hc + c, lo);
                            tmem_ld16(acc + hc + half + c, hi);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            if (dst == nullptr) continue;
                            uint32_t w1[8], w2[8];
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                float4 b1 = make_float4(0.f, 0.f, 0.f, 0.f), b2 = b1;
                                if (p.bias) {
                                    b1 = *reinterpret_cast<const float4*>(p.bias + y0 + hc + c + 4 * q4);
                                    b2 = *reinterpret_cast<const float4*>(p.bias + y0 + hc + half + c + 4 * q4);
                                }
                                const float bb1[4] = {b1.x, b1.y, b1.z, b1.w}, bb2[4] = {b2.x, b2.y, b2.z, b2.w};
                                const float* cc = cs + 4 * q4;
                                const float* ss = sn + 4 * q4;
                                float o1[4], o2[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float a1 = __fadd_rn(__fmul_rn(__uint_as_float(lo[4 * q4 + e]), row_scale), bb1[e]);
                                    const float a2 = __fadd_rn(__fmul_rn(__uint_as_float(hi[4 * q4 + e]), row_scale), bb2[e]);
                                    o1[e] = rotate ? __fadd_rn(__fmul_rn(a1, cc[e]), __fmul_rn(-a2, ss[e])) : a1;
                                    o2[e] = rotate ? __fadd_rn(__fmul_rn(a2, cc[e]), __fmul_rn(a1, ss[e])) : a2;
                                }
                                __nv_bfloat162 v;
                                v = __floats2bfloat162_rn(o1[0], o1[1]); w1[2 * q4] = *reinterpret_cast<uint32_t*>(&v);
                                v = __floats2bfloat162_rn(o1[2], o1[3]); w1[2 * q4 + 1] = *reinterpret_cast<uint32_t*>(&v);
                                v = __floats2bfloat162_rn(o2[0], o2[1]); w2[2 * q4] = *reinterpret_cast<uint32_t*>(&v);
                                v = __floats2bfloat162_rn(o2[2], o2[3]); w2[2 * q4 + 1] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            st_global_32B(dst + c, w1);
                            st_global_32B(dst + half + c, w2);
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) hand_back(buf);
                    continue;
                }
            }
            int c_begin = 0;
            [[maybe_unused]] bool folded_in_lines = false;
            if constexpr (!X_CONTIGUOUS_OUT && FOLD == 1 && GW == 64) {
                if (fix == 1 && scale_ssq == nullptr && n_kb > 0) {
                    // The residual fold in whole lines.  A thread that owns a token row would touch 32 different
                    // 128-byte lines of the fp32 stream per instruction with its warp (rows lie kilobytes apart), so
                    // the accumulator values of 32 columns go through shared memory (the bf16 staging area: 32 rows of
                    // 128 bytes per warp) and the warp works on four rows per instruction, eight lanes per row of
                    // 128 bytes: residual read, sum written back, sum of squares, activations (sum x norm weight) as
                    // bf16.  The residual values of the next 32 columns are fetched while these are worked on.
                    constexpr int UW = 32;
                    const int units = min(BN, p.y_rows - y0) / UW;
                    const int rsub = lane >> 3, piece = lane & 7;
                    const int row0 = x0 + quarter * 32;
                    float part[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) part[i] = 0.f;
                    float4 cur[8], nxt[8];
                    auto fetch = [&](int u, float4 (&dst)[8]) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int grow = row0 + i * 4 + rsub;
                            dst[i] = (alive && grow < p.x_rows)
                                ? *reinterpret_cast<const float4*>(p.resid + (size_t)grow * p.y_rows + y0 + u * UW + piece * 4)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    };
                    if (units > 0) fetch(0, cur);
#pragma unroll 1
                    for (int u = 0; u < units; ++u) {
                        if (u + 1 < units) fetch(u + 1, nxt);
                        uint32_t r0[16], r1[16];
                        __syncwarp();     // every lane has read the staging area of the unit before
                        tmem_ld16(acc + u * UW, r0);
                        tmem_ld16(acc + u * UW + 16, r1);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(out_stage + lane * L::OUT_PITCH + q * 16),
                                         "r"(r0[4 * q]), "r"(r0[4 * q + 1]), "r"(r0[4 * q + 2]), "r"(r0[4 * q + 3]) : "memory");
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(out_stage + lane * L::OUT_PITCH + 64 + q * 16),
                                         "r"(r1[4 * q]), "r"(r1[4 * q + 1]), "r"(r1[4 * q + 2]), "r"(r1[4 * q + 3]) : "memory");
                        }
                        __syncwarp();
                        const int col = y0 + u * UW + piece * 4;
                        const float4 w4 = *reinterpret_cast<const float4*>(p.norm_w + col);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = i * 4 + rsub, grow = row0 + rr;
                            uint32_t a0, a1, a2, a3;
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                                         : "r"(out_stage + rr * L::OUT_PITCH + piece * 16) : "memory");
                            if (alive && grow < p.x_rows) {
                                float4 v = cur[i];
                                v.x += __uint_as_float(a0); v.y += __uint_as_float(a1);
                                v.z += __uint_as_float(a2); v.w += __uint_as_float(a3);
                                *reinterpret_cast<float4*>(p.resid + (size_t)grow * p.y_rows + col) = v;
                                part[i] = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, fmaf(v.x, v.x, part[i]))));
                                __nv_bfloat162 lo = __floats2bfloat162_rn(__fmul_rn(v.x, w4.x), __fmul_rn(v.y, w4.y));
                                __nv_bfloat162 hi = __floats2bfloat162_rn(__fmul_rn(v.z, w4.z), __fmul_rn(v.w, w4.w));
                                *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + (long long)grow * p.stride_x + col) =
                                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
                    }
                    // a row's sum of squares: over its eight lanes, then to the thread that owns the row
                    // (row i * 4 + rsub sits in lanes 8 rsub .. 8 rsub + 7; the owner of row r is lane r)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        part[i] += __shfl_xor_sync(0xffffffffu, part[i], 1);
                        part[i] += __shfl_xor_sync(0xffffffffu, part[i], 2);
                        part[i] += __shfl_xor_sync(0xffffffffu, part[i], 4);
                        const float mine = __shfl_sync(0xffffffffu, part[i], 8 * (lane & 3));
                        if ((lane >> 2) == i) row_ssq = mine;
                    }
                    c_begin = units * UW;
                    folded_in_lines = true;
                }
            }
            if constexpr (!X_CONTIGUOUS_OUT && GW == 64) {
                if (p.out_f32 && n_kb > 0 && fix == 0) {
                    // fp32 partial sums of a split K, in whole lines as well: 32 columns of the warp's 32 rows go
                    // through the staging area and leave as 128 bytes per row, four rows per instruction (a thread
                    // storing 16 bytes of its own row makes its warp touch 32 lines per instruction, and with one
                    // tile per CTA nothing hides this epilogue)
                    const int units = min(BN, p.y_rows - y0) / 32;
                    const int rsub = lane >> 3, piece = lane & 7;
                    const int row0 = x0 + quarter * 32;
#pragma unroll 1
                    for (int u = 0; u < units; ++u) {
                        uint32_t r0[16], r1[16];
                        __syncwarp();     // every lane has read the staging area of the unit before
                        tmem_ld16(acc + u * 32, r0);
                        tmem_ld16(acc + u * 32 + 16, r1);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (scale_ssq != nullptr) {
#pragma unroll
                            for (int q = 0; q < 16; ++q) {
                                r0[q] = __float_as_uint(__uint_as_float(r0[q]) * row_scale);
                                r1[q] = __float_as_uint(__uint_as_float(r1[q]) * row_scale);
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(out_stage + lane * L::OUT_PITCH + q * 16),
                                         "r"(r0[4 * q]), "r"(r0[4 * q + 1]), "r"(r0[4 * q + 2]), "r"(r0[4 * q + 3]) : "memory");
                            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(out_stage + lane * L::OUT_PITCH + 64 + q * 16),
                                         "r"(r1[4 * q]), "r"(r1[4 * q + 1]), "r"(r1[4 * q + 2]), "r"(r1[4 * q + 3]) : "memory");
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = i * 4 + rsub, grow = row0 + rr;
                            uint32_t a0, a1, a2, a3;
                            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                                         : "r"(out_stage + rr * L::OUT_PITCH + piece * 16) : "memory");
                            if (alive && grow < p.x_rows)
                                *reinterpret_cast<uint4*>((float*)p.out + (long long)blockIdx.z * p.split_stride +
                                                          (long long)grow * p.stride_x + y0 + u * 32 + piece * 4) = make_uint4(a0, a1, a2, a3);
                        }
                    }
                    c_begin = units * 32;
                }
            }
            if constexpr (!X_CONTIGUOUS_OUT && GW > 0) {
                if (!folded_in_lines && !p.out_f32 && n_kb > 0) {
                    const int whole = min(BN, p.y_rows - y0) / GW;      // groups of GW columns inside the matrix
#pragma unroll 1
                    for (int gq = 0; gq < whole; ++gq) {
                        uint32_t w[GW / 2];
                        // the fold's residual values of the whole group go out at once: one round trip to memory per
                        // group of GW columns, not one per 16
                        float4 xg[GW / 4];
                        const bool prefetched = fix1_rows && alive && xr < p.x_rows;
                        if (prefetched) {
                            const float4* src = reinterpret_cast<const float4*>(p.resid + (size_t)xr * p.y_rows + y0 + gq * GW);
#pragma unroll
                            for (int i = 0; i < GW / 4; ++i) xg[i] = src[i];
                        }
#pragma unroll
                        for (int cc = 0; cc < GW; cc += 16) {
                            uint32_t r[16];
                            __syncwarp();
                            tmem_ld16(acc + gq * GW + cc, r);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            if (fix1_rows) fold16(r, y0 + gq * GW + cc, prefetched ? &xg[cc / 4] : nullptr);
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * q]) * row_scale, __uint_as_float(r[2 * q + 1]) * row_scale);
                                w[cc / 2 + q] = *reinterpret_cast<uint32_t*>(&v);
                            }
                        }
                        store_lines(w, y0 + gq * GW, p.stride_x);
                    }
                    c_begin = whole * GW;
                }
            }
#pragma unroll 1
            for (int c = c_begin; c < BN; c += 16) {
                uint32_t r[16];
                __syncwarp();   // tcgen05.ld is warp-wide: converge after the per-thread stores
                if (n_kb > 0) {
                    tmem_ld16(acc + c, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int q = 0; q < 16; ++q) r[q] = 0u;
                }
                if constexpr (!X_CONTIGUOUS_OUT) {
                    if (fix1_rows) fold16(r, y0 + c, nullptr);
                    if (scale_ssq != nullptr) {
#pragma unroll
                        for (int q = 0; q < 16; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * row_scale);
                    }
                }
                if (!alive || xr >= p.x_rows) {
                    // nothing to store for this thread
                } else if constexpr (!X_CONTIGUOUS_OUT) {
                    // a thread owns a row of the output: 16 consecutive elements (stride_y == 1)
                    const int yc = y0 + c;
                    if (yc + 16 <= p.y_rows) {
                        if (p.out_f32) {
                            float4* dst = reinterpret_cast<float4*>((float*)p.out + out_base + yc);
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                dst[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                     __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                        } else {
                            uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + out_base + yc);
                            uint32_t w[8];
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1]));
                                w[q] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    } else {
                        for (int q = 0; q < 16 && yc + q < p.y_rows; ++q) {
                            const float v = __uint_as_float(r[q]);
                            if (p.out_f32) ((float*)p.out)[out_base + yc + q] = v;
                            else ((__nv_bfloat16*)p.out)[out_base + yc + q] = __float2bfloat16_rn(v);
                        }
                    }
                } else {
                    // transposed store: for each y the 32 lanes write 32 consecutive x (stride_x == 1)
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        const int y = y0 + c + q;
                        if (y < p.y_rows) {
                            float v = __uint_as_float(r[q]);
                            if constexpr (X_CONTIGUOUS_OUT) { if (scale_ssq) v *= rstd_s[c + q]; }
                            if (p.out_f32) ((float*)p.out)[out_base + (long long)y * p.stride_y] = v;
                            else ((__nv_bfloat16*)p.out)[out_base + (long long)y * p.stride_y] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
            // this warp has read its quarter of the accumulator: hand the buffer back to the MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) hand_back(buf);
            if constexpr (!X_CONTIGUOUS_OUT) {
                if (fix1_rows && alive && xr < p.x_rows) p.ssq_out[(size_t)(tile / p.tiles_x) * p.x_rows + xr] = row_ssq;
            }
            if constexpr (X_CONTIGUOUS_OUT && BN <= 128) {
                if (fix != 0) {
                    // ---- fix-up: every split of this tile has stored its partial sums; the CTA that arrives last
                    // adds them up (in split order, whichever CTA does it) and finishes the tile
                    __threadfence();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (epi_tid == 0) {
                        int last = 1;
                        if (gridDim.z > 1) {
                            last = atomicAdd(p.tile_counters + tile, 1) == (int)gridDim.z - 1;
                            if (last) p.tile_counters[tile] = 0;      // ready for the next launch
                        }
                        *last_s = last;
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (*last_s && alive) {
                        __threadfence();
                        const int n0 = x0 + 4 * lane;                       // this lane's four features of the tile
                        const bool in = n0 < p.x_rows;                      // x_rows % 4 == 0: all four or none
                        const int t_end = min(y0 + BN, p.y_rows);
                        const float* parts = (const float*)p.out;
                        const int n_parts = (int)gridDim.z;
                        if (fix == 1) {
                            float4 w4 = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (in) w4 = *reinterpret_cast<const float4*>(p.norm_w + n0);
#pragma unroll 2
                            for (int t = y0 + quarter; t < t_end; t += 4) {           // a warp per token
                                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (in) {
                                    const size_t at = (size_t)t * p.stride_y + n0;
                                    float4 acc = __ldcg(reinterpret_cast<const float4*>(parts + at));
                                    for (int z = 1; z < n_parts; ++z) {
                                        const float4 q = __ldcg(reinterpret_cast<const float4*>(parts + (size_t)z * p.split_stride + at));
                                        acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
                                    }
                                    float* xr4 = p.resid + (size_t)t * p.x_rows + n0;
                                    v = *reinterpret_cast<const float4*>(xr4);
                                    v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
                                    *reinterpret_cast<float4*>(xr4) = v;
                                    __nv_bfloat162 lo = __floats2bfloat162_rn(__fmul_rn(v.x, w4.x), __fmul_rn(v.y, w4.y));
                                    __nv_bfloat162 hi = __floats2bfloat162_rn(__fmul_rn(v.z, w4.z), __fmul_rn(v.w, w4.w));
                                    *reinterpret_cast<uint2*>(p.h_out + (size_t)t * p.x_rows + n0) =
                                        make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                                }
                                float ss = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, v.x * v.x)));
                                ss = warp_sum(ss);
                                if (lane == 0) p.ssq_out[(size_t)(tile % p.tiles_x) * p.y_rows + t] = ss;
                            }
                        } else {
                            const int hd = p.hd, half = p.rot >> 1;
                            const int head = n0 / hd, d = n0 - head * hd;
                            const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
                            const bool rotate = p.rot > 0 && (is_q || is_k);
                            const int jj = d < half ? d : d - half;
                            float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (in && p.bias) b4 = *reinterpret_cast<const float4*>(p.bias + n0);
#pragma unroll 2
                            for (int t = y0 + quarter; t < t_end; t += 4) {
                                float4 x4 = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (in) {
                                    const size_t at = (size_t)t * p.stride_y + n0;
                                    x4 = __ldcg(reinterpret_cast<const float4*>(parts + at));
                                    for (int z = 1; z < n_parts; ++z) {
                                        const float4 q = __ldcg(reinterpret_cast<const float4*>(parts + (size_t)z * p.split_stride + at));
                                        x4.x += q.x; x4.y += q.y; x4.z += q.z; x4.w += q.w;
                                    }
                                    x4.x += b4.x; x4.y += b4.y; x4.z += b4.z; x4.w += b4.w;
                                }
                                // the other half of the rotation's pairs sits hd / 8 lanes away (every lane takes part)
                                float4 o4;
                                o4.x = __shfl_xor_sync(0xffffffffu, x4.x, hd >> 3);
                                o4.y = __shfl_xor_sync(0xffffffffu, x4.y, hd >> 3);
                                o4.z = __shfl_xor_sync(0xffffffffu, x4.z, hd >> 3);
                                o4.w = __shfl_xor_sync(0xffffffffu, x4.w, hd >> 3);
                                if (!in) continue;
                                if (rotate) {
                                    const float4 c4 = *reinterpret_cast<const float4*>(p.cos_t + (size_t)t * half + jj);
                                    const float4 s4 = *reinterpret_cast<const float4*>(p.sin_t + (size_t)t * half + jj);
                                    if (d < half) {      // out[j] = x[j] cos - x[j + half] sin, products rounded apart
                                        x4.x = __fadd_rn(__fmul_rn(x4.x, c4.x), __fmul_rn(-o4.x, s4.x));
                                        x4.y = __fadd_rn(__fmul_rn(x4.y, c4.y), __fmul_rn(-o4.y, s4.y));
                                        x4.z = __fadd_rn(__fmul_rn(x4.z, c4.z), __fmul_rn(-o4.z, s4.z));
                                        x4.w = __fadd_rn(__fmul_rn(x4.w, c4.w), __fmul_rn(-o4.w, s4.w));
                                    } else {             // out[j + half] = x[j + half] cos + x[j] sin
                                        x4.x = __fadd_rn(__fmul_rn(x4.x, c4.x), __fmul_rn(o4.x, s4.x));
                                        x4.y = __fadd_rn(__fmul_rn(x4.y, c4.y), __fmul_rn(o4.y, s4.y));
                                        x4.z = __fadd_rn(__fmul_rn(x4.z, c4.z), __fmul_rn(o4.z, s4.z));
                                        x4.w = __fadd_rn(__fmul_rn(x4.w, c4.w), __fmul_rn(o4.w, s4.w));
                                    }
                                }
                                __nv_bfloat162 lo = __floats2bfloat162_rn(x4.x, x4.y), hi = __floats2bfloat162_rn(x4.z, x4.w);
                                const uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                                if (is_q) {
                                    *reinterpret_cast<uint2*>(p.q_out + ((size_t)t * p.nh + head) * hd + d) = packed;
                                } else if (p.kv_cache != nullptr) {
                                    const int slot = pyre_checked_slot(p.slot_mapping[t], p.n_pages, p.page_size, p.err_flag);
                                    if (slot >= 0) {
                                        const int page = slot / p.page_size, off = slot - page * p.page_size;
                                        const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
                                        const size_t row = ((size_t)(page * 2 + (is_k ? 0 : 1)) * p.nkv + kvh) * p.page_size + off;
                                        *reinterpret_cast<uint2*>(p.kv_cache + row * hd + d) = packed;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    // ---------------- teardown: all tensor-memory reads are done before the columns are freed
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (CTAS == 2) cluster_sync_all();     // neither CTA leaves while the other may still touch its memory or barriers
    else __syncthreads();
    if (warp == 1) {
        __syncwarp();
        if constexpr (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- host side
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

// [rows, K] bf16 row-major with leading dimension ld (elements); boxes of box_rows x 64, 128B swizzle.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return PYRE_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : PYRE_ERR_BAD_ARG;
}

template <int BN, int STAGES, bool XC, int CTAS = 1, int FOLD = 1>
int launch(const CUtensorMap& mx, const CUtensorMap& my, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES, XC, CTAS>;
    static_assert(L::TOTAL <= 232448, "the ring does not fit into shared memory");
    static bool configured_on[PYRE_MAX_DEVICES] = {};      // the attributes are per device
    bool& configured = configured_on[pyre_current_device()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, XC, CTAS, FOLD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e;
    if constexpr (CTAS == 2) {
        // pairs of CTAs: a cluster of two along x (the two SMs of a TPC), with the dependent-launch attribute as everywhere
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = (size_t)L::TOTAL;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pyre_pdl_enabled() ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES, XC, CTAS, FOLD>, mx, my, p);
    } else {
        e = pyre_launch(gemm_tc_kernel<BN, STAGES, XC, CTAS, FOLD>, grid, dim3(THREADS), (size_t)L::TOTAL, stream, mx, my, p);
    }
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

// The row store of one CTA per tile: the variant without the folded work exists at 128 columns only, the one with the
// rotary epilogue at 128 and 256.
template <int BN, int STAGES>
int launch_rows(const CUtensorMap& mx, const CUtensorMap& my, const GemmParams& p, dim3 grid, cudaStream_t stream, bool fold) {
    if constexpr (BN == 128) {
        if (!fold) return launch<BN, STAGES, false, 1, 0>(mx, my, p, grid, stream);
    }
    if (p.fix == 2) {          // the rotary epilogue: tiles of whole heads, 128 or 256 columns
        if constexpr (BN == 128 || BN == 256) return launch<BN, STAGES, false, 1, 2>(mx, my, p, grid, stream);
        else return PYRE_ERR_BAD_ARG;
    }
    return launch<BN, STAGES, false>(mx, my, p, grid, stream);
}

}  // namespace

// D[x, y] = sum_k X[x, k] Y[y, k] for bf16 X [x_rows, K] (leading dimension ldx) and Y [y_rows, K] (ldy).
// out[z * split_stride + x * stride_x + y * stride_y] receives split z's partial sum (fp32 if
// out_f32 else bf16).  One of stride_x, stride_y must be 1: stride_x == 1 selects the transposed
// store (X = weights), stride_y == 1 the row store (X = tokens).  bn: tile width along y, one of
// 16, 32, 64, 128, 256, and for the row store also 160, 192, 208, 224.  splits >= 1 divides the K blocks among blockIdx.z.  x_is_constant says
// which operand holds weights: its first tiles are fetched before the kernel waits for the
// kernels before it in the stream (programmatic dependent launch).  gated: the weight operand holds gate
// and up rows interleaved in blocks of 64 (64 gate rows, the up rows of the same features, ...); the output is
// silu(gate product) * (up product), half as many features: row store (weights = Y, bn 256, out[x, j]) or
// transposed store (weights = X, bn <= 128, out[y * stride_y + j]); one split, bf16 out.  pair: two CTAs of a
// cluster share each 256 x bn tile (row store, bn 128, 160, 192, 208, 224 or 256).
//
// fx (may be null): work folded into a product with the transposed store (weights = X, at most 128 tokens = Y in one
// tile): `scale_ssq` scales the rows of the result by the 1/rms of a norm whose weight the activations already carry;
// `fix` = 1 / 2 has the CTA that finishes a tile last add up the splits' partial sums (out must be fp32 partials
// [splits][y_rows][x_rows]) and turn them into the residual update with the next norm's preparation, or into the
// rotated queries and the cache's keys and values.  See GemmParams.
struct PyreGemmFix {
    int fix;
    int scale_tiles;
    float scale_n, scale_eps;
    const float* scale_ssq;
    int* tile_counters;
    float* resid;
    const float* norm_w;
    void* h_out;
    float* ssq_out;
    const float* bias;
    const float* cos_t;
    const float* sin_t;
    void* q_out;
    void* kv_cache;
    const int* slot_mapping;
    int nh, nkv, hd, rot, page_size;
    long long n_pages;
};

static int gemm_tc_impl(const void* X, int x_rows, long long ldx, const void* Y, int y_rows, long long ldy, int K,
                        void* out, int out_f32, long long stride_x, long long stride_y, long long split_stride,
                        int splits, int bn, int x_is_constant, int gated, int pair, int* err_flag, const PyreGemmFix* fx,
                        cudaStream_t stream) {
    if (x_rows <= 0 || y_rows <= 0) return 0;
    if (fx && (fx->fix != 0 || fx->scale_ssq != nullptr) && stride_x != 1) {
        // row store (tokens on the rows): every thread of the epilogue owns a token row, so the row scale and the
        // residual fold (fix == 1) need no exchange between CTAs; one split, no gate with the fold, bf16 out
        if (fx->scale_ssq && fx->scale_tiles < 1) return PYRE_ERR_BAD_ARG;
        if (fx->fix == 1 && (splits != 1 || gated || out_f32 || !fx->resid || !fx->norm_w || !fx->ssq_out)) return PYRE_ERR_BAD_ARG;
        if (fx->fix == 2) {
            // bias + rotary + cache write in the epilogue: whole heads per tile, pairs in chunks of 16
            if (splits != 1 || gated || out_f32) return PYRE_ERR_BAD_ARG;
            if (fx->hd <= 0 || fx->hd % 32 || bn % fx->hd || (fx->rot != 0 && fx->rot != fx->hd) || !fx->q_out ||
                y_rows != (fx->nh + 2 * fx->nkv) * fx->hd || fx->page_size <= 0 || (fx->kv_cache && !fx->slot_mapping) ||
                (fx->rot && (!fx->cos_t || !fx->sin_t)))
                return PYRE_ERR_UNSUPPORTED;
            // the epilogue moves 32 bytes per request: tables, queries and cache rows start on such boundaries
            if ((((uintptr_t)fx->q_out | (uintptr_t)fx->kv_cache | (uintptr_t)fx->cos_t | (uintptr_t)fx->sin_t) & 31) != 0) return PYRE_ERR_UNSUPPORTED;
        }
        if (fx->fix != 0 && fx->fix != 1 && fx->fix != 2) return PYRE_ERR_BAD_ARG;
    } else if (fx && (fx->fix != 0 || fx->scale_ssq != nullptr)) {
        if (stride_x != 1 || bn > 128 || y_rows > bn || pair) return PYRE_ERR_BAD_ARG;      // transposed store, one tile of tokens
        if (fx->scale_ssq && fx->scale_tiles < 1) return PYRE_ERR_BAD_ARG;
        if (fx->fix != 0) {
            if (gated || !out_f32 || x_rows % 4 || stride_y != x_rows || !fx->tile_counters) return PYRE_ERR_BAD_ARG;
            if (fx->fix == 1 && (!fx->resid || !fx->norm_w || !fx->h_out || !fx->ssq_out)) return PYRE_ERR_BAD_ARG;
            if (fx->fix == 2) {
                if (fx->hd <= 0 || 128 % fx->hd || fx->hd % 8 || (fx->rot != 0 && fx->rot != fx->hd) || !fx->q_out ||
                    x_rows != (fx->nh + 2 * fx->nkv) * fx->hd || fx->page_size <= 0 || (fx->kv_cache && !fx->slot_mapping) ||
                    (fx->rot && (!fx->cos_t || !fx->sin_t)))
                    return PYRE_ERR_UNSUPPORTED;
            } else if (fx->fix != 1) return PYRE_ERR_BAD_ARG;
        }
    }
    // the gated epilogue: whole tiles of gate/up rows interleaved in blocks of 64, one split, bf16 out; with the
    // tokens on the row side 256-wide tiles, with the weights on the row side at most 128 tokens per tile
    if (gated && (splits != 1 || out_f32)) return PYRE_ERR_BAD_ARG;
    if (gated && stride_y == 1 && stride_x != 1 && (bn != 256 || y_rows % 256)) return PYRE_ERR_BAD_ARG;
    if (gated && stride_x == 1 && (bn > 128 || x_rows % 128)) return PYRE_ERR_BAD_ARG;
    if (K <= 0 || K % 8 || ldx % 8 || ldy % 8 || splits < 1) return PYRE_ERR_UNSUPPORTED;
    if (((uintptr_t)X & 15) || ((uintptr_t)Y & 15)) return PYRE_ERR_UNSUPPORTED;
    if (stride_x != 1 && stride_y != 1) return PYRE_ERR_BAD_ARG;
    const bool xc = (stride_x == 1);
    if (!xc && ((stride_x % 8) || ((uintptr_t)out & 15))) return PYRE_ERR_UNSUPPORTED;  // vector stores of a row
    if (pair && (xc || bn < 128)) return PYRE_ERR_BAD_ARG;     // pairs of CTAs serve the row store, widths from 128
    CUtensorMap mx, my;
    int rc = make_map(&mx, X, x_rows, K, ldx, BM);
    if (rc) return rc;
    rc = make_map(&my, Y, y_rows, K, ldy, pair ? bn / 2 : bn);      // a CTA of a pair fetches half of the tile's Y rows
    if (rc) return rc;
    const int total_kb = (K + BK - 1) / BK;
    if (splits > total_kb) splits = total_kb;
    GemmParams p;
    p.x_rows = x_rows; p.y_rows = y_rows; p.K = K;
    p.k_blocks_per_split = (total_kb + splits - 1) / splits;
    p.stride_x = stride_x; p.stride_y = stride_y; p.split_stride = split_stride;
    p.out = out; p.out_f32 = out_f32; p.x_is_constant = x_is_constant; p.err_flag = err_flag; p.gated = gated ? 1 : 0;
    p.scale_ssq = nullptr; p.scale_tiles = 0; p.scale_n = 0.f; p.scale_eps = 0.f; p.fix = 0; p.tile_counters = nullptr;
    p.resid = nullptr; p.norm_w = nullptr; p.h_out = nullptr; p.ssq_out = nullptr; p.bias = nullptr; p.cos_t = p.sin_t = nullptr;
    p.q_out = nullptr; p.kv_cache = nullptr; p.slot_mapping = nullptr; p.nh = p.nkv = p.hd = p.rot = p.page_size = 0; p.n_pages = 0;
    if (fx) {
        p.scale_ssq = fx->scale_ssq; p.scale_tiles = fx->scale_tiles; p.scale_n = fx->scale_n; p.scale_eps = fx->scale_eps;
        p.fix = fx->fix; p.tile_counters = fx->tile_counters; p.resid = fx->resid; p.norm_w = fx->norm_w;
        p.h_out = (__nv_bfloat16*)fx->h_out; p.ssq_out = fx->ssq_out; p.bias = fx->bias; p.cos_t = fx->cos_t; p.sin_t = fx->sin_t;
        p.q_out = (__nv_bfloat16*)fx->q_out; p.kv_cache = (__nv_bfloat16*)fx->kv_cache; p.slot_mapping = fx->slot_mapping;
        p.nh = fx->nh; p.nkv = fx->nkv; p.hd = fx->hd; p.rot = fx->rot; p.page_size = fx->page_size; p.n_pages = fx->n_pages;
    }
    p.tiles_x = ceil_div(x_rows, pair ? 2 * BM : BM); p.tiles_y = ceil_div(y_rows, bn);
    const long long n_tiles = (long long)p.tiles_x * p.tiles_y;
    // one CTA per SM stays resident and walks the tiles (a split K keeps one CTA per tile and split)
    const int sm_count = pyre_sm_count();
    long long ctas = splits > 1 ? n_tiles : (n_tiles < sm_count ? n_tiles : sm_count);
    if (xc && splits == 1 && n_tiles > sm_count) {
        // A weight stream (few tokens) is bound by memory: what counts is that no round of the persistent CTAs
        // runs nearly empty at the end while the memory system idles.  Take the CTA count, at least 7/8 of the
        // SMs, that fills the rounds best (1188 tiles: 132 CTAs x 9 rounds instead of 148 x 8 + 4).
        long long best = sm_count, best_waste = ((n_tiles + sm_count - 1) / sm_count) * sm_count - n_tiles;
        for (long long g = sm_count - 1; g >= sm_count - sm_count / 8 && best_waste > 0; --g) {
            const long long waste = ((n_tiles + g - 1) / g) * g - n_tiles;
            if (waste * sm_count < best_waste * g) { best = g; best_waste = waste; }
        }
        ctas = best;
    }
    if (pair) {
        // one pair per TPC stays resident (a split K keeps one pair per tile and split)
        const long long pairs = splits > 1 ? n_tiles : (n_tiles < sm_count / 2 ? n_tiles : sm_count / 2);
        dim3 grid2((unsigned)(2 * pairs), 1, splits);
        if (p.fix == 2) {      // the rotary epilogue: tiles of whole heads
            switch (bn) {
                case 128: return launch<128, 8, false, 2, 2>(mx, my, p, grid2, stream);
                case 256: return launch<256, 6, false, 2, 2>(mx, my, p, grid2, stream);
                default: return PYRE_ERR_BAD_ARG;
            }
        }
        // plain products (decode steps of 129-256 requests) run the variant without the folded work: few registers,
        // so that the next kernels' CTAs find room beside the draining pairs
        const bool plain = p.fix == 0 && p.scale_ssq == nullptr;
#define GO2(BN_, ST_) return plain ? launch<BN_, ST_, false, 2, 0>(mx, my, p, grid2, stream) : launch<BN_, ST_, false, 2, 1>(mx, my, p, grid2, stream)
        switch (bn) {
            case 128: GO2(128, 8);
            case 160: GO2(160, 7);
            case 192: GO2(192, 7);
            case 208: GO2(208, 7);
            case 224: GO2(224, 6);
            case 256: GO2(256, 6);
            default: return PYRE_ERR_BAD_ARG;
        }
#undef GO2
    }
    dim3 grid((unsigned)ctas, 1, splits);
    // the plain products run the variant without that code: the weight stream always, the row store at the one width
    // that decode steps of 33-128 tokens use (96 registers, held there by its launch bounds, instead of 183: two of the attention's CTAs fit beside it)
    const bool fold = p.fix != 0 || p.scale_ssq != nullptr;
#define GO(BN_, ST_)                                                              \
    rc = !xc ? launch_rows<BN_, ST_>(mx, my, p, grid, stream, fold)                               \
        : fold ? launch<BN_, ST_, true, 1, 1>(mx, my, p, grid, stream)                              \
               : launch<BN_, ST_, true, 1, 0>(mx, my, p, grid, stream)
    switch (bn) {
        case 16: GO(16, 10); break;
        case 32: GO(32, 10); break;
        case 64: GO(64, 8); break;
        case 128: GO(128, 6); break;
        case 256: GO(256, 4); break;
        // widths between 128 and 256 exist for the row-store orientation only: they let the planner pick the
        // tile count that fills the rounds of the persistent CTAs best
        case 160: if (xc || p.fix == 2) return PYRE_ERR_BAD_ARG; rc = launch<160, 5, false>(mx, my, p, grid, stream); break;
        case 192: if (xc || p.fix == 2) return PYRE_ERR_BAD_ARG; rc = launch<192, 5, false>(mx, my, p, grid, stream); break;
        case 208: if (xc || p.fix == 2) return PYRE_ERR_BAD_ARG; rc = launch<208, 5, false>(mx, my, p, grid, stream); break;
        case 224: if (xc || p.fix == 2) return PYRE_ERR_BAD_ARG; rc = launch<224, 5, false>(mx, my, p, grid, stream); break;
        default: return PYRE_ERR_BAD_ARG;
    }
#undef GO
    return rc;
}

PYRE_API int pyre_gemm_tc(const void* X, int x_rows, long long ldx, const void* Y, int y_rows, long long ldy, int K,
                          void* out, int out_f32, long long stride_x, long long stride_y, long long split_stride,
                          int splits, int bn, int x_is_constant, int gated, int pair, int* err_flag,
                          const PyreGemmFix* fx, cudaStream_t stream) {
    return gemm_tc_impl(X, x_rows, ldx, Y, y_rows, ldy, K, out, out_f32, stride_x, stride_y, split_stride, splits, bn,
                        x_is_constant, gated, pair, err_flag, fx, stream);
}
