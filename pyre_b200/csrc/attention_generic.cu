// Paged attention over the block table, any head size that is a multiple of 16, any
// page size, float32 or bfloat16 storage, fp32 arithmetic throughout.
//
// This is the exact kernel: it serves the whole 32-bit path and every head size the
// tensor-core kernels do not cover.  One warp owns one (query token, query head) and
// walks the keys of that token's sequence in chunks of 32, from the start of its
// window to the token's own position, with an online softmax (running maximum m, sum l
// and an fp32 accumulator).  Prompt portions and single decoded tokens are the same
// case: a query at absolute position p sees the cached keys lo..p, where
// lo = max(0, p - window + 1) with a window and 0 without; the keys of the current
// portion were written to the pages before this kernel runs.
//
// The arithmetic of one (token, head) depends on nothing but its own keys: the chunks
// are aligned to multiples of 32 from position 0 and every sum has a fixed order, so
// the result is bit-identical however the tokens were cut into steps, whatever else is
// in the batch and wherever the pages lie.
//
// Formula: pyre/model.py:104-124 (scores = (q k^T) * scale, causal mask, fp32 softmax,
// probs v) and pyre/kernels/paged_attn.py:43-71 (online softmax over the block table);
// query head h reads key/value head h / (nh / nkv) (pyre/model.py:66-72).
#include "common.cuh"

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* q,             // [n_tokens, nh, hd]
    const T* cache,         // one layer: [page][2][nkv][page_size][hd]
    T* out,                 // [n_tokens, nh * hd]
    const int* block_table, // [n_seqs, bt_stride] logical page -> physical page (or -1)
    int bt_stride,
    const int* seq_of_token,  // [n_tokens]
    const int* positions,     // [n_tokens]
    int n_tokens, int nh, int nkv, int hd, int page_size, int window, float scale, long long n_pages, int* err_flag) {
    extern __shared__ float q_smem[];  // [warps][hd]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)n_tokens * nh) return;  // whole warp leaves together
    const int t = (int)(item / nh), h = (int)(item - (long long)t * nh);
    const int kvh = h / (nh / nkv);
    const int seq = seq_of_token[t];
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (size_t)seq * bt_stride;

    float* qs = q_smem + warp * hd;
    const T* qrow = q + ((size_t)t * nh + h) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    const int n_own = (hd + 31) / 32;  // output dims per lane: d = lane + 32 i
    float acc[8];                      // hd <= 256
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int c = (lo / 32) * 32; c <= pos; c += 32) {
        const int j = c + lane;
        const bool valid = j >= lo && j <= pos;
        float score = -INFINITY;
        int vrow = -1;  // row index of this key's value vector, in units of hd elements
        if (valid) {
            const int page = pyre_checked_page(table[j / page_size], n_pages, err_flag);
            const int off = j % page_size;
            const size_t krow = ((size_t)(page * 2) * nkv + kvh) * page_size + off;
            vrow = (int)(((size_t)(page * 2 + 1) * nkv + kvh) * page_size + off);
            const T* kp = cache + krow * hd;
            // four interleaved chains (dims e, e + 4 of every 8), added as a tree: shorter sums round less
            float dot[4] = {0.f, 0.f, 0.f, 0.f};
            for (int d = 0; d < hd; d += 8) {
                Vec<T, 8> kv = load_vec<T, 8>(kp + d);
#pragma unroll
                for (int e = 0; e < 8; ++e) dot[e & 3] = fmaf(qs[d + e], to_f32<T>(kv.v[e]), dot[e & 3]);
            }
            score = ((dot[0] + dot[1]) + (dot[2] + dot[3])) * scale;
        }
        const float m_new = fmaxf(m, warp_max(score));
        const float p = valid ? expf(score - m_new) : 0.f;
        const float alpha = expf(m - m_new);  // m = -inf at the start: exp(-inf) = 0
        l = l * alpha + warp_sum(p);
        float part[8];  // this chunk's share of the output, summed on its own and then added to the older keys'
#pragma unroll
        for (int i = 0; i < 8; ++i) part[i] = 0.f;
        const int n_keys = min(32, pos - c + 1);
        if constexpr (sizeof(T) == 4) {
            // float32 storage: four keys at a time.  Their value rows are fetched together (one key after the other,
            // the loads were a chain of memory latencies: 2.5 times the time of a decode step's launch), then added
            // in the order of the keys, as below: the same sums, bit for bit.  (With 2-byte values the wider loop is
            // slower; they keep the plain one.)
            for (int j0 = 0; j0 < n_keys; j0 += 4) {
                float pj[4];
                int vr[4];
                float val[4][8];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    pj[u] = __shfl_sync(0xffffffffu, p, (j0 + u) & 31);
                    vr[u] = (j0 + u < n_keys) ? __shfl_sync(0xffffffffu, vrow, (j0 + u) & 31) : -1;   // -1: before the window, or past the chunk's keys
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const T* vp = cache + (size_t)(vr[u] < 0 ? 0 : vr[u]) * hd;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int d = lane + 32 * i;
                        val[u][i] = (vr[u] >= 0 && i < n_own && d < hd) ? to_f32<T>(vp[d]) : 0.f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (vr[u] < 0) continue;  // the same for the whole warp
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int d = lane + 32 * i;
                        if (i < n_own && d < hd) part[i] = fmaf(pj[u], val[u][i], part[i]);
                    }
                }
            }
        } else {
            for (int jj = 0; jj < n_keys; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const int vr = __shfl_sync(0xffffffffu, vrow, jj);
                if (vr < 0) continue;  // before the window: same for the whole warp
                const T* vp = cache + (size_t)vr * hd;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int d = lane + 32 * i;
                    if (i < n_own && d < hd) part[i] = fmaf(pj, to_f32<T>(vp[d]), part[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(acc[i], alpha, part[i]);
        m = m_new;
    }
    const float inv_l = 1.0f / l;
    T* orow = out + ((size_t)t * nh + h) * hd;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (i < n_own && d < hd) orow[d] = from_f32<T>(acc[i] * inv_l);
    }
}

PYRE_API int pyre_paged_attention_generic(const void* q, const void* cache, void* out, const int* block_table,
                                          int bt_stride, const int* seq_of_token, const int* positions,
                                          int n_tokens, int nh, int nkv, int hd, int page_size, int window,
                                          float scale, int dtype, long long n_pages, int* err_flag,
                                          cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 8 || hd > 256 || hd <= 0 || nkv <= 0 || nh % nkv || page_size <= 0) return PYRE_ERR_BAD_ARG;
    const int warps = 4;
    const long long items = (long long)n_tokens * nh;
    const int blocks = (int)ceil_div_ll(items, warps);
    const size_t smem = (size_t)warps * hd * sizeof(float);
    if (dtype == PYRE_F32)
        pyre_launch(paged_attention_generic_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream, 
            (const float*)q, (const float*)cache, (float*)out, block_table, bt_stride, seq_of_token, positions,
            n_tokens, nh, nkv, hd, page_size, window, scale, n_pages, err_flag);
    else if (dtype == PYRE_BF16)
        pyre_launch(paged_attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, block_table, bt_stride,
            seq_of_token, positions, n_tokens, nh, nkv, hd, page_size, window, scale, n_pages, err_flag);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}
