// Memory-bound kernels of the decoder step: embedding lookup, fused residual-add +
// RMSNorm (with optional row gather), rotary tables, bias + rotary + paged K/V write,
// and SiLU(gate) * up.  All arithmetic is fp32; `dtype` is the type of the
// activations and of the cache (0 = float32, 1 = bfloat16).  The residual stream is
// always float32.
//
// Formulas follow the reference's model code (Lalitaditya-tickoo/pyre):
//   RMSNorm   pyre/model.py:33-38     rotary  pyre/model.py:41-63
//   SwiGLU    pyre/model.py:128-139   embed   pyre/model.py:196
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[t, :] = float(table[ids[t], :]).  An id outside [0, V) gives a zero row
// and raises the error flag (the host checks ids first; this only guards memory).
// ---------------------------------------------------------------------------
template <typename T, int VEC>
__global__ void embedding_kernel(const T* table, const int* ids, float* x,
                                 int H, int V, int* err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* dst = x + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && err) atomicExch(err, 1);
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * H;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        Vec<T, VEC> a = load_vec<T, VEC>(src + i);
        Vec<float, VEC> o;
#pragma unroll
        for (int k = 0; k < VEC; ++k) o.v[k] = to_f32<T>(a.v[k]);
        store_vec<float, VEC>(dst + i, o);
    }
}

PYRE_API int pyre_embedding(const void* table, int dtype, const int* ids, float* x, int n_tokens, int H, int V,
                            int* err_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const bool vec = (H % 4 == 0);
    const int threads = vec ? min(256, max(32, ((H / 4 + 31) / 32) * 32)) : 256;
    if (dtype == PYRE_F32) {
        if (vec) pyre_launch(embedding_kernel<float, 4>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, x, H, V, err_flag);
        else pyre_launch(embedding_kernel<float, 1>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, x, H, V, err_flag);
    } else if (dtype == PYRE_BF16) {
        if (vec) pyre_launch(embedding_kernel<__nv_bfloat16, 4>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, x, H, V, err_flag);
        else pyre_launch(embedding_kernel<__nv_bfloat16, 1>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, x, H, V, err_flag);
    } else {
        return PYRE_ERR_BAD_ARG;
    }
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Fused residual add + RMSNorm.
//   src = rows ? rows[r] : r
//   v   = x[src] + (delta ? delta[src] : 0)          (fp32 sum)
//   if update_x: x[src] = v                           (only without a row gather)
//   out[r] = (v * (1 / sqrt(mean(v^2) + eps))) * w    (the reference's order of products)
// One block per output row; the block size depends on H only, so a row's sum of
// squares is added in the same order whatever the batch holds.
// ---------------------------------------------------------------------------
// delta may come as `n_partials` fp32 partial sums [n_partials][T][H] (a product whose K
// was split over CTAs): they are added in index order, then to x.
template <typename T, int VEC>
__device__ __forceinline__ void load_delta(Vec<float, VEC>& a, const T* dr, const float* pr, int n_partials,
                                           long long partial_stride, int i) {
    if (pr) {
        Vec<float, VEC> acc = load_vec<float, VEC>(pr + i);
        for (int s = 1; s < n_partials; ++s) {
            Vec<float, VEC> q = load_vec<float, VEC>(pr + (size_t)s * partial_stride + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc.v[k] += q.v[k];
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) a.v[k] = a.v[k] + acc.v[k];
    } else {
        Vec<T, VEC> d = load_vec<T, VEC>(dr + i);
#pragma unroll
        for (int k = 0; k < VEC; ++k) a.v[k] = a.v[k] + to_f32<T>(d.v[k]);
    }
}

// KEEP: vectors of the row that a thread keeps in registers between the sum of squares and the scaling (the row is
// then read once; every global round trip counts in a kernel that handles a few rows of a decode step); 0: the row
// is read again for the scaling (any width).
template <typename T, int VEC, int KEEP>
__global__ void add_rmsnorm_kernel(float* x, const T* delta, const float* partials,
                                   int n_partials, long long partial_stride, const float* w,
                                   T* out, const int* rows, int H, float eps, int update_x) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * H;
    const T* dr = delta ? delta + (size_t)src * H : nullptr;
    const float* pr = partials ? partials + (size_t)src * H : nullptr;
    const bool has_delta = dr || pr;
    T* orow = out + (size_t)r * H;

    [[maybe_unused]] Vec<float, VEC> kept[KEEP > 0 ? KEEP : 1];
    float ss = 0.f;
    if constexpr (KEEP > 0) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * VEC;
            if (i < H) {
                Vec<float, VEC> a = load_vec<float, VEC>(xr + i);
                if (has_delta) {
                    load_delta<T, VEC>(a, dr, pr, n_partials, partial_stride, i);
                    if (update_x) store_vec<float, VEC>(xr + i, a);
                }
                kept[j] = a;
#pragma unroll
                for (int k = 0; k < VEC; ++k) ss = fmaf(a.v[k], a.v[k], ss);
            }
        }
    } else {
        for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
            Vec<float, VEC> a = load_vec<float, VEC>(xr + i);
            if (has_delta) {
                load_delta<T, VEC>(a, dr, pr, n_partials, partial_stride, i);
                if (update_x) store_vec<float, VEC>(xr + i, a);
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k) ss = fmaf(a.v[k], a.v[k], ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)H + eps);

    if constexpr (KEEP > 0) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * VEC;
            if (i < H) {
                Vec<float, VEC> g = load_vec<float, VEC>(w + i);
                Vec<T, VEC> o;
#pragma unroll
                for (int k = 0; k < VEC; ++k) o.v[k] = from_f32<T>(__fmul_rn(__fmul_rn(kept[j].v[k], rstd), g.v[k]));
                store_vec<T, VEC>(orow + i, o);
            }
        }
    } else {
        for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
            Vec<float, VEC> a = load_vec<float, VEC>(xr + i);
            if (has_delta && !update_x) load_delta<T, VEC>(a, dr, pr, n_partials, partial_stride, i);
            Vec<float, VEC> g = load_vec<float, VEC>(w + i);
            Vec<T, VEC> o;
#pragma unroll
            for (int k = 0; k < VEC; ++k) o.v[k] = from_f32<T>(__fmul_rn(__fmul_rn(a.v[k], rstd), g.v[k]));
            store_vec<T, VEC>(orow + i, o);
        }
    }
}

// delta: activation dtype [T, H] or null; partials: fp32 [n_partials][T][H] (stride between
// partials in elements) or null; at most one of the two.
PYRE_API int pyre_add_rmsnorm(float* x, const void* delta, const float* partials, int n_partials,
                              long long partial_stride, const float* weight, void* out, const int* rows,
                              int n_rows, int H, float eps, int update_x, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (rows && update_x) return PYRE_ERR_BAD_ARG;  // two output rows could name one source row
    if (delta && partials) return PYRE_ERR_BAD_ARG;
    if (partials && n_partials < 1) return PYRE_ERR_BAD_ARG;
    const bool vec = (H % 4 == 0);
    const int per = vec ? H / 4 : H;
    const int threads = min(512, max(32, ((per + 31) / 32) * 32));
    // a row of up to 4 vectors per thread stays in registers between the two passes (the same sums in the same order)
    const int per_thread = ceil_div(per, threads);
#define LAUNCH_K(TT, V, KP) pyre_launch(add_rmsnorm_kernel<TT, V, KP>, dim3(n_rows), dim3(threads), 0, stream, x, (const TT*)delta, partials, n_partials, partial_stride, weight, (TT*)out, rows, H, eps, update_x)
#define LAUNCH(TT, V) do { if (per_thread <= 2) LAUNCH_K(TT, V, 2); else if (per_thread <= 4) LAUNCH_K(TT, V, 4); else LAUNCH_K(TT, V, 0); } while (0)
    if (dtype == PYRE_F32) { if (vec) LAUNCH(float, 4); else LAUNCH(float, 1); }
    else if (dtype == PYRE_BF16) { if (vec) LAUNCH(__nv_bfloat16, 4); else LAUNCH(__nv_bfloat16, 1); }
    else return PYRE_ERR_BAD_ARG;
#undef LAUNCH
#undef LAUNCH_K
    PYRE_LAUNCH_CHECK();
    return 0;
}

// x[t, :] += delta[t, :] (fp32 sum), for a residual that no norm follows.
template <typename T>
__global__ void add_residual_kernel(float* x, const T* delta, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = x[i] + to_f32<T>(delta[i]);
}

PYRE_API int pyre_add_residual(float* x, const void* delta, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll(n, threads));
    if (dtype == PYRE_F32) pyre_launch(add_residual_kernel<float>, dim3(blocks), dim3(threads), 0, stream, x, (const float*)delta, (size_t)n);
    else if (dtype == PYRE_BF16) pyre_launch(add_residual_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, x, (const __nv_bfloat16*)delta, (size_t)n);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Rotary tables of one step: cos/sin[t, j] of angle = float(position[t]) * inv_freq[j],
// all in fp32 (accurate sincosf; this file is never built with fast-math).  Computed
// once per step and shared by every layer with the same rotary settings.
// ---------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* positions, const float* inv_freq,
                                  float* cos_out, float* sin_out, int n_tokens, int half) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    const int t = i / half, j = i - t * half;
    const float ang = __fmul_rn((float)__ldcg(positions + t), inv_freq[j]);   // positions may come from an earlier kernel: no read-only load
    float s, c;
    sincosf(ang, &s, &c);
    cos_out[i] = c;
    sin_out[i] = s;
}

PYRE_API int pyre_rope_table(const int* positions, const float* inv_freq, float* cos_out, float* sin_out,
                             int n_tokens, int half, cudaStream_t stream) {
    const long long n = (long long)n_tokens * half;
    if (n <= 0) return 0;
    pyre_launch(rope_table_kernel, dim3((int)ceil_div_ll(n, 256)), dim3(256), 0, stream, positions, inv_freq, cos_out, sin_out, n_tokens, half);
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Bias + rotary + paged K/V write.
//   qkv  [T, (nh + 2 nkv) * hd]   product of the fused q/k/v projection, no bias yet
//   bias [(nh + 2 nkv) * hd] fp32 or null
//   q_out[T, nh * hd]             rotated queries
//   cache: one layer of a paged pool, [page][2 (K,V)][nkv][page_size][hd]
//   slot_mapping[t] = page * page_size + offset of token t, or < 0: do not store
//   n_pages, err_flag: the pool's page count and the device's error word, for the debug checks (common.cuh)
// Rotation (half-split pairs over the first `rot` dims of a head, pyre/model.py:54-63):
//   out[j]        = x[j] * cos[j]        - x[j + rot/2] * sin[j]
//   out[j + rot/2] = x[j + rot/2] * cos[j] + x[j]        * sin[j]
// computed in fp32 with separately rounded products, as the reference's fp32 path does.
// Dims at and beyond `rot`, and the whole of v, pass through (plus bias).
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void load_qkv4(float (&v)[4], const T* in, const float* pin, int n_partials,
                                          long long partial_stride, int idx) {
    if (pin) {
        Vec<float, 4> acc = load_vec<float, 4>(pin + idx);
        for (int s = 1; s < n_partials; ++s) {
            Vec<float, 4> q = load_vec<float, 4>(pin + (size_t)s * partial_stride + idx);
#pragma unroll
            for (int k = 0; k < 4; ++k) acc.v[k] += q.v[k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = acc.v[k];
    } else {
        Vec<T, 4> a = load_vec<T, 4>(in + idx);
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = to_f32<T>(a.v[k]);
    }
}

template <typename T>
__global__ void qkv_rope_write_kernel(const T* qkv, const float* partials, int n_partials,
                                      long long partial_stride, const float* bias,
                                      const float* cos_t, const float* sin_t,
                                      T* q_out, T* cache,
                                      const int* slot_mapping, int nh, int nkv, int hd, int rot,
                                      int page_size, long long n_pages, int* err_flag) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;   // one token per blockIdx.x; blockIdx.y strides over its items
    const int half = rot / 2;
    const int chunks = hd / 4;
    const int n_heads_all = nh + 2 * nkv;
    const T* in = qkv ? qkv + (size_t)t * n_heads_all * hd : nullptr;
    const float* pin = partials ? partials + (size_t)t * n_heads_all * hd : nullptr;
    const float* ct = cos_t + (size_t)t * half;
    const float* st = sin_t + (size_t)t * half;
    const int slot = (cache && slot_mapping) ? pyre_checked_slot(slot_mapping[t], n_pages, page_size, err_flag) : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot - page * page_size : 0;

    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_heads_all * chunks; item += gridDim.y * blockDim.x) {
        const int h = item / chunks;
        const int d0 = (item - h * chunks) * 4;
        const bool is_v = h >= nh + nkv;
        const bool is_k = !is_v && h >= nh;
        // destination row of this head
        T* dst;
        if (!is_k && !is_v) {
            dst = q_out + ((size_t)t * nh + h) * hd;
        } else {
            if (slot < 0) continue;
            const int kvh = is_k ? h - nh : h - nh - nkv;
            const size_t row = ((size_t)(page * 2 + (is_v ? 1 : 0)) * nkv + kvh) * page_size + off;
            dst = cache + row * hd;
        }
        const int hoff = h * hd;
        const float* b = bias ? bias + (size_t)h * hd : nullptr;
        if (is_v || d0 >= rot) {
            float a[4];
            load_qkv4<T>(a, in, pin, n_partials, partial_stride, hoff + d0);
            Vec<T, 4> o;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float v = a[k];
                if (b) v = v + b[d0 + k];
                o.v[k] = from_f32<T>(v);
            }
            store_vec<T, 4>(dst + d0, o);
        } else if (d0 < half) {
            float a1[4], a2[4];
            load_qkv4<T>(a1, in, pin, n_partials, partial_stride, hoff + d0);
            load_qkv4<T>(a2, in, pin, n_partials, partial_stride, hoff + d0 + half);
            Vec<T, 4> o1, o2;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float x1 = a1[k];
                float x2 = a2[k];
                if (b) { x1 = x1 + b[d0 + k]; x2 = x2 + b[d0 + half + k]; }
                const float c = ct[d0 + k], s = st[d0 + k];
                o1.v[k] = from_f32<T>(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, s)));
                o2.v[k] = from_f32<T>(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
            }
            store_vec<T, 4>(dst + d0, o1);
            store_vec<T, 4>(dst + d0 + half, o2);
        }  // chunks in [half, rot) are written by their partner
    }
}

// The common case, rotary over the whole head (rot == hd): one item is a pair of VEC-wide chunks (d0, d0 + hd / 2)
// of one head, the two halves that a rotation mixes (for v: two plain chunks), so no thread idles and every access
// is VEC elements wide.  Same arithmetic as the general kernel above.
template <typename T, int VEC>
__device__ __forceinline__ void load_qkv_vec(float (&v)[VEC], const T* in, const float* pin, int n_partials,
                                             long long partial_stride, int idx) {
    if (pin) {
        Vec<float, VEC> acc = load_vec<float, VEC>(pin + idx);
        for (int s = 1; s < n_partials; ++s) {
            Vec<float, VEC> q = load_vec<float, VEC>(pin + (size_t)s * partial_stride + idx);
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc.v[k] += q.v[k];
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = acc.v[k];
    } else {
        Vec<T, VEC> a = load_vec<T, VEC>(in + idx);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = to_f32<T>(a.v[k]);
    }
}

template <typename T, int VEC>
__global__ void qkv_rope_write_full_kernel(const T* qkv, const float* partials, int n_partials,
                                           long long partial_stride, const float* bias,
                                           const float* cos_t, const float* sin_t,
                                           T* q_out, T* cache,
                                           const int* slot_mapping, int nh, int nkv, int hd, int page_size,
                                           long long n_pages, int* err_flag) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = hd / 2;
    const int per_head = half / VEC;
    const int n_heads_all = nh + 2 * nkv;
    const T* in = qkv ? qkv + (size_t)t * n_heads_all * hd : nullptr;
    const float* pin = partials ? partials + (size_t)t * n_heads_all * hd : nullptr;
    const float* ct = cos_t + (size_t)t * half;
    const float* st = sin_t + (size_t)t * half;
    const int slot = (cache && slot_mapping) ? pyre_checked_slot(slot_mapping[t], n_pages, page_size, err_flag) : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? slot - page * page_size : 0;
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_heads_all * per_head; item += gridDim.y * blockDim.x) {
        const int h = item / per_head;
        const int d0 = (item - h * per_head) * VEC;
        const bool is_v = h >= nh + nkv;
        const bool is_k = !is_v && h >= nh;
        T* dst;
        if (!is_k && !is_v) {
            dst = q_out + ((size_t)t * nh + h) * hd;
        } else {
            if (slot < 0) continue;
            const int kvh = is_k ? h - nh : h - nh - nkv;
            dst = cache + (((size_t)(page * 2 + (is_v ? 1 : 0)) * nkv + kvh) * page_size + off) * hd;
        }
        float a1[VEC], a2[VEC];
        load_qkv_vec<T, VEC>(a1, in, pin, n_partials, partial_stride, h * hd + d0);
        load_qkv_vec<T, VEC>(a2, in, pin, n_partials, partial_stride, h * hd + d0 + half);
        // bias, cos and sin come four floats at a time (VEC is 4 or 8 and d0 a multiple of it)
        if (bias) {
            const float* b = bias + (size_t)h * hd;
#pragma unroll
            for (int k4 = 0; k4 < VEC; k4 += 4) {
                const Vec<float, 4> b1 = load_vec<float, 4>(b + d0 + k4), b2 = load_vec<float, 4>(b + d0 + half + k4);
#pragma unroll
                for (int k = 0; k < 4; ++k) { a1[k4 + k] = a1[k4 + k] + b1.v[k]; a2[k4 + k] = a2[k4 + k] + b2.v[k]; }
            }
        }
        Vec<T, VEC> o1, o2;
        if (is_v) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) { o1.v[k] = from_f32<T>(a1[k]); o2.v[k] = from_f32<T>(a2[k]); }
        } else {
#pragma unroll
            for (int k4 = 0; k4 < VEC; k4 += 4) {
                const Vec<float, 4> c4 = load_vec<float, 4>(ct + d0 + k4), s4 = load_vec<float, 4>(st + d0 + k4);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float c = c4.v[k], s_ = s4.v[k];
                    o1.v[k4 + k] = from_f32<T>(__fadd_rn(__fmul_rn(a1[k4 + k], c), __fmul_rn(-a2[k4 + k], s_)));
                    o2.v[k4 + k] = from_f32<T>(__fadd_rn(__fmul_rn(a2[k4 + k], c), __fmul_rn(a1[k4 + k], s_)));
                }
            }
        }
        store_vec<T, VEC>(dst + d0, o1);
        store_vec<T, VEC>(dst + d0 + half, o2);
    }
}

// qkv: activation dtype [T, width] or null; partials: fp32 [n_partials][T][width] or null (one of the two).
PYRE_API int pyre_qkv_rope_write(const void* qkv, const float* partials, int n_partials, long long partial_stride,
                                 const float* bias, const float* cos_t, const float* sin_t,
                                 void* q_out, void* cache, const int* slot_mapping, int n_tokens, int nh, int nkv,
                                 int hd, int rot, int page_size, int dtype, long long n_pages, int* err_flag,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 8 || rot % 8 || rot > hd || rot < 0 || page_size <= 0) return PYRE_ERR_BAD_ARG;
    if ((qkv == nullptr) == (partials == nullptr)) return PYRE_ERR_BAD_ARG;
    if (partials && n_partials < 1) return PYRE_ERR_BAD_ARG;
    // rotary over the whole head and many tokens (a bandwidth-bound pass): the pair kernel, 8 bf16 (4 fp32) per
    // access; few tokens (a latency-bound pass) keep the narrower items of the general kernel: more threads, shorter chains
    const int vec = dtype == PYRE_BF16 ? 8 : 4;
    const bool full = rot == hd && hd % (2 * vec) == 0 && n_tokens >= 256;
    const int items = full ? (nh + 2 * nkv) * (hd / (2 * vec)) : (nh + 2 * nkv) * (hd / 4);
    const int threads = min(128, max(32, ((items + 31) / 32) * 32));
    // few tokens: spread a token's items over several blocks (one item per thread); many tokens:
    // one block per token is plenty of parallelism
    const int by = n_tokens >= 256 ? 1 : min(ceil_div(items, threads), 64);
    if (full && dtype == PYRE_F32)
        pyre_launch(qkv_rope_write_full_kernel<float, 4>, dim3(n_tokens, by), dim3(threads), 0, stream, (const float*)qkv, partials, n_partials, partial_stride, bias, cos_t, sin_t, (float*)q_out, (float*)cache, slot_mapping, nh, nkv, hd, page_size, n_pages, err_flag);
    else if (full && dtype == PYRE_BF16)
        pyre_launch(qkv_rope_write_full_kernel<__nv_bfloat16, 8>, dim3(n_tokens, by), dim3(threads), 0, stream, (const __nv_bfloat16*)qkv, partials, n_partials, partial_stride, bias, cos_t, sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, slot_mapping, nh, nkv, hd, page_size, n_pages, err_flag);
    else if (dtype == PYRE_F32)
        pyre_launch(qkv_rope_write_kernel<float>, dim3(n_tokens, by), dim3(threads), 0, stream, (const float*)qkv, partials, n_partials, partial_stride, bias, cos_t, sin_t, (float*)q_out, (float*)cache, slot_mapping, nh, nkv, hd, rot, page_size, n_pages, err_flag);
    else if (dtype == PYRE_BF16)
        pyre_launch(qkv_rope_write_kernel<__nv_bfloat16>, dim3(n_tokens, by), dim3(threads), 0, stream, (const __nv_bfloat16*)qkv, partials, n_partials, partial_stride, bias, cos_t, sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, slot_mapping, nh, nkv, hd, rot, page_size, n_pages, err_flag);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, I + i],  silu(z) = z / (1 + exp(-z))  in fp32.
// ---------------------------------------------------------------------------
template <typename T, int VEC>
__global__ void silu_mul_kernel(const T* gu, T* out, int n_tokens, int I, int block) {
    pdl_trigger();
    pdl_wait();
    const size_t per_row = (size_t)(I / VEC);
    const size_t total = per_row * n_tokens;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / per_row;
        const int i = (int)(idx - t * per_row) * VEC;
        const T* row = gu + t * (size_t)(2 * I);
        // block == 0: [all gates | all ups]; else gates and ups alternate in blocks of `block` features
        const int gi = block ? (i / block) * 2 * block + i % block : i;
        const int ui = block ? gi + block : I + i;
        Vec<T, VEC> g = load_vec<T, VEC>(row + gi);
        Vec<T, VEC> u = load_vec<T, VEC>(row + ui);
        Vec<T, VEC> o;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float z = to_f32<T>(g.v[k]);
            const float s = z / (1.0f + expf(-z));
            o.v[k] = from_f32<T>(__fmul_rn(s, to_f32<T>(u.v[k])));
        }
        store_vec<T, VEC>(out + t * (size_t)I + i, o);
    }
}

// block: 0 for gate_up = [gates | ups]; n > 0 for gates and ups interleaved in blocks of n features
// (n a multiple of 8 that divides I).
PYRE_API int pyre_silu_mul(const void* gu, void* out, int n_tokens, int I, int block, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || I <= 0) return 0;
    if (block < 0 || (block > 0 && (block % 8 || I % block))) return PYRE_ERR_BAD_ARG;
    const int threads = 256;
#define LAUNCH(TT, V)                                                                                      \
    do {                                                                                                   \
        long long total = (long long)n_tokens * (I / V);                                                   \
        int blocks = (int)min((long long)pyre_sm_count() * 16, ceil_div_ll(total, threads));                           \
        pyre_launch(silu_mul_kernel<TT, V>, dim3(blocks), dim3(threads), 0, stream, (const TT*)gu, (TT*)out, n_tokens, I, block);      \
    } while (0)
    if (dtype == PYRE_F32) { if (I % 4 == 0) LAUNCH(float, 4); else LAUNCH(float, 1); }
    else if (dtype == PYRE_BF16) { if (I % 8 == 0) LAUNCH(__nv_bfloat16, 8); else if (I % 4 == 0) LAUNCH(__nv_bfloat16, 4); else LAUNCH(__nv_bfloat16, 1); }
    else return PYRE_ERR_BAD_ARG;
#undef LAUNCH
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[i] = sum_s partials[s * split_stride + i]: adds up the fp32 partial sums of a
// product whose K was split over CTAs, in a fixed order, and converts.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void sum_partials_kernel(const float* partials, int n_splits, long long split_stride,
                                    T* out, long long n) {
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float acc = partials[i];
        for (int s = 1; s < n_splits; ++s) acc += partials[(long long)s * split_stride + i];
        out[i] = from_f32<T>(acc);
    }
}

PYRE_API int pyre_sum_partials(const float* partials, int n_splits, long long split_stride, void* out, long long n,
                               int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n_splits < 1) return PYRE_ERR_BAD_ARG;
    const int threads = 256;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll(n, threads));
    if (dtype == PYRE_F32) pyre_launch(sum_partials_kernel<float>, dim3(blocks), dim3(threads), 0, stream, partials, n_splits, split_stride, (float*)out, n);
    else if (dtype == PYRE_BF16) pyre_launch(sum_partials_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, partials, n_splits, split_stride, (__nv_bfloat16*)out, n);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// ids[dst[i]] = prev[src[i]] for every i with dst[i] >= 0: the tokens that the last step
// sampled become inputs of the next step without a trip through the host.
// ---------------------------------------------------------------------------
__global__ void feed_tokens_kernel(int* ids, const int* dst, const int* src,
                                   const int* prev, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int d = dst[i];
    if (d >= 0) ids[d] = prev[src[i]];
}

PYRE_API int pyre_feed_tokens(int* ids, const int* dst, const int* src, const int* prev, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    pyre_launch(feed_tokens_kernel, dim3(ceil_div(n, 128)), dim3(128), 0, stream, ids, dst, src, prev, n);
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// A kernel that does nothing for `ns` nanoseconds (at most one second): queued before a measured
// region, it keeps the GPU behind the host, so that every launch of the region is in the stream
// before the GPU reaches it and event timestamps show device time, not the host's launch rate.
// ---------------------------------------------------------------------------
__global__ void delay_kernel(unsigned long long ns) {
    const unsigned long long t0 = pyre_now_ns();
    while (pyre_now_ns() - t0 < ns) __nanosleep(2000);
}

PYRE_API int pyre_delay(long long ns, cudaStream_t stream) {
    if (ns <= 0) return 0;
    if (ns > 1000000000ll) return PYRE_ERR_BAD_ARG;
    delay_kernel<<<1, 1, 0, stream>>>((unsigned long long)ns);
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[t, i] = bf16(float(rows[t, i]) * rstd[t]),  rstd[t] = 1 / sqrt(sum_j ssq[j][t] / H + eps):
// activations that carry a norm's weight but not yet its 1/rms (left so by a product's fix-up, whose
// consumer normally applies the factor in its own epilogue), made plain for any other consumer.
// ---------------------------------------------------------------------------
__global__ void scale_rows_kernel(const __nv_bfloat16* rows, const float* ssq, int n_tiles,
                                  __nv_bfloat16* out, int n_tokens, int H, float eps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    float s = 0.f;
    for (int j = 0; j < n_tiles; ++j) s += ssq[(size_t)j * n_tokens + t];
    const float rstd = 1.0f / sqrtf(s / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)t * H + i] = __float2bfloat16_rn(__bfloat162float(rows[(size_t)t * H + i]) * rstd);
}

PYRE_API int pyre_scale_rows(const void* rows, const float* ssq, int n_tiles, void* out, int n_tokens, int H, float eps,
                             cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0) return 0;
    if (n_tiles < 1) return PYRE_ERR_BAD_ARG;
    pyre_launch(scale_rows_kernel, dim3(n_tokens), dim3(256), 0, stream, (const __nv_bfloat16*)rows, ssq, n_tiles,
                (__nv_bfloat16*)out, n_tokens, H, eps);
    PYRE_LAUNCH_CHECK();
    return 0;
}
