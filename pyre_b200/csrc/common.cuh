// Shared helpers of the sm_100a kernels: element types, conversions, reductions and
// the C calling convention.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and the
// CUDA stream to launch on, allocates nothing and returns 0 or a cudaError_t value
// (the launch error); the Python side turns a non-zero code into an exception.
// Activations and weights are either float (the 32-bit path) or __nv_bfloat16; the
// `dtype` argument says which: 0 = float32, 1 = bfloat16.  All arithmetic is fp32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PYRE_API extern "C" __attribute__((visibility("default")))

enum PyreDType : int { PYRE_F32 = 0, PYRE_BF16 = 1 };

// Error codes of argument checks (outside the cudaError_t range that launches return).
#define PYRE_ERR_BAD_ARG 100001
#define PYRE_ERR_UNSUPPORTED 100002

#define PYRE_LAUNCH_CHECK()                      \
    do {                                         \
        cudaError_t e__ = cudaGetLastError();    \
        if (e__ != cudaSuccess) return (int)e__; \
    } while (0)

template <typename T> struct ElemOps;

template <> struct ElemOps<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};

template <> struct ElemOps<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A vector of N elements of T that is loaded and stored in one transaction.
template <typename T, int N> struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

template <typename T, int N> __device__ __forceinline__ Vec<T, N> load_vec(const T* p) {
    return *reinterpret_cast<const Vec<T, N>*>(p);
}
template <typename T, int N> __device__ __forceinline__ void store_vec(T* p, const Vec<T, N>& x) {
    *reinterpret_cast<Vec<T, N>*>(p) = x;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions is fixed by the thread layout, so a row's result does not depend on
// what else the launch holds.  `scratch` is 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the decoder step is launched with the
// "programmatic stream serialization" attribute: it may be scheduled while the kernel
// before it in the stream is still running, as soon as that kernel's CTAs have called
// pdl_trigger().  Whatever a kernel does before pdl_wait() must not touch memory that an
// earlier kernel of the step writes or still reads (only its own set-up and constant
// weights); pdl_wait() returns when the kernel before it has completed and its writes
// are visible, which, by induction along the stream, holds for all earlier kernels too.
// Without the attribute both calls do nothing.  PYRE_PDL=0 in the environment turns the
// attribute off.
//
// NO READ-ONLY LOADS of anything an earlier kernel writes.  "Visible" holds for ordinary loads.  A load
// through the read-only path (ld.global.nc: what the compiler makes of a `const T* __restrict__`
// parameter, and what __ldg() is) promises that the data does not change while the kernel lives, and under
// this attribute a kernel lives while its predecessors still write: such a load returned stale activations
// (seen in the fp32 tile product of tiny models, where three kernels of a chain sit on one SM at once;
// gone with an ordinary load).  So no kernel parameter in this directory is `__restrict__`, nothing uses
// __ldg(), and tests/test_bindings.py compiles every source to PTX and fails if an ld.global.nc appears
// (the one in sincosf's table of 2/pi apart).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Spin-waits in the kernels (mbarriers of the TMA / tcgen05 pipelines) are bounded by time, not by a
// count of polls: a wait may legitimately last as long as the kernels before it in the stream run (a CTA
// can be resident and polling while its predecessor drains), but never long: a quarter of a second is some
// seventy decode steps of a 7B model.  After PYRE_WAIT_NS the waiter gives up, raises the error word and the
// kernel winds down.
constexpr unsigned long long PYRE_WAIT_NS = 250000000ull;
__device__ __forceinline__ unsigned long long pyre_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
static inline bool pyre_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("PYRE_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t pyre_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pyre_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Per-device host state.  Function attributes (dynamic shared memory, cluster size) and the multiprocessor
// count belong to a device, not to the process: they are kept by the index of the device that is current at
// the call.  Written without a lock: two host threads that race here write the same values.
constexpr int PYRE_MAX_DEVICES = 64;
static inline int pyre_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PYRE_MAX_DEVICES) dev = 0;
    return dev;
}
static inline int pyre_sm_count() {
    static int count[PYRE_MAX_DEVICES] = {};
    const int dev = pyre_current_device();
    if (!count[dev]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        count[dev] = n > 0 ? n : 148;
    }
    return count[dev];
}

// ---------------------------------------------------------------------------
// Debug checks (-DPYRE_DEBUG_CHECKS; PYRE_DEBUG_CHECKS=1 in the environment builds and loads such libraries).
// Every page number that an attention kernel takes from a block table for a key it reads, and every cache slot
// that the K/V write takes from the slot mapping, is checked against the pool: 0 <= page < n_pages (the pages
// that requests own and the scratch page after them; n_pages <= 0 means "not known": only the sign is checked).
// A page number outside (a -1 inside the live range of a sequence, a number beyond the pool) raises the
// device's error word with PYRE_ERRWORD_BAD_PAGE and the access is not made: a read goes to page 0 instead, a
// write is dropped.  The host side refuses such tables before a step starts (the allocator's hard errors,
// pyre/paged_cache.py:62-77 of the reference); this is the device-side net under it.  Off, the helpers are
// the identity and cost nothing.
// ---------------------------------------------------------------------------
constexpr int PYRE_ERRWORD_BAD_PAGE = 6;
#ifdef PYRE_DEBUG_CHECKS
__device__ __forceinline__ int pyre_checked_page(int page, long long n_pages, int* err) {
    if (page < 0 || (n_pages > 0 && page >= n_pages)) {
        if (err) atomicExch(err, PYRE_ERRWORD_BAD_PAGE);
        return 0;
    }
    return page;
}
// slot = page * page_size + offset of a token's keys and values, or < 0 for "store nothing"
__device__ __forceinline__ int pyre_checked_slot(int slot, long long n_pages, int page_size, int* err) {
    if (slot >= 0 && n_pages > 0 && slot >= n_pages * page_size) {
        if (err) atomicExch(err, PYRE_ERRWORD_BAD_PAGE);
        return -1;
    }
    return slot;
}
#else
__device__ __forceinline__ int pyre_checked_page(int page, long long, int*) { return page; }
__device__ __forceinline__ int pyre_checked_slot(int slot, long long, int, int*) { return slot; }
#endif

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }
