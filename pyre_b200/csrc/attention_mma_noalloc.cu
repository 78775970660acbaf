// The allocation-free variant of the tensor-core paged attention; see
// attention_mma_noalloc.h for who needs it, its cost and its rules.
//
// It is the same kernel as pyre_paged_attention_mma (this file includes that
// translation unit, so the code is one), launched with its split-KV scratch pointing into
// a file-scope device array instead of caller-provided memory.
#include "attention_mma.cu"
#include "attention_mma_noalloc.h"

// Scratch of every call of the entry point below on this device.  In host code this name
// is only a handle for the runtime's symbol table, not a device address: the address is
// fetched once per device with cudaGetSymbolAddress and passed to the kernels.
static __device__ __align__(256) float g_noalloc_scratch[PYRE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {};  // per device, filled by the first call on that device
}  // namespace

PYRE_API long long pyre_paged_attention_mma_noalloc_capacity(void) { return PYRE_NOALLOC_SCRATCH_FLOATS; }

PYRE_API int pyre_paged_attention_mma_noalloc(const void* q, const void* cache, void* out, const int* block_table,
                                              int bt_stride, const int* cu_seqlens, const int* positions,
                                              int n_tokens, int n_seqs, int nh, int nkv, int hd, int page_size,
                                              int window, float scale, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_splits < 1 || nh <= 0 || hd <= 0) return PYRE_ERR_BAD_ARG;
    const long long need = pyre_attention_mma_scratch_floats(n_tokens, nh, hd, n_splits);
    if (need > PYRE_NOALLOC_SCRATCH_FLOATS) return PYRE_ERR_SCRATCH_TOO_LARGE;

    float* scratch = nullptr;
    if (need > 0) {
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= MAX_DEVICES) return PYRE_ERR_TOO_MANY_DEVICES;
        if (g_scratch_addr[dev] == nullptr) {
            // first call on this device: resolve the array's device address (not during a capture)
            void* addr = nullptr;
            e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            g_scratch_addr[dev] = static_cast<float*>(addr);
        }
        scratch = g_scratch_addr[dev];
    }
    return pyre_paged_attention_mma(q, cache, out, scratch, block_table, bt_stride, cu_seqlens, positions, n_tokens,
                                    n_seqs, nh, nkv, hd, page_size, window, scale, n_splits, 0, 0, 0, nullptr, stream);
}
