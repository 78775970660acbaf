/* Allocation-free paged attention: one extra C entry point.
 *
 * This entry point has no counterpart in the reference (Lalitaditya-tickoo/pyre has no
 * native code at all); it exists for callers of this library that are not allowed to
 * allocate device memory.
 *
 * Who that is.  pyre_paged_attention_mma() splits long contexts over several CTAs and
 * needs a few megabytes of scratch for the partial results; its caller passes a scratch
 * pointer, which in practice comes from cudaMalloc or from a framework's allocator.  Some
 * callers cannot do that at the point where they call attention: a latency-critical
 * serving loop whose memory budget was fixed at start-up and must never grow or
 * fragment, a plug-in hosted by a runtime that owns all device memory and hands none
 * out, or a thin C or Rust host that links this library without a device allocator of
 * its own.  For them the scratch lives inside the library, in a file-scope
 * `static __device__` array, and the entry point below uses it.
 *
 * What it costs.  The array is PYRE_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on
 * which this library is loaded holds that memory from the load of the module until the
 * process exits, whether or not the entry point is ever called.  The library is separate
 * (libpyre_attention_mma_noalloc.so), so only programs that ask for it pay.
 *
 * Limit.  A call needs n_tokens * nh * n_splits * (hd + 2) floats when n_splits > 1 and
 * none when n_splits == 1.  A call that needs more than the array holds is refused with
 * PYRE_ERR_SCRATCH_TOO_LARGE and nothing is launched; lower n_splits or the batch.
 *
 * Set-up.  The first call on each device looks up the device address of the array
 * (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call
 * outside any stream capture.  The calling thread's current device must be the device
 * that owns the pointers passed in.
 *
 * Sharing.  All calls on one device share the one array, and it keeps what the last call
 * left.  Nothing in it has to be zero: every slot that the combining step reads is
 * written earlier in the same call.  Two calls whose kernels overlap on the GPU (issued on
 * different streams without an ordering between them) race on the array and corrupt
 * each other's results; order them on one stream or with events.
 *
 * Threads.  The table of resolved addresses is filled without a lock.  Two host threads
 * that make their first call on one device at the same time both look the address up and
 * store the same value, which is harmless; no other host state is shared.
 *
 * The entry point calls no cudaMalloc, cudaFree or other allocating routine.
 * Arguments: those of pyre_paged_attention_mma() without `scratch` (built in), and without
 * `max_len`, `n_pages`, `uniform_len` and `err_flag`, which are passed as 0 / null: every
 * entry of the batch is served whatever its length, and, because no page count is given, no
 * tensor map over the pages is built, so keys and values always travel by cp.async copies
 * (the other entry point moves them by TMA when the page size is a power of two and the head
 * size a multiple of 64).  The result is the same bit for bit; long contexts are somewhat
 * slower than through pyre_paged_attention_mma().
 * bfloat16 q [T, nh, hd], one layer of the paged cache [page][2][nkv][page_size][hd],
 * bfloat16 out [T, nh * hd], int32 block_table [n_seqs, bt_stride], cu_seqlens
 * [n_seqs + 1], positions [T].  Returns 0, a cudaError_t value, or a PYRE_ERR_* code.
 */
#pragma once
#include <cuda_runtime.h>

#define PYRE_NOALLOC_SCRATCH_FLOATS (4ll * 1024 * 1024)
#define PYRE_ERR_SCRATCH_TOO_LARGE 100003
#define PYRE_ERR_TOO_MANY_DEVICES 100004

#ifdef __cplusplus
extern "C" {
#endif

int pyre_paged_attention_mma_noalloc(const void* q, const void* cache, void* out, const int* block_table,
                                     int bt_stride, const int* cu_seqlens, const int* positions, int n_tokens,
                                     int n_seqs, int nh, int nkv, int hd, int page_size, int window, float scale,
                                     int n_splits, cudaStream_t stream);

/* Capacity of the built-in scratch in floats (PYRE_NOALLOC_SCRATCH_FLOATS). */
long long pyre_paged_attention_mma_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
