// One C entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference project.  It exists for hosts that embed the library under a memory
// regime of their own: a process whose device memory was handed out in full at start-up by its own pool, a
// real-time loop that may not call into the allocator, or a plugin that is only allowed to touch the buffers it is
// given.  Such callers cannot use the ordinary split
// attention path, because that path needs a float32 workspace for the per-split partial results and the Python
// wrapper allocates it on every call.
//
// akv_paged_attention_noalloc runs the general paged attention kernel (key splits + merge) with that workspace
// taken from a fixed array inside the library instead.  The caller passes inputs and outputs exactly as for the
// ordinary entry point; nothing is allocated or freed, by this function or by anything it calls.
//
// Limit.  The workspace is AKV_NOALLOC_SCRATCH_BYTES (16 MiB) per GPU, resident from the moment the library is
// loaded on that GPU until the process ends.  A call needs tokens * heads * splits * (head_dim + 2) floats; a
// call that needs more is refused with an error (nothing is launched).
//
// Sharing.  Every call on a GPU uses the same array.  Its contents after a call are whatever that call left; a
// call never relies on them (each partial is written before it is read, nothing has to start at zero).  Two calls
// whose kernels may run at the same time on one GPU (different streams, different threads) would overwrite each
// other's partials: callers must order them.
//
// First call.  The first call on each GPU looks up the array's device address (cudaGetSymbolAddress, with that
// GPU current) and remembers it.  Make that first call outside any stream capture.
#pragma once

#include <stdint.h>

#define AKV_NOALLOC_SCRATCH_BYTES (16ll * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success.  On failure returns a non-zero code, launches nothing, and akv_noalloc_last_error()
// describes the reason (valid until the calling thread's next call).
//   dtype: 0 = float32, 1 = bfloat16 (type of q, out and the cache pages)
//   stream: a cudaStream_t (0 = the default stream); status: int32[1] device word for bad indices, or null
// All pointers are device pointers on the current device; shapes as in launchers.h (PagedAttentionParams).
int akv_paged_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                const int32_t* block_table, const int32_t* cu_q, const int32_t* ctx_lens,
                                const int32_t* tile_seq, const int32_t* tile_q0, const int32_t* tile_nq,
                                int64_t num_tokens, int num_tiles, int q_tile, int num_splits, int num_seqs,
                                int table_width, int num_heads, int num_kv_heads, int head_dim, int page_size,
                                int64_t num_pages, int window, float scale, int dtype, int* status, void* stream);

const char* akv_noalloc_last_error(void);

// Size of the built-in workspace in bytes (AKV_NOALLOC_SCRATCH_BYTES).
int64_t akv_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
