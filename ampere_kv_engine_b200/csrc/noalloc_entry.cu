// akv_paged_attention_noalloc: the general paged attention (key splits + merge) with its partial-result
// workspace in a fixed device array of this library, for callers that must not allocate.  See noalloc_entry.h
// for who needs it, the size limit and the sharing rules.  No counterpart in the reference project.
#include "noalloc_entry.h"

#include <cuda_runtime.h>

#include <mutex>
#include <stdio.h>

#include "launchers.h"

namespace {

// The workspace itself: one copy per GPU that loads the library, alive until the process exits.
static __device__ __align__(256) unsigned char g_scratch[AKV_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};   // device address of g_scratch on each GPU, looked up once
std::mutex g_setup_mutex;
thread_local char g_error[512] = "";

int fail(int code, const char* text) {
  snprintf(g_error, sizeof(g_error), "%s", text);
  return code;
}

// In host code `g_scratch` is only a handle of the symbol, not a device address: the address that kernels can
// use has to be asked for, on the GPU that will run them.
int scratch_for_current_device(float** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(2, cudaGetErrorString(err));
  if (device < 0 || device >= kMaxDevices) return fail(2, "akv_paged_attention_noalloc: device index out of range");
  std::lock_guard<std::mutex> guard(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_scratch);
    if (err != cudaSuccess) {
      snprintf(g_error, sizeof(g_error), "akv_paged_attention_noalloc: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(err));
      return 2;
    }
    g_scratch_address[device] = static_cast<float*>(address);
  }
  *out = g_scratch_address[device];
  return 0;
}

}  // namespace

extern "C" int akv_paged_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           const int32_t* block_table, const int32_t* cu_q,
                                           const int32_t* ctx_lens, const int32_t* tile_seq,
                                           const int32_t* tile_q0, const int32_t* tile_nq, int64_t num_tokens,
                                           int num_tiles, int q_tile, int num_splits, int num_seqs,
                                           int table_width, int num_heads, int num_kv_heads, int head_dim,
                                           int page_size, int64_t num_pages, int window, float scale, int dtype,
                                           int* status, void* stream) {
  g_error[0] = '\0';
  if (!q || !k_cache || !v_cache || !out || !block_table || !cu_q || !ctx_lens || !tile_seq || !tile_q0 || !tile_nq)
    return fail(1, "akv_paged_attention_noalloc: a required pointer is null");
  if (dtype != 0 && dtype != 1) return fail(1, "akv_paged_attention_noalloc: dtype must be 0 (float32) or 1 (bfloat16)");
  if (num_tokens < 0 || num_tiles < 0 || q_tile < 1 || num_splits < 1 || num_seqs < 1 || table_width < 1 ||
      num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads || page_size < 1 || num_pages < 1 || window < 0)
    return fail(1, "akv_paged_attention_noalloc: a size argument is out of range");
  if (head_dim % 16 || head_dim < 16 || head_dim > 256)
    return fail(1, "akv_paged_attention_noalloc: head_dim must be a multiple of 16 up to 256");
  // tokens * heads * splits * (head_dim + 2) floats of partial results must fit in the built-in workspace
  const double need = (double)num_tokens * num_heads * num_splits * (head_dim + 2) * sizeof(float);
  if (need > (double)AKV_NOALLOC_SCRATCH_BYTES) {
    snprintf(g_error, sizeof(g_error),
             "akv_paged_attention_noalloc: the call needs %.0f bytes of workspace (tokens %lld x heads %d x splits %d x "
             "(head_dim %d + 2) floats), the built-in workspace holds %lld; use fewer splits or fewer tokens per call",
             need, (long long)num_tokens, num_heads, num_splits, head_dim, (long long)AKV_NOALLOC_SCRATCH_BYTES);
    return 3;
  }
  float* scratch = nullptr;
  const int setup = scratch_for_current_device(&scratch);
  if (setup != 0) return setup;

  akv::PagedAttentionParams p{};
  p.q = q;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.out = out;
  p.block_table = block_table;
  p.cu_q = cu_q;
  p.ctx_lens = ctx_lens;
  p.tile_seq = tile_seq;
  p.tile_q0 = tile_q0;
  p.tile_nq = tile_nq;
  p.partials = scratch;          // every (row, split) partial is written before the merge reads it
  p.num_tokens = num_tokens;
  p.num_tiles = num_tiles;
  p.q_tile = q_tile;
  p.num_splits = num_splits;
  p.num_seqs = num_seqs;
  p.table_width = table_width;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.head_dim = head_dim;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.window = window;
  p.kernel = 1;                  // the general kernel: its only memory beyond inputs and outputs is `partials`
  p.scale = scale;
  p.dtype = dtype;
  p.status = status;
  const int err = akv::launch_paged_attention(p, static_cast<cudaStream_t>(stream));
  if (err != 0) {
    snprintf(g_error, sizeof(g_error), "akv_paged_attention_noalloc: launch failed: %s",
             cudaGetErrorString(static_cast<cudaError_t>(err)));
    return 4;
  }
  return 0;
}

extern "C" const char* akv_noalloc_last_error(void) { return g_error; }

extern "C" int64_t akv_noalloc_scratch_bytes(void) { return AKV_NOALLOC_SCRATCH_BYTES; }
