// Host launchers of the hand-written kernels.  Plain C++ signatures over raw device
// pointers so that the .cu files compile without any tensor-library header; bindings.cpp
// checks shapes, dtypes, devices and contiguity before it calls these.
//
// `dtype` is akv::DType (0 = float32, 1 = bfloat16) and names the storage type of
// activations / matrices / cache pages; norm weights, rotary tables and logits are float32.
// Every launcher enqueues on `stream` and returns the launch's cudaError_t as int.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace akv {

// Streaming multiprocessors of the current device, asked once per device.  When no device answers (a build box
// without a GPU) the count of the B200 this package is written for stands in.
constexpr int kFallbackSmCount = 148;
int sm_count();

// Runs the package's bounded mbarrier wait on a barrier that nothing completes, `limit` tries (at most a million),
// and reports kWaitTimeout in `status`: a self-test of the path a production kernel takes when a wait gives up.
int launch_wait_selftest(uint32_t limit, int* status, cudaStream_t stream);

int launch_smoke_add(const float* a, const float* b, float* out, int64_t n, cudaStream_t stream);

// hidden[n, :] = float(table[ids[n], :]).  With `sampled` (may be null), an id of -(r + 1) stands for sampled[r]:
// the token the previous step chose in its row r, still on the device.
int launch_embedding(const int32_t* ids, const int32_t* sampled, int64_t num_sampled, const void* table,
                     float* hidden, int64_t num_tokens, int64_t hidden_size, int64_t vocab, int dtype, int* status,
                     cudaStream_t stream);

// hidden += delta (if delta); out = rmsnorm(hidden) * weight.  With `rows` (num_rows entries)
// only those rows are read, hidden is left untouched and out is [num_rows, hidden_size].
// delta_parts > 0: delta is float32 [delta_parts, tokens, hidden], partial sums that are added up.
int launch_add_rmsnorm(float* hidden, const void* delta, int delta_parts, const float* weight, void* out,
                       const int32_t* rows, int64_t num_rows, int64_t num_tokens, int64_t hidden_size,
                       float eps, int dtype, int* status, cudaStream_t stream);

// out[n, i] = silu(gate(n, i)) * up(n, i).  The gate and up columns of gate_up [tokens, 2 inter] alternate in runs
// of `block` columns (block == inter: all gate columns first, the stored form of separate matrices; block == 64:
// the form that lets one 128-row GEMM tile hold both).  parts > 0: gate_up is float32 [parts, tokens, 2 inter]
// partial sums.
int launch_silu_mul(const void* gate_up, int parts, void* out, int64_t num_tokens, int64_t inter, int64_t block,
                    int dtype, cudaStream_t stream);

// Split-K weight-streaming product for few tokens (gemm_tc.cu), x [tokens, k] and w [features, k] bfloat16.
// Either out [tokens, features] (out_dtype: float32 or bfloat16; the splits are added up inside the kernel,
// splits in {1, 2, 4, 8}) or parts [splits, tokens, features] float32 (each split's sum as it is).
bool small_m_gemm_supported(int64_t tokens, int64_t features, int64_t k);
int small_m_gemm_splits(int64_t features, int64_t k);
// What the kernel does with a finished output tile besides storing it.
//   kEpilogueGated: w holds gate and up rows alternating in runs of 64, so that a 128-row tile has both for 64
//   outputs; out is [tokens, features / 2] bfloat16 = silu(gate) * up, with gate and up rounded to bfloat16 first
//   (what the unfused pair, product then launch_silu_mul, computes).
//   kEpilogueQkv: w holds the q, k and v projections of heads of 128 dims, one head per 128-row tile; the tile's
//   values, rounded to bfloat16, then go through what launch_qk_norm_rope_write does (per-head RMSNorm of q and
//   k, rotation of the whole head by position) and land in q_out / the cache pages (GemmQkv); nothing else is
//   stored.
//   kEpilogueResidual: the tile, rounded to bfloat16, is added to the float32 residual stream in place
//   (GemmResidual::hidden [tokens, features]), and the sum of squares of the new values over the tile's 128
//   features goes to ssq [tiles, tokens]: the next product can then apply the RMS norm itself (GemmNormedX).
enum GemmEpilogue : int { kEpiloguePlain = 0, kEpilogueGated = 1, kEpilogueQkv = 2, kEpilogueResidual = 3 };
struct GemmQkv {
  const int32_t* positions;  // [tokens]
  const int32_t* slots;      // [tokens] page * page_size + offset, or -1; null: K and V are not kept
  const float* q_weight;     // [128] or null: no norm
  const float* k_weight;
  const float* inv_freq;     // [64] or null: no rotation
  void* q_out;               // [tokens, num_heads * 128] bfloat16
  void* k_cache;             // [num_pages, num_kv_heads, page_size, 128] bfloat16, or null
  void* v_cache;
  int num_heads, num_kv_heads, page_size;
  int64_t num_pages;
  float eps;
};
struct GemmResidual {
  float* hidden;             // [tokens, features] float32, updated in place
  float* ssq;                // [ceil(features / 128), tokens] float32, written
};
// The token operand made inside the kernel instead of read from x: x[t, k] = hidden[t, k] * inv_rms[t] * weight[k]
// rounded to bfloat16, with inv_rms[t] = rsqrt(sum over tiles of ssq[tile, t] / k + eps): the RMS norm of
// launch_add_rmsnorm applied to a residual stream whose sums of squares a kEpilogueResidual product left behind.
struct GemmNormedX {
  const float* hidden;       // [tokens, k] float32
  const float* ssq;          // [ssq_tiles, tokens]
  const float* weight;       // [k]
  int ssq_tiles;
  float eps;
};
struct GemmFusion {
  int epilogue = kEpiloguePlain;
  GemmQkv qkv = {};
  GemmResidual residual = {};
  bool normed_x = false;     // x is null and normed says how to make it
  GemmNormedX normed = {};
};
int launch_small_m_gemm(const void* x, const void* w, void* out, int out_dtype, float* parts, int64_t tokens,
                        int64_t features, int64_t k, int splits, const GemmFusion* fusion, int* status,
                        cudaStream_t stream);

// A chain of weight-streaming products in one persistent kernel (stream_phases.cu): up to kMaxStreamPhases
// products x W^T for at most 16 bfloat16 tokens, each depending on the one before, with the epilogues of
// launch_small_m_gemm.  The token operand of a phase is a bfloat16 tensor, or the RMS norm of the float32 residual
// stream `hidden` (its sums of squares come from the last residual phase of the launch, or are added up in the kernel
// when there is none).
constexpr int kMaxStreamPhases = 4;
enum StreamX : int { kStreamXTensor = 0, kStreamXNormed = 1 };
struct StreamPhase {
  const void* w;             // [features, k] bfloat16
  int64_t features, k;
  int x_kind;                // StreamX
  const void* x;             // kStreamXTensor: [tokens, k] bfloat16
  const float* norm_weight;  // kStreamXNormed: [k]
  float eps;
  int epilogue;              // GemmEpilogue; kEpilogueResidual adds into `hidden` (features == hidden_size)
  void* out;                 // plain: bfloat16 [tokens, features]; gated: bfloat16 [tokens, features / 2]
  GemmQkv qkv;               // kEpilogueQkv
};
// CTAs the kernel asks for (one per SM, in clusters of four), and the scratch a launch needs: float32 words for
// partial tiles (none: they stay in shared memory) and int32 counters, one per phase, zero at launch.
int stream_phases_grid();
void stream_phases_scratch(const StreamPhase* phases, int num_phases, int64_t* part_floats, int64_t* sync_ints);
// `trace` (null in production): int64 [grid, kMaxStreamPhases, 16] that receives nanosecond stamps of each CTA's
// progress through each phase, for measurements.
int launch_stream_phases(const StreamPhase* phases, int num_phases, int64_t tokens, float* hidden,
                         int64_t hidden_size, float* ssq, float* parts, int* sync, int* status,
                         cudaStream_t stream, unsigned long long* trace = nullptr);

struct QkRopeWriteParams {
  const void* qkv;          // [N, (NH + 2 NKV) * D]; with qkv_parts > 0: float32 [qkv_parts, N, ...] partial sums
  int qkv_parts;
  const int32_t* positions; // [N]
  const int32_t* slots;     // [N] page * page_size + offset, or -1: do not write; may be null
  const float* q_weight;    // [D] or null: no norm
  const float* k_weight;    // [D] or null
  const float* inv_freq;    // [rotary_dim / 2] or null: no rotation
  void* q_out;              // [N, NH * D]
  void* k_out;              // [N, NKV * D] or null
  void* v_out;              // [N, NKV * D] or null
  void* k_cache;            // [num_pages, NKV, page_size, D] or null
  void* v_cache;
  int64_t num_tokens;
  int num_heads, num_kv_heads, head_dim, rotary_dim, page_size;
  int64_t num_pages;
  float eps;
  int dtype;
  int* status;
};
int launch_qk_norm_rope_write(const QkRopeWriteParams& p, cudaStream_t stream);

// Copy k, v [N, NKV * D] into their cache slots.
int launch_kv_write(const void* k, const void* v, const int32_t* slots, void* k_cache, void* v_cache,
                    int64_t num_tokens, int num_kv_heads, int head_dim, int page_size, int64_t num_pages,
                    int dtype, int* status, cudaStream_t stream);

struct PagedAttentionParams {
  const void* q;               // [N, NH * D]
  const void* k_cache;         // [num_pages, NKV, page_size, D]
  const void* v_cache;
  void* out;                   // [N, NH * D]
  const int32_t* block_table;  // [S, table_width]
  const int32_t* cu_q;         // [S + 1] first batch row of each sequence
  const int32_t* ctx_lens;     // [S] keys of each sequence once this step's tokens are in
  const int32_t* tile_seq;     // [tiles] sequence of each query tile
  const int32_t* tile_q0;      // [tiles] first batch row of the tile
  const int32_t* tile_nq;      // [tiles] rows in the tile (<= q_tile)
  float* partials;             // [N * NH, num_splits, D + 2] when num_splits > 1
  int64_t num_tokens;
  int num_tiles, q_tile, num_splits;
  int num_seqs, table_width;
  int num_heads, num_kv_heads, head_dim, page_size;
  int64_t num_pages;
  int window;                  // 0 = all keys
  int kernel;                  // 0 = best kernel that takes the sizes, 1 = the general kernel, 2 = no tcgen05 prompt
                               // kernel, 3 / 4 = the tcgen05 prompt kernel's narrow / wide form whatever the grid
  float scale;
  int dtype;
  int* status;
};
int launch_paged_attention(const PagedAttentionParams& p, cudaStream_t stream);
// The tensor-core kernels (attention_tc.cu): whether they take the problem, and their launch (without the merge).
bool attention_tc_supported(const PagedAttentionParams& p);
int launch_attention_tc(const PagedAttentionParams& p, cudaStream_t stream);
bool attention_tc_merges_in_kernel(const PagedAttentionParams& p);
// The tcgen05 prompt kernel (attention_tcgen05.cu): bfloat16, head size 128, groups of 2, 4 or 8 q-heads.
bool attention_tcgen05_supported(const PagedAttentionParams& p);
int launch_attention_tcgen05(const PagedAttentionParams& p, cudaStream_t stream);

// tokens[r] = argmax(logits[r]) where temperature[r] == 0, else the inverse-CDF draw of
// softmax(logits[r] / temperature[r]) at uniform[r].
// A row is cut into kSampleSlices slices, a block each.  Workspaces: part_max / part_arg / part_sum hold
// num_rows * kSampleSlices entries (written before they are read); tickets holds num_rows counters that must be zero
// when the kernel starts and are zero again when it ends.
constexpr int kSampleSlices = 8;
int launch_sample(const float* logits, const float* temperature, const float* uniform, int32_t* tokens,
                  int64_t num_rows, int64_t vocab, float* part_max, int* part_arg, double* part_sum, int* tickets,
                  cudaStream_t stream);

}  // namespace akv
