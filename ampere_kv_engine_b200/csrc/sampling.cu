// Token choice on the device: greedy argmax (lowest index wins a tie, as torch.argmax does for
// the reference, ampere_kv/runner.py:346 and ampere_kv/scheduler.py:142,189) and temperature
// sampling by inverse CDF of softmax(logits / T) at a uniform number the host derives from
// (seed, request, step).  The reference samples greedily only; temperature is this package's.
//
// One block per row.  Thread t owns the contiguous chunk [t*C, (t+1)*C) of the vocabulary, so
// the cumulative sum has a fixed order: chunk sums in double, an exclusive scan over threads,
// then the owning thread walks its chunk.
#include "common.cuh"
#include "launchers.h"

#include <math_constants.h>

namespace akv {

constexpr int kSampleThreads = 1024;

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int32_t* __restrict__ tokens, int64_t vocab) {
  __shared__ float s_max[32];
  __shared__ int s_arg[32];
  __shared__ double s_sum[kSampleThreads];
  __shared__ int s_winner;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const float* x = logits + row * vocab;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // 1. max and its first index (strided pass: coalesced).  Rows whose length and start allow it are read as
  // float4, four of them in flight per thread: with one float per load the pass was a chain of ~150 dependent
  // round trips to L2 per thread (20 us per step for a handful of rows).
  float best = -CUDART_INF_F;
  int arg = 0x7fffffff;
  auto take = [&](float v, int64_t i) {
    if (v > best || (v == best && (int)i < arg)) { best = v; arg = (int)i; }
  };
  if (vocab % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int64_t quads = vocab / 4;
    int64_t q = tid;
    for (; q + 3 * kSampleThreads < quads; q += 4 * kSampleThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = x4[q + u * kSampleThreads];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = (q + u * kSampleThreads) * 4;
        take(v[u].x, i); take(v[u].y, i + 1); take(v[u].z, i + 2); take(v[u].w, i + 3);
      }
    }
    for (; q < quads; q += kSampleThreads) {
      const float4 v = x4[q];
      take(v.x, q * 4); take(v.y, q * 4 + 1); take(v.z, q * 4 + 2); take(v.w, q * 4 + 3);
    }
  } else {
    for (int64_t i = tid; i < vocab; i += kSampleThreads) take(x[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
  }
  if (lane == 0) { s_max[warp] = best; s_arg[warp] = arg; }
  __syncthreads();
  if (warp == 0) {
    best = s_max[lane];
    arg = s_arg[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (lane == 0) { s_max[0] = best; s_arg[0] = arg; }
  }
  __syncthreads();
  best = s_max[0];
  arg = s_arg[0];
  const float temp = temperature[row];
  if (!(temp > 0.f) || arg == 0x7fffffff) {
    if (tid == 0) tokens[row] = arg == 0x7fffffff ? 0 : arg;
    return;
  }

  // 2. chunk sums of exp((x - max) / T)
  const int64_t chunk = (vocab + kSampleThreads - 1) / kSampleThreads;
  const int64_t begin = tid * chunk, stop = min(vocab, begin + chunk);
  const float inv_t = 1.f / temp;
  double local = 0.0;
  for (int64_t i = begin; i < stop; ++i) local += (double)expf((x[i] - best) * inv_t);
  s_sum[tid] = local;
  __syncthreads();
  // 3. inclusive scan over the 1024 chunk sums (Hillis-Steele, fixed order)
  for (int o = 1; o < kSampleThreads; o <<= 1) {
    const double add = tid >= o ? s_sum[tid - o] : 0.0;
    __syncthreads();
    s_sum[tid] += add;
    __syncthreads();
  }
  const double total = s_sum[kSampleThreads - 1];
  const double target = (double)uniform[row] * total;
  const double before = tid > 0 ? s_sum[tid - 1] : 0.0;
  // 4. the last non-empty chunk whose start is <= target owns the draw
  if (tid == 0) s_winner = -1;
  __syncthreads();
  if (local > 0.0 && before <= target) atomicMax(&s_winner, tid);
  __syncthreads();
  if (tid == s_winner) {
    double run = before;
    int64_t pick = begin;
    for (int64_t i = begin; i < stop; ++i) {
      const double pr = (double)expf((x[i] - best) * inv_t);
      if (pr > 0.0) pick = i;  // last index with mass so far: the answer if rounding overshoots
      run += pr;
      if (run > target) break;
    }
    tokens[row] = (int32_t)pick;
  }
  if (s_winner < 0 && tid == 0) tokens[row] = arg;
}

int launch_sample(const float* logits, const float* temperature, const float* uniform, int32_t* tokens,
                  int64_t num_rows, int64_t vocab, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  if (vocab <= 0 || vocab > 0x7ffffffeLL || num_rows > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(sample_kernel, dim3((unsigned)num_rows), dim3(kSampleThreads), 0, stream, dim3(1, 1, 1),
                           logits, temperature, uniform, tokens, vocab);
}

}  // namespace akv
