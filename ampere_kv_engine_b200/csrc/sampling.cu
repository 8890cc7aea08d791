// Token choice on the device: greedy argmax (lowest index wins a tie, as torch.argmax does for
// the reference, ampere_kv/runner.py:346 and ampere_kv/scheduler.py:142,189) and temperature
// sampling by inverse CDF of softmax(logits / T) at a uniform number the host derives from
// (seed, request, step).  The reference samples greedily only; temperature is this package's.
//
// A row of logits is cut into up to kSampleSlices contiguous slices, one block each, so that a decode step of a
// handful of rows still has dozens of blocks reading (many rows get fewer slices each).  A block finds its
// slice's maximum (and the first index of it) and, for a row that is sampled, the slice's sum of
// exp((x - slice max) / T).  The block that finishes a row last (a
// ticket counter per row, which that block resets for the next launch) combines the slices in slice order: the
// row's maximum, the slice sums rescaled to it, the slice the draw falls into; then it walks that one slice: thread
// t owns the contiguous chunk [t*C, (t+1)*C) of it, chunk sums in double, an inclusive scan over threads, and the
// owning thread walks its chunk.  Every sum has a fixed order, so a draw is reproducible.
#include "common.cuh"
#include "launchers.h"

#include <math_constants.h>

namespace akv {

constexpr int kSampleThreads = 1024;
constexpr int kNoIndex = 0x7fffffff;

// (max, first index of it) over the block; every thread gets the result.
__device__ __forceinline__ void block_argmax(float& best, int& arg, float* s_max, int* s_arg) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
}

// Sum over the block in a fixed order (a shuffle tree per warp, then warp 0 over the warps' sums); every thread
// gets it.  `scratch` holds 33 doubles.
__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double t = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int32_t* __restrict__ tokens, int64_t vocab, int64_t slice_len,
              int slices, float* __restrict__ part_max, int* __restrict__ part_arg,
              double* __restrict__ part_sum, int* __restrict__ tickets) {
  __shared__ float s_max[32];
  __shared__ int s_arg[32];
  __shared__ double s_sum[kSampleThreads];
  __shared__ double s_scratch[33];
  __shared__ int s_flag;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x / slices;
  const int slice = (int)(blockIdx.x - row * slices);
  const float* x = logits + row * vocab;
  const int tid = threadIdx.x;
  const int64_t lo = min(vocab, (int64_t)slice * slice_len), hi = min(vocab, lo + slice_len);
  const float temp = temperature[row];
  const bool drawn = temp > 0.f;
  const float inv_t = drawn ? 1.f / temp : 0.f;

  // 1. the slice's maximum and its first index.  Slices start on multiples of four; where the row does too, the
  // pass reads float4, four loads in flight per thread (one float per load made it a chain of dependent round trips).
  float best = -CUDART_INF_F;
  int arg = kNoIndex;
  auto take = [&](float v, int64_t i) {
    if (v > best || (v == best && (int)i < arg)) { best = v; arg = (int)i; }
  };
  if (vocab % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int64_t q_hi = hi / 4;
    int64_t q = lo / 4 + tid;
    for (; q + 3 * kSampleThreads < q_hi; q += 4 * kSampleThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = x4[q + u * kSampleThreads];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = (q + u * kSampleThreads) * 4;
        take(v[u].x, i); take(v[u].y, i + 1); take(v[u].z, i + 2); take(v[u].w, i + 3);
      }
    }
    for (; q < q_hi; q += kSampleThreads) {
      const float4 v = x4[q];
      take(v.x, q * 4); take(v.y, q * 4 + 1); take(v.z, q * 4 + 2); take(v.w, q * 4 + 3);
    }
  } else {
    for (int64_t i = lo + tid; i < hi; i += kSampleThreads) take(x[i], i);
  }
  block_argmax(best, arg, s_max, s_arg);

  // 2. a drawn row: the slice's sum of exp((x - slice max) / T), strided partial sums in double
  double slice_sum = 0.0;
  if (drawn && arg != kNoIndex) {
    double local = 0.0;
    for (int64_t i = lo + tid; i < hi; i += kSampleThreads) local += (double)expf((x[i] - best) * inv_t);
    slice_sum = block_sum_double(local, s_scratch);
  }
  if (tid == 0) {
    part_max[blockIdx.x] = best;
    part_arg[blockIdx.x] = arg;
    part_sum[blockIdx.x] = slice_sum;
    __threadfence();
    s_flag = atomicAdd(&tickets[row], 1) == slices - 1;
  }
  __syncthreads();
  if (!s_flag) return;

  // 3. the block that finished the row last combines the slices, in slice order
  __threadfence();
  __syncthreads();                     // everyone has read s_flag before it is reused below
  if (tid == 0) tickets[row] = 0;      // for the next launch
  const int64_t first = row * slices;
  float row_max = -CUDART_INF_F;
  int row_arg = kNoIndex;
  for (int s = 0; s < slices; ++s) {
    const float m = __ldcg(part_max + first + s);
    const int a = __ldcg(part_arg + first + s);
    if (a != kNoIndex && (row_arg == kNoIndex || m > row_max)) { row_max = m; row_arg = a; }
  }
  if (!drawn || row_arg == kNoIndex) {
    if (tid == 0) tokens[row] = row_arg == kNoIndex ? 0 : row_arg;
    return;
  }
  double weight[kSampleSlices], total = 0.0;
  for (int s = 0; s < slices; ++s) {
    weight[s] = 0.0;
    if (__ldcg(part_arg + first + s) != kNoIndex)
      weight[s] = __ldcg(part_sum + first + s) * (double)expf((__ldcg(part_max + first + s) - row_max) * inv_t);
    total += weight[s];
  }
  const double target_row = (double)uniform[row] * total;
  // the last slice with mass whose start is <= the target owns the draw
  int owner = -1;
  double before_owner = 0.0, run = 0.0;
  for (int s = 0; s < slices; ++s) {
    if (weight[s] > 0.0 && run <= target_row) { owner = s; before_owner = run; }
    run += weight[s];
  }
  if (owner < 0) {
    if (tid == 0) tokens[row] = row_arg;
    return;
  }
  const double target = target_row - before_owner;      // within the owning slice, in exp((x - row max) / T) units
  const int64_t o_lo = min(vocab, (int64_t)owner * slice_len), o_hi = min(vocab, o_lo + slice_len);
  const int64_t chunk = (o_hi - o_lo + kSampleThreads - 1) / kSampleThreads;
  const int64_t begin = min(o_hi, o_lo + tid * chunk), stop = min(o_hi, begin + chunk);
  double local = 0.0;
  for (int64_t i = begin; i < stop; ++i) local += (double)expf((x[i] - row_max) * inv_t);
  s_sum[tid] = local;
  __syncthreads();
  // inclusive scan over the 1024 chunk sums (Hillis-Steele, fixed order)
  for (int o = 1; o < kSampleThreads; o <<= 1) {
    const double add = tid >= o ? s_sum[tid - o] : 0.0;
    __syncthreads();
    s_sum[tid] += add;
    __syncthreads();
  }
  const double before = tid > 0 ? s_sum[tid - 1] : 0.0;
  // the last non-empty chunk whose start is <= the target owns the draw
  if (tid == 0) s_flag = -1;
  __syncthreads();
  if (local > 0.0 && before <= target) atomicMax(&s_flag, tid);
  __syncthreads();
  if (tid == s_flag) {
    double acc = before;
    int64_t pick = begin;
    for (int64_t i = begin; i < stop; ++i) {
      const double pr = (double)expf((x[i] - row_max) * inv_t);
      if (pr > 0.0) pick = i;  // last index with mass so far: the answer if rounding overshoots
      acc += pr;
      if (acc > target) break;
    }
    tokens[row] = (int32_t)pick;
  }
  if (s_flag < 0 && tid == 0) tokens[row] = row_arg;
}

int launch_sample(const float* logits, const float* temperature, const float* uniform, int32_t* tokens,
                  int64_t num_rows, int64_t vocab, float* part_max, int* part_arg, double* part_sum, int* tickets,
                  cudaStream_t stream) {
  if (num_rows == 0) return 0;
  if (vocab <= 0 || vocab > 0x7ffffffeLL || num_rows * kSampleSlices > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  // as many slices per row as keep a few hundred blocks in flight: 8 for a handful of rows, 1 from 75 rows on
  // (measured at 64 rows: 8 slices 19.9 us, 1 slice 14.2 us for the arg-max; at 8 rows: 5.6 us against 7.4 us)
  int slices = kSampleSlices;
  while (slices > 1 && num_rows * slices > sm_count()) slices /= 2;
  if (part_max == nullptr || part_arg == nullptr || part_sum == nullptr || tickets == nullptr)
    return (int)cudaErrorInvalidValue;
  int64_t slice_len = (vocab + slices - 1) / slices;
  slice_len = (slice_len + 3) / 4 * 4;
  return (int)launch_chain(sample_kernel, dim3((unsigned)(num_rows * slices)), dim3(kSampleThreads), 0, stream,
                           dim3(1, 1, 1), logits, temperature, uniform, tokens, vocab, slice_len, slices, part_max,
                           part_arg, part_sum, tickets);
}

}  // namespace akv
