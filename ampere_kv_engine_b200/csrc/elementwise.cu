// Row-wise kernels: embedding gather, fused residual-add + RMSNorm (whole batch or gathered
// rows), SiLU-mul, and the toolchain smoke kernel.
//
// What they replace in the reference: the embedding gather of ampere_kv/runner.py:282, the
// five element-wise/reduce library launches of rms_norm (runner.py:48-57) together with the
// residual sums of runner.py:167 and :179, silu(gate) * up of runner.py:176, and
// csrc/smoke_cuda.cu:11-23.  The residual stream is float32 in both precisions: sums of
// squares, rsqrt, the scale by the weight and the residual sum are 32-bit, one rounding per
// stored tensor.
#include "common.cuh"
#include "launchers.h"

#include <stdlib.h>

namespace akv {

bool pdl_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("AKV_NO_PDL");
    return !(v != nullptr && v[0] != '\0' && v[0] != '0');
  }();
  return enabled;
}

__global__ void smoke_add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                 float* __restrict__ out, int64_t n) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};      // 0: not asked yet (a race writes the same value twice)
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    return kFallbackSmCount;
  }
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) {
      cudaGetLastError();
      return kFallbackSmCount;
    }
    cached[device] = count;
  }
  return cached[device];
}

// Self-test of the bounded wait: one thread initialises an mbarrier that nobody ever arrives on and on which no
// copy is in flight, waits on it through the package's one wait loop with the given limit, finds that the wait ran
// out, reports kWaitTimeout as every production kernel would, and returns.  Nothing hangs and nothing faults.
__global__ void wait_selftest_kernel(uint32_t limit, int* status) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bar);
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(1u));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (!mbar_wait_bounded(addr, 0u, limit)) set_status(status, kWaitTimeout);
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(addr) : "memory");
}

int launch_wait_selftest(uint32_t limit, int* status, cudaStream_t stream) {
  if (limit == 0 || limit > 1000u * 1000u || status == nullptr) return (int)cudaErrorInvalidValue;
  wait_selftest_kernel<<<1, 1, 0, stream>>>(limit, status);
  return (int)cudaGetLastError();
}

int launch_smoke_add(const float* a, const float* b, float* out, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  const int threads = 256;
  smoke_add_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(a, b, out, n);
  return (int)cudaGetLastError();
}

template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ sampled,
                                 int64_t num_sampled, const T* __restrict__ table, float* __restrict__ hidden,
                                 int64_t hidden_size, int64_t vocab, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = blockIdx.x;
  int64_t id = ids[token];
  // -(r + 1): the token that the previous step chose in its row r, which the host has not read yet
  if (id < 0 && sampled != nullptr && -id - 1 < num_sampled) id = sampled[-id - 1];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) set_status(status, kBadToken);
    id = 0;
  }
  const T* row = table + id * hidden_size;
  float* dst = hidden + token * hidden_size;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) dst[i] = to_float<T>(row[i]);
}

int launch_embedding(const int32_t* ids, const int32_t* sampled, int64_t num_sampled, const void* table,
                     float* hidden, int64_t num_tokens, int64_t hidden_size, int64_t vocab, int dtype, int* status,
                     cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int threads = (int)(hidden_size >= 1024 ? 256 : (hidden_size >= 128 ? 128 : 32));
  if (dtype == kBFloat16)
    return (int)launch_chain(embedding_kernel<__nv_bfloat16>, dim3((unsigned)num_tokens), dim3(threads), 0, stream,
                             dim3(1, 1, 1), ids, sampled, num_sampled, (const __nv_bfloat16*)table, hidden, hidden_size,
                             vocab, status);
  return (int)launch_chain(embedding_kernel<float>, dim3((unsigned)num_tokens), dim3(threads), 0, stream,
                           dim3(1, 1, 1), ids, sampled, num_sampled, (const float*)table, hidden, hidden_size, vocab,
                           status);
}

// ---------------------------------------------------------------------------------------------------------
// Residual-add + RMSNorm.  One block per output row.  The row is read once (residual stream float32, delta in the
// activation type or as float32 split-K partial sums), kept in registers (fast path: hidden size a multiple of 4
// and at most 16384) or in shared memory (any size), the sum of squares is reduced over the block, and the
// normalised, weighted row is written.  PARTS > 0 at compile time means "delta is [num_parts, tokens, hidden]
// float32 partial sums"; the common path carries no such loop.
template <typename TD>
__device__ __forceinline__ float read_delta(const TD* d, int64_t i, int num_parts, int64_t part_stride) {
  float add = 0.f;
  for (int s = 0; s < num_parts; ++s) add += to_float<TD>(d[s * part_stride + i]);
  return add;
}

template <typename T, typename TD, bool PARTS>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const TD* __restrict__ delta, int num_parts,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int32_t* __restrict__ rows, int64_t num_tokens,
                                   int64_t hidden_size, float eps, int* status) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];  // hidden_size floats
  pdl_launch_dependents();
  pdl_wait();
  const int64_t out_row = blockIdx.x;
  int64_t src = out_row;
  const bool gathered = rows != nullptr;
  if (gathered) {
    src = rows[out_row];
    if (src < 0 || src >= num_tokens) {
      if (threadIdx.x == 0) set_status(status, kBadRow);
      src = 0;
    }
  }
  float* h = hidden + src * hidden_size;
  const TD* d = delta ? delta + src * hidden_size : nullptr;
  const int64_t part_stride = num_tokens * hidden_size;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    float v = h[i];
    if (d) {
      v += PARTS ? read_delta<TD>(d, i, num_parts, part_stride) : to_float<TD>(d[i]);
      if (!gathered) h[i] = v;
    }
    row_cache[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden_size + eps);
  T* o = out + out_row * hidden_size;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x)
    o[i] = from_float<T>(row_cache[i] * inv * weight[i]);
}

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// Fast path: 4 elements per thread per round, at most ITERS rounds, the row stays in registers.
template <typename T, int ITERS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int32_t* __restrict__ rows, int64_t num_tokens, int hidden_size,
                                       float eps, int* status) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t out_row = blockIdx.x;
  int64_t src = out_row;
  const bool gathered = rows != nullptr;
  if (gathered) {
    src = rows[out_row];
    if (src < 0 || src >= num_tokens) {
      if (threadIdx.x == 0) set_status(status, kBadRow);
      src = 0;
    }
  }
  float* h = hidden + src * hidden_size;
  const T* d = delta ? delta + src * hidden_size : nullptr;
  float v[ITERS][4];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < hidden_size) {
      load4<float>(h + i, v[it]);
      if (d) {
        float dv[4];
        load4<T>(d + i, dv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[it][e] += dv[e];
        if (!gathered) store4<float>(h + i, v[it]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += v[it][e] * v[it][e];
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden_size + eps);
  T* o = out + out_row * hidden_size;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < hidden_size) {
      float w[4], r[4];
      load4<float>(weight + i, w);
#pragma unroll
      for (int e = 0; e < 4; ++e) r[e] = v[it][e] * inv * w[e];
      store4<T>(o + i, r);
    }
  }
}

template <typename T, typename TD, bool PARTS>
static int launch_add_rmsnorm_general(float* hidden, const void* delta, int num_parts, const float* weight, void* out,
                                      const int32_t* rows, int64_t n, int64_t num_tokens, int64_t hidden_size,
                                      float eps, int* status, cudaStream_t stream) {
  const size_t smem = (size_t)hidden_size * sizeof(float);
  int threads = 32;
  while (threads < 512 && threads * 4 < hidden_size) threads *= 2;
  auto kernel = add_rmsnorm_kernel<T, TD, PARTS>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  return (int)launch_chain(kernel, dim3((unsigned)n), dim3(threads), smem, stream, dim3(1, 1, 1), hidden,
                           (const TD*)delta, num_parts, weight, (T*)out, rows, num_tokens, hidden_size, eps, status);
}

template <typename T>
static int launch_add_rmsnorm_fast(float* hidden, const void* delta, const float* weight, void* out,
                                   const int32_t* rows, int64_t n, int64_t num_tokens, int64_t hidden_size,
                                   float eps, int* status, cudaStream_t stream) {
  const int quads = (int)(hidden_size / 4);
  int threads = 32;
  while (threads < 512 && threads * 2 <= quads) threads *= 2;      // two rounds per thread when the row is long
  const int iters = (quads + threads - 1) / threads;
#define AKV_NORM(IT)                                                                                           \
  launch_chain(add_rmsnorm_vec_kernel<T, IT>, dim3((unsigned)n), dim3(threads), 0, stream, dim3(1, 1, 1), hidden, \
               (const T*)delta, weight, (T*)out, rows, num_tokens, (int)hidden_size, eps, status)
  if (iters <= 1) return (int)AKV_NORM(1);
  if (iters <= 2) return (int)AKV_NORM(2);
  if (iters <= 4) return (int)AKV_NORM(4);
  return (int)AKV_NORM(8);
#undef AKV_NORM
}

int launch_add_rmsnorm(float* hidden, const void* delta, int delta_parts, const float* weight, void* out,
                       const int32_t* rows, int64_t num_rows, int64_t num_tokens, int64_t hidden_size,
                       float eps, int dtype, int* status, cudaStream_t stream) {
  const int64_t n = rows ? num_rows : num_tokens;
  if (n == 0) return 0;
  if ((size_t)hidden_size * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;  // refused by the caller first
  const bool aligned = hidden_size % 4 == 0 && hidden_size <= 16384 &&
                       (reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(delta) |
                        reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (delta_parts > 0) {
    if (dtype == kBFloat16)
      return launch_add_rmsnorm_general<__nv_bfloat16, float, true>(hidden, delta, delta_parts, weight, out, rows, n,
                                                                     num_tokens, hidden_size, eps, status, stream);
    return launch_add_rmsnorm_general<float, float, true>(hidden, delta, delta_parts, weight, out, rows, n, num_tokens,
                                                          hidden_size, eps, status, stream);
  }
  if (dtype == kBFloat16) {
    if (aligned)
      return launch_add_rmsnorm_fast<__nv_bfloat16>(hidden, delta, weight, out, rows, n, num_tokens, hidden_size, eps,
                                                    status, stream);
    return launch_add_rmsnorm_general<__nv_bfloat16, __nv_bfloat16, false>(hidden, delta, 1, weight, out, rows, n,
                                                                            num_tokens, hidden_size, eps, status,
                                                                            stream);
  }
  if (aligned)
    return launch_add_rmsnorm_fast<float>(hidden, delta, weight, out, rows, n, num_tokens, hidden_size, eps, status,
                                          stream);
  return launch_add_rmsnorm_general<float, float, false>(hidden, delta, 1, weight, out, rows, n, num_tokens,
                                                         hidden_size, eps, status, stream);
}

// ---------------------------------------------------------------------------------------------------------
// SiLU-mul.  Fast path: 8 elements (bfloat16) or 4 (float32) per thread; general path: one element per thread,
// any size, optional float32 partial sums.
template <typename T, typename TI, bool PARTS>
__global__ void silu_mul_kernel(const TI* __restrict__ gate_up, int num_parts, T* __restrict__ out, int64_t inter,
                                int64_t total, int64_t part_stride, int64_t block) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t token = idx / inter, i = idx - token * inter;
  const TI* row = gate_up + token * 2 * inter;
  // gate and up columns alternate in runs of `block` (block == inter: all gate columns, then all up columns)
  const int64_t gi = i / block * 2 * block + i % block, ui = gi + block;
  float g, u;
  if (PARTS) {
    g = u = 0.f;
    for (int s = 0; s < num_parts; ++s) {
      g += to_float<TI>(row[s * part_stride + gi]);
      u += to_float<TI>(row[s * part_stride + ui]);
    }
  } else {
    g = to_float<TI>(row[gi]);
    u = to_float<TI>(row[ui]);
  }
  out[idx] = from_float<T>(silu_mul_value<T>(g, u));
}

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter_vecs,
                                    int64_t total_vecs, int block) {
  constexpr int V = 16 / sizeof(T);     // elements per 16-byte vector
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= total_vecs) return;
  const int64_t token = idx / inter_vecs;
  const int i = (int)(idx - token * inter_vecs) * V;
  const int64_t inter = (int64_t)inter_vecs * V;
  const T* row = gate_up + token * 2 * inter;
  const int gi = i / block * 2 * block + i % block;     // `block` is a multiple of V
  float g[V], u[V], r[V];
  if constexpr (sizeof(T) == 2) {
    load8<T>(row + gi, g);
    load8<T>(row + gi + block, u);
  } else {
    load4<T>(row + gi, g);
    load4<T>(row + gi + block, u);
  }
#pragma unroll
  for (int e = 0; e < V; ++e) r[e] = silu_mul_value<T>(g[e], u[e]);
  T* o = out + token * inter + i;
  if constexpr (sizeof(T) == 2) {
    float lo[4] = {r[0], r[1], r[2], r[3]}, hi[4] = {r[4], r[5], r[6], r[7]};
    store4<T>(o, lo);
    store4<T>(o + 4, hi);
  } else {
    store4<T>(o, r);
  }
}

int launch_silu_mul(const void* gate_up, int parts, void* out, int64_t num_tokens, int64_t inter, int64_t block,
                    int dtype, cudaStream_t stream) {
  const int64_t total = num_tokens * inter;
  if (total == 0) return 0;
  if (block <= 0 || inter % block != 0) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const int vec = dtype == kBFloat16 ? 8 : 4;
  const bool aligned = parts == 0 && inter % vec == 0 && block % vec == 0 && inter < 0x3fffffffLL &&
                       (reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (aligned) {
    const int64_t total_vecs = total / vec;
    const int64_t blocks = (total_vecs + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    if (dtype == kBFloat16)
      return (int)launch_chain(silu_mul_vec_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                               dim3(1, 1, 1), (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (int)(inter / vec),
                               total_vecs, (int)block);
    return (int)launch_chain(silu_mul_vec_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                             dim3(1, 1, 1), (const float*)gate_up, (float*)out, (int)(inter / vec), total_vecs, (int)block);
  }
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const int64_t part_stride = num_tokens * 2 * inter;
  if (parts > 0) {
    if (dtype == kBFloat16)
      silu_mul_kernel<__nv_bfloat16, float, true><<<(unsigned)blocks, threads, 0, stream>>>(
          (const float*)gate_up, parts, (__nv_bfloat16*)out, inter, total, part_stride, block);
    else
      silu_mul_kernel<float, float, true><<<(unsigned)blocks, threads, 0, stream>>>(
          (const float*)gate_up, parts, (float*)out, inter, total, part_stride, block);
  } else if (dtype == kBFloat16) {
    silu_mul_kernel<__nv_bfloat16, __nv_bfloat16, false><<<(unsigned)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)gate_up, 1, (__nv_bfloat16*)out, inter, total, part_stride, block);
  } else {
    silu_mul_kernel<float, float, false><<<(unsigned)blocks, threads, 0, stream>>>(
        (const float*)gate_up, 1, (float*)out, inter, total, part_stride, block);
  }
  return (int)cudaGetLastError();
}

}  // namespace akv
