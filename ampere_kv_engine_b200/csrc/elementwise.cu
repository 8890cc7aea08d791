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

namespace akv {

__global__ void smoke_add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                 float* __restrict__ out, int64_t n) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}

int launch_smoke_add(const float* a, const float* b, float* out, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  const int threads = 256;
  smoke_add_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(a, b, out, n);
  return (int)cudaGetLastError();
}

template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ hidden, int64_t hidden_size, int64_t vocab,
                                 int* status) {
  const int64_t token = blockIdx.x;
  int64_t id = ids[token];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) set_status(status, kBadToken);
    id = 0;
  }
  const T* row = table + id * hidden_size;
  float* dst = hidden + token * hidden_size;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) dst[i] = to_float<T>(row[i]);
}

int launch_embedding(const int32_t* ids, const void* table, float* hidden, int64_t num_tokens,
                     int64_t hidden_size, int64_t vocab, int dtype, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int threads = (int)(hidden_size >= 1024 ? 256 : (hidden_size >= 128 ? 128 : 32));
  if (dtype == kBFloat16)
    embedding_kernel<__nv_bfloat16><<<(unsigned)num_tokens, threads, 0, stream>>>(
        ids, (const __nv_bfloat16*)table, hidden, hidden_size, vocab, status);
  else
    embedding_kernel<float><<<(unsigned)num_tokens, threads, 0, stream>>>(
        ids, (const float*)table, hidden, hidden_size, vocab, status);
  return (int)cudaGetLastError();
}

// One block per output row.  Pass 1 adds the delta into the residual stream (whole-batch form) and accumulates
// the sum of squares; pass 2 reads the row back from shared memory and writes the normalised, weighted values.
// The delta is either one tensor in the activation type or `num_parts` float32 partial sums of a split-K product
// ([num_parts, tokens, hidden]) that are added up here.
template <typename T, typename TD>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const TD* __restrict__ delta, int num_parts,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int32_t* __restrict__ rows, int64_t num_tokens,
                                   int64_t hidden_size, float eps, int* status) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];  // hidden_size floats
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
      float add = 0.f;
      for (int s = 0; s < num_parts; ++s) add += to_float<TD>(d[s * part_stride + i]);
      v += add;
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

template <typename T, typename TD>
static int launch_add_rmsnorm_typed(float* hidden, const void* delta, int num_parts, const float* weight, void* out,
                                    const int32_t* rows, int64_t n, int64_t num_tokens, int64_t hidden_size,
                                    float eps, int* status, cudaStream_t stream) {
  const size_t smem = (size_t)hidden_size * sizeof(float);
  int threads = 32;
  while (threads < 512 && threads * 4 < hidden_size) threads *= 2;
  auto kernel = add_rmsnorm_kernel<T, TD>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  kernel<<<(unsigned)n, threads, smem, stream>>>(hidden, (const TD*)delta, num_parts, weight, (T*)out, rows,
                                                 num_tokens, hidden_size, eps, status);
  return (int)cudaGetLastError();
}

int launch_add_rmsnorm(float* hidden, const void* delta, int delta_parts, const float* weight, void* out,
                       const int32_t* rows, int64_t num_rows, int64_t num_tokens, int64_t hidden_size,
                       float eps, int dtype, int* status, cudaStream_t stream) {
  const int64_t n = rows ? num_rows : num_tokens;
  if (n == 0) return 0;
  if ((size_t)hidden_size * sizeof(float) > 200 * 1024) return (int)cudaErrorInvalidValue;  // refused by the caller first
  if (dtype == kBFloat16) {
    if (delta_parts > 0)
      return launch_add_rmsnorm_typed<__nv_bfloat16, float>(hidden, delta, delta_parts, weight, out, rows, n,
                                                            num_tokens, hidden_size, eps, status, stream);
    return launch_add_rmsnorm_typed<__nv_bfloat16, __nv_bfloat16>(hidden, delta, 1, weight, out, rows, n, num_tokens,
                                                                  hidden_size, eps, status, stream);
  }
  return launch_add_rmsnorm_typed<float, float>(hidden, delta, delta_parts > 0 ? delta_parts : 1, weight, out, rows,
                                                n, num_tokens, hidden_size, eps, status, stream);
}

template <typename T, typename TI>
__global__ void silu_mul_kernel(const TI* __restrict__ gate_up, int num_parts, T* __restrict__ out, int64_t inter,
                                int64_t total) {
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t token = idx / inter, i = idx - token * inter;
  const int64_t part_stride = (total / inter) * 2 * inter;
  const TI* row = gate_up + token * 2 * inter;
  float g = 0.f, u = 0.f;
  for (int s = 0; s < num_parts; ++s) {
    g += to_float<TI>(row[s * part_stride + i]);
    u += to_float<TI>(row[s * part_stride + inter + i]);
  }
  // silu(g) = g * sigmoid(g), in float (ampere_kv/runner.py:176)
  out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
}

int launch_silu_mul(const void* gate_up, int parts, void* out, int64_t num_tokens, int64_t inter, int dtype,
                    cudaStream_t stream) {
  const int64_t total = num_tokens * inter;
  if (total == 0) return 0;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (dtype == kBFloat16) {
    if (parts > 0)
      silu_mul_kernel<__nv_bfloat16, float><<<(unsigned)blocks, threads, 0, stream>>>(
          (const float*)gate_up, parts, (__nv_bfloat16*)out, inter, total);
    else
      silu_mul_kernel<__nv_bfloat16, __nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
          (const __nv_bfloat16*)gate_up, 1, (__nv_bfloat16*)out, inter, total);
  } else {
    silu_mul_kernel<float, float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)gate_up,
                                                                            parts > 0 ? parts : 1, (float*)out,
                                                                            inter, total);
  }
  return (int)cudaGetLastError();
}

}  // namespace akv
