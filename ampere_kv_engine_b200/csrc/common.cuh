// Shared device helpers for the sm_100a kernels of this package.
//
// Every kernel is templated on the storage type T of activations / weights / cache
// (float or __nv_bfloat16) and does its arithmetic in float.  No kernel traps, asserts or
// spins without a bound: inputs are validated on the host (bindings.cpp), and a kernel that
// meets an impossible index records a code in a status word and skips the access.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace akv {

enum DType : int { kFloat32 = 0, kBFloat16 = 1 };

// Codes a kernel may leave in the status word (first writer wins; 0 = fine).
enum Status : int {
  kOk = 0,
  kBadPage = 1,      // a block-table entry outside [0, num_pages)
  kBadSlot = 2,      // a cache slot outside the pool
  kBadToken = 3,     // a token id outside the vocabulary
  kBadRow = 4,       // a gathered row outside the batch
  kWaitTimeout = 5,  // a bounded mbarrier wait gave up
};

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load 8 consecutive elements (16-byte aligned for bf16, 32-byte for float) as floats.
template <typename T>
__device__ __forceinline__ void load8(const T* __restrict__ p, float (&out)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* __restrict__ p, float (&out)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // a bf16 is the upper half of a float
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// silu(g) * u = g * sigmoid(g) * u (ampere_kv/runner.py:176).  A float32 result keeps the exact division and
// exponential; a result that is rounded to bfloat16 anyway takes the approximate ones (relative error about 1e-6
// against a rounding step of 4e-3), which is a fifth of the instructions: the activation kernel was bound by
// instruction issue, not by memory.
template <typename T>
__device__ __forceinline__ float silu_mul_value(float g, float u) {
  if constexpr (sizeof(T) == 2) return __fdividef(g, 1.f + __expf(-g)) * u;
  else return g / (1.f + expf(-g)) * u;
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

// Sum over a whole block (any multiple of 32 threads up to 1024); every thread gets the result.
// `scratch` must hold 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // protect scratch from a previous use
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// The one bounded wait of the package: poll an mbarrier (shared-memory address) for the given phase parity at most
// `limit` times.  False when the phase did not complete; the caller then records kWaitTimeout, stops issuing work,
// and leaves the kernel in order.  Every mbarrier wait of the TMA / tcgen05 kernels goes through this loop.
constexpr uint32_t kWaitLimit = 20u * 1000u * 1000u;     // about a second
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar_addr, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Programmatic dependent launch.  A kernel of the step's chain lets the next kernel start while it still runs
// (pdl_launch_dependents, at its top) and waits for the previous kernel's results right before it first touches
// them (pdl_wait).  What a kernel does before pdl_wait must not depend on the previous kernel: set-up, barrier
// initialisation, and, in the weight-streaming GEMM, filling the TMA ring with weights.  Both are no-ops in a
// kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with the programmatic-stream-serialization attribute (and, if cluster_z/cluster_y > 1, a cluster).
// AKV_NO_PDL=1 in the environment launches without it (for comparisons).
bool pdl_enabled();

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chain(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = cluster.x;
    attrs[n].val.clusterDim.y = cluster.y;
    attrs[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  config.attrs = attrs;
  config.numAttrs = n;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

}  // namespace akv
