// Fused per-head QK RMSNorm + rotate-half RoPE + KV page write, and the page write alone.
//
// Replaces, in one pass over the fused projection output: the per-head norms of
// ampere_kv/runner.py:73-75, apply_rope (runner.py:80-98: angle = position * inv_freq in
// float32, both halves share the angle, x*cos + rotate_half(x)*sin) and the page-write
// kernels csrc/paged_decode.cu:90-111 and :500-525 (post-rotation K and un-rotated V go to
// slot (page, offset) of a [page, kv_head, offset, dim] pool).
//
// One warp per (token, head).  Lane l owns the rotation pairs (j, j + D/2) for
// j = l, l + 32, ... so any even head size works.  rotary_dim <= D may rotate only the first
// rotary_dim dims of a head (pairs (j, j + rotary_dim/2)); the rest pass through.
#include "common.cuh"
#include "launchers.h"

namespace akv {

constexpr int kMaxPairsPerLane = 8;  // head_dim <= 512

template <typename T, typename TI>
__global__ void qk_norm_rope_write_kernel(QkRopeWriteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_heads = p.num_heads + 2 * p.num_kv_heads;
  const int head = blockIdx.x * (blockDim.x >> 5) + warp;
  const int64_t token = blockIdx.y + (int64_t)blockIdx.z * 65535;
  if (head >= total_heads || token >= p.num_tokens) return;
  const int D = p.head_dim, half = D / 2;
  const TI* src = (const TI*)p.qkv + (token * total_heads + head) * (int64_t)D;
  const int parts = p.qkv_parts > 0 ? p.qkv_parts : 1;
  const int64_t part_stride = p.num_tokens * (int64_t)total_heads * D;

  // which kind of head, and where its results go
  const bool is_q = head < p.num_heads;
  const bool is_k = !is_q && head < p.num_heads + p.num_kv_heads;
  const int local = is_q ? head : (is_k ? head - p.num_heads : head - p.num_heads - p.num_kv_heads);
  T* dense_out = nullptr;
  if (is_q) dense_out = (T*)p.q_out + (token * p.num_heads + local) * (int64_t)D;
  else if (is_k && p.k_out) dense_out = (T*)p.k_out + (token * p.num_kv_heads + local) * (int64_t)D;
  else if (!is_k && p.v_out) dense_out = (T*)p.v_out + (token * p.num_kv_heads + local) * (int64_t)D;
  T* cache_out = nullptr;
  if (!is_q && p.slots != nullptr && p.k_cache != nullptr) {
    const int64_t slot = p.slots[token];
    if (slot >= 0) {
      if (slot >= p.num_pages * p.page_size) {
        if (lane == 0) set_status(p.status, kBadSlot);
      } else {
        const int64_t page = slot / p.page_size, off = slot % p.page_size;
        T* base = (T*)(is_k ? p.k_cache : p.v_cache);
        cache_out = base + ((page * p.num_kv_heads + local) * p.page_size + off) * (int64_t)D;
      }
    }
  }

  // load the head: lane owns elements j and j + half
  float lo[kMaxPairsPerLane], hi[kMaxPairsPerLane];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kMaxPairsPerLane; ++c) {
    const int j = c * 32 + lane;
    if (j < half) {
      float a = 0.f, b = 0.f;
      for (int s = 0; s < parts; ++s) {      // float32 partial sums of a split-K product are added here
        a += to_float<TI>(src[s * part_stride + j]);
        b += to_float<TI>(src[s * part_stride + j + half]);
      }
      lo[c] = a;
      hi[c] = b;
      ss += lo[c] * lo[c] + hi[c] * hi[c];
    } else {
      lo[c] = hi[c] = 0.f;
    }
  }
  const float* w = is_q ? p.q_weight : (is_k ? p.k_weight : nullptr);
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
    for (int c = 0; c < kMaxPairsPerLane; ++c) {
      const int j = c * 32 + lane;
      if (j < half) {
        lo[c] = lo[c] * inv * w[j];
        hi[c] = hi[c] * inv * w[j + half];
      }
    }
  }
  const bool rotate = !(!is_q && !is_k) && p.inv_freq != nullptr && p.rotary_dim > 0;
  if (rotate && p.rotary_dim == D) {
    const float pos = (float)p.positions[token];
#pragma unroll
    for (int c = 0; c < kMaxPairsPerLane; ++c) {
      const int j = c * 32 + lane;
      if (j < half) {
        const float angle = pos * p.inv_freq[j];
        float s, co;
        sincosf(angle, &s, &co);
        const float a = lo[c], b = hi[c];
        lo[c] = a * co - b * s;  // x*cos + (-x[j+half])*sin
        hi[c] = b * co + a * s;  // x*cos + ( x[j])*sin
      }
    }
  }
  // store (a partial rotary_dim is handled below, after the values are in memory order)
  if (rotate && p.rotary_dim != D) {
    // general case: rotation pairs are (j, j + rotary_dim/2) inside the first rotary_dim dims,
    // which does not match the (j, j + D/2) ownership; go through shared memory per warp.
    extern __shared__ float head_buf[];
    float* buf = head_buf + warp * D;
#pragma unroll
    for (int c = 0; c < kMaxPairsPerLane; ++c) {
      const int j = c * 32 + lane;
      if (j < half) { buf[j] = lo[c]; buf[j + half] = hi[c]; }
    }
    __syncwarp();
    const int rh = p.rotary_dim / 2;
    const float pos = (float)p.positions[token];
    for (int j = lane; j < rh; j += 32) {
      const float angle = pos * p.inv_freq[j];
      float s, co;
      sincosf(angle, &s, &co);
      const float a = buf[j], b = buf[j + rh];
      buf[j] = a * co - b * s;
      buf[j + rh] = b * co + a * s;
    }
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      const T v = from_float<T>(buf[d]);
      if (dense_out) dense_out[d] = v;
      if (cache_out) cache_out[d] = v;
    }
    return;
  }
#pragma unroll
  for (int c = 0; c < kMaxPairsPerLane; ++c) {
    const int j = c * 32 + lane;
    if (j < half) {
      const T a = from_float<T>(lo[c]), b = from_float<T>(hi[c]);
      if (dense_out) { dense_out[j] = a; dense_out[j + half] = b; }
      if (cache_out) { cache_out[j] = a; cache_out[j + half] = b; }
    }
  }
}

// Fast path (head size a multiple of 4, the whole head rotated or none of it, one input tensor): a block of 8 warps
// takes 24 heads of one token, three per warp, whose loads are all issued before the first is used (a warp with
// one head's 256 bytes in flight left the kernel latency-bound: 45 us for 2,048 tokens of 48 heads).  The token's
// cos/sin table is computed once per block in shared memory; every lane owns two adjacent elements of the low
// half and their partners in the high half (4- or 8-byte accesses).
template <typename T>
struct Pair;
template <>
struct Pair<float> {
  static __device__ __forceinline__ void load(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
  }
  static __device__ __forceinline__ void store(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
  }
};
template <>
struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float& a, float& b) {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(raw << 16); b = __uint_as_float(raw & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<uint32_t*>(&v);
  }
};

constexpr int kFastWarps = 8;
constexpr int kHeadsPerWarp = 3;      // loads of three heads are in flight per warp before any is used
constexpr int kMaxUnitsPerLane = 4;   // head_dim <= 512

// UPL: units of 4 elements per lane, 1 for heads up to 128 dims, 2 up to 256, 4 up to 512 (fewer registers, more
// warps per SM).
template <typename T, int UPL>
__global__ void __launch_bounds__(kFastWarps * 32) qk_norm_rope_write_fast_kernel(QkRopeWriteParams p) {
  extern __shared__ float cs[];   // [2][half]: cos, sin of this token's angles
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_heads = p.num_heads + 2 * p.num_kv_heads;
  const int64_t token = blockIdx.y + (int64_t)blockIdx.z * 65535;
  if (token >= p.num_tokens) return;
  const int D = p.head_dim, half = D / 2, units = D / 4;
  const bool rotary = p.inv_freq != nullptr && p.rotary_dim == D;
  // the token's cache slot, once
  int64_t slot = -1;
  if (p.slots != nullptr && p.k_cache != nullptr) {
    slot = p.slots[token];
    if (slot >= p.num_pages * p.page_size) {
      if (threadIdx.x == 0) set_status(p.status, kBadSlot);
      slot = -1;
    }
  }
  const int first_head = (blockIdx.x * kFastWarps + warp) * kHeadsPerWarp;
  float lo[kHeadsPerWarp][UPL][2], hi[kHeadsPerWarp][UPL][2];
  // 1. every load of this warp's heads, before anything waits for one
#pragma unroll
  for (int hh = 0; hh < kHeadsPerWarp; ++hh) {
    const int head = first_head + hh;
    if (head < total_heads) {
      const T* src = (const T*)p.qkv + (token * total_heads + head) * (int64_t)D;
#pragma unroll
      for (int c = 0; c < UPL; ++c) {
        const int u = c * 32 + lane;
        if (u < units) {
          Pair<T>::load(src + 2 * u, lo[hh][c][0], lo[hh][c][1]);
          Pair<T>::load(src + half + 2 * u, hi[hh][c][0], hi[hh][c][1]);
        }
      }
    }
  }
  // the token's cos/sin table, while the loads are under way
  if (rotary) {
    const float pos = (float)p.positions[token];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float sn, co;
      sincosf(pos * p.inv_freq[j], &sn, &co);
      cs[j] = co;
      cs[half + j] = sn;
    }
    __syncthreads();
  }
  // 2. norm, rotation, stores, head by head
#pragma unroll
  for (int hh = 0; hh < kHeadsPerWarp; ++hh) {
    const int head = first_head + hh;
    if (head >= total_heads) break;
    const bool is_q = head < p.num_heads;
    const bool is_k = !is_q && head < p.num_heads + p.num_kv_heads;
    const int local = is_q ? head : (is_k ? head - p.num_heads : head - p.num_heads - p.num_kv_heads);
    T* dense_out = nullptr;
    if (is_q) dense_out = (T*)p.q_out + (token * p.num_heads + local) * (int64_t)D;
    else if (is_k && p.k_out) dense_out = (T*)p.k_out + (token * p.num_kv_heads + local) * (int64_t)D;
    else if (!is_k && p.v_out) dense_out = (T*)p.v_out + (token * p.num_kv_heads + local) * (int64_t)D;
    T* cache_out = nullptr;
    if (!is_q && slot >= 0) {
      const int64_t page = slot / p.page_size, off = slot % p.page_size;
      T* base = (T*)(is_k ? p.k_cache : p.v_cache);
      cache_out = base + ((page * p.num_kv_heads + local) * p.page_size + off) * (int64_t)D;
    }
    const float* w = is_q ? p.q_weight : (is_k ? p.k_weight : nullptr);
    if (w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < UPL; ++c) {
        const int u = c * 32 + lane;
        if (u < units)
          ss += lo[hh][c][0] * lo[hh][c][0] + lo[hh][c][1] * lo[hh][c][1] + hi[hh][c][0] * hi[hh][c][0] +
                hi[hh][c][1] * hi[hh][c][1];
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
      for (int c = 0; c < UPL; ++c) {
        const int u = c * 32 + lane;
        if (u < units) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            lo[hh][c][e] = lo[hh][c][e] * inv * w[2 * u + e];
            hi[hh][c][e] = hi[hh][c][e] * inv * w[half + 2 * u + e];
          }
        }
      }
    }
    if (rotary && (is_q || is_k)) {
#pragma unroll
      for (int c = 0; c < UPL; ++c) {
        const int u = c * 32 + lane;
        if (u < units) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float co = cs[2 * u + e], sn = cs[half + 2 * u + e];
            const float a = lo[hh][c][e], b = hi[hh][c][e];
            lo[hh][c][e] = a * co - b * sn;
            hi[hh][c][e] = b * co + a * sn;
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < UPL; ++c) {
      const int u = c * 32 + lane;
      if (u < units) {
        if (dense_out) {
          Pair<T>::store(dense_out + 2 * u, lo[hh][c][0], lo[hh][c][1]);
          Pair<T>::store(dense_out + half + 2 * u, hi[hh][c][0], hi[hh][c][1]);
        }
        if (cache_out) {
          Pair<T>::store(cache_out + 2 * u, lo[hh][c][0], lo[hh][c][1]);
          Pair<T>::store(cache_out + half + 2 * u, hi[hh][c][0], hi[hh][c][1]);
        }
      }
    }
  }
}

// bfloat16 heads of 64, 128 or 256 dims, rotated whole or not at all, with 16-byte accesses: LPH = D / 16 lanes
// share a head, lane s of them owns dims [8s, 8s + 8) of the low half and their partners in the high half, so a warp
// takes 32 / LPH heads at a time and a block of four warps all heads of one token in a few passes.  The kernel above
// spends about 50 instructions per element on indexing when every lane owns four elements (it was bound by
// instruction issue: 32 us for 2,048 tokens of 48 heads, a tenth of the DRAM bandwidth); here a lane owns 16.
template <int LPH>
__global__ void __launch_bounds__(128) qk_norm_rope_write_vec_kernel(QkRopeWriteParams p) {
  constexpr int D = LPH * 16, half = D / 2, kHeadsPerWarp = 32 / LPH;
  __shared__ float cs[D];   // cos [half], sin [half] of this token's angles
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_heads = p.num_heads + 2 * p.num_kv_heads;
  const int64_t token = blockIdx.x;
  const bool rotary = p.inv_freq != nullptr;
  // A block lives for a few microseconds, most of them waiting: for the token's position, then its angles, then
  // its row.  The row does not depend on the angles: the loads of the first passes over the heads (all of them
  // for up to 64 heads) are issued first and travel while the angle table is made.
  constexpr int kAhead = 4;
  const int sub = lane % LPH, d0 = sub * 8;
  const __nv_bfloat16* row = (const __nv_bfloat16*)p.qkv + token * (int64_t)total_heads * D;
  uint4 ahead_lo[kAhead], ahead_hi[kAhead];
#pragma unroll
  for (int i = 0; i < kAhead; ++i) {
    const int head = (i * 4 + warp) * kHeadsPerWarp + lane / LPH;
    ahead_lo[i] = ahead_hi[i] = make_uint4(0u, 0u, 0u, 0u);
    if (head < total_heads) {
      ahead_lo[i] = *reinterpret_cast<const uint4*>(row + head * D + d0);
      ahead_hi[i] = *reinterpret_cast<const uint4*>(row + head * D + half + d0);
    }
  }
  if (rotary && threadIdx.x < half) {
    float sn, co;
    sincosf((float)p.positions[token] * p.inv_freq[threadIdx.x], &sn, &co);
    cs[threadIdx.x] = co;
    cs[half + threadIdx.x] = sn;
  }
  // the token's cache slot, once, in 32-bit arithmetic (the host checked that the pool's slots fit)
  int page = -1, off = 0;
  if (p.slots != nullptr && p.k_cache != nullptr) {
    const int slot = p.slots[token];
    if (slot >= (int)(p.num_pages * p.page_size)) {
      if (threadIdx.x == 0) set_status(p.status, kBadSlot);
    } else if (slot >= 0) {
      page = slot / p.page_size;
      off = slot - page * p.page_size;
    }
  }
  __syncthreads();
  auto unpack = [](const uint4& raw, float (&out)[8]) {
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(pairs[e]);
      out[2 * e] = f.x;
      out[2 * e + 1] = f.y;
    }
  };
  int pass = 0;
  for (int base = 0; base < total_heads; base += 4 * kHeadsPerWarp, ++pass) {
    const int head = base + warp * kHeadsPerWarp + lane / LPH;
    const bool active = head < total_heads;
    float lo[8], hi[8];
    if (pass < kAhead) {      // fetched above (zeros for a head that does not exist)
      uint4 raw_lo = ahead_lo[0], raw_hi = ahead_hi[0];
#pragma unroll
      for (int i = 1; i < kAhead; ++i)
        if (pass == i) {
          raw_lo = ahead_lo[i];
          raw_hi = ahead_hi[i];
        }
      unpack(raw_lo, lo);
      unpack(raw_hi, hi);
    } else if (active) {
      load8<__nv_bfloat16>(row + head * D + d0, lo);
      load8<__nv_bfloat16>(row + head * D + half + d0, hi);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) lo[e] = hi[e] = 0.f;
    }
    const bool is_q = head < p.num_heads;
    const bool is_k = !is_q && head < p.num_heads + p.num_kv_heads;
    const int local = is_q ? head : (is_k ? head - p.num_heads : head - p.num_heads - p.num_kv_heads);
    const float* w = is_q ? p.q_weight : (is_k ? p.k_weight : nullptr);
    // the sum of squares is taken by all lanes (inactive heads sum zeros), so the shuffles stay warp-wide
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!active) continue;
    if (w != nullptr) {
      const float inv = rsqrtf(ss / (float)D + p.eps);
      float wl[8], wh[8];
      load8<float>(w + d0, wl);
      load8<float>(w + half + d0, wh);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        lo[e] = lo[e] * inv * wl[e];
        hi[e] = hi[e] * inv * wh[e];
      }
    }
    if (rotary && (is_q || is_k)) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float co = cs[d0 + e], sn = cs[half + d0 + e];
        const float a = lo[e], b = hi[e];
        lo[e] = a * co - b * sn;
        hi[e] = b * co + a * sn;
      }
    }
    uint4 out_lo, out_hi;
    {
      __nv_bfloat162 v0 = __floats2bfloat162_rn(lo[0], lo[1]), v1 = __floats2bfloat162_rn(lo[2], lo[3]);
      __nv_bfloat162 v2 = __floats2bfloat162_rn(lo[4], lo[5]), v3 = __floats2bfloat162_rn(lo[6], lo[7]);
      out_lo = make_uint4(*reinterpret_cast<uint32_t*>(&v0), *reinterpret_cast<uint32_t*>(&v1),
                          *reinterpret_cast<uint32_t*>(&v2), *reinterpret_cast<uint32_t*>(&v3));
      v0 = __floats2bfloat162_rn(hi[0], hi[1]); v1 = __floats2bfloat162_rn(hi[2], hi[3]);
      v2 = __floats2bfloat162_rn(hi[4], hi[5]); v3 = __floats2bfloat162_rn(hi[6], hi[7]);
      out_hi = make_uint4(*reinterpret_cast<uint32_t*>(&v0), *reinterpret_cast<uint32_t*>(&v1),
                          *reinterpret_cast<uint32_t*>(&v2), *reinterpret_cast<uint32_t*>(&v3));
    }
    __nv_bfloat16* dense = nullptr;
    if (is_q) dense = (__nv_bfloat16*)p.q_out + (token * p.num_heads + local) * (int64_t)D;
    else if (is_k && p.k_out) dense = (__nv_bfloat16*)p.k_out + (token * p.num_kv_heads + local) * (int64_t)D;
    else if (!is_k && p.v_out) dense = (__nv_bfloat16*)p.v_out + (token * p.num_kv_heads + local) * (int64_t)D;
    if (dense != nullptr) {
      *reinterpret_cast<uint4*>(dense + d0) = out_lo;
      *reinterpret_cast<uint4*>(dense + half + d0) = out_hi;
    }
    if (!is_q && page >= 0) {
      __nv_bfloat16* cache = (__nv_bfloat16*)(is_k ? p.k_cache : p.v_cache) +
                             (((int64_t)page * p.num_kv_heads + local) * p.page_size + off) * D;
      *reinterpret_cast<uint4*>(cache + d0) = out_lo;
      *reinterpret_cast<uint4*>(cache + half + d0) = out_hi;
    }
  }
}

int launch_qk_norm_rope_write(const QkRopeWriteParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.head_dim % 2 || p.head_dim / 2 > 32 * kMaxPairsPerLane) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const int total_heads = p.num_heads + 2 * p.num_kv_heads;
  const int64_t ny = p.num_tokens < 65535 ? p.num_tokens : 65535;
  const int64_t nz = (p.num_tokens + 65534) / 65535;
  if (nz > 65535) return (int)cudaErrorInvalidValue;
  const bool whole_or_none = p.inv_freq == nullptr || p.rotary_dim == p.head_dim || p.rotary_dim == 0;
  const auto aligned16 = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
  if (p.dtype == kBFloat16 && p.qkv_parts == 0 && whole_or_none && p.num_tokens <= 0x7fffffffLL &&
      (p.head_dim == 64 || p.head_dim == 128 || p.head_dim == 256) &&
      p.num_pages * (int64_t)p.page_size <= 0x7fffffffLL && aligned16(p.qkv) && aligned16(p.q_out) &&
      aligned16(p.k_out) && aligned16(p.v_out) && aligned16(p.k_cache) && aligned16(p.v_cache) &&
      aligned16(p.q_weight) && aligned16(p.k_weight)) {
    QkRopeWriteParams q = p;
    if (q.rotary_dim != q.head_dim) q.inv_freq = nullptr;
    const dim3 grid((unsigned)p.num_tokens), block(128), one(1, 1, 1);
    if (p.head_dim == 64) return (int)launch_chain(qk_norm_rope_write_vec_kernel<4>, grid, block, 0, stream, one, q);
    if (p.head_dim == 128) return (int)launch_chain(qk_norm_rope_write_vec_kernel<8>, grid, block, 0, stream, one, q);
    return (int)launch_chain(qk_norm_rope_write_vec_kernel<16>, grid, block, 0, stream, one, q);
  }
  if (p.qkv_parts == 0 && p.head_dim % 4 == 0 && whole_or_none && p.head_dim / 4 <= 32 * kMaxUnitsPerLane) {
    QkRopeWriteParams q = p;
    if (q.rotary_dim != q.head_dim) q.inv_freq = nullptr;
    const int per_block = kFastWarps * kHeadsPerWarp;
    dim3 fast_grid((unsigned)((total_heads + per_block - 1) / per_block), (unsigned)ny, (unsigned)nz);
    const size_t table = q.inv_freq ? (size_t)p.head_dim * sizeof(float) : 0;
    const dim3 block(kFastWarps * 32), one(1, 1, 1);
#define AKV_QK_FAST(T, UPL) \
  return (int)launch_chain(qk_norm_rope_write_fast_kernel<T, UPL>, fast_grid, block, table, stream, one, q)
    if (p.dtype == kBFloat16) {
      if (p.head_dim <= 128) AKV_QK_FAST(__nv_bfloat16, 1);
      if (p.head_dim <= 256) AKV_QK_FAST(__nv_bfloat16, 2);
      AKV_QK_FAST(__nv_bfloat16, 4);
    }
    if (p.head_dim <= 128) AKV_QK_FAST(float, 1);
    if (p.head_dim <= 256) AKV_QK_FAST(float, 2);
    AKV_QK_FAST(float, 4);
#undef AKV_QK_FAST
  }
  dim3 grid((unsigned)((total_heads + warps - 1) / warps), (unsigned)ny, (unsigned)nz);
  const size_t smem = (p.rotary_dim != p.head_dim && p.inv_freq) ? (size_t)warps * p.head_dim * sizeof(float) : 0;
  if (p.dtype == kBFloat16) {
    if (p.qkv_parts > 0)
      qk_norm_rope_write_kernel<__nv_bfloat16, float><<<grid, warps * 32, smem, stream>>>(p);
    else
      qk_norm_rope_write_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, warps * 32, smem, stream>>>(p);
  } else {
    qk_norm_rope_write_kernel<float, float><<<grid, warps * 32, smem, stream>>>(p);
  }
  return (int)cudaGetLastError();
}

template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ k, const T* __restrict__ v,
                                const int32_t* __restrict__ slots, T* __restrict__ k_cache,
                                T* __restrict__ v_cache, int64_t num_tokens, int num_kv_heads, int head_dim,
                                int page_size, int64_t num_pages, int* status) {
  const int64_t token = blockIdx.x;
  const int64_t slot = slots[token];
  if (slot < 0) return;
  if (slot >= num_pages * page_size) {
    if (threadIdx.x == 0) set_status(status, kBadSlot);
    return;
  }
  const int64_t page = slot / page_size, off = slot % page_size;
  const int width = num_kv_heads * head_dim;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int head = i / head_dim, d = i % head_dim;
    const int64_t dst = ((page * num_kv_heads + head) * page_size + off) * (int64_t)head_dim + d;
    k_cache[dst] = k[token * width + i];
    v_cache[dst] = v[token * width + i];
  }
}

int launch_kv_write(const void* k, const void* v, const int32_t* slots, void* k_cache, void* v_cache,
                    int64_t num_tokens, int num_kv_heads, int head_dim, int page_size, int64_t num_pages,
                    int dtype, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int threads = 128;
  if (dtype == kBFloat16)
    kv_write_kernel<__nv_bfloat16><<<(unsigned)num_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, slots, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, num_tokens, num_kv_heads, head_dim, page_size, num_pages, status);
  else
    kv_write_kernel<float><<<(unsigned)num_tokens, threads, 0, stream>>>(
        (const float*)k, (const float*)v, slots, (float*)k_cache, (float*)v_cache, num_tokens, num_kv_heads,
        head_dim, page_size, num_pages, status);
  return (int)cudaGetLastError();
}

}  // namespace akv
