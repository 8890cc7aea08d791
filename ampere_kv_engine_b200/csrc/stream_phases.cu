// A chain of weight-streaming products for a few tokens in ONE persistent kernel (sm_100a).
//
// A decode step of a few tokens is bound by reading the weights once.  Run as one kernel per product, every product
// pays for its start (barriers, tensor memory, the first copies' latency) and its end (the reduction of K splits,
// the epilogue) with the memory system idle: measured on B200 about 3.5 us per kernel boundary, five boundaries a
// layer.  Here a launch takes a list of up to kMaxPhases products ("phases") that depend on one another in order,
// for instance
//     o-projection (+ residual)  ->  norm + gate/up (+ SiLU-mul)  ->  down (+ residual)  ->  norm + q/k/v of the
//     next layer (+ per-head norm, rotation, cache write)
// and streams ALL their weights through one TMA ring per SM without a pause: the copy warp runs ahead through the
// phases' weight tiles as fast as ring slots free up, whatever the other warps wait for.  The reference has no
// counterpart (its products are library calls, ampere_kv/runner.py:64-66, 165, 174-177).
//
// Work.  One CTA per SM.  A phase is the matrix W [features, k] cut into tiles of 128 features x 64 k ("blocks",
// 16 KB), numbered tile-major.  CTA c of G takes the blocks [c B / G, (c + 1) B / G) of every phase: an equal share
// to within one block whatever the shape.  A run of blocks of one tile within a CTA's share is a "segment": its
// product is accumulated in tensor memory (two accumulators, so the next segment's MMAs run under this one's
// epilogue) and stored as a float32 partial tile; the CTA that stores a tile's last partial (a ticket counter)
// adds the partials up in slot order (the result does not depend on who came last) and applies the phase's
// epilogue.
//
// Warps (320 threads): 0 copies weights (TMA), 1 issues tcgen05.mma, 2-5 make the token operand of each block in
// shared memory (from a bfloat16 tensor, or as the RMS norm of the float32 residual stream), 6-9 are the epilogue.
// A phase's token operand needs the phase before it finished everywhere: the operand warps wait on a counter of
// finished tiles in global memory.  Everything another CTA wrote in this launch is read past the L1 (ld.cg).
//
// No wait is unbounded: mbarrier waits and the counter polls give up after about a second, record kWaitTimeout,
// and the CTA leaves in order (copies in flight awaited, tensor memory freed).  Groups of warps that meet at a named
// barrier decide to give up together (the barrier carries the vote), so nobody is left waiting at it.
#include "common.cuh"
#include "launchers.h"
#include "tensor_map.h"

#include <cuda.h>

namespace akv {

namespace {

constexpr int kTileM = 128;
constexpr int kTileK = 64;
constexpr int kBN = 16;                         // token rows of the MMA (the launch takes up to 16 tokens)
constexpr int kWBytes = kTileM * kTileK * 2;    // 16 KB of weights per block
constexpr int kXBytes = kBN * kTileK * 2;       // 2 KB of tokens per block
constexpr int kStageBytes = kWBytes + kXBytes;
constexpr int kThreads = 320;
constexpr int kXWarps = 4;                      // warps 2..5
constexpr int kFirstXWarp = 2;
constexpr int kFirstEpiWarp = 6;
constexpr uint32_t kPollLimit = 4u * 1000u * 1000u;     // polls of a global counter (with a short sleep each)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  return mbar_wait_bounded(smem_u32(bar), parity, kWaitLimit);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// K-major tile with rows of 128 bytes, 128-byte swizzle, 1024 bytes between groups of 8 rows.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  desc |= (uint64_t)1 << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// float32 accumulator, bfloat16 A and B, both K-major, M = 128, N = kBN.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) |
                            ((uint32_t)(kTileM >> 4) << 24);
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// A named barrier over `count` threads that also ORs a vote: true for everybody if anybody voted true.
__device__ __forceinline__ bool bar_any(int id, int count, bool vote) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %1, 0;\n"
      "barrier.cta.red.or.pred q, %2, %3, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(out)
      : "r"((uint32_t)vote), "r"(id), "r"(count)
      : "memory");
  return out != 0;
}
__device__ __forceinline__ void bar_sync(int id, int count) {
  asm volatile("barrier.cta.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// Loads that go past the L1: data another CTA of this launch wrote.
__device__ __forceinline__ float ld_cg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float4 ld_cg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ uint4 ld_cg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct StreamPhaseDev {
  int features, k;
  int tiles, kb;             // ceil(features / 128), ceil(k / 64)
  int x_kind;                // kStreamXTensor / kStreamXNormed
  int epilogue;              // GemmEpilogue
  int slots;                 // most CTAs that share one tile
  int ctas;                  // CTAs that take blocks of this phase: min(grid, blocks), so that each of them has one
  int ssq_from_hidden;       // normed x without sums of squares left by a residual phase: add them up here
  const __nv_bfloat16* x;    // [tokens, k]
  const float* norm_weight;  // [k]
  float eps;
  void* out;                 // plain: bfloat16 [tokens, features]; gated: bfloat16 [tokens, features / 2]
  int64_t part_offset;       // floats into `parts`
  int sync_offset;           // ints into `sync`: tickets [tiles], then the count of finished tiles
  GemmQkv qkv;
};

struct StreamParamsDev {
  int num_phases, tokens, hidden_size, grid;
  float* hidden;             // [tokens, hidden_size] float32: normed-x source, residual target
  float* ssq;                // [ceil(hidden_size / 128), tokens]
  float* parts;
  int* sync;
  int* status;
  StreamPhaseDev phase[kMaxStreamPhases];
};

struct BlockRange {
  int lo, hi;
};
__device__ __forceinline__ BlockRange cta_range(const StreamPhaseDev& ph, int cta) {
  if (cta >= ph.ctas) return {0, 0};
  const int64_t blocks = (int64_t)ph.tiles * ph.kb;
  return {(int)(blocks * cta / ph.ctas), (int)(blocks * (cta + 1) / ph.ctas)};
}
// The CTA whose share holds block b: the largest c with floor(c B / G) <= b.
__device__ __forceinline__ int cta_of_block(int64_t b, int64_t blocks, int grid) {
  return (int)(((b + 1) * grid - 1) / blocks);
}

template <int kStages>
struct StreamSmem {
  static constexpr int kRing = kStages * kStageBytes;
  // barriers: w_full, x_full, empty per stage; acc_full, acc_empty per accumulator
  static constexpr int kBars = (3 * kStages + 4) * 8;
  static constexpr int kScratch = 16 + 16 * 4 + 16 * 4 * 4 + 2 * kTileM * 4 + 2 * 4 * 4 + 16;
  static constexpr int kBytes = kRing + kBars + kScratch + 1024;
};

template <int kStages>
__global__ void __launch_bounds__(kThreads, 1)
stream_phases_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                     const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3,
                     const __grid_constant__ StreamParamsDev p) {
  static_assert(kStages % kXWarps == 0, "a ring slot is always written by the same operand warp");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* w_full = reinterpret_cast<uint64_t*>(smem + StreamSmem<kStages>::kRing);
  uint64_t* x_full = w_full + kStages;
  uint64_t* empty = x_full + kStages;
  uint64_t* acc_full = empty + kStages;      // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* inv_rms = reinterpret_cast<float*>(tmem_holder + 4);       // [16]
  float* red_tok = inv_rms + 16;                                    // [16][4] per-token warp sums (residual)
  float* xch = red_tok + 64;                                        // [2][128] rotation partners (qkv)
  float* red_it = xch + 2 * kTileM;                                 // [2][4] per-head warp sums (qkv)
  int* flags = reinterpret_cast<int*>(red_it + 8);                  // [0]: ticket broadcast
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const CUtensorMap* maps[kMaxStreamPhases] = {&map0, &map1, &map2, &map3};

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&w_full[s], 1);
      mbar_init(&x_full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);      // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(32u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  bool ok = true;

  if (warp == 0) {
    // ---- weights: run ahead through every phase's share as fast as ring slots free up
    if (lane == 0) {
      int issued = 0;
      for (int ph = 0; ph < p.num_phases && ok; ++ph) {
        const StreamPhaseDev& P = p.phase[ph];
        const BlockRange r = cta_range(P, cta);
        for (int b = r.lo; b < r.hi; ++b, ++issued) {
          const int s = issued % kStages;
          if (issued >= kStages && !mbar_wait(&empty[s], ((issued / kStages) - 1) & 1)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&w_full[s], kWBytes);
          tma_load_2d(smem + s * kStageBytes, maps[ph], (b % P.kb) * kTileK, (b / P.kb) * kTileM, &w_full[s]);
        }
      }
      if (!ok) {
        // copies already issued must land before the CTA's shared memory goes away
        const int first = issued > kStages ? issued - kStages : 0;
        for (int i = first; i < issued; ++i) mbar_wait(&w_full[i % kStages], (i / kStages) & 1);
      }
    }
  } else if (warp == 1) {
    // ---- tensor cores: one thread walks the same blocks and issues the MMAs
    if (lane == 0) {
      int done_blocks = 0, seg = 0;
      for (int ph = 0; ph < p.num_phases && ok; ++ph) {
        const StreamPhaseDev& P = p.phase[ph];
        const BlockRange r = cta_range(P, cta);
        int b = r.lo;
        while (b < r.hi && ok) {
          const int tile = b / P.kb;
          const int seg_end = min(r.hi, (tile + 1) * P.kb);
          const int buf = seg & 1;
          if (seg >= 2 && !mbar_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t acc = tmem_base + (uint32_t)(buf * kBN);
          for (int first = 1; b < seg_end; ++b, ++done_blocks, first = 0) {
            const int s = done_blocks % kStages;
            const uint32_t parity = (done_blocks / kStages) & 1;
            if (!mbar_wait(&w_full[s], parity) || !mbar_wait(&x_full[s], parity)) {
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
            const uint32_t b_addr = a_addr + kWBytes;
#pragma unroll
            for (int k = 0; k < kTileK / 16; ++k)
              umma_bf16(acc, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), (first && k == 0) ? 0u : 1u);
            umma_commit(&empty[s]);
          }
          if (ok) umma_commit(&acc_full[buf]);
          ++seg;
        }
      }
    }
  } else if (warp < kFirstEpiWarp) {
    // ---- token operand: warp xw makes the blocks xw, xw + 4, ... of this CTA's walk
    const int xw = warp - kFirstXWarp;
    pdl_wait();       // the first phase's tokens and the residual stream come from the kernels before this one
    int walked = 0;   // blocks of earlier phases
    for (int ph = 0; ph < p.num_phases; ++ph) {
      const StreamPhaseDev& P = p.phase[ph];
      const BlockRange r = cta_range(P, cta);
      const int count = r.hi - r.lo;
      bool fail = !ok;
      if (ph > 0 && count > 0) {
        // the phase before must have finished everywhere
        const StreamPhaseDev& Q = p.phase[ph - 1];
        const int* finished = p.sync + Q.sync_offset + Q.tiles;
        if (lane == 0) {
          uint32_t tries = 0;
          while (ld_acquire(finished) < Q.tiles) {
            if (++tries > kPollLimit) {
              fail = true;
              break;
            }
            __nanosleep(64);
          }
        }
        fail = __shfl_sync(0xffffffffu, (int)fail, 0) != 0;
        __threadfence();
      }
      if (P.x_kind == kStreamXNormed && count > 0) {
        // 1 / rms of every token's row of the residual stream
        if (!fail) {
          for (int t = xw; t < p.tokens; t += kXWarps) {
            float ss = 0.f;
            if (P.ssq_from_hidden) {
              const float* row = p.hidden + (int64_t)t * P.k;
              for (int i = lane * 4; i < P.k; i += 128) {
                const float4 v = ld_cg4(row + i);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
              }
            } else {
              const int ssq_tiles = (P.k + kTileM - 1) / kTileM;
              for (int i = lane; i < ssq_tiles; i += 32) ss += ld_cg(p.ssq + (int64_t)i * p.tokens + t);
            }
            ss = warp_sum(ss);
            if (lane == 0) inv_rms[t] = rsqrtf(ss / (float)P.k + P.eps);
          }
        }
        fail = bar_any(2, kXWarps * 32, fail);
      } else if (ph > 0 && count > 0) {
        fail = bar_any(2, kXWarps * 32, fail);
      }
      if (fail) {
        ok = false;
        break;
      }
      for (int i = 0; i < count; ++i) {
        const int g = walked + i;                       // index in the CTA's whole walk
        if (g % kXWarps != xw) continue;
        const int s = g % kStages;
        if (g >= kStages && !mbar_wait(&empty[s], ((g / kStages) - 1) & 1)) {
          ok = false;
          break;
        }
        const int b = r.lo + i;
        const int k_base = (b % P.kb) * kTileK;
        uint8_t* x_tile = smem + s * kStageBytes + kWBytes;
        for (int task = lane; task < kBN * 8; task += 32) {
          const int row = task >> 3, c = task & 7;
          const int k0 = k_base + c * 8;
          uint4 packed = make_uint4(0u, 0u, 0u, 0u);    // rows past the tokens and columns past K: zeros
          if (row < p.tokens && k0 < P.k) {
            if (P.x_kind == kStreamXNormed) {
              const float* src = p.hidden + (int64_t)row * P.k + k0;
              const float4 h0 = ld_cg4(src), h1 = ld_cg4(src + 4);
              const float4 w0 = *reinterpret_cast<const float4*>(P.norm_weight + k0);
              const float4 w1 = *reinterpret_cast<const float4*>(P.norm_weight + k0 + 4);
              const float inv = inv_rms[row];
              __nv_bfloat162 v0 = __floats2bfloat162_rn(h0.x * inv * w0.x, h0.y * inv * w0.y);
              __nv_bfloat162 v1 = __floats2bfloat162_rn(h0.z * inv * w0.z, h0.w * inv * w0.w);
              __nv_bfloat162 v2 = __floats2bfloat162_rn(h1.x * inv * w1.x, h1.y * inv * w1.y);
              __nv_bfloat162 v3 = __floats2bfloat162_rn(h1.z * inv * w1.z, h1.w * inv * w1.w);
              packed = make_uint4(*reinterpret_cast<uint32_t*>(&v0), *reinterpret_cast<uint32_t*>(&v1),
                                  *reinterpret_cast<uint32_t*>(&v2), *reinterpret_cast<uint32_t*>(&v3));
            } else {
              packed = ld_cg16(P.x + (int64_t)row * P.k + k0);
            }
          }
          *reinterpret_cast<uint4*>(x_tile + row * 128 + ((c ^ (row & 7)) << 4)) = packed;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the tensor core reads through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&x_full[s]);
      }
      if (!ok) break;
      walked += count;
    }
  } else {
    // ---- epilogue: every segment's partial tile, and the tiles this CTA completes
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    pdl_wait();       // the epilogues write what earlier kernels may still read
    int seg = 0;
    for (int ph = 0; ph < p.num_phases && ok; ++ph) {
      const StreamPhaseDev& P = p.phase[ph];
      const BlockRange r = cta_range(P, cta);
      const int64_t blocks = (int64_t)P.tiles * P.kb;
      int* tickets = p.sync + P.sync_offset;
      int b = r.lo;
      while (b < r.hi) {
        const int tile = b / P.kb;
        const int seg_end = min(r.hi, (tile + 1) * P.kb);
        const int buf = seg & 1;
        bool fail = !mbar_wait(&acc_full[buf], (seg >> 1) & 1);
        fail = bar_any(1, 128, fail);
        if (fail) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t v[16];
        tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kBN), v);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        // who shares this tile: the CTAs from the one that holds its first block to the one that holds its last
        const int first_cta = cta_of_block((int64_t)tile * P.kb, blocks, P.ctas);
        const int last_cta = cta_of_block((int64_t)(tile + 1) * P.kb - 1, blocks, P.ctas);
        const int sharers = last_cta - first_cta + 1;
        float* tile_parts = p.parts + P.part_offset + (int64_t)tile * P.slots * (kBN * kTileM);
        float* mine = tile_parts + (int64_t)(cta - first_cta) * (kBN * kTileM);
        if (sharers > 1) {
#pragma unroll
          for (int t = 0; t < kBN; ++t)
            if (t < p.tokens) mine[t * kTileM + row] = __uint_as_float(v[t]);
          __threadfence();
          bar_sync(1, 128);
          if (threadIdx.x == kFirstEpiWarp * 32) flags[0] = atomicAdd(&tickets[tile], 1);
          bar_sync(1, 128);
        }
        const bool last = sharers == 1 || flags[0] == sharers - 1;
        if (last) {
          // the tile is whole: add the partials up in slot order and apply the phase's epilogue
          __threadfence();
          float sum[kBN];
#pragma unroll
          for (int t = 0; t < kBN; ++t) sum[t] = 0.f;
          if (sharers == 1) {
#pragma unroll
            for (int t = 0; t < kBN; ++t) sum[t] = __uint_as_float(v[t]);
          } else if (P.epilogue != kEpilogueGated) {
            for (int s = 0; s < sharers; ++s) {
              const float* part = tile_parts + (int64_t)s * (kBN * kTileM);
#pragma unroll
              for (int t = 0; t < kBN; ++t)
                if (t < p.tokens) sum[t] += ld_cg(part + t * kTileM + row);
            }
          }
          if (P.epilogue == kEpilogueResidual) {
            const int feature = tile * kTileM + row;
#pragma unroll
            for (int t = 0; t < kBN; ++t) {
              if (t >= p.tokens) break;
              float h = 0.f;
              if (feature < P.features) {
                float* cell = p.hidden + (int64_t)t * P.features + feature;
                h = ld_cg(cell) + __bfloat162float(__float2bfloat16_rn(sum[t]));
                *cell = h;
              }
              const float ss = warp_sum(h * h);
              if (lane == 0) red_tok[t * 4 + quarter] = ss;
            }
            bar_sync(1, 128);
            if (row < p.tokens)
              p.ssq[(int64_t)tile * p.tokens + row] =
                  red_tok[row * 4] + red_tok[row * 4 + 1] + red_tok[row * 4 + 2] + red_tok[row * 4 + 3];
          } else if (P.epilogue == kEpilogueGated) {
            // rows 0-63 are gate rows, rows 64-127 the up rows of the same 64 outputs.  A thread takes output j of
            // every other token and needs both of its rows: through shared memory when the tile is this CTA's
            // alone, else from the partials.
            const int j = row & 63, half = row >> 6;
            const int out_features = P.features / 2;
            const int feature = tile * (kTileM / 2) + j;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(P.out);
            if (sharers == 1) {
              // stage the tile [token][row] in the partial slot of its own (an L2 round trip, a few hundred bytes)
#pragma unroll
              for (int t = 0; t < kBN; ++t)
                if (t < p.tokens) mine[t * kTileM + row] = sum[t];
              __threadfence();
              bar_sync(1, 128);
            }
            for (int t = half; t < p.tokens; t += 2) {
              float g = 0.f, u = 0.f;
              for (int s = 0; s < sharers; ++s) {
                const float* part = tile_parts + (int64_t)s * (kBN * kTileM) + t * kTileM;
                g += ld_cg(part + j);
                u += ld_cg(part + j + 64);
              }
              g = __bfloat162float(__float2bfloat16_rn(g));
              u = __bfloat162float(__float2bfloat16_rn(u));
              if (feature < out_features)
                out[(int64_t)t * out_features + feature] = __float2bfloat16_rn(silu_mul_value<__nv_bfloat16>(g, u));
            }
          } else if (P.epilogue == kEpilogueQkv) {
            // the tile is one head of 128 dims; a thread owns dim `row` of it
            const GemmQkv& e = P.qkv;
            const int head = tile;
            const bool is_q = head < e.num_heads, is_k = !is_q && head < e.num_heads + e.num_kv_heads;
            const int local = is_q ? head : (is_k ? head - e.num_heads : head - e.num_heads - e.num_kv_heads);
            const float* nw = is_q ? e.q_weight : (is_k ? e.k_weight : nullptr);
            const bool normed = nw != nullptr;
            const bool rotate = (is_q || is_k) && e.inv_freq != nullptr;
            const float wd = normed ? nw[row] : 1.f;
            const float freq = rotate ? e.inv_freq[row & 63] : 0.f;
#pragma unroll
            for (int t = 0; t < kBN; ++t) {
              if (t >= p.tokens) break;
              float val = __bfloat162float(__float2bfloat16_rn(sum[t]));
              if (normed) {
                const float ss = warp_sum(val * val);
                float* red = red_it + (t & 1) * 4;
                if (lane == 0) red[quarter] = ss;
                bar_sync(1, 128);
                val = val * rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)kTileM + e.eps) * wd;
              }
              if (rotate) {
                float sn, co;
                sincosf((float)e.positions[t] * freq, &sn, &co);
                float* x2 = xch + (t & 1) * kTileM;
                x2[row] = val;
                bar_sync(1, 128);
                const float partner = x2[row ^ 64];
                val = row < 64 ? val * co - partner * sn : val * co + partner * sn;
              }
              __nv_bfloat16* dst = nullptr;
              if (is_q) {
                dst = (__nv_bfloat16*)e.q_out + ((int64_t)t * e.num_heads + local) * kTileM;
              } else if (e.slots != nullptr && e.k_cache != nullptr) {
                const int64_t slot = e.slots[t];
                if (slot >= e.num_pages * e.page_size) {
                  if (row == 0) set_status(p.status, kBadSlot);
                } else if (slot >= 0) {
                  const int64_t page = slot / e.page_size, off = slot % e.page_size;
                  dst = (__nv_bfloat16*)(is_k ? e.k_cache : e.v_cache) +
                        ((page * e.num_kv_heads + local) * e.page_size + off) * (int64_t)kTileM;
                }
              }
              if (dst != nullptr) dst[row] = __float2bfloat16_rn(val);
            }
          } else {
            const int feature = tile * kTileM + row;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(P.out);
            if (feature < P.features) {
#pragma unroll
              for (int t = 0; t < kBN; ++t)
                if (t < p.tokens) out[(int64_t)t * P.features + feature] = __float2bfloat16_rn(sum[t]);
            }
          }
          // the tile is finished: make it visible, then count it
          __threadfence();
          bar_sync(1, 128);
          if (threadIdx.x == kFirstEpiWarp * 32) atomicAdd(tickets + P.tiles, 1);
        }
        b = seg_end;
        ++seg;
      }
    }
  }
  if (!ok) set_status(p.status, kWaitTimeout);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
  }
}

template <int kStages>
int launch_stages(const CUtensorMap* maps, const StreamParamsDev& p, cudaStream_t stream) {
  auto kernel = stream_phases_kernel<kStages>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           StreamSmem<kStages>::kBytes);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  return (int)launch_chain(kernel, dim3((unsigned)p.grid), dim3(kThreads), StreamSmem<kStages>::kBytes, stream,
                           dim3(1, 1, 1), maps[0], maps[1], maps[2], maps[3], p);
}

int64_t blocks_of(const StreamPhase& ph) {
  return ((ph.features + kTileM - 1) / kTileM) * ((ph.k + kTileK - 1) / kTileK);
}

// CTAs that take blocks of a phase: every one of them has at least one block, so the CTAs that share a tile are
// consecutive.
int ctas_of(const StreamPhase& ph, int grid) {
  const int64_t blocks = blocks_of(ph);
  return (int)(blocks < grid ? blocks : grid);
}

// Most CTAs that share one tile of a phase, for a grid of `grid` CTAs.
int slots_of(const StreamPhase& ph, int grid_all) {
  const int64_t tiles = (ph.features + kTileM - 1) / kTileM, kb = (ph.k + kTileK - 1) / kTileK, blocks = tiles * kb;
  const int grid = ctas_of(ph, grid_all);
  int most = 1;
  for (int64_t t = 0; t < tiles; ++t) {
    const int first = (int)(((t * kb + 1) * grid - 1) / blocks);
    const int last = (int)((((t + 1) * kb) * grid - 1) / blocks);
    most = last - first + 1 > most ? last - first + 1 : most;
  }
  return most;
}

}  // namespace

int stream_phases_grid() { return sm_count(); }

void stream_phases_scratch(const StreamPhase* phases, int num_phases, int64_t* part_floats, int64_t* sync_ints) {
  const int grid = stream_phases_grid();
  int64_t parts = 0, sync = 0;
  for (int i = 0; i < num_phases; ++i) {
    const int64_t tiles = (phases[i].features + kTileM - 1) / kTileM;
    parts += tiles * slots_of(phases[i], grid) * (kBN * kTileM);
    sync += tiles + 1;
  }
  *part_floats = parts;
  *sync_ints = sync;
}

int launch_stream_phases(const StreamPhase* phases, int num_phases, int64_t tokens, float* hidden,
                         int64_t hidden_size, float* ssq, float* parts, int* sync, int* status,
                         cudaStream_t stream) {
  if (num_phases < 1 || num_phases > kMaxStreamPhases || tokens < 1 || tokens > kBN || hidden == nullptr ||
      ssq == nullptr || parts == nullptr || sync == nullptr)
    return (int)cudaErrorInvalidValue;
  StreamParamsDev p = {};
  p.num_phases = num_phases;
  p.tokens = (int)tokens;
  p.hidden_size = (int)hidden_size;
  p.grid = stream_phases_grid();
  p.hidden = hidden;
  p.ssq = ssq;
  p.parts = parts;
  p.sync = sync;
  p.status = status;
  CUtensorMap maps[kMaxStreamPhases];
  int64_t part_offset = 0;
  int sync_offset = 0;
  bool ssq_ready = false;       // a residual phase of this launch has left the sums of squares
  for (int i = 0; i < num_phases; ++i) {
    const StreamPhase& in = phases[i];
    if (in.w == nullptr || in.features < 1 || in.k < kTileK || in.k % 8 != 0) return (int)cudaErrorInvalidValue;
    StreamPhaseDev& d = p.phase[i];
    d.features = (int)in.features;
    d.k = (int)in.k;
    d.tiles = (int)((in.features + kTileM - 1) / kTileM);
    d.kb = (int)((in.k + kTileK - 1) / kTileK);
    d.x_kind = in.x_kind;
    d.epilogue = in.epilogue;
    d.slots = slots_of(in, p.grid);
    d.ctas = ctas_of(in, p.grid);
    d.x = reinterpret_cast<const __nv_bfloat16*>(in.x);
    d.norm_weight = in.norm_weight;
    d.eps = in.eps;
    d.out = in.out;
    d.qkv = in.qkv;
    d.part_offset = part_offset;
    d.sync_offset = sync_offset;
    part_offset += (int64_t)d.tiles * d.slots * (kBN * kTileM);
    sync_offset += d.tiles + 1;
    if (in.x_kind == kStreamXNormed) {
      if (in.norm_weight == nullptr || in.k != hidden_size || hidden_size % 8 != 0) return (int)cudaErrorInvalidValue;
      d.ssq_from_hidden = ssq_ready ? 0 : 1;
    } else if (in.x_kind == kStreamXTensor) {
      if (in.x == nullptr) return (int)cudaErrorInvalidValue;
    } else {
      return (int)cudaErrorInvalidValue;
    }
    switch (in.epilogue) {
      case kEpilogueResidual:
        if (in.features != hidden_size) return (int)cudaErrorInvalidValue;
        ssq_ready = true;
        break;
      case kEpilogueGated:
        if (in.out == nullptr || in.features % kTileM != 0) return (int)cudaErrorInvalidValue;
        break;
      case kEpilogueQkv:
        if (in.qkv.q_out == nullptr || in.qkv.positions == nullptr ||
            in.features != (int64_t)(in.qkv.num_heads + 2 * in.qkv.num_kv_heads) * kTileM)
          return (int)cudaErrorInvalidValue;
        break;
      case kEpiloguePlain:
        if (in.out == nullptr) return (int)cudaErrorInvalidValue;
        break;
      default:
        return (int)cudaErrorInvalidValue;
    }
    if (!weight_tensor_map(in.w, in.features, in.k, kTileM, &maps[i])) return (int)cudaErrorInvalidValue;
  }
  for (int i = num_phases; i < kMaxStreamPhases; ++i) maps[i] = maps[0];
  // Ring depth: twelve slots of 18 KB fill the SM; AKV_STREAM_STAGES=8 leaves room for another kernel's CTA.
  static const int stages = [] {
    const char* v = getenv("AKV_STREAM_STAGES");
    const int n = v ? atoi(v) : 0;
    return n == 8 ? 8 : 12;
  }();
  if (stages == 8) return launch_stages<8>(maps, p, stream);
  return launch_stages<12>(maps, p, stream);
}

}  // namespace akv
