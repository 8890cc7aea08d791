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
// Warps (320 threads): 0 copies weights (TMA), 1 issues tcgen05.mma, 2-5 make the token operand, 6-9 are the
// epilogue.  The token operand of a phase (a bfloat16 tensor, or the RMS norm of the float32 residual stream) is
// made ONCE per phase for all the K blocks this CTA's share touches and stays in shared memory: at most 8 tokens, so
// a K block of it is one 8-row swizzle atom of 1 KB, which the MMA (N = 16) reads twice (the stride between its two
// 8-row groups is 0; the duplicate columns are not used).  Made block by block instead, with the memory system busy
// streaming weights, every block waited microseconds for its tokens.  The operand is built in eight groups in the
// order the blocks are used, each with its own barrier, so the MMAs start after the first group.  A phase's token
// operand needs the phase before it finished everywhere: the operand warps wait on a counter of finished tiles in
// global memory.  Everything another CTA wrote in this launch is read past the L1 (ld.cg).
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
constexpr int kBN = 16;                         // token columns of the MMA
constexpr int kRows = 8;                        // tokens a launch takes at most: one 8-row swizzle atom per K block
constexpr int kWBytes = kTileM * kTileK * 2;    // 16 KB of weights per block
constexpr int kXBytes = kRows * kTileK * 2;     // 1 KB of tokens per K block
constexpr int kStageBytes = kWBytes;
constexpr int kMaxStages = 12;
constexpr int kXGroups = 8;                     // the operand of a phase becomes ready in this many parts
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
template <uint32_t kGroupStride = 1024>
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  desc |= (uint64_t)1 << 16;
  desc |= (uint64_t)(kGroupStride >> 4) << 32;
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
// Counter updates that publish what this CTA wrote before a CTA barrier (release at GPU scope: cumulative over the
// writes of the threads that met at the barrier) and take in what others published (acquire).
__device__ __forceinline__ int atom_add_acq_rel(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_add_release(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
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
  int stages;                // ring slots of 16 KB
  int xslots;                // K blocks of token operand the buffer holds (the most any CTA needs in any phase)
  float* hidden;             // [tokens, hidden_size] float32: normed-x source, residual target
  float* ssq;                // [ceil(hidden_size / 128), tokens]
  float* parts;
  int* sync;
  int* status;
  unsigned long long* trace;   // null, or [grid][phases][8] nanosecond stamps (measurement only)
  StreamPhaseDev phase[kMaxStreamPhases];
};

// Slots of the measurement trace [grid][phases][kTraceSlots]: where a CTA's warps are in a phase, in nanoseconds.
constexpr int kTraceSlots = 16;
enum TraceSlot : int {
  kTraceFirstCopy = 0, kTraceLastCopy = 1, kTraceFirstMma = 2, kTraceLastMma = 3, kTraceOperandMayStart = 4,
  kTraceOperandFirstGroup = 5, kTraceOperandDone = 6, kTraceLastEpilogue = 7,
  // of the CTA's last segment in the phase:
  kTraceSegAccumulated = 8, kTraceSegPartialStored = 9, kTraceSegTicket = 10, kTraceSegFinalizeStart = 11,
  kTraceSegFinalizeMath = 12, kTraceSegPublished = 13,
};
__device__ __forceinline__ void stamp(const StreamParamsDev& p, int cta, int ph, int what) {
  if (p.trace != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.trace[((int64_t)cta * kMaxStreamPhases + ph) * kTraceSlots + what] = t;
  }
}

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

// One CTA's walk through its blocks of every phase, in order: the phase, the K block and the first feature row of
// the block to come.  All by increments.
struct BlockWalk {
  int ph, k, y, left;      // left: blocks of this phase still to come, this one included
  __device__ BlockWalk(const StreamParamsDev& p, int cta) : ph(-1), k(0), y(0), left(0) { enter(p, cta); }
  __device__ void enter(const StreamParamsDev& p, int cta) {
    while (left == 0 && ++ph < p.num_phases) {
      const BlockRange r = cta_range(p.phase[ph], cta);
      left = r.hi - r.lo;
      if (left > 0) {
        k = r.lo % p.phase[ph].kb;
        y = (r.lo / p.phase[ph].kb) * kTileM;
      }
    }
  }
  __device__ bool valid() const { return left > 0; }
  __device__ void next(const StreamParamsDev& p, int cta) {
    if (++k == p.phase[ph].kb) {
      k = 0;
      y += kTileM;
    }
    if (--left == 0) enter(p, cta);
  }
};

// Shared memory of a launch with `stages` ring slots and `xslots` K blocks of token operand.
struct StreamSmem {
  // barriers: w_full, empty per ring slot; acc_full, acc_empty per accumulator; x_ready per operand group;
  // mma_phase_done
  static constexpr int kBars = (2 * kMaxStages + 4 + kXGroups + 1) * 8;
  static constexpr int kScratch = 16 + 16 * 4 + 16 * 4 * 4 + 2 * kTileM * 4 + 2 * 4 * 4 + 16 + kRows * kTileM * 4;
  static constexpr int kFixed = kBars + kScratch + 1024;      // + alignment slack
  static int bytes(int stages, int xslots) { return stages * kStageBytes + xslots * kXBytes + kFixed; }
};

// The K blocks of a phase that a CTA's share touches, in the order it uses them: `count` of them from `first`,
// wrapping around at kb.  Block k has its tokens in slot (k - first) mod kb of the operand buffer.
struct XSpan {
  int first, count;
};
__device__ __forceinline__ XSpan x_span(const StreamPhaseDev& P, const BlockRange& r) {
  const int blocks = r.hi - r.lo;
  return {blocks > 0 ? r.lo % P.kb : 0, blocks < P.kb ? blocks : P.kb};
}
__device__ __forceinline__ int x_slot(const StreamPhaseDev& P, const XSpan& span, int k) {
  const int d = k - span.first;
  return d < 0 ? d + P.kb : d;
}
__device__ __forceinline__ int x_group_size(const XSpan& span) { return (span.count + kXGroups - 1) / kXGroups; }

__global__ void __launch_bounds__(kThreads, 1)
stream_phases_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                     const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3,
                     const __grid_constant__ StreamParamsDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* xbuf = smem + stages * kStageBytes;                     // [xslots][8 rows][128 bytes], swizzled
  uint64_t* w_full = reinterpret_cast<uint64_t*>(xbuf + p.xslots * kXBytes);
  uint64_t* empty = w_full + kMaxStages;
  uint64_t* acc_full = empty + kMaxStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* x_ready = acc_empty + 2;         // [kXGroups]
  uint64_t* mma_phase_done = x_ready + kXGroups;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(mma_phase_done + 1);
  float* inv_rms = reinterpret_cast<float*>(tmem_holder + 4);       // [16]
  float* red_tok = inv_rms + 16;                                    // [16][4] per-token warp sums (residual)
  float* xch = red_tok + 64;                                        // [2][128] rotation partners (qkv)
  float* red_it = xch + 2 * kTileM;                                 // [2][4] per-head warp sums (qkv)
  int* flags = reinterpret_cast<int*>(red_it + 8);                  // [0]: ticket broadcast
  float* tile_buf = reinterpret_cast<float*>(flags + 4);            // [8][128] a finished tile (qkv)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const CUtensorMap* maps[kMaxStreamPhases] = {&map0, &map1, &map2, &map3};

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&w_full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);      // one arrival per epilogue warp
    }
    for (int g = 0; g < kXGroups; ++g) mbar_init(&x_ready[g], kXWarps);
    mbar_init(mma_phase_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(32u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // rows of the operand past the tokens are never written: zero them once (their columns are not used, but they
  // should not hold whatever the last kernel left)
  for (int i = threadIdx.x; i < p.xslots * kXBytes / 16; i += kThreads)
    reinterpret_cast<uint4*>(xbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  bool ok = true;

  if (warp == 0) {
    // ---- weights: run ahead through every phase's share as fast as ring slots free up.  (One thread walks the
    // blocks; every index is kept by increments: a division per block made this loop, not the memory, the limit.)
    // (A second cursor that asked the L2 for blocks ahead of the ring, so that the memory would keep streaming
    // while the MMAs wait for a phase to finish everywhere, made the chain slower the further ahead it ran, with
    // and without eviction priorities: 108 / 113 / 120 / 135 us at 0 / 8 / 16 / 32 blocks.  It was taken out.)
    if (lane == 0) {
      BlockWalk load(p, cta);
      int s = 0;                 // ring slot of the next block
      uint32_t round = 0;        // parity of the times the ring has been gone around
      bool lapped = false;       // the ring has been filled once: a slot must be waited for
      int stamped = -1;
      while (load.valid()) {
        if (load.ph != stamped) {
          if (stamped >= 0) stamp(p, cta, stamped, kTraceLastCopy);
          stamped = load.ph;
          stamp(p, cta, stamped, kTraceFirstCopy);
        }
        if (lapped && !mbar_wait(&empty[s], round ^ 1u)) {
          ok = false;
          break;
        }
        mbar_expect_tx(&w_full[s], kWBytes);
        tma_load_2d(smem + s * kStageBytes, maps[load.ph], load.k * kTileK, load.y, &w_full[s]);
        load.next(p, cta);
        if (++s == stages) {
          s = 0;
          round ^= 1u;
          lapped = true;
        }
      }
      if (stamped >= 0) stamp(p, cta, stamped, kTraceLastCopy);
      if (!ok) {
        // copies already issued must land before the CTA's shared memory goes away: every slot whose copy has not
        // been consumed completes its current phase (bounded waits; a slot never used returns at once)
        for (int i = 0; i < stages; ++i) mbar_wait(&w_full[i], (i < s ? round : round ^ 1u));
      }
    }
  } else if (warp == 1) {
    // ---- tensor cores: one thread walks the same blocks and issues the MMAs
    if (lane == 0) {
      int s = 0, seg = 0;
      uint32_t round = 0;
      for (int ph = 0; ph < p.num_phases && ok; ++ph) {
        const StreamPhaseDev& P = p.phase[ph];
        const BlockRange r = cta_range(P, cta);
        const XSpan span = x_span(P, r);
        const int group_size = x_group_size(span);
        int groups_ready = 0, slots_ready = 0;      // operand groups waited for, and the slots they cover
        int slot = 0;                                // operand slot of the next block: they are used in order
        int k = r.hi > r.lo ? r.lo % P.kb : 0;
        int b = r.lo;
        while (b < r.hi && ok) {
          const int seg_blocks = min(r.hi - b, P.kb - k);      // to the end of the tile or of the share
          const int buf = seg & 1;
          if (seg >= 2 && !mbar_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t acc = tmem_base + (uint32_t)(buf * kBN);
          for (int i = 0; i < seg_blocks; ++i) {
            while (slot >= slots_ready && groups_ready < kXGroups && ok) {
              if (!mbar_wait(&x_ready[groups_ready], ph & 1)) ok = false;
              ++groups_ready;
              slots_ready += group_size;
            }
            if (!ok || !mbar_wait(&w_full[s], round)) {
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (b == r.lo && i == 0) stamp(p, cta, ph, kTraceFirstMma);
            const uint32_t a_addr = smem_u32(smem) + (uint32_t)s * kStageBytes;
            const uint32_t b_addr = smem_u32(xbuf) + (uint32_t)slot * kXBytes;
#pragma unroll
            for (int kk = 0; kk < kTileK / 16; ++kk)
              umma_bf16(acc, umma_desc<1024>(a_addr + kk * 32), umma_desc<0>(b_addr + kk * 32),
                        (i == 0 && kk == 0) ? 0u : 1u);
            umma_commit(&empty[s]);
            if (++s == stages) {
              s = 0;
              round ^= 1u;
            }
            if (++slot == P.kb) slot = 0;
          }
          if (ok) umma_commit(&acc_full[buf]);
          b += seg_blocks;
          k += seg_blocks;
          if (k == P.kb) k = 0;
          ++seg;
        }
        // every operand group of the phase is waited for, used or not, so that the barriers' phases stay in step
        while (groups_ready < kXGroups && ok) {
          if (!mbar_wait(&x_ready[groups_ready], ph & 1)) ok = false;
          ++groups_ready;
        }
        stamp(p, cta, ph, kTraceLastMma);
        if (ok) umma_commit(mma_phase_done);      // arrives once every MMA of the phase has read the operand
      }
    }
  } else if (warp < kFirstEpiWarp) {
    // ---- token operand: all K blocks this CTA's share touches, once per phase, in the order they are used
    const int xw = warp - kFirstXWarp;
    const int xt = xw * 32 + lane;      // 0..127
    pdl_wait();       // the first phase's tokens and the residual stream come from the kernels before this one
    for (int ph = 0; ph < p.num_phases; ++ph) {
      const StreamPhaseDev& P = p.phase[ph];
      const BlockRange r = cta_range(P, cta);
      const XSpan span = x_span(P, r);
      bool fail = false;
      if (ph > 0) {
        // this CTA's MMAs of the phase before have read the operand buffer ...
        if (!mbar_wait(mma_phase_done, (ph - 1) & 1)) fail = true;
        // ... and, if it has work in this phase, the phase before has finished everywhere
        if (span.count > 0 && !fail) {
          const StreamPhaseDev& Q = p.phase[ph - 1];
          const int* finished = p.sync + Q.sync_offset + Q.tiles;
          if (lane == 0) {
            uint32_t tries = 0;
            while (ld_acquire(finished) < Q.tiles) {
              if (++tries > kPollLimit) {
                fail = true;
                break;
              }
              __nanosleep(20);
            }
          }
          fail = __shfl_sync(0xffffffffu, (int)fail, 0) != 0;
        }
      }
      if (P.x_kind == kStreamXNormed && span.count > 0 && !fail) {
        // 1 / rms of every token's row of the residual stream
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
      if (fail) {
        ok = false;
        break;
      }
      if (xt == 0) stamp(p, cta, ph, kTraceOperandMayStart);
      const int group_size = x_group_size(span);
      for (int group = 0; group < kXGroups; ++group) {
        const int slot_lo = group * group_size;
        const int slot_hi = span.count < slot_lo + group_size ? span.count : slot_lo + group_size;
        // a task is 8 elements (16 bytes) of one token's row of one K block
        const int tasks = (slot_hi > slot_lo ? slot_hi - slot_lo : 0) * p.tokens * 8;
        for (int task = xt; task < tasks; task += kXWarps * 32) {
          const int c = task & 7;
          const int row = (task >> 3) % p.tokens;
          const int slot = slot_lo + (task >> 3) / p.tokens;
          int kblock = span.first + slot;
          if (kblock >= P.kb) kblock -= P.kb;
          const int k0 = kblock * kTileK + c * 8;
          uint4 packed = make_uint4(0u, 0u, 0u, 0u);    // columns past K: zeros
          if (k0 < P.k) {
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
          *reinterpret_cast<uint4*>(xbuf + slot * kXBytes + row * 128 + ((c ^ (row & 7)) << 4)) = packed;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the tensor core reads through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&x_ready[group]);
        if (xt == 0 && group == 0) stamp(p, cta, ph, kTraceOperandFirstGroup);
      }
      if (xt == 0) stamp(p, cta, ph, kTraceOperandDone);
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
        const bool stamper = threadIdx.x == kFirstEpiWarp * 32;
        if (stamper) stamp(p, cta, ph, kTraceSegAccumulated);
        uint32_t v[16];
        tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kBN), v);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        // who shares this tile: the CTAs from the one that holds its first block to the one that holds its last
        const int first_cta = cta_of_block((int64_t)tile * P.kb, blocks, P.ctas);
        const int last_cta = cta_of_block((int64_t)(tile + 1) * P.kb - 1, blocks, P.ctas);
        const int sharers = last_cta - first_cta + 1;
        float* tile_parts = p.parts + P.part_offset + (int64_t)tile * P.slots * (kRows * kTileM);
        float* mine = tile_parts + (int64_t)(cta - first_cta) * (kRows * kTileM);
        if (sharers > 1) {
#pragma unroll
          for (int t = 0; t < kRows; ++t)
            if (t < p.tokens) mine[t * kTileM + row] = __uint_as_float(v[t]);
          if (stamper) stamp(p, cta, ph, kTraceSegPartialStored);
          bar_sync(1, 128);       // everybody's partial is written (CTA scope) ...
          if (threadIdx.x == kFirstEpiWarp * 32) flags[0] = atom_add_acq_rel(&tickets[tile], 1);   // ... and published
          bar_sync(1, 128);
          if (stamper) stamp(p, cta, ph, kTraceSegTicket);
        }
        const bool last = sharers == 1 || flags[0] == sharers - 1;
        if (last) {
          // the tile is whole (the ticket's acquire, passed on by the barrier, lets everybody see the partials):
          // add them up in slot order and apply the phase's epilogue
          if (stamper) stamp(p, cta, ph, kTraceSegFinalizeStart);
          float sum[kRows];
#pragma unroll
          for (int t = 0; t < kRows; ++t) sum[t] = 0.f;
          if (sharers == 1) {
#pragma unroll
            for (int t = 0; t < kRows; ++t) sum[t] = __uint_as_float(v[t]);
          } else if (P.epilogue != kEpilogueGated) {
            // eight sharers' partials under way at a time (one round trip to the L2), added in slot order
            for (int s0 = 0; s0 < sharers; s0 += 8) {
              float part[8][kRows];
#pragma unroll
              for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int t = 0; t < kRows; ++t)
                  part[j][t] = (s0 + j < sharers && t < p.tokens)
                                   ? ld_cg(tile_parts + (int64_t)(s0 + j) * (kRows * kTileM) + t * kTileM + row)
                                   : 0.f;
#pragma unroll
              for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int t = 0; t < kRows; ++t) sum[t] += part[j][t];      // absent ones add an exact zero
            }
          }
          if (P.epilogue == kEpilogueResidual) {
            const int feature = tile * kTileM + row;
            // the stream's old values of all tokens first (one round trip; a load after each store waited for one
            // each), then the sums and the stores
            float old[kRows];
#pragma unroll
            for (int t = 0; t < kRows; ++t)
              old[t] = (t < p.tokens && feature < P.features) ? ld_cg(p.hidden + (int64_t)t * P.features + feature)
                                                              : 0.f;
#pragma unroll
            for (int t = 0; t < kRows; ++t) {
              if (t >= p.tokens) break;
              float h = 0.f;
              if (feature < P.features) {
                h = old[t] + __bfloat162float(__float2bfloat16_rn(sum[t]));
                p.hidden[(int64_t)t * P.features + feature] = h;
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
            // every other token and needs both of its rows: through the tile's first partial slot when the tile is
            // this CTA's alone, else from the partials.
            const int j = row & 63, half = row >> 6;
            const int out_features = P.features / 2;
            const int feature = tile * (kTileM / 2) + j;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(P.out);
            if (sharers == 1) {
#pragma unroll
              for (int t = 0; t < kRows; ++t)
                if (t < p.tokens) mine[t * kTileM + row] = sum[t];
              __threadfence();
              bar_sync(1, 128);
            }
            // this thread's tokens (every other one: at most four), all of their loads under way before the
            // first sum
            float gs[kRows / 2], us[kRows / 2];
#pragma unroll
            for (int i = 0; i < kRows / 2; ++i) gs[i] = us[i] = 0.f;
            for (int s0 = 0; s0 < sharers; s0 += 4) {
              float pg[4][kRows / 2], pu[4][kRows / 2];
#pragma unroll
              for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                for (int i = 0; i < kRows / 2; ++i) {
                  const int t = half + 2 * i;
                  const bool live = s0 + jj < sharers && t < p.tokens;
                  const float* part = tile_parts + (int64_t)(s0 + jj) * (kRows * kTileM) + t * kTileM;
                  pg[jj][i] = live ? ld_cg(part + j) : 0.f;
                  pu[jj][i] = live ? ld_cg(part + j + 64) : 0.f;
                }
#pragma unroll
              for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                for (int i = 0; i < kRows / 2; ++i) {
                  gs[i] += pg[jj][i];
                  us[i] += pu[jj][i];
                }
            }
#pragma unroll
            for (int i = 0; i < kRows / 2; ++i) {
              const int t = half + 2 * i;
              if (t >= p.tokens) break;
              const float g = __bfloat162float(__float2bfloat16_rn(gs[i]));
              const float u = __bfloat162float(__float2bfloat16_rn(us[i]));
              if (feature < out_features)
                out[(int64_t)t * out_features + feature] = __float2bfloat16_rn(silu_mul_value<__nv_bfloat16>(g, u));
            }
          } else if (P.epilogue == kEpilogueQkv) {
            // The tile is one head of 128 dims.  Its values, rounded as the stored product would be, go through
            // shared memory once; then a warp takes a token: a lane holds dims lane, lane + 32, lane + 64,
            // lane + 96, so the norm is a sum within the warp and a dim's rotation partner (dim ^ 64) sits in the
            // same lane.  No barrier per token.
            const GemmQkv& e = P.qkv;
            const int head = tile;
            const bool is_q = head < e.num_heads, is_k = !is_q && head < e.num_heads + e.num_kv_heads;
            const int local = is_q ? head : (is_k ? head - e.num_heads : head - e.num_heads - e.num_kv_heads);
            const float* nw = is_q ? e.q_weight : (is_k ? e.k_weight : nullptr);
            const bool rotate = (is_q || is_k) && e.inv_freq != nullptr;
#pragma unroll
            for (int t = 0; t < kRows; ++t)
              if (t < p.tokens) tile_buf[t * kTileM + row] = __bfloat162float(__float2bfloat16_rn(sum[t]));
            bar_sync(1, 128);
            for (int t = quarter; t < p.tokens; t += 4) {
              float val[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) val[j] = tile_buf[t * kTileM + lane + 32 * j];
              if (nw != nullptr) {
                const float ss = warp_sum(val[0] * val[0] + val[1] * val[1] + val[2] * val[2] + val[3] * val[3]);
                const float inv = rsqrtf(ss / (float)kTileM + e.eps);
#pragma unroll
                for (int j = 0; j < 4; ++j) val[j] = val[j] * inv * nw[lane + 32 * j];
              }
              if (rotate) {
                const float pos = (float)e.positions[t];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  float sn, co;
                  sincosf(pos * e.inv_freq[lane + 32 * j], &sn, &co);
                  const float lo = val[j], hi = val[j + 2];
                  val[j] = lo * co - hi * sn;
                  val[j + 2] = hi * co + lo * sn;
                }
              }
              __nv_bfloat16* dst = nullptr;
              if (is_q) {
                dst = (__nv_bfloat16*)e.q_out + ((int64_t)t * e.num_heads + local) * kTileM;
              } else if (e.slots != nullptr && e.k_cache != nullptr) {
                const int64_t slot = e.slots[t];
                if (slot >= e.num_pages * e.page_size) {
                  if (lane == 0) set_status(p.status, kBadSlot);
                } else if (slot >= 0) {
                  const int64_t page = slot / e.page_size, off = slot % e.page_size;
                  dst = (__nv_bfloat16*)(is_k ? e.k_cache : e.v_cache) +
                        ((page * e.num_kv_heads + local) * e.page_size + off) * (int64_t)kTileM;
                }
              }
              if (dst != nullptr) {
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(val[j]);
              }
            }
          } else {
            const int feature = tile * kTileM + row;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(P.out);
            if (feature < P.features) {
#pragma unroll
              for (int t = 0; t < kRows; ++t)
                if (t < p.tokens) out[(int64_t)t * P.features + feature] = __float2bfloat16_rn(sum[t]);
            }
          }
          // the tile is finished: count it, publishing what everybody wrote before the barrier
          if (stamper) stamp(p, cta, ph, kTraceSegFinalizeMath);
          bar_sync(1, 128);
          if (threadIdx.x == kFirstEpiWarp * 32) red_add_release(tickets + P.tiles, 1);
          if (stamper) stamp(p, cta, ph, kTraceSegPublished);
        }
        b = seg_end;
        ++seg;
        if (threadIdx.x == kFirstEpiWarp * 32) stamp(p, cta, ph, kTraceLastEpilogue);
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

int launch_kernel(const CUtensorMap* maps, const StreamParamsDev& p, cudaStream_t stream) {
  auto kernel = stream_phases_kernel;
  const int bytes = StreamSmem::bytes(p.stages, p.xslots);
  static int configured = 0;
  if (configured < bytes) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (err != cudaSuccess) return (int)err;
    configured = bytes;
  }
  return (int)launch_chain(kernel, dim3((unsigned)p.grid), dim3(kThreads), (size_t)bytes, stream, dim3(1, 1, 1),
                           maps[0], maps[1], maps[2], maps[3], p);
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
    parts += tiles * slots_of(phases[i], grid) * (kRows * kTileM);
    sync += tiles + 1;
  }
  *part_floats = parts;
  *sync_ints = sync;
}

int launch_stream_phases(const StreamPhase* phases, int num_phases, int64_t tokens, float* hidden,
                         int64_t hidden_size, float* ssq, float* parts, int* sync, int* status,
                         cudaStream_t stream, unsigned long long* trace) {
  if (num_phases < 1 || num_phases > kMaxStreamPhases || tokens < 1 || tokens > kRows || hidden == nullptr ||
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
  p.trace = trace;
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
    part_offset += (int64_t)d.tiles * d.slots * (kRows * kTileM);
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
  // The operand buffer holds the most K blocks any CTA touches in any phase; the ring takes what is left of the
  // SM's shared memory (at most kMaxStages slots; AKV_STREAM_STAGES=n caps it for measurements).
  int xslots = 1;
  for (int i = 0; i < num_phases; ++i) {
    const int64_t blocks = (int64_t)p.phase[i].tiles * p.phase[i].kb;
    const int64_t most = (blocks + p.phase[i].ctas - 1) / p.phase[i].ctas;
    const int need = (int)(most < p.phase[i].kb ? most : p.phase[i].kb);
    xslots = need > xslots ? need : xslots;
  }
  static const int cap = [] {
    const char* v = getenv("AKV_STREAM_STAGES");
    const int n = v ? atoi(v) : 0;
    return (n >= 2 && n <= kMaxStages) ? n : kMaxStages;
  }();
  constexpr int kSmemLimit = 227 * 1024;
  int stages = (kSmemLimit - StreamSmem::kFixed - xslots * kXBytes) / kStageBytes;
  stages = stages > cap ? cap : stages;
  if (stages < 2) return (int)cudaErrorInvalidValue;
  p.stages = stages;
  p.xslots = xslots;
  return launch_kernel(maps, p, stream);
}

}  // namespace akv
