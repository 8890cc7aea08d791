// A chain of weight-streaming products for a few tokens in ONE persistent kernel (sm_100a).
//
// A decode step of a few tokens is bound by reading the weights once.  Run as one kernel per product, every product
// pays for its start (barriers, tensor memory, the first copies' latency) and its end (the reduction of K splits,
// the epilogue) with the memory system idle: measured on B200 about 3.5 us per kernel boundary, five boundaries a
// layer.  Here a launch takes a list of up to kMaxStreamPhases products ("phases") that depend on one another in
// order, for instance
//     o-projection (+ residual)  ->  norm + gate/up (+ SiLU-mul)  ->  down (+ residual)  ->  norm + q/k/v of the
//     next layer (+ per-head norm, rotation, cache write)
// and streams ALL their weights through one TMA ring per SM without a pause: the copy warp runs ahead through the
// phases' weight tiles as fast as ring slots free up, whatever the other warps wait for.  The reference has no
// counterpart (its products are library calls, ampere_kv/runner.py:64-66, 165, 174-177).
//
// Work.  One CTA per SM, in clusters of four.  A phase is the matrix W [features, k] cut into tiles of 128 features;
// cluster c of C takes the tiles c, c + C, ...; within a tile each of the cluster's four CTAs takes a quarter of K
// (blocks of 64: 16 KB of weights each).  A CTA accumulates its quarter of a tile in tensor memory (two
// accumulators, so the next tile's MMAs run under this one's epilogue), puts the float32 partial tile into its own
// shared memory and tells its three neighbours (an mbarrier in each one's shared memory); then every CTA adds up,
// in rank order, the four partials of the tokens it is responsible for (token t belongs to rank t mod 4), reading
// the neighbours' through distributed shared memory, and applies the phase's epilogue to them.  (A first version
// reduced through global memory, with stream-K shares, a ticket per tile and the last sharer summing: balanced to
// the block, but each hand-over between phases cost 7 to 10 us; measured, see the profile of the narrow products.)
//
// Warps (320 threads): 0 copies weights (TMA), 1 issues tcgen05.mma, 2-5 make the token operand, 6-9 are the
// epilogue.  The token operand of a phase (a bfloat16 tensor, or the RMS norm of the float32 residual stream) is
// made ONCE per phase for the CTA's quarter of K and stays in shared memory: at most 8 tokens, so a K block of it
// is one 8-row swizzle atom of 1 KB, which the MMA (N = 16) reads twice (the stride between its two 8-row groups
// is 0; the duplicate columns are not used).  It is built in eight groups in the order the blocks are used, each
// with its own barrier, so the MMAs start after the first group.  A phase's token operand needs the phase before it
// finished everywhere: every CTA counts itself in a counter in global memory when it has finished a phase
// (release), and the operand warps wait for the count (acquire).  Everything another CTA wrote in this launch is
// read past the L1 (ld.cg).
//
// No wait is unbounded: mbarrier waits and the counter polls give up after about a second, record kWaitTimeout,
// and the CTA leaves in order (copies in flight awaited, tensor memory freed, the cluster met once more so that
// nobody's shared memory goes away under a neighbour's read).  Groups of warps that meet at a named barrier decide
// to give up together (the barrier carries the vote), so nobody is left waiting at it.
#include "common.cuh"
#include "launchers.h"
#include "tensor_map.h"

#include <cuda.h>

#include <map>
#include <mutex>
#include <utility>

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
constexpr int kCluster = 4;                     // CTAs that share a tile's K
constexpr int kPartBytes = kRows * kTileM * 4;  // a float32 partial tile [token][feature]
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
// A counter update that publishes what this CTA wrote before a CTA barrier (release at GPU scope: cumulative over
// the writes of the threads that met at the barrier); the readers' loads acquire.
__device__ __forceinline__ void red_add_release(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---- cluster: neighbours' shared memory and barriers
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t peer_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float ld_peer(uint32_t remote_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote_addr) : "memory");
  return v;
}
// Arrive on a barrier in a neighbour's (or one's own) shared memory.  The arrival itself is relaxed: whoever has
// something to publish runs ONE cluster-scope fence before its four arrivals (four releasing arrivals cost four
// fences, about half a microsecond each).
__device__ __forceinline__ void peer_arrive(uint32_t remote_bar_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// The bounded wait with cluster-scope acquire: what neighbours wrote before they arrived is visible afterwards.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void cluster_meet() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

struct StreamPhaseDev {
  int features, k;
  int tiles, kb;             // ceil(features / 128), ceil(k / 64)
  int x_kind;                // kStreamXTensor / kStreamXNormed
  int epilogue;              // GemmEpilogue
  int ssq_from_hidden;       // normed x without sums of squares left by a residual phase: add them up here
  int sync_offset;           // ints into `sync`: the count of CTAs that have finished the phase
  const __nv_bfloat16* x;    // [tokens, k]
  const float* norm_weight;  // [k]
  float eps;
  void* out;                 // plain: bfloat16 [tokens, features]; gated: bfloat16 [tokens, features / 2]
  GemmQkv qkv;
};

struct StreamParamsDev {
  int num_phases, tokens, hidden_size;
  int clusters;              // the grid is clusters * kCluster CTAs
  int stages;                // ring slots of 16 KB
  int xslots;                // K blocks of token operand the buffer holds (a quarter of the longest K, rounded up)
  float* hidden;             // [tokens, hidden_size] float32: normed-x source, residual target
  float* ssq;                // [ceil(hidden_size / 128), tokens]
  int* sync;
  int* status;
  unsigned long long* trace;   // null, or [grid][phases][kTraceSlots] nanosecond stamps (measurement only)
  StreamPhaseDev phase[kMaxStreamPhases];
};

// Slots of the measurement trace [grid][phases][kTraceSlots]: where a CTA's warps are in a phase, in nanoseconds.
constexpr int kTraceSlots = 16;
enum TraceSlot : int {
  kTraceFirstCopy = 0, kTraceLastCopy = 1, kTraceFirstMma = 2, kTraceLastMma = 3, kTraceOperandMayStart = 4,
  kTraceOperandFirstGroup = 5, kTraceOperandDone = 6, kTraceLastEpilogue = 7,
  // of the CTA's last tile in the phase:
  kTraceTileAccumulated = 8, kTraceTilePartialTold = 9, kTraceTilePartialsHere = 10, kTraceTileSummed = 11,
  kTraceTileEpilogueDone = 12,
};
__device__ __forceinline__ void stamp(const StreamParamsDev& p, int cta, int ph, int what) {
  if (p.trace != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    p.trace[((int64_t)cta * kMaxStreamPhases + ph) * kTraceSlots + what] = t;
  }
}

// A CTA's share of a phase: the tiles of its cluster (first, first + clusters, ...) and its quarter of K.
struct Share {
  int first_tile, num_tiles, stride;
  int k_lo, nkb;
};
__device__ __forceinline__ Share share_of(const StreamPhaseDev& P, int cluster, int clusters, int rank) {
  Share s;
  s.first_tile = cluster;
  s.stride = clusters;
  s.num_tiles = cluster < P.tiles ? (P.tiles - cluster + clusters - 1) / clusters : 0;
  const int base = P.kb / kCluster, extra = P.kb % kCluster;
  s.k_lo = rank * base + min(rank, extra);
  s.nkb = base + (rank < extra ? 1 : 0);
  return s;
}
__device__ __forceinline__ int x_group_size(int nkb) { return (nkb + kXGroups - 1) / kXGroups; }

// Shared memory of a launch with `stages` ring slots and `xslots` K blocks of token operand.
struct StreamSmem {
  // barriers: w_full, empty per ring slot; acc_full, acc_empty per accumulator; x_ready per operand group;
  // mma_phase_done; part_ready, part_free per partial buffer
  static constexpr int kBars = (2 * kMaxStages + 4 + kXGroups + 1 + 4) * 8;
  static constexpr int kScratch = 16 + 16 * 4 + 16 * 4 * 4 + 2 * 4 * 4 + 16 + kRows * kTileM * 4;
  static constexpr int kFixed = kBars + kScratch + 2 * kPartBytes + 1024;      // + alignment slack
  static int bytes(int stages, int xslots) { return stages * kStageBytes + xslots * kXBytes + kFixed; }
};

__global__ void __launch_bounds__(kThreads, 1)
stream_phases_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                     const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3,
                     const __grid_constant__ StreamParamsDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* xbuf = smem + stages * kStageBytes;                     // [xslots][8 rows][128 bytes], swizzled
  float* part = reinterpret_cast<float*>(xbuf + p.xslots * kXBytes);   // [2][8 tokens][128 features]
  uint64_t* w_full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(part) + 2 * kPartBytes);
  uint64_t* empty = w_full + kMaxStages;
  uint64_t* acc_full = empty + kMaxStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* x_ready = acc_empty + 2;         // [kXGroups]
  uint64_t* mma_phase_done = x_ready + kXGroups;
  uint64_t* part_ready = mma_phase_done + 1; // [2] the four partials of a tile are in their CTAs' buffer b
  uint64_t* part_free = part_ready + 2;      // [2] the four CTAs have read this CTA's buffer b
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(part_free + 2);
  float* inv_rms = reinterpret_cast<float*>(tmem_holder + 4);       // [16]
  float* red_tok = inv_rms + 16;                                    // [16][4] per-token warp sums (residual)
  int* flags = reinterpret_cast<int*>(red_tok + 64 + 8);            // spare
  float* tile_buf = reinterpret_cast<float*>(flags + 4);            // [8][128] summed tokens (gated, qkv)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int rank = (int)cluster_rank();
  const int cluster = cta / kCluster;
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
      mbar_init(&part_ready[b], kCluster);
      mbar_init(&part_free[b], kCluster);
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
  cluster_meet();      // every neighbour's barriers exist before anybody arrives on them
  const uint32_t tmem_base = *tmem_holder;
  bool ok = true;

  if (warp == 0) {
    // ---- weights: run ahead through every phase's share as fast as ring slots free up.  (One thread walks the
    // blocks; every index is kept by increments: a division per block made this loop, not the memory, the limit.
    // Asking the L2 for blocks ahead of the ring, with and without eviction priorities, made the chain slower the
    // further ahead it ran, and was taken out.)
    if (lane == 0) {
      int s = 0;                 // ring slot of the next block
      uint32_t round = 0;        // parity of the times the ring has been gone around
      bool lapped = false;       // the ring has been filled once: a slot must be waited for
      for (int ph = 0; ph < p.num_phases && ok; ++ph) {
        const StreamPhaseDev& P = p.phase[ph];
        const Share sh = share_of(P, cluster, p.clusters, rank);
        stamp(p, cta, ph, kTraceFirstCopy);
        for (int i = 0, tile = sh.first_tile; i < sh.num_tiles && ok; ++i, tile += sh.stride) {
          for (int k = sh.k_lo; k < sh.k_lo + sh.nkb; ++k) {
            if (lapped && !mbar_wait(&empty[s], round ^ 1u)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&w_full[s], kWBytes);
            tma_load_2d(smem + s * kStageBytes, maps[ph], k * kTileK, tile * kTileM, &w_full[s]);
            if (++s == stages) {
              s = 0;
              round ^= 1u;
              lapped = true;
            }
          }
        }
        stamp(p, cta, ph, kTraceLastCopy);
      }
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
        const Share sh = share_of(P, cluster, p.clusters, rank);
        const int work = sh.num_tiles > 0 ? sh.nkb : 0;
        const int group_size = x_group_size(work);
        int groups_ready = 0, slots_ready = 0;      // operand groups waited for, and the slots they cover
        for (int i = 0; i < sh.num_tiles && ok && work > 0; ++i) {
          const int buf = seg & 1;
          if (seg >= 2 && !mbar_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t acc = tmem_base + (uint32_t)(buf * kBN);
          for (int slot = 0; slot < work; ++slot) {
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
            if (i == 0 && slot == 0) stamp(p, cta, ph, kTraceFirstMma);
            const uint32_t a_addr = smem_u32(smem) + (uint32_t)s * kStageBytes;
            const uint32_t b_addr = smem_u32(xbuf) + (uint32_t)slot * kXBytes;
#pragma unroll
            for (int kk = 0; kk < kTileK / 16; ++kk)
              umma_bf16(acc, umma_desc<1024>(a_addr + kk * 32), umma_desc<0>(b_addr + kk * 32),
                        (slot == 0 && kk == 0) ? 0u : 1u);
            umma_commit(&empty[s]);
            if (++s == stages) {
              s = 0;
              round ^= 1u;
            }
          }
          if (ok) umma_commit(&acc_full[buf]);
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
    // ---- token operand: the CTA's quarter of K, once per phase, in the order the blocks are used
    const int xw = warp - kFirstXWarp;
    const int xt = xw * 32 + lane;      // 0..127
    pdl_wait();       // the first phase's tokens and the residual stream come from the kernels before this one
    for (int ph = 0; ph < p.num_phases; ++ph) {
      const StreamPhaseDev& P = p.phase[ph];
      const Share sh = share_of(P, cluster, p.clusters, rank);
      const int work = sh.num_tiles > 0 ? sh.nkb : 0;
      bool fail = false;
      if (ph > 0) {
        // this CTA's MMAs of the phase before have read the operand buffer ...
        if (!mbar_wait(mma_phase_done, (ph - 1) & 1)) fail = true;
        // ... and, if it has work in this phase, the phase before has finished everywhere
        if (work > 0 && !fail) {
          const int* finished = p.sync + p.phase[ph - 1].sync_offset;
          const int everybody = p.clusters * kCluster;
          if (lane == 0) {
            uint32_t tries = 0;
            while (ld_acquire(finished) < everybody) {
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
      if (P.x_kind == kStreamXNormed && work > 0 && !fail) {
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
      const int group_size = x_group_size(work);
      for (int group = 0; group < kXGroups; ++group) {
        const int slot_lo = group * group_size;
        const int slot_hi = work < slot_lo + group_size ? work : slot_lo + group_size;
        // a task is 8 elements (16 bytes) of one token's row of one K block
        const int tasks = (slot_hi > slot_lo ? slot_hi - slot_lo : 0) * p.tokens * 8;
        for (int task = xt; task < tasks; task += kXWarps * 32) {
          const int c = task & 7;
          const int row = (task >> 3) % p.tokens;
          const int slot = slot_lo + (task >> 3) / p.tokens;
          const int k0 = (sh.k_lo + slot) * kTileK + c * 8;
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
    // ---- epilogue: this CTA's partial of every tile of its cluster, and its tokens of the tile's sum
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool leader = threadIdx.x == kFirstEpiWarp * 32;
    pdl_wait();       // the epilogues write what earlier kernels may still read
    int seg = 0;      // accumulators used so far
    int use = 0;      // partial buffers used so far (the same count in all four CTAs of the cluster)
    for (int ph = 0; ph < p.num_phases && ok; ++ph) {
      const StreamPhaseDev& P = p.phase[ph];
      const Share sh = share_of(P, cluster, p.clusters, rank);
      for (int i = 0, tile = sh.first_tile; i < sh.num_tiles; ++i, tile += sh.stride, ++use) {
        const int pb = use & 1;
        float* mine = part + pb * (kRows * kTileM);
        bool fail = false;
        // the neighbours have read what this buffer held two tiles ago
        if (use >= 2 && !mbar_wait_cluster(&part_free[pb], ((use >> 1) - 1) & 1)) fail = true;
        uint32_t v[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) v[t] = 0u;
        if (sh.nkb > 0) {
          const int buf = seg & 1;
          if (!fail && !mbar_wait(&acc_full[buf], (seg >> 1) & 1)) fail = true;
          fail = bar_any(1, 128, fail);
          if (fail) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (leader) stamp(p, cta, ph, kTraceTileAccumulated);
          tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kBN), v);
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          ++seg;
        } else {
          fail = bar_any(1, 128, fail);
          if (fail) {
            ok = false;
            break;
          }
        }
#pragma unroll
        for (int t = 0; t < kRows; ++t)
          if (t < p.tokens) mine[t * kTileM + row] = __uint_as_float(v[t]);
        bar_sync(1, 128);       // the whole partial is written (CTA scope) ...
        if (leader) {           // ... and told to the four CTAs of the cluster, this one included (cluster scope)
          fence_cluster();
          const uint32_t bar = smem_u32(&part_ready[pb]);
#pragma unroll
          for (int q = 0; q < kCluster; ++q) peer_arrive(peer_addr(bar, (uint32_t)q));
          stamp(p, cta, ph, kTraceTilePartialTold);
        }
        fail = !mbar_wait_cluster(&part_ready[pb], (use >> 1) & 1);
        fail = bar_any(1, 128, fail);
        if (fail) {
          ok = false;
          break;
        }
        if (leader) stamp(p, cta, ph, kTraceTilePartialsHere);
        // this CTA's tokens: rank, rank + 4.  All eight loads under way, then the sums in rank order.
        float sum[2];
        {
          float got[2][kCluster];
          const uint32_t base = smem_u32(mine) + (uint32_t)row * 4u;
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int q = 0; q < kCluster; ++q) {
              const int t = rank + kCluster * j;
              got[j][q] = t < p.tokens ? ld_peer(peer_addr(base + (uint32_t)(t * kTileM) * 4u, (uint32_t)q)) : 0.f;
            }
#pragma unroll
          for (int j = 0; j < 2; ++j) sum[j] = ((got[j][0] + got[j][1]) + got[j][2]) + got[j][3];
        }
        bar_sync(1, 128);       // everybody has read ...
        if (leader) {           // ... so each owner may reuse its buffer
          const uint32_t bar = smem_u32(&part_free[pb]);
#pragma unroll
          for (int q = 0; q < kCluster; ++q) peer_arrive(peer_addr(bar, (uint32_t)q));
          stamp(p, cta, ph, kTraceTileSummed);
        }
        // ---- the phase's epilogue on this CTA's tokens of the tile
        if (P.epilogue == kEpilogueResidual) {
          const int feature = tile * kTileM + row;
          float old[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int t = rank + kCluster * j;
            old[j] = (t < p.tokens && feature < P.features) ? ld_cg(p.hidden + (int64_t)t * P.features + feature) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int t = rank + kCluster * j;
            float h = 0.f;
            if (t < p.tokens && feature < P.features) {
              h = old[j] + __bfloat162float(__float2bfloat16_rn(sum[j]));
              p.hidden[(int64_t)t * P.features + feature] = h;
            }
            const float ss = warp_sum(h * h);
            if (lane == 0) red_tok[j * 4 + quarter] = ss;
          }
          bar_sync(1, 128);
          if (row < 2) {
            const int t = rank + kCluster * row;
            if (t < p.tokens)
              p.ssq[(int64_t)tile * p.tokens + t] =
                  red_tok[row * 4] + red_tok[row * 4 + 1] + red_tok[row * 4 + 2] + red_tok[row * 4 + 3];
          }
          bar_sync(1, 128);     // red_tok may be written again
        } else if (P.epilogue == kEpilogueGated || P.epilogue == kEpilogueQkv) {
          // the summed tokens go through shared memory once: the gate needs its up row, a head its other dims
#pragma unroll
          for (int j = 0; j < 2; ++j) tile_buf[j * kTileM + row] = sum[j];
          bar_sync(1, 128);
          if (P.epilogue == kEpilogueGated) {
            // rows 0-63 are gate rows, rows 64-127 the up rows of the same 64 outputs: thread (half, j) takes
            // output j of this CTA's token `half`
            const int j = row & 63, half = row >> 6;
            const int t = rank + kCluster * half;
            const int out_features = P.features / 2;
            const int feature = tile * (kTileM / 2) + j;
            if (t < p.tokens && feature < out_features) {
              const float g = __bfloat162float(__float2bfloat16_rn(tile_buf[half * kTileM + j]));
              const float u = __bfloat162float(__float2bfloat16_rn(tile_buf[half * kTileM + j + 64]));
              reinterpret_cast<__nv_bfloat16*>(P.out)[(int64_t)t * out_features + feature] =
                  __float2bfloat16_rn(silu_mul_value<__nv_bfloat16>(g, u));
            }
          } else {
            // The tile is one head of 128 dims; a warp takes a token: a lane holds dims lane, lane + 32,
            // lane + 64, lane + 96, so the norm is a sum within the warp and a dim's rotation partner (dim ^ 64)
            // sits in the same lane.
            const GemmQkv& e = P.qkv;
            const int head = tile;
            const bool is_q = head < e.num_heads, is_k = !is_q && head < e.num_heads + e.num_kv_heads;
            const int local = is_q ? head : (is_k ? head - e.num_heads : head - e.num_heads - e.num_kv_heads);
            const float* nw = is_q ? e.q_weight : (is_k ? e.k_weight : nullptr);
            const bool rotate = (is_q || is_k) && e.inv_freq != nullptr;
            const int t = rank + kCluster * quarter;       // warps 0 and 1 of the group have a token each
            if (quarter < 2 && t < p.tokens) {
              float val[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                val[j] = __bfloat162float(__float2bfloat16_rn(tile_buf[quarter * kTileM + lane + 32 * j]));
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
          }
          bar_sync(1, 128);     // tile_buf may be written again
        } else {
          const int feature = tile * kTileM + row;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int t = rank + kCluster * j;
            if (t < p.tokens && feature < P.features)
              reinterpret_cast<__nv_bfloat16*>(P.out)[(int64_t)t * P.features + feature] = __float2bfloat16_rn(sum[j]);
          }
        }
        if (leader) {
          stamp(p, cta, ph, kTraceTileEpilogueDone);
          stamp(p, cta, ph, kTraceLastEpilogue);
        }
      }
      if (!ok) break;
      // this CTA has finished the phase: count it, publishing what its epilogue threads wrote
      bar_sync(1, 128);
      if (leader) red_add_release(p.sync + P.sync_offset, 1);
    }
  }
  if (!ok) set_status(p.status, kWaitTimeout);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
  }
  cluster_meet();      // nobody's shared memory goes away while a neighbour may still read it or arrive on it
}

struct Launch {
  int clusters, stages, xslots, bytes;
};

// How many clusters of four the device holds at once with this much shared memory (the kernel needs every CTA of
// the grid resident: they wait for one another), 0 if the query fails.
int resident_clusters(int bytes) {
  static std::mutex mutex;
  static std::map<std::pair<int, int>, int> cache;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> guard(mutex);
  auto it = cache.find({device, bytes});
  if (it != cache.end()) return it->second;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(sm_count() / kCluster * kCluster));
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = (size_t)bytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = kCluster;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, stream_phases_kernel, &config) != cudaSuccess) {
    cudaGetLastError();
    clusters = 0;
  }
  cache[{device, bytes}] = clusters;
  return clusters;
}

int launch_kernel(const CUtensorMap* maps, const StreamParamsDev& p, int bytes, cudaStream_t stream) {
  return (int)launch_chain(stream_phases_kernel, dim3((unsigned)(p.clusters * kCluster)), dim3(kThreads),
                           (size_t)bytes, stream, dim3(kCluster, 1, 1), maps[0], maps[1], maps[2], maps[3], p);
}

}  // namespace

int stream_phases_grid() { return sm_count() / kCluster * kCluster; }

void stream_phases_scratch(const StreamPhase* phases, int num_phases, int64_t* part_floats, int64_t* sync_ints) {
  (void)phases;
  *part_floats = 0;          // partial tiles stay in shared memory
  *sync_ints = num_phases;   // one counter of finished CTAs per phase
}

int launch_stream_phases(const StreamPhase* phases, int num_phases, int64_t tokens, float* hidden,
                         int64_t hidden_size, float* ssq, float* parts, int* sync, int* status,
                         cudaStream_t stream, unsigned long long* trace) {
  (void)parts;
  if (num_phases < 1 || num_phases > kMaxStreamPhases || tokens < 1 || tokens > kRows || hidden == nullptr ||
      ssq == nullptr || sync == nullptr)
    return (int)cudaErrorInvalidValue;
  StreamParamsDev p = {};
  p.num_phases = num_phases;
  p.tokens = (int)tokens;
  p.hidden_size = (int)hidden_size;
  p.hidden = hidden;
  p.ssq = ssq;
  p.sync = sync;
  p.status = status;
  p.trace = trace;
  CUtensorMap maps[kMaxStreamPhases];
  bool ssq_ready = false;       // a residual phase of this launch has left the sums of squares
  int xslots = 1;
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
    d.x = reinterpret_cast<const __nv_bfloat16*>(in.x);
    d.norm_weight = in.norm_weight;
    d.eps = in.eps;
    d.out = in.out;
    d.qkv = in.qkv;
    d.sync_offset = i;
    const int quarter = (d.kb + kCluster - 1) / kCluster;
    xslots = quarter > xslots ? quarter : xslots;
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
  // The operand buffer holds a quarter of the longest K; the ring takes what is left of the SM's shared memory (at
  // most kMaxStages slots; AKV_STREAM_STAGES=n caps it for measurements).
  static const int cap = [] {
    const char* v = getenv("AKV_STREAM_STAGES");
    const int n = v ? atoi(v) : 0;
    return (n >= 2 && n <= kMaxStages) ? n : kMaxStages;
  }();
  constexpr int kSmemLimit = 227 * 1024;
  int stages = (kSmemLimit - StreamSmem::kFixed - xslots * kXBytes) / kStageBytes;
  stages = stages > cap ? cap : stages;
  if (stages < 2) return (int)cudaErrorInvalidValue;
  const int bytes = StreamSmem::bytes(stages, xslots);
  static int configured = 0;
  if (configured < bytes) {
    cudaError_t err = cudaFuncSetAttribute(stream_phases_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (err != cudaSuccess) return (int)err;
    configured = bytes;
  }
  // every CTA waits for every other one: the grid is what the device holds at once
  const int clusters = resident_clusters(bytes);
  if (clusters < 1) return (int)cudaErrorInvalidConfiguration;
  p.clusters = clusters;
  p.stages = stages;
  p.xslots = xslots;
  return launch_kernel(maps, p, bytes, stream);
}

}  // namespace akv
