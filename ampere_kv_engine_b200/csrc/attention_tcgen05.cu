// Causal paged attention for prompt portions on the 5th-generation tensor cores (tcgen05), bfloat16, head
// size 128.  One CTA owns up to 128 query rows = TQ tokens x G q-heads of one kv head (any G from 1 to 16;
// TQ = 128 / G rounded down, so a group of 5 fills 125 rows and the last three stay dead) and walks the keys 64 at
// a time:
//     S  = Q K^T          tcgen05.mma (M = 128, N = 64, K = 16 x 8), Q and K from shared memory, S in TMEM
//     P  = softmax part   128 threads, one query row each: tcgen05.ld of the row, mask, running max and sum in
//                         float32, P written to shared memory as bfloat16 in the swizzled operand layout
//     O += P V            tcgen05.mma (M = 128, N = 128, K = 16 x 4), V straight from its page rows (an
//                         MN-major operand), O accumulated in TMEM over all blocks
// The running maximum a row's probabilities are taken against is only raised when the new maximum exceeds it by
// more than 8 (in log2 units, a factor of 256): then the row's O in TMEM is rescaled (tcgen05.ld, multiply,
// tcgen05.st) by the threads of its warp; otherwise P = 2^(s - reference) may exceed 1, which float32 sums and
// bfloat16 probabilities hold without loss, and O / l at the end is exact either way.  Scores are double-buffered
// in TMEM and P in shared memory, so the tensor core works on the next block's scores while the threads are in
// the softmax of this one.
// Warps 0-3 are the softmax / accumulate threads (TMEM lanes 0-127), warp 4 issues the TMA loads (Q tile once,
// then a ring of K/V stages, one box per page and 64-dim half, no multicast), warp 5 issues the MMAs.  The
// mathematics is the reference's (ampere_kv/kv_cache.py:76-94): score = q.k * scale, key j visible to the query at
// position t iff j <= t (and j > t - window), q-head h reads kv-head h / G.
//
//
// That is the narrow form, for launches of more CTAs than SMs (two CTAs share an SM and fill each other's waits).
// Launches that fit in one wave (short prompts, portions of long ones) take the wide form further down: one CTA
// per SM with all of its tensor memory, 128-key blocks, two threads per query row and an issuing thread each for
// the scores and for P V.
//
// Every wait is bounded; a wait that runs out sets kWaitTimeout in the status word and the CTA frees its TMEM and
// leaves without writing results.
#include "common.cuh"
#include "launchers.h"

#include <cuda.h>
#include <math_constants.h>
#include <stdlib.h>

#include <map>
#include <mutex>
#include <tuple>

namespace akv {

namespace {

constexpr int kD = 128;             // head size
constexpr int kRows = 128;          // query rows per CTA
constexpr int kKeys = 64;           // keys per block
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
  return mbar_wait_bounded(s_addr(bar), parity, kWaitLimit);
}
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(s_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(s_addr(bar))
      : "memory");
}
__device__ __forceinline__ void tma_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(s_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(s_addr(bar))
      : "memory");
}

// Shared-memory operand descriptors, 128-byte swizzle, version 1 (Blackwell).
//   K-major tile (rows of 128 bytes): leading offset unused (1), 1024 bytes between 8-row groups.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
//   MN-major tile (V: one row of 128 bytes = 64 head dims of one key): `atom_bytes` between the 64-dim halves
//   (leading offset), 1024 bytes between groups of 8 keys (stride offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t atom_bytes) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(atom_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: float32 accumulator, bfloat16 operands, M = 128, N = n, A K-major, B K- or MN-major.
__device__ __forceinline__ constexpr uint32_t idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kRows >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate)
      : "memory");
}
// The same with the A operand read from tensor memory (lane = row, a 32-bit column = two consecutive K elements).
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t id,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(id), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bar))
               : "memory");
}
struct FaParams {
  PagedAttentionParams p;
  int tq;          // tokens per CTA = 128 / G
  int subtiles;    // CTAs per batch tile
  int box_rows;    // rows of one K/V box = min(page_size, 64)
};

// Shared memory: Q [2 halves][128 rows][128 B] | K/V ring: per stage K [2][64][128 B], V [2][64][128 B] |
// P [2 buffers][128 rows][128 B] | barriers | TMEM base.
template <int kStagesKV>
struct FaSmemT {
  static constexpr int kQ = 2 * kRows * 128;
  static constexpr int kK = 2 * kKeys * 128;
  static constexpr int kStage = 2 * kK;
  static constexpr int kBars = (1 + 4 * kStagesKV + 2 + 2 + 2) * 8;
  static constexpr int kBytes = kQ + kStagesKV * kStage + kBars + 16 + 1024;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

constexpr float kRescaleThreshold = 8.f;     // log2 units

// kStagesKV = 2: 96 KB of shared memory and at most 168 registers, two CTAs per SM (each takes half of the SM's
// tensor memory): one CTA's softmax fills the other's waits.  kStagesKV = 4: one CTA per SM with a deeper K/V ring,
// for launches with fewer CTAs than SMs.
template <int kStagesKV>
__global__ void __launch_bounds__(192, kStagesKV <= 2 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map, FaParams fp) {
  using FaSmem = FaSmemT<kStagesKV>;
  const PagedAttentionParams& p = fp.p;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + FaSmem::kQ;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(kv_smem + kStagesKV * FaSmem::kStage);
  uint64_t* k_full = q_full + 1;                 // [stages]
  uint64_t* v_full = k_full + kStagesKV;         // [stages]
  uint64_t* k_empty = v_full + kStagesKV;        // [stages] the scores of the stage's block are computed: K may go
  uint64_t* kv_empty = k_empty + kStagesKV;      // [stages] P V of the stage's block is done: V may go
  uint64_t* s_ready = kv_empty + kStagesKV;      // [2] scores of a block are in TMEM buffer (block & 1)
  // P of a block is in shared memory buffer (block & 1): 128 arrivals.  One barrier per buffer, because a softmax
  // warp may run one block ahead of another (the scores are double-buffered), and its arrival for block j + 1 must
  // not count towards block j.
  uint64_t* p_ready = s_ready + 2;               // [2]
  // O holds the sum through block j: barrier (j & 1), phase (j >> 1).  Two barriers, because a softmax thread
  // that did not rescale has not watched them: what it knows is that P V of block j - 2 is done once it has seen
  // the scores of block j, and with one barrier per parity of j that is exactly the phase before the one it
  // waits for, so that a parity wait cannot be answered by an older or a newer phase.
  uint64_t* pv_done = p_ready + 2;               // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 2);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.num_heads / p.num_kv_heads, NH = p.num_heads, P = p.page_size;
  const int kvh = blockIdx.y;
  constexpr uint32_t kTmemCols = 256;            // S: columns 0-63 and 64-127, O: columns 128-255

  pdl_launch_dependents();
  // CTAs start in index order and a sequence's later tiles see more keys: walk the tiles backwards, longest first
  const int slot = blockIdx.x / fp.subtiles, sub = blockIdx.x - slot * fp.subtiles;
  const int batch_tile = (int)(gridDim.x / fp.subtiles) - 1 - slot;
  const int seq = p.tile_seq[batch_tile];
  const int q0 = p.tile_q0[batch_tile] + fp.tq * sub;
  const int nq = min(fp.tq, p.tile_nq[batch_tile] - fp.tq * sub);
  if (nq <= 0) return;
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  const int tile_pos = ctx - q_len + (q0 - seq_q0);
  int lo = p.window > 0 ? max(0, tile_pos - p.window + 1) : 0;
  lo = lo / fp.box_rows * fp.box_rows;
  const int hi = tile_pos + nq;
  const int num_blocks = (hi - lo + kKeys - 1) / kKeys;

  if (tid == 0) {
    bar_init(q_full, 1);
    for (int s = 0; s < kStagesKV; ++s) {
      bar_init(&k_full[s], 1);
      bar_init(&v_full[s], 1);
      bar_init(&k_empty[s], 1);
      bar_init(&kv_empty[s], 1);
    }
    bar_init(&s_ready[0], 1);
    bar_init(&s_ready[1], 1);
    bar_init(&p_ready[0], kRows);
    bar_init(&p_ready[1], kRows);
    bar_init(&pv_done[0], 1);
    bar_init(&pv_done[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_holder)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_holder;
  pdl_wait();      // q and this step's K/V pages come from the previous kernels
  bool ok = true;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      // tq tokens x G heads: all 128 rows when G divides 128, else fewer (rows past them are dead: never live)
      bar_expect_tx(q_full, 2u * (uint32_t)(fp.tq * G) * 128u);
      // rows of the tile in (token, head) order: box {64 dims, G heads, tq tokens} per 64-dim half
      tma_3d(q_smem, &q_map, 0, kvh * G, q0, q_full);
      tma_3d(q_smem + kRows * 128, &q_map, 64, kvh * G, q0, q_full);
    }
    const int32_t* table = p.block_table + (int64_t)seq * p.table_width;
    // One copy per lane: lane = 4 * box + kind, kind = K low half, K high half, V low half, V high half.  The
    // lanes look their pages up and issue their copies side by side; one thread doing the block's up to
    // sixteen look-ups and copies in turn took longer than the tensor cores need for the block.  The look-up
    // of a block is started one block early, so that its latency hides behind the wait for the stage.
    const int boxes = kKeys / fp.box_rows;
    const int x = lane >> 2, kind = lane & 3;
    auto row_of = [&](int blk) -> int {       // first cache row of this lane's box in block blk, -1: no box
      const int key = lo + blk * kKeys + x * fp.box_rows;
      if (blk >= num_blocks || x >= boxes || key >= hi) return -1;
      const int logical = key / P;
      int page = logical < p.table_width ? table[logical] : -1;
      if (page < 0 || page >= p.num_pages) {
        set_status(p.status, kBadPage);
        page = 0;     // keep the byte count honest; the result is flagged
      }
      return (page * p.num_kv_heads + kvh) * P + key % P;
    };
    // K of a stage is free as soon as the scores of its block are computed, V only after P V: K runs one block
    // ahead of V (the issuer computes the scores of block b + 1 before P V of block b), so each iteration fetches
    // K of block b + 1 and V of block b.  With two stages that is what hides the copy's latency.
    auto fetch = [&](int blk, int y, bool keys) -> bool {      // this lane's copies of K or V of block blk
      const int s = blk % kStagesKV;
      if (blk >= kStagesKV) {
        const bool freed = bar_wait(keys ? &k_empty[s] : &kv_empty[s], ((blk / kStagesKV) - 1) & 1);
        if (!__all_sync(0xffffffffu, freed)) return false;       // the warp decides together: it votes below
      }
      const bool mine = y >= 0 && (kind < 2) == keys;
      const uint32_t valid_boxes = __popc(__ballot_sync(0xffffffffu, y >= 0 && kind == 0));
      uint64_t* full = keys ? &k_full[s] : &v_full[s];
      if (lane == 0) bar_expect_tx(full, valid_boxes * (uint32_t)fp.box_rows * 256u);
      __syncwarp();
      if (mine) {
        uint8_t* dst = kv_smem + s * FaSmem::kStage + (keys ? 0 : FaSmem::kK);
        const uint32_t off = (uint32_t)(kind & 1) * (kKeys * 128) + (uint32_t)x * fp.box_rows * 128;
        tma_2d(dst + off, keys ? &k_map : &v_map, (kind & 1) * 64, y, full);
      }
      return true;
    };
    if constexpr (kStagesKV <= 2) {
      int y_cur = row_of(0), y_next = row_of(1);
      if (num_blocks > 0 && !fetch(0, y_cur, true)) ok = false;
      for (int b = 0; b < num_blocks && ok; ++b) {
        const int y_after = row_of(b + 2);                       // looked up two blocks early
        if (b + 1 < num_blocks && !fetch(b + 1, y_next, true)) { ok = false; break; }
        if (!fetch(b, y_cur, false)) { ok = false; break; }
        y_cur = y_next;
        y_next = y_after;
      }
    } else {
      // a deep ring has the slack already: K and V of a block are fetched together once P V of the stage's last
      // tenant is done (measured: the split order costs 15 % on a 512-token portion after 7,680 keys)
      int y_next = row_of(0);
      for (int b = 0; b < num_blocks && ok; ++b) {
        const int s = b % kStagesKV;
        const int y = y_next;
        y_next = row_of(b + 1);
        if (b >= kStagesKV) {
          const bool freed = bar_wait(&kv_empty[s], ((b / kStagesKV) - 1) & 1);
          if (!__all_sync(0xffffffffu, freed)) {
            ok = false;
            break;
          }
        }
        const uint32_t valid_boxes = __popc(__ballot_sync(0xffffffffu, y >= 0 && kind == 0));
        if (lane == 0) {
          bar_expect_tx(&k_full[s], valid_boxes * (uint32_t)fp.box_rows * 256u);
          bar_expect_tx(&v_full[s], valid_boxes * (uint32_t)fp.box_rows * 256u);
        }
        __syncwarp();
        if (y >= 0) {
          uint8_t* dst = kv_smem + s * FaSmem::kStage + (kind < 2 ? 0 : FaSmem::kK);
          const uint32_t off = (uint32_t)(kind & 1) * (kKeys * 128) + (uint32_t)x * fp.box_rows * 128;
          tma_2d(dst + off, kind < 2 ? &k_map : &v_map, (kind & 1) * 64, y, kind < 2 ? &k_full[s] : &v_full[s]);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_s = idesc(kKeys, false), id_o = idesc(kD, true);
      const uint32_t q_addr = s_addr(q_smem);
      auto issue_scores = [&](int b) -> bool {
        const int s = b % kStagesKV;
        if (!bar_wait(&k_full[s], (b / kStagesKV) & 1)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = s_addr(kv_smem + s * FaSmem::kStage);
#pragma unroll
        for (int t = 0; t < kD / 16; ++t) {
          const uint32_t off = (t >> 2) * (kRows * 128) + (t & 3) * 32;          // half, then 32 bytes per k-step
          const uint32_t koff = (t >> 2) * (kKeys * 128) + (t & 3) * 32;
          umma(tmem + (b & 1) * 64, desc_k_major(q_addr + off), desc_k_major(k_addr + koff), id_s, t > 0 ? 1u : 0u);
        }
        umma_commit(&s_ready[b & 1]);
        umma_commit(&k_empty[s]);
        return true;
      };
      if (!bar_wait(q_full, 0)) ok = false;
      if (ok && num_blocks > 0 && !issue_scores(0)) ok = false;
      for (int b = 0; b < num_blocks && ok; ++b) {
        const int s = b % kStagesKV;
        // the next block's scores go into the other TMEM buffer; its previous tenant (block b - 1) was read
        // before p_ready(b - 1), which the previous iteration waited for
        if (b + 1 < num_blocks && !issue_scores(b + 1)) { ok = false; break; }
        // O += P V once P is in shared memory (and any rescaling of O is done) and V has landed
        if (!bar_wait(&p_ready[b & 1], (b >> 1) & 1)) { ok = false; break; }
        if (!bar_wait(&v_full[s], (b / kStagesKV) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = s_addr(kv_smem + s * FaSmem::kStage) + FaSmem::kK;
        const uint32_t p_tmem = tmem + (b & 1) * 64;      // P lies over the first half of the block's scores
#pragma unroll
        for (int t = 0; t < kKeys / 16; ++t) {
          // A = P from tensor memory: 16 keys = 8 columns; B = V: 16 keys = 16 rows of 128 bytes
          umma_a_tmem(tmem + 128, p_tmem + t * 8, desc_mn_major(v_addr + t * 16 * 128, kKeys * 128), id_o,
                      (b > 0 || t > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[b & 1]);
        umma_commit(&kv_empty[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: one query row per thread
    const int row = tid;                               // TMEM lane
    const int token_local = row / G, head_local = row - token_local * G;
    const bool live = token_local < nq;
    const int pos = tile_pos + token_local;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const float scale_log2 = p.scale * kLog2e;
    float m_ref = -CUDART_INF_F, l = 0.f;

    for (int b = 0; b < num_blocks; ++b) {
      const int s = b % kStagesKV;
      const int key0 = lo + b * kKeys;
      const int nvalid = min(kKeys, hi - key0);
      if (ok && !bar_wait(&s_ready[b & 1], (b >> 1) & 1)) ok = false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t raw[2][32];
      if (ok) {
        tmem_ld32_nowait(lane_base + (b & 1) * 64, raw[0]);
        tmem_ld32_nowait(lane_base + (b & 1) * 64 + 32, raw[1]);
        tmem_wait_ld();
      }
      // Unscaled scores stay where the load put them; masked keys become -inf.  Most blocks lie wholly below the
      // diagonal, inside the window and inside the sequence: no masks there.  The maximum is taken along four
      // independent chains (one chain of 64 dependent maxima was a quarter of the block's time).
      const bool plain = ok && nvalid == kKeys && key0 + kKeys - 1 <= tile_pos &&
                         (p.window <= 0 || key0 > tile_pos + nq - 1 - p.window);
      float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      if (plain && live) {
#pragma unroll
        for (int j = 0; j < kKeys; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(raw[j >> 5][j & 31]));
      } else {
#pragma unroll
        for (int j = 0; j < kKeys; ++j) {
          const int key = key0 + j;
          const bool visible = ok && live && j < nvalid && key <= pos && (p.window <= 0 || key > pos - p.window);
          if (!visible) raw[j >> 5][j & 31] = 0xff800000u;     // -inf
          mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(raw[j >> 5][j & 31]));
        }
      }
      const float bmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;     // the scale is positive
      // raise the reference maximum only when it pays; then O (in TMEM) and l are rescaled
      const bool raise = bmax > m_ref + kRescaleThreshold || (m_ref == -CUDART_INF_F && bmax > -CUDART_INF_F);
      if (__any_sync(0xffffffffu, raise)) {
        const float alpha = (raise && m_ref != -CUDART_INF_F) ? ex2(m_ref - bmax) : 1.f;
        if (b > 0) {
          // O must hold all earlier blocks and no MMA may be adding to it: P V of block b - 1 is done
          if (ok && !bar_wait(&pv_done[(b - 1) & 1], ((b - 1) >> 1) & 1)) ok = false;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (ok) {
#pragma unroll
            for (int c = 0; c < kD / 32; ++c) {
              uint32_t o[32];
              tmem_ld32_nowait(lane_base + 128 + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(lane_base + 128 + c * 32, o);
            }
            tmem_wait_st();
          }
        }
        if (raise) {
          l *= alpha;
          m_ref = bmax;
        }
      }
      // A row that has seen no key yet subtracts 0, so that 2^(-inf - 0) = 0 and not 2^(-inf + inf).
      const float m_sub = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      // P as bfloat16 pairs, one 32-bit column per pair, written over the first 32 score columns of this
      // thread's lane (its 64 scores are in registers by now): P V reads its A operand from tensor memory
      uint32_t packed[32];
      float part[4] = {0.f, 0.f, 0.f, 0.f};     // four chains for the row sum as well
#pragma unroll
      for (int j = 0; j < kKeys; j += 2) {
        // 2^(score * scale - m): one multiply-add; -inf stays -inf and gives 0
        const float pa = ex2(fmaf(__uint_as_float(raw[j >> 5][j & 31]), scale_log2, -m_sub));
        const float pb = ex2(fmaf(__uint_as_float(raw[(j + 1) >> 5][(j + 1) & 31]), scale_log2, -m_sub));
        part[(j >> 1) & 3] += pa + pb;
        __nv_bfloat162 h = __floats2bfloat162_rn(pa, pb);
        packed[j >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      if (ok) {
        tmem_st32(lane_base + (b & 1) * 64, packed);
        tmem_wait_st();
      }
      l += (part[0] + part[1]) + (part[2] + part[3]);
      if (nvalid < kKeys) {
        // V rows of keys past the end may hold anything (a page's tail, or nothing was loaded): zero them, or
        // 0 * NaN would poison the product.  V has to have landed first.
        if (ok && !bar_wait(&v_full[s], (b / kStagesKV) & 1)) ok = false;
        uint8_t* v_area = kv_smem + s * FaSmem::kStage + FaSmem::kK;
        for (int i = tid; i < (kKeys - nvalid) * 16; i += kRows) {
          const int r = nvalid + (i >> 4), c = i & 15;
          *reinterpret_cast<uint4*>(v_area + (c >> 3) * (kKeys * 128) + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        // generic-proxy writes must be visible to the tensor core's async-proxy reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      bar_arrive(&p_ready[b & 1]);
    }
    // O / l: the products run in order, so the last one done means all are
    if (num_blocks > 0 && ok && !bar_wait(&pv_done[(num_blocks - 1) & 1], ((num_blocks - 1) >> 1) & 1)) ok = false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    __nv_bfloat16* out = (__nv_bfloat16*)p.out + ((int64_t)(q0 + token_local) * NH + kvh * G + head_local) * kD;
#pragma unroll
    for (int c = 0; c < kD / 32; ++c) {
      uint32_t o[32];
      if (ok) {
        tmem_ld32_nowait(lane_base + 128 + c * 32, o);
        tmem_wait_ld();
      }
      if (ok && live) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[v * 8 + 2 * e]) * inv,
                                                      __uint_as_float(o[v * 8 + 2 * e + 1]) * inv);
            packed[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(out + c * 32 + v * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
  }
  if (!ok && lane == 0) set_status(p.status, kWaitTimeout);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ the wide form
// The same mathematics with the work shaped by three measurements: one thread issues a tcgen05.mma about every 100
// cycles whatever its size, so the MMAs should be as wide as the tensor core allows and the scores and P V should
// have an issuing thread each; and a softmax thread that owns a whole row keeps the tensor core waiting.  One CTA
// per SM with all of its tensor memory: blocks of 128 keys (S = Q K^T is eight MMAs of 128 columns per block
// instead of sixteen of 64), two score buffers of 128 columns, eight softmax warps (warps w and w + 4 share the
// TMEM lanes 32 (w % 4) .. + 31 and take keys 0-63 and 64-127 of each block: per block a thread still handles 64
// scores, but two blocks' worth of keys; the halves' maxima and sums meet through shared memory at a named
// barrier of 64 threads), warp 8 copies (K of a stage released as soon as its scores are computed, V after P V),
// warp 9 issues the scores, warp 10 issues P V.
constexpr int kWideKeys = 128;
constexpr int kWideSoftmax = 256;
constexpr int kWideThreads = kWideSoftmax + 96;      // + the copy warp and the two issuing warps
constexpr int kWideStages = 2;
struct FaWideSmem {
  static constexpr int kQ = 2 * kRows * 128;
  static constexpr int kK = 2 * kWideKeys * 128;
  static constexpr int kStage = 2 * kK;
  static constexpr int kBars = (1 + 4 * kWideStages + 2 + 2 + 2) * 8;
  static constexpr int kExchange = 2 * 2 * kRows * 4;      // [block parity][half][row]: maxima, at the end sums
  static constexpr int kBytes = kQ + kWideStages * kStage + kBars + 16 + kExchange + 1024;
};
__device__ __forceinline__ void pair_sync(int id) { asm volatile("barrier.cta.sync %0, 64;" ::"r"(id) : "memory"); }

__global__ void __launch_bounds__(kWideThreads, 1)
attention_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                              const __grid_constant__ CUtensorMap v_map, FaParams fp) {
  using FaSmem = FaWideSmem;
  constexpr int kStagesKV = kWideStages;
  const PagedAttentionParams& p = fp.p;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + FaSmem::kQ;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(kv_smem + kStagesKV * FaSmem::kStage);
  uint64_t* k_full = q_full + 1;                 // [stages]
  uint64_t* v_full = k_full + kStagesKV;         // [stages]
  uint64_t* k_empty = v_full + kStagesKV;        // [stages] the scores of the stage's block are computed: K may go
  uint64_t* kv_empty = k_empty + kStagesKV;      // [stages] P V of the stage's block is done: V may go
  uint64_t* s_ready = kv_empty + kStagesKV;      // [2] scores of a block are in TMEM buffer (block & 1)
  uint64_t* p_ready = s_ready + 2;               // [2] P of a block is in tensor memory: 256 arrivals
  uint64_t* pv_done = p_ready + 2;               // [2] O holds the sum through block j: barrier (j & 1), phase (j >> 1)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_done + 2);
  float* exchange = reinterpret_cast<float*>(tmem_holder + 4);      // [2][2][128]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.num_heads / p.num_kv_heads, NH = p.num_heads, P = p.page_size;
  const int kvh = blockIdx.y;
  constexpr uint32_t kTmemCols = 512;            // S: columns 0-127 and 128-255, O: columns 256-383
  constexpr int kCopyWarp = 8, kScoreWarp = 9, kPvWarp = 10;

  pdl_launch_dependents();
  // CTAs start in index order and a sequence's later tiles see more keys: walk the tiles backwards, longest first
  const int slot = blockIdx.x / fp.subtiles, sub = blockIdx.x - slot * fp.subtiles;
  const int batch_tile = (int)(gridDim.x / fp.subtiles) - 1 - slot;
  const int seq = p.tile_seq[batch_tile];
  const int q0 = p.tile_q0[batch_tile] + fp.tq * sub;
  const int nq = min(fp.tq, p.tile_nq[batch_tile] - fp.tq * sub);
  if (nq <= 0) return;
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  const int tile_pos = ctx - q_len + (q0 - seq_q0);
  int lo = p.window > 0 ? max(0, tile_pos - p.window + 1) : 0;
  lo = lo / fp.box_rows * fp.box_rows;
  const int hi = tile_pos + nq;
  const int num_blocks = (hi - lo + kWideKeys - 1) / kWideKeys;

  if (tid == 0) {
    bar_init(q_full, 1);
    for (int s = 0; s < kStagesKV; ++s) {
      bar_init(&k_full[s], 1);
      bar_init(&v_full[s], 1);
      bar_init(&k_empty[s], 1);
      bar_init(&kv_empty[s], 1);
    }
    bar_init(&s_ready[0], 1);
    bar_init(&s_ready[1], 1);
    bar_init(&p_ready[0], kWideSoftmax);
    bar_init(&p_ready[1], kWideSoftmax);
    bar_init(&pv_done[0], 1);
    bar_init(&pv_done[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kScoreWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_holder)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_holder;
  pdl_wait();      // q and this step's K/V pages come from the previous kernels
  bool ok = true;

  if (warp == kCopyWarp) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bar_expect_tx(q_full, 2u * (uint32_t)(fp.tq * G) * 128u);
      tma_3d(q_smem, &q_map, 0, kvh * G, q0, q_full);
      tma_3d(q_smem + kRows * 128, &q_map, 64, kvh * G, q0, q_full);
    }
    const int32_t* table = p.block_table + (int64_t)seq * p.table_width;
    // one copy per lane: lane = 4 * box + kind, kind = K low half, K high half, V low half, V high half
    const int boxes = kWideKeys / fp.box_rows;
    const int x = lane >> 2, kind = lane & 3;
    auto row_of = [&](int blk) -> int {       // first cache row of this lane's box in block blk, -1: no box
      const int key = lo + blk * kWideKeys + x * fp.box_rows;
      if (blk >= num_blocks || x >= boxes || key >= hi) return -1;
      const int logical = key / P;
      int page = logical < p.table_width ? table[logical] : -1;
      if (page < 0 || page >= p.num_pages) {
        set_status(p.status, kBadPage);
        page = 0;     // keep the byte count honest; the result is flagged
      }
      return (page * p.num_kv_heads + kvh) * P + key % P;
    };
    auto fetch = [&](int blk, int y, bool keys) -> bool {      // this lane's copies of K or V of block blk
      const int s = blk % kStagesKV;
      if (blk >= kStagesKV) {
        const bool freed = bar_wait(keys ? &k_empty[s] : &kv_empty[s], ((blk / kStagesKV) - 1) & 1);
        if (!__all_sync(0xffffffffu, freed)) return false;       // the warp decides together: it votes below
      }
      const bool mine = y >= 0 && (kind < 2) == keys;
      const uint32_t valid_boxes = __popc(__ballot_sync(0xffffffffu, y >= 0 && kind == 0));
      uint64_t* full = keys ? &k_full[s] : &v_full[s];
      if (lane == 0) bar_expect_tx(full, valid_boxes * (uint32_t)fp.box_rows * 256u);
      __syncwarp();
      if (mine) {
        uint8_t* dst = kv_smem + s * FaSmem::kStage + (keys ? 0 : FaSmem::kK);
        const uint32_t off = (uint32_t)(kind & 1) * (kWideKeys * 128) + (uint32_t)x * fp.box_rows * 128;
        tma_2d(dst + off, keys ? &k_map : &v_map, (kind & 1) * 64, y, full);
      }
      return true;
    };
    int y_cur = row_of(0), y_next = row_of(1);
    if (num_blocks > 0 && !fetch(0, y_cur, true)) ok = false;
    for (int b = 0; b < num_blocks && ok; ++b) {
      const int y_after = row_of(b + 2);                       // looked up two blocks early
      if (b + 1 < num_blocks && !fetch(b + 1, y_next, true)) { ok = false; break; }
      if (!fetch(b, y_cur, false)) { ok = false; break; }
      y_cur = y_next;
      y_next = y_after;
    }
  } else if (warp == kScoreWarp) {
    // ---------------------------------------------------------------- MMA issuer: scores
    if (lane == 0) {
      constexpr uint32_t id_s = idesc(kWideKeys, false);
      const uint32_t q_addr = s_addr(q_smem);
      if (!bar_wait(q_full, 0)) ok = false;
      for (int b = 0; b < num_blocks && ok; ++b) {
        const int s = b % kStagesKV;
        // the scores of block b go into buffer b & 1, where P of block b - 2 lay: P V of that block must be done
        if (b >= 2 && !bar_wait(&pv_done[b & 1], ((b - 2) >> 1) & 1)) { ok = false; break; }
        if (!bar_wait(&k_full[s], (b / kStagesKV) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = s_addr(kv_smem + s * FaSmem::kStage);
#pragma unroll
        for (int t = 0; t < kD / 16; ++t) {
          const uint32_t off = (t >> 2) * (kRows * 128) + (t & 3) * 32;          // half, then 32 bytes per k-step
          const uint32_t koff = (t >> 2) * (kWideKeys * 128) + (t & 3) * 32;
          umma(tmem + (b & 1) * kWideKeys, desc_k_major(q_addr + off), desc_k_major(k_addr + koff), id_s, t > 0 ? 1u : 0u);
        }
        umma_commit(&s_ready[b & 1]);
        umma_commit(&k_empty[s]);
      }
    }
  } else if (warp == kPvWarp) {
    // ---------------------------------------------------------------- MMA issuer: O += P V
    if (lane == 0) {
      constexpr uint32_t id_o = idesc(kD, true);
      for (int b = 0; b < num_blocks && ok; ++b) {
        const int s = b % kStagesKV;
        // once P is in tensor memory (and any rescaling of O is done) and V has landed
        if (!bar_wait(&p_ready[b & 1], (b >> 1) & 1)) { ok = false; break; }
        if (!bar_wait(&v_full[s], (b / kStagesKV) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = s_addr(kv_smem + s * FaSmem::kStage) + FaSmem::kK;
        const uint32_t p_tmem = tmem + (b & 1) * kWideKeys;      // P lies over the first half of the block's scores
#pragma unroll
        for (int t = 0; t < kWideKeys / 16; ++t) {
          // A = P from tensor memory: 16 keys = 8 columns; B = V: 16 keys = 16 rows of 128 bytes
          umma_a_tmem(tmem + 256, p_tmem + t * 8, desc_mn_major(v_addr + t * 16 * 128, kWideKeys * 128), id_o,
                      (b > 0 || t > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[b & 1]);
        umma_commit(&kv_empty[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: two threads per query row
    const int half = warp >> 2;                        // which 64 of a block's 128 keys
    const int row = (warp & 3) * 32 + lane;            // TMEM lane
    const int pair_bar = 1 + (warp & 3);               // the named barrier of this warp and its partner
    const int token_local = row / G, head_local = row - token_local * G;
    const bool live = token_local < nq;
    const int pos = tile_pos + token_local;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float scale_log2 = p.scale * kLog2e;
    float m_ref = -CUDART_INF_F, l = 0.f;              // l: this half's share of the row sum

    for (int b = 0; b < num_blocks; ++b) {
      const int s = b % kStagesKV;
      const int key0 = lo + b * kWideKeys + half * 64;      // this thread's first key of the block
      const int nvalid_block = min(kWideKeys, hi - (lo + b * kWideKeys));
      const int nvalid = max(0, min(64, nvalid_block - half * 64));
      if (ok && !bar_wait(&s_ready[b & 1], (b >> 1) & 1)) ok = false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t raw[2][32];
      if (ok) {
        tmem_ld32_nowait(lane_base + (b & 1) * kWideKeys + half * 64, raw[0]);
        tmem_ld32_nowait(lane_base + (b & 1) * kWideKeys + half * 64 + 32, raw[1]);
        tmem_wait_ld();
      }
      const bool plain = ok && nvalid == 64 && key0 + 63 <= tile_pos &&
                         (p.window <= 0 || key0 > tile_pos + nq - 1 - p.window);
      float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      if (plain && live) {
#pragma unroll
        for (int j = 0; j < 64; ++j) mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(raw[j >> 5][j & 31]));
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int key = key0 + j;
          const bool visible = ok && live && j < nvalid && key <= pos && (p.window <= 0 || key > pos - p.window);
          if (!visible) raw[j >> 5][j & 31] = 0xff800000u;     // -inf
          mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(raw[j >> 5][j & 31]));
        }
      }
      // the row's maximum over the block: this half's and the partner's, through shared memory.  Both have their
      // scores in registers once they meet, so either may then write P over the other's score columns.
      float* xmax = exchange + (b & 1) * 2 * kRows;
      const float hmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;     // the scale is positive
      xmax[half * kRows + row] = hmax;
      pair_sync(pair_bar);
      const float bmax = fmaxf(hmax, xmax[(half ^ 1) * kRows + row]);
      // raise the reference maximum only when it pays; then O (in TMEM) and l are rescaled.  Both halves of a row
      // see the same bmax and m_ref, so they decide alike; each rescales its 64 of the row's 128 columns of O.
      const bool raise = bmax > m_ref + kRescaleThreshold || (m_ref == -CUDART_INF_F && bmax > -CUDART_INF_F);
      if (__any_sync(0xffffffffu, raise)) {
        const float alpha = (raise && m_ref != -CUDART_INF_F) ? ex2(m_ref - bmax) : 1.f;
        if (b > 0) {
          // O must hold all earlier blocks and no MMA may be adding to it: P V of block b - 1 is done
          if (ok && !bar_wait(&pv_done[(b - 1) & 1], ((b - 1) >> 1) & 1)) ok = false;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (ok) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {      // 16 columns at a time: the block's scores are alive beside them
              uint32_t o[16];
              tmem_ld16_nowait(lane_base + 256 + half * 64 + c * 16, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st16(lane_base + 256 + half * 64 + c * 16, o);
            }
            tmem_wait_st();
          }
        }
        if (raise) {
          l *= alpha;
          m_ref = bmax;
        }
      }
      // A row that has seen no key yet subtracts 0, so that 2^(-inf - 0) = 0 and not 2^(-inf + inf).
      const float m_sub = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      // P as bfloat16 pairs, one 32-bit column per pair: this half's 64 keys are columns 32 half .. + 31 of the
      // block's score buffer (P of the whole block lies over the first 64 score columns)
      uint32_t packed[32];
      float part[4] = {0.f, 0.f, 0.f, 0.f};     // four chains for the row sum as well
#pragma unroll
      for (int j = 0; j < 64; j += 2) {
        const float pa = ex2(fmaf(__uint_as_float(raw[j >> 5][j & 31]), scale_log2, -m_sub));
        const float pb = ex2(fmaf(__uint_as_float(raw[(j + 1) >> 5][(j + 1) & 31]), scale_log2, -m_sub));
        part[(j >> 1) & 3] += pa + pb;
        __nv_bfloat162 h = __floats2bfloat162_rn(pa, pb);
        packed[j >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      if (ok) {
        tmem_st32(lane_base + (b & 1) * kWideKeys + half * 32, packed);
        tmem_wait_st();
      }
      l += (part[0] + part[1]) + (part[2] + part[3]);
      if (nvalid_block < kWideKeys) {
        // V rows of keys past the end may hold anything (a page's tail, or nothing was loaded): zero them, or
        // 0 * NaN would poison the product.  V has to have landed first.
        if (ok && !bar_wait(&v_full[s], (b / kStagesKV) & 1)) ok = false;
        uint8_t* v_area = kv_smem + s * FaSmem::kStage + FaSmem::kK;
        for (int i = tid; i < (kWideKeys - nvalid_block) * 16; i += kWideSoftmax) {
          const int r = nvalid_block + (i >> 4), c = i & 15;
          *reinterpret_cast<uint4*>(v_area + (c >> 3) * (kWideKeys * 128) + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
        // generic-proxy writes must be visible to the tensor core's async-proxy reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      bar_arrive(&p_ready[b & 1]);
    }
    // the row sum: this half's share and the partner's, first half first
    float* xsum = exchange + (num_blocks & 1) * 2 * kRows;
    xsum[half * kRows + row] = l;
    pair_sync(pair_bar);
    l = xsum[row] + xsum[kRows + row];
    // O / l: the products run in order, so the last one done means all are
    if (num_blocks > 0 && ok && !bar_wait(&pv_done[(num_blocks - 1) & 1], ((num_blocks - 1) >> 1) & 1)) ok = false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    __nv_bfloat16* out = (__nv_bfloat16*)p.out + ((int64_t)(q0 + token_local) * NH + kvh * G + head_local) * kD +
                         half * 64;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t o[32];
      if (ok) {
        tmem_ld32_nowait(lane_base + 256 + half * 64 + c * 32, o);
        tmem_wait_ld();
      }
      if (ok && live) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[v * 8 + 2 * e]) * inv,
                                                      __uint_as_float(o[v * 8 + 2 * e + 1]) * inv);
            packed[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(out + c * 32 + v * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
  }
  if (!ok && lane == 0) set_status(p.status, kWaitTimeout);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kScoreWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

bool encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
            const cuuint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct MapCache {
  std::mutex mutex;
  std::map<std::tuple<const void*, int64_t, int, int>, CUtensorMap> maps;
};

// [rows, 128] bfloat16 cache tensor: boxes of 64 columns by box_rows rows
bool cache_map(const void* base, int64_t rows, int box_rows, CUtensorMap* out) {
  static MapCache cache;
  std::lock_guard<std::mutex> guard(cache.mutex);
  const auto key = std::make_tuple(base, rows, box_rows, 0);
  auto it = cache.maps.find(key);
  if (it != cache.maps.end()) { *out = it->second; return true; }
  const cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kD * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  CUtensorMap map;
  if (!encode(&map, base, 2, dims, strides, box)) return false;
  cache.maps[key] = map;
  *out = map;
  return true;
}

// q [tokens, heads, 128]: boxes of 64 dims x G heads x tq tokens, so a tile's rows come out in (token, head) order
bool q_map_for(const void* base, int64_t tokens, int heads, int group, int tq, CUtensorMap* out) {
  static MapCache cache;
  std::lock_guard<std::mutex> guard(cache.mutex);
  const auto key = std::make_tuple(base, tokens, heads, group * 1000 + tq);
  auto it = cache.maps.find(key);
  if (it != cache.maps.end()) { *out = it->second; return true; }
  const cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)heads, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)heads * kD * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)tq};
  CUtensorMap map;
  if (!encode(&map, base, 3, dims, strides, box)) return false;
  if (cache.maps.size() > 4096) cache.maps.clear();
  cache.maps[key] = map;
  *out = map;
  return true;
}

}  // namespace

// Prompt portions, bfloat16, head size 128, groups of 1 to 16 q-heads, pages of 16 tokens or more (a power of
// two).  AKV_PROMPT_KERNEL=mma keeps the mma.sync kernel (for comparisons).
bool attention_tcgen05_supported(const PagedAttentionParams& p) {
  static const bool disabled = [] {
    const char* v = getenv("AKV_PROMPT_KERNEL");
    return v != nullptr && v[0] == 'm';
  }();
  if (disabled || p.dtype != kBFloat16 || p.head_dim != kD || p.q_tile <= 1) return false;
  if (!(p.scale > 0.f)) return false;      // the kernel takes the maximum before it scales
  if (p.num_heads % p.num_kv_heads) return false;
  const int G = p.num_heads / p.num_kv_heads;
  if (G < 1 || G > 16) return false;
  if (p.page_size < 16 || (p.page_size & (p.page_size - 1))) return false;
  if (p.num_kv_heads > 65535) return false;
  return encode_fn() != nullptr;
}

namespace {
template <int kStagesKV>
int launch_stages(const CUtensorMap& q_map, const CUtensorMap& k_map, const CUtensorMap& v_map, const FaParams& fp,
                  dim3 grid, cudaStream_t stream) {
  auto kernel = attention_tcgen05_kernel<kStagesKV>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           FaSmemT<kStagesKV>::kBytes);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  return (int)launch_chain(kernel, grid, dim3(192), FaSmemT<kStagesKV>::kBytes, stream, dim3(1, 1, 1), q_map, k_map,
                           v_map, fp);
}
}  // namespace

int launch_attention_tcgen05(const PagedAttentionParams& p, cudaStream_t stream) {
  const int G = p.num_heads / p.num_kv_heads;
  const int tq = kRows / G;
  const int subtiles = (p.q_tile + tq - 1) / tq;
  const int box_rows = p.page_size < kKeys ? p.page_size : kKeys;
  const int64_t rows = p.num_pages * p.num_kv_heads * (int64_t)p.page_size;
  CUtensorMap q_map, k_map, v_map;
  if (!q_map_for(p.q, p.num_tokens, p.num_heads, G, tq, &q_map) || !cache_map(p.k_cache, rows, box_rows, &k_map) ||
      !cache_map(p.v_cache, rows, box_rows, &v_map))
    return (int)cudaErrorInvalidValue;
  FaParams fp{p, tq, subtiles, box_rows};
  const dim3 grid((unsigned)(p.num_tiles * subtiles), (unsigned)p.num_kv_heads, 1u);
  // the narrow form's ring (AKV_PROMPT_STAGES=2 | 4 forces it): two stages and two CTAs per SM when there are more
  // CTAs than SMs, else four stages and one CTA per SM
  static const int forced = [] {
    const char* v = getenv("AKV_PROMPT_STAGES");
    const int n = v ? atoi(v) : 0;
    return (n == 2 || n == 4) ? n : 0;
  }();
  // Two forms.  More CTAs than SMs: the narrow form, two CTAs per SM with two K/V stages each, whose CTAs fill
  // each other's waits.  No more CTAs than SMs (a short prompt, a portion of a long one): the wide form, one CTA
  // per SM with 128-key blocks, two threads per row and an issuing thread each for the scores and for P V.
  // Measured: a 2,048-token prompt (512 CTAs) 81 us narrow against 84 us wide, an 8,192-token prompt 826 against
  // 643 TFLOP/s; a 512-token portion after 7,680 keys (128 CTAs) 126 us wide against 148 us for the narrow form
  // with a four-stage ring, a 256-token prompt 22 against 26 us.  AKV_PROMPT_FORM=1 | 2 forces wide | narrow.
  static const int form = [] {
    const char* v = getenv("AKV_PROMPT_FORM");
    const int n = v ? atoi(v) : 0;
    return (n == 1 || n == 2) ? n : 0;
  }();
  const int sms = sm_count();
  const bool few = (int64_t)grid.x * grid.y <= sms;
  const bool wide_form = p.kernel == 4 || (p.kernel != 3 && (form == 1 || (form == 0 && few)));
  if (wide_form) {
    const int wide_rows = p.page_size < 64 ? p.page_size : 64;      // a box holds at most 64 keys (8 KB per half)
    CUtensorMap kw, vw;
    if (!cache_map(p.k_cache, rows, wide_rows, &kw) || !cache_map(p.v_cache, rows, wide_rows, &vw))
      return (int)cudaErrorInvalidValue;
    FaParams wide{p, tq, subtiles, wide_rows};
    static bool configured = false;
    if (!configured) {
      cudaError_t err = cudaFuncSetAttribute(attention_tcgen05_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             FaWideSmem::kBytes);
      if (err != cudaSuccess) return (int)err;
      configured = true;
    }
    return (int)launch_chain(attention_tcgen05_wide_kernel, grid, dim3(kWideThreads), FaWideSmem::kBytes, stream,
                             dim3(1, 1, 1), q_map, kw, vw, wide);
  }
  const bool shallow = forced ? forced == 2 : !few;
  if (shallow) return launch_stages<2>(q_map, k_map, v_map, fp, grid, stream);
  return launch_stages<4>(q_map, k_map, v_map, fp, grid, stream);
}

}  // namespace akv
