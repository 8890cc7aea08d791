// Weight-streaming bfloat16 GEMM for few tokens (decode steps), on the 5th-generation tensor cores:
//     out[t, f] = sum_k x[t, k] * w[f, k]
// The weight matrix [features, K] is the M operand (128 features per CTA), the tokens are the N operand
// (padded to 16/32/64), so every byte of weight is read exactly once by one CTA and feeds a full-width
// tcgen05.mma.  K is cut into 1/2/4/8 splits so that a thin output still occupies the whole GPU.  The CTAs of
// one output tile form a thread-block cluster: each leaves its float32 partial tile in its own shared memory,
// and after a cluster barrier the CTA of split s adds up, in split order, the tokens s, s + S, ... of the tile
// read from its peers' shared memory (distributed shared memory) and stores them, rounded once.  In that tail a
// warp owns tokens and a lane four consecutive features: the partial sums arrive as 16-byte loads, as many under
// way as the round trip (about a microsecond when every CTA reduces at once) is worth; a token's 128 features are
// one warp's, so the epilogues that work across a tile (norm over a head, rotation, the sum of squares for the
// next RMS norm) need shuffles only and no warp waits for another.  With ``parts`` instead of ``out`` the float32
// partial tiles are stored as they are, [splits, tokens, features].
//
// One CTA = 6 warps: warp 0 issues the TMA loads (128-byte swizzled tiles of 64 K-elements, a 4-stage ring
// guarded by full/empty mbarriers, no multicast), warp 1 allocates TMEM and issues tcgen05.mma (one thread,
// accumulator in TMEM, tcgen05.commit frees each stage and finally signals the epilogue), warps 2-5 read the
// accumulator with tcgen05.ld.  Two or three CTAs share an SM, so one CTA's set-up and epilogue overlap the
// others' streaming.  It replaces the library GEMMs the reference calls for its
// projections (ampere_kv/runner.py:64-66, 165, 174-177, 297) for up to 64 tokens; larger batches (prompts) stay
// on the library GEMM.
//
// Every wait is bounded; a wait that runs out sets kWaitTimeout in the status word, and the CTA still frees
// its TMEM and leaves.
#include "common.cuh"
#include "launchers.h"
#include "tensor_map.h"

#include <cuda.h>
#include <stdlib.h>

#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

namespace akv {

namespace {

constexpr int kTileM = 128;      // features per CTA
constexpr int kTileK = 64;       // K elements per stage: 128 bytes, one swizzle row

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// start address, leading offset 1 (unused with this swizzle), 1024 bytes between 8-row groups, version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  desc |= (uint64_t)1 << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

// Instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
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

struct GemmParams {
  float* parts;        // [splits, tokens, features] float32 partial tiles, or null
  void* out;           // [tokens, features] in OutT (cluster reduction), or null
  int tokens, features, k;
  int kb_total;        // K blocks of 64 in all
  int splits;
  int* status;
  GemmQkv qkv;            // kEpilogueQkv only
  GemmResidual residual;  // kEpilogueResidual only
  GemmNormedX normed;     // kNormedX only
};

template <int BN, int kStages>
struct GemmSmem {
  static constexpr int kA = kTileM * kTileK * 2;
  static constexpr int kB = BN * kTileK * 2;
  static constexpr int kStage = kA + kB;
  static constexpr int kReduce = BN * kTileM * 4;                      // float32 partial tile, reuses the stages
  static_assert(kReduce <= kStages * kStage, "the partial tile must fit in the stage ring");
  static constexpr int kBars = (2 * kStages + 1) * 8 + 16;             // barriers, TMEM base
  static constexpr int kBytes = kStages * kStage + kBars + 64 * 4 + 1024;   // + inverse RMS per token (kNormedX)
};

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// The meeting before a CTA leaves: it only has to know that its neighbours have read its shared memory (their
// loads are complete when they arrive, since they have used the values).  Nothing is published, so the arrival does
// not wait for this CTA's own global stores as a releasing arrival does.
__device__ __forceinline__ void cluster_meet_to_leave() {
  asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
  asm volatile("barrier.cluster.wait;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Sums over the cluster's CTAs (one per K split, in split order) of kPlaces groups of four consecutive floats of
// the partial tiles, every load issued before the first is used: ONE round trip through distributed shared
// memory (about a microsecond when all CTAs reduce at once).  offset[i] is the group's byte offset in the partial
// tile (a multiple of 16), or kNoPlace.
constexpr uint32_t kNoPlace = 0xffffffffu;
template <int kPlaces, int S>
__device__ __forceinline__ void gather_sums(uint32_t tile_addr, const uint32_t (&offset)[kPlaces], float4 (&sum)[kPlaces]) {
  uint32_t peer[S];
#pragma unroll
  for (int s = 0; s < S; ++s)
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[s]) : "r"(tile_addr), "r"((uint32_t)s));
  float4 v[kPlaces][S];
#pragma unroll
  for (int i = 0; i < kPlaces; ++i)
#pragma unroll
    for (int s = 0; s < S; ++s) {
      v[i][s] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (offset[i] != kNoPlace)
        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v[i][s].x), "=f"(v[i][s].y), "=f"(v[i][s].z), "=f"(v[i][s].w)
                     : "r"(peer[s] + offset[i])
                     : "memory");
    }
#pragma unroll
  for (int i = 0; i < kPlaces; ++i) {
    sum[i] = v[i][0];
#pragma unroll
    for (int s = 1; s < S; ++s) {
      sum[i].x += v[i][s].x;
      sum[i].y += v[i][s].y;
      sum[i].z += v[i][s].z;
      sum[i].w += v[i][s].w;
    }
  }
}

// (sin a, cos a, sin b, cos b).  Not inlined: the epilogue needs it in two places, and its code is long.
__device__ __noinline__ float4 sincos_pair(float a, float b) {
  float4 r;
  sincosf(a, &r.x, &r.y);
  sincosf(b, &r.z, &r.w);
  return r;
}
// Sines and cosines of a token's rotation for the four dims of each lane (dims 4 * lane + i, frequencies
// 4 * (lane & 15) + i): lane j computes the angles of frequencies 2j and 2j + 1 (`freq2`), the lanes that need
// them fetch them from there, so that a warp computes each of the head's 64 angles once.
__device__ __forceinline__ void rotation_of(float pos, float2 freq2, float4* sn, float4* co) {
  const float4 mine = sincos_pair(pos * freq2.x, pos * freq2.y);
  const int src = 2 * (threadIdx.x & 15);
  sn->x = __shfl_sync(0xffffffffu, mine.x, src);
  co->x = __shfl_sync(0xffffffffu, mine.y, src);
  sn->y = __shfl_sync(0xffffffffu, mine.z, src);
  co->y = __shfl_sync(0xffffffffu, mine.w, src);
  sn->z = __shfl_sync(0xffffffffu, mine.x, src + 1);
  co->z = __shfl_sync(0xffffffffu, mine.y, src + 1);
  sn->w = __shfl_sync(0xffffffffu, mine.z, src + 1);
  co->w = __shfl_sync(0xffffffffu, mine.w, src + 1);
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int BN, typename OutT, int kStages, int kEpilogue, bool kNormedX>
__global__ void __launch_bounds__(192, 3)
small_m_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                    GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * GemmSmem<BN, kStages>::kStage);
  uint64_t* empty = full + kStages;
  uint64_t* acc_ready = empty + kStages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_ready + 1);
  float* inv_rms = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(acc_ready) + 8 + 16);     // [64], kNormedX
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;

  // this split's K blocks: an even share, the first (kb_total % splits) splits take one more
  const int base = p.kb_total / p.splits, extra = p.kb_total % p.splits;
  const int kb_begin = split * base + min(split, extra);
  const int num_kb = base + (split < extra ? 1 : 0);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], kNormedX ? 2 : 1);     // the TMA issuer, and the warp that writes the token tile
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  bool ok = true;
  // In the tail a warp owns tokens and a lane four consecutive features of the tile (rows 4 * lane .. + 3).  Fetched
  // ahead of the product, kEpilogueQkv: the norm weights and rotation frequencies of the lane's dims, position and
  // cache slot of the warp's tokens (lane i holds those of the warp's i-th token), sine and cosine for its first.
  float4 qkv_w = make_float4(1.f, 1.f, 1.f, 1.f);
  float2 qkv_f = make_float2(0.f, 0.f);      // rotation frequencies 2 * lane and 2 * lane + 1
  float4 qkv_sn = make_float4(0.f, 0.f, 0.f, 0.f), qkv_co = make_float4(1.f, 1.f, 1.f, 1.f);
  int qkv_pos = 0;
  int64_t qkv_slot = -1;
  float4 res_old = make_float4(0.f, 0.f, 0.f, 0.f);     // kEpilogueResidual: the stream's old values, first token

  if (warp == 0) {
    // The weights do not depend on the kernel before this one: fill the ring's weight halves first, then wait
    // for that kernel and fetch the activations.  (kNormedX: warps 2-5 make the token tiles.)  The first copies
    // are issued by one lane per stage, side by side: a thread spends about 100 ns on each copy it issues, and
    // the activation copies come after the wait, where that time is not hidden.
    constexpr uint32_t kTxBytes = kNormedX ? GemmSmem<BN, kStages>::kA : GemmSmem<BN, kStages>::kStage;
    const int ahead = min(num_kb, kStages);
    if (lane < ahead) {
      mbar_expect_tx(&full[lane], kTxBytes);
      tma_load_2d(smem + lane * GemmSmem<BN, kStages>::kStage, &w_map, (kb_begin + lane) * kTileK, tile * kTileM, &full[lane]);
    }
    if constexpr (!kNormedX) {
      pdl_wait();
      if (lane < ahead)
        tma_load_2d(smem + lane * GemmSmem<BN, kStages>::kStage + GemmSmem<BN, kStages>::kA, &x_map,
                    (kb_begin + lane) * kTileK, 0, &full[lane]);
    }
    __syncwarp();
    if (lane == 0) {
      for (int kb = ahead; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait(&empty[s], ((kb / kStages) - 1) & 1)) {
          ok = false;
          break;
        }
        uint8_t* stage = smem + s * GemmSmem<BN, kStages>::kStage;
        mbar_expect_tx(&full[s], kTxBytes);
        const int k0 = (kb_begin + kb) * kTileK;
        tma_load_2d(stage, &w_map, k0, tile * kTileM, &full[s]);
        if constexpr (!kNormedX) tma_load_2d(stage + GemmSmem<BN, kStages>::kA, &x_map, k0, 0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait(&full[s], (kb / kStages) & 1)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(smem + s * GemmSmem<BN, kStages>::kStage);
        const uint32_t b_addr = a_addr + GemmSmem<BN, kStages>::kA;
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          // 16 K-elements = 32 bytes further along the swizzled row
          umma_bf16(tmem_base, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc,
                    (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);     // arrives once these MMAs have read the stage
      }
      if (ok) umma_commit(acc_ready);
    }
  } else {
    // epilogue: warp (2..5) reads the TMEM lanes of its quarter; lane = feature, column = token
    const int quarter = warp & 3;
    if constexpr (kNormedX) {
      // The token operand is the RMS norm of the residual stream, made here: x = hidden * inv_rms * weight,
      // rounded to bfloat16 and laid out as the TMA would (rows of 128 bytes, 16-byte chunk c of row r at
      // c ^ (r & 7)).  Warp q makes the K blocks kb = q, q + 4, ...: up to four blocks are under way at a time.
      const GemmNormedX& nx = p.normed;
      // A stage must always be written by the same warp, so that the warp sees each of the stage's "empty" phases
      // in turn (a parity wait two phases late answers wrongly): with three stages three warps work.
      constexpr int kXWarps = kStages < 4 ? kStages : 4;
      // The product cannot start before its first token tiles exist, and they wait for two things from memory one
      // after the other: the sums of squares (for the scale), then the rows.  With few tokens (two 16-byte pieces
      // of a tile per lane, both of the same 8 K elements) a warp fetches the rows of its first K block together
      // with the sums of squares, and the norm weights, which are the model's, before it waits for the previous
      // kernel at all.  (Fetching the rows of its second block as well was measured slower: 3.41 against 3.29 ms
      // a step at batch 8.)
      const bool pre = p.tokens * 8 <= 64 && quarter < kXWarps && quarter < num_kb;
      float pre_h[2][8], pre_w[8];
      auto piece_k0 = [&](int kb, int task) { return (kb_begin + kb) * kTileK + (task & 7) * 8; };
      if (pre && piece_k0(quarter, lane) < p.k) load8<float>(nx.weight + piece_k0(quarter, lane), pre_w);
      pdl_wait();      // hidden and its sums of squares come from the kernels before this one
      if (pre) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int task = lane + 32 * j;
          if (task < p.tokens * 8 && piece_k0(quarter, task) < p.k)
            load8<float>(nx.hidden + (int64_t)(task >> 3) * p.k + piece_k0(quarter, task), pre_h[j]);
        }
      }
      // a warp per token, a lane per tile: the partial sums of a token arrive in one round trip (one thread adding
      // a token's 32 tiles up in turn waited for each load)
      for (int t = quarter; t < p.tokens; t += 4) {
        float ss = 0.f;
        for (int i = lane; i < nx.ssq_tiles; i += 32) ss += nx.ssq[(int64_t)i * p.tokens + t];
        ss = warp_sum(ss);
        if (lane == 0) inv_rms[t] = rsqrtf(ss / (float)p.k + nx.eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // x = hidden * inv_rms * weight of one 16-byte piece (token r, 8 K elements), rounded, to its swizzled place
      auto put = [&](uint8_t* x_tile, int task, const float (&h)[8], const float (&w)[8], bool inside) {
        const int r = task >> 3, c = task & 7;
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);       // past the end of K: zeros (the weights' are zeros too)
        if (inside) {
          const float inv = inv_rms[r];
          uint32_t u[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 v = __floats2bfloat162_rn(h[2 * e] * inv * w[2 * e], h[2 * e + 1] * inv * w[2 * e + 1]);
            u[e] = *reinterpret_cast<uint32_t*>(&v);
          }
          packed = make_uint4(u[0], u[1], u[2], u[3]);
        }
        *reinterpret_cast<uint4*>(x_tile + r * 128 + ((c ^ (r & 7)) << 4)) = packed;
      };
      for (int kb = quarter; quarter < kXWarps && kb < num_kb && ok; kb += kXWarps) {
        const int s = kb % kStages;
        if (kb >= kStages && !mbar_wait(&empty[s], ((kb / kStages) - 1) & 1)) {
          ok = false;
          break;
        }
        uint8_t* x_tile = smem + s * GemmSmem<BN, kStages>::kStage + GemmSmem<BN, kStages>::kA;
        if (pre && kb == quarter) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int task = lane + 32 * j;
            if (task < p.tokens * 8) put(x_tile, task, pre_h[j], pre_w, piece_k0(kb, task) < p.k);
          }
        } else {
          // a lane's pieces of a tile are all of the same 8 K elements (32 is a multiple of 8): one fetch of the
          // norm weights, and the rows of four pieces under way at a time (one piece at a time paid a round trip
          // to the L2 per piece: with 16 tokens four in a row per tile)
          const int k0 = piece_k0(kb, lane);
          const bool inside = k0 < p.k;
          float w[8];
          if (inside) load8<float>(nx.weight + k0, w);
#pragma unroll 1
          for (int base = lane; base < p.tokens * 8; base += 4 * 32) {
            float h[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int task = base + 32 * j;
              if (inside && task < p.tokens * 8) load8<float>(nx.hidden + (int64_t)(task >> 3) * p.k + k0, h[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int task = base + 32 * j;
              if (task < p.tokens * 8) put(x_tile, task, h[j], w, inside);
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
      }
    }
    if constexpr (kEpilogue == kEpilogueQkv) {
      // while the product runs (and after this warp's part in making the token operand, which the product waits
      // for): what the tail needs besides the product.  None of it comes from the previous kernel.
      const GemmQkv& e = p.qkv;
      const bool is_q = tile < e.num_heads, is_k = !is_q && tile < e.num_heads + e.num_kv_heads;
      const float* w = is_q ? e.q_weight : (is_k ? e.k_weight : nullptr);
      if (w != nullptr) qkv_w = *reinterpret_cast<const float4*>(w + 4 * lane);
      const bool rotate = (is_q || is_k) && e.inv_freq != nullptr;
      if (rotate) qkv_f = *reinterpret_cast<const float2*>(e.inv_freq + 2 * lane);
      const int mine = split + (quarter + 4 * lane) * p.splits;       // the warp's lane-th token
      if (mine < p.tokens) {
        qkv_pos = e.positions[mine];
        if (!is_q && e.slots != nullptr) qkv_slot = e.slots[mine];
      }
      if (rotate && split + quarter * p.splits < p.tokens)      // the warp has a first token
        rotation_of((float)__shfl_sync(0xffffffffu, qkv_pos, 0), qkv_f, &qkv_sn, &qkv_co);
    }
    if constexpr (kEpilogue == kEpilogueResidual) {
      // the residual stream's old values for the warp's first token, fetched while the product runs
      if constexpr (!kNormedX) pdl_wait();
      const int token = split + quarter * p.splits, feature = tile * kTileM + 4 * lane;
      if (token < p.tokens && (p.features & 3) == 0 && feature < p.features)
        res_old = *reinterpret_cast<const float4*>(p.residual.hidden + (int64_t)token * p.features + feature);
    }
    // The tail runs once per CTA: its loops over token columns are not unrolled further than they must be (measured:
    // fetching the instructions of a fully unrolled copy of 64 columns took 4 us, executing them 0.5 us).
    const int row = quarter * 32 + lane;
    const int feature = tile * kTileM + row;
    float* reduce = reinterpret_cast<float*>(smem);     // [token][128 features]; the stages are drained by then
    float* part_out = p.parts ? p.parts + (int64_t)split * p.tokens * p.features : nullptr;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    if (!mbar_wait(acc_ready, 0)) ok = false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
      // accumulator -> shared memory (or the caller's partial tiles), 16 token columns at a time
#pragma unroll 1
      for (int c = 0; c < BN / 16; ++c) {
        uint32_t v[16];
        if (ok) {
          tmem_load16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16, v);
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) v[t] = 0u;
        }
        if (part_out) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const int token = c * 16 + t;
            if (token < p.tokens && feature < p.features)
              part_out[(int64_t)token * p.features + feature] = __uint_as_float(v[t]);
          }
        } else {
          float* dst = reduce + c * 16 * kTileM + row;
#pragma unroll
          for (int t = 0; t < 16; ++t) dst[t * kTileM] = __uint_as_float(v[t]);
        }
      }
    }
    if (!ok) set_status(p.status, kWaitTimeout);
    if (p.out != nullptr) {
      // every CTA of the tile has its partial in shared memory: add them up across the cluster, in split order
      cluster_sync_all();
      const uint32_t tile_addr = smem_u32(smem);
      // This CTA owns the tokens split, split + S, ...; warp w of the four takes the w-th, (w + 4)-th, ... of them,
      // U at a time with U * S loads of 16 bytes under way, and a lane four consecutive features: a token's 128
      // features are one warp's, so the norm over a head and the sum of squares are warp sums, the rotation's
      // partner dim (+-64) sits 16 lanes away, and no warp waits for another.
      auto tail = [&](auto splits_tag) {
        constexpr int S = decltype(splits_tag)::value;
        constexpr int U = 8 / S;
        [[maybe_unused]] const int feature = tile * kTileM + 4 * lane;      // the lane's first feature
        [[maybe_unused]] const bool whole = (p.features & 3) == 0;          // output rows start on 16-byte boundaries
        int round = 0;
#pragma unroll 1
        for (int o = quarter; split + o * S < p.tokens; o += 4 * U, ++round) {
          uint32_t off[U];
          float4 sum[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int tok = split + (o + 4 * u) * S;
            off[u] = tok < p.tokens ? (uint32_t)(tok * kTileM + 4 * lane) * 4u : kNoPlace;
          }
          gather_sums<U, S>(tile_addr, off, sum);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int tok = split + (o + 4 * u) * S;
            if (tok >= p.tokens) break;
            const float4 v = sum[u];
            if constexpr (kEpilogue == kEpilogueGated) {
              // rows 0-63 of the tile are gate rows, rows 64-127 the up rows of the same 64 outputs: lanes 0-15
              // hold four gates each, lane + 16 the four ups that go with them
              const float u0 = __shfl_xor_sync(0xffffffffu, v.x, 16), u1 = __shfl_xor_sync(0xffffffffu, v.y, 16);
              const float u2 = __shfl_xor_sync(0xffffffffu, v.z, 16), u3 = __shfl_xor_sync(0xffffffffu, v.w, 16);
              const int out_features = p.features / 2;
              const int gated_feature = tile * (kTileM / 2) + 4 * lane;
              if (lane < 16 && gated_feature < out_features) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(silu_mul_value<OutT>(bf16_round(v.x), bf16_round(u0)),
                                                          silu_mul_value<OutT>(bf16_round(v.y), bf16_round(u1)));
                __nv_bfloat162 hi = __floats2bfloat162_rn(silu_mul_value<OutT>(bf16_round(v.z), bf16_round(u2)),
                                                          silu_mul_value<OutT>(bf16_round(v.w), bf16_round(u3)));
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)tok * out_features + gated_feature) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
              }
            } else if constexpr (kEpilogue == kEpilogueQkv) {
              // The tile is one head of 128 dims.  The sums rounded as the stored product would be, norm over the
              // head, rotation with the partner dim, store to q_out or to the token's cache slot.
              const GemmQkv& e = p.qkv;
              const int head = tile;
              const bool is_q = head < e.num_heads, is_k = !is_q && head < e.num_heads + e.num_kv_heads;
              const int local = is_q ? head : (is_k ? head - e.num_heads : head - e.num_heads - e.num_kv_heads);
              const bool normed = (is_q ? e.q_weight : (is_k ? e.k_weight : nullptr)) != nullptr;
              const bool rotate = (is_q || is_k) && e.inv_freq != nullptr;
              float x[4] = {bf16_round(v.x), bf16_round(v.y), bf16_round(v.z), bf16_round(v.w)};
              if (normed) {
                const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
                const float inv = rsqrtf(ss / (float)kTileM + e.eps);
                x[0] *= inv * qkv_w.x;
                x[1] *= inv * qkv_w.y;
                x[2] *= inv * qkv_w.z;
                x[3] *= inv * qkv_w.w;
              }
              const int nth = round * U + u;      // this token is the warp's nth
              if (rotate) {
                float4 sn = qkv_sn, co = qkv_co;
                if (nth > 0)      // the first token's were computed while the product ran
                  rotation_of((float)__shfl_sync(0xffffffffu, qkv_pos, nth), qkv_f, &sn, &co);
                const float sign = lane < 16 ? -1.f : 1.f;      // dims below 64: x cos - partner sin
                const float p0 = __shfl_xor_sync(0xffffffffu, x[0], 16), p1 = __shfl_xor_sync(0xffffffffu, x[1], 16);
                const float p2 = __shfl_xor_sync(0xffffffffu, x[2], 16), p3 = __shfl_xor_sync(0xffffffffu, x[3], 16);
                x[0] = x[0] * co.x + sign * p0 * sn.x;
                x[1] = x[1] * co.y + sign * p1 * sn.y;
                x[2] = x[2] * co.z + sign * p2 * sn.z;
                x[3] = x[3] * co.w + sign * p3 * sn.w;
              }
              __nv_bfloat16* dst = nullptr;
              if (is_q) {
                dst = (__nv_bfloat16*)e.q_out + ((int64_t)tok * e.num_heads + local) * kTileM;
              } else if (e.slots != nullptr && e.k_cache != nullptr) {
                const int64_t slot = __shfl_sync(0xffffffffu, qkv_slot, nth);
                if (slot >= e.num_pages * e.page_size) {
                  if (lane == 0) set_status(p.status, kBadSlot);
                } else if (slot >= 0) {
                  const int64_t page = slot / e.page_size, in_page = slot % e.page_size;
                  dst = (__nv_bfloat16*)(is_k ? e.k_cache : e.v_cache) +
                        ((page * e.num_kv_heads + local) * e.page_size + in_page) * (int64_t)kTileM;
                }
              }
              if (dst != nullptr) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
                *reinterpret_cast<uint2*>(dst + 4 * lane) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
              }
            } else if constexpr (kEpilogue == kEpilogueResidual) {
              // hidden += the tile (rounded as the stored product would be); the new values' squares, summed over
              // the tile's features, are this tile's share of the token's mean square.
              float* cell = p.residual.hidden + (int64_t)tok * p.features + feature;
              float h[4] = {0.f, 0.f, 0.f, 0.f};
              const float add[4] = {bf16_round(v.x), bf16_round(v.y), bf16_round(v.z), bf16_round(v.w)};
              if (whole && feature < p.features) {
                const float4 old = (round == 0 && u == 0) ? res_old : *reinterpret_cast<const float4*>(cell);
                h[0] = old.x + add[0];
                h[1] = old.y + add[1];
                h[2] = old.z + add[2];
                h[3] = old.w + add[3];
                *reinterpret_cast<float4*>(cell) = make_float4(h[0], h[1], h[2], h[3]);
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  if (feature + i < p.features) {
                    h[i] = cell[i] + add[i];
                    cell[i] = h[i];
                  }
              }
              const float ss = warp_sum(h[0] * h[0] + h[1] * h[1] + h[2] * h[2] + h[3] * h[3]);
              if (lane == 0) p.residual.ssq[(int64_t)tile * p.tokens + tok] = ss;
            } else {
              OutT* dst = out + (int64_t)tok * p.features + feature;
              const float x[4] = {v.x, v.y, v.z, v.w};
              if (whole && feature < p.features) {
                if constexpr (sizeof(OutT) == 4) {
                  *reinterpret_cast<float4*>(dst) = v;
                } else {
                  __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
                  *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                }
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  if (feature + i < p.features) dst[i] = from_float<OutT>(x[i]);
              }
            }
          }
        }
      };
      switch (p.splits) {
        case 1: tail(std::integral_constant<int, 1>{}); break;
        case 2: tail(std::integral_constant<int, 2>{}); break;
        case 4: tail(std::integral_constant<int, 4>{}); break;
        default: tail(std::integral_constant<int, 8>{}); break;
      }
      cluster_meet_to_leave();      // nobody leaves while a peer may still read its shared memory
    }
  }
  if (warp < 2) {
    if (!ok) set_status(p.status, kWaitTimeout);
    if (p.out != nullptr) {
      cluster_sync_all();      // with warps 2-5: the partials are in place, then everybody is done reading
      cluster_meet_to_leave();
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

// Map over a row-major bfloat16 matrix [rows, cols]: boxes of 64 columns by `box_rows` rows, 128-byte swizzle,
// zeros outside the matrix.
bool matrix_map(const void* base, int64_t rows, int64_t cols, int box_rows, CUtensorMap* out) {
  static std::mutex mutex;
  static std::map<std::tuple<const void*, int64_t, int64_t, int>, CUtensorMap> cache;
  std::lock_guard<std::mutex> guard(mutex);
  const auto key = std::make_tuple(base, rows, cols, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult res = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return false;
  if (cache.size() > 8192) cache.clear();
  cache[key] = map;
  *out = map;
  return true;
}

template <int BN, typename OutT, int kStages, int kEpilogue, bool kNormedX>
int launch_stages(const CUtensorMap& w_map, const CUtensorMap& x_map, const GemmParams& p, cudaStream_t stream) {
  auto kernel = small_m_gemm_kernel<BN, OutT, kStages, kEpilogue, kNormedX>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN, kStages>::kBytes);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const dim3 grid((unsigned)((p.features + kTileM - 1) / kTileM), (unsigned)p.splits);
  const dim3 cluster(1, p.out != nullptr ? (unsigned)p.splits : 1u, 1);   // the splits of a tile form the cluster
  return (int)launch_chain(kernel, grid, dim3(192), GemmSmem<BN, kStages>::kBytes, stream, cluster, w_map, x_map, p);
}

// Stages of the TMA ring of the plain product when AKV_GEMM_STAGES=2|3|4|8 is set in the environment (for
// measurements); 0: the default of the token count.
int ring_stages() {
  static const int stages = [] {
    const char* v = getenv("AKV_GEMM_STAGES");
    const int n = v ? atoi(v) : 0;
    return (n == 2 || n == 3 || n == 4 || n == 8) ? n : 0;
  }();
  return stages;
}

template <int BN, bool kNormedX>
int launch_bn(const CUtensorMap& w_map, const CUtensorMap& x_map, const GemmParams& p, int epilogue, bool bf16_out,
              cudaStream_t stream) {
  // 16 tokens: four stages of 18 KB; 32 and 64 tokens: three stages of 20 and 24 KB.  Either way three CTAs share
  // an SM (with four stages of 20 KB only two did, and the wide projections took 27 % longer).  A narrow product
  // whose grid two CTAs per SM already hold (the o and down projections: 256 CTAs) gains nothing from the third CTA
  // and takes the deeper ring instead (64 tokens, o: 12.8 -> 11.5 us, down: 23.6 -> 21.7 us).
  constexpr int kDefault = BN == 16 ? 4 : 3;
  const int64_t ctas = (int64_t)((p.features + kTileM - 1) / kTileM) * p.splits;
  const bool deep = BN > 16 && ctas <= 2 * sm_count();
  switch (epilogue) {
    case kEpilogueGated:
      return launch_stages<BN, __nv_bfloat16, kDefault, kEpilogueGated, kNormedX>(w_map, x_map, p, stream);
    case kEpilogueQkv:
      return launch_stages<BN, __nv_bfloat16, kDefault, kEpilogueQkv, kNormedX>(w_map, x_map, p, stream);
    case kEpilogueResidual:
      if constexpr (kNormedX) return (int)cudaErrorInvalidValue;
      else return deep ? launch_stages<BN, float, 4, kEpilogueResidual, false>(w_map, x_map, p, stream)
                       : launch_stages<BN, float, kDefault, kEpilogueResidual, false>(w_map, x_map, p, stream);
    default: break;
  }
  if constexpr (!kNormedX) {
    int stages = ring_stages();
    if (stages == 0 && deep) stages = 4;
    if (stages == 2)
      return bf16_out ? launch_stages<BN, __nv_bfloat16, 2, kEpiloguePlain, false>(w_map, x_map, p, stream)
                      : launch_stages<BN, float, 2, kEpiloguePlain, false>(w_map, x_map, p, stream);
    if (stages == 8)
      return bf16_out ? launch_stages<BN, __nv_bfloat16, 8, kEpiloguePlain, false>(w_map, x_map, p, stream)
                      : launch_stages<BN, float, 8, kEpiloguePlain, false>(w_map, x_map, p, stream);
    if (stages == 7 - kDefault)      // the other of 3 and 4
      return bf16_out ? launch_stages<BN, __nv_bfloat16, 7 - kDefault, kEpiloguePlain, false>(w_map, x_map, p, stream)
                      : launch_stages<BN, float, 7 - kDefault, kEpiloguePlain, false>(w_map, x_map, p, stream);
  }
  return bf16_out ? launch_stages<BN, __nv_bfloat16, kDefault, kEpiloguePlain, kNormedX>(w_map, x_map, p, stream)
                  : launch_stages<BN, float, kDefault, kEpiloguePlain, kNormedX>(w_map, x_map, p, stream);
}

template <bool kNormedX>
int launch_tokens(int bn, const CUtensorMap& w_map, const CUtensorMap& x_map, const GemmParams& p, int epilogue,
                  bool bf16_out, cudaStream_t stream) {
  if (bn == 16) return launch_bn<16, kNormedX>(w_map, x_map, p, epilogue, bf16_out, stream);
  if (bn == 32) return launch_bn<32, kNormedX>(w_map, x_map, p, epilogue, bf16_out, stream);
  return launch_bn<64, kNormedX>(w_map, x_map, p, epilogue, bf16_out, stream);
}

}  // namespace

bool weight_tensor_map(const void* base, int64_t rows, int64_t cols, int box_rows, CUtensorMap* out) {
  return matrix_map(base, rows, cols, box_rows, out);
}

bool small_m_gemm_supported(int64_t tokens, int64_t features, int64_t k) {
  return tokens >= 1 && tokens <= 64 && k >= 64 && k % 8 == 0 && features >= 1 && encode_fn() != nullptr &&
         (features + kTileM - 1) / kTileM <= 0x7fffffffLL;
}

// 1, 2, 4 or 8 splits of K: enough CTAs for about two per SM, at least four K blocks each.
int small_m_gemm_splits(int64_t features, int64_t k) {
  const int64_t tiles = (features + kTileM - 1) / kTileM;
  const int64_t kb_total = (k + kTileK - 1) / kTileK;
  int splits = 1;
  while (splits < 8 && tiles * splits < 2 * sm_count() && kb_total / (splits * 2) >= 4) splits *= 2;
  return splits;
}

// out_dtype: akv::DType of `out` when the split partials are reduced inside the kernel; parts (float32
// [splits, tokens, features]) is written instead when `out` is null.  `fusion` (null: none) names what else the
// kernel does: an epilogue on the output tile, a token operand made from the residual stream.
int launch_small_m_gemm(const void* x, const void* w, void* out, int out_dtype, float* parts, int64_t tokens,
                        int64_t features, int64_t k, int splits, const GemmFusion* fusion, int* status,
                        cudaStream_t stream) {
  if (!small_m_gemm_supported(tokens, features, k) || splits < 1) return (int)cudaErrorInvalidValue;
  const GemmFusion plain;
  const GemmFusion& f = fusion != nullptr ? *fusion : plain;
  if (f.epilogue == kEpilogueQkv) {
    // the results go where qkv says; `out` only selects the in-kernel reduction and is never written
    if (f.qkv.q_out == nullptr || parts != nullptr || f.qkv.positions == nullptr) return (int)cudaErrorInvalidValue;
    if (features != (int64_t)(f.qkv.num_heads + 2 * f.qkv.num_kv_heads) * kTileM) return (int)cudaErrorInvalidValue;
    out = f.qkv.q_out;
    out_dtype = kBFloat16;
  } else if (f.epilogue == kEpilogueResidual) {
    if (f.residual.hidden == nullptr || f.residual.ssq == nullptr || parts != nullptr || f.normed_x)
      return (int)cudaErrorInvalidValue;
    out = f.residual.hidden;
    out_dtype = kFloat32;
  } else if (f.epilogue == kEpilogueGated) {
    if (out == nullptr || out_dtype != kBFloat16 || features % kTileM != 0) return (int)cudaErrorInvalidValue;
  } else if (f.epilogue != kEpiloguePlain) {
    return (int)cudaErrorInvalidValue;
  }
  if ((out == nullptr) == (parts == nullptr)) return (int)cudaErrorInvalidValue;
  if (f.normed_x) {
    if (x != nullptr || f.normed.hidden == nullptr || f.normed.ssq == nullptr || f.normed.weight == nullptr ||
        f.normed.ssq_tiles < 1 || parts != nullptr)
      return (int)cudaErrorInvalidValue;
  } else if (x == nullptr) {
    return (int)cudaErrorInvalidValue;
  }
  const int bn = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : 64);
  const int kb_total = (int)((k + kTileK - 1) / kTileK);
  if (splits > kb_total) return (int)cudaErrorInvalidValue;
  if (out != nullptr && splits != 1 && splits != 2 && splits != 4 && splits != 8) return (int)cudaErrorInvalidValue;
  CUtensorMap w_map, x_map;
  if (!matrix_map(w, features, k, kTileM, &w_map)) return (int)cudaErrorInvalidValue;
  if (f.normed_x) x_map = w_map;      // unused
  else if (!matrix_map(x, tokens, k, bn, &x_map)) return (int)cudaErrorInvalidValue;
  GemmParams p{parts, out, (int)tokens, (int)features, (int)k, kb_total, splits, status, f.qkv, f.residual, f.normed};
  const bool bf16_out = out != nullptr && out_dtype == kBFloat16;
  if (f.normed_x) return launch_tokens<true>(bn, w_map, x_map, p, f.epilogue, bf16_out, stream);
  return launch_tokens<false>(bn, w_map, x_map, p, f.epilogue, bf16_out, stream);
}

}  // namespace akv
