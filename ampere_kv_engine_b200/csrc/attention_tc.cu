// Tensor-core paged attention for bfloat16 caches: K/V pages are brought into shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, mbarrier completion, no multicast), scores and the weighted sum of
// V run on mma.sync m16n8k16 with float32 accumulators, the softmax is an online float32 softmax in registers.
//
// Two kernels:
//   * prompt portions: one CTA per (query tile of up to 16 tokens, kv head); warp g owns q-head kvh*G + g, its
//     16 MMA rows are the tile's tokens; the G warps share every K/V tile (one read per GQA group).
//   * decoded tokens: one CTA per (token, kv head, key split); the MMA rows are the G q-heads of the group; the
//     consumer warps work on the same 32-key block together; 2, 4 or 8 key splits form a thread-block cluster
//     and are merged through distributed shared memory (other split counts leave (acc, max, sum) partials for
//     the merge kernel of paged_attention.cu).
//
// Same mathematics as the general kernel and as the reference (ampere_kv/kv_cache.py:76-94,
// csrc/paged_decode.cu:166-243): score = q.k * scale, key j visible to the query at position t iff j <= t (and
// j > t - window), float32 softmax, q-head h reads kv-head h / G.
//
// Every mbarrier wait is bounded: a wait that runs out records kWaitTimeout in the status word and the CTA
// leaves without writing results.  Keys past a sequence's end inside its last page may hold anything: their
// scores are replaced (not multiplied) and their V rows are zeroed in shared memory before use.
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

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
// Returns false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  return mbar_wait_bounded(smem_addr(bar), parity, kWaitLimit);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct TcParams {
  PagedAttentionParams p;
  int box_rows;     // rows of one TMA box = min(page_size, keys per stage)
};

// Byte offset of (key k, 16-byte chunk c of the head) inside one stage's K or V area.  The area is laid out
// as [64-dim half][key][128 bytes]; TMA's 128-byte swizzle xors the chunk-in-row with the row's low 3 bits.
// (Fetching both halves of a page with one 3-D box, [key][half][128 bytes], was tried: it halves the number of
// TMA instructions, changes decode attention by 3 % and costs the prompt kernel 70 % through two-way ldmatrix
// bank conflicts.)
template <int D, int KT>
__device__ __forceinline__ uint32_t tile_offset_d(int k, int chunk) {
  const int half = chunk >> 3, c = chunk & 7;
  return (uint32_t)(half * KT * 128 + k * 128 + ((c ^ (k & 7)) << 4));
}

// One warp's share of a key block: scores for its 16 rows against KT keys, online softmax, P.V.
//   q_frag: A fragments of the warp's 16 query rows, D/16 k-steps of 4 registers
//   row_pos[2]: absolute position of rows (lane/4) and (lane/4 + 8), -1 for a row that does not exist
template <int D, int KT>
__device__ __forceinline__ void process_block(const uint32_t (&q_frag)[D / 16][4], uint32_t k_base, uint32_t v_base,
                                              int key0, int nvalid, const int (&row_pos)[2], int window,
                                              float scale_log2, float (&m)[2], float (&l)[2],
                                              float (&o)[D / 8][4]) {
  const int lane = threadIdx.x & 31;
  constexpr int NT = KT / 8;   // score n-tiles
  float s[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
  }
  // S = Q K^T
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    if (j * 8 < nvalid) {
#pragma unroll
      for (int t = 0; t < D / 16; t += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = j * 8 + (lane & 7);
        const int chunk = 2 * t + (lane >> 3);
        ldmatrix_x4(k_base + tile_offset_d<D, KT>(key, chunk), b0, b1, b2, b3);
        mma_bf16(s[j], q_frag[t], b0, b1);
        mma_bf16(s[j], q_frag[t + 1], b2, b3);
      }
    }
  }
  // mask, scale, block max
  float bmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
      const bool visible = (j * 8 + (lane & 3) * 2 + (e & 1)) < nvalid && key <= row_pos[r] &&
                           (window <= 0 || key > row_pos[r] - window);
      const float v = visible ? s[j][e] * scale_log2 : -CUDART_INF_F;
      s[j][e] = v;
      bmax[r] = fmaxf(bmax[r], v);
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 1));
    bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 2));
  }
  float alpha[2], m_new[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    m_new[r] = fmaxf(m[r], bmax[r]);
    alpha[r] = (m_new[r] == -CUDART_INF_F) ? 1.f : exp2f(m[r] - m_new[r]);
    m[r] = m_new[r];
    l[r] *= alpha[r];
  }
#pragma unroll
  for (int v = 0; v < D / 8; ++v) {
    o[v][0] *= alpha[0];
    o[v][1] *= alpha[0];
    o[v][2] *= alpha[1];
    o[v][3] *= alpha[1];
  }
  // P = exp2(S - m), row sums (per-lane partial sums; reduced over the quad at the end)
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const float pv = (s[j][e] == -CUDART_INF_F) ? 0.f : exp2f(s[j][e] - m_new[r]);
      s[j][e] = pv;
      l[r] += pv;
    }
  }
  // O += P V, 16 keys at a time
#pragma unroll
  for (int u = 0; u < KT / 16; ++u) {
    if (u * 16 < nvalid) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * u][0], s[2 * u][1]);
      a[1] = pack_bf16(s[2 * u][2], s[2 * u][3]);
      a[2] = pack_bf16(s[2 * u + 1][0], s[2 * u + 1][1]);
      a[3] = pack_bf16(s[2 * u + 1][2], s[2 * u + 1][3]);
#pragma unroll
      for (int v = 0; v < D / 8; v += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = u * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = v + (lane >> 4);
        ldmatrix_x4_trans(v_base + tile_offset_d<D, KT>(key, chunk), b0, b1, b2, b3);
        mma_bf16(o[v], a, b0, b1);
        mma_bf16(o[v + 1], a, b2, b3);
      }
    }
  }
}

// Shared-memory layout of the prompt kernel: [stage][K area | V area], each area KT * D * 2 bytes, then the
// mbarriers.
template <int D, int KT, int STAGES>
struct Smem {
  static constexpr int kArea = KT * D * 2;
  static constexpr int kStage = 2 * kArea;
  static constexpr int kBytes = STAGES * kStage + 2 * STAGES * 8 + 1024;   // + alignment slack
};

// The producer warp's view of the block table: each lane holds one entry of the current run of 32 logical
// pages, so a dependent global load is paid once per 32 pages, not once per key block.
struct TableWindow {
  const int32_t* table;
  int width;
  int first;      // logical page of lane 0's entry, -1 before the first load
  int entry;
  __device__ __forceinline__ int page(int logical, int lane) {
    const int base = logical & ~31;
    if (base != first) {
      first = base;
      const int mine = base + lane;
      entry = mine < width ? table[mine] : -1;
    }
    return __shfl_sync(0xffffffffu, entry, logical & 31);
  }
};

// Issue this producer warp's share of the TMA loads of the key block starting at key0 into `stage`.  Issuing a
// tensor copy costs the issuing thread on the order of a hundred cycles, and a block of 16-token pages needs
// eight of them, so the copies of a block are dealt out to `num_producers` warps (copy i to warp i mod n); each
// announces its own bytes on the stage's barrier, which counts `num_producers` arrivals.
template <int D, int KT>
__device__ __forceinline__ void issue_block(const TcParams& tp, const CUtensorMap* k_map, const CUtensorMap* v_map,
                                            TableWindow& window, int kvh, int key0, int key_end, uint8_t* stage,
                                            uint64_t* bar, int producer, int num_producers) {
  const PagedAttentionParams& p = tp.p;
  const int lane = threadIdx.x & 31;
  const int P = p.page_size, rows = tp.box_rows;
  const int boxes = KT / rows;
  constexpr int H = D / 64;
  uint32_t bytes = 0;
  int page_of[KT / 8];   // rows >= 8, so at most KT / 8 boxes
#pragma unroll
  for (int b = 0; b < KT / 8; ++b) {
    page_of[b] = -1;
    if (b < boxes) {
      const int key = key0 + b * rows;
      if (key < key_end) {
        int page = window.page(key / P, lane);
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) set_status(p.status, kBadPage);
          page = -1;
        }
        page_of[b] = page;
        if (page >= 0) {
#pragma unroll
          for (int c = 0; c < 2 * H; ++c)
            if ((b * 2 * H + c) % num_producers == producer) bytes += (uint32_t)rows * 128u;
        }
      }
    }
  }
  // One copy per lane (lane = box * 2H + copy), issued side by side: one thread issuing a block's copies in turn
  // spends about 150 ns on each, which capped a CTA at 13-15 GB/s.
  if (lane == 0) mbar_expect_tx(bar, bytes);
  __syncwarp();
  const int my_box = lane / (2 * H), c = lane % (2 * H);
  int my_page = -1;
#pragma unroll
  for (int b = 0; b < KT / 8; ++b)
    if (b == my_box && b < boxes) my_page = page_of[b];
  if (my_page >= 0 && lane % num_producers == producer) {
    const int key = key0 + my_box * rows;
    const int y = (my_page * p.num_kv_heads + kvh) * P + key % P;
    const int h = c >> 1;
    if (c & 1)
      tma_load_2d(stage + KT * D * 2 + h * KT * 128 + my_box * rows * 128, v_map, h * 64, y, bar);
    else
      tma_load_2d(stage + h * KT * 128 + my_box * rows * 128, k_map, h * 64, y, bar);
  }
}

// Zero the V rows [first, KT) of a stage (keys past the end of the sequence).
template <int D, int KT>
__device__ __forceinline__ void zero_v_rows(uint8_t* stage, int first, int tid, int nthreads) {
  uint8_t* v_area = stage + KT * D * 2;
  const int chunks_per_row = 8;   // 128 bytes
  for (int h = 0; h < D / 64; ++h) {
    const int total = (KT - first) * chunks_per_row;
    for (int i = tid; i < total; i += nthreads) {
      const int row = first + i / chunks_per_row, c = i % chunks_per_row;
      *reinterpret_cast<uint4*>(v_area + h * KT * 128 + row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
    }
  }
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync(int consumers) {
  asm volatile("bar.sync 1, %0;" ::"r"(consumers * 32) : "memory");
}
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
__device__ __forceinline__ float ld_peer_smem(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// Merge of one output row across the key splits of a cluster (at most 8 CTAs): row layout in every CTA's shared
// memory is (acc[D], max in log2 units, sum).  A thread's first dim is fetched together with the maxima and the
// sums, all loads issued before the first is used: one round trip through distributed shared memory for the row
// when the CTA has a thread per dim, not one for the weights and another for the values.  The sums run in split
// order.
template <int D>
__device__ __forceinline__ void merge_row_over_splits(uint32_t base, int splits, int tid, int nthreads,
                                                      __nv_bfloat16* out) {
  float mv[8], lv[8], v[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    mv[s] = s < splits ? ld_peer_smem(base + D * 4u, (uint32_t)s) : -CUDART_INF_F;
    lv[s] = s < splits ? ld_peer_smem(base + (D + 1) * 4u, (uint32_t)s) : 0.f;
    v[s] = (s < splits && tid < D) ? ld_peer_smem(base + tid * 4u, (uint32_t)s) : 0.f;
  }
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int s = 0; s < 8; ++s)
    if (lv[s] > 0.f) mx = fmaxf(mx, mv[s]);
  float w[8], den = 0.f;
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    w[s] = lv[s] > 0.f ? exp2f(mv[s] - mx) : 0.f;
    den += w[s] * lv[s];
  }
  for (int d = tid; d < D; d += nthreads) {
    if (d != tid) {
#pragma unroll
      for (int s = 0; s < 8; ++s) v[s] = s < splits ? ld_peer_smem(base + d * 4u, (uint32_t)s) : 0.f;
    }
    float num = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) num += w[s] * v[s];
    out[d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
  }
}

// Producer warps of one CTA.  Measured on B200: one is best; more producers only add warps that spin on the
// barriers (decode at batch 64, 1,152 keys: 102 us with one producer, 184 us with four).
constexpr int kProducers = 1;

// The prompt kernel.  Warps 0 .. consumers-1 compute (warp g = q-head g of the group); the last kProducers warps
// are the producers: they walk the block table and keep the TMA ring full.  full[s]: the stage's bytes have
// landed; empty[s]: every consumer warp is done with the stage.
template <int D, int KT, int STAGES, int WARPS, int MIN_CTAS>
__global__ void __launch_bounds__(32 * (WARPS + kProducers), MIN_CTAS) attention_tc_kernel(const __grid_constant__ CUtensorMap k_map,
                                    const __grid_constant__ CUtensorMap v_map, TcParams tp) {
  const PagedAttentionParams& p = tp.p;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Smem<D, KT, STAGES>::kStage);
  uint64_t* empty = full + STAGES;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int consumers = (int)(blockDim.x >> 5) - kProducers;
  const bool is_producer = warp >= consumers;
  const int G = p.num_heads / p.num_kv_heads, NH = p.num_heads;
  const int tile = blockIdx.x, kvh = blockIdx.y;

  pdl_launch_dependents();
  // a batch tile holds up to q_tile tokens; this kernel's CTAs take 16 of them each
  const int subtiles = (p.q_tile + 15) / 16;
  const int batch_tile = tile / subtiles, sub = tile - batch_tile * subtiles;
  const int seq = p.tile_seq[batch_tile];
  const int q0 = p.tile_q0[batch_tile] + 16 * sub;
  const int nq = min(16, p.tile_nq[batch_tile] - 16 * sub);
  if (nq <= 0) return;
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  const int tile_pos = ctx - q_len + (q0 - seq_q0);

  const int pos_first = tile_pos, pos_last = tile_pos + nq - 1;
  int lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  lo = lo / tp.box_rows * tp.box_rows;     // boxes start on box boundaries inside a page
  const int hi = pos_last + 1;
  const int range_lo = lo, range_hi = hi;
  const int num_blocks = range_hi > range_lo ? (range_hi - range_lo + KT - 1) / KT : 0;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], kProducers);
      mbar_init(&empty[s], consumers);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();      // q and this step's K/V pages come from the previous kernels

  bool ok = true;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
  int row_pos[2] = {-1, -1}, row_token[2] = {0, 0}, row_head[2] = {0, 0};

  if (is_producer) {
    TableWindow window{p.block_table + (int64_t)seq * p.table_width, p.table_width, -1, -1};
    for (int b = 0; b < num_blocks; ++b) {
      const int s = b % STAGES;
      if (b >= STAGES && !mbar_wait(&empty[s], ((b / STAGES) - 1) & 1)) {
        ok = false;
        break;
      }
      issue_block<D, KT>(tp, &k_map, &v_map, window, kvh, range_lo + b * KT, range_hi,
                         smem + s * Smem<D, KT, STAGES>::kStage, &full[s], warp - consumers, kProducers);
    }
  } else {
    // rows of this warp: the tile's tokens, of head (kvh*G + warp)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = (lane >> 2) + 8 * r;
      row_token[r] = q0 + row;
      row_head[r] = kvh * G + warp;
      row_pos[r] = row < nq ? tile_pos + row : -1;
    }
    // query fragments straight from global memory
    uint32_t q_frag[D / 16][4];
    {
      const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
#pragma unroll
      for (int t = 0; t < D / 16; ++t) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int col = t * 16 + (lane & 3) * 2;
          uint32_t lo_pair = 0, hi_pair = 0;
          if (row_pos[r] >= 0) {
            const __nv_bfloat16* src = q + ((int64_t)row_token[r] * NH + row_head[r]) * D + col;
            lo_pair = *reinterpret_cast<const uint32_t*>(src);
            hi_pair = *reinterpret_cast<const uint32_t*>(src + 8);
          }
          q_frag[t][r] = lo_pair;
          q_frag[t][2 + r] = hi_pair;
        }
      }
    }
#pragma unroll
    for (int v = 0; v < D / 8; ++v) o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.f;
    const float scale_log2 = p.scale * kLog2e;

    // Every consumer warp (one q-head each) works on every block.  A warp whose wait ran out keeps walking the
    // loop (the consumers' barriers stay matched) but computes nothing.
    for (int b = 0; b < num_blocks; ++b) {
      const int s = b % STAGES;
      uint8_t* stage = smem + s * Smem<D, KT, STAGES>::kStage;
      if (ok && !mbar_wait(&full[s], (b / STAGES) & 1)) ok = false;
      const int key0 = range_lo + b * KT;
      const int nvalid = min(KT, range_hi - key0);
      if (nvalid < KT) {
        // V rows past the end may hold anything (or were never loaded): make them zero before P.V reads them.
        // This only ever happens in a range's last block, so no later TMA load touches these rows.
        zero_v_rows<D, KT>(stage, nvalid, tid, consumers * 32);
        consumer_sync(consumers);
      }
      if (ok)
        process_block<D, KT>(q_frag, smem_addr(stage), smem_addr(stage + KT * D * 2), key0, nvalid, row_pos,
                             p.window, scale_log2, m, l, o);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
  }
  if (!ok && lane == 0) set_status(p.status, kWaitTimeout);

  if (is_producer || !ok) return;

  // every warp writes its own head's rows
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (row_pos[r] < 0) continue;
    const int64_t row = (int64_t)row_token[r] * NH + row_head[r];
    __nv_bfloat16* out = (__nv_bfloat16*)p.out + row * D;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
    for (int v = 0; v < D / 8; ++v) {
      const int col = v * 8 + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(out + col) = pack_bf16(o[v][2 * r] * inv, o[v][2 * r + 1] * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------- decode, cooperative
// Decoded tokens: the consumer warps of a CTA work on the SAME 32-key block, so a stage of the
// TMA ring is held for a quarter of the time and the ring turns over four times faster (decode attention is bound
// by how many bytes a CTA keeps in flight, not by arithmetic).  Warp w scores keys [8w, 8w + 8) of the block
// (Q K^T, one 16 x 8 tile over all of D), the warps exchange their row maxima and their probabilities through
// shared memory, then warp w accumulates P V for head dims [w D/4, (w + 1) D/4).  The MMA rows are the G q-heads
// of the group, as before; 2, 4 or 8 key splits form a cluster and are merged through distributed shared memory.
constexpr int kPRow = 40;      // bf16 elements per row of the probability tile: 32 keys + padding against bank conflicts

template <int D, int STAGES, int kCoopWarps>
struct CoopSmem {
  static constexpr int KT = 32;
  static constexpr int kStage = 2 * KT * D * 2;
  static constexpr int kExchange = 2 * (kCoopWarps * 16 * 4 + 16 * kPRow * 2);   // double-buffered maxima + P tile
  static constexpr int kMerge = 16 * (D + 2) * 4;
  static_assert(kMerge <= STAGES * kStage, "the merge buffer must fit in the stage ring");
  static constexpr int kBytes = STAGES * kStage + kExchange + 2 * STAGES * 8 + kCoopWarps * 16 * 4 + 1024;
};

template <int D, int STAGES, bool CLUSTER, int kCoopWarps>
__global__ void __launch_bounds__((kCoopWarps + 1) * 32)
attention_decode_coop_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             TcParams tp) {
  constexpr int KT = 32;
  constexpr int NV = D / 8 / kCoopWarps;       // P.V n-tiles (8 dims each) per warp
  using Layout = CoopSmem<D, STAGES, kCoopWarps>;
  constexpr int NQ = KT / 8 / kCoopWarps;      // score n-tiles (8 keys each) per warp
  const PagedAttentionParams& p = tp.p;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* smax = reinterpret_cast<float*>(smem + STAGES * Layout::kStage);                  // [2][warps][16]
  __nv_bfloat16* ptile = reinterpret_cast<__nv_bfloat16*>(smax + 2 * kCoopWarps * 16);     // [2][16][kPRow]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Layout::kStage + Layout::kExchange);
  uint64_t* empty = full + STAGES;
  float* lpart = reinterpret_cast<float*>(empty + STAGES);                                 // [warps][16] row sums
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool is_producer = warp == kCoopWarps;
  const int G = p.num_heads / p.num_kv_heads, NH = p.num_heads;
  // CTAs start in the order of blockIdx.x, then .y: taken tile-major, all kv heads of the first tile start before
  // any of the second, so that the host's order of the tiles (longest context first) is the order of the work
  const int linear = blockIdx.y * gridDim.x + blockIdx.x;
  const int tile = linear / gridDim.y, kvh = linear - tile * gridDim.y, split = blockIdx.z;

  pdl_launch_dependents();
  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int nq = p.tile_nq[tile];
  if (nq <= 0) return;     // padding of a captured layout; the whole cluster sees the same tile
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  const int pos = ctx - q_len + (q0 - seq_q0);

  int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  lo = lo / tp.box_rows * tp.box_rows;
  const int hi = pos + 1;
  int range_lo = lo, range_hi = hi;
  if (p.num_splits > 1) {
    int per = (hi - lo + p.num_splits - 1) / p.num_splits;
    per = (per + KT - 1) / KT * KT;
    range_lo = lo + split * per;
    range_hi = min(hi, range_lo + per);
  }
  const int num_blocks = range_hi > range_lo ? (range_hi - range_lo + KT - 1) / KT : 0;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCoopWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  bool ok = true;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  float o[NV][4];
#pragma unroll
  for (int v = 0; v < NV; ++v) o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.f;

  if (is_producer) {
    TableWindow window{p.block_table + (int64_t)seq * p.table_width, p.table_width, -1, -1};
    // Keys before this step's tokens were written by earlier steps: their blocks are fetched while the previous
    // kernel (which writes this step's K and V) still runs, as far as the ring has room.
    const int first_new = ctx - q_len;
    int b = 0;
    for (; b < num_blocks && b < STAGES && min(range_lo + (b + 1) * KT, range_hi) <= first_new; ++b)
      issue_block<D, KT>(tp, &k_map, &v_map, window, kvh, range_lo + b * KT, range_hi, smem + b * Layout::kStage,
                         &full[b], 0, 1);
    pdl_wait();      // this step's K/V pages come from the previous kernels
    for (; b < num_blocks; ++b) {
      const int s = b % STAGES;
      if (b >= STAGES && !mbar_wait(&empty[s], ((b / STAGES) - 1) & 1)) {
        ok = false;
        break;
      }
      issue_block<D, KT>(tp, &k_map, &v_map, window, kvh, range_lo + b * KT, range_hi, smem + s * Layout::kStage,
                         &full[s], 0, 1);
    }
  } else {
    pdl_wait();      // q comes from the previous kernel
    // query fragments: rows are the heads of the group (row < G), all D/16 k-steps
    const int row_a = lane >> 2, row_b = row_a + 8;
    uint32_t q_frag[D / 16][4];
    {
      const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
#pragma unroll
      for (int t = 0; t < D / 16; ++t) {
        const int col = t * 16 + (lane & 3) * 2;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = r ? row_b : row_a;
          uint32_t lo_pair = 0, hi_pair = 0;
          if (row < G) {
            const __nv_bfloat16* src = q + ((int64_t)q0 * NH + kvh * G + row) * D + col;
            lo_pair = *reinterpret_cast<const uint32_t*>(src);
            hi_pair = *reinterpret_cast<const uint32_t*>(src + 8);
          }
          q_frag[t][r] = lo_pair;
          q_frag[t][2 + r] = hi_pair;
        }
      }
    }
    const float scale_log2 = p.scale * kLog2e;
    const bool live[2] = {row_a < G, row_b < G};

    for (int b = 0; b < num_blocks; ++b) {
      const int s = b % STAGES;
      uint8_t* stage = smem + s * Layout::kStage;
      const uint32_t k_base = smem_addr(stage), v_base = smem_addr(stage + KT * D * 2);
      float* my_max = smax + (b & 1) * kCoopWarps * 16;
      __nv_bfloat16* my_p = ptile + (b & 1) * 16 * kPRow;
      if (ok && !mbar_wait(&full[s], (b / STAGES) & 1)) ok = false;
      const int key0 = range_lo + b * KT;
      const int nvalid = min(KT, range_hi - key0);
      if (nvalid < KT) zero_v_rows<D, KT>(stage, nvalid, tid, kCoopWarps * 32);   // made visible by the barriers below

      // scores of this warp's keys: NQ tiles of 8
      float sc[NQ][4];
#pragma unroll
      for (int j = 0; j < NQ; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        const int first = (warp * NQ + j) * 8;
        if (ok && first < nvalid) {
#pragma unroll
          for (int t = 0; t < D / 16; t += 2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + tile_offset_d<D, KT>(first + (lane & 7), 2 * t + (lane >> 3)), b0, b1, b2, b3);
            mma_bf16(sc[j], q_frag[t], b0, b1);
            mma_bf16(sc[j], q_frag[t + 1], b2, b3);
          }
        }
      }
      float bmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int in_block = (warp * NQ + j) * 8 + (lane & 3) * 2 + (e & 1);
          const int key = key0 + in_block;
          const bool visible = ok && live[r] && in_block < nvalid && key <= pos &&
                               (p.window <= 0 || key > pos - p.window);
          sc[j][e] = visible ? sc[j][e] * scale_log2 : -CUDART_INF_F;
          bmax[r] = fmaxf(bmax[r], sc[j][e]);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 1));
        bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 2));
      }
      if ((lane & 3) == 0) {
        my_max[warp * 16 + row_a] = bmax[0];
        my_max[warp * 16 + row_b] = bmax[1];
      }
      consumer_sync(kCoopWarps);
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = r ? row_b : row_a;
        float mx = m[r];
#pragma unroll
        for (int w = 0; w < kCoopWarps; ++w) mx = fmaxf(mx, my_max[w * 16 + row]);
        alpha[r] = (mx == -CUDART_INF_F) ? 1.f : exp2f(m[r] - mx);
        m[r] = mx;
        l[r] *= alpha[r];
      }
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        float pr[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          pr[e] = (sc[j][e] == -CUDART_INF_F) ? 0.f : exp2f(sc[j][e] - m[r]);
          l[r] += pr[e];
        }
        const int col = (warp * NQ + j) * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(my_p + row_a * kPRow + col) = pack_bf16(pr[0], pr[1]);
        *reinterpret_cast<uint32_t*>(my_p + row_b * kPRow + col) = pack_bf16(pr[2], pr[3]);
      }
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        o[v][0] *= alpha[0];
        o[v][1] *= alpha[0];
        o[v][2] *= alpha[1];
        o[v][3] *= alpha[1];
      }
      consumer_sync(kCoopWarps);
      // O[:, this warp's dims] += P V
      if (ok) {
#pragma unroll
        for (int u = 0; u < KT / 16; ++u) {
          if (u * 16 < nvalid) {
            uint32_t a[4];
            // A fragment of P: rows (lane & 15), 16-byte column chunk (lane >> 4) of the 16 keys of group u
            ldmatrix_x4(smem_addr(my_p + (lane & 15) * kPRow + u * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int v = 0; v < NV; v += 2) {
              uint32_t b0, b1, b2, b3;
              const int key = u * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
              const int chunk = warp * NV + v + (lane >> 4);
              ldmatrix_x4_trans(v_base + tile_offset_d<D, KT>(key, chunk), b0, b1, b2, b3);
              mma_bf16(o[v], a, b0, b1);
              if (v + 1 < NV) mma_bf16(o[v + 1], a, b2, b3);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    if ((lane & 3) == 0) {
      lpart[warp * 16 + row_a] = ok ? l[0] : 0.f;     // each warp summed the probabilities of its own keys
      lpart[warp * 16 + row_b] = ok ? l[1] : 0.f;
    }
  }
  if (!ok && lane == 0) set_status(p.status, kWaitTimeout);

  // the CTA's (acc, max, sum) for its rows, in the (idle) stage ring: every warp owns its own head dims
  __syncthreads();
  float* merge = reinterpret_cast<float*>(smem);
  constexpr int kRow = D + 2;
  if (!is_producer) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = (lane >> 2) + 8 * r;
      if (row < G) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const int col = (warp * NV + v) * 8 + (lane & 3) * 2;
          merge[row * kRow + col] = ok ? o[v][2 * r] : 0.f;
          merge[row * kRow + col + 1] = ok ? o[v][2 * r + 1] : 0.f;
        }
        if (warp == 0 && (lane & 3) == 0) {
          merge[row * kRow + D] = m[r];          // log2 units; the same in every warp
          float total = 0.f;
#pragma unroll
          for (int w = 0; w < kCoopWarps; ++w) total += lpart[w * 16 + row];     // fixed order
          merge[row * kRow + D + 1] = total;
        }
      }
    }
  }
  __syncthreads();
  if (CLUSTER) {
    cluster_sync_all();
    for (int row = split; row < G; row += p.num_splits) {
      const uint32_t base = smem_addr(merge) + (uint32_t)(row * kRow) * 4u;
      merge_row_over_splits<D>(base, p.num_splits, tid, blockDim.x,
                               (__nv_bfloat16*)p.out + ((int64_t)q0 * NH + kvh * G + row) * D);
    }
    cluster_meet_to_leave();      // nobody leaves while a peer may still read its shared memory
    return;
  }
  for (int idx = tid; idx < G * D; idx += blockDim.x) {
    const int row = idx / D, d = idx - row * D;
    const int64_t out_row = (int64_t)q0 * NH + kvh * G + row;
    const float sum = merge[row * kRow + D + 1];
    if (p.num_splits == 1) {
      ((__nv_bfloat16*)p.out)[out_row * D + d] = __float2bfloat16_rn(sum > 0.f ? merge[row * kRow + d] / sum : 0.f);
    } else {
      float* part = p.partials + (out_row * p.num_splits + split) * (int64_t)kRow;
      part[d] = merge[row * kRow + d];
      if (d == 0) {
        part[D] = merge[row * kRow + D] * kLn2;
        part[D + 1] = sum;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- host side

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

// A 2-D map over a cache tensor seen as [pages * kv_heads * page_size rows, head_dim] bfloat16, boxes of
// 64 columns (128 bytes) by `box_rows` rows, 128-byte swizzle.
bool cache_map(const void* base, int64_t rows, int head_dim, int box_rows, CUtensorMap* out) {
  static std::mutex mutex;
  static std::map<std::tuple<const void*, int64_t, int, int>, CUtensorMap> cache;
  std::lock_guard<std::mutex> guard(mutex);
  const auto key = std::make_tuple(base, rows, head_dim, box_rows);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult res = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return false;
  cache[key] = map;
  *out = map;
  return true;
}

template <int D, int KT, int STAGES, int WARPS, int MIN_CTAS>
int launch_prompt(const PagedAttentionParams& p, int box_rows, const CUtensorMap& k_map, const CUtensorMap& v_map,
                  cudaStream_t stream) {
  auto kernel = attention_tc_kernel<D, KT, STAGES, WARPS, MIN_CTAS>;
  constexpr int smem = Smem<D, KT, STAGES>::kBytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int G = p.num_heads / p.num_kv_heads;
  TcParams tp{p, box_rows};
  const dim3 grid((unsigned)(p.num_tiles * ((p.q_tile + 15) / 16)), (unsigned)p.num_kv_heads, 1u);
  const dim3 block(32 * (G + kProducers));      // one consumer warp per q-head of the group, and the producer
  return (int)launch_chain(kernel, grid, block, smem, stream, dim3(1, 1, 1), k_map, v_map, tp);
}

template <int D, int STAGES, bool CLUSTER, int kCoopWarps>
int launch_coop(const PagedAttentionParams& p, int box_rows, const CUtensorMap& k_map, const CUtensorMap& v_map,
                cudaStream_t stream) {
  auto kernel = attention_decode_coop_kernel<D, STAGES, CLUSTER, kCoopWarps>;
  constexpr int smem = CoopSmem<D, STAGES, kCoopWarps>::kBytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  TcParams tp{p, box_rows};
  const dim3 grid((unsigned)p.num_tiles, (unsigned)p.num_kv_heads, (unsigned)p.num_splits);
  const dim3 cluster(1, 1, CLUSTER ? (unsigned)p.num_splits : 1u);
  return (int)launch_chain(kernel, grid, dim3((kCoopWarps + 1) * 32), smem, stream, cluster, k_map, v_map, tp);
}

// Shape of the decode kernel's CTAs: (TMA ring stages of 16 KB at head size 128, consumer warps).  Bandwidth comes
// from CTAs per SM, and a cluster's CTAs must all fit at once: rings of 4 or more stages (64 KB and up) made the
// batch-8 kernel 25 us instead of 15 us.  Three stages pay since the producer fetches the blocks of old keys
// before it waits for the previous kernel.  Two consumer warps (more CTAs per SM by registers) do best wherever a
// CTA walks more than a few key blocks; four (the block is done sooner) only for the shortest walks, a few
// tokens cut into eight splits.  Measured per step with (3,4) | (3,2): batch 1 3.18 | 3.23 ms, batch 8 at 1,064
// keys 3.48 | 3.49 ms, batch 16 3.96 | 3.89 ms, batch 32 4.70 | 4.65 ms, batch 64 5.56 | 5.47 ms, batch 8 at 8,192
// keys 4.88 | 4.81 ms; (2,2) is 1-4 % behind everywhere.  AKV_ATTN_CONFIG=2|3|4|6 forces (2,2) | (3,4) | (2,4) | (3,2).
int decode_config(int splits, int64_t blocks_per_cta) {
  static const int forced = [] {
    const char* v = getenv("AKV_ATTN_CONFIG");
    const int n = v ? atoi(v) : 0;
    return (n == 2 || n == 3 || n == 4 || n == 6) ? n : 0;
  }();
  if (forced) return forced;
  return (splits >= 8 && blocks_per_cta < 16) ? 3 : 6;
}

}  // namespace

// Whether the tensor-core kernels take this problem; otherwise the caller uses the general kernel.
bool attention_tc_supported(const PagedAttentionParams& p) {
  if (p.dtype != kBFloat16) return false;
  if (p.head_dim != 64 && p.head_dim != 128) return false;
  const int G = p.num_heads / p.num_kv_heads;
  if (p.num_heads % p.num_kv_heads || G < 1 || G > 16) return false;
  if (p.page_size < 8 || (p.page_size & (p.page_size - 1))) return false;   // boxes of 8.. rows, power of two
  if (p.num_kv_heads > 65535 || p.num_splits > 65535) return false;
  if (p.q_tile > 128) return false;
  if (p.q_tile > 1 && G > 8) return false;    // prompt kernel: one warp per q-head of the group
  return encode_fn() != nullptr;
}

// Decode with 2, 4 or 8 key splits merges them inside the kernel (a cluster per token and kv head).
bool attention_tc_merges_in_kernel(const PagedAttentionParams& p) {
  return p.q_tile == 1 && (p.num_splits == 2 || p.num_splits == 4 || p.num_splits == 8);
}

int launch_attention_tc(const PagedAttentionParams& p, cudaStream_t stream) {
  const bool decode = p.q_tile == 1;
  const int G_all = p.num_heads / p.num_kv_heads;
  const char* prompt_config = getenv("AKV_PROMPT_CONFIG");
  const bool narrow_prompt = prompt_config != nullptr && atoi(prompt_config) == 32 && G_all <= 4 && p.page_size <= 32;
  const int kt = (decode || narrow_prompt) ? 32 : 64;
  const int box_rows = p.page_size < kt ? p.page_size : kt;
  const int64_t rows = p.num_pages * p.num_kv_heads * (int64_t)p.page_size;
  CUtensorMap k_map, v_map;
  if (!cache_map(p.k_cache, rows, p.head_dim, box_rows, &k_map) ||
      !cache_map(p.v_cache, rows, p.head_dim, box_rows, &v_map))
    return (int)cudaErrorInvalidValue;
  if (decode) {
    const bool merge = attention_tc_merges_in_kernel(p);
#define AKV_COOP(ST, W)                                                                                       \
  if (p.head_dim == 128)                                                                                      \
    return merge ? launch_coop<128, ST, true, W>(p, box_rows, k_map, v_map, stream)                           \
                 : launch_coop<128, ST, false, W>(p, box_rows, k_map, v_map, stream);                         \
  return merge ? launch_coop<64, ST, true, W>(p, box_rows, k_map, v_map, stream)                              \
               : launch_coop<64, ST, false, W>(p, box_rows, k_map, v_map, stream);
    // an upper bound of the 32-key blocks a CTA walks: the block table's width over the splits
    const int64_t bound_keys = p.window > 0 ? (int64_t)p.window : (int64_t)p.table_width * p.page_size;
    switch (decode_config(p.num_splits, bound_keys / (p.num_splits > 0 ? p.num_splits : 1) / 32)) {
      case 2: AKV_COOP(2, 2)
      case 4: AKV_COOP(2, 4)
      case 6: AKV_COOP(3, 2)
      default: AKV_COOP(3, 4)
    }
#undef AKV_COOP
  }
  // Prompt tiles: 64-key blocks, three stages, two CTAs per SM.  A variant with 32-key blocks and three CTAs per SM
  // (AKV_PROMPT_CONFIG=32, groups of up to four q-heads) measured the same on a 2,048-token prompt (294 vs 290 us)
  // and worse on a 512-token portion after 7,680 keys (638 vs 510 us).
  if (kt == 32) {
    if (p.head_dim == 128) return launch_prompt<128, 32, 3, 4, 3>(p, box_rows, k_map, v_map, stream);
    return launch_prompt<64, 32, 3, 4, 3>(p, box_rows, k_map, v_map, stream);
  }
  if (p.head_dim == 128) return launch_prompt<128, 64, 3, 8, 1>(p, box_rows, k_map, v_map, stream);
  return launch_prompt<64, 64, 3, 8, 1>(p, box_rows, k_map, v_map, stream);
}

}  // namespace akv
