// Paged causal GQA attention over the block tables, for prompt portions and decoded tokens in
// one launch: the general kernel (float arithmetic on CUDA cores, any head size that is a
// multiple of 16 up to 256, any group size, float32 or bfloat16 pages).  It is the whole
// attention of the float32 path and the fallback of the bfloat16 path for sizes its
// tensor-core kernels do not take.
//
// What it replaces: F.scaled_dot_product_attention over a gathered copy of the history
// (ampere_kv/kv_cache.py:76-94 with the read-back of ampere_kv/paged_cache.py:109-121) and
// the decode kernels csrc/paged_decode.cu:119-257 / :404-496 with their merge :528-544.
// Same mathematics: score = q.k * scale, query at absolute position t sees key j iff j <= t
// (and j > t - window when a window is set), softmax and the weighted sum of V in float32,
// q-head h reads kv-head h / G.
//
// Work split.  A query tile is up to q_tile consecutive tokens of one sequence; its rows are
// (token, head-in-group) pairs, R to a warp.  One warp owns (tile, kv head, row group, key
// split): it walks its key range 32 keys at a time, lane = key for the scores (K row read
// once for all R rows, q broadcast from shared memory), then lane = dims for P.V.  Keys are
// never re-read per q-head of a group.  With one split the warp writes the output row; with
// more it writes (acc, max, sum) partials and a second kernel merges them in split order.
#include "common.cuh"
#include "launchers.h"

#include <math_constants.h>

namespace akv {

constexpr int kAttnWarps = 4;
constexpr int kAttnRows = 8;

template <typename T, int DC>
__global__ void __launch_bounds__(kAttnWarps * 32)
paged_attention_kernel(PagedAttentionParams p, int row_groups, int64_t total_items) {
  constexpr int R = kAttnRows;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t item = (int64_t)blockIdx.x * kAttnWarps + warp;
  if (item >= total_items) return;
  const int D = p.head_dim, NH = p.num_heads, NKV = p.num_kv_heads, G = NH / NKV, P = p.page_size;
  const int rg = (int)(item % row_groups);
  const int kvh = (int)((item / row_groups) % NKV);
  const int split = (int)((item / ((int64_t)row_groups * NKV)) % p.num_splits);
  const int tile = (int)(item / ((int64_t)row_groups * NKV * p.num_splits));

  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int nq = p.tile_nq[tile];
  const int rows_in_tile = nq * G;
  const int row0 = rg * R;
  if (row0 >= rows_in_tile) return;
  const int nrows = min(R, rows_in_tile - row0);
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  // absolute position of the tile's first token
  const int tile_pos = ctx - q_len + (q0 - seq_q0);

  extern __shared__ float smem[];
  float* qs = smem + warp * (R * D + R * 32);
  float* ps = qs + R * D;

  const T* q = (const T*)p.q;
  for (int idx = lane; idx < R * D; idx += 32) {
    const int r = idx / D, d = idx - r * D;
    float v = 0.f;
    if (r < nrows) {
      const int rr = row0 + r;
      const int64_t token = q0 + rr / G;
      const int head = kvh * G + rr % G;
      v = to_float<T>(q[(token * NH + head) * (int64_t)D + d]) * p.scale;
    }
    qs[idx] = v;
  }
  __syncwarp();

  int pos[R];
#pragma unroll
  for (int r = 0; r < R; ++r) pos[r] = (r < nrows) ? tile_pos + (row0 + r) / G : -1;
  const int pos_first = tile_pos + row0 / G;
  const int pos_last = tile_pos + (row0 + nrows - 1) / G;
  const int lo_item = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int hi_item = pos_last + 1;
  int per = (hi_item - lo_item + p.num_splits - 1) / p.num_splits;
  per = (per + 31) & ~31;
  const int start = lo_item + split * per;
  const int end = min(hi_item, start + per);

  float m[R], l[R], acc[R][DC];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -CUDART_INF_F;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  }

  const T* k_cache = (const T*)p.k_cache;
  const T* v_cache = (const T*)p.v_cache;
  const int32_t* table = p.block_table + (int64_t)seq * p.table_width;

  for (int kb = start; kb < end; kb += 32) {
    const int key = kb + lane;
    bool kvalid = key < end;
    int page = 0;
    if (kvalid) {
      const int logical = key / P;
      page = logical < p.table_width ? table[logical] : -1;
      if (page < 0 || page >= p.num_pages) {
        set_status(p.status, kBadPage);
        kvalid = false;
        page = 0;
      }
    }
    const int off = key % P;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = 0.f;
    if (kvalid) {
      const T* kptr = k_cache + (((int64_t)page * NKV + kvh) * P + off) * (int64_t)D;
#pragma unroll 2
      for (int d0 = 0; d0 < D; d0 += 8) {
        float kf[8];
        load8<T>(kptr + d0, kf);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(qs + r * D + d0);
          const float4 b = *reinterpret_cast<const float4*>(qs + r * D + d0 + 4);
          s[r] += a.x * kf[0] + a.y * kf[1] + a.z * kf[2] + a.w * kf[3] + b.x * kf[4] + b.y * kf[5] +
                  b.z * kf[6] + b.w * kf[7];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool visible = kvalid && key <= pos[r] && (p.window <= 0 || key > pos[r] - p.window);
      const float sr = visible ? s[r] : -CUDART_INF_F;
      const float m_new = fmaxf(m[r], warp_max(sr));
      const float alpha = (m_new == -CUDART_INF_F) ? 1.f : expf(m[r] - m_new);
      const float pr = visible ? expf(sr - m_new) : 0.f;
      l[r] = l[r] * alpha + pr;
      m[r] = m_new;
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] *= alpha;
      ps[r * 32 + lane] = pr;
    }
    __syncwarp();
    const int nk = min(32, end - kb);
    for (int j = 0; j < nk; ++j) {
      const int pj = __shfl_sync(0xffffffffu, page, j);
      const int offj = (kb + j) % P;
      const T* vptr = v_cache + (((int64_t)pj * NKV + kvh) * P + offj) * (int64_t)D;
      float vv[DC];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = c * 32 + lane;
        vv[c] = d < D ? to_float<T>(vptr[d]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float pr = ps[r * 32 + j];
#pragma unroll
        for (int c = 0; c < DC; ++c) acc[r][c] += pr * vv[c];
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (r >= nrows) continue;
    const float total = warp_sum(l[r]);
    const int rr = row0 + r;
    const int64_t token = q0 + rr / G;
    const int head = kvh * G + rr % G;
    const int64_t row = token * NH + head;
    if (p.num_splits == 1) {
      T* o = (T*)p.out + row * (int64_t)D;
      const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = c * 32 + lane;
        if (d < D) o[d] = from_float<T>(acc[r][c] * inv);
      }
    } else {
      float* part = p.partials + (row * p.num_splits + split) * (int64_t)(D + 2);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = c * 32 + lane;
        if (d < D) part[d] = acc[r][c];
      }
      if (lane == 0) {
        part[D] = m[r];
        part[D + 1] = total;
      }
    }
  }
}

// out[row] = sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) l_s, splits taken in order.  One block per (tile, row
// of the tile, q-head): only the rows of the call's tiles are merged and written.  (A batch may be covered by two
// calls with different tiles and split counts; the other call's rows have no partial sums in this call's
// workspace and their results must stay.)
template <typename T>
__global__ void merge_splits_kernel(const float* __restrict__ partials, T* __restrict__ out,
                                    const int32_t* __restrict__ tile_q0, const int32_t* __restrict__ tile_nq,
                                    int q_tile, int num_heads, int num_splits, int head_dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t per_tile = (int64_t)q_tile * num_heads;
  const int64_t tile = blockIdx.x / per_tile;
  const int in_tile = (int)(blockIdx.x - tile * per_tile);
  const int r = in_tile / num_heads, head = in_tile - r * num_heads;
  if (r >= tile_nq[tile]) return;
  const int64_t row = ((int64_t)tile_q0[tile] + r) * num_heads + head;
  const float* base = partials + row * num_splits * (int64_t)(head_dim + 2);
  float m = -CUDART_INF_F;
  for (int s = 0; s < num_splits; ++s) {
    const float* part = base + (int64_t)s * (head_dim + 2);
    if (part[head_dim + 1] > 0.f) m = fmaxf(m, part[head_dim]);
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float* part = base + (int64_t)s * (head_dim + 2);
      const float ls = part[head_dim + 1];
      if (ls > 0.f) {
        const float w = expf(part[head_dim] - m);
        num += w * part[d];
        den += w * ls;
      }
    }
    out[row * head_dim + d] = from_float<T>(den > 0.f ? num / den : 0.f);
  }
}

template <typename T>
static int launch_merge(const PagedAttentionParams& p, cudaStream_t stream) {
  const int64_t blocks = (int64_t)p.num_tiles * p.q_tile * p.num_heads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (blocks == 0) return 0;
  const int threads = p.head_dim <= 32 ? 32 : (p.head_dim <= 64 ? 64 : 128);
  merge_splits_kernel<T><<<(unsigned)blocks, threads, 0, stream>>>(p.partials, (T*)p.out, p.tile_q0, p.tile_nq, p.q_tile,
                                                                    p.num_heads, p.num_splits, p.head_dim);
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_typed(const PagedAttentionParams& p, cudaStream_t stream) {
  const int G = p.num_heads / p.num_kv_heads;
  const int row_groups = (p.q_tile * G + kAttnRows - 1) / kAttnRows;
  const int64_t total = (int64_t)p.num_tiles * p.num_kv_heads * row_groups * p.num_splits;
  const int64_t blocks = (total + kAttnWarps - 1) / kAttnWarps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)kAttnWarps * (kAttnRows * p.head_dim + kAttnRows * 32) * sizeof(float);
  const int dc = (p.head_dim + 31) / 32;
#define AKV_LAUNCH(DCV)                                                                             \
  case DCV:                                                                                         \
    paged_attention_kernel<T, DCV><<<(unsigned)blocks, kAttnWarps * 32, smem, stream>>>(p, row_groups, \
                                                                                         total);    \
    break;
  switch (dc) {
    AKV_LAUNCH(1) AKV_LAUNCH(2) AKV_LAUNCH(3) AKV_LAUNCH(4)
    AKV_LAUNCH(5) AKV_LAUNCH(6) AKV_LAUNCH(7) AKV_LAUNCH(8)
    default: return (int)cudaErrorInvalidValue;
  }
#undef AKV_LAUNCH
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return (int)err;
  return p.num_splits > 1 ? launch_merge<T>(p, stream) : 0;
}

int launch_paged_attention(const PagedAttentionParams& p, cudaStream_t stream) {
  if (p.num_tiles == 0 || p.num_tokens == 0) return 0;
  if (p.head_dim % 16 || p.head_dim > 256 || p.num_heads % p.num_kv_heads || p.num_splits < 1)
    return (int)cudaErrorInvalidValue;
  if ((p.kernel == 0 || p.kernel == 3 || p.kernel == 4) && p.q_tile > 1 && attention_tcgen05_supported(p)) {
    PagedAttentionParams q = p;
    q.num_splits = 1;
    return launch_attention_tcgen05(q, stream);
  }
  if (p.kernel != 1 && attention_tc_supported(p)) {
    PagedAttentionParams q = p;
    if (q.q_tile > 1) q.num_splits = 1;          // the prompt kernel walks all keys of a tile itself
    const int err = launch_attention_tc(q, stream);
    if (err != 0) return err;
    return (q.num_splits > 1 && !attention_tc_merges_in_kernel(q)) ? launch_merge<__nv_bfloat16>(q, stream) : 0;
  }
  return p.dtype == kBFloat16 ? launch_typed<__nv_bfloat16>(p, stream) : launch_typed<float>(p, stream);
}

}  // namespace akv
