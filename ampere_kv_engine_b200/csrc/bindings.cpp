// Python bindings of the extension `_C`: one function per kernel family.  Every function
// validates device, dtype, shape and contiguity of what it is given and raises a Python
// error that names the argument; nothing is allocated here (callers pass outputs and
// workspaces), so every call can be captured into a CUDA graph.  The reference's extension
// has the same split between checked entry points and launchers (csrc/bindings.cpp:43-73,
// csrc/paged_decode.cu:567-632), but guards indices with device asserts; here a bad index
// sets a code in the `status` tensor instead and the access is skipped.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <pybind11/stl.h>

#include <string>
#include <utility>
#include <vector>

#include "launchers.h"

namespace py = pybind11;

namespace {

using at::Tensor;
using OptTensor = c10::optional<at::Tensor>;

// Error text is put together with std::string only (no iostream formatting in this file).
inline std::string text(const std::string& v) { return v; }
inline std::string text(const char* v) { return std::string(v); }
inline std::string text(int64_t v) { return std::to_string(v); }
inline std::string text(int v) { return std::to_string(v); }
inline std::string text(double v) { return std::to_string(v); }
inline std::string text(at::ScalarType v) { return std::string(c10::toString(v)); }
inline std::string join() { return std::string(); }
template <typename First, typename... Rest>
std::string join(const First& first, const Rest&... rest) { return text(first) + join(rest...); }

#define AKV_CHECK(cond, ...)                          \
  do {                                                \
    if (!(cond)) {                                    \
      const std::string akv_message = join(__VA_ARGS__); \
      TORCH_CHECK(false, akv_message);                \
    }                                                 \
  } while (0)

void check_cuda(const Tensor& t, const char* name) {
  AKV_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  AKV_CHECK(t.is_contiguous(), name, " must be contiguous");
}

int dtype_code(const Tensor& t, const char* name) {
  if (t.scalar_type() == at::kFloat) return 0;
  if (t.scalar_type() == at::kBFloat16) return 1;
  AKV_CHECK(false, name, " must be float32 or bfloat16, got ", t.scalar_type());
  return -1;
}

void check_same(const Tensor& a, const Tensor& b, const char* an, const char* bn) {
  AKV_CHECK(a.scalar_type() == b.scalar_type(), an, " and ", bn, " must have the same dtype");
  AKV_CHECK(a.device() == b.device(), an, " and ", bn, " must be on the same device");
}

void check_i32(const Tensor& t, const char* name, int64_t numel = -1) {
  check_cuda(t, name);
  AKV_CHECK(t.scalar_type() == at::kInt, name, " must be int32");
  if (numel >= 0) AKV_CHECK(t.numel() >= numel, name, " must hold at least ", numel, " entries, has ", t.numel());
}

void check_f32(const Tensor& t, const char* name, int64_t numel = -1) {
  check_cuda(t, name);
  AKV_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
  if (numel >= 0) AKV_CHECK(t.numel() == numel, name, " must hold ", numel, " entries, has ", t.numel());
}

int* status_ptr(const OptTensor& status) {
  if (!status.has_value()) return nullptr;
  check_i32(*status, "status", 1);
  return status->data_ptr<int>();
}

void check_launch(int err, const char* what) {
  AKV_CHECK(err == 0, what, ": launch failed: ", cudaGetErrorString((cudaError_t)err));
}

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

Tensor smoke_add(const Tensor& a, const Tensor& b) {
  check_f32(a, "a");
  check_f32(b, "b", a.numel());
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = at::empty_like(a);
  check_launch(akv::launch_smoke_add(a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(), a.numel(),
                                     stream_of(a)),
               "smoke_add");
  return out;
}

void wait_selftest(int64_t limit, Tensor& status) {
  check_i32(status, "status", 1);
  AKV_CHECK(limit >= 1 && limit <= 1000000, "limit must be between 1 and 1000000 tries");
  c10::cuda::CUDAGuard guard(status.device());
  check_launch(akv::launch_wait_selftest((uint32_t)limit, status.data_ptr<int>(), stream_of(status)), "wait_selftest");
}

void embedding(const Tensor& ids, const Tensor& table, Tensor& hidden, const OptTensor& status,
               const OptTensor& sampled) {
  check_cuda(table, "table");
  AKV_CHECK(table.dim() == 2, "table must be [vocab, hidden]");
  const int64_t n = ids.numel(), h = table.size(1);
  check_i32(ids, "ids");
  check_f32(hidden, "hidden", n * h);
  const int* sampled_ptr = nullptr;
  int64_t num_sampled = 0;
  if (sampled.has_value()) {
    check_i32(*sampled, "sampled");
    sampled_ptr = sampled->data_ptr<int>();
    num_sampled = sampled->numel();
  }
  c10::cuda::CUDAGuard guard(table.device());
  check_launch(akv::launch_embedding(ids.data_ptr<int>(), sampled_ptr, num_sampled, table.data_ptr(),
                                     hidden.data_ptr<float>(), n, h,
                                     table.size(0), dtype_code(table, "table"), status_ptr(status),
                                     stream_of(table)),
               "embedding");
}

void add_rmsnorm(Tensor& hidden, const OptTensor& delta, const Tensor& weight, Tensor& out, const OptTensor& rows,
                 double eps, const OptTensor& status) {
  check_cuda(hidden, "hidden");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && hidden.dim() == 2, "hidden must be float32 [tokens, hidden]");
  const int64_t n = hidden.size(0), h = hidden.size(1);
  check_f32(weight, "weight", h);
  check_cuda(out, "out");
  const int code = dtype_code(out, "out");
  AKV_CHECK(h * 4 <= 200 * 1024, "add_rmsnorm: hidden size ", h, " exceeds the kernel's limit of 51200");
  const void* delta_ptr = nullptr;
  int delta_parts = 0;
  if (delta.has_value()) {
    check_cuda(*delta, "delta");
    if (delta->dim() == 3) {
      // float32 partial sums of a split-K product, [parts, tokens, hidden]
      AKV_CHECK(delta->scalar_type() == at::kFloat, "a 3-D delta holds float32 partial sums");
      AKV_CHECK(delta->size(0) >= 1 && delta->size(1) == n && delta->size(2) == h,
                "a 3-D delta must be [parts, tokens, hidden]");
      delta_parts = (int)delta->size(0);
    } else {
      check_same(*delta, out, "delta", "out");
      AKV_CHECK(delta->numel() == n * h, "delta must be [tokens, hidden]");
    }
    delta_ptr = delta->data_ptr();
  }
  const int* rows_ptr = nullptr;
  int64_t num_rows = 0;
  if (rows.has_value()) {
    check_i32(*rows, "rows");
    rows_ptr = rows->data_ptr<int>();
    num_rows = rows->numel();
    AKV_CHECK(out.numel() == num_rows * h, "out must be [rows, hidden]");
  } else {
    AKV_CHECK(out.numel() == n * h, "out must be [tokens, hidden]");
  }
  c10::cuda::CUDAGuard guard(hidden.device());
  check_launch(akv::launch_add_rmsnorm(hidden.data_ptr<float>(), delta_ptr, delta_parts, weight.data_ptr<float>(),
                                       out.data_ptr(),
                                       rows_ptr, num_rows, n, h, (float)eps, code, status_ptr(status),
                                       stream_of(hidden)),
               "add_rmsnorm");
}

void silu_mul(const Tensor& gate_up, Tensor& out, int64_t block) {
  check_cuda(gate_up, "gate_up");
  check_cuda(out, "out");
  int parts = 0;
  Tensor first = gate_up;
  if (gate_up.dim() == 3) {
    AKV_CHECK(gate_up.scalar_type() == at::kFloat, "a 3-D gate_up holds float32 partial sums");
    parts = (int)gate_up.size(0);
    AKV_CHECK(parts >= 1, "gate_up must hold at least one part");
    first = gate_up.select(0, 0);
    AKV_CHECK(first.device() == out.device(), "gate_up and out must be on the same device");
  } else {
    check_same(gate_up, out, "gate_up", "out");
  }
  AKV_CHECK(first.dim() == 2 && first.size(1) % 2 == 0, "gate_up must be [tokens, 2 * intermediate]");
  const int64_t n = first.size(0), inter = first.size(1) / 2;
  AKV_CHECK(out.numel() == n * inter, "out must be [tokens, intermediate]");
  if (block == 0) block = inter;
  AKV_CHECK(inter == 0 || (block > 0 && inter % block == 0),
            "the run length of gate and up columns must divide the intermediate size, got ", block, " for ", inter);
  c10::cuda::CUDAGuard guard(gate_up.device());
  check_launch(akv::launch_silu_mul(gate_up.data_ptr(), parts, out.data_ptr(), n, inter, block,
                                    dtype_code(out, "out"), stream_of(out)),
               "silu_mul");
}

// The token operand of the small-batch product: either x [tokens, k] bfloat16, or the RMS norm of a float32
// residual stream that the kernel applies itself (hidden [tokens, k], ssq [tiles, tokens] partial sums of squares
// left by a product with the residual epilogue, the norm's weight [k] and eps).
struct TokenOperand {
  const void* x = nullptr;
  akv::GemmNormedX normed = {};
  bool is_normed = false;
  int64_t tokens = 0, k = 0;
  const Tensor* anchor = nullptr;     // device and stream
};

TokenOperand token_operand(const OptTensor& x, const OptTensor& nx_hidden, const OptTensor& nx_ssq,
                           const OptTensor& nx_weight, double nx_eps, const Tensor& w) {
  check_cuda(w, "w");
  AKV_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2, "w must be bfloat16 [features, k]");
  AKV_CHECK(reinterpret_cast<uintptr_t>(w.data_ptr()) % 16 == 0, "w must be 16-byte aligned");
  TokenOperand t;
  if (x.has_value()) {
    AKV_CHECK(!nx_hidden.has_value(), "give x or the residual stream to norm, not both");
    check_cuda(*x, "x");
    AKV_CHECK(x->scalar_type() == at::kBFloat16 && x->dim() == 2 && x->size(1) == w.size(1),
              "x must be bfloat16 [tokens, k] for w [features, k]");
    AKV_CHECK(reinterpret_cast<uintptr_t>(x->data_ptr()) % 16 == 0, "x must be 16-byte aligned");
    t.x = x->data_ptr();
    t.tokens = x->size(0);
    t.anchor = &*x;
  } else {
    AKV_CHECK(nx_hidden.has_value() && nx_ssq.has_value() && nx_weight.has_value(),
              "without x the product needs the residual stream, its sums of squares and the norm's weight");
    check_cuda(*nx_hidden, "hidden");
    AKV_CHECK(nx_hidden->scalar_type() == at::kFloat && nx_hidden->dim() == 2 && nx_hidden->size(1) == w.size(1),
              "hidden must be float32 [tokens, k] for w [features, k]");
    AKV_CHECK(reinterpret_cast<uintptr_t>(nx_hidden->data_ptr()) % 16 == 0, "hidden must be 16-byte aligned");
    t.tokens = nx_hidden->size(0);
    check_cuda(*nx_ssq, "ssq");
    AKV_CHECK(nx_ssq->scalar_type() == at::kFloat && nx_ssq->dim() == 2 && nx_ssq->size(0) >= 1 &&
                  nx_ssq->size(1) == t.tokens, "ssq must be float32 [tiles, tokens]");
    check_f32(*nx_weight, "the norm's weight", w.size(1));
    AKV_CHECK(reinterpret_cast<uintptr_t>(nx_weight->data_ptr()) % 16 == 0, "the norm's weight must be 16-byte aligned");
    t.is_normed = true;
    t.normed.hidden = nx_hidden->data_ptr<float>();
    t.normed.ssq = nx_ssq->data_ptr<float>();
    t.normed.weight = nx_weight->data_ptr<float>();
    t.normed.ssq_tiles = (int)nx_ssq->size(0);
    t.normed.eps = (float)nx_eps;
    t.anchor = &*nx_hidden;
  }
  t.k = w.size(1);
  AKV_CHECK(w.device() == t.anchor->device(), "w and the token operand must be on the same device");
  AKV_CHECK(akv::small_m_gemm_supported(t.tokens, w.size(0), t.k),
            "small_m_gemm takes 1..64 tokens and a K that is a multiple of 8 and at least 64; got ", t.tokens,
            " tokens, K = ", t.k);
  return t;
}

void check_cluster_splits(int64_t splits, int64_t k) {
  AKV_CHECK((splits == 1 || splits == 2 || splits == 4 || splits == 8) && splits <= (k + 63) / 64,
            "splits must be 1, 2, 4 or 8 and at most the number of 64-element K blocks, got ", splits);
}

// x @ w^T for few tokens on the tcgen05 tensor cores.  `out` is either [tokens, features] (float32 or bfloat16:
// the K splits are added up inside the kernel) or a 3-D float32 [splits, tokens, features] that receives every
// split's partial sum as it is.  gated: w holds gate and up rows in alternating runs of 64 and out is
// silu(gate) * up, [tokens, features / 2] bfloat16.
void small_m_gemm(const OptTensor& x, const Tensor& w, Tensor& out, int64_t splits, const OptTensor& status,
                  bool gated, const OptTensor& nx_hidden, const OptTensor& nx_ssq, const OptTensor& nx_weight,
                  double nx_eps) {
  const TokenOperand t = token_operand(x, nx_hidden, nx_ssq, nx_weight, nx_eps, w);
  check_cuda(out, "out");
  AKV_CHECK(out.device() == w.device(), "out and w must be on the same device");
  void* out_ptr = nullptr;
  float* parts_ptr = nullptr;
  int out_code = 0;
  if (out.dim() == 3) {
    AKV_CHECK(out.scalar_type() == at::kFloat && out.size(1) == t.tokens && out.size(2) == w.size(0),
              "a 3-D out must be float32 [splits, tokens, features]");
    splits = out.size(0);
    AKV_CHECK(splits >= 1 && splits <= (t.k + 63) / 64, "splits must be between 1 and the number of 64-element K blocks");
    AKV_CHECK(!gated && !t.is_normed, "partial sums come from the plain product of a given x only");
    parts_ptr = out.data_ptr<float>();
  } else {
    if (gated) {
      AKV_CHECK(w.size(0) % 128 == 0 && out.scalar_type() == at::kBFloat16,
                "the gated epilogue takes a weight of gate and up rows in alternating runs of 64 (rows a multiple "
                "of 128) and a bfloat16 out");
      AKV_CHECK(out.dim() == 2 && out.size(0) == t.tokens && out.size(1) * 2 == w.size(0),
                "a gated out must be [tokens, features / 2]");
    } else {
      AKV_CHECK(out.dim() == 2 && out.size(0) == t.tokens && out.size(1) == w.size(0),
                "out must be [tokens, features]");
    }
    check_cluster_splits(splits, t.k);
    out_code = dtype_code(out, "out");
    out_ptr = out.data_ptr();
  }
  akv::GemmFusion f;
  f.epilogue = gated ? akv::kEpilogueGated : akv::kEpiloguePlain;
  f.normed_x = t.is_normed;
  f.normed = t.normed;
  c10::cuda::CUDAGuard guard(w.device());
  check_launch(akv::launch_small_m_gemm(t.x, w.data_ptr(), out_ptr, out_code, parts_ptr, t.tokens, w.size(0), t.k,
                                        (int)splits, &f, status_ptr(status), stream_of(*t.anchor)),
               "small_m_gemm");
}

// The product added to the float32 residual stream in place: hidden [tokens, features] += bfloat16(x @ w^T), and
// ssq [ceil(features / 128), tokens] receives each 128-feature tile's sum of squares of the new values.
void small_m_gemm_residual(const Tensor& x, const Tensor& w, Tensor& hidden, Tensor& ssq, int64_t splits,
                           const OptTensor& status) {
  const TokenOperand t = token_operand(x, OptTensor(), OptTensor(), OptTensor(), 0.0, w);
  check_cuda(hidden, "hidden");
  check_cuda(ssq, "ssq");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && hidden.dim() == 2 && hidden.size(0) == t.tokens &&
                hidden.size(1) == w.size(0) && hidden.device() == w.device(),
            "hidden must be float32 [tokens, features] on w's device");
  AKV_CHECK(ssq.scalar_type() == at::kFloat && ssq.dim() == 2 && ssq.size(0) == (w.size(0) + 127) / 128 &&
                ssq.size(1) == t.tokens && ssq.device() == w.device(),
            "ssq must be float32 [ceil(features / 128), tokens] on w's device");
  check_cluster_splits(splits, t.k);
  akv::GemmFusion f;
  f.epilogue = akv::kEpilogueResidual;
  f.residual.hidden = hidden.data_ptr<float>();
  f.residual.ssq = ssq.data_ptr<float>();
  c10::cuda::CUDAGuard guard(w.device());
  check_launch(akv::launch_small_m_gemm(t.x, w.data_ptr(), nullptr, 0, nullptr, t.tokens, w.size(0), t.k, (int)splits,
                                        &f, status_ptr(status), stream_of(x)),
               "small_m_gemm_residual");
}

bool small_m_gemm_supported(int64_t tokens, int64_t features, int64_t k) {
  return akv::small_m_gemm_supported(tokens, features, k);
}

int64_t small_m_gemm_splits(int64_t features, int64_t k) { return akv::small_m_gemm_splits(features, k); }

struct CacheGeometry {
  int64_t num_pages;
  int num_kv_heads, page_size, head_dim;
};

CacheGeometry check_cache(const Tensor& k_cache, const Tensor& v_cache, int num_kv_heads, int head_dim,
                          const Tensor& like) {
  check_cuda(k_cache, "k_cache");
  check_cuda(v_cache, "v_cache");
  check_same(k_cache, v_cache, "k_cache", "v_cache");
  check_same(k_cache, like, "k_cache", "activations");
  AKV_CHECK(k_cache.dim() == 4 && k_cache.sizes() == v_cache.sizes(),
              "k_cache and v_cache must both be [pages, kv_heads, page_size, head_dim]");
  AKV_CHECK(k_cache.size(1) == num_kv_heads && k_cache.size(3) == head_dim, "cache pages are [",
              k_cache.size(1), " kv heads, ", k_cache.size(3), " dims], the call says [", num_kv_heads, ", ",
              head_dim, "]");
  return {k_cache.size(0), num_kv_heads, (int)k_cache.size(2), head_dim};
}

// The q/k/v projection of few tokens with per-head norm, rotation and the cache write done on the output tile
// (heads of 128 dims, the whole head rotated or none of it).  q_out [tokens, heads * 128]; K and V go to the
// slots of the cache pages when slots and caches are given, and are dropped otherwise.
void small_m_gemm_qkv(const OptTensor& x, const Tensor& w, Tensor& q_out, const Tensor& positions,
                      const OptTensor& slots, const OptTensor& q_weight, const OptTensor& k_weight,
                      const OptTensor& inv_freq, const OptTensor& k_cache, const OptTensor& v_cache,
                      int64_t num_heads, int64_t num_kv_heads, double eps, int64_t splits, const OptTensor& status,
                      const OptTensor& nx_hidden, const OptTensor& nx_ssq, const OptTensor& nx_weight,
                      double nx_eps) {
  const TokenOperand t = token_operand(x, nx_hidden, nx_ssq, nx_weight, nx_eps, w);
  check_cuda(q_out, "q_out");
  AKV_CHECK(q_out.scalar_type() == at::kBFloat16 && q_out.device() == w.device(),
            "q_out must be bfloat16 on w's device");
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && w.size(0) == (num_heads + 2 * num_kv_heads) * 128,
            "w must hold (heads + 2 kv_heads) heads of 128 rows each, got ", w.size(0), " rows");
  const int64_t n = t.tokens;
  check_cluster_splits(splits, t.k);
  AKV_CHECK(q_out.is_contiguous() && q_out.numel() == n * num_heads * 128, "q_out must be [tokens, heads * 128]");
  check_i32(positions, "positions", n);
  akv::GemmQkv e{};
  e.positions = positions.data_ptr<int>();
  e.q_out = q_out.data_ptr();
  if (slots.has_value()) {
    check_i32(*slots, "slots", n);
    e.slots = slots->data_ptr<int>();
  }
  if (q_weight.has_value()) { check_f32(*q_weight, "q_weight", 128); e.q_weight = q_weight->data_ptr<float>(); }
  if (k_weight.has_value()) { check_f32(*k_weight, "k_weight", 128); e.k_weight = k_weight->data_ptr<float>(); }
  if (inv_freq.has_value()) { check_f32(*inv_freq, "inv_freq", 64); e.inv_freq = inv_freq->data_ptr<float>(); }
  AKV_CHECK(k_cache.has_value() == v_cache.has_value(), "k_cache and v_cache come together");
  if (k_cache.has_value()) {
    AKV_CHECK(slots.has_value(), "a cache to write needs slots");
    const CacheGeometry g = check_cache(*k_cache, *v_cache, (int)num_kv_heads, 128, q_out);
    e.k_cache = k_cache->data_ptr();
    e.v_cache = v_cache->data_ptr();
    e.num_pages = g.num_pages;
    e.page_size = g.page_size;
  }
  e.num_heads = (int)num_heads;
  e.num_kv_heads = (int)num_kv_heads;
  e.eps = (float)eps;
  akv::GemmFusion f;
  f.epilogue = akv::kEpilogueQkv;
  f.qkv = e;
  f.normed_x = t.is_normed;
  f.normed = t.normed;
  c10::cuda::CUDAGuard guard(w.device());
  check_launch(akv::launch_small_m_gemm(t.x, w.data_ptr(), nullptr, 0, nullptr, n, w.size(0), t.k, (int)splits, &f,
                                        status_ptr(status), stream_of(*t.anchor)),
               "small_m_gemm_qkv");
}

// A chain of products in one persistent kernel (launchers.h: launch_stream_phases).  `phases` is a list of dicts:
//   w [features, k] bfloat16; x [tokens, k] bfloat16 or None with norm_weight [k] float32 and eps (the token operand
//   is then the RMS norm of `hidden`); epilogue: "residual" (adds into hidden), "gated" (out [tokens, features / 2]),
//   "plain" (out [tokens, features]) or "qkv" (q_out, positions, slots, q_weight, k_weight, inv_freq, k_cache,
//   v_cache, num_heads, num_kv_heads, qk_eps: the arguments of small_m_gemm_qkv).
// ssq [ceil(hidden / 128), tokens] float32 scratch; parts and sync as stream_phases_scratch says, sync zeroed.
akv::StreamPhase parse_stream_phase(const py::dict& d, const Tensor& hidden, int64_t tokens) {
  akv::StreamPhase ph = {};
  const Tensor w = d["w"].cast<Tensor>();
  check_cuda(w, "w");
  AKV_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.device() == hidden.device(),
            "a phase's w must be a bfloat16 matrix on hidden's device");
  ph.w = w.data_ptr();
  ph.features = w.size(0);
  ph.k = w.size(1);
  AKV_CHECK(reinterpret_cast<uintptr_t>(ph.w) % 16 == 0 && ph.k % 8 == 0 && ph.k >= 64,
            "a phase's w must be 16-byte aligned with k a multiple of 8, at least 64");
  const std::string epilogue = d["epilogue"].cast<std::string>();
  if (d.contains("x") && !d["x"].is_none()) {
    const Tensor x = d["x"].cast<Tensor>();
    check_cuda(x, "x");
    AKV_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(0) == tokens && x.size(1) == ph.k &&
                  x.device() == hidden.device() && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0,
              "a phase's x must be bfloat16 [tokens, k], 16-byte aligned, on hidden's device");
    ph.x_kind = akv::kStreamXTensor;
    ph.x = x.data_ptr();
  } else {
    const Tensor nw = d["norm_weight"].cast<Tensor>();
    check_f32(nw, "norm_weight", ph.k);
    AKV_CHECK(ph.k == hidden.size(1) && reinterpret_cast<uintptr_t>(nw.data_ptr()) % 16 == 0,
              "a normed token operand has the residual stream's width and a 16-byte aligned weight");
    ph.x_kind = akv::kStreamXNormed;
    ph.norm_weight = nw.data_ptr<float>();
    ph.eps = d["eps"].cast<float>();
  }
  if (epilogue == "residual") {
    ph.epilogue = akv::kEpilogueResidual;
    AKV_CHECK(ph.features == hidden.size(1), "a residual phase has as many features as the residual stream");
  } else if (epilogue == "gated" || epilogue == "plain") {
    ph.epilogue = epilogue == "gated" ? akv::kEpilogueGated : akv::kEpiloguePlain;
    Tensor out = d["out"].cast<Tensor>();
    check_cuda(out, "out");
    const int64_t width = epilogue == "gated" ? ph.features / 2 : ph.features;
    AKV_CHECK(out.scalar_type() == at::kBFloat16 && out.numel() == tokens * width && out.device() == hidden.device(),
              "a phase's out must be bfloat16 [tokens, ", width, "] on hidden's device");
    AKV_CHECK(epilogue != "gated" || ph.features % 128 == 0, "a gated phase needs features in whole tiles of 128");
    ph.out = out.data_ptr();
  } else if (epilogue == "qkv") {
    ph.epilogue = akv::kEpilogueQkv;
    akv::GemmQkv& e = ph.qkv;
    e.num_heads = d["num_heads"].cast<int>();
    e.num_kv_heads = d["num_kv_heads"].cast<int>();
    e.eps = d["qk_eps"].cast<float>();
    AKV_CHECK(e.num_heads > 0 && e.num_kv_heads > 0 && ph.features == (int64_t)(e.num_heads + 2 * e.num_kv_heads) * 128,
              "a qkv phase's w holds (heads + 2 kv_heads) heads of 128 rows each");
    Tensor q_out = d["q_out"].cast<Tensor>();
    check_cuda(q_out, "q_out");
    AKV_CHECK(q_out.scalar_type() == at::kBFloat16 && q_out.numel() == tokens * e.num_heads * 128 &&
                  q_out.device() == hidden.device(), "q_out must be bfloat16 [tokens, heads * 128]");
    e.q_out = q_out.data_ptr();
    const Tensor positions = d["positions"].cast<Tensor>();
    check_i32(positions, "positions", tokens);
    e.positions = positions.data_ptr<int>();
    auto opt = [&](const char* key) -> OptTensor {
      if (!d.contains(key) || d[key].is_none()) return c10::nullopt;
      return d[key].cast<Tensor>();
    };
    const OptTensor slots = opt("slots"), qw = opt("q_weight"), kw = opt("k_weight"), freq = opt("inv_freq");
    const OptTensor k_cache = opt("k_cache"), v_cache = opt("v_cache");
    if (slots.has_value()) { check_i32(*slots, "slots", tokens); e.slots = slots->data_ptr<int>(); }
    if (qw.has_value()) { check_f32(*qw, "q_weight", 128); e.q_weight = qw->data_ptr<float>(); }
    if (kw.has_value()) { check_f32(*kw, "k_weight", 128); e.k_weight = kw->data_ptr<float>(); }
    if (freq.has_value()) { check_f32(*freq, "inv_freq", 64); e.inv_freq = freq->data_ptr<float>(); }
    AKV_CHECK(k_cache.has_value() == v_cache.has_value(), "k_cache and v_cache come together");
    if (k_cache.has_value()) {
      AKV_CHECK(slots.has_value(), "a cache to write needs slots");
      const CacheGeometry g = check_cache(*k_cache, *v_cache, e.num_kv_heads, 128, q_out);
      e.k_cache = k_cache->data_ptr();
      e.v_cache = v_cache->data_ptr();
      e.num_pages = g.num_pages;
      e.page_size = g.page_size;
    }
  } else {
    AKV_CHECK(false, "unknown epilogue '", epilogue, "' (residual, gated, plain, qkv)");
  }
  return ph;
}

void stream_phases(Tensor& hidden, const py::list& phases, Tensor& ssq, Tensor& parts, Tensor& sync,
                   const OptTensor& status, const OptTensor& trace) {
  check_cuda(hidden, "hidden");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && hidden.dim() == 2 && hidden.is_contiguous(),
            "hidden must be a contiguous float32 [tokens, hidden] tensor");
  const int64_t tokens = hidden.size(0), width = hidden.size(1);
  AKV_CHECK(tokens >= 1 && tokens <= 16, "stream_phases takes 1 to 16 tokens, got ", tokens);
  const int64_t n = (int64_t)phases.size();
  AKV_CHECK(n >= 1 && n <= akv::kMaxStreamPhases, "stream_phases takes 1 to ", akv::kMaxStreamPhases, " phases, got ", n);
  akv::StreamPhase list[akv::kMaxStreamPhases];
  for (int64_t i = 0; i < n; ++i) list[i] = parse_stream_phase(phases[i].cast<py::dict>(), hidden, tokens);
  int64_t part_floats = 0, sync_ints = 0;
  akv::stream_phases_scratch(list, (int)n, &part_floats, &sync_ints);
  check_f32(ssq, "ssq");
  check_f32(parts, "parts");
  check_i32(sync, "sync");
  AKV_CHECK(ssq.numel() >= (width + 127) / 128 * tokens, "ssq must hold ceil(hidden / 128) * tokens floats");
  AKV_CHECK(parts.numel() >= part_floats, "parts must hold ", part_floats, " floats, has ", parts.numel());
  AKV_CHECK(sync.numel() >= sync_ints, "sync must hold ", sync_ints, " ints, has ", sync.numel());
  AKV_CHECK(ssq.device() == hidden.device() && parts.device() == hidden.device() && sync.device() == hidden.device(),
            "scratch tensors must be on hidden's device");
  unsigned long long* trace_ptr = nullptr;
  if (trace.has_value()) {
    check_cuda(*trace, "trace");
    AKV_CHECK(trace->scalar_type() == at::kLong && trace->is_contiguous() &&
                  trace->numel() >= (int64_t)akv::stream_phases_grid() * akv::kMaxStreamPhases * 16,
              "trace must be int64 [grid, ", akv::kMaxStreamPhases, ", 16]");
    trace_ptr = reinterpret_cast<unsigned long long*>(trace->data_ptr<int64_t>());
  }
  c10::cuda::CUDAGuard guard(hidden.device());
  check_launch(akv::launch_stream_phases(list, (int)n, tokens, hidden.data_ptr<float>(), width, ssq.data_ptr<float>(),
                                         parts.data_ptr<float>(), sync.data_ptr<int>(), status_ptr(status),
                                         stream_of(hidden), trace_ptr),
               "stream_phases");
}

// (floats of partial tiles, ints of counters) a launch over matrices of the given (features, k) shapes needs.
std::pair<int64_t, int64_t> stream_phases_scratch(const std::vector<std::pair<int64_t, int64_t>>& shapes) {
  AKV_CHECK(!shapes.empty() && (int64_t)shapes.size() <= akv::kMaxStreamPhases, "1 to ", akv::kMaxStreamPhases, " shapes");
  akv::StreamPhase list[akv::kMaxStreamPhases] = {};
  for (size_t i = 0; i < shapes.size(); ++i) {
    list[i].features = shapes[i].first;
    list[i].k = shapes[i].second;
  }
  int64_t part_floats = 0, sync_ints = 0;
  akv::stream_phases_scratch(list, (int)shapes.size(), &part_floats, &sync_ints);
  return {part_floats, sync_ints};
}

void qk_norm_rope_write(const Tensor& qkv, const Tensor& positions, const OptTensor& slots,
                        const OptTensor& q_weight, const OptTensor& k_weight, const OptTensor& inv_freq,
                        Tensor& q_out, const OptTensor& k_out, const OptTensor& v_out, const OptTensor& k_cache,
                        const OptTensor& v_cache, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                        int64_t rotary_dim, double eps, const OptTensor& status) {
  check_cuda(qkv, "qkv");
  check_cuda(q_out, "q_out");
  int qkv_parts = 0;
  if (qkv.dim() == 3) {
    AKV_CHECK(qkv.scalar_type() == at::kFloat && qkv.size(0) >= 1, "a 3-D qkv holds float32 partial sums");
    AKV_CHECK(qkv.device() == q_out.device(), "qkv and q_out must be on the same device");
    qkv_parts = (int)qkv.size(0);
  } else {
    check_same(qkv, q_out, "qkv", "q_out");
  }
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && head_dim > 0, "head counts and head_dim must be positive");
  AKV_CHECK(head_dim % 2 == 0 && head_dim <= 512, "qk_norm_rope_write: head_dim must be even and <= 512, got ",
              head_dim);
  const int64_t width = (num_heads + 2 * num_kv_heads) * head_dim;
  AKV_CHECK((qkv.dim() == 2 || qkv.dim() == 3) && qkv.size(-1) == width,
            "qkv must be [tokens, (heads + 2 kv_heads) * head_dim = ", width, "]");
  const int64_t n = qkv.size(-2);
  check_i32(positions, "positions", n);
  AKV_CHECK(q_out.numel() == n * num_heads * head_dim, "q_out must be [tokens, heads * head_dim]");
  akv::QkRopeWriteParams p{};
  p.qkv = qkv.data_ptr();
  p.qkv_parts = qkv_parts;
  p.positions = positions.data_ptr<int>();
  p.q_out = q_out.data_ptr();
  if (slots.has_value()) {
    check_i32(*slots, "slots", n);
    p.slots = slots->data_ptr<int>();
  }
  if (q_weight.has_value()) { check_f32(*q_weight, "q_weight", head_dim); p.q_weight = q_weight->data_ptr<float>(); }
  if (k_weight.has_value()) { check_f32(*k_weight, "k_weight", head_dim); p.k_weight = k_weight->data_ptr<float>(); }
  if (inv_freq.has_value()) {
    AKV_CHECK(rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim,
                "rotary_dim must be even and in (0, head_dim], got ", rotary_dim);
    check_f32(*inv_freq, "inv_freq", rotary_dim / 2);
    p.inv_freq = inv_freq->data_ptr<float>();
  }
  if (k_out.has_value()) {
    check_cuda(*k_out, "k_out"); check_same(*k_out, q_out, "k_out", "q_out");
    AKV_CHECK(k_out->numel() == n * num_kv_heads * head_dim, "k_out must be [tokens, kv_heads * head_dim]");
    p.k_out = k_out->data_ptr();
  }
  if (v_out.has_value()) {
    check_cuda(*v_out, "v_out"); check_same(*v_out, q_out, "v_out", "q_out");
    AKV_CHECK(v_out->numel() == n * num_kv_heads * head_dim, "v_out must be [tokens, kv_heads * head_dim]");
    p.v_out = v_out->data_ptr();
  }
  AKV_CHECK(k_cache.has_value() == v_cache.has_value(), "k_cache and v_cache come together");
  if (k_cache.has_value()) {
    AKV_CHECK(slots.has_value(), "a cache to write needs slots");
    const CacheGeometry g = check_cache(*k_cache, *v_cache, (int)num_kv_heads, (int)head_dim, q_out);
    p.k_cache = k_cache->data_ptr();
    p.v_cache = v_cache->data_ptr();
    p.num_pages = g.num_pages;
    p.page_size = g.page_size;
  }
  p.num_tokens = n;
  p.num_heads = (int)num_heads;
  p.num_kv_heads = (int)num_kv_heads;
  p.head_dim = (int)head_dim;
  p.rotary_dim = (int)rotary_dim;
  p.eps = (float)eps;
  p.dtype = dtype_code(q_out, "q_out");
  p.status = status_ptr(status);
  c10::cuda::CUDAGuard guard(qkv.device());
  check_launch(akv::launch_qk_norm_rope_write(p, stream_of(qkv)), "qk_norm_rope_write");
}

void kv_write(const Tensor& k, const Tensor& v, const Tensor& slots, Tensor& k_cache, Tensor& v_cache,
              const OptTensor& status) {
  check_cuda(k, "k");
  check_cuda(v, "v");
  check_same(k, v, "k", "v");
  AKV_CHECK(k.dim() == 2 && k.sizes() == v.sizes(), "k and v must both be [tokens, kv_heads * head_dim]");
  AKV_CHECK(k_cache.dim() == 4, "k_cache must be [pages, kv_heads, page_size, head_dim]");
  const int nkv = (int)k_cache.size(1), d = (int)k_cache.size(3);
  const CacheGeometry g = check_cache(k_cache, v_cache, nkv, d, k);
  AKV_CHECK(k.size(1) == (int64_t)nkv * d, "k is ", k.size(1), " wide, the cache wants ", (int64_t)nkv * d);
  check_i32(slots, "slots", k.size(0));
  c10::cuda::CUDAGuard guard(k.device());
  check_launch(akv::launch_kv_write(k.data_ptr(), v.data_ptr(), slots.data_ptr<int>(), k_cache.data_ptr(),
                                    v_cache.data_ptr(), k.size(0), nkv, d, g.page_size, g.num_pages,
                                    dtype_code(k, "k"), status_ptr(status), stream_of(k)),
               "kv_write");
}

void paged_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, Tensor& out,
                     const Tensor& block_table, const Tensor& cu_q, const Tensor& ctx_lens, const Tensor& tile_seq,
                     const Tensor& tile_q0, const Tensor& tile_nq, const OptTensor& partials, int64_t num_tiles,
                     int64_t q_tile, int64_t num_splits, int64_t num_heads, int64_t num_kv_heads, int64_t window,
                     double scale, const OptTensor& status, int64_t kernel) {
  check_cuda(q, "q");
  check_cuda(out, "out");
  check_same(q, out, "q", "out");
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0,
              "paged_attention: heads (", num_heads, ") must be a positive multiple of kv heads (", num_kv_heads, ")");
  AKV_CHECK(q.dim() == 2 && q.size(1) % num_heads == 0, "q must be [tokens, heads * head_dim]");
  const int64_t n = q.size(0), d = q.size(1) / num_heads;
  AKV_CHECK(d % 16 == 0 && d <= 256, "paged_attention: head_dim must be a multiple of 16 up to 256, got ", d);
  AKV_CHECK(out.numel() == q.numel(), "out must have q's shape");
  const CacheGeometry g = check_cache(k_cache, v_cache, (int)num_kv_heads, (int)d, q);
  check_i32(block_table, "block_table");
  AKV_CHECK(block_table.dim() == 2, "block_table must be [sequences, width]");
  const int64_t s = block_table.size(0);
  check_i32(cu_q, "cu_q", s + 1);
  check_i32(ctx_lens, "ctx_lens", s);
  AKV_CHECK(num_tiles >= 0 && q_tile >= 1 && num_splits >= 1 && window >= 0, "bad tile / split / window counts");
  check_i32(tile_seq, "tile_seq", num_tiles);
  check_i32(tile_q0, "tile_q0", num_tiles);
  check_i32(tile_nq, "tile_nq", num_tiles);
  akv::PagedAttentionParams p{};
  if (num_splits > 1) {
    AKV_CHECK(partials.has_value(), "num_splits > 1 needs a partials workspace");
    check_cuda(*partials, "partials");
    AKV_CHECK(partials->scalar_type() == at::kFloat && partials->numel() >= n * num_heads * num_splits * (d + 2),
                "partials must be float32 with at least tokens * heads * splits * (head_dim + 2) entries");
    p.partials = partials->data_ptr<float>();
  }
  p.q = q.data_ptr();
  p.k_cache = k_cache.data_ptr();
  p.v_cache = v_cache.data_ptr();
  p.out = out.data_ptr();
  p.block_table = block_table.data_ptr<int>();
  p.cu_q = cu_q.data_ptr<int>();
  p.ctx_lens = ctx_lens.data_ptr<int>();
  p.tile_seq = tile_seq.data_ptr<int>();
  p.tile_q0 = tile_q0.data_ptr<int>();
  p.tile_nq = tile_nq.data_ptr<int>();
  p.num_tokens = n;
  p.num_tiles = (int)num_tiles;
  p.q_tile = (int)q_tile;
  p.num_splits = (int)num_splits;
  p.num_seqs = (int)s;
  p.table_width = (int)block_table.size(1);
  p.num_heads = (int)num_heads;
  p.num_kv_heads = (int)num_kv_heads;
  p.head_dim = (int)d;
  p.page_size = g.page_size;
  p.num_pages = g.num_pages;
  p.window = (int)window;
  p.kernel = (int)kernel;
  p.scale = (float)scale;
  p.dtype = dtype_code(q, "q");
  p.status = status_ptr(status);
  c10::cuda::CUDAGuard guard(q.device());
  check_launch(akv::launch_paged_attention(p, stream_of(q)), "paged_attention");
}

int64_t sample_slices() { return akv::kSampleSlices; }

// parts: float32 workspace of 4 * rows * slices entries (maxima, indices and, as doubles, sums); tickets: int32, at
// least `rows` entries, all zero (the kernel leaves them zero).
void sample(const Tensor& logits, const Tensor& temperature, const Tensor& uniform, Tensor& tokens, Tensor& parts,
            Tensor& tickets) {
  check_cuda(logits, "logits");
  AKV_CHECK(logits.scalar_type() == at::kFloat && logits.dim() == 2, "logits must be float32 [rows, vocab]");
  const int64_t rows = logits.size(0), cells = rows * akv::kSampleSlices;
  check_f32(temperature, "temperature", rows);
  check_f32(uniform, "uniform", rows);
  check_i32(tokens, "tokens", rows);
  check_f32(parts, "parts");
  check_i32(tickets, "tickets");
  AKV_CHECK(parts.numel() >= 4 * cells && reinterpret_cast<uintptr_t>(parts.data_ptr()) % 8 == 0,
            "parts must hold 4 * rows * slices float32 entries, 8-byte aligned");
  AKV_CHECK(tickets.numel() >= rows, "tickets must hold a counter per row");
  AKV_CHECK(parts.device() == logits.device() && tickets.device() == logits.device(),
            "the workspaces must be on the logits' device");
  float* base = parts.data_ptr<float>();
  c10::cuda::CUDAGuard guard(logits.device());
  check_launch(akv::launch_sample(logits.data_ptr<float>(), temperature.data_ptr<float>(), uniform.data_ptr<float>(),
                                  tokens.data_ptr<int>(), rows, logits.size(1), base + 2 * cells,
                                  reinterpret_cast<int*>(base + 3 * cells), reinterpret_cast<double*>(base),
                                  tickets.data_ptr<int>(), stream_of(logits)),
               "sample");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "sm_100a kernels of the engine";
  namespace py = pybind11;
  m.def("smoke_add", &smoke_add, "a + b on the device (toolchain check)");
  m.def("wait_selftest", &wait_selftest, py::arg("limit"), py::arg("status"),
        "a bounded wait on a barrier that nothing completes: leaves the wait-timeout code in status");
  m.def("embedding", &embedding, py::arg("ids"), py::arg("table"), py::arg("hidden"), py::arg("status") = py::none(),
        py::arg("sampled") = py::none());
  m.def("add_rmsnorm", &add_rmsnorm, py::arg("hidden"), py::arg("delta"), py::arg("weight"), py::arg("out"),
        py::arg("rows"), py::arg("eps"), py::arg("status") = py::none());
  m.def("silu_mul", &silu_mul, py::arg("gate_up"), py::arg("out"), py::arg("block") = 0);
  m.def("small_m_gemm", &small_m_gemm, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("splits") = 1,
        py::arg("status") = py::none(), py::arg("gated") = false, py::arg("nx_hidden") = py::none(),
        py::arg("nx_ssq") = py::none(), py::arg("nx_weight") = py::none(), py::arg("nx_eps") = 0.0);
  m.def("small_m_gemm_residual", &small_m_gemm_residual, py::arg("x"), py::arg("w"), py::arg("hidden"),
        py::arg("ssq"), py::arg("splits") = 1, py::arg("status") = py::none());
  m.def("small_m_gemm_qkv", &small_m_gemm_qkv, py::arg("x"), py::arg("w"), py::arg("q_out"), py::arg("positions"),
        py::arg("slots"), py::arg("q_weight"), py::arg("k_weight"), py::arg("inv_freq"), py::arg("k_cache"),
        py::arg("v_cache"), py::arg("num_heads"), py::arg("num_kv_heads"), py::arg("eps"), py::arg("splits") = 1,
        py::arg("status") = py::none(), py::arg("nx_hidden") = py::none(), py::arg("nx_ssq") = py::none(),
        py::arg("nx_weight") = py::none(), py::arg("nx_eps") = 0.0);
  m.def("stream_phases", &stream_phases, py::arg("hidden"), py::arg("phases"), py::arg("ssq"), py::arg("parts"),
        py::arg("sync"), py::arg("status") = py::none(), py::arg("trace") = py::none(),
        "a chain of dependent products for up to 16 tokens in one persistent kernel");
  m.def("stream_phases_scratch", &stream_phases_scratch, py::arg("shapes"));
  m.def("stream_phases_max", []() { return (int64_t)akv::kMaxStreamPhases; });
  m.def("stream_phases_grid", []() { return (int64_t)akv::stream_phases_grid(); });
  m.def("small_m_gemm_supported", &small_m_gemm_supported);
  m.def("small_m_gemm_splits", &small_m_gemm_splits);
  m.def("qk_norm_rope_write", &qk_norm_rope_write, py::arg("qkv"), py::arg("positions"), py::arg("slots"),
        py::arg("q_weight"), py::arg("k_weight"), py::arg("inv_freq"), py::arg("q_out"), py::arg("k_out"),
        py::arg("v_out"), py::arg("k_cache"), py::arg("v_cache"), py::arg("num_heads"), py::arg("num_kv_heads"),
        py::arg("head_dim"), py::arg("rotary_dim"), py::arg("eps"), py::arg("status") = py::none());
  m.def("kv_write", &kv_write, py::arg("k"), py::arg("v"), py::arg("slots"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("status") = py::none());
  m.def("paged_attention", &paged_attention, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"),
        py::arg("block_table"), py::arg("cu_q"), py::arg("ctx_lens"), py::arg("tile_seq"), py::arg("tile_q0"),
        py::arg("tile_nq"), py::arg("partials"), py::arg("num_tiles"), py::arg("q_tile"), py::arg("num_splits"),
        py::arg("num_heads"), py::arg("num_kv_heads"), py::arg("window"), py::arg("scale"),
        py::arg("status") = py::none(), py::arg("kernel") = 0);
  m.def("sample", &sample, py::arg("logits"), py::arg("temperature"), py::arg("uniform"), py::arg("tokens"),
        py::arg("parts"), py::arg("tickets"));
  m.def("sample_slices", &sample_slices);
  m.def("sm_count", &akv::sm_count, "streaming multiprocessors of the current device");
}
