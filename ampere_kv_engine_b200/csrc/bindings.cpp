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
               const OptTensor& sampled, double scale, const OptTensor& positions, const OptTensor& position_rows) {
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
  const int* positions_ptr = nullptr;
  const void* rows_ptr = nullptr;
  int64_t max_positions = 0;
  if (position_rows.has_value()) {
    AKV_CHECK(positions.has_value(), "position_rows needs positions");
    check_cuda(*position_rows, "position_rows");
    check_same(*position_rows, table, "position_rows", "table");
    AKV_CHECK(position_rows->dim() == 2 && position_rows->size(1) == h, "position_rows must be [positions, hidden]");
    check_i32(*positions, "positions", n);
    positions_ptr = positions->data_ptr<int>();
    rows_ptr = position_rows->data_ptr();
    max_positions = position_rows->size(0);
  }
  c10::cuda::CUDAGuard guard(table.device());
  check_launch(akv::launch_embedding(ids.data_ptr<int>(), sampled_ptr, num_sampled, table.data_ptr(),
                                     hidden.data_ptr<float>(), n, h,
                                     table.size(0), dtype_code(table, "table"), status_ptr(status),
                                     stream_of(table), (float)scale, positions_ptr, rows_ptr, max_positions),
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
                  double nx_eps, int64_t activation) {
  const TokenOperand t = token_operand(x, nx_hidden, nx_ssq, nx_weight, nx_eps, w);
  check_cuda(out, "out");
  AKV_CHECK(out.device() == w.device(), "out and w must be on the same device");
  AKV_CHECK(activation >= -1 && activation <= 2 &&
                (activation < 0 || (!gated && out.dim() == 2 && out.scalar_type() == at::kBFloat16)),
            "an activation (0 relu squared, 1 tanh GELU, 2 SiLU) goes with the plain product and a bfloat16 out");
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
  f.activation = (int)activation;
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

// A paged storage of rows: [pages, heads, page_size, width], contiguous.
void check_pages(const Tensor& cache, const char* name, int64_t heads, int64_t min_width, const Tensor& like) {
  check_cuda(cache, name);
  check_same(cache, like, name, "activations");
  AKV_CHECK(cache.dim() == 4 && cache.size(1) == heads && cache.size(3) >= min_width, name,
            " must be [pages, ", heads, " heads, page_size, at least ", min_width, " elements]");
}

// Attention with reshaped scores and keys / values of different widths (see launchers.h).  k_cache
// [pages, kv heads, page_size, >= key width]; v_cache likewise for the value width, or the same tensor when a value
// is the first v_dim elements of its key row.
void scored_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, Tensor& out,
                      const Tensor& block_table, const Tensor& cu_q, const Tensor& ctx_lens, const Tensor& tile_seq,
                      const Tensor& tile_q0, const Tensor& tile_nq, const OptTensor& partials, int64_t num_tiles,
                      int64_t q_tile, int64_t num_splits, int64_t num_heads, int64_t num_kv_heads, int64_t v_dim,
                      int64_t window, int64_t chunk, double scale, double softcap, const OptTensor& slopes,
                      const OptTensor& gate, const OptTensor& status, int64_t kernel, int64_t keep_first,
                      bool sigmoid_weights, const OptTensor& head_bias, double out_scale) {
  check_cuda(q, "q");
  check_cuda(out, "out");
  check_same(q, out, "q", "out");
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0,
            "scored_attention: heads (", num_heads, ") must be a positive multiple of kv heads (", num_kv_heads, ")");
  AKV_CHECK(q.dim() == 2 && q.size(1) % num_heads == 0, "q must be [tokens, heads * key width]");
  const int64_t n = q.size(0), d = q.size(1) / num_heads;
  AKV_CHECK(d >= 1 && d <= 1024, "scored_attention: the key width must be between 1 and 1024, got ", d);
  AKV_CHECK(v_dim >= 1 && v_dim <= 512, "scored_attention: the value width must be between 1 and 512, got ", v_dim);
  AKV_CHECK(out.dim() == 2 && out.size(0) == n && out.size(1) == num_heads * v_dim,
            "out must be [tokens, heads * value width]");
  check_pages(k_cache, "k_cache", num_kv_heads, d, q);
  check_pages(v_cache, "v_cache", num_kv_heads, v_dim, q);
  AKV_CHECK(k_cache.size(0) == v_cache.size(0) && k_cache.size(2) == v_cache.size(2),
            "k_cache and v_cache must have the same pages and page size");
  check_i32(block_table, "block_table");
  AKV_CHECK(block_table.dim() == 2, "block_table must be [sequences, width]");
  const int64_t s = block_table.size(0);
  check_i32(cu_q, "cu_q", s + 1);
  check_i32(ctx_lens, "ctx_lens", s);
  AKV_CHECK(num_tiles >= 0 && q_tile >= 1 && num_splits >= 1 && window >= 0 && chunk >= 0 && softcap >= 0,
            "bad tile / split / window / chunk / softcap");
  check_i32(tile_seq, "tile_seq", num_tiles);
  check_i32(tile_q0, "tile_q0", num_tiles);
  check_i32(tile_nq, "tile_nq", num_tiles);
  akv::ScoredAttentionParams sp{};
  akv::PagedAttentionParams& p = sp.base;
  if (num_splits > 1) {
    AKV_CHECK(partials.has_value(), "num_splits > 1 needs a partials workspace");
    check_cuda(*partials, "partials");
    AKV_CHECK(partials->scalar_type() == at::kFloat && partials->numel() >= n * num_heads * num_splits * (v_dim + 2),
              "partials must be float32 with at least tokens * heads * splits * (value width + 2) entries");
    p.partials = partials->data_ptr<float>();
  }
  if (slopes.has_value()) {
    check_f32(*slopes, "slopes", num_heads);
    sp.slopes = slopes->data_ptr<float>();
  }
  if (gate.has_value()) {
    check_f32(*gate, "gate", n * num_heads);
    sp.gate = gate->data_ptr<float>();
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
  p.page_size = (int)k_cache.size(2);
  p.num_pages = k_cache.size(0);
  p.window = (int)window;
  p.kernel = (int)kernel;          // 0: the best kernel that takes the sizes; 1: the general kernel
  p.scale = (float)scale;
  p.dtype = dtype_code(q, "q");
  p.status = status_ptr(status);
  sp.v_dim = (int)v_dim;
  sp.k_row_stride = k_cache.size(3);
  sp.v_row_stride = v_cache.size(3);
  sp.softcap = (float)softcap;
  sp.chunk = (int)chunk;
  AKV_CHECK(keep_first >= 0 && (keep_first == 0 || (window > 0 && chunk == 0)),
            "scored_attention: keep_first goes with a window and without blocks");
  sp.keep_first = (int)keep_first;
  sp.sigmoid_weights = sigmoid_weights ? 1 : 0;
  if (head_bias.has_value()) {
    AKV_CHECK(sigmoid_weights, "scored_attention: head_bias is read with sigmoid_weights only");
    check_f32(*head_bias, "head_bias", num_heads);
    sp.head_bias = head_bias->data_ptr<float>();
  }
  sp.out_scale = (float)out_scale;
  c10::cuda::CUDAGuard guard(q.device());
  check_launch(akv::launch_scored_attention(sp, stream_of(q)), "scored_attention");
}

void head_prep(const Tensor& x, const OptTensor& slots, Tensor& q_out, const OptTensor& k_cache,
               const OptTensor& v_cache, const OptTensor& v_keep, const OptTensor& v_other,
               const OptTensor& blend_weight, const OptTensor& gate_out, int64_t num_heads, int64_t num_kv_heads,
               int64_t head_dim, int64_t v_dim, bool unit_norm, double eps, const OptTensor& status,
               const OptTensor& q_weight, const OptTensor& k_weight, bool has_kv) {
  check_cuda(x, "x");
  check_cuda(q_out, "q_out");
  check_same(x, q_out, "x", "q_out");
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && head_dim > 0 && v_dim > 0, "head_prep: sizes must be positive");
  AKV_CHECK(has_kv || !(k_cache.has_value() || v_keep.has_value() || v_other.has_value() || k_weight.has_value()),
            "head_prep: without k and v columns there is nothing to cache, keep, blend or weigh");
  const int64_t width = num_heads * head_dim + (has_kv ? num_kv_heads * (head_dim + v_dim) : 0) +
                        (gate_out.has_value() ? num_heads : 0);
  AKV_CHECK(x.dim() == 2 && x.size(1) == width, "x must be [tokens, ", width, "], the q, k, v (and gate) columns");
  const int64_t n = x.size(0);
  AKV_CHECK(q_out.numel() == n * num_heads * head_dim, "q_out must be [tokens, heads * head_dim]");
  akv::HeadPrepParams p{};
  p.x = x.data_ptr();
  p.q_out = q_out.data_ptr();
  if (slots.has_value()) {
    check_i32(*slots, "slots", n);
    p.slots = slots->data_ptr<int>();
  }
  if (k_cache.has_value()) {
    AKV_CHECK(v_cache.has_value() && slots.has_value(), "k_cache needs v_cache and slots");
    check_pages(*k_cache, "k_cache", num_kv_heads, head_dim, x);
    check_pages(*v_cache, "v_cache", num_kv_heads, v_dim, x);
    AKV_CHECK(k_cache->size(0) == v_cache->size(0) && k_cache->size(2) == v_cache->size(2),
              "k_cache and v_cache must have the same pages and page size");
    p.k_cache = k_cache->data_ptr();
    p.v_cache = v_cache->data_ptr();
    p.page_size = (int)k_cache->size(2);
    p.num_pages = k_cache->size(0);
    p.k_row_stride = k_cache->size(3);
    p.v_row_stride = v_cache->size(3);
  }
  auto dense_v = [&](const OptTensor& t, const char* name) -> void* {
    if (!t.has_value()) return nullptr;
    check_cuda(*t, name);
    check_same(*t, x, name, "x");
    AKV_CHECK(t->numel() == n * num_kv_heads * v_dim, name, " must be [tokens, kv heads * value width]");
    return t->data_ptr();
  };
  p.v_keep = dense_v(v_keep, "v_keep");
  p.v_other = dense_v(v_other, "v_other");
  if (v_other.has_value()) {
    AKV_CHECK(blend_weight.has_value(), "v_other needs blend_weight");
    check_f32(*blend_weight, "blend_weight", 1);
    p.blend_weight = blend_weight->data_ptr<float>();
  }
  if (gate_out.has_value()) {
    check_f32(*gate_out, "gate_out", n * num_heads);
    p.gate_out = gate_out->data_ptr<float>();
  }
  p.num_tokens = n;
  p.num_heads = (int)num_heads;
  p.num_kv_heads = (int)num_kv_heads;
  p.head_dim = (int)head_dim;
  p.v_dim = (int)v_dim;
  p.unit_norm = unit_norm ? 1 : 0;
  p.eps = (float)eps;
  p.dtype = dtype_code(x, "x");
  p.status = status_ptr(status);
  if (q_weight.has_value()) {
    check_f32(*q_weight, "q_weight", head_dim);
    p.q_weight = q_weight->data_ptr<float>();
  }
  if (k_weight.has_value()) {
    check_f32(*k_weight, "k_weight", head_dim);
    p.k_weight = k_weight->data_ptr<float>();
  }
  p.no_kv = has_kv ? 0 : 1;
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_head_prep(p, stream_of(x)), "head_prep");
}

void latent_prep(const Tensor& x, const Tensor& positions, const OptTensor& slots, const Tensor& q_weight,
                 const Tensor& kv_weight, const Tensor& inv_freq, Tensor& q_latent, const OptTensor& cache,
                 int64_t q_rank, int64_t kv_rank, int64_t rot_dim, int64_t rotary_dims, double eps,
                 const OptTensor& status) {
  check_cuda(x, "x");
  check_cuda(q_latent, "q_latent");
  check_same(x, q_latent, "x", "q_latent");
  AKV_CHECK(q_rank > 0 && kv_rank > 0 && rot_dim >= 0 && rotary_dims >= 0 && rotary_dims <= rot_dim &&
                rotary_dims % 2 == 0,
            "latent_prep: ranks must be positive and rotary_dims an even number up to rot_dim");
  AKV_CHECK(x.dim() == 2 && x.size(1) == q_rank + kv_rank + rot_dim,
            "x must be [tokens, q_rank + kv_rank + rot_dim]");
  const int64_t n = x.size(0);
  check_i32(positions, "positions", n);
  check_f32(q_weight, "q_weight", q_rank);
  check_f32(kv_weight, "kv_weight", kv_rank);
  check_f32(inv_freq, "inv_freq", rotary_dims / 2);
  AKV_CHECK(q_latent.numel() == n * q_rank, "q_latent must be [tokens, q_rank]");
  akv::LatentPrepParams p{};
  p.x = x.data_ptr();
  p.positions = positions.data_ptr<int>();
  if (slots.has_value()) {
    check_i32(*slots, "slots", n);
    p.slots = slots->data_ptr<int>();
  }
  p.q_weight = q_weight.data_ptr<float>();
  p.kv_weight = kv_weight.data_ptr<float>();
  p.inv_freq = inv_freq.data_ptr<float>();
  p.q_latent = q_latent.data_ptr();
  if (cache.has_value()) {
    AKV_CHECK(slots.has_value(), "cache needs slots");
    check_pages(*cache, "cache", 1, kv_rank + rot_dim, x);
    p.cache = cache->data_ptr();
    p.page_size = (int)cache->size(2);
    p.num_pages = cache->size(0);
    p.row_stride = cache->size(3);
  }
  p.num_tokens = n;
  p.q_rank = (int)q_rank;
  p.kv_rank = (int)kv_rank;
  p.rot_dim = (int)rot_dim;
  p.rotary_dims = (int)rotary_dims;
  p.eps = (float)eps;
  p.dtype = dtype_code(x, "x");
  p.status = status_ptr(status);
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_latent_prep(p, stream_of(x)), "latent_prep");
}

void rotate_pairs(const Tensor& in, Tensor& out, const Tensor& positions, const Tensor& inv_freq, int64_t heads,
                  int64_t cols, int64_t rotary_dims, int64_t in_offset, int64_t out_offset) {
  check_cuda(in, "in");
  check_cuda(out, "out");
  check_same(in, out, "in", "out");
  AKV_CHECK(in.dim() == 2 && out.dim() == 2 && in.size(0) == out.size(0) && heads > 0 && in.size(1) % heads == 0 &&
                out.size(1) % heads == 0,
            "in and out must be [tokens, heads * width]");
  const int64_t n = in.size(0), in_width = in.size(1) / heads, out_width = out.size(1) / heads;
  AKV_CHECK(cols >= 0 && in_offset >= 0 && out_offset >= 0 && in_offset + cols <= in_width &&
                out_offset + cols <= out_width && rotary_dims >= 0 && rotary_dims <= cols && rotary_dims % 2 == 0,
            "rotate_pairs: the column range must lie inside both tensors and rotary_dims be even and inside it");
  check_i32(positions, "positions", n);
  check_f32(inv_freq, "inv_freq", rotary_dims / 2);
  c10::cuda::CUDAGuard guard(in.device());
  check_launch(akv::launch_rotate_pairs(in.data_ptr(), out.data_ptr(), positions.data_ptr<int>(),
                                        inv_freq.data_ptr<float>(), n, (int)heads, (int)cols, (int)rotary_dims,
                                        in_width, (int)in_offset, out_width, (int)out_offset, dtype_code(in, "in"),
                                        stream_of(in)),
               "rotate_pairs");
}

void activation(const Tensor& in, Tensor& out, int64_t kind) {
  check_cuda(in, "in");
  check_cuda(out, "out");
  check_same(in, out, "in", "out");
  AKV_CHECK(in.numel() == out.numel(), "in and out must have the same number of elements");
  AKV_CHECK(kind >= 0 && kind <= 2, "activation: kind must be 0 (relu squared), 1 (tanh GELU) or 2 (SiLU)");
  c10::cuda::CUDAGuard guard(in.device());
  check_launch(akv::launch_activation(in.data_ptr(), out.data_ptr(), in.numel(), (int)kind, dtype_code(in, "in"),
                                      stream_of(in)),
               "activation");
}

void add_layernorm(Tensor& hidden, const OptTensor& delta, const Tensor& weight, Tensor& out, const OptTensor& rows,
                   double eps, const OptTensor& status) {
  check_cuda(hidden, "hidden");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && hidden.dim() == 2, "hidden must be float32 [tokens, hidden]");
  const int64_t n = hidden.size(0), h = hidden.size(1);
  check_f32(weight, "weight", h);
  check_cuda(out, "out");
  const int code = dtype_code(out, "out");
  AKV_CHECK(h * 4 <= 200 * 1024, "add_layernorm: hidden size ", h, " exceeds the kernel's limit of 51200");
  const void* delta_ptr = nullptr;
  if (delta.has_value()) {
    check_cuda(*delta, "delta");
    check_same(*delta, out, "delta", "out");
    AKV_CHECK(delta->numel() == n * h, "delta must be [tokens, hidden]");
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
  check_launch(akv::launch_add_layernorm(hidden.data_ptr<float>(), delta_ptr, weight.data_ptr<float>(), out.data_ptr(),
                                         rows_ptr, num_rows, n, h, (float)eps, code, status_ptr(status),
                                         stream_of(hidden)),
               "add_layernorm");
}

void branch_layernorm(Tensor& hidden, const Tensor& branch, const Tensor& weight, const OptTensor& copy, double eps) {
  check_cuda(hidden, "hidden");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && hidden.dim() == 2, "hidden must be float32 [tokens, hidden]");
  const int64_t n = hidden.size(0), h = hidden.size(1);
  check_f32(weight, "weight", h);
  check_cuda(branch, "branch");
  AKV_CHECK(branch.numel() == n * h && branch.device() == hidden.device(), "branch must be [tokens, hidden]");
  AKV_CHECK(h * 4 <= 200 * 1024, "branch_layernorm: hidden size ", h, " exceeds the kernel's limit of 51200");
  void* copy_ptr = nullptr;
  int copy_code = 0;
  if (copy.has_value()) {
    check_cuda(*copy, "copy");
    AKV_CHECK(copy->scalar_type() == at::kBFloat16 && copy->numel() == n * h && copy->device() == hidden.device(),
              "copy must be bfloat16 [tokens, hidden]");
    copy_ptr = copy->data_ptr();
    copy_code = 1;
  }
  c10::cuda::CUDAGuard guard(hidden.device());
  check_launch(akv::launch_branch_layernorm(hidden.data_ptr<float>(), branch.data_ptr(), dtype_code(branch, "branch"),
                                            weight.data_ptr<float>(), copy_ptr, copy_code, n, h, (float)eps,
                                            stream_of(hidden)),
               "branch_layernorm");
}

void branch_layernorm_parts(Tensor& hidden, const Tensor& parts, const OptTensor& shared, const Tensor& weight,
                            const OptTensor& copy, double eps, int64_t top) {
  check_cuda(hidden, "hidden");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && hidden.dim() == 2, "hidden must be float32 [tokens, hidden]");
  const int64_t n = hidden.size(0), h = hidden.size(1);
  check_f32(weight, "weight", h);
  AKV_CHECK(top >= 1, "top must be positive");
  check_f32(parts, "parts", n * top * h);
  AKV_CHECK(parts.device() == hidden.device(), "parts must be on the stream's device");
  AKV_CHECK(h * 4 <= 200 * 1024, "branch_layernorm_parts: hidden size ", h, " exceeds the kernel's limit of 51200");
  const void* shared_ptr = nullptr;
  int shared_code = 0;
  if (shared.has_value()) {
    check_cuda(*shared, "shared");
    AKV_CHECK(shared->numel() == n * h && shared->device() == hidden.device(), "shared must be [tokens, hidden]");
    shared_ptr = shared->data_ptr();
    shared_code = dtype_code(*shared, "shared");
  }
  void* copy_ptr = nullptr;
  int copy_code = 0;
  if (copy.has_value()) {
    check_cuda(*copy, "copy");
    AKV_CHECK(copy->scalar_type() == at::kBFloat16 && copy->numel() == n * h && copy->device() == hidden.device(),
              "copy must be bfloat16 [tokens, hidden]");
    copy_ptr = copy->data_ptr();
    copy_code = 1;
  }
  c10::cuda::CUDAGuard guard(hidden.device());
  check_launch(akv::launch_branch_layernorm_parts(hidden.data_ptr<float>(), parts.data_ptr<float>(), (int)top, shared_ptr,
                                                  shared_code, weight.data_ptr<float>(), copy_ptr, copy_code, n, h,
                                                  (float)eps, stream_of(hidden)),
               "branch_layernorm_parts");
}

void stream_copy(const Tensor& hidden, Tensor& out) {
  check_cuda(hidden, "hidden");
  check_cuda(out, "out");
  AKV_CHECK(hidden.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16 && out.numel() == hidden.numel() &&
                out.device() == hidden.device(),
            "stream_copy: float32 in, bfloat16 out of the same size");
  c10::cuda::CUDAGuard guard(hidden.device());
  check_launch(akv::launch_stream_copy(hidden.data_ptr<float>(), out.data_ptr(), hidden.numel(), stream_of(hidden)),
               "stream_copy");
}

void glu(const Tensor& gate_up, Tensor& out, int64_t kind, int64_t block, double limit, double slope) {
  check_cuda(gate_up, "gate_up");
  check_cuda(out, "out");
  check_same(gate_up, out, "gate_up", "out");
  AKV_CHECK(gate_up.dim() == 2 && gate_up.size(1) % 2 == 0, "gate_up must be [tokens, 2 * intermediate]");
  const int64_t n = gate_up.size(0), inter = gate_up.size(1) / 2;
  AKV_CHECK(out.numel() == n * inter, "out must be [tokens, intermediate]");
  AKV_CHECK(kind >= 0 && kind <= 2, "glu: kind must be 0 (SiLU), 1 (tanh GELU) or 2 (clamped swish)");
  AKV_CHECK(kind != 2 || limit > 0, "glu: the clamped form needs a positive limit");
  if (block == 0) block = inter;
  AKV_CHECK(block > 0 && inter % block == 0, "glu: block must divide the intermediate size");
  c10::cuda::CUDAGuard guard(gate_up.device());
  check_launch(akv::launch_glu(gate_up.data_ptr(), out.data_ptr(), n, inter, block, (int)kind, (float)limit,
                               (float)slope, dtype_code(gate_up, "gate_up"), stream_of(gate_up)),
               "glu");
}

void softcap(Tensor& logits, double cap) {
  check_cuda(logits, "logits");
  AKV_CHECK(logits.scalar_type() == at::kFloat, "logits must be float32");
  AKV_CHECK(cap > 0, "softcap: cap must be positive");
  c10::cuda::CUDAGuard guard(logits.device());
  check_launch(akv::launch_softcap(logits.data_ptr<float>(), logits.numel(), (float)cap, stream_of(logits)), "softcap");
}

akv::DeltaParams delta_params(const Tensor& x, const Tensor& state, const Tensor& cu_q, const Tensor& state_slots,
                              int64_t num_heads, int64_t num_kv_heads, int64_t head_dim, int64_t v_dim, int64_t taps) {
  check_cuda(x, "x");
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && head_dim > 0 && v_dim > 0,
            "delta rule: sizes must be positive and heads a multiple of the q/k heads");
  AKV_CHECK(head_dim <= akv::kDeltaMaxDim && v_dim <= akv::kDeltaMaxDim && akv::delta_scan_supported((int)head_dim, (int)v_dim),
            "delta rule: a head of ", head_dim, " x ", v_dim, " is outside what the kernels take");
  AKV_CHECK(taps >= 1 && taps <= akv::kDeltaMaxTaps, "delta rule: taps must be between 1 and ", (int64_t)akv::kDeltaMaxTaps);
  const int64_t channels = 2 * num_kv_heads * head_dim + num_heads * v_dim;
  const int64_t width = channels + num_heads * v_dim + 2 * num_heads;
  AKV_CHECK(x.dim() == 2 && x.size(1) == width, "x must be [tokens, ", width, "]: q, k, v, gate, beta, step");
  const int64_t memory = akv::delta_memory_floats((int)num_heads, (int)head_dim, (int)v_dim);
  const int64_t floats = (memory + (taps - 1) * channels + 3) / 4 * 4;
  check_cuda(state, "state");
  AKV_CHECK(state.scalar_type() == at::kFloat && state.dim() == 2 && state.size(1) == floats && state.device() == x.device(),
            "state must be float32 [slots, ", floats, "]");
  check_i32(cu_q, "cu_q", 1);
  const int64_t num_seqs = cu_q.numel() - 1;
  check_i32(state_slots, "state_slots", num_seqs);
  akv::DeltaParams p{};
  p.x = x.data_ptr();
  p.state = state.data_ptr<float>();
  p.cu_q = cu_q.data_ptr<int>();
  p.state_slots = state_slots.data_ptr<int>();
  p.num_tokens = x.size(0);
  p.state_stride = state.size(1);
  p.memory = memory;
  p.num_seqs = (int)num_seqs;
  p.num_slots = (int)state.size(0);
  p.num_heads = (int)num_heads;
  p.num_kv_heads = (int)num_kv_heads;
  p.head_dim = (int)head_dim;
  p.v_dim = (int)v_dim;
  p.taps = (int)taps;
  p.dtype = dtype_code(x, "x");
  return p;
}

void delta_prep(const Tensor& x, const Tensor& conv, const Tensor& rate_log, const Tensor& step_bias, const Tensor& state,
                const Tensor& cu_q, const Tensor& state_slots, Tensor& qkv, Tensor& coef, int64_t num_heads,
                int64_t num_kv_heads, int64_t head_dim, int64_t v_dim, int64_t taps, double unit_eps) {
  akv::DeltaParams p = delta_params(x, state, cu_q, state_slots, num_heads, num_kv_heads, head_dim, v_dim, taps);
  const int64_t channels = 2 * num_kv_heads * head_dim + num_heads * v_dim;
  check_f32(conv, "conv", channels * taps);
  check_f32(rate_log, "rate_log", num_heads);
  check_f32(step_bias, "step_bias", num_heads);
  check_f32(qkv, "qkv", p.num_tokens * channels);
  check_f32(coef, "coef", p.num_tokens * 2 * num_heads);
  p.conv = conv.data_ptr<float>();
  p.rate_log = rate_log.data_ptr<float>();
  p.step_bias = step_bias.data_ptr<float>();
  p.qkv = qkv.data_ptr<float>();
  p.coef = coef.data_ptr<float>();
  p.unit_eps = (float)unit_eps;
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_delta_prep(p, stream_of(x)), "delta_prep");
}

void delta_scan(const Tensor& qkv, const Tensor& coef, const Tensor& x, const Tensor& norm_weight, Tensor& state,
                const Tensor& cu_q, const Tensor& state_slots, Tensor& scratch, Tensor& out, int64_t num_heads,
                int64_t num_kv_heads, int64_t head_dim, int64_t v_dim, int64_t taps, double norm_eps) {
  akv::DeltaParams p = delta_params(x, state, cu_q, state_slots, num_heads, num_kv_heads, head_dim, v_dim, taps);
  const int64_t channels = 2 * num_kv_heads * head_dim + num_heads * v_dim;
  check_f32(qkv, "qkv", p.num_tokens * channels);
  check_f32(coef, "coef", p.num_tokens * 2 * num_heads);
  check_f32(norm_weight, "norm_weight", v_dim);
  check_f32(scratch, "scratch", p.num_tokens * num_heads * v_dim);
  check_cuda(out, "out");
  check_same(out, x, "out", "x");
  AKV_CHECK(out.numel() == p.num_tokens * num_heads * v_dim, "out must be [tokens, heads * v_dim]");
  p.qkv = qkv.data_ptr<float>();
  p.coef = coef.data_ptr<float>();
  p.norm_weight = norm_weight.data_ptr<float>();
  p.scratch = scratch.data_ptr<float>();
  p.out = out.data_ptr();
  p.norm_eps = (float)norm_eps;
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_delta_scan(p, stream_of(x)), "delta_scan");
}

// Linear attention with a decaying matrix memory (see launchers.h).  x: one product's output; state
// [slots, floats per slot] float32 (a view whose rows may be wider than this mixer's share: its stride is passed on).
void linear_scan(const Tensor& x, Tensor& state, const Tensor& cu_q, const Tensor& state_slots, Tensor& out,
                 int64_t num_heads, int64_t head_dim, int64_t v_dim, int64_t mode, int64_t q_off, int64_t k_off,
                 int64_t v_off, const OptTensor& gate_bias, const OptTensor& lower, const OptTensor& decay,
                 int64_t qk_group, int64_t decay_off) {
  check_cuda(x, "x");
  AKV_CHECK(x.dim() == 2, "x must be [tokens, columns]");
  AKV_CHECK(num_heads > 0 && akv::linear_scan_state_floats((int)num_heads, (int)head_dim, (int)v_dim) > 0,
            "linear_scan: ", num_heads, " heads of ", head_dim, " x ", v_dim, " are outside what the kernel takes (each up to ",
            (int64_t)akv::kLinearScanMaxDim, ")");
  AKV_CHECK(qk_group >= 1 && num_heads % qk_group == 0, "linear_scan: qk_group must divide the heads");
  const int64_t n = x.size(0), qk = num_heads / qk_group * head_dim, vw = num_heads * v_dim;
  const bool prepared = mode == akv::kPlainDecay || mode == akv::kTokenDecay;
  AKV_CHECK(!prepared || x.scalar_type() == at::kFloat, "linear_scan: modes 2 and 3 read float32 rows");
  AKV_CHECK(prepared || qk_group == 1, "linear_scan: shared q and k heads come with the prepared modes");
  AKV_CHECK(mode != akv::kTokenDecay || (decay_off >= 0 && decay_off + num_heads <= x.size(1)),
            "linear_scan: the decay columns must lie inside x");
  AKV_CHECK(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + qk <= x.size(1) && k_off + qk <= x.size(1) &&
            v_off + vw <= x.size(1), "linear_scan: the q, k and v columns must lie inside x");
  AKV_CHECK(state.is_cuda() && state.scalar_type() == at::kFloat && state.dim() == 2 && state.stride(1) == 1 &&
            state.size(1) >= akv::linear_scan_state_floats((int)num_heads, (int)head_dim, (int)v_dim),
            "state must be float32 [slots, at least the memory's floats] with unit stride in a row");
  check_i32(cu_q, "cu_q");
  const int64_t seqs = cu_q.numel() - 1;
  check_i32(state_slots, "state_slots", seqs);
  check_f32(out, "out", n * vw);
  akv::LinearScanParams p{};
  p.x = x.data_ptr();
  p.x_stride = x.size(1);
  p.q_off = (int)q_off;
  p.k_off = (int)k_off;
  p.v_off = (int)v_off;
  if (gate_bias.has_value()) {
    check_f32(*gate_bias, "gate_bias", qk);
    p.gate_bias = gate_bias->data_ptr<float>();
  }
  if (lower.has_value()) {
    check_f32(*lower, "lower", qk);
    p.lower = lower->data_ptr<float>();
  }
  if (decay.has_value()) {
    check_f32(*decay, "decay", num_heads);
    p.decay = decay->data_ptr<float>();
  }
  AKV_CHECK(mode == akv::kGatedWrite ? lower.has_value()
                                     : (mode == akv::kTokenDecay ||
                                        ((mode == akv::kConstantDecay || mode == akv::kPlainDecay) && decay.has_value())),
            "linear_scan: mode 0 needs lower, modes 1 and 2 need decay, mode 3 decay columns");
  // a step that holds more than single tokens: activations and gates are worked out once per token by a kernel of
  // their own, into scratch that the scan's staging warps copy from
  Tensor act;
  if (n > 2 * seqs) {
    if (prepared) {
      p.act = (float*)x.data_ptr();        // the rows are float32 and final: the staging warps copy from them
    } else {
      act = at::empty({n, 2 * qk + vw}, x.options().dtype(at::kFloat));
      p.act = act.data_ptr<float>();
    }
  }
  p.qk_group = (int)qk_group;
  p.decay_off = (int)decay_off;
  p.state = state.data_ptr<float>();
  p.state_stride = state.stride(0);
  p.cu_q = cu_q.data_ptr<int>();
  p.state_slots = state_slots.data_ptr<int>();
  p.out = out.data_ptr<float>();
  p.num_tokens = n;
  p.num_seqs = (int)seqs;
  p.num_heads = (int)num_heads;
  p.head_dim = (int)head_dim;
  p.v_dim = (int)v_dim;
  p.mode = (int)mode;
  p.dtype = dtype_code(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_linear_scan(p, stream_of(x)), "linear_scan");
}

void group_norm_gate(const Tensor& in, Tensor& out, const OptTensor& weight, int64_t group, double eps, double factor,
                     const OptTensor& x, int64_t gate_off, int64_t gate_kind, bool gate_first, const OptTensor& skip,
                     int64_t skip_off, const OptTensor& skip_coef, int64_t skip_head) {
  check_cuda(in, "in");
  check_cuda(out, "out");
  AKV_CHECK(in.scalar_type() == at::kFloat && in.dim() == 2, "in must be float32 [tokens, width]");
  const int64_t n = in.size(0), width = in.size(1);
  AKV_CHECK(out.numel() == n * width, "out must be [tokens, width]");
  AKV_CHECK(group >= 1 && width % group == 0, "group_norm_gate: the group (", group, ") must divide the width (", width, ")");
  akv::GroupNormGateParams p{};
  if (weight.has_value()) {
    check_cuda(*weight, "weight");
    AKV_CHECK(weight->scalar_type() == at::kFloat && (weight->numel() == group || weight->numel() == width),
              "weight must be float32 with a group's or the whole width's entries");
    p.weight = weight->data_ptr<float>();
    p.weight_len = (int)weight->numel();
  }
  if (x.has_value()) {
    check_cuda(*x, "x");
    check_same(*x, out, "x", "out");
    AKV_CHECK(x->dim() == 2 && x->size(0) == n && gate_off >= 0 && gate_off + width <= x->size(1),
              "the gate columns must lie inside x");
    AKV_CHECK(gate_kind == 0 || gate_kind == 1, "gate_kind: 0 sigmoid, 1 SiLU");
    p.x = x->data_ptr();
    p.x_stride = x->size(1);
  }
  if (skip.has_value()) {
    check_cuda(*skip, "skip");
    AKV_CHECK(skip->scalar_type() == at::kFloat && skip->dim() == 2 && skip->size(0) == n && skip_off >= 0 &&
                  skip_off + width <= skip->size(1), "the skip columns must lie inside skip (float32 [tokens, columns])");
    AKV_CHECK(skip_coef.has_value() && skip_head >= 1 && width % skip_head == 0,
              "skip needs a coefficient per run of skip_head columns");
    check_f32(*skip_coef, "skip_coef", width / skip_head);
    p.skip = skip->data_ptr<float>();
    p.skip_stride = skip->size(1);
    p.skip_off = (int)skip_off;
    p.skip_coef = skip_coef->data_ptr<float>();
    p.skip_head = (int)skip_head;
  }
  p.in = in.data_ptr<float>();
  p.out = out.data_ptr();
  p.num_tokens = n;
  p.width = (int)width;
  p.group = (int)group;
  p.eps = (float)eps;
  p.factor = (float)factor;
  p.gate_off = (int)gate_off;
  p.gate_kind = (int)gate_kind;
  p.gate_first = gate_first ? 1 : 0;
  p.dtype = dtype_code(out, "out");
  c10::cuda::CUDAGuard guard(in.device());
  check_launch(akv::launch_group_norm_gate(p, stream_of(in)), "group_norm_gate");
}

void rotary_prep(const Tensor& x, const Tensor& positions, const OptTensor& slots, const Tensor& freq, Tensor& q_out,
                 const OptTensor& k_cache, const OptTensor& v_cache, int64_t num_heads, int64_t num_kv_heads,
                 int64_t head_dim, int64_t v_dim, int64_t rotary_dims, int64_t layout, double factor,
                 bool value_from_key, bool value_norm, double eps, const OptTensor& status, const OptTensor& q_norm,
                 const OptTensor& k_norm, double row_norm_eps, int64_t x_off) {
  check_cuda(x, "x");
  check_cuda(q_out, "q_out");
  check_same(x, q_out, "x", "q_out");
  AKV_CHECK(num_heads > 0 && num_kv_heads > 0 && head_dim > 0 && v_dim > 0, "rotary_prep: sizes must be positive");
  AKV_CHECK(rotary_dims >= 0 && rotary_dims % 2 == 0 && rotary_dims <= head_dim && (layout == 0 || layout == 1),
            "rotary_prep: rotary_dims must be even and at most the head's width; layout 0 or 1");
  AKV_CHECK(!value_from_key || v_dim == head_dim, "rotary_prep: a value that is its key has the key's width");
  const int64_t width = (num_heads + num_kv_heads) * head_dim + (value_from_key ? 0 : num_kv_heads * v_dim);
  AKV_CHECK(x.dim() == 2 && x_off >= 0 && x.size(1) >= x_off + width,
            "x must hold the ", width, " q, k (and v) columns of a token from column x_off on");
  const int64_t n = x.size(0);
  check_i32(positions, "positions", n);
  check_f32(freq, "freq", rotary_dims / 2);
  AKV_CHECK(q_out.numel() == n * num_heads * head_dim, "q_out must be [tokens, heads * head_dim]");
  akv::RotaryPrepParams p{};
  p.x = static_cast<const char*>(x.data_ptr()) + x_off * x.element_size();
  p.x_stride = x.size(1);
  p.positions = positions.data_ptr<int>();
  p.freq = freq.data_ptr<float>();
  p.q_out = q_out.data_ptr();
  if (slots.has_value()) {
    check_i32(*slots, "slots", n);
    p.slots = slots->data_ptr<int>();
  }
  if (k_cache.has_value()) {
    AKV_CHECK(v_cache.has_value() && slots.has_value(), "k_cache needs v_cache and slots");
    check_pages(*k_cache, "k_cache", num_kv_heads, head_dim, x);
    check_pages(*v_cache, "v_cache", num_kv_heads, v_dim, x);
    AKV_CHECK(k_cache->size(0) == v_cache->size(0) && k_cache->size(2) == v_cache->size(2),
              "k_cache and v_cache must have the same pages and page size");
    p.k_cache = k_cache->data_ptr();
    p.v_cache = v_cache->data_ptr();
    p.page_size = (int)k_cache->size(2);
    p.num_pages = k_cache->size(0);
    p.k_row_stride = k_cache->size(3);
    p.v_row_stride = v_cache->size(3);
  }
  p.num_tokens = n;
  p.num_heads = (int)num_heads;
  p.num_kv_heads = (int)num_kv_heads;
  p.head_dim = (int)head_dim;
  p.v_dim = (int)v_dim;
  p.rotary_dims = (int)rotary_dims;
  p.layout = (int)layout;
  p.factor = (float)factor;
  p.value_from_key = value_from_key ? 1 : 0;
  p.value_norm = value_norm ? 1 : 0;
  p.eps = (float)eps;
  AKV_CHECK(q_norm.has_value() == k_norm.has_value(), "rotary_prep: q_norm and k_norm come together");
  if (q_norm.has_value()) {
    check_f32(*q_norm, "q_norm", num_heads * head_dim);
    check_f32(*k_norm, "k_norm", num_kv_heads * head_dim);
    p.q_norm = q_norm->data_ptr<float>();
    p.k_norm = k_norm->data_ptr<float>();
    p.row_norm_eps = (float)row_norm_eps;
  }
  p.dtype = dtype_code(x, "x");
  p.status = status_ptr(status);
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_rotary_prep(p, stream_of(x)), "rotary_prep");
}

void pair_rows_add(Tensor& hidden, const Tensor& ids, const OptTensor& sampled, const Tensor& positions,
                   const Tensor& cu_q, const Tensor& state_slots, Tensor& last_token, const Tensor& table,
                   int64_t vocab, int64_t buckets, int64_t mul_prev, int64_t mul_cur) {
  check_cuda(table, "table");
  AKV_CHECK(table.dim() == 2 && table.size(0) == buckets + 1 && buckets >= 1, "table must be [buckets + 1, hidden]");
  const int64_t n = ids.numel(), h = table.size(1);
  check_i32(ids, "ids");
  check_f32(hidden, "hidden", n * h);
  check_i32(positions, "positions", n);
  check_i32(cu_q, "cu_q");
  const int64_t seqs = cu_q.numel() - 1;
  AKV_CHECK(seqs >= 1, "cu_q must hold at least one sequence");
  check_i32(state_slots, "state_slots", seqs);
  AKV_CHECK(last_token.is_cuda() && last_token.scalar_type() == at::kInt && last_token.dim() == 2 &&
            last_token.size(1) >= 1, "last_token must be int32 [slots, at least 1]");
  akv::PairRowsParams p{};
  p.ids = ids.data_ptr<int>();
  if (sampled.has_value()) {
    check_i32(*sampled, "sampled");
    p.sampled = sampled->data_ptr<int>();
    p.num_sampled = sampled->numel();
  }
  p.positions = positions.data_ptr<int>();
  p.cu_q = cu_q.data_ptr<int>();
  p.state_slots = state_slots.data_ptr<int>();
  p.last_token = last_token.data_ptr<int>();
  p.state_stride = last_token.stride(0);
  p.table = table.data_ptr();
  p.hidden = hidden.data_ptr<float>();
  p.num_tokens = n;
  p.hidden_size = h;
  p.vocab = vocab;
  p.buckets = buckets;
  p.mul_prev = mul_prev;
  p.mul_cur = mul_cur;
  p.num_seqs = (int)seqs;
  p.dtype = dtype_code(table, "table");
  c10::cuda::CUDAGuard guard(table.device());
  check_launch(akv::launch_pair_rows_add(p, stream_of(table)), "pair_rows_add");
}

void stream_add(Tensor& hidden, const Tensor& other) {
  check_f32(hidden, "hidden");
  check_f32(other, "other", hidden.numel());
  c10::cuda::CUDAGuard guard(hidden.device());
  check_launch(akv::launch_stream_add(hidden.data_ptr<float>(), other.data_ptr<float>(), hidden.numel(),
                                      stream_of(hidden)), "stream_add");
}

void scaled_sum(const Tensor& a, const Tensor& b, Tensor& out, double sa, double sb) {
  check_cuda(a, "a");
  check_cuda(b, "b");
  check_cuda(out, "out");
  check_same(a, b, "a", "b");
  check_same(a, out, "a", "out");
  AKV_CHECK(a.numel() == b.numel() && a.numel() == out.numel(), "a, b and out must have the same size");
  c10::cuda::CUDAGuard guard(a.device());
  check_launch(akv::launch_scaled_sum(a.data_ptr(), b.data_ptr(), out.data_ptr(), (float)sa, (float)sb, a.numel(),
                                      dtype_code(a, "a"), stream_of(a)), "scaled_sum");
}

// The q, k and v heads of one product as float32 rows [q | k | v], q and k turned by position (see launchers.h).
void rotary_rows(const Tensor& x, const Tensor& positions, const Tensor& freq, Tensor& out, int64_t num_heads,
                 int64_t head_dim, int64_t v_dim, int64_t rotary_dims, int64_t q_off, int64_t k_off, int64_t v_off,
                 double q_scale, double k_scale) {
  check_cuda(x, "x");
  AKV_CHECK(x.dim() == 2 && num_heads > 0 && head_dim > 0 && v_dim > 0, "rotary_rows: x [tokens, columns], positive sizes");
  AKV_CHECK(rotary_dims >= 0 && rotary_dims % 2 == 0 && rotary_dims <= head_dim,
            "rotary_rows: rotary_dims must be even and at most the head's width");
  const int64_t n = x.size(0), qk = num_heads * head_dim, vw = num_heads * v_dim;
  AKV_CHECK(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + qk <= x.size(1) && k_off + qk <= x.size(1) &&
            v_off + vw <= x.size(1), "rotary_rows: the q, k and v columns must lie inside x");
  check_i32(positions, "positions", n);
  check_f32(freq, "freq", rotary_dims / 2);
  check_cuda(out, "out");
  AKV_CHECK(out.scalar_type() == at::kFloat && out.dim() == 2 && out.size(0) == n && out.size(1) >= 2 * qk + vw,
            "out must be float32 [tokens, at least 2 * heads * head_dim + heads * v_dim]");
  akv::RotaryRowsParams p{};
  p.x = x.data_ptr();
  p.x_stride = x.size(1);
  p.q_off = (int)q_off;
  p.k_off = (int)k_off;
  p.v_off = (int)v_off;
  p.positions = positions.data_ptr<int>();
  p.freq = freq.data_ptr<float>();
  p.out = out.data_ptr<float>();
  p.out_stride = out.size(1);
  p.num_tokens = n;
  p.num_heads = (int)num_heads;
  p.head_dim = (int)head_dim;
  p.v_dim = (int)v_dim;
  p.rotary_dims = (int)rotary_dims;
  p.q_scale = (float)q_scale;
  p.k_scale = (float)k_scale;
  p.dtype = dtype_code(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_rotary_rows(p, stream_of(x)), "rotary_rows");
}

// Hyper-connections (see launchers.h).  x [tokens, streams, width] float32; y the pending sublayer result.
akv::HyperStepParams hyper_params(Tensor& x, const OptTensor& y, const OptTensor& mix, const OptTensor& write,
                                  const OptTensor& scale) {
  check_cuda(x, "x");
  AKV_CHECK(x.scalar_type() == at::kFloat && x.dim() == 3, "x must be float32 [tokens, streams, width]");
  const int64_t n = x.size(0), streams = x.size(1), width = x.size(2);
  AKV_CHECK(streams >= 1 && streams <= akv::kHyperMaxStreams, "hyper: 1 to ", (int64_t)akv::kHyperMaxStreams, " streams");
  akv::HyperStepParams p{};
  p.x = x.data_ptr<float>();
  p.num_tokens = n;
  p.streams = (int)streams;
  p.width = (int)width;
  if (y.has_value()) {
    check_cuda(*y, "y");
    AKV_CHECK(y->numel() == n * width && y->device() == x.device(), "y must be [tokens, width]");
    AKV_CHECK(mix.has_value() && write.has_value(), "y needs mix and write");
    check_f32(*mix, "mix", streams * streams);
    check_f32(*write, "write", streams);
    p.y = y->data_ptr();
    p.y_dtype = dtype_code(*y, "y");
    p.mix = mix->data_ptr<float>();
    p.write = write->data_ptr<float>();
    if (scale.has_value()) {
      check_f32(*scale, "scale", width);
      p.scale = scale->data_ptr<float>();
    }
  }
  return p;
}

void hyper_step(Tensor& x, const OptTensor& y, const OptTensor& mix, const OptTensor& write, const OptTensor& scale,
                const OptTensor& read, const OptTensor& weight, double eps, const OptTensor& out, const OptTensor& rows,
                const OptTensor& status) {
  akv::HyperStepParams p = hyper_params(x, y, mix, write, scale);
  AKV_CHECK(y.has_value() || out.has_value(), "hyper_step: nothing to do");
  if (out.has_value()) {
    AKV_CHECK(read.has_value() && weight.has_value(), "out needs read and weight");
    check_f32(*read, "read", p.streams);
    check_f32(*weight, "weight", p.width);
    check_cuda(*out, "out");
    int64_t out_rows = p.num_tokens;
    if (rows.has_value()) {
      AKV_CHECK(!y.has_value(), "hyper_step: gathered rows go without a write");
      check_i32(*rows, "rows");
      out_rows = rows->numel();
      p.rows = rows->data_ptr<int>();
      p.num_rows = out_rows;
    }
    AKV_CHECK(out->numel() == out_rows * p.width && out->device() == x.device(), "out must be [rows, width]");
    p.read = read->data_ptr<float>();
    p.weight = weight->data_ptr<float>();
    p.eps = (float)eps;
    p.out = out->data_ptr();
    p.dtype = dtype_code(*out, "out");
  }
  p.status = status_ptr(status);
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_hyper_step(p, stream_of(x)), "hyper_step");
}

void hyper_collapse(Tensor& x, const OptTensor& y, const OptTensor& mix, const OptTensor& write, const OptTensor& scale,
                    Tensor& sum) {
  akv::HyperStepParams p = hyper_params(x, y, mix, write, scale);
  check_f32(sum, "sum", p.num_tokens * p.width);
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_hyper_collapse(p, sum.data_ptr<float>(), stream_of(x)), "hyper_collapse");
}

void hyper_expand(const Tensor& in, Tensor& x) {
  check_cuda(x, "x");
  AKV_CHECK(x.scalar_type() == at::kFloat && x.dim() == 3, "x must be float32 [tokens, streams, width]");
  check_f32(in, "in", x.size(0) * x.size(2));
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_hyper_expand(in.data_ptr<float>(), x.data_ptr<float>(), x.size(0), (int)x.size(1),
                                        (int)x.size(2), stream_of(x)), "hyper_expand");
}

void normed_pair_sum(const Tensor& a, const Tensor& b, const Tensor& wa, const Tensor& wb, Tensor& out, double eps,
                     double sa, double sb) {
  check_cuda(out, "out");
  AKV_CHECK(a.dim() == 2, "a must be [tokens, width]");
  const int64_t n = a.size(0), width = a.size(1);
  check_f32(a, "a", n * width);
  check_f32(b, "b", n * width);
  check_f32(wa, "wa", width);
  check_f32(wb, "wb", width);
  AKV_CHECK(out.numel() == n * width && out.device() == a.device(), "out must be [tokens, width]");
  c10::cuda::CUDAGuard guard(a.device());
  check_launch(akv::launch_normed_pair_sum(a.data_ptr<float>(), b.data_ptr<float>(), wa.data_ptr<float>(),
                                           wb.data_ptr<float>(), out.data_ptr(), n, (int)width, (float)eps, (float)sa,
                                           (float)sb, dtype_code(out, "out"), stream_of(a)), "normed_pair_sum");
}

// A selective state-space mixer's preparation (see launchers.h).
void ssm_prep(const Tensor& x, const Tensor& conv, const OptTensor& conv_bias, const Tensor& step_bias,
              const Tensor& rate_log, const Tensor& state, int64_t tail_off, const Tensor& cu_q, const Tensor& state_slots,
              Tensor& out, int64_t num_heads, int64_t v_dim, int64_t state_dim, int64_t groups, int64_t taps,
              int64_t conv_off, int64_t step_off) {
  check_cuda(x, "x");
  AKV_CHECK(x.dim() == 2 && num_heads >= 1 && num_heads <= akv::kSsmMaxHeads && v_dim >= 1 && state_dim >= 1 &&
                groups >= 1 && num_heads % groups == 0 && taps >= 1 && taps <= akv::kConvMaxTaps,
            "ssm_prep: up to ", (int64_t)akv::kSsmMaxHeads, " heads in equal groups, 1 to ", (int64_t)akv::kConvMaxTaps, " taps");
  const int64_t n = x.size(0), inner = num_heads * v_dim, gn = groups * state_dim, channels = inner + 2 * gn;
  AKV_CHECK(conv_off >= 0 && conv_off + channels <= x.size(1) && step_off >= 0 && step_off + num_heads <= x.size(1),
            "ssm_prep: the convolved channels and the step columns must lie inside x");
  check_f32(conv, "conv", channels * taps);
  check_f32(step_bias, "step_bias", num_heads);
  check_f32(rate_log, "rate_log", num_heads);
  AKV_CHECK(state.is_cuda() && state.scalar_type() == at::kFloat && state.dim() == 2 && state.stride(1) == 1 &&
                tail_off >= 0 && tail_off + (taps - 1) * channels <= state.size(1),
            "state must be float32 [slots, floats] with room for the convolutions' inputs behind tail_off");
  check_i32(cu_q, "cu_q");
  const int64_t seqs = cu_q.numel() - 1;
  check_i32(state_slots, "state_slots", seqs);
  check_cuda(out, "out");
  AKV_CHECK(out.scalar_type() == at::kFloat && out.dim() == 2 && out.size(0) == n && out.size(1) >= 2 * gn + 2 * inner + num_heads,
            "out must be float32 [tokens, at least 2 * groups * state + 2 * heads * v_dim + heads]");
  akv::SsmPrepParams p{};
  p.x = x.data_ptr();
  p.x_stride = x.size(1);
  p.conv_off = (int)conv_off;
  p.step_off = (int)step_off;
  p.conv = conv.data_ptr<float>();
  if (conv_bias.has_value()) {
    check_f32(*conv_bias, "conv_bias", channels);
    p.conv_bias = conv_bias->data_ptr<float>();
  }
  p.step_bias = step_bias.data_ptr<float>();
  p.rate_log = rate_log.data_ptr<float>();
  p.state = state.data_ptr<float>();
  p.state_stride = state.stride(0);
  p.tail_off = tail_off;
  p.cu_q = cu_q.data_ptr<int>();
  p.state_slots = state_slots.data_ptr<int>();
  p.out = out.data_ptr<float>();
  p.out_stride = out.size(1);
  p.num_tokens = n;
  p.num_seqs = (int)seqs;
  p.num_slots = (int)state.size(0);
  p.num_heads = (int)num_heads;
  p.v_dim = (int)v_dim;
  p.state_dim = (int)state_dim;
  p.groups = (int)groups;
  p.taps = (int)taps;
  p.dtype = dtype_code(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_ssm_prep(p, stream_of(x)), "ssm_prep");
}

// The last taps - 1 inputs of `channels` convolved columns of x, per sequence, into the state slot behind tail_off.
void conv_tail(const Tensor& x, Tensor& state, int64_t tail_off, const Tensor& cu_q, const Tensor& state_slots,
               int64_t conv_off, int64_t channels, int64_t taps) {
  check_cuda(x, "x");
  AKV_CHECK(x.dim() == 2 && channels >= 1 && taps >= 1 && taps <= akv::kConvMaxTaps && conv_off >= 0 &&
                conv_off + channels <= x.size(1), "conv_tail: the channels must lie inside x; 1 to ",
            (int64_t)akv::kConvMaxTaps, " taps");
  AKV_CHECK(state.is_cuda() && state.scalar_type() == at::kFloat && state.dim() == 2 && state.stride(1) == 1 &&
                tail_off >= 0 && tail_off + (taps - 1) * channels <= state.size(1),
            "state must be float32 [slots, floats] with room for the inputs behind tail_off");
  check_i32(cu_q, "cu_q");
  const int64_t seqs = cu_q.numel() - 1;
  check_i32(state_slots, "state_slots", seqs);
  akv::ConvTailParams p{};
  p.x = x.data_ptr();
  p.x_stride = x.size(1);
  p.conv_off = (int)conv_off;
  p.channels = (int)channels;
  p.taps = (int)taps;
  p.state = state.data_ptr<float>();
  p.state_stride = state.stride(0);
  p.tail_off = tail_off;
  p.cu_q = cu_q.data_ptr<int>();
  p.state_slots = state_slots.data_ptr<int>();
  p.num_seqs = (int)seqs;
  p.num_slots = (int)state.size(0);
  p.dtype = dtype_code(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_conv_tail(p, stream_of(x)), "conv_tail");
}

void moe_route(const Tensor& logits, const OptTensor& correction, Tensor& chosen, Tensor& weights, int64_t groups,
               int64_t keep_groups, int64_t group_top, double scale, double weight_eps, int64_t score_kind) {
  check_cuda(logits, "logits");
  AKV_CHECK(logits.scalar_type() == at::kFloat && logits.dim() == 2, "logits must be float32 [tokens, experts]");
  const int64_t n = logits.size(0), experts = logits.size(1);
  check_i32(chosen, "chosen");
  AKV_CHECK(chosen.dim() == 2 && chosen.size(0) == n, "chosen must be [tokens, top]");
  const int64_t top = chosen.size(1);
  check_f32(weights, "weights", n * top);
  AKV_CHECK(experts >= 1 && experts <= akv::kMoeMaxExperts && top >= 1 && top <= 32 && top <= experts,
            "moe_route: up to ", (int64_t)akv::kMoeMaxExperts, " experts and a top of up to 32");
  AKV_CHECK(groups >= 1 && experts % groups == 0 && keep_groups >= 1 && keep_groups <= groups && group_top >= 1 &&
                top <= keep_groups * (experts / groups),
            "moe_route: the groups must divide the experts and the kept groups hold the top");
  akv::MoeRouteParams p{};
  p.logits = logits.data_ptr<float>();
  if (correction.has_value()) {
    check_f32(*correction, "correction", experts);
    p.correction = correction->data_ptr<float>();
  }
  p.chosen = chosen.data_ptr<int>();
  p.weights = weights.data_ptr<float>();
  p.num_tokens = n;
  p.experts = (int)experts;
  p.top = (int)top;
  p.groups = (int)groups;
  p.keep_groups = (int)keep_groups;
  p.group_top = (int)group_top;
  p.scale = (float)scale;
  p.weight_eps = (float)weight_eps;
  AKV_CHECK(score_kind == 0 || score_kind == 1, "moe_route: score_kind 0 (sigmoid) or 1 (softmax)");
  p.score_kind = (int)score_kind;
  c10::cuda::CUDAGuard guard(logits.device());
  check_launch(akv::launch_moe_route(p, stream_of(logits)), "moe_route");
}

void moe_router(const Tensor& x, const Tensor& w, Tensor& logits) {
  check_cuda(x, "x");
  check_cuda(w, "w");
  check_same(x, w, "x", "w");
  AKV_CHECK(x.dim() == 2 && w.dim() == 2 && w.size(1) == x.size(1), "moe_router: x [tokens, hidden], w [experts, hidden]");
  check_f32(logits, "logits", x.size(0) * w.size(0));
  AKV_CHECK(x.size(0) <= 65535, "moe_router: at most 65535 tokens");
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_moe_router(x.data_ptr(), w.data_ptr(), logits.data_ptr<float>(), x.size(0), (int)w.size(0),
                                      (int)x.size(1), dtype_code(x, "x"), stream_of(x)),
               "moe_router");
}

void moe_sort(const Tensor& chosen, Tensor& order, Tensor& offsets) {
  check_i32(chosen, "chosen");
  check_i32(order, "order", chosen.numel());
  check_i32(offsets, "offsets", 2);
  const int64_t experts = offsets.numel() - 1;
  AKV_CHECK(experts <= akv::kMoeMaxExperts, "moe_sort: up to ", (int64_t)akv::kMoeMaxExperts, " experts");
  c10::cuda::CUDAGuard guard(chosen.device());
  check_launch(akv::launch_moe_sort(chosen.data_ptr<int>(), order.data_ptr<int>(), offsets.data_ptr<int>(),
                                    chosen.numel(), (int)experts, stream_of(chosen)),
               "moe_sort");
}

void moe_gate_up(const Tensor& x, const Tensor& w, const Tensor& order, const Tensor& offsets, Tensor& act, int64_t top,
                 double limit, double slope, int64_t form, double up_offset) {
  check_cuda(x, "x");
  check_cuda(w, "w");
  check_cuda(act, "act");
  check_same(x, w, "x", "w");
  check_same(x, act, "x", "act");
  AKV_CHECK(x.dim() == 2 && w.dim() == 3 && w.size(2) == x.size(1) && w.size(1) % 2 == 0,
            "moe_gate_up: x [tokens, hidden], w [experts, 2 * intermediate, hidden]");
  const int64_t pairs = order.numel(), experts = w.size(0), inter = w.size(1) / 2;
  check_i32(order, "order");
  check_i32(offsets, "offsets", experts + 1);
  AKV_CHECK(top >= 1 && pairs == x.size(0) * top && act.numel() == pairs * inter && limit > 0,
            "moe_gate_up: order holds tokens * top pairs, act [pairs, intermediate], a positive limit");
  akv::MoeGemmParams p{};
  p.a = x.data_ptr();
  p.w = w.data_ptr();
  p.order = order.data_ptr<int>();
  p.offsets = offsets.data_ptr<int>();
  p.out = act.data_ptr();
  p.pairs = pairs;
  p.experts = (int)experts;
  p.k = (int)x.size(1);
  p.n = (int)inter;
  p.top = (int)top;
  p.limit = (float)limit;
  p.slope = (float)slope;
  p.up_offset = (float)up_offset;
  p.dtype = dtype_code(x, "x");
  AKV_CHECK(form >= 0 && form <= 3, "form: 0 by size, 1 float arithmetic, 2 mma.sync tiles, 3 few rows");
  p.force_plain = (int)form;
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(akv::launch_moe_gemm(p, true, stream_of(x)), "moe_gate_up");
}

void moe_down(const Tensor& act, const Tensor& w, const Tensor& order, const Tensor& offsets, const Tensor& weights,
              Tensor& out, int64_t form) {
  check_cuda(act, "act");
  check_cuda(w, "w");
  check_same(act, w, "act", "w");
  AKV_CHECK(act.dim() == 2 && w.dim() == 3 && w.size(2) == act.size(1), "moe_down: act [pairs, intermediate], w [experts, hidden, intermediate]");
  const int64_t pairs = act.size(0), experts = w.size(0), hidden = w.size(1);
  check_i32(order, "order", pairs);
  check_i32(offsets, "offsets", experts + 1);
  check_f32(weights, "weights", pairs);
  check_f32(out, "out", pairs * hidden);
  AKV_CHECK(order.numel() == pairs, "moe_down: a pair per row of act");
  akv::MoeGemmParams p{};
  p.a = act.data_ptr();
  p.w = w.data_ptr();
  p.order = order.data_ptr<int>();
  p.offsets = offsets.data_ptr<int>();
  p.weights = weights.data_ptr<float>();
  p.out = out.data_ptr();
  p.pairs = pairs;
  p.experts = (int)experts;
  p.k = (int)act.size(1);
  p.n = (int)hidden;
  p.top = 1;
  p.dtype = dtype_code(act, "act");
  AKV_CHECK(form >= 0 && form <= 3, "form: 0 by size, 1 float arithmetic, 2 mma.sync tiles, 3 few rows");
  p.force_plain = (int)form;
  c10::cuda::CUDAGuard guard(act.device());
  check_launch(akv::launch_moe_gemm(p, false, stream_of(act)), "moe_down");
}

void moe_combine(const Tensor& parts, const OptTensor& shared, Tensor& out, int64_t top) {
  check_cuda(parts, "parts");
  AKV_CHECK(parts.scalar_type() == at::kFloat && parts.dim() == 2 && top >= 1 && parts.size(0) % top == 0,
            "moe_combine: parts must be float32 [tokens * top, hidden]");
  const int64_t n = parts.size(0) / top, h = parts.size(1);
  check_f32(out, "out", n * h);
  const void* shared_ptr = nullptr;
  int shared_code = 0;
  if (shared.has_value()) {
    check_cuda(*shared, "shared");
    AKV_CHECK(shared->numel() == n * h && shared->device() == parts.device(), "shared must be [tokens, hidden]");
    shared_ptr = shared->data_ptr();
    shared_code = dtype_code(*shared, "shared");
  }
  c10::cuda::CUDAGuard guard(parts.device());
  check_launch(akv::launch_moe_combine(parts.data_ptr<float>(), shared_ptr, shared_code, out.data_ptr<float>(), n, h,
                                       (int)top, stream_of(parts)),
               "moe_combine");
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
        py::arg("sampled") = py::none(), py::arg("scale") = 1.0, py::arg("positions") = py::none(),
        py::arg("position_rows") = py::none());
  m.def("add_rmsnorm", &add_rmsnorm, py::arg("hidden"), py::arg("delta"), py::arg("weight"), py::arg("out"),
        py::arg("rows"), py::arg("eps"), py::arg("status") = py::none());
  m.def("silu_mul", &silu_mul, py::arg("gate_up"), py::arg("out"), py::arg("block") = 0);
  m.def("small_m_gemm", &small_m_gemm, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("splits") = 1,
        py::arg("status") = py::none(), py::arg("gated") = false, py::arg("nx_hidden") = py::none(),
        py::arg("nx_ssq") = py::none(), py::arg("nx_weight") = py::none(), py::arg("nx_eps") = 0.0,
        py::arg("activation") = -1);
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
  m.def("scored_attention", &scored_attention, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"),
        py::arg("block_table"), py::arg("cu_q"), py::arg("ctx_lens"), py::arg("tile_seq"), py::arg("tile_q0"),
        py::arg("tile_nq"), py::arg("partials"), py::arg("num_tiles"), py::arg("q_tile"), py::arg("num_splits"),
        py::arg("num_heads"), py::arg("num_kv_heads"), py::arg("v_dim"), py::arg("window"), py::arg("chunk"),
        py::arg("scale"), py::arg("softcap"), py::arg("slopes") = py::none(), py::arg("gate") = py::none(),
        py::arg("status") = py::none(), py::arg("kernel") = 0, py::arg("keep_first") = 0, py::arg("sigmoid_weights") = false,
        py::arg("head_bias") = py::none(), py::arg("out_scale") = 1.0);
  m.def("head_prep", &head_prep, py::arg("x"), py::arg("slots"), py::arg("q_out"), py::arg("k_cache"),
        py::arg("v_cache"), py::arg("v_keep"), py::arg("v_other"), py::arg("blend_weight"), py::arg("gate_out"),
        py::arg("num_heads"), py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("v_dim"), py::arg("unit_norm"),
        py::arg("eps"), py::arg("status") = py::none(), py::arg("q_weight") = py::none(),
        py::arg("k_weight") = py::none(), py::arg("has_kv") = true);
  m.def("latent_prep", &latent_prep, py::arg("x"), py::arg("positions"), py::arg("slots"), py::arg("q_weight"),
        py::arg("kv_weight"), py::arg("inv_freq"), py::arg("q_latent"), py::arg("cache"), py::arg("q_rank"),
        py::arg("kv_rank"), py::arg("rot_dim"), py::arg("rotary_dims"), py::arg("eps"), py::arg("status") = py::none());
  m.def("rotate_pairs", &rotate_pairs, py::arg("in"), py::arg("out"), py::arg("positions"), py::arg("inv_freq"),
        py::arg("heads"), py::arg("cols"), py::arg("rotary_dims"), py::arg("in_offset"), py::arg("out_offset"));
  m.def("activation", &activation, py::arg("in"), py::arg("out"), py::arg("kind"));
  m.def("add_layernorm", &add_layernorm, py::arg("hidden"), py::arg("delta"), py::arg("weight"), py::arg("out"),
        py::arg("rows"), py::arg("eps"), py::arg("status") = py::none());
  m.def("branch_layernorm", &branch_layernorm, py::arg("hidden"), py::arg("branch"), py::arg("weight"), py::arg("copy"),
        py::arg("eps"));
  m.def("branch_layernorm_parts", &branch_layernorm_parts, py::arg("hidden"), py::arg("parts"), py::arg("shared"),
        py::arg("weight"), py::arg("copy"), py::arg("eps"), py::arg("top"));
  m.def("stream_copy", &stream_copy, py::arg("hidden"), py::arg("out"));
  m.def("glu", &glu, py::arg("gate_up"), py::arg("out"), py::arg("kind"), py::arg("block") = 0, py::arg("limit") = 0.0,
        py::arg("slope") = 1.0);
  m.def("softcap", &softcap, py::arg("logits"), py::arg("cap"));
  m.def("delta_prep", &delta_prep, py::arg("x"), py::arg("conv"), py::arg("rate_log"), py::arg("step_bias"),
        py::arg("state"), py::arg("cu_q"), py::arg("state_slots"), py::arg("qkv"), py::arg("coef"), py::arg("num_heads"),
        py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("v_dim"), py::arg("taps"), py::arg("unit_eps"));
  m.def("delta_scan", &delta_scan, py::arg("qkv"), py::arg("coef"), py::arg("x"), py::arg("norm_weight"), py::arg("state"),
        py::arg("cu_q"), py::arg("state_slots"), py::arg("scratch"), py::arg("out"), py::arg("num_heads"),
        py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("v_dim"), py::arg("taps"), py::arg("norm_eps"));
  m.def("delta_scan_supported", [](int64_t dim, int64_t v_dim) { return akv::delta_scan_supported((int)dim, (int)v_dim); });
  m.def("delta_memory_floats", [](int64_t heads, int64_t dim, int64_t v_dim) {
    return akv::delta_memory_floats((int)heads, (int)dim, (int)v_dim);
  });
  m.def("linear_scan", &linear_scan, py::arg("x"), py::arg("state"), py::arg("cu_q"), py::arg("state_slots"),
        py::arg("out"), py::arg("num_heads"), py::arg("head_dim"), py::arg("v_dim"), py::arg("mode"), py::arg("q_off"),
        py::arg("k_off"), py::arg("v_off"), py::arg("gate_bias") = py::none(), py::arg("lower") = py::none(),
        py::arg("decay") = py::none(), py::arg("qk_group") = 1, py::arg("decay_off") = 0);
  m.def("linear_scan_state_floats", [](int64_t heads, int64_t dim, int64_t v_dim) {
    return (int64_t)akv::linear_scan_state_floats((int)heads, (int)dim, (int)v_dim);
  });
  m.def("group_norm_gate", &group_norm_gate, py::arg("in"), py::arg("out"), py::arg("weight"), py::arg("group"),
        py::arg("eps"), py::arg("factor") = 1.0, py::arg("x") = py::none(), py::arg("gate_off") = 0,
        py::arg("gate_kind") = 0, py::arg("gate_first") = false, py::arg("skip") = py::none(), py::arg("skip_off") = 0,
        py::arg("skip_coef") = py::none(), py::arg("skip_head") = 1);
  m.def("rotary_prep", &rotary_prep, py::arg("x"), py::arg("positions"), py::arg("slots"), py::arg("freq"),
        py::arg("q_out"), py::arg("k_cache"), py::arg("v_cache"), py::arg("num_heads"), py::arg("num_kv_heads"),
        py::arg("head_dim"), py::arg("v_dim"), py::arg("rotary_dims"), py::arg("layout"), py::arg("factor") = 1.0,
        py::arg("value_from_key") = false, py::arg("value_norm") = false, py::arg("eps") = 0.0,
        py::arg("status") = py::none(), py::arg("q_norm") = py::none(), py::arg("k_norm") = py::none(),
        py::arg("row_norm_eps") = 0.0, py::arg("x_off") = 0);
  m.def("pair_rows_add", &pair_rows_add, py::arg("hidden"), py::arg("ids"), py::arg("sampled"), py::arg("positions"),
        py::arg("cu_q"), py::arg("state_slots"), py::arg("last_token"), py::arg("table"), py::arg("vocab"),
        py::arg("buckets"), py::arg("mul_prev"), py::arg("mul_cur"));
  m.def("stream_add", &stream_add, py::arg("hidden"), py::arg("other"));
  m.def("rotary_rows", &rotary_rows, py::arg("x"), py::arg("positions"), py::arg("freq"), py::arg("out"),
        py::arg("num_heads"), py::arg("head_dim"), py::arg("v_dim"), py::arg("rotary_dims"), py::arg("q_off"),
        py::arg("k_off"), py::arg("v_off"), py::arg("q_scale") = 1.0, py::arg("k_scale") = 1.0);
  m.def("hyper_step", &hyper_step, py::arg("x"), py::arg("y"), py::arg("mix"), py::arg("write"), py::arg("scale"),
        py::arg("read"), py::arg("weight"), py::arg("eps"), py::arg("out"), py::arg("rows") = py::none(),
        py::arg("status") = py::none());
  m.def("hyper_collapse", &hyper_collapse, py::arg("x"), py::arg("y"), py::arg("mix"), py::arg("write"),
        py::arg("scale"), py::arg("sum"));
  m.def("hyper_expand", &hyper_expand, py::arg("in"), py::arg("x"));
  m.def("normed_pair_sum", &normed_pair_sum, py::arg("a"), py::arg("b"), py::arg("wa"), py::arg("wb"), py::arg("out"),
        py::arg("eps"), py::arg("sa"), py::arg("sb"));
  m.def("ssm_prep", &ssm_prep, py::arg("x"), py::arg("conv"), py::arg("conv_bias"), py::arg("step_bias"),
        py::arg("rate_log"), py::arg("state"), py::arg("tail_off"), py::arg("cu_q"), py::arg("state_slots"),
        py::arg("out"), py::arg("num_heads"), py::arg("v_dim"), py::arg("state_dim"), py::arg("groups"), py::arg("taps"),
        py::arg("conv_off"), py::arg("step_off"));
  m.def("conv_tail", &conv_tail, py::arg("x"), py::arg("state"), py::arg("tail_off"), py::arg("cu_q"),
        py::arg("state_slots"), py::arg("conv_off"), py::arg("channels"), py::arg("taps"));
  m.def("scaled_sum", &scaled_sum, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("sa"), py::arg("sb"));
  m.def("moe_route", &moe_route, py::arg("logits"), py::arg("correction"), py::arg("chosen"), py::arg("weights"),
        py::arg("groups"), py::arg("keep_groups"), py::arg("group_top"), py::arg("scale"), py::arg("weight_eps"),
        py::arg("score_kind") = 0);
  m.def("moe_router", &moe_router, py::arg("x"), py::arg("w"), py::arg("logits"));
  m.def("moe_sort", &moe_sort, py::arg("chosen"), py::arg("order"), py::arg("offsets"));
  m.def("moe_gate_up", &moe_gate_up, py::arg("x"), py::arg("w"), py::arg("order"), py::arg("offsets"), py::arg("act"),
        py::arg("top"), py::arg("limit"), py::arg("slope"), py::arg("form") = 0, py::arg("up_offset") = 1.0);
  m.def("moe_down", &moe_down, py::arg("act"), py::arg("w"), py::arg("order"), py::arg("offsets"), py::arg("weights"),
        py::arg("out"), py::arg("form") = 0);
  m.def("moe_combine", &moe_combine, py::arg("parts"), py::arg("shared"), py::arg("out"), py::arg("top"));
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
