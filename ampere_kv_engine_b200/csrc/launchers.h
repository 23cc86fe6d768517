// Host launchers of the hand-written kernels.  Plain C++ signatures over raw device
// pointers so that the .cu files compile without any tensor-library header; bindings.cpp
// checks shapes, dtypes, devices and contiguity before it calls these.
//
// `dtype` is akv::DType (0 = float32, 1 = bfloat16) and names the storage type of
// activations / matrices / cache pages; norm weights, rotary tables and logits are float32.
// Every launcher enqueues on `stream` and returns the launch's cudaError_t as int.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace akv {

// Streaming multiprocessors of the current device, asked once per device.  When no device answers (a build box
// without a GPU) the count of the B200 this package is written for stands in.
constexpr int kFallbackSmCount = 148;
int sm_count();

// Runs the package's bounded mbarrier wait on a barrier that nothing completes, `limit` tries (at most a million),
// and reports kWaitTimeout in `status`: a self-test of the path a production kernel takes when a wait gives up.
int launch_wait_selftest(uint32_t limit, int* status, cudaStream_t stream);

int launch_smoke_add(const float* a, const float* b, float* out, int64_t n, cudaStream_t stream);

// hidden[n, :] = float(table[ids[n], :]) * scale (+ float(position_rows[positions[n], :]) when a position table is
// given).  With `sampled` (may be null), an id of -(r + 1) stands for sampled[r]: the token the previous step chose
// in its row r, still on the device.
int launch_embedding(const int32_t* ids, const int32_t* sampled, int64_t num_sampled, const void* table,
                     float* hidden, int64_t num_tokens, int64_t hidden_size, int64_t vocab, int dtype, int* status,
                     cudaStream_t stream, float scale = 1.f, const int32_t* positions = nullptr,
                     const void* position_rows = nullptr, int64_t max_positions = 0);

// hidden += delta (if delta; same dtype as out); out = (x - mean) / sqrt(var + eps) * weight of every row, the
// variance being the mean of the squared deviations.  With `rows` only those rows are read and hidden is untouched.
int launch_add_layernorm(float* hidden, const void* delta, const float* weight, void* out, const int32_t* rows,
                         int64_t num_rows, int64_t num_tokens, int64_t hidden_size, float eps, int dtype, int* status,
                         cudaStream_t stream);

// hidden += LayerNorm(branch) * weight, row by row; `copy` (bfloat16 or null) receives the new hidden rounded.
int launch_branch_layernorm(float* hidden, const void* branch, int branch_dtype, const float* weight, void* copy,
                            int copy_dtype, int64_t num_tokens, int64_t hidden_size, float eps, cudaStream_t stream);

// The same with row t of the branch given as the sum of parts[t * top .. t * top + top) (float32 rows) and shared[t]
// (may be null), added in that order.
int launch_branch_layernorm_parts(float* hidden, const float* parts, int top, const void* shared, int shared_dtype,
                                  const float* weight, void* copy, int copy_dtype, int64_t num_tokens,
                                  int64_t hidden_size, float eps, cudaStream_t stream);

// out (bfloat16) = in (float32), element by element.
int launch_stream_copy(const float* in, void* out, int64_t total, cudaStream_t stream);

// out[n, i] = act(gate(n, i)) * up(n, i) over gate_up [tokens, 2 inter] whose gate and up columns alternate in runs
// of `block` columns.  kGluClampedSwish: g = min(gate, limit), u = clamp(up, -limit, limit),
// g * sigmoid(slope * g) * (u + 1).
enum Glu : int { kGluSilu = 0, kGluGeluTanh = 1, kGluClampedSwish = 2 };
int launch_glu(const void* gate_up, void* out, int64_t num_tokens, int64_t inter, int64_t block, int kind, float limit,
               float slope, int dtype, cudaStream_t stream);

// x = cap * tanh(x / cap) in place.
int launch_softcap(float* x, int64_t total, float cap, cudaStream_t stream);

// hidden += delta (if delta); out = rmsnorm(hidden) * weight.  With `rows` (num_rows entries)
// only those rows are read, hidden is left untouched and out is [num_rows, hidden_size].
// delta_parts > 0: delta is float32 [delta_parts, tokens, hidden], partial sums that are added up.
int launch_add_rmsnorm(float* hidden, const void* delta, int delta_parts, const float* weight, void* out,
                       const int32_t* rows, int64_t num_rows, int64_t num_tokens, int64_t hidden_size,
                       float eps, int dtype, int* status, cudaStream_t stream);

// out[n, i] = silu(gate(n, i)) * up(n, i).  The gate and up columns of gate_up [tokens, 2 inter] alternate in runs
// of `block` columns (block == inter: all gate columns first, the stored form of separate matrices; block == 64:
// the form that lets one 128-row GEMM tile hold both).  parts > 0: gate_up is float32 [parts, tokens, 2 inter]
// partial sums.
int launch_silu_mul(const void* gate_up, int parts, void* out, int64_t num_tokens, int64_t inter, int64_t block,
                    int dtype, cudaStream_t stream);

// Split-K weight-streaming product for few tokens (gemm_tc.cu), x [tokens, k] and w [features, k] bfloat16.
// Either out [tokens, features] (out_dtype: float32 or bfloat16; the splits are added up inside the kernel,
// splits in {1, 2, 4, 8}) or parts [splits, tokens, features] float32 (each split's sum as it is).
bool small_m_gemm_supported(int64_t tokens, int64_t features, int64_t k);
int small_m_gemm_splits(int64_t features, int64_t k);
// What the kernel does with a finished output tile besides storing it.
//   kEpilogueGated: w holds gate and up rows alternating in runs of 64, so that a 128-row tile has both for 64
//   outputs; out is [tokens, features / 2] bfloat16 = silu(gate) * up, with gate and up rounded to bfloat16 first
//   (what the unfused pair, product then launch_silu_mul, computes).
//   kEpilogueQkv: w holds the q, k and v projections of heads of 128 dims, one head per 128-row tile; the tile's
//   values, rounded to bfloat16, then go through what launch_qk_norm_rope_write does (per-head RMSNorm of q and
//   k, rotation of the whole head by position) and land in q_out / the cache pages (GemmQkv); nothing else is
//   stored.
//   kEpilogueResidual: the tile, rounded to bfloat16, is added to the float32 residual stream in place
//   (GemmResidual::hidden [tokens, features]), and the sum of squares of the new values over the tile's 128
//   features goes to ssq [tiles, tokens]: the next product can then apply the RMS norm itself (GemmNormedX).
enum GemmEpilogue : int { kEpiloguePlain = 0, kEpilogueGated = 1, kEpilogueQkv = 2, kEpilogueResidual = 3 };
struct GemmQkv {
  const int32_t* positions;  // [tokens]
  const int32_t* slots;      // [tokens] page * page_size + offset, or -1; null: K and V are not kept
  const float* q_weight;     // [128] or null: no norm
  const float* k_weight;
  const float* inv_freq;     // [64] or null: no rotation
  void* q_out;               // [tokens, num_heads * 128] bfloat16
  void* k_cache;             // [num_pages, num_kv_heads, page_size, 128] bfloat16, or null
  void* v_cache;
  int num_heads, num_kv_heads, page_size;
  int64_t num_pages;
  float eps;
};
struct GemmResidual {
  float* hidden;             // [tokens, features] float32, updated in place
  float* ssq;                // [ceil(features / 128), tokens] float32, written
};
// The token operand made inside the kernel instead of read from x: x[t, k] = hidden[t, k] * inv_rms[t] * weight[k]
// rounded to bfloat16, with inv_rms[t] = rsqrt(sum over tiles of ssq[tile, t] / k + eps): the RMS norm of
// launch_add_rmsnorm applied to a residual stream whose sums of squares a kEpilogueResidual product left behind.
struct GemmNormedX {
  const float* hidden;       // [tokens, k] float32
  const float* ssq;          // [ssq_tiles, tokens]
  const float* weight;       // [k]
  int ssq_tiles;
  float eps;
};
struct GemmFusion {
  int epilogue = kEpiloguePlain;
  GemmQkv qkv = {};
  GemmResidual residual = {};
  bool normed_x = false;     // x is null and normed says how to make it
  GemmNormedX normed = {};
  // kEpiloguePlain with a bfloat16 out only: an Activation applied to the product (rounded to bfloat16 first, as the
  // stored product would be) before it is stored; -1: none
  int activation = -1;
};
int launch_small_m_gemm(const void* x, const void* w, void* out, int out_dtype, float* parts, int64_t tokens,
                        int64_t features, int64_t k, int splits, const GemmFusion* fusion, int* status,
                        cudaStream_t stream);

// A chain of weight-streaming products in one persistent kernel (stream_phases.cu): up to kMaxStreamPhases
// products x W^T for at most 16 bfloat16 tokens, each depending on the one before, with the epilogues of
// launch_small_m_gemm.  The token operand of a phase is a bfloat16 tensor, or the RMS norm of the float32 residual
// stream `hidden` (its sums of squares come from the last residual phase of the launch, or are added up in the kernel
// when there is none).
constexpr int kMaxStreamPhases = 4;
enum StreamX : int { kStreamXTensor = 0, kStreamXNormed = 1 };
struct StreamPhase {
  const void* w;             // [features, k] bfloat16
  int64_t features, k;
  int x_kind;                // StreamX
  const void* x;             // kStreamXTensor: [tokens, k] bfloat16
  const float* norm_weight;  // kStreamXNormed: [k]
  float eps;
  int epilogue;              // GemmEpilogue; kEpilogueResidual adds into `hidden` (features == hidden_size)
  void* out;                 // plain: bfloat16 [tokens, features]; gated: bfloat16 [tokens, features / 2]
  GemmQkv qkv;               // kEpilogueQkv
};
// CTAs the kernel asks for (one per SM, in clusters of four), and the scratch a launch needs: float32 words for
// partial tiles (none: they stay in shared memory) and int32 counters, one per phase, zero at launch.
int stream_phases_grid();
void stream_phases_scratch(const StreamPhase* phases, int num_phases, int64_t* part_floats, int64_t* sync_ints);
// `trace` (null in production): int64 [grid, kMaxStreamPhases, 16] that receives nanosecond stamps of each CTA's
// progress through each phase, for measurements.
int launch_stream_phases(const StreamPhase* phases, int num_phases, int64_t tokens, float* hidden,
                         int64_t hidden_size, float* ssq, float* parts, int* sync, int* status,
                         cudaStream_t stream, unsigned long long* trace = nullptr);

struct QkRopeWriteParams {
  const void* qkv;          // [N, (NH + 2 NKV) * D]; with qkv_parts > 0: float32 [qkv_parts, N, ...] partial sums
  int qkv_parts;
  const int32_t* positions; // [N]
  const int32_t* slots;     // [N] page * page_size + offset, or -1: do not write; may be null
  const float* q_weight;    // [D] or null: no norm
  const float* k_weight;    // [D] or null
  const float* inv_freq;    // [rotary_dim / 2] or null: no rotation
  void* q_out;              // [N, NH * D]
  void* k_out;              // [N, NKV * D] or null
  void* v_out;              // [N, NKV * D] or null
  void* k_cache;            // [num_pages, NKV, page_size, D] or null
  void* v_cache;
  int64_t num_tokens;
  int num_heads, num_kv_heads, head_dim, rotary_dim, page_size;
  int64_t num_pages;
  float eps;
  int dtype;
  int* status;
};
int launch_qk_norm_rope_write(const QkRopeWriteParams& p, cudaStream_t stream);

// Copy k, v [N, NKV * D] into their cache slots.
int launch_kv_write(const void* k, const void* v, const int32_t* slots, void* k_cache, void* v_cache,
                    int64_t num_tokens, int num_kv_heads, int head_dim, int page_size, int64_t num_pages,
                    int dtype, int* status, cudaStream_t stream);

struct PagedAttentionParams {
  const void* q;               // [N, NH * D]
  const void* k_cache;         // [num_pages, NKV, page_size, D]
  const void* v_cache;
  void* out;                   // [N, NH * D]
  const int32_t* block_table;  // [S, table_width]
  const int32_t* cu_q;         // [S + 1] first batch row of each sequence
  const int32_t* ctx_lens;     // [S] keys of each sequence once this step's tokens are in
  const int32_t* tile_seq;     // [tiles] sequence of each query tile
  const int32_t* tile_q0;      // [tiles] first batch row of the tile
  const int32_t* tile_nq;      // [tiles] rows in the tile (<= q_tile)
  float* partials;             // [N * NH, num_splits, D + 2] when num_splits > 1
  int64_t num_tokens;
  int num_tiles, q_tile, num_splits;
  int num_seqs, table_width;
  int num_heads, num_kv_heads, head_dim, page_size;
  int64_t num_pages;
  int window;                  // 0 = all keys
  int kernel;                  // 0 = best kernel that takes the sizes, 1 = the general kernel, 2 = no tcgen05 prompt
                               // kernel, 3 / 4 = the tcgen05 prompt kernel's narrow / wide form whatever the grid
  float scale;
  int dtype;
  int* status;
};
int launch_paged_attention(const PagedAttentionParams& p, cudaStream_t stream);
// The tensor-core kernels (attention_tc.cu): whether they take the problem, and their launch (without the merge).
bool attention_tc_supported(const PagedAttentionParams& p);
int launch_attention_tc(const PagedAttentionParams& p, cudaStream_t stream);
bool attention_tc_merges_in_kernel(const PagedAttentionParams& p);
// The tcgen05 prompt kernel (attention_tcgen05.cu): bfloat16, head size 128, groups of 2, 4 or 8 q-heads.
bool attention_tcgen05_supported(const PagedAttentionParams& p);
int launch_attention_tcgen05(const PagedAttentionParams& p, cudaStream_t stream);

// Attention whose scores are reshaped before the softmax and whose keys and values may differ in width
// (scored_attention.cu).  `base` is read as for launch_paged_attention with these differences: head_dim is the width
// of a query / key row, out is [N, NH * v_dim], partials hold v_dim + 2 floats per (row, split), `kernel` is ignored.
struct ScoredAttentionParams {
  PagedAttentionParams base;
  int v_dim;                   // width of a value row and of a head's output
  int64_t k_row_stride;        // elements between consecutive (page, kv head, offset) rows of the key storage
  int64_t v_row_stride;        // the same for the value storage (which may be the key storage: a value that is a
                               // prefix of its key row)
  float softcap;               // > 0: score <- softcap * tanh(score / softcap)
  const float* slopes;         // [NH] or null: score <- score - slopes[h] * (query position - key position)
  int chunk;                   // > 0: a query sees only the keys of its own block of `chunk` positions
  const float* gate;           // [N, NH] or null: a head's output is multiplied by its gate
  int keep_first;              // > 0 (with a window): the keys at positions below it stay visible behind the window
  int sigmoid_weights;         // 1: a visible key weighs sigmoid(score + head_bias[h]); the weights are not normalised
  const float* head_bias;      // [NH] or null (read with sigmoid_weights)
  float out_scale;             // every output is multiplied by it (1: nothing)
};
int launch_scored_attention(const ScoredAttentionParams& p, cudaStream_t stream);
// The tcgen05 prompt kernel's scored form (attention_tcgen05.cu): bfloat16 prompt tiles with keys and values of 128
// dims, whatever modifiers; `base.kernel` == 1 keeps the general kernel.
// The mma.sync decode kernel's scored form (attention_tc.cu): single-token tiles with keys and values of the same 64
// or 128 dims, 1, 2, 4 or 8 key splits.
bool attention_tc_scored_supported(const ScoredAttentionParams& p);
int launch_attention_tc_scored(const ScoredAttentionParams& p, cudaStream_t stream);
// The mma.sync kernel for rows that are key and value at once (scored_attention_mma.cu): bfloat16, k_cache == v_cache,
// key width a multiple of 16 up to 576, value width 64, 128, 256 or 512; any tiles and splits (without the merge).
bool scored_attention_mma_supported(const ScoredAttentionParams& p);
int launch_scored_attention_mma(const ScoredAttentionParams& p, cudaStream_t stream);
bool attention_tcgen05_scored_supported(const ScoredAttentionParams& p);
int launch_attention_tcgen05_scored(const ScoredAttentionParams& p, cudaStream_t stream);

// What stands between one product that holds [q heads | k heads | v heads | a gate column per q head] of every token
// and the attention over them (mixer_prep.cu): q and k heads scaled to unit RMS, v blended with another layer's
// values of the same token, k and v written to their cache slots, gates through a sigmoid.
struct HeadPrepParams {
  const void* x;               // [N, NH * D + NKV * D + NKV * DV (+ NH)]
  const int32_t* slots;        // [N] page * page_size + offset, or -1: not written; may be null
  void* q_out;                 // [N, NH * D]
  void* k_cache;               // [num_pages, NKV, page_size, k_row_stride] or null
  void* v_cache;               // [num_pages, NKV, page_size, v_row_stride] or null
  void* v_keep;                // [N, NKV * DV] or null: receives this layer's own values before the blend
  const void* v_other;         // [N, NKV * DV] or null: v <- (1 - w) v + w v_other
  const float* blend_weight;   // one float on the device (read when v_other is given)
  float* gate_out;             // [N, NH] or null: sigmoid of the gate columns (null: x has no gate columns)
  int64_t num_tokens;
  int num_heads, num_kv_heads, head_dim, v_dim, page_size;
  int64_t num_pages, k_row_stride, v_row_stride;
  int unit_norm;               // 1: q and k heads are divided by sqrt(mean(x^2) + eps)
  float eps;
  int dtype;
  int* status;
  const float* q_weight;       // [D] or null: q heads are multiplied by it after the norm
  const float* k_weight;       // [D] or null: likewise for k heads
  int no_kv;                   // 1: x holds no k and v columns (the mixer reads another position's pages)
};
int launch_head_prep(const HeadPrepParams& p, cudaStream_t stream);

// What stands between one product that holds [query latent | key/value latent | rotated key part] of every token and
// what comes next: RMS norm with a plain weight on each latent, rotary positions on neighbouring pairs of the first
// rotary_dims dims of the rotated part; the normed key/value latent and the rotated part go side by side into the
// token's cache row [kv_rank + rot_dim].
struct LatentPrepParams {
  const void* x;               // [N, q_rank + kv_rank + rot_dim]
  const int32_t* positions;    // [N]
  const int32_t* slots;        // [N] or null
  const float* q_weight;       // [q_rank]
  const float* kv_weight;      // [kv_rank]
  const float* inv_freq;       // [rotary_dims / 2]
  void* q_latent;              // [N, q_rank]
  void* cache;                 // [num_pages, 1, page_size, row_stride] or null
  int64_t num_tokens;
  int q_rank, kv_rank, rot_dim, rotary_dims, page_size;
  int64_t num_pages, row_stride;
  float eps;
  int dtype;
  int* status;
};
int launch_latent_prep(const LatentPrepParams& p, cudaStream_t stream);

// out[t, h, out_offset + c] = rotated in[t, h, in_offset + c] for c < cols: dims 2i and 2i + 1 turn by
// positions[t] * inv_freq[i] while 2i + 1 < rotary_dims, the rest passes unchanged.
int launch_rotate_pairs(const void* in, void* out, const int32_t* positions, const float* inv_freq,
                        int64_t num_tokens, int heads, int cols, int rotary_dims, int64_t in_width, int in_offset,
                        int64_t out_width, int out_offset, int dtype, cudaStream_t stream);

// The gated delta rule (delta_rule.cu).  x [N, q | k | v | gate | beta | step] with num_kv_heads heads of head_dim
// for q and k, num_heads heads of v_dim for v and gate, one column per head for beta and step.  state
// [num_slots, state_stride] float32: per slot heads * v_dim * head_dim floats of S ([head][value column][dim]) at
// offset 0 (in the scan kernel's own order, delta_memory_floats() of them) and (taps - 1) * channels convolution
// inputs at offset `memory`.
constexpr int kDeltaMaxDim = 256;
constexpr int kDeltaMaxTaps = 16;
struct DeltaParams {
  const void* x;
  const float* conv;           // [channels, taps], channels = 2 * num_kv_heads * head_dim + num_heads * v_dim
  const float* rate_log;       // [num_heads]
  const float* step_bias;      // [num_heads]
  const float* norm_weight;    // [v_dim]
  float* state;
  const int32_t* cu_q;         // [num_seqs + 1]
  const int32_t* state_slots;  // [num_seqs]; negative: the sequence is padding
  float* qkv;                  // [N, channels]: unit q, unit k, v
  float* coef;                 // [N, 2 * num_heads]: beta, decay
  float* scratch;              // [N, num_heads * v_dim]: o before its norm
  void* out;                   // [N, num_heads * v_dim]
  int64_t num_tokens, state_stride, memory;
  int num_seqs, num_slots, num_heads, num_kv_heads, head_dim, v_dim, taps;
  float unit_eps, norm_eps;
  int dtype;
};
int launch_delta_prep(const DeltaParams& p, cudaStream_t stream);
int launch_delta_scan(const DeltaParams& p, cudaStream_t stream);
bool delta_scan_supported(int dim, int v_dim);
int64_t delta_memory_floats(int num_heads, int dim, int v_dim);

// Routed experts (routed_experts.cu).
constexpr int kMoeMaxExperts = 512;
struct MoeRouteParams {
  const float* logits;         // [N, experts]
  const float* correction;     // [experts] or null: added to the scores for the choice only
  int32_t* chosen;             // [N, top]
  float* weights;              // [N, top]
  int64_t num_tokens;
  int experts, top, groups, keep_groups, group_top;
  float scale, weight_eps;
  int score_kind;              // 0: sigmoid of each logit; 1: softmax over all experts
};
int launch_moe_route(const MoeRouteParams& p, cudaStream_t stream);
// logits[t, e] = x[t, :] . w[e, :] in float, a warp per (token, expert): for steps of a few tokens.
int launch_moe_router(const void* x, const void* w, float* logits, int64_t tokens, int experts, int k, int dtype,
                      cudaStream_t stream);
// order [pairs]: the (token, choice) pairs (token * top + choice) sorted by expert; offsets [experts + 1].
int launch_moe_sort(const int32_t* chosen, int32_t* order, int32_t* offsets, int64_t pairs, int experts,
                    cudaStream_t stream);
struct MoeGemmParams {
  const void* a;               // gated: x [tokens, k]; else the activations [pairs, k] in sorted order
  const void* w;               // gated: [experts, 2 n, k] (gate rows, then up rows); else [experts, n, k]
  const int32_t* order;        // [pairs]
  const int32_t* offsets;      // [experts + 1]
  const float* weights;        // [pairs] by pair (not gated)
  void* out;                   // gated: [pairs, n] in sorted order, type of a; else float32 [pairs, n] by pair
  int64_t pairs;
  int experts, k, n, top;
  float limit, slope;
  float up_offset;             // the gated product's activation is g sigmoid(slope g) (u + up_offset)
  int dtype;
  int force_plain;             // 0: the form is chosen by size; 1: float arithmetic; 2: mma.sync tiles; 3: few rows
};
// steps with at most this many (token, choice) pairs run the few-rows form of the gated product (measured at 8
// tokens, 64 experts of 1,024 x 4,096: 103 against 111 us; the down product is faster in tiles: 59 against 89 us)
constexpr int kMoeFewRowPairs = 128;
int launch_moe_gemm(const MoeGemmParams& p, bool gated, cudaStream_t stream);
// out[t] = sum over c < top of parts[t * top + c] (+ shared[t]), float32.
int launch_moe_combine(const float* parts, const void* shared, int shared_dtype, float* out, int64_t num_tokens,
                       int64_t width, int top, cudaStream_t stream);

enum Activation : int { kActReluSquared = 0, kActGeluTanh = 1, kActSilu = 2 };
int launch_activation(const void* in, void* out, int64_t total, int kind, int dtype, cudaStream_t stream);

// tokens[r] = argmax(logits[r]) where temperature[r] == 0, else the inverse-CDF draw of
// softmax(logits[r] / temperature[r]) at uniform[r].
// A row is cut into kSampleSlices slices, a block each.  Workspaces: part_max / part_arg / part_sum hold
// num_rows * kSampleSlices entries (written before they are read); tickets holds num_rows counters that must be zero
// when the kernel starts and are zero again when it ends.
constexpr int kSampleSlices = 8;
int launch_sample(const float* logits, const float* temperature, const float* uniform, int32_t* tokens,
                  int64_t num_rows, int64_t vocab, float* part_max, int* part_arg, double* part_sum, int* tickets,
                  cudaStream_t stream);

// Linear attention with a decaying matrix memory per head (linear_memory.cu): S_t = diag(a_t) S_(t-1) + k_t v_t^T,
// o_t = S_t^T q_t, float32, from and into the requests' state slots.  x [N, x_stride] is one product's output whose
// columns hold q (num_heads * head_dim from q_off), the gate or key columns (the same count from k_off) and v
// (num_heads * v_dim from v_off).
enum LinearScanMode : int {
  kGatedWrite = 0,      // a = f, k = 1 - f, f = lower + (1 - lower) sigmoid(x_k + gate_bias); q = silu(x_q); v = x_v
  kConstantDecay = 1,   // a = decay[head]; k = silu(x_k); q = silu(x_q); v = silu(x_v)
  kPlainDecay = 2,      // a = decay[head]; q, k, v as they stand in x, which is float32 (prepared by another kernel)
  kTokenDecay = 3,      // a = x[decay_off + head] of the token; q, k, v as they stand in x (float32); qk_group heads
                        // in a row share a q and a k
};
constexpr int kLinearScanMaxDim = 256;
struct LinearScanParams {
  const void* x;
  int64_t x_stride;
  int q_off, k_off, v_off;
  const float* gate_bias;      // [NH * D] or null
  const float* lower;          // [NH * D] (kGatedWrite)
  const float* decay;          // [NH] (kConstantDecay)
  float* state;                // [slots, state_stride]; a slot's first linear_scan_state_floats() floats are S
  float* act;                  // [N, 2 * NH * D + NH * DV] float32 scratch for steps that hold prompts, or null:
                               // q, a-or-k and v after their activations and gates, written by a kernel of its own
  int64_t state_stride;
  const int32_t* cu_q;         // [num_seqs + 1]
  const int32_t* state_slots;  // [num_seqs], negative: a padded sequence, left alone
  float* out;                  // [N, NH * DV] float32
  int64_t num_tokens;
  int num_seqs, num_heads, head_dim, v_dim, mode, dtype;
  int qk_group;                // heads that share one q and one k (0 or 1: every head its own)
  int decay_off;               // kTokenDecay: column of x where the token's decays (a float per head) begin
  // filled in by the launcher: where the prompt form's staging warps find q, k and v in `act`
  int64_t act_stride;
  int act_q_off, act_k_off, act_v_off, act_aligned;
};
bool linear_scan_shape(int head_dim, int v_dim, int* rows, int* lanes);
int64_t linear_scan_state_floats(int num_heads, int head_dim, int v_dim);
int launch_linear_scan(const LinearScanParams& p, cudaStream_t stream);
// v = in (+ skip_coef[c / skip_head] * skip[t, skip_off + c]) (* gate, if gate_first);
// out[t, c] = v / sqrt(mean over c's group of `group` columns of v^2 + eps) * weight[c % weight_len] * factor
// (* gate unless gate_first), gate = sigmoid or SiLU of x[t, gate_off + c] when x is given; in float32 [N, width],
// out in `dtype`, x in `dtype`, skip float32.
struct GroupNormGateParams {
  const float* in;
  void* out;
  const float* weight;         // [weight_len] or null: no weight
  int weight_len;
  int64_t num_tokens;
  int width, group;
  float eps, factor;
  const void* x;               // gate columns, or null
  int64_t x_stride;
  int gate_off;
  int gate_kind;               // 0: sigmoid, 1: SiLU
  int gate_first;              // 1: the gate multiplies before the norm
  const float* skip;           // [N, skip_stride] or null
  int64_t skip_stride;
  int skip_off;
  const float* skip_coef;      // a coefficient per run of skip_head columns
  int skip_head;
  int dtype;
};
int launch_group_norm_gate(const GroupNormGateParams& p, cudaStream_t stream);

// Rotary positions on the q and k heads of one product, the value's preparation and the cache write (rotary_prep.cu).
struct RotaryPrepParams {
  const void* x;               // [N, x_stride]: NH * D of q, NKV * D of k, then NKV * DV of v unless value_from_key
  int64_t x_stride;
  const int32_t* positions;    // [N]
  const int32_t* slots;        // [N] page * page_size + offset, negative: not stored; may be null
  const float* freq;           // [rotary_dims / 2]
  void* q_out;                 // [N, NH * D]
  void* k_cache;               // [num_pages, NKV, page_size, k_row_stride] or null
  void* v_cache;
  int64_t num_tokens, num_pages, k_row_stride, v_row_stride;
  int num_heads, num_kv_heads, head_dim, v_dim, page_size;
  int rotary_dims;             // the first so many dims of a head are turned
  int layout;                  // 0: dim i pairs with i + rotary_dims / 2; 1: dim 2i with 2i + 1
  float factor;                // on cos and sin
  int value_from_key;          // 1: the value is the key head before the turn
  int value_norm;              // 1: the value head is divided by sqrt(mean(v^2) + eps)
  float eps;
  const float* q_norm;         // [NH * D] or null: q is divided by the root mean square of ALL its heads' entries (plus
  const float* k_norm;         // row_norm_eps) and multiplied by this weight before the turn; [NKV * D] likewise for k
  float row_norm_eps;
  int dtype;
  int* status;
};
int launch_rotary_prep(const RotaryPrepParams& p, cudaStream_t stream);

// The q, k and v heads of one product as float32 rows [q | k | v] for a scan: the first rotary_dims dims of every q and
// k head turned in the half layout (dim i with i + rotary_dims / 2), q times q_scale and k times k_scale afterwards.
struct RotaryRowsParams {
  const void* x;               // [N, x_stride], q from q_off (NH * D), k from k_off (NH * D), v from v_off (NH * DV)
  int64_t x_stride;
  int q_off, k_off, v_off;
  const int32_t* positions;    // [N]
  const float* freq;           // [rotary_dims / 2]
  float* out;                  // [N, out_stride]: q at 0, k at NH * D, v at 2 * NH * D
  int64_t out_stride;
  int64_t num_tokens;
  int num_heads, head_dim, v_dim, rotary_dims;
  float q_scale, k_scale;
  int dtype;
};
int launch_rotary_rows(const RotaryRowsParams& p, cudaStream_t stream);

// Hyper-connections: a residual stream in `streams` copies per token (hyper_streams.cu).
constexpr int kHyperMaxStreams = 8;
struct HyperStepParams {
  float* x;                    // [N, streams, width] float32
  const void* y;               // [N, width] the sublayer's result to write back, or null
  int y_dtype;
  const float* mix;            // [streams, streams], from x to
  const float* write;          // [streams]
  const float* scale;          // [width] on y, or null
  const float* read;           // [streams]: the next sublayer's mixture, with out
  const float* weight;         // [width]: the norm's factor
  float eps;
  void* out;                   // [N or num_rows, width] the normed mixture in `dtype`, or null
  const int32_t* rows;         // gather for out (then y must be null), or null
  int64_t num_rows;
  int64_t num_tokens;
  int streams, width, dtype;
  int* status;
};
int launch_hyper_step(const HyperStepParams& p, cudaStream_t stream);
int launch_hyper_collapse(const HyperStepParams& p, float* sum, cudaStream_t stream);
int launch_hyper_expand(const float* in, float* x, int64_t num_tokens, int streams, int width, cudaStream_t stream);
int launch_normed_pair_sum(const float* a, const float* b, const float* wa, const float* wb, void* out,
                           int64_t num_tokens, int width, float eps, float sa, float sb, int dtype, cudaStream_t stream);

// A selective state-space mixer's preparation (state_space.cu).
constexpr int kSsmMaxHeads = 1024;
constexpr int kConvMaxTaps = 16;
struct SsmPrepParams {
  const void* x;               // [N, x_stride]: the convolved channels [x (H * P) | B (G * N) | C (G * N)] from conv_off,
  int64_t x_stride;            // the step columns (H) from step_off
  int conv_off, step_off;
  const float* conv;           // [channels, taps]
  const float* conv_bias;      // [channels] or null
  const float* step_bias;      // [H]
  const float* rate_log;       // [H]
  const float* state;          // [slots, state_stride]; the convolutions' last taps - 1 inputs from tail_off
  int64_t state_stride, tail_off;
  const int32_t* cu_q;
  const int32_t* state_slots;
  float* out;                  // [N, out_stride]: [C | B | dt x | decay | x]
  int64_t out_stride;
  int64_t num_tokens;
  int num_seqs, num_slots, num_heads, v_dim, state_dim, groups, taps, dtype;
};
int launch_ssm_prep(const SsmPrepParams& p, cudaStream_t stream);
struct ConvTailParams {
  const void* x;
  int64_t x_stride;
  int conv_off, channels, taps;
  float* state;
  int64_t state_stride, tail_off;
  const int32_t* cu_q;
  const int32_t* state_slots;
  int num_seqs, num_slots, dtype;
};
int launch_conv_tail(const ConvTailParams& p, cudaStream_t stream);

// hidden[t] += table[(previous token * mul_prev + token * mul_cur) mod buckets] (row `buckets` at position 0); the
// token before a step's first row comes from, and the step's last token goes to, last_token[slot * state_stride]
// (stream_ops.cu).
struct PairRowsParams {
  const int32_t* ids;          // [N]; -(r + 1) stands for sampled[r]
  const int32_t* sampled;
  int64_t num_sampled;
  const int32_t* positions;    // [N]
  const int32_t* cu_q;         // [num_seqs + 1]
  const int32_t* state_slots;  // [num_seqs]
  int32_t* last_token;
  int64_t state_stride;        // int32 elements between two slots
  const void* table;           // [buckets + 1, hidden]
  float* hidden;               // [N, hidden]
  int64_t num_tokens, hidden_size, vocab, buckets, mul_prev, mul_cur;
  int num_seqs, dtype;
};
int launch_pair_rows_add(const PairRowsParams& p, cudaStream_t stream);
int launch_stream_add(float* hidden, const float* other, int64_t n, cudaStream_t stream);
int launch_scaled_sum(const void* a, const void* b, void* out, float sa, float sb, int64_t n, int dtype,
                      cudaStream_t stream);

}  // namespace akv
