// What stands between one product that holds [q heads | k heads (| v heads)] of every token (biases already added)
// and attention over pages, for mixers whose queries and keys are turned by the token's position:
//
//   q, k  <- the first rotary_dims dims of every head turned: the pair (u, v) becomes
//            (u c - v s, v c + u s) with c = cos(position * freq[i]) * factor, s = sin(position * freq[i]) * factor;
//            pair i is dims (i, i + rotary_dims / 2) (layout 0) or dims (2i, 2i + 1) (layout 1)
//   v     <- the key head as it was before the turn (value_from_key; the product has no v columns), or the v head,
//            optionally divided by sqrt(mean(v^2) + eps) (value_norm)
//   q goes to q_out, k and v to the token's cache slot.
//   Optionally, before the turn, q and k are RMS-normed over ALL their heads' entries at once (one root mean square
//   for the q row, one for the k row) with a learned weight per entry.
// A second kernel (rotary_rows) writes the turned q and k and the plain v of a product as float32 rows [q | k | v],
// each of q and k times a constant: the input of a linear-attention scan that keeps everything in float32.
//
// Positions, angles, cos and sin are float32; freq comes from the host (it carries whatever rescaling of the
// frequencies the encoding has).  A warp per (token, q head) and per (token, kv head): the latter writes the key and
// its value.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

constexpr int kPrepWarps = 4;
constexpr int kRowWarps = 4;     // of the form with norms over whole rows: a block per token, or a cluster of them

// One head: src (T) -> dst (U), the first `rot` dims turned; every entry first times inv * w[d] when w is given (a
// norm over the whole row of heads, whose root mean square the caller worked out), and times `scale` at the end.
template <typename T, typename U>
__device__ __forceinline__ void turn_head(const T* __restrict__ src, U* __restrict__ dst, int D, int rot, int layout,
                                          float position, const float* __restrict__ freq, float factor, int lane,
                                          const float* __restrict__ w = nullptr, float inv = 1.f, float scale = 1.f) {
  const int half = rot / 2;
  for (int i = lane; i < half; i += 32) {
    const int a = layout == 0 ? i : 2 * i, b = layout == 0 ? i + half : 2 * i + 1;
    float s, c;
    sincosf(position * freq[i], &s, &c);
    s *= factor;
    c *= factor;
    float u = to_float<T>(src[a]), v = to_float<T>(src[b]);
    if (w != nullptr) {
      u *= inv * w[a];
      v *= inv * w[b];
    }
    dst[a] = from_float<U>((u * c - v * s) * scale);
    dst[b] = from_float<U>((v * c + u * s) * scale);
  }
  for (int d = rot + lane; d < D; d += 32) {
    float u = to_float<T>(src[d]);
    if (w != nullptr) u *= inv * w[d];
    dst[d] = from_float<U>(u * scale);
  }
}

// what a warp does for head h of a token: a q head goes to q_out, a k head with its value to the token's cache slot
template <typename T>
__device__ __forceinline__ void prep_head(const RotaryPrepParams& p, int64_t token, int h, int lane, float inv_q,
                                          float inv_k) {
  const int NH = p.num_heads, NKV = p.num_kv_heads, D = p.head_dim, DV = p.v_dim;
  const T* row = (const T*)p.x + token * p.x_stride;
  const float position = (float)p.positions[token];
  if (h < NH) {
    turn_head<T, T>(row + (int64_t)h * D, (T*)p.q_out + (token * NH + h) * (int64_t)D, D, p.rotary_dims, p.layout,
                    position, p.freq, p.factor, lane, p.q_norm != nullptr ? p.q_norm + (int64_t)h * D : nullptr, inv_q);
    return;
  }
  const int g = h - NH;
  if (p.k_cache == nullptr) return;
  const int64_t slot = p.slots != nullptr ? p.slots[token] : -1;
  if (slot < 0) return;                                 // a padded token: nothing to store
  const int64_t page = slot / p.page_size;
  if (page >= p.num_pages) {
    if (lane == 0) set_status(p.status, kBadSlot);
    return;
  }
  const int64_t at = (page * NKV + g) * p.page_size + slot % p.page_size;
  const T* ksrc = row + (int64_t)NH * D + (int64_t)g * D;
  turn_head<T, T>(ksrc, (T*)p.k_cache + at * p.k_row_stride, D, p.rotary_dims, p.layout, position, p.freq, p.factor,
                  lane, p.k_norm != nullptr ? p.k_norm + (int64_t)g * D : nullptr, inv_k);
  T* vdst = (T*)p.v_cache + at * p.v_row_stride;
  if (p.value_from_key) {
    for (int d = lane; d < DV; d += 32) vdst[d] = ksrc[d];
    return;
  }
  const T* vsrc = row + (int64_t)(NH + NKV) * D + (int64_t)g * DV;
  float inv = 1.f;
  if (p.value_norm) {
    float ss = 0.f;
    for (int d = lane; d < DV; d += 32) {
      const float v = to_float<T>(vsrc[d]);
      ss += v * v;
    }
    inv = 1.f / sqrtf(warp_sum(ss) / (float)DV + p.eps);
  }
  for (int d = lane; d < DV; d += 32) vdst[d] = from_float<T>(to_float<T>(vsrc[d]) * inv);
}

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32) rotary_prep_kernel(RotaryPrepParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int units = p.num_heads + p.num_kv_heads;
  const int64_t item = (int64_t)blockIdx.x * kPrepWarps + (threadIdx.x >> 5);
  if (item >= p.num_tokens * units) return;
  prep_head<T>(p, item / units, (int)(item % units), lane, 1.f, 1.f);
}

// The form with norms over the whole q row and the whole k row: a block per token adds up both rows' squares once,
// then its warps take the heads in turn.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32) rotary_prep_rows_kernel(RotaryPrepParams p) {
  __shared__ float scratch[34];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t token = blockIdx.x;
  const int qw = p.num_heads * p.head_dim, kw = p.num_kv_heads * p.head_dim;
  const T* row = (const T*)p.x + token * p.x_stride;
  // the blocks of a token (grid y, one cluster) take every gridDim.y-th run of the row for the sums, then every
  // gridDim.y-th group of heads
  const int first = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
  float sq = 0.f, sk = 0.f;
  for (int c = first; c < qw; c += stride) {
    const float v = to_float<T>(row[c]);
    sq = fmaf(v, v, sq);
  }
  for (int c = first; c < kw; c += stride) {
    const float v = to_float<T>(row[qw + c]);
    sk = fmaf(v, v, sk);
  }
  sq = cluster_sum(sq, scratch);
  sk = cluster_sum(sk, scratch);
  const float inv_q = 1.f / sqrtf(sq / (float)qw + p.row_norm_eps), inv_k = 1.f / sqrtf(sk / (float)kw + p.row_norm_eps);
  for (int h = blockIdx.y * kRowWarps + (threadIdx.x >> 5); h < p.num_heads + p.num_kv_heads; h += gridDim.y * kRowWarps)
    prep_head<T>(p, token, h, lane, inv_q, inv_k);
}

// [q | k | v] of a token as float32 for a scan: a warp per (token, head) turns the head's q and k and copies its v
template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32) rotary_rows_kernel(RotaryRowsParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int NH = p.num_heads, D = p.head_dim, DV = p.v_dim;
  const int64_t item = (int64_t)blockIdx.x * kPrepWarps + (threadIdx.x >> 5);
  if (item >= p.num_tokens * NH) return;
  const int64_t token = item / NH;
  const int h = (int)(item % NH);
  const T* row = (const T*)p.x + token * p.x_stride;
  float* out = p.out + token * p.out_stride;
  const float position = (float)p.positions[token];
  turn_head<T, float>(row + p.q_off + (int64_t)h * D, out + (int64_t)h * D, D, p.rotary_dims, 0, position, p.freq, 1.f,
                      lane, nullptr, 1.f, p.q_scale);
  turn_head<T, float>(row + p.k_off + (int64_t)h * D, out + (int64_t)(NH + h) * D, D, p.rotary_dims, 0, position, p.freq,
                      1.f, lane, nullptr, 1.f, p.k_scale);
  const T* vsrc = row + p.v_off + (int64_t)h * DV;
  float* vdst = out + 2 * (int64_t)NH * D + (int64_t)h * DV;
  for (int d = lane; d < DV; d += 32) vdst[d] = to_float<T>(vsrc[d]);
}

}  // namespace

int launch_rotary_prep(const RotaryPrepParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.rotary_dims < 0 || p.rotary_dims % 2 || p.rotary_dims > p.head_dim || (p.layout != 0 && p.layout != 1) ||
      (p.value_from_key && p.v_dim != p.head_dim))
    return (int)cudaErrorInvalidValue;
  if ((p.q_norm == nullptr) != (p.k_norm == nullptr)) return (int)cudaErrorInvalidValue;
  if (p.q_norm != nullptr) {
    if (p.num_tokens > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    // few tokens: up to eight blocks (a cluster) share a token's heads
    int parts = 1;
    while (parts < 8 && p.num_tokens * parts < 128 && (p.num_heads + p.num_kv_heads) >= 2 * parts * kRowWarps) parts *= 2;
    const dim3 grid((unsigned)p.num_tokens, (unsigned)parts), cluster(1, parts, 1);
    if (p.dtype == kBFloat16)
      return (int)launch_chain(rotary_prep_rows_kernel<__nv_bfloat16>, grid, dim3(kRowWarps * 32), 0, stream, cluster, p);
    return (int)launch_chain(rotary_prep_rows_kernel<float>, grid, dim3(kRowWarps * 32), 0, stream, cluster, p);
  }
  const int64_t items = p.num_tokens * (p.num_heads + p.num_kv_heads);
  const int64_t blocks = (items + kPrepWarps - 1) / kPrepWarps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(rotary_prep_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(rotary_prep_kernel<float>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), 0, stream,
                           dim3(1, 1, 1), p);
}

int launch_rotary_rows(const RotaryRowsParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.rotary_dims < 0 || p.rotary_dims % 2 || p.rotary_dims > p.head_dim || p.num_heads < 1)
    return (int)cudaErrorInvalidValue;
  const int64_t blocks = (p.num_tokens * p.num_heads + kPrepWarps - 1) / kPrepWarps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(rotary_rows_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(rotary_rows_kernel<float>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), 0, stream,
                           dim3(1, 1, 1), p);
}

}  // namespace akv
