// What stands between one product that holds [q heads | k heads (| v heads)] of every token (biases already added)
// and attention over pages, for mixers whose queries and keys are turned by the token's position:
//
//   q, k  <- the first rotary_dims dims of every head turned: the pair (u, v) becomes
//            (u c - v s, v c + u s) with c = cos(position * freq[i]) * factor, s = sin(position * freq[i]) * factor;
//            pair i is dims (i, i + rotary_dims / 2) (layout 0) or dims (2i, 2i + 1) (layout 1)
//   v     <- the key head as it was before the turn (value_from_key; the product has no v columns), or the v head,
//            optionally divided by sqrt(mean(v^2) + eps) (value_norm)
//   q goes to q_out, k and v to the token's cache slot.
//
// Positions, angles, cos and sin are float32; freq comes from the host (it carries whatever rescaling of the
// frequencies the encoding has).  A warp per (token, q head) and per (token, kv head): the latter writes the key and
// its value.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

constexpr int kPrepWarps = 4;

template <typename T>
__device__ __forceinline__ void turn_head(const T* __restrict__ src, T* __restrict__ dst, int D, int rot, int layout,
                                          float position, const float* __restrict__ freq, float factor, int lane) {
  const int half = rot / 2;
  for (int i = lane; i < half; i += 32) {
    const int a = layout == 0 ? i : 2 * i, b = layout == 0 ? i + half : 2 * i + 1;
    float s, c;
    sincosf(position * freq[i], &s, &c);
    s *= factor;
    c *= factor;
    const float u = to_float<T>(src[a]), v = to_float<T>(src[b]);
    dst[a] = from_float<T>(u * c - v * s);
    dst[b] = from_float<T>(v * c + u * s);
  }
  for (int d = rot + lane; d < D; d += 32) dst[d] = src[d];
}

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32) rotary_prep_kernel(RotaryPrepParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int NH = p.num_heads, NKV = p.num_kv_heads, D = p.head_dim, DV = p.v_dim;
  const int64_t item = (int64_t)blockIdx.x * kPrepWarps + (threadIdx.x >> 5);
  if (item >= p.num_tokens * (NH + NKV)) return;
  const int64_t token = item / (NH + NKV);
  const int h = (int)(item % (NH + NKV));
  const T* row = (const T*)p.x + token * p.x_stride;
  const float position = (float)p.positions[token];
  if (h < NH) {
    turn_head<T>(row + (int64_t)h * D, (T*)p.q_out + (token * NH + h) * (int64_t)D, D, p.rotary_dims, p.layout, position,
                 p.freq, p.factor, lane);
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
  turn_head<T>(ksrc, (T*)p.k_cache + at * p.k_row_stride, D, p.rotary_dims, p.layout, position, p.freq, p.factor, lane);
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

}  // namespace

int launch_rotary_prep(const RotaryPrepParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.rotary_dims < 0 || p.rotary_dims % 2 || p.rotary_dims > p.head_dim || (p.layout != 0 && p.layout != 1) ||
      (p.value_from_key && p.v_dim != p.head_dim))
    return (int)cudaErrorInvalidValue;
  const int64_t items = p.num_tokens * (p.num_heads + p.num_kv_heads);
  const int64_t blocks = (items + kPrepWarps - 1) / kPrepWarps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(rotary_prep_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(rotary_prep_kernel<float>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), 0, stream,
                           dim3(1, 1, 1), p);
}

}  // namespace akv
