// What stands between the input product of a selective state-space mixer (Mamba-2) and the scan over its memory.
//
// The product holds, per token, [gate z (H * P) | convolved channels: x (H * P), B (G * N), C (G * N) | step (H)].
//
//   ssm_prep:   the channels pass a short causal convolution over the sequence's own earlier tokens (weights
//               [channels, taps], last tap the current token's, a bias per channel; the inputs before the step's first
//               token come from the request's state slot, which holds zeros at a sequence's start) and SiLU;
//               dt = softplus(step + step_bias), decay = exp(-exp(rate_log) * dt).  It writes one float32 row per token
//               in the order the linear scan reads: [C (G * N) | B (G * N) | dt * x (H * P) | decay (H) | x (H * P)],
//               so that with q = C, k = B, v = dt x the recurrence S <- decay S + k v^T, o = S^T q is the scan's
//               per-token-decay mode with H / G heads sharing a q and k.
//   conv_tail:  moves each sequence's last taps - 1 inputs of the convolved channels into the state slot; a thread per
//               (sequence, channel) reads all it needs before it writes.
//
// Everything after the product is float32.  A sequence whose state slot is negative (padding of a captured step) is
// left alone and its rows are zero.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ int sequence_of(const int32_t* cu_q, int num_seqs, int64_t token) {
  int lo = 0, hi = num_seqs;          // invariant: cu_q[lo] <= token < cu_q[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_q[mid] <= token) lo = mid; else hi = mid;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(256) ssm_prep_kernel(SsmPrepParams p) {
  __shared__ float dt_s[kSsmMaxHeads];
  pdl_launch_dependents();
  pdl_wait();
  const int H = p.num_heads, P = p.v_dim, N = p.state_dim, G = p.groups, taps = p.taps;
  const int inner = H * P, gn = G * N, channels = inner + 2 * gn;
  const int64_t token = blockIdx.x;
  const T* x = (const T*)p.x;
  float* out = p.out + token * p.out_stride;
  const int s = sequence_of(p.cu_q, p.num_seqs, token);
  const int slot = p.state_slots[s];
  const int width = 2 * gn + 2 * inner + H;
  if (slot < 0 || slot >= p.num_slots) {
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) out[c] = 0.f;
    return;
  }
  // the blocks of a token (grid y) take every gridDim.y-th run of the channels; each works out the steps it needs
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = softplus_f(to_float<T>(x[token * p.x_stride + p.step_off + h]) + p.step_bias[h]);
    dt_s[h] = dt;
    if (blockIdx.y == 0) out[2 * gn + inner + h] = expf(-expf(p.rate_log[h]) * dt);
  }
  __syncthreads();
  const int64_t seq_first = p.cu_q[s];
  const int offset = (int)(token - seq_first);               // tokens of this sequence before this one in the step
  const float* before = p.state + (int64_t)slot * p.state_stride + p.tail_off;      // [taps - 1, channels]
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float* w = p.conv + (int64_t)c * taps;
    float y = p.conv_bias != nullptr ? p.conv_bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = offset - (taps - 1) + j;              // index within the step's tokens of this sequence
      const float in = back >= 0 ? to_float<T>(x[(seq_first + back) * p.x_stride + p.conv_off + c])
                                 : before[(int64_t)(taps - 1 + back) * channels + c];
      y = fmaf(w[j], in, y);
    }
    y = y / (1.f + expf(-y));
    if (c < inner) {
      out[2 * gn + c] = dt_s[c / P] * y;                     // v = dt x
      out[2 * gn + inner + H + c] = y;                       // x itself, for the skip term
    } else if (c < inner + gn) {
      out[gn + (c - inner)] = y;                             // B: the scan's k
    } else {
      out[c - inner - gn] = y;                               // C: the scan's q
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) conv_tail_kernel(ConvTailParams p, int channel_blocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x / channel_blocks;
  const int c = (blockIdx.x - s * channel_blocks) * blockDim.x + threadIdx.x;
  const int64_t first = p.cu_q[s];
  const int n = (int)(p.cu_q[s + 1] - first);
  const int slot = p.state_slots[s];
  if (c >= p.channels || n <= 0 || slot < 0 || slot >= p.num_slots) return;
  const int keep = p.taps - 1;
  const T* x = (const T*)p.x;
  float* before = p.state + (int64_t)slot * p.state_stride + p.tail_off;
  float kept[kConvMaxTaps - 1];
#pragma unroll
  for (int i = 0; i < kConvMaxTaps - 1; ++i) {
    kept[i] = 0.f;
    if (i < keep) {
      const int back = n - keep + i;          // index within the step's tokens of this sequence
      kept[i] = back >= 0 ? to_float<T>(x[(first + back) * p.x_stride + p.conv_off + c])
                          : before[(int64_t)(i + n) * p.channels + c];
    }
  }
#pragma unroll
  for (int i = 0; i < kConvMaxTaps - 1; ++i)
    if (i < keep) before[(int64_t)i * p.channels + c] = kept[i];
}

}  // namespace

int launch_ssm_prep(const SsmPrepParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.num_heads < 1 || p.num_heads > kSsmMaxHeads || p.groups < 1 || p.num_heads % p.groups || p.taps < 1 ||
      p.taps > kConvMaxTaps || p.num_tokens > 0x7fffffffLL || p.num_seqs < 1)
    return (int)cudaErrorInvalidValue;
  const int channels = p.num_heads * p.v_dim + 2 * p.groups * p.state_dim;
  int across = 1;                       // few tokens: several blocks share a token's channels
  while (across < 16 && p.num_tokens * across < 256 && channels >= 2 * across * 256) across *= 2;
  const dim3 grid((unsigned)p.num_tokens, (unsigned)across);
  if (p.dtype == kBFloat16)
    return (int)launch_chain(ssm_prep_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, dim3(1, 1, 1), p);
  return (int)launch_chain(ssm_prep_kernel<float>, grid, dim3(256), 0, stream, dim3(1, 1, 1), p);
}

int launch_conv_tail(const ConvTailParams& p, cudaStream_t stream) {
  if (p.num_seqs == 0 || p.taps <= 1) return 0;
  if (p.taps > kConvMaxTaps || p.channels < 1) return (int)cudaErrorInvalidValue;
  const int channel_blocks = (p.channels + 127) / 128;
  const int64_t blocks = (int64_t)p.num_seqs * channel_blocks;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(conv_tail_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, stream, dim3(1, 1, 1),
                             p, channel_blocks);
  return (int)launch_chain(conv_tail_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, dim3(1, 1, 1), p,
                           channel_blocks);
}

}  // namespace akv
