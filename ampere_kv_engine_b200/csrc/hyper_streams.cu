// A residual stream kept in several copies ("hyper-connections"): x_1 .. x_S per token, float32, [N, S, W].
//
// A sublayer reads one mixture of the copies and writes its result back into all of them:
//
//   u     = sum_s read[s] x_s                                  what the sublayer's norm sees
//   x_t  <- sum_s mix[s, t] x_s + write[t] * scale[c] * y      all t at once from the old copies; y the sublayer's
//                                                              result, scale an optional vector over the width
//
// hyper_step does the write of one sublayer and the read and RMS norm of the next in one pass over a token's rows
// (either half may be absent): the copies are read once, the new ones stored, the mixture u kept in shared memory
// between the sum of squares and the output.  hyper_collapse gives sum_t x_t with a write still pending, which is
// what a final norm reads.  hyper_expand makes the S copies from one row.  Everything is float32; y may be float32
// or bfloat16, the normed output is in the serving dtype.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

__device__ __forceinline__ float load_y(const void* y, int y_dtype, int64_t i) {
  return y_dtype == kBFloat16 ? __bfloat162float(((const __nv_bfloat16*)y)[i]) : ((const float*)y)[i];
}

template <typename T>
__global__ void __launch_bounds__(256) hyper_step_kernel(HyperStepParams p) {
  extern __shared__ float hyper_smem[];
  __shared__ float scratch[33];
  __shared__ float coef[kHyperMaxStreams * kHyperMaxStreams + 2 * kHyperMaxStreams];
  pdl_launch_dependents();
  const int S = p.streams, W = p.width;
  float* mix = coef;                                   // [from, to]
  float* write = coef + kHyperMaxStreams * kHyperMaxStreams;
  float* read = write + kHyperMaxStreams;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix[i] = p.y != nullptr ? p.mix[i] : ((i / S == i % S) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    write[i] = p.y != nullptr ? p.write[i] : 0.f;
    read[i] = p.out != nullptr ? p.read[i] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  int64_t token = blockIdx.x;
  if (p.rows != nullptr) {
    token = p.rows[blockIdx.x];
    if (token < 0 || token >= p.num_tokens) {
      if (threadIdx.x == 0) set_status(p.status, kBadRow);
      return;
    }
  }
  float* x = p.x + token * (int64_t)S * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float old[kHyperMaxStreams];
#pragma unroll
    for (int s = 0; s < kHyperMaxStreams; ++s) old[s] = s < S ? x[(int64_t)s * W + c] : 0.f;
    float u = 0.f;
    if (p.y != nullptr) {
      float y = load_y(p.y, p.y_dtype, token * W + c);
      if (p.scale != nullptr) y *= p.scale[c];
#pragma unroll
      for (int t = 0; t < kHyperMaxStreams; ++t) {
        if (t >= S) break;
        float v = write[t] * y;
#pragma unroll
        for (int s = 0; s < kHyperMaxStreams; ++s)
          if (s < S) v = fmaf(mix[s * S + t], old[s], v);
        x[(int64_t)t * W + c] = v;
        u = fmaf(read[t], v, u);
      }
    } else {
#pragma unroll
      for (int s = 0; s < kHyperMaxStreams; ++s)
        if (s < S) u = fmaf(read[s], old[s], u);
    }
    if (p.out != nullptr) {
      hyper_smem[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (p.out == nullptr) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)W + p.eps);
  T* out = (T*)p.out + (int64_t)blockIdx.x * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) out[c] = from_float<T>(hyper_smem[c] * inv * p.weight[c]);
}

// out[n, c] = sum_t x_t after the pending write (if any): sum_s (sum_t mix[s, t]) x_s + (sum_t write[t]) scale y
__global__ void __launch_bounds__(256) hyper_collapse_kernel(HyperStepParams p, float* __restrict__ sum) {
  __shared__ float col[kHyperMaxStreams + 1];
  pdl_launch_dependents();
  const int S = p.streams, W = p.width;
  if (threadIdx.x <= S) {
    float v = 0.f;
    if (threadIdx.x < S) {
      if (p.y == nullptr) v = 1.f;
      else for (int t = 0; t < S; ++t) v += p.mix[threadIdx.x * S + t];
    } else if (p.y != nullptr) {
      for (int t = 0; t < S; ++t) v += p.write[t];
    }
    col[threadIdx.x] = v;
  }
  pdl_wait();
  __syncthreads();
  const int64_t token = blockIdx.x;
  const float* x = p.x + token * (int64_t)S * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = 0.f;
    if (p.y != nullptr) {
      v = col[S] * load_y(p.y, p.y_dtype, token * W + c);
      if (p.scale != nullptr) v *= p.scale[c];
    }
    for (int s = 0; s < S; ++s) v = fmaf(col[s], x[(int64_t)s * W + c], v);
    sum[token * W + c] = v;
  }
}

__global__ void __launch_bounds__(256) hyper_expand_kernel(const float* __restrict__ in, float* __restrict__ x, int S, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = in[token * W + c];
    for (int s = 0; s < S; ++s) x[(token * S + s) * (int64_t)W + c] = v;
  }
}

// out = sa * a / sqrt(mean(a^2) + eps) * wa + sb * b / sqrt(mean(b^2) + eps) * wb, a row per block; a and b float32
template <typename T>
__global__ void __launch_bounds__(256) normed_pair_sum_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                              const float* __restrict__ wa, const float* __restrict__ wb,
                                                              T* __restrict__ out, int W, float eps, float sa, float sb) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = blockIdx.x;
  const float* ra = a + token * W;
  const float* rb = b + token * W;
  float ssa = 0.f, ssb = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    ssa = fmaf(ra[c], ra[c], ssa);
    ssb = fmaf(rb[c], rb[c], ssb);
  }
  ssa = block_sum(ssa, scratch);
  ssb = block_sum(ssb, scratch);
  const float ia = sa / sqrtf(ssa / (float)W + eps), ib = sb / sqrtf(ssb / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    out[token * W + c] = from_float<T>(ra[c] * ia * wa[c] + rb[c] * ib * wb[c]);
}

int threads_for(int width) { return width >= 1024 ? 256 : (width >= 256 ? 128 : 64); }

}  // namespace

int launch_hyper_step(const HyperStepParams& p, cudaStream_t stream) {
  const int64_t blocks = p.rows != nullptr ? p.num_rows : p.num_tokens;
  if (blocks == 0) return 0;
  if (p.streams < 1 || p.streams > kHyperMaxStreams || p.width < 1 || blocks > 0x7fffffffLL ||
      (p.y == nullptr && p.out == nullptr) || (p.rows != nullptr && p.y != nullptr) ||
      (p.y != nullptr && (p.mix == nullptr || p.write == nullptr)) ||
      (p.out != nullptr && (p.read == nullptr || p.weight == nullptr)))
    return (int)cudaErrorInvalidValue;
  const size_t smem = p.out != nullptr ? (size_t)p.width * sizeof(float) : 0;
  auto kernel = p.dtype == kBFloat16 ? hyper_step_kernel<__nv_bfloat16> : hyper_step_kernel<float>;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  return (int)launch_chain(kernel, dim3((unsigned)blocks), dim3(threads_for(p.width)), smem, stream, dim3(1, 1, 1), p);
}

int launch_hyper_collapse(const HyperStepParams& p, float* sum, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.streams < 1 || p.streams > kHyperMaxStreams || p.width < 1 || p.num_tokens > 0x7fffffffLL ||
      (p.y != nullptr && (p.mix == nullptr || p.write == nullptr)))
    return (int)cudaErrorInvalidValue;
  return (int)launch_chain(hyper_collapse_kernel, dim3((unsigned)p.num_tokens), dim3(threads_for(p.width)), 0, stream,
                           dim3(1, 1, 1), p, sum);
}

int launch_hyper_expand(const float* in, float* x, int64_t num_tokens, int streams, int width, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (streams < 1 || streams > kHyperMaxStreams || width < 1 || num_tokens > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(hyper_expand_kernel, dim3((unsigned)num_tokens), dim3(threads_for(width)), 0, stream,
                           dim3(1, 1, 1), in, x, streams, width);
}

int launch_normed_pair_sum(const float* a, const float* b, const float* wa, const float* wb, void* out,
                           int64_t num_tokens, int width, float eps, float sa, float sb, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (width < 1 || num_tokens > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (dtype == kBFloat16)
    return (int)launch_chain(normed_pair_sum_kernel<__nv_bfloat16>, dim3((unsigned)num_tokens), dim3(threads_for(width)),
                             0, stream, dim3(1, 1, 1), a, b, wa, wb, (__nv_bfloat16*)out, width, eps, sa, sb);
  return (int)launch_chain(normed_pair_sum_kernel<float>, dim3((unsigned)num_tokens), dim3(threads_for(width)), 0,
                           stream, dim3(1, 1, 1), a, b, wa, wb, (float*)out, width, eps, sa, sb);
}

}  // namespace akv
