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
#include <algorithm>

#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

__device__ __forceinline__ float load_y(const void* y, int y_dtype, int64_t i) {
  return y_dtype == kBFloat16 ? __bfloat162float(((const __nv_bfloat16*)y)[i]) : ((const float*)y)[i];
}

template <int VEC>
__device__ __forceinline__ void load_vec(const float* p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    v[0] = *p;
  }
}
template <int VEC>
__device__ __forceinline__ void store_vec(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else *p = v[0];
}
template <int VEC>
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  } else {
    *p = __float2bfloat16_rn(v[0]);
  }
}
template <int VEC>
__device__ __forceinline__ void load_y_vec(const void* y, int y_dtype, int64_t i, float (&v)[VEC]) {
  if (y_dtype == kBFloat16) {
    const __nv_bfloat16* p = (const __nv_bfloat16*)y + i;
    if constexpr (VEC == 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(p);
      v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
      v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      v[0] = __bfloat162float(*p);
    }
  } else {
    load_vec<VEC>((const float*)y + i, v);
  }
}

// A block per (row, slice of the columns); the blocks of a row form a cluster (grid y) and add up their sums of
// squares through distributed shared memory.  VEC columns per thread and access (4 where the width allows 16-byte
// accesses).
template <typename T, int VEC>
__global__ void __launch_bounds__(256) hyper_step_kernel(HyperStepParams p, int chunk) {
  extern __shared__ __align__(16) float hyper_smem[];
  __shared__ float scratch[34];
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
  bool bad = false;
  if (p.rows != nullptr) {
    token = p.rows[blockIdx.x];
    if (token < 0 || token >= p.num_tokens) {            // every block of the row sees the same: they skip together
      if (threadIdx.x == 0) set_status(p.status, kBadRow);
      bad = true;
      token = 0;
    }
  }
  const int c0 = blockIdx.y * chunk, c1 = min(W, c0 + chunk);
  float* x = p.x + token * (int64_t)S * W;
  float ss = 0.f;
  for (int c = c0 + threadIdx.x * VEC; c < c1 && !bad; c += blockDim.x * VEC) {
    float old[kHyperMaxStreams][VEC];
#pragma unroll
    for (int s = 0; s < kHyperMaxStreams; ++s)
      if (s < S) load_vec<VEC>(x + (int64_t)s * W + c, old[s]);
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] = 0.f;
    if (p.y != nullptr) {
      float y[VEC];
      load_y_vec<VEC>(p.y, p.y_dtype, token * W + c, y);
      if (p.scale != nullptr) {
        float sc[VEC];
        load_vec<VEC>(p.scale + c, sc);
#pragma unroll
        for (int e = 0; e < VEC; ++e) y[e] *= sc[e];
      }
#pragma unroll
      for (int t = 0; t < kHyperMaxStreams; ++t) {
        if (t >= S) break;
        float v[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = write[t] * y[e];
#pragma unroll
        for (int s = 0; s < kHyperMaxStreams; ++s) {
          if (s < S) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = fmaf(mix[s * S + t], old[s][e], v[e]);
          }
        }
        store_vec<VEC>(x + (int64_t)t * W + c, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) u[e] = fmaf(read[t], v[e], u[e]);
      }
    } else {
#pragma unroll
      for (int s = 0; s < kHyperMaxStreams; ++s) {
        if (s < S) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = fmaf(read[s], old[s][e], u[e]);
        }
      }
    }
    if (p.out != nullptr) {
      store_vec<VEC>(hyper_smem + (c - c0), u);
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(u[e], u[e], ss);
    }
  }
  if (p.out == nullptr) return;
  ss = cluster_sum(ss, scratch);
  if (bad) return;
  const float inv = 1.f / sqrtf(ss / (float)W + p.eps);
  T* out = (T*)p.out + (int64_t)blockIdx.x * W;
  for (int c = c0 + threadIdx.x * VEC; c < c1; c += blockDim.x * VEC) {
    float u[VEC], w[VEC];
    load_vec<VEC>(hyper_smem + (c - c0), u);
    load_vec<VEC>(p.weight + c, w);
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] *= inv * w[e];
    store_vec<VEC>(out + c, u);
  }
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

// out = sa * a / sqrt(mean(a^2) + eps) * wa + sb * b / sqrt(mean(b^2) + eps) * wb; a block per (row, slice of the
// columns), the blocks of a row a cluster (grid y); a and b float32
template <typename T>
__global__ void __launch_bounds__(256) normed_pair_sum_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                              const float* __restrict__ wa, const float* __restrict__ wb,
                                                              T* __restrict__ out, int W, int chunk, float eps, float sa,
                                                              float sb) {
  __shared__ float scratch[34];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = blockIdx.x;
  const int c0 = blockIdx.y * chunk, c1 = min(W, c0 + chunk);
  const float* ra = a + token * W;
  const float* rb = b + token * W;
  float ssa = 0.f, ssb = 0.f;
  for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
    ssa = fmaf(ra[c], ra[c], ssa);
    ssb = fmaf(rb[c], rb[c], ssb);
  }
  ssa = cluster_sum(ssa, scratch);
  ssb = cluster_sum(ssb, scratch);
  const float ia = sa / sqrtf(ssa / (float)W + eps), ib = sb / sqrtf(ssb / (float)W + eps);
  for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x)
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
  // 16-byte accesses where every row, slice and operand starts on a 16-byte boundary
  auto aligned = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
  const bool wide = p.width % 4 == 0 && aligned(p.x) && aligned(p.y) && aligned(p.scale) && aligned(p.weight) &&
                    aligned(p.out);
  const int vec = wide ? 4 : 1;
  const int parts = row_cluster(blocks, p.width);
  const int chunk = ((p.width / vec + parts - 1) / parts) * vec;
  const size_t smem = p.out != nullptr ? (size_t)chunk * sizeof(float) : 0;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  void (*kernel)(HyperStepParams, int) =
      p.dtype == kBFloat16 ? (wide ? hyper_step_kernel<__nv_bfloat16, 4> : hyper_step_kernel<__nv_bfloat16, 1>)
                           : (wide ? hyper_step_kernel<float, 4> : hyper_step_kernel<float, 1>);
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int threads = std::min(256, std::max(32, (chunk / vec + 31) / 32 * 32));
  return (int)launch_chain(kernel, dim3((unsigned)blocks, (unsigned)parts), dim3(threads), smem, stream,
                           dim3(1, parts, 1), p, chunk);
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
  const int parts = row_cluster(num_tokens, width);
  const int chunk = (width + parts - 1) / parts;
  const int threads = std::min(256, std::max(32, (chunk + 31) / 32 * 32));
  const dim3 grid((unsigned)num_tokens, (unsigned)parts), cluster(1, parts, 1);
  if (dtype == kBFloat16)
    return (int)launch_chain(normed_pair_sum_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, cluster, a, b, wa, wb,
                             (__nv_bfloat16*)out, width, chunk, eps, sa, sb);
  return (int)launch_chain(normed_pair_sum_kernel<float>, grid, dim3(threads), 0, stream, cluster, a, b, wa, wb,
                           (float*)out, width, chunk, eps, sa, sb);
}

}  // namespace akv
