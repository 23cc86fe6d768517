// Small kernels on the float32 residual stream and on branch outputs:
//
//   pair_rows_add   hidden[t] += table[(prev(t) * mul_prev + token(t) * mul_cur) mod buckets], and row `buckets` for a
//                   sequence's first token (position 0).  prev(t) is the token before t in the same sequence: the row
//                   above inside a step, and for a step's first row the last token of the step before, which the
//                   request keeps in its state slot (one int32).  The block of a sequence's first row reads that
//                   token and then stores the sequence's newest one; no other block touches the slot.
//   stream_add      hidden += other (both float32)
//   scaled_sum      out = a * sa + b * sb, formed in float32 and rounded once
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

__device__ __forceinline__ int64_t resolve_token(int64_t id, const int32_t* sampled, int64_t num_sampled, int64_t vocab) {
  if (id < 0 && sampled != nullptr && -id - 1 < num_sampled) id = sampled[-id - 1];
  return (id < 0 || id >= vocab) ? 0 : id;             // the embedding kernel has reported it
}

template <typename T>
__global__ void pair_rows_add_kernel(PairRowsParams p) {
  __shared__ int64_t prev_shared;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = blockIdx.x;
  // the sequence whose rows hold this token: the last s with cu_q[s] <= token
  int lo = 0, hi = p.num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (p.cu_q[mid] <= token) lo = mid;
    else hi = mid - 1;
  }
  const int seq = lo;
  const bool first_row = token == p.cu_q[seq];
  const int slot = p.state_slots[seq];
  const int64_t cur = resolve_token(p.ids[token], p.sampled, p.num_sampled, p.vocab);
  if (threadIdx.x == 0) {
    int64_t prev = 0;
    if (!first_row) prev = resolve_token(p.ids[token - 1], p.sampled, p.num_sampled, p.vocab);
    else if (slot >= 0) prev = p.last_token[(int64_t)slot * p.state_stride];
    prev_shared = prev;
    if (first_row && slot >= 0) {
      const int64_t last = p.cu_q[seq + 1] - 1;
      if (last >= token && last < p.num_tokens)
        p.last_token[(int64_t)slot * p.state_stride] =
            (int32_t)resolve_token(p.ids[last], p.sampled, p.num_sampled, p.vocab);
    }
  }
  __syncthreads();
  int64_t row = p.buckets;
  if (p.positions[token] > 0) {
    row = (prev_shared * p.mul_prev + cur * p.mul_cur) % p.buckets;
    if (row < 0) row += p.buckets;
  }
  const T* src = (const T*)p.table + row * p.hidden_size;
  float* dst = p.hidden + token * p.hidden_size;
  for (int64_t i = threadIdx.x; i < p.hidden_size; i += blockDim.x) dst[i] += to_float<T>(src[i]);
}

__global__ void stream_add_kernel(float* __restrict__ hidden, const float* __restrict__ other, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 a = *reinterpret_cast<float4*>(hidden + i);
    const float4 b = *reinterpret_cast<const float4*>(other + i);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    *reinterpret_cast<float4*>(hidden + i) = a;
  } else {
    for (int64_t k = i; k < n; ++k) hidden[k] += other[k];
  }
}

template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, float sa,
                                  float sb, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<T>(to_float<T>(a[i]) * sa + to_float<T>(b[i]) * sb);
}

}  // namespace

int launch_pair_rows_add(const PairRowsParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.buckets < 1 || p.num_seqs < 1) return (int)cudaErrorInvalidValue;
  const int threads = (int)(p.hidden_size >= 1024 ? 256 : (p.hidden_size >= 128 ? 128 : 32));
  if (p.dtype == kBFloat16)
    return (int)launch_chain(pair_rows_add_kernel<__nv_bfloat16>, dim3((unsigned)p.num_tokens), dim3(threads), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(pair_rows_add_kernel<float>, dim3((unsigned)p.num_tokens), dim3(threads), 0, stream,
                           dim3(1, 1, 1), p);
}

int launch_stream_add(float* hidden, const float* other, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  const int64_t blocks = ((n + 3) / 4 + 255) / 256;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(stream_add_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, dim3(1, 1, 1), hidden, other, n);
}

int launch_scaled_sum(const void* a, const void* b, void* out, float sa, float sb, int64_t n, int dtype,
                      cudaStream_t stream) {
  if (n == 0) return 0;
  const int64_t blocks = (n + 255) / 256;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (dtype == kBFloat16)
    return (int)launch_chain(scaled_sum_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, dim3(1, 1, 1),
                             (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, sa, sb, n);
  return (int)launch_chain(scaled_sum_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, dim3(1, 1, 1),
                           (const float*)a, (const float*)b, (float*)out, sa, sb, n);
}

}  // namespace akv
