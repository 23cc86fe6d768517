// Linear attention with a matrix memory per head that decays row by row, carried from token to token:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t            S: [dim, v_dim] float32 per (request, head)
//
// Two ways to fill a_t and k_t from one product's columns:
//   kGatedWrite      a = f, k = 1 - f with f = lower + (1 - lower) * sigmoid(x_f + bias)  (a forget gate per row that
//                    also decides what is written), q = silu(x_q), v = x_v
//   kConstantDecay   a = decay[head] for every row, k = silu(x_k), q = silu(x_q), v = silu(x_v)
// Everything after the product is float32: gates, activations, the memory and both products with it.
//
// Work split: a block owns (sequence, head, 32 value columns) for the whole step.  A value column of S lives in the
// registers of `lanes` neighbouring lanes (ROWS rows each), so writing a token is thread-local and reading it out is
// one sum over those lanes.  Tokens are staged through shared memory CHUNK at a time (activations and gates are
// worked out once per chunk by all threads).  S moves between registers and the request's state slot in an order of
// its own ([head][slice][row in lane][column][lane]), so that the loads and stores of a decode step are coalesced.
// Tokens are walked one by one whatever the step holds: the memory after a token does not depend on how the tokens
// were cut into steps.
//
// A second kernel norms what the scan read out: RMS over groups of columns (a head, or all heads together), a
// weight, a constant factor, and optionally a sigmoid gate from further columns of the product.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

constexpr int kScanColumns = 32;     // value columns per block
constexpr int kScanChunk = 16;       // tokens staged at a time

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

template <typename T, int MODE, int ROWS>
__global__ void __launch_bounds__(256)
linear_scan_kernel(LinearScanParams p, int lanes, int slices) {
  pdl_launch_dependents();
  pdl_wait();
  const int H = p.num_heads, D = p.head_dim, DV = p.v_dim;
  const int DP = lanes * ROWS;                         // rows of S with padding
  const int slice = blockIdx.x % slices;
  const int head = (blockIdx.x / slices) % H;
  const int seq = blockIdx.x / (slices * H);
  const int slot = p.state_slots[seq];
  const int t0 = p.cu_q[seq];
  const int n = p.cu_q[seq + 1] - t0;
  if (slot < 0 || n <= 0) return;                      // a padded sequence: nothing is read or written
  const int tid = threadIdx.x, threads = blockDim.x;
  const int sub = tid % lanes, col = tid / lanes;
  const int j = slice * kScanColumns + col;

  extern __shared__ float smem[];
  float* qs = smem;                                    // [CHUNK][DP]
  float* as = qs + kScanChunk * DP;                    // [CHUNK][DP]: f (gated write) or k (constant decay)
  float* vs = as + kScanChunk * DP;                    // [CHUNK][32]

  float* mem = p.state + (int64_t)slot * p.state_stride +
               ((int64_t)head * slices + slice) * ROWS * (int64_t)threads + tid;
  float S[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) S[r] = mem[(int64_t)r * threads];
  const float decay = MODE == kConstantDecay ? p.decay[head] : 0.f;

  const T* x = (const T*)p.x;
  const int wide = H * DV;
  for (int c0 = 0; c0 < n; c0 += kScanChunk) {
    const int nt = min(kScanChunk, n - c0);
    for (int idx = tid; idx < nt * DP; idx += threads) {
      const int t = idx / DP, d = idx - t * DP;
      float qv = 0.f, av = MODE == kGatedWrite ? 1.f : 0.f;      // padded rows stay zero
      if (d < D) {
        const T* row = x + (int64_t)(t0 + c0 + t) * p.x_stride;
        const int ch = head * D + d;
        qv = silu_f(to_float<T>(row[p.q_off + ch]));
        const float raw = to_float<T>(row[p.k_off + ch]);
        if (MODE == kGatedWrite) {
          const float low = p.lower[ch];
          av = low + (1.f - low) * sigmoid_f(raw + (p.gate_bias != nullptr ? p.gate_bias[ch] : 0.f));
        } else {
          av = silu_f(raw);
        }
      }
      qs[idx] = qv;
      as[idx] = av;
    }
    for (int idx = tid; idx < nt * kScanColumns; idx += threads) {
      const int t = idx / kScanColumns, c = idx - t * kScanColumns;
      const int jj = slice * kScanColumns + c;
      float vv = 0.f;
      if (jj < DV) {
        vv = to_float<T>(x[(int64_t)(t0 + c0 + t) * p.x_stride + p.v_off + head * DV + jj]);
        if (MODE == kConstantDecay) vv = silu_f(vv);
      }
      vs[idx] = vv;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = vs[t * kScanColumns + col];
      const float4* q4 = reinterpret_cast<const float4*>(qs + t * DP + sub * ROWS);
      const float4* a4 = reinterpret_cast<const float4*>(as + t * DP + sub * ROWS);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int r4 = 0; r4 < ROWS / 4; ++r4) {
        const float4 q = q4[r4], a = a4[r4];
        const float qa[4] = {q.x, q.y, q.z, q.w}, aa[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = r4 * 4 + e;
          if (MODE == kGatedWrite) S[r] = aa[e] * S[r] + (1.f - aa[e]) * v;
          else S[r] = decay * S[r] + aa[e] * v;
          if (e & 1) o1 += S[r] * qa[e];
          else o0 += S[r] * qa[e];
        }
      }
      float o = o0 + o1;
      for (int w = 1; w < lanes; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (sub == 0 && j < DV) p.out[(int64_t)(t0 + c0 + t) * wide + head * DV + j] = o;
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) mem[(int64_t)r * threads] = S[r];
}

// out[t, c] = in[t, c] / sqrt(mean over c's group of in^2 + eps) * weight[c % weight_len] * factor
//             (* sigmoid(x[t, gate_off + c]));   one block per (token, group)
template <typename T>
__global__ void group_norm_gate_kernel(const float* __restrict__ in, T* __restrict__ out, const float* __restrict__ weight,
                                       int weight_len, int group, int width, float eps, float factor,
                                       const T* __restrict__ x, int64_t x_stride, int gate_off) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int groups = width / group;
  const int64_t token = blockIdx.x / groups;
  const int g = blockIdx.x % groups;
  const float* src = in + token * width + (int64_t)g * group;
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) ss += src[i] * src[i];
  ss = block_sum(ss, scratch);
  const float inv = factor / sqrtf(ss / (float)group + eps);
  T* dst = out + token * width + (int64_t)g * group;
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const int c = g * group + i;
    float y = src[i] * inv * weight[c % weight_len];
    if (x != nullptr) y *= sigmoid_f(to_float<T>(x[token * x_stride + gate_off + c]));
    dst[i] = from_float<T>(y);
  }
}

}  // namespace

bool linear_scan_shape(int head_dim, int v_dim, int* rows, int* lanes) {
  if (head_dim < 1 || head_dim > kLinearScanMaxDim || v_dim < 1 || v_dim > kLinearScanMaxDim) return false;
  const int r = head_dim <= 128 ? 16 : 32;
  int l = 1;
  while (l * r < head_dim) l *= 2;
  if (l > 8) return false;
  *rows = r;
  *lanes = l;
  return true;
}

int64_t linear_scan_state_floats(int num_heads, int head_dim, int v_dim) {
  int rows = 0, lanes = 0;
  if (!linear_scan_shape(head_dim, v_dim, &rows, &lanes)) return -1;
  const int slices = (v_dim + kScanColumns - 1) / kScanColumns;
  return (int64_t)num_heads * slices * kScanColumns * rows * lanes;
}

template <typename T, int MODE, int ROWS>
static int launch_scan(const LinearScanParams& p, int lanes, cudaStream_t stream) {
  const int slices = (p.v_dim + kScanColumns - 1) / kScanColumns;
  const int64_t blocks = (int64_t)p.num_seqs * p.num_heads * slices;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)kScanChunk * (2 * lanes * ROWS + kScanColumns) * sizeof(float);
  return (int)launch_chain(linear_scan_kernel<T, MODE, ROWS>, dim3((unsigned)blocks), dim3(kScanColumns * lanes), smem,
                           stream, dim3(1, 1, 1), p, lanes, slices);
}

template <typename T>
static int launch_scan_typed(const LinearScanParams& p, int rows, int lanes, cudaStream_t stream) {
  if (p.mode == kGatedWrite)
    return rows == 16 ? launch_scan<T, kGatedWrite, 16>(p, lanes, stream) : launch_scan<T, kGatedWrite, 32>(p, lanes, stream);
  return rows == 16 ? launch_scan<T, kConstantDecay, 16>(p, lanes, stream)
                    : launch_scan<T, kConstantDecay, 32>(p, lanes, stream);
}

int launch_linear_scan(const LinearScanParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0 || p.num_seqs == 0) return 0;
  int rows = 0, lanes = 0;
  if (!linear_scan_shape(p.head_dim, p.v_dim, &rows, &lanes) || p.num_heads < 1 ||
      (p.mode != kGatedWrite && p.mode != kConstantDecay))
    return (int)cudaErrorInvalidValue;
  if (p.mode == kGatedWrite ? p.lower == nullptr : p.decay == nullptr) return (int)cudaErrorInvalidValue;
  return p.dtype == kBFloat16 ? launch_scan_typed<__nv_bfloat16>(p, rows, lanes, stream)
                              : launch_scan_typed<float>(p, rows, lanes, stream);
}

int launch_group_norm_gate(const float* in, void* out, const float* weight, int weight_len, int64_t num_tokens,
                           int width, int group, float eps, float factor, const void* x, int64_t x_stride,
                           int gate_off, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (group < 1 || width % group || weight_len < 1) return (int)cudaErrorInvalidValue;
  const int64_t blocks = num_tokens * (width / group);
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const int threads = group >= 1024 ? 256 : (group >= 128 ? 128 : (group > 32 ? 64 : 32));
  if (dtype == kBFloat16)
    return (int)launch_chain(group_norm_gate_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                             dim3(1, 1, 1), in, (__nv_bfloat16*)out, weight, weight_len, group, width, eps, factor,
                             (const __nv_bfloat16*)x, x_stride, gate_off);
  return (int)launch_chain(group_norm_gate_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                           in, (float*)out, weight, weight_len, group, width, eps, factor, (const float*)x, x_stride,
                           gate_off);
}

}  // namespace akv
