// A feed-forward of routed experts, entirely on the device (no host read of the routing).
//
//   moe_router:   the router's logits for a few tokens (a warp per token and expert); larger steps use the library.
//   moe_route:    per token: s = sigmoid(logits); choice = s + correction; the experts form equal groups of
//                 neighbours, a group's score is the sum of its group_top largest choice scores, only experts of the
//                 keep best groups can be chosen; the top largest remaining choice scores are chosen (ties: the lower
//                 index); weights = chosen s / (their sum + eps) * scale.  One warp per token, all in float.
//   moe_sort:     a counting sort of the (token, choice) pairs by expert: where each expert's run begins, and the
//                 pairs in that order (within an expert in no particular order: every row is computed by itself).
//   moe_gate_up:  for the sorted rows of every expert, both products with the expert's matrices and the clamped
//                 activation on the output tile.
//   moe_down:     the third product, times the pair's weight, written to the pair's own row (float32).
//   moe_combine:  a token's rows added up in the order of its choices, plus the shared expert's row.
//
// The grouped products tile the sorted rows expert by expert: a block finds its (expert, row tile) by walking the
// run starts, so the grid depends on the batch layout alone.  Each output element is one dot product accumulated
// in float in the order of k, whatever tile it falls in: a row's result does not depend on the rest of the batch.
#include "common.cuh"
#include "launchers.h"

#include <float.h>
#include <stdlib.h>

namespace akv {

namespace {

constexpr int kRouteWarps = 4;

__device__ __forceinline__ bool better(float v, int i, float best, int best_i) {
  return v > best || (v == best && i < best_i);
}

}  // namespace

__global__ void moe_route_kernel(MoeRouteParams p) {
  extern __shared__ float route_smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t token = (int64_t)blockIdx.x * kRouteWarps + warp;
  if (token >= p.num_tokens) return;
  const int E = p.experts, groups = p.groups, per = E / groups;
  float* score = route_smem + (size_t)warp * (2 * E + 2 * groups);     // s
  float* choice = score + E;                                            // s + correction, later masked
  float* group_score = choice + E;
  float* group_kept = group_score + groups;
  const float* z = p.logits + token * E;
  // softmax scores: the row's maximum and the sum of the exponentials first (a row of padding may hold anything)
  float row_max = 0.f, row_inv = 1.f;
  if (p.score_kind == 1) {
    float m = -FLT_MAX;
    for (int e = lane; e < E; e += 32)
      if (z[e] == z[e]) m = fmaxf(m, fminf(z[e], FLT_MAX));
    row_max = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - row_max);
    sum = warp_sum(sum);
    row_inv = 1.f / sum;
  }
  for (int e = lane; e < E; e += 32) {
    const float s = p.score_kind == 1 ? expf(z[e] - row_max) * row_inv : 1.f / (1.f + expf(-z[e]));
    float c = p.correction != nullptr ? s + p.correction[e] : s;
    if (!(c == c)) c = -FLT_MAX;          // a row of padding may hold anything; the choice must still be an expert
    score[e] = s;
    choice[e] = c;
  }
  __syncwarp();
  if (groups > 1) {
    const int take = min(p.group_top, per);
    for (int g = lane; g < groups; g += 32) {
      // the sum of the group's `take` largest choice scores: repeated maximum, skipping what was taken
      const float* c = choice + g * per;
      float sum = 0.f;
      float last = FLT_MAX;
      int last_i = -1;
      for (int r = 0; r < take; ++r) {
        float best = -FLT_MAX;
        int best_i = -1;
        for (int i = 0; i < per; ++i) {
          // candidates: everything after (last, last_i) in the order (value descending, index ascending)
          const bool after = c[i] < last || (c[i] == last && i > last_i);
          if (after && (best_i < 0 || better(c[i], i, best, best_i))) {
            best = c[i];
            best_i = i;
          }
        }
        if (best_i < 0) break;
        sum += best;
        last = best;
        last_i = best_i;
      }
      group_score[g] = sum;
    }
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
      int rank = 0;
      for (int o = 0; o < groups; ++o)
        rank += (group_score[o] > group_score[g] || (group_score[o] == group_score[g] && o < g)) ? 1 : 0;
      group_kept[g] = rank < p.keep_groups ? 1.f : 0.f;
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32)
      if (group_kept[e / per] == 0.f) choice[e] = -INFINITY;
    __syncwarp();
  }
  // the `top` largest choice scores, one after the other
  float picked_sum = 0.f;
  float my_score = 0.f;           // lane r keeps the r-th choice
  int my_expert = 0;
  for (int r = 0; r < p.top; ++r) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (c != c) continue;       // marks of what was chosen already
      if (better(c, e, best, best_i) || best_i == 0x7fffffff) {
        best = c;
        best_i = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_i = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (other_i != 0x7fffffff && (best_i == 0x7fffffff || better(other, other_i, best, best_i))) {
        best = other;
        best_i = other_i;
      }
    }
    if (best_i == 0x7fffffff) best_i = 0;       // more choices than experts: cannot happen with a checked config
    const float s = score[best_i];
    picked_sum += s;
    if (lane == r % 32) {
      my_score = s;
      my_expert = best_i;
    }
    if (lane == 0) choice[best_i] = __int_as_float(0x7fc00000);   // NaN: taken
    __syncwarp();
  }
  if (lane < p.top) {          // top <= 32 (checked by the launcher)
    p.chosen[token * p.top + lane] = my_expert;
    p.weights[token * p.top + lane] = my_score / (picked_sum + p.weight_eps) * p.scale;
  }
}

// Router logits of a few tokens: a warp per (token, expert), the dot product over the hidden size in float.  (The
// library's product of a handful of rows with a matrix of a few dozen rows runs on one or two SMs.)
template <typename T>
__global__ void __launch_bounds__(256) moe_router_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                         float* __restrict__ logits, int experts, int k) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int expert = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t token = blockIdx.y;
  if (expert >= experts) return;
  const T* a = x + token * k;
  const T* b = w + (int64_t)expert * k;
  float sum = 0.f;
  constexpr int kVec = 16 / sizeof(T);
  if (k % kVec == 0 && (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % 16 == 0) {
    float s0 = 0.f, s1 = 0.f;
    for (int c = lane * kVec; c < k; c += 32 * kVec) {
      if constexpr (sizeof(T) == 2) {
        float u[8], v[8];
        load8<T>(a + c, u);
        load8<T>(b + c, v);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          s0 = fmaf(u[i], v[i], s0);
          s1 = fmaf(u[i + 1], v[i + 1], s1);
        }
      } else {
        const float4 u = *reinterpret_cast<const float4*>(a + c), v = *reinterpret_cast<const float4*>(b + c);
        s0 = fmaf(u.x, v.x, s0); s1 = fmaf(u.y, v.y, s1); s0 = fmaf(u.z, v.z, s0); s1 = fmaf(u.w, v.w, s1);
      }
    }
    sum = s0 + s1;
  } else {
    for (int c = lane; c < k; c += 32) sum = fmaf(to_float<T>(a[c]), to_float<T>(b[c]), sum);
  }
  sum = warp_sum(sum);
  if (lane == 0) logits[token * experts + expert] = sum;
}

int launch_moe_router(const void* x, const void* w, float* logits, int64_t tokens, int experts, int k, int dtype,
                      cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (experts <= 0 || k <= 0 || tokens > 65535) return (int)cudaErrorInvalidValue;
  const dim3 grid((unsigned)((experts + 7) / 8), (unsigned)tokens);
  if (dtype == kBFloat16)
    return (int)launch_chain(moe_router_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, dim3(1, 1, 1),
                             (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, logits, experts, k);
  return (int)launch_chain(moe_router_kernel<float>, grid, dim3(256), 0, stream, dim3(1, 1, 1), (const float*)x,
                           (const float*)w, logits, experts, k);
}

int launch_moe_route(const MoeRouteParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.experts <= 0 || p.experts > kMoeMaxExperts || p.top <= 0 || p.top > 32 || p.top > p.experts || p.groups <= 0 ||
      p.experts % p.groups || p.keep_groups <= 0 || p.keep_groups > p.groups || p.group_top <= 0 ||
      (p.score_kind != 0 && p.score_kind != 1))
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)kRouteWarps * (2 * p.experts + 2 * p.groups) * sizeof(float);
  const int64_t blocks = (p.num_tokens + kRouteWarps - 1) / kRouteWarps;
  if (blocks > 0x7fffffffLL || smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(moe_route_kernel, dim3((unsigned)blocks), dim3(kRouteWarps * 32), smem, stream, dim3(1, 1, 1), p);
}

// One block: counts per expert in shared memory, their running sum, then every pair takes the next place of its
// expert's run.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t* __restrict__ chosen, int32_t* __restrict__ order,
                                                        int32_t* __restrict__ offsets, int64_t pairs, int experts) {
  __shared__ int counts[kMoeMaxExperts];
  __shared__ int starts[kMoeMaxExperts + 1];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = min(max(chosen[i], 0), experts - 1);
    atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      starts[e] = run;
      run += counts[e];
    }
    starts[experts] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = starts[e];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = min(max(chosen[i], 0), experts - 1);
    order[starts[e] + atomicAdd(&counts[e], 1)] = (int32_t)i;
  }
}

int launch_moe_sort(const int32_t* chosen, int32_t* order, int32_t* offsets, int64_t pairs, int experts,
                    cudaStream_t stream) {
  if (experts <= 0 || experts > kMoeMaxExperts || pairs > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, dim3(1, 1, 1), chosen, order, offsets, pairs,
                           experts);
}

// ---------------------------------------------------------------------------------------------------------
// The grouped products.  A block computes kTileRows sorted rows of one expert times kTileCols output features (of
// the gate and the up matrix at once in the first product), K in steps of kTileK through shared memory (operands
// widened to float there), 2 x 4 outputs per thread.
namespace {
constexpr int kTileRows = 32, kTileCols = 64, kTileK = 32, kGemmThreads = 256;

// the (expert, first sorted row, rows) of row tile `tile`, or rows = 0 when the batch has fewer tiles
__device__ __forceinline__ void find_tile(const int32_t* offsets, int experts, int tile, int& expert, int& row0,
                                          int& rows) {
  rows = 0;
  expert = row0 = 0;
  int seen = 0;
  for (int e = 0; e < experts; ++e) {
    const int begin = offsets[e], count = offsets[e + 1] - begin;
    const int tiles = (count + kTileRows - 1) / kTileRows;
    if (tile < seen + tiles) {
      expert = e;
      row0 = begin + (tile - seen) * kTileRows;
      rows = min(kTileRows, begin + count - row0);
      return;
    }
    seen += tiles;
  }
}
}  // namespace

template <typename T, bool GATED>
__global__ void __launch_bounds__(kGemmThreads) moe_gemm_kernel(MoeGemmParams p) {
  __shared__ float a_tile[kTileK][kTileRows + 1];
  __shared__ float w_tile[GATED ? 2 : 1][kTileK][kTileCols + 1];
  __shared__ int tile_info[3];
  __shared__ int64_t row_source[kTileRows];
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int e, r0, n;
    find_tile(p.offsets, p.experts, blockIdx.y, e, r0, n);
    tile_info[0] = e;
    tile_info[1] = r0;
    tile_info[2] = n;
  }
  __syncthreads();
  const int expert = tile_info[0], row0 = tile_info[1], rows = tile_info[2];
  if (rows == 0) return;
  const int K = p.k, N = p.n;                       // N: output features (per matrix in the gated product)
  const int col0 = blockIdx.x * kTileCols;
  if (threadIdx.x < kTileRows) {
    const int r = threadIdx.x;
    int64_t src = -1;
    if (r < rows) src = GATED ? (int64_t)(p.order[row0 + r] / p.top) : (int64_t)(row0 + r);
    row_source[r] = src;
  }
  __syncthreads();
  const T* a = (const T*)p.a;
  const T* w = (const T*)p.w + (int64_t)expert * (GATED ? 2 : 1) * N * K;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[GATED ? 2 : 1][2][4] = {};
  for (int k0 = 0; k0 < K; k0 += kTileK) {
    for (int i = threadIdx.x; i < kTileRows * kTileK; i += kGemmThreads) {
      const int r = i / kTileK, kk = i % kTileK;
      const int64_t src = row_source[r];
      a_tile[kk][r] = (src >= 0 && k0 + kk < K) ? to_float<T>(a[src * K + k0 + kk]) : 0.f;
    }
    for (int i = threadIdx.x; i < kTileCols * kTileK; i += kGemmThreads) {
      const int c = i / kTileK, kk = i % kTileK;
      const bool inside = col0 + c < N && k0 + kk < K;
      w_tile[0][kk][c] = inside ? to_float<T>(w[(int64_t)(col0 + c) * K + k0 + kk]) : 0.f;
      if (GATED) w_tile[1][kk][c] = inside ? to_float<T>(w[(int64_t)(N + col0 + c) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kTileK; ++kk) {
      const float a0 = a_tile[kk][ty * 2], a1 = a_tile[kk][ty * 2 + 1];
#pragma unroll
      for (int m = 0; m < (GATED ? 2 : 1); ++m) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float b = w_tile[m][kk][tx * 4 + j];
          acc[m][0][j] = fmaf(a0, b, acc[m][0][j]);
          acc[m][1][j] = fmaf(a1, b, acc[m][1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
    if (GATED) {
      T* dst = (T*)p.out + (int64_t)(row0 + r) * N;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = col0 + tx * 4 + j;
        if (c >= N) continue;
        const float g = fminf(acc[0][i][j], p.limit);
        const float u = fminf(fmaxf(acc[GATED ? 1 : 0][i][j], -p.limit), p.limit);
        dst[c] = from_float<T>(g / (1.f + expf(-p.slope * g)) * (u + p.up_offset));
      }
    } else {
      const int pair = p.order[row0 + r];
      const float weight = p.weights[pair];
      float* dst = (float*)p.out + (int64_t)pair * N;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = col0 + tx * 4 + j;
        if (c < N) dst[c] = weight * acc[0][i][j];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// The same products on the tensor cores, for bfloat16 with k a multiple of eight (16-byte copies): 64 sorted rows of
// one expert times 128 weight rows (gated: 64 gate rows and the 64 up rows of the same features), k in steps of 32
// through a three-stage cp.async ring, ldmatrix + mma.sync m16n8k16 with float accumulators.  Eight warps, two along
// the rows and four along the features; in the gated product a warp holds 16 gate features and the same 16 up
// features, so the activation is applied to its own accumulators.
namespace {
constexpr int kMmaRows = 64, kMmaWeightRows = 128, kMmaK = 32, kMmaStages = 3, kMmaPitch = kMmaK + 8;

__device__ __forceinline__ void cp_async_16(void* smem, const void* global, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;                 // zero bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(global), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void find_tile_of(const int32_t* offsets, int experts, int tile, int tile_rows, int& expert,
                                             int& row0, int& rows) {
  rows = 0;
  expert = row0 = 0;
  int seen = 0;
  for (int e = 0; e < experts; ++e) {
    const int begin = offsets[e], count = offsets[e + 1] - begin;
    const int tiles = (count + tile_rows - 1) / tile_rows;
    if (tile < seen + tiles) {
      expert = e;
      row0 = begin + (tile - seen) * tile_rows;
      rows = min(tile_rows, begin + count - row0);
      return;
    }
    seen += tiles;
  }
}
}  // namespace

template <bool GATED, int BM>
__global__ void __launch_bounds__(256) moe_gemm_mma_kernel(MoeGemmParams p) {
  // BM sorted rows of one expert per CTA (64, or 128 where experts have rows enough to fill such tiles: a warp then
  // holds 64 x 32 of the output and every weight fragment it fetches serves four row fragments instead of two)
  extern __shared__ __align__(16) unsigned char mma_smem[];
  typedef __nv_bfloat16 (*ATile)[BM][kMmaPitch];
  typedef __nv_bfloat16 (*WTile)[kMmaWeightRows][kMmaPitch];
  ATile a_smem = reinterpret_cast<ATile>(mma_smem);
  WTile w_smem = reinterpret_cast<WTile>(mma_smem + sizeof(__nv_bfloat16) * kMmaStages * BM * kMmaPitch);
  __shared__ int tile_info[3];
  __shared__ int64_t row_source[BM];
  constexpr int MI = BM / 32;                       // 16-row fragments per warp
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int e, r0, n;
    find_tile_of(p.offsets, p.experts, blockIdx.y, BM, e, r0, n);
    tile_info[0] = e;
    tile_info[1] = r0;
    tile_info[2] = n;
  }
  __syncthreads();
  const int expert = tile_info[0], row0 = tile_info[1], rows = tile_info[2];
  if (rows == 0) return;
  const int K = p.k, N = p.n;
  constexpr int kCols = GATED ? kMmaWeightRows / 2 : kMmaWeightRows;      // output features of the tile
  const int col0 = blockIdx.x * kCols;
  if (threadIdx.x < BM) {
    const int r = threadIdx.x;
    int64_t src = -1;
    if (r < rows) src = GATED ? (int64_t)(p.order[row0 + r] / p.top) : (int64_t)(row0 + r);
    row_source[r] = src;
  }
  __syncthreads();
  const __nv_bfloat16* a = (const __nv_bfloat16*)p.a;
  const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (int64_t)expert * (GATED ? 2 : 1) * N * K;

  // this thread's copies of a stage: BM / 64 16-byte pieces of the rows' tile, two of the weights' tile
  const int piece = threadIdx.x & 3;
  int64_t a_src[BM / 64];
#pragma unroll
  for (int i = 0; i < BM / 64; ++i) a_src[i] = row_source[(threadIdx.x >> 2) + 64 * i];
  int64_t w_src[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int wr = (threadIdx.x >> 2) + 64 * i;               // row of the weights' tile
    int64_t row;
    if (GATED) row = wr < 64 ? (int64_t)col0 + wr : (int64_t)N + col0 + (wr - 64);
    else row = (int64_t)col0 + wr;
    const bool inside = GATED ? (col0 + (wr & 63) < N) : (col0 + wr < N);
    w_src[i] = inside ? row : -1;
  }
  auto issue = [&](int stage, int k0) {
    const int k = k0 + piece * 8;
    const bool in_k = k < K;
#pragma unroll
    for (int i = 0; i < BM / 64; ++i)
      cp_async_16(&a_smem[stage][(threadIdx.x >> 2) + 64 * i][piece * 8], a + (a_src[i] >= 0 && in_k ? a_src[i] * K + k : 0),
                  a_src[i] >= 0 && in_k);
#pragma unroll
    for (int i = 0; i < 2; ++i)
      cp_async_16(&w_smem[stage][(threadIdx.x >> 2) + 64 * i][piece * 8], w + (w_src[i] >= 0 && in_k ? w_src[i] * K + k : 0),
                  w_src[i] >= 0 && in_k);
  };

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wm = warp >> 2, wn = warp & 3;                    // 2 x 4 warps
  // the four 8-feature tiles of this warp, as rows of the weights' tile
  int n_base[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    n_base[j] = GATED ? (j < 2 ? wn * 16 + j * 8 : 64 + wn * 16 + (j - 2) * 8) : wn * 32 + j * 8;
  float acc[MI][4][4] = {};
  const int steps = (K + kMmaK - 1) / kMmaK;
#pragma unroll
  for (int s = 0; s < kMmaStages - 1; ++s) {
    if (s < steps) issue(s, s * kMmaK);
    cp_async_commit();
  }
  for (int step = 0; step < steps; ++step) {
    cp_async_wait<kMmaStages - 2>();
    __syncthreads();
    const int next = step + kMmaStages - 1;
    if (next < steps) issue(next % kMmaStages, next * kMmaK);
    cp_async_commit();
    const int stage = step % kMmaStages;
#pragma unroll
    for (int kk = 0; kk < kMmaK; kk += 16) {
      uint32_t af[MI][4];
#pragma unroll
      for (int i = 0; i < MI; ++i)
        ldmatrix_x4(af[i], &a_smem[stage][wm * (BM / 2) + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        // two 8-feature tiles at a time: lanes 0-15 address the first, 16-31 the second; within each, lanes 8-15 the
        // upper half of k
        uint32_t bf[4];
        const int nb = (lane < 16) ? n_base[j] : n_base[j + 1];
        ldmatrix_x4(bf, &w_smem[stage][nb + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int i = 0; i < MI; ++i) {
          mma_bf16(acc[i][j], af[i], bf[0], bf[1]);
          mma_bf16(acc[i][j + 1], af[i], bf[2], bf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // accumulator element e of tile (i, j): row wm * BM / 2 + i * 16 + lane / 4 (+ 8 for e >= 2), feature (lane % 4) * 2 + (e & 1)
#pragma unroll
  for (int i = 0; i < MI; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * (BM / 2) + i * 16 + (lane >> 2) + half * 8;
      if (r >= rows) continue;
      if (GATED) {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (int64_t)(row0 + r) * N;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = col0 + wn * 16 + j * 8 + (lane & 3) * 2 + e;
            if (c >= N) continue;
            const float g = fminf(acc[i][j][half * 2 + e], p.limit);
            const float u = fminf(fmaxf(acc[i][j + 2][half * 2 + e], -p.limit), p.limit);
            dst[c] = __float2bfloat16_rn(g / (1.f + expf(-p.slope * g)) * (u + p.up_offset));
          }
        }
      } else {
        const int pair = p.order[row0 + r];
        const float weight = p.weights[pair];
        float* dst = (float*)p.out + (int64_t)pair * N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = col0 + wn * 32 + j * 8 + (lane & 3) * 2 + e;
            if (c < N) dst[c] = weight * acc[i][j][half * 2 + e];
          }
        }
      }
    }
  }
}

static bool moe_gemm_takes_mma(const MoeGemmParams& p) {
  return p.dtype == kBFloat16 && p.k % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.w)) % 16 == 0;
}

template <bool GATED, int BM>
static int launch_moe_mma(const MoeGemmParams& p, cudaStream_t stream) {
  const int64_t row_tiles = p.pairs / BM + (p.pairs < p.experts ? p.pairs : p.experts);
  const int cols = GATED ? kMmaWeightRows / 2 : kMmaWeightRows;
  const int64_t col_tiles = (p.n + cols - 1) / cols;
  if (row_tiles > 65535 || col_tiles > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(__nv_bfloat16) * kMmaStages * (BM + kMmaWeightRows) * kMmaPitch;
  auto kernel = moe_gemm_mma_kernel<GATED, BM>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  return (int)launch_chain(kernel, dim3((unsigned)col_tiles, (unsigned)row_tiles), dim3(256), smem, stream, dim3(1, 1, 1), p);
}

// ---------------------------------------------------------------------------------------------------------
// The same products when an expert has a handful of rows (decode steps): nothing is reused enough to stage, so a
// warp streams the weight rows of its features straight from global memory in 16-byte pieces and multiplies them
// with up to four of the expert's rows at a time (their pieces come from L1).  A block per (32 features, expert);
// an expert without rows costs a look at two integers.  bfloat16, k a multiple of eight.
namespace {
constexpr int kGemvRows = 4, kGemvFeatures = 32, kGemvWarps = 8;

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
}  // namespace

template <bool GATED>
__global__ void __launch_bounds__(kGemvWarps * 32) moe_gemv_kernel(MoeGemmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int expert = blockIdx.y;
  const int begin = p.offsets[expert], rows = p.offsets[expert + 1] - begin;
  if (rows <= 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int K = p.k, N = p.n, chunks = K / 8;
  const __nv_bfloat16* a = (const __nv_bfloat16*)p.a;
  const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (int64_t)expert * (GATED ? 2 : 1) * N * K;
  constexpr int kPerWarp = kGemvFeatures / kGemvWarps;
  for (int r0 = 0; r0 < rows; r0 += kGemvRows) {
    const int count = min(kGemvRows, rows - r0);
    const uint4* x[kGemvRows];
    int pair[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const int sorted = begin + r0 + min(r, count - 1);        // rows beyond the group repeat its last one, unused
      pair[r] = p.order[sorted];
      const int64_t src = GATED ? (int64_t)(pair[r] / p.top) : (int64_t)sorted;
      x[r] = reinterpret_cast<const uint4*>(a + src * K);
    }
    for (int f = 0; f < kPerWarp; ++f) {
      const int feature = blockIdx.x * kGemvFeatures + warp * kPerWarp + f;
      if (feature >= N) break;                                    // the same for the whole warp
      const uint4* wg = reinterpret_cast<const uint4*>(w + (int64_t)feature * K);
      const uint4* wu = GATED ? reinterpret_cast<const uint4*>(w + (int64_t)(N + feature) * K) : wg;
      float acc[GATED ? 2 : 1][kGemvRows] = {};
#pragma unroll 2
      for (int c = lane; c < chunks; c += 32) {
        float g[8], u[8];
        unpack8(wg[c], g);
        if (GATED) unpack8(wu[c], u);
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
          float v[8];
          unpack8(x[r][c], v);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            acc[0][r] = fmaf(g[i], v[i], acc[0][r]);
            if (GATED) acc[GATED ? 1 : 0][r] = fmaf(u[i], v[i], acc[GATED ? 1 : 0][r]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        acc[0][r] = warp_sum(acc[0][r]);
        if (GATED) acc[GATED ? 1 : 0][r] = warp_sum(acc[GATED ? 1 : 0][r]);
      }
      if (lane < count) {
        float first = 0.f, second = 0.f;
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
          if (r == lane) {
            first = acc[0][r];
            second = acc[GATED ? 1 : 0][r];
          }
        }
        if (GATED) {
          const float g = fminf(first, p.limit);
          const float u = fminf(fmaxf(second, -p.limit), p.limit);
          ((__nv_bfloat16*)p.out)[(int64_t)(begin + r0 + lane) * N + feature] =
              __float2bfloat16_rn(g / (1.f + expf(-p.slope * g)) * (u + p.up_offset));
        } else {
          int mine = pair[0];
#pragma unroll
          for (int r = 1; r < kGemvRows; ++r)
            if (r == lane) mine = pair[r];
          ((float*)p.out)[(int64_t)mine * N + feature] = p.weights[mine] * first;
        }
      }
    }
  }
}

int launch_moe_gemm(const MoeGemmParams& p, bool gated, cudaStream_t stream) {
  if (p.pairs == 0) return 0;
  if (p.experts <= 0 || p.experts > kMoeMaxExperts || p.k <= 0 || p.n <= 0 || p.top <= 0) return (int)cudaErrorInvalidValue;
  // 0: by size; 1: float arithmetic; 2: mma.sync tiles; 3: the few-rows form
  const bool tensor_ok = moe_gemm_takes_mma(p);
  if ((p.force_plain == 2 || p.force_plain == 3) && !tensor_ok) return (int)cudaErrorInvalidValue;
  if (p.force_plain == 3 || (p.force_plain == 0 && tensor_ok && gated && p.pairs <= kMoeFewRowPairs)) {
    const int64_t col_tiles = (p.n + kGemvFeatures - 1) / kGemvFeatures;
    if (col_tiles > 0x7fffffffLL || p.experts > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)col_tiles, (unsigned)p.experts);
    if (gated) return (int)launch_chain(moe_gemv_kernel<true>, grid, dim3(kGemvWarps * 32), 0, stream, dim3(1, 1, 1), p);
    return (int)launch_chain(moe_gemv_kernel<false>, grid, dim3(kGemvWarps * 32), 0, stream, dim3(1, 1, 1), p);
  }
  if (tensor_ok && p.force_plain != 1) {
    // tiles of 128 rows where the experts' runs are long enough to fill them.  Measured (gated / down product, us):
    // 256 rows an expert 244 / 142 against 234 / 138 with tiles of 64; 128 rows 669 / 388 against 652 / 371; 512 rows
    // 1,937 / 1,203 against 2,141 / 1,268.  AKV_MOE_TALL_ROWS moves the threshold (a measurement switch).
    static const int64_t tall_rows = [] {
      const char* v = getenv("AKV_MOE_TALL_ROWS");
      return v != nullptr && v[0] != '\0' ? (int64_t)atoll(v) : (int64_t)384;
    }();
    const bool tall = p.pairs >= tall_rows * p.experts;
    if (gated) return tall ? launch_moe_mma<true, 128>(p, stream) : launch_moe_mma<true, 64>(p, stream);
    return tall ? launch_moe_mma<false, 128>(p, stream) : launch_moe_mma<false, 64>(p, stream);
  }
  // every expert may end in a tile that is not full
  const int64_t row_tiles = p.pairs / kTileRows + (p.pairs < p.experts ? p.pairs : p.experts);
  const int64_t col_tiles = (p.n + kTileCols - 1) / kTileCols;
  if (row_tiles > 65535 || col_tiles > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const dim3 grid((unsigned)col_tiles, (unsigned)row_tiles);
  if (p.dtype == kBFloat16) {
    if (gated) return (int)launch_chain(moe_gemm_kernel<__nv_bfloat16, true>, grid, dim3(kGemmThreads), 0, stream, dim3(1, 1, 1), p);
    return (int)launch_chain(moe_gemm_kernel<__nv_bfloat16, false>, grid, dim3(kGemmThreads), 0, stream, dim3(1, 1, 1), p);
  }
  if (gated) return (int)launch_chain(moe_gemm_kernel<float, true>, grid, dim3(kGemmThreads), 0, stream, dim3(1, 1, 1), p);
  return (int)launch_chain(moe_gemm_kernel<float, false>, grid, dim3(kGemmThreads), 0, stream, dim3(1, 1, 1), p);
}

template <typename TS>
__global__ void moe_combine_kernel(const float* __restrict__ parts, const TS* __restrict__ shared,
                                   float* __restrict__ out, int64_t total, int64_t width, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t token = idx / width, c = idx - token * width;
  float sum = 0.f;
  for (int s = 0; s < top; ++s) sum += parts[(token * top + s) * width + c];
  if (shared != nullptr) sum += to_float<TS>(shared[idx]);
  out[idx] = sum;
}

int launch_moe_combine(const float* parts, const void* shared, int shared_dtype, float* out, int64_t num_tokens,
                       int64_t width, int top, cudaStream_t stream) {
  const int64_t total = num_tokens * width;
  if (total == 0) return 0;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (shared != nullptr && shared_dtype == kBFloat16)
    return (int)launch_chain(moe_combine_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                             dim3(1, 1, 1), parts, (const __nv_bfloat16*)shared, out, total, width, top);
  return (int)launch_chain(moe_combine_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                           parts, (const float*)shared, out, total, width, top);
}

}  // namespace akv
