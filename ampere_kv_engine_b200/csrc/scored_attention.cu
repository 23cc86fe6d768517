// Paged causal attention whose scores are reshaped before the softmax and whose keys and values
// need not have the same width: the general kernel (float arithmetic on CUDA cores, float32 or
// bfloat16 pages) for mixers that the plain kernel of paged_attention.cu does not describe.
//
//   score(i, j) = q_i . k_j * scale
//   cap  > 0:     score <- cap * tanh(score / cap)
//   slopes:       score <- score - slopes[h] * (i - j)            (a bias that grows with the distance)
//   visible(i,j): j <= i, j > i - window (window > 0), floor(j / chunk) == floor(i / chunk) (chunk > 0);
//                 with keep_first > 0 the keys j < keep_first stay visible behind a window (at their true positions)
//   out_i = softmax over the visible j of score(i, j) applied to v_j, times gate[i, h] (if given), times out_scale
//   sigmoid_weights: the weight of a visible key is sigmoid(score + head_bias[h]) instead, not normalised over keys
//
// Keys are rows of `head_dim` elements, values rows of `v_dim`; both live in paged storage
// [pages, kv heads, page size, row stride] whose row strides are given, so a value may be a
// prefix of the key row it shares (a cache that keeps one compressed latent per token, read as
// key and, in its first v_dim elements, as value).
//
// Work split, as in the plain general kernel: a warp owns (tile, kv head, R rows of the tile,
// key split); rows are (token, head-in-group) pairs.  It walks its key range 32 keys at a time,
// lane = key for the scores (the key row is read once for all R rows, q comes from shared
// memory), lane = value dims for P.V.  With several splits the partial (acc, max, sum) go to a
// workspace and a second kernel merges them in split order.
#include "common.cuh"
#include "launchers.h"

#include <math_constants.h>

namespace akv {

constexpr int kScoredWarps = 4;

template <typename T, int DC, int R>
__global__ void __launch_bounds__(kScoredWarps * 32)
scored_attention_kernel(ScoredAttentionParams sp, int row_groups, int64_t total_items, int vec) {
  const PagedAttentionParams& p = sp.base;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t item = (int64_t)blockIdx.x * kScoredWarps + warp;
  if (item >= total_items) return;
  const int D = p.head_dim, DV = sp.v_dim, NH = p.num_heads, NKV = p.num_kv_heads, G = NH / NKV, P = p.page_size;
  const int rg = (int)(item % row_groups);
  const int kvh = (int)((item / row_groups) % NKV);
  const int split = (int)((item / ((int64_t)row_groups * NKV)) % p.num_splits);
  const int tile = (int)(item / ((int64_t)row_groups * NKV * p.num_splits));

  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int nq = p.tile_nq[tile];
  const int rows_in_tile = nq * G;
  const int row0 = rg * R;
  if (row0 >= rows_in_tile) return;
  const int nrows = min(R, rows_in_tile - row0);
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  const int tile_pos = ctx - q_len + (q0 - seq_q0);      // absolute position of the tile's first token

  extern __shared__ float smem[];
  float* qs = smem + warp * (R * D + R * 32);
  float* ps = qs + R * D;

  const T* q = (const T*)p.q;
  for (int idx = lane; idx < R * D; idx += 32) {
    const int r = idx / D, d = idx - r * D;
    float v = 0.f;
    if (r < nrows) {
      const int rr = row0 + r;
      const int64_t token = q0 + rr / G;
      const int head = kvh * G + rr % G;
      v = to_float<T>(q[(token * NH + head) * (int64_t)D + d]) * p.scale;
    }
    qs[idx] = v;
  }
  __syncwarp();

  int pos[R], first_key[R];
  float slope[R], bias[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const bool live = r < nrows;
    pos[r] = live ? tile_pos + (row0 + r) / G : -1;
    int first = 0;
    if (live && p.window > 0) first = max(first, pos[r] - p.window + 1);
    if (live && sp.chunk > 0) first = max(first, pos[r] / sp.chunk * sp.chunk);
    first_key[r] = first;
    slope[r] = (live && sp.slopes != nullptr) ? sp.slopes[kvh * G + (row0 + r) % G] : 0.f;
    bias[r] = (live && sp.head_bias != nullptr) ? sp.head_bias[kvh * G + (row0 + r) % G] : 0.f;
  }
  const int pos_last = tile_pos + (row0 + nrows - 1) / G;
  const int lo_item = first_key[0];        // rows are in position order: the first row's first key is the lowest
  const int hi_item = pos_last + 1;
  // The keys this item walks are [0, kept) and [lo_item, hi_item): the first keys a window keeps, then the window.
  // They are numbered in one run ("walk index" w: key = w below kept, lo_item + w - kept from there on), which the
  // splits cut; without kept keys the walk index is the key less lo_item.
  const int kept = min(sp.keep_first, lo_item);
  int per = (max(hi_item - lo_item, 0) + kept + p.num_splits - 1) / p.num_splits;
  per = (per + 31) & ~31;
  const int start = split * per;
  const int end = min(hi_item - lo_item + kept, start + per);
  const int jump = lo_item - kept;          // added to a walk index from `kept` on
  const float inv_cap = sp.softcap > 0.f ? 1.f / sp.softcap : 0.f;

  float m[R], l[R], acc[R][DC];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -CUDART_INF_F;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  }

  const T* k_cache = (const T*)p.k_cache;
  const T* v_cache = (const T*)p.v_cache;
  const int32_t* table = p.block_table + (int64_t)seq * p.table_width;

  for (int kb = start; kb < end; kb += 32) {
    const int walk = kb + lane;
    const int key = walk < kept ? walk : walk + jump;
    bool kvalid = walk < end;
    int page = 0;
    if (kvalid) {
      const int logical = key / P;
      page = logical < p.table_width ? table[logical] : -1;
      if (page < 0 || page >= p.num_pages) {
        set_status(p.status, kBadPage);
        kvalid = false;
        page = 0;
      }
    }
    const int off = key % P;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) s[r] = 0.f;
    if (kvalid) {
      const T* kptr = k_cache + (((int64_t)page * NKV + kvh) * P + off) * sp.k_row_stride;
      if (vec) {
#pragma unroll 2
        for (int d0 = 0; d0 < D; d0 += 8) {
          float kf[8];
          load8<T>(kptr + d0, kf);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float4 a = *reinterpret_cast<const float4*>(qs + r * D + d0);
            const float4 b = *reinterpret_cast<const float4*>(qs + r * D + d0 + 4);
            s[r] += a.x * kf[0] + a.y * kf[1] + a.z * kf[2] + a.w * kf[3] + b.x * kf[4] + b.y * kf[5] +
                    b.z * kf[6] + b.w * kf[7];
          }
        }
      } else {
        for (int d = 0; d < D; ++d) {
          const float kf = to_float<T>(kptr[d]);
#pragma unroll
          for (int r = 0; r < R; ++r) s[r] += qs[r * D + d] * kf;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool visible = kvalid && key <= pos[r] && (key >= first_key[r] || key < sp.keep_first);
      float sr = s[r];
      if (sp.softcap > 0.f) sr = sp.softcap * tanhf(sr * inv_cap);
      sr -= slope[r] * (float)(pos[r] - key);
      if (sp.sigmoid_weights) {
        // no softmax: every visible key weighs sigmoid(score + bias of the head), whatever the other keys do
        const float pr = visible ? 1.f / (1.f + expf(-(sr + bias[r]))) : 0.f;
        ps[r * 32 + lane] = pr;
        continue;
      }
      sr = visible ? sr : -CUDART_INF_F;
      const float m_new = fmaxf(m[r], warp_max(sr));
      const float alpha = (m_new == -CUDART_INF_F) ? 1.f : expf(m[r] - m_new);
      const float pr = visible ? expf(sr - m_new) : 0.f;
      l[r] = l[r] * alpha + pr;
      m[r] = m_new;
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] *= alpha;
      ps[r * 32 + lane] = pr;
    }
    __syncwarp();
    const int nk = min(32, end - kb);
    for (int j = 0; j < nk; ++j) {
      const int pj = __shfl_sync(0xffffffffu, page, j);
      const int offj = __shfl_sync(0xffffffffu, off, j);
      const T* vptr = v_cache + (((int64_t)pj * NKV + kvh) * P + offj) * sp.v_row_stride;
      float vv[DC];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = c * 32 + lane;
        vv[c] = d < DV ? to_float<T>(vptr[d]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float pr = ps[r * 32 + j];
#pragma unroll
        for (int c = 0; c < DC; ++c) acc[r][c] += pr * vv[c];
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (r >= nrows) continue;
    const float total = warp_sum(l[r]);
    const int rr = row0 + r;
    const int64_t token = q0 + rr / G;
    const int head = kvh * G + rr % G;
    const int64_t row = token * NH + head;
    if (p.num_splits == 1) {
      T* o = (T*)p.out + row * (int64_t)DV;
      float inv = sp.sigmoid_weights ? 1.f : (total > 0.f ? 1.f / total : 0.f);
      if (sp.gate != nullptr) inv *= sp.gate[row];
      inv *= sp.out_scale;
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = c * 32 + lane;
        if (d < DV) o[d] = from_float<T>(acc[r][c] * inv);
      }
    } else {
      float* part = p.partials + (row * p.num_splits + split) * (int64_t)(DV + 2);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = c * 32 + lane;
        if (d < DV) part[d] = acc[r][c];
      }
      if (lane == 0) {
        part[DV] = m[r];
        part[DV + 1] = total;
      }
    }
  }
}

// out[row] = gate[row] * sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) l_s, splits taken in order; one block per
// (tile, row of the tile, q-head), so only the rows of the call's tiles are written.  The splits' weights are worked
// out once per block (thread s takes split s) and left in shared memory; after that a thread only adds up its dims.
constexpr int kMergeSplits = 64;       // most key splits of a call
template <typename T>
__global__ void scored_merge_kernel(const float* __restrict__ partials, T* __restrict__ out,
                                    const int32_t* __restrict__ tile_q0, const int32_t* __restrict__ tile_nq,
                                    const float* __restrict__ gate, int q_tile, int num_heads, int num_splits,
                                    int v_dim, int plain_sum, float out_scale) {
  __shared__ float weight[kMergeSplits];
  __shared__ float scale_out;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t per_tile = (int64_t)q_tile * num_heads;
  const int64_t tile = blockIdx.x / per_tile;
  const int in_tile = (int)(blockIdx.x - tile * per_tile);
  const int r = in_tile / num_heads, head = in_tile - r * num_heads;
  if (r >= tile_nq[tile]) return;
  const int64_t row = ((int64_t)tile_q0[tile] + r) * num_heads + head;
  const float* base = partials + row * num_splits * (int64_t)(v_dim + 2);
  if (plain_sum) {
    // weights that were never normalised over the keys: the splits' sums are added as they are
    for (int s = threadIdx.x; s < num_splits; s += blockDim.x) weight[s] = 1.f;
    if (threadIdx.x == 0) scale_out = (gate != nullptr ? gate[row] : 1.f) * out_scale;
  } else if (threadIdx.x < 32) {
    // one warp: the maximum over the splits, each split's weight, the weighted sum of the row sums in split order
    float ms[(kMergeSplits + 31) / 32], ls[(kMergeSplits + 31) / 32];
    float m = -CUDART_INF_F;
#pragma unroll
    for (int c = 0; c < (kMergeSplits + 31) / 32; ++c) {
      const int s = c * 32 + threadIdx.x;
      ms[c] = -CUDART_INF_F;
      ls[c] = 0.f;
      if (s < num_splits) {
        const float* part = base + (int64_t)s * (v_dim + 2);
        ls[c] = part[v_dim + 1];
        if (ls[c] > 0.f) ms[c] = part[v_dim];
      }
      m = fmaxf(m, ms[c]);
    }
    m = warp_max(m);
#pragma unroll
    for (int c = 0; c < (kMergeSplits + 31) / 32; ++c) {
      const int s = c * 32 + threadIdx.x;
      if (s < num_splits) weight[s] = ls[c] > 0.f ? expf(ms[c] - m) : 0.f;
    }
    __syncwarp();
    if (threadIdx.x == 0) {
      float den = 0.f;
      for (int s = 0; s < num_splits; ++s) den += weight[s] * base[(int64_t)s * (v_dim + 2) + v_dim + 1];
      scale_out = den > 0.f ? (gate != nullptr ? gate[row] : 1.f) * out_scale / den : 0.f;
    }
  }
  __syncthreads();
  const float g = scale_out;
  for (int d = threadIdx.x; d < v_dim; d += blockDim.x) {
    float num = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = weight[s];
      if (w > 0.f) num += w * base[(int64_t)s * (v_dim + 2) + d];
    }
    out[row * v_dim + d] = from_float<T>(g * num);
  }
}

template <typename T>
static int launch_scored_merge(const ScoredAttentionParams& sp, cudaStream_t stream) {
  const PagedAttentionParams& p = sp.base;
  const int64_t merge_blocks = (int64_t)p.num_tiles * p.q_tile * p.num_heads;
  if (merge_blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const int threads = sp.v_dim <= 32 ? 32 : (sp.v_dim <= 64 ? 64 : 128);
  return (int)launch_chain(scored_merge_kernel<T>, dim3((unsigned)merge_blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                           (const float*)p.partials, (T*)p.out, p.tile_q0, p.tile_nq, sp.gate, p.q_tile, p.num_heads,
                           p.num_splits, sp.v_dim, sp.sigmoid_weights, sp.out_scale);
}

template <typename T, int DC, int R>
static int launch_rows(const ScoredAttentionParams& sp, cudaStream_t stream) {
  const PagedAttentionParams& p = sp.base;
  const int G = p.num_heads / p.num_kv_heads;
  const int row_groups = (p.q_tile * G + R - 1) / R;
  const int64_t total = (int64_t)p.num_tiles * p.num_kv_heads * row_groups * p.num_splits;
  const int64_t blocks = (total + kScoredWarps - 1) / kScoredWarps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)kScoredWarps * (R * p.head_dim + R * 32) * sizeof(float);
  auto kernel = scored_attention_kernel<T, DC, R>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  // 16-byte loads of the key rows and of q in shared memory need rows that start on such a boundary
  const int per16 = 16 / (int)sizeof(T);
  const int vec = (p.head_dim % 8 == 0 && sp.k_row_stride % per16 == 0 &&
                   reinterpret_cast<uintptr_t>(p.k_cache) % 16 == 0) ? 1 : 0;
  cudaError_t err = launch_chain(kernel, dim3((unsigned)blocks), dim3(kScoredWarps * 32), smem, stream, dim3(1, 1, 1), sp,
                                 row_groups, total, vec);
  if (err != cudaSuccess) return (int)err;
  return p.num_splits > 1 ? launch_scored_merge<T>(sp, stream) : 0;
}

template <typename T>
static int launch_scored_typed(const ScoredAttentionParams& sp, cudaStream_t stream) {
  const int dc = (sp.v_dim + 31) / 32;
#define AKV_SCORED(DCV, RV) \
  case DCV: return launch_rows<T, DCV, RV>(sp, stream);
  switch (dc) {
    AKV_SCORED(1, 8) AKV_SCORED(2, 8) AKV_SCORED(3, 8) AKV_SCORED(4, 8)
    AKV_SCORED(5, 8) AKV_SCORED(6, 8) AKV_SCORED(7, 8) AKV_SCORED(8, 8)
    default: break;
  }
#undef AKV_SCORED
  // wide values (a compressed latent read as value): fewer rows per warp keep the accumulators in registers
  if (dc <= 12) return launch_rows<T, 12, 4>(sp, stream);
  if (dc <= 16) return launch_rows<T, 16, 4>(sp, stream);
  return (int)cudaErrorInvalidValue;
}

int launch_scored_attention(const ScoredAttentionParams& sp, cudaStream_t stream) {
  const PagedAttentionParams& p = sp.base;
  if (p.num_tiles == 0 || p.num_tokens == 0) return 0;
  if (p.head_dim < 1 || sp.v_dim < 1 || sp.v_dim > 512 || p.num_heads % p.num_kv_heads || p.num_splits < 1 ||
      p.num_splits > kMergeSplits ||
      sp.k_row_stride < p.head_dim || sp.v_row_stride < sp.v_dim || sp.chunk < 0 || sp.softcap < 0.f ||
      sp.keep_first < 0 || (sp.keep_first > 0 && (p.window <= 0 || sp.chunk > 0)))
    return (int)cudaErrorInvalidValue;
  // kept first keys, weights without a softmax and an output factor: the tcgen05 prompt kernel, the tensor-core
  // kernel for single tokens and the general kernel
  if (p.kernel != 1 && p.q_tile > 1 && attention_tcgen05_scored_supported(sp))
    return launch_attention_tcgen05_scored(sp, stream);
  if (p.kernel != 1 && p.q_tile == 1 && attention_tc_scored_supported(sp)) return launch_attention_tc_scored(sp, stream);
  const bool general_only = sp.keep_first > 0 || sp.sigmoid_weights || sp.head_bias != nullptr || sp.out_scale != 1.f;
  if (general_only)
    return p.dtype == kBFloat16 ? launch_scored_typed<__nv_bfloat16>(sp, stream) : launch_scored_typed<float>(sp, stream);
  if (p.kernel != 1 && scored_attention_mma_supported(sp)) {
    const int err = launch_scored_attention_mma(sp, stream);
    if (err != 0) return err;
    return p.num_splits > 1 ? launch_scored_merge<__nv_bfloat16>(sp, stream) : 0;
  }
  return p.dtype == kBFloat16 ? launch_scored_typed<__nv_bfloat16>(sp, stream)
                              : launch_scored_typed<float>(sp, stream);
}

}  // namespace akv
