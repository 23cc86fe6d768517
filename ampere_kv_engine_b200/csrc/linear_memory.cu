// Linear attention with a matrix memory per head that decays row by row, carried from token to token:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t            S: [dim, v_dim] float32 per (request, head)
//
// Two ways to fill a_t and k_t from one product's columns:
//   kGatedWrite      a = f, k = 1 - f with f = lower + (1 - lower) * sigmoid(x_f + bias)  (a row keeps f of itself and
//                    takes 1 - f of the value), q = silu(x_q), v = x_v
//   kConstantDecay   a = decay[head] for every row, k = silu(x_k), q = silu(x_q), v = silu(x_v)
//   kPlainDecay      a = decay[head]; q, k and v are taken as they are: a kernel before the scan has prepared them
//                    (a rotation by position, a scale) and x is its float32 output
//   kTokenDecay      a = x[decay_off + head] of the token (a scalar per head and token); q, k and v as they are;
//                    qk_group heads in a row share one q and one k (a state-space mixer's groups)
// Everything after the product is float32: gates, activations, the memory and both products with it.
//
// Work split: a block owns (sequence, head, 32 value columns) for the whole step; a thread holds ROWS rows of one
// column of S in registers, `lanes` threads a column, so writing a token is thread-local.  Tokens are staged through
// two shared-memory buffers CHUNK at a time, and there is one block barrier per chunk.
//   Decode form (steps of a token or two per sequence): a column's threads are neighbouring lanes and add up their
//   parts of a token's output with shuffles; every thread stages its share of the next tokens itself (loads,
//   activations, gates).
//   Prompt form (everything else): a kernel of its own first writes every token's q, a-or-k and v after activations
//   and gates as float32 (once per token, not once per block of a head's value slices).  In the scan a warp holds
//   the same rows of all 32 columns, so its reads of q and of the gates are broadcasts; it leaves its part of every
//   token's output in shared memory, and when the chunk is walked the walking warps add the parts up, a thread per
//   (token, column).  Further warps do nothing but copy the next chunk from the float32 scratch, asynchronously.
// S moves between registers and the request's state slot in an order of its own ([head][slice][row in lane][column]
// [lane]), the same in both forms, so that the loads and stores of a decode step are coalesced.
// Tokens are walked one by one whatever the step holds: the memory after a token does not depend on how the tokens
// were cut into steps, and a token's output only in the order in which `lanes` parts are added.
//
// A second kernel norms what the scan read out: RMS over groups of columns (a head, or all heads together), a
// weight, a constant factor, and optionally a sigmoid gate from further columns of the product.
#include <algorithm>

#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

constexpr int kScanColumns = 32;     // value columns per block
constexpr int kScanProducers = 128;  // threads that only copy tokens into shared memory, in the prompt form
constexpr int kScanBatch = 8;        // tokens whose loads a staging thread has in flight at a time (decode form)

// The quotient is a reciprocal and a product (two units in the last place), inline: the staging threads work on many
// entries at a time and a division's subroutine would put them in a row.  The denominator is at least one; where
// expf overflows the quotient is zero.
__device__ __forceinline__ float sigmoid_f(float z) { return __fdividef(1.f, 1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return __fdividef(z, 1.f + expf(-z)); }

// floats between two lanes' rows of q (or of a) in shared memory: padded where several lanes share a column, so that
// the float4 reads of a group's lanes fall into different banks
__host__ __device__ constexpr int scan_pitch(int rows, int lanes) { return lanes > 1 ? rows + 4 : rows; }

// staged entries per staging thread and token: [q (dim) | f or k (dim) | v (32)] over 32 * lanes threads (dim at most
// rows * lanes), or over the producers (dim at most 8 * rows)
__host__ __device__ constexpr int scan_rounds(int rows, int producers) {
  return producers > 0 ? (2 * 8 * rows + kScanColumns + producers - 1) / producers : 3;
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* global) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(global)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* global) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(global)
               : "memory");
}

// act[t] = [q (NH * D) | a or k (NH * D) | v (NH * DV)] of token t after activations and gates, float32: what every
// block of a head's value slices would otherwise work out again for itself while it stages a prompt's tokens.
template <typename T, int MODE>
__global__ void linear_prep_kernel(LinearScanParams p, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int qk = p.num_heads * p.head_dim;
  const int64_t t = blockIdx.x;                        // a block row per token, blockIdx.y over its columns
  const T* row = (const T*)p.x + t * p.x_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float y;
    if (c < qk) {
      y = silu_f(to_float<T>(row[p.q_off + c]));
    } else if (c < 2 * qk) {
      const int ch = c - qk;
      const float z = to_float<T>(row[p.k_off + ch]);
      if (MODE == kGatedWrite) {
        const float low = p.lower[ch];
        y = low + (1.f - low) * sigmoid_f(z + (p.gate_bias != nullptr ? p.gate_bias[ch] : 0.f));
      } else {
        y = silu_f(z);
      }
    } else {
      const float z = to_float<T>(row[p.v_off + c - 2 * qk]);
      y = MODE == kGatedWrite ? z : silu_f(z);
    }
    p.act[t * width + c] = y;
  }
}

// PRODUCERS == 0: the decode form.  PRODUCERS > 0: the prompt form with that many further threads that only copy
// the next chunk from p.act into shared memory beside the walk of the current one.
template <typename T, int MODE, int ROWS, int CHUNK, int PRODUCERS>
__global__ void __launch_bounds__(256 + PRODUCERS)
linear_scan_kernel(LinearScanParams p, int lanes, int slices) {
  constexpr int kRounds = scan_rounds(ROWS, PRODUCERS);
  constexpr bool kPrepared = MODE == kPlainDecay || MODE == kTokenDecay;     // no activation, float32 input
  constexpr int kExtra = MODE == kTokenDecay ? 4 : 0;                        // a token's decay, behind its v
  constexpr int kBatch = CHUNK < kScanBatch ? CHUNK : (ROWS >= 32 ? kScanBatch / 2 : kScanBatch);
  pdl_launch_dependents();
  pdl_wait();
  const int H = p.num_heads, D = p.head_dim, DV = p.v_dim;
  const int slice = blockIdx.x % slices;
  const int head = (blockIdx.x / slices) % H;
  const int seq = blockIdx.x / (slices * H);
  const int slot = p.state_slots[seq];
  const int t0 = p.cu_q[seq];
  const int n = p.cu_q[seq + 1] - t0;
  if (slot < 0 || n <= 0) return;                      // a padded sequence: nothing is read or written
  const int tid = threadIdx.x;
  const int threads = kScanColumns * lanes;            // threads that own rows of S
  const bool walker = tid < threads;
  const bool stager = PRODUCERS > 0 ? !walker : true;
  const int stage_id = PRODUCERS > 0 ? tid - threads : tid;
  const int stagers = PRODUCERS > 0 ? PRODUCERS : threads;
  // which rows (sub) of which column (col) of S a thread owns.  Decode form: a column's lanes are neighbours, so that
  // they can add up with shuffles.  Prompt form: a warp holds the same rows of all 32 columns, so that its reads of
  // q and of the gates are one broadcast each and no shuffle stands between two tokens.
  const int sub = PRODUCERS > 0 ? tid / kScanColumns : tid % lanes;
  const int col = PRODUCERS > 0 ? tid % kScanColumns : tid / lanes;
  const int j = slice * kScanColumns + col;
  const int pitch = scan_pitch(ROWS, lanes);
  const int vec = lanes * pitch;                       // floats of a token's q (or a) in shared memory
  const int per_token = 2 * vec + kScanColumns + kExtra;   // [q | a | v (| decay)]
  const int qk_head = head / p.qk_group;               // whose q and k this head reads
  const int per_buffer = CHUNK * per_token;

  extern __shared__ __align__(16) float smem[];

  float* mem = p.state + (int64_t)slot * p.state_stride +
               ((int64_t)head * slices + slice) * ROWS * (int64_t)threads + col * lanes + sub;
  float S[ROWS];
  if (walker) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) S[r] = mem[(int64_t)r * threads];
  }
  const float decay = (MODE == kConstantDecay || MODE == kPlainDecay) ? p.decay[head] : 0.f;

  // What a staging thread stages of every token: entry i = stage_id + round * stagers of [q (D) | f or k (D) | v (the
  // slice's columns)].  Its column of x, its place in a token's shared-memory row and its gate constants are worked
  // out once.
  const int mine_cols = min(kScanColumns, DV - slice * kScanColumns);
  const int fetch_per_token = 2 * D + mine_cols;
  const T* src[kRounds];
  int dst[kRounds], kind[kRounds];                     // kind 0: q, 1: f or k, 2: v, 3: the token's decay
  float low[kRounds], bias[kRounds];
  const T* x = (const T*)p.x + (int64_t)t0 * p.x_stride;
#pragma unroll
  for (int r = 0; r < kRounds; ++r) {
    const int i = stage_id + r * stagers;
    src[r] = nullptr;
    dst[r] = kind[r] = 0;
    low[r] = bias[r] = 0.f;
    if (PRODUCERS == 0 && i < fetch_per_token) {
      if (i < D) {
        src[r] = x + p.q_off + qk_head * D + i;
        dst[r] = i / ROWS * pitch + i % ROWS;
      } else if (i < 2 * D) {
        const int d = i - D, ch = qk_head * D + d;
        src[r] = x + p.k_off + ch;
        dst[r] = vec + d / ROWS * pitch + d % ROWS;
        kind[r] = 1;
        if (MODE == kGatedWrite) {
          low[r] = p.lower[ch];
          bias[r] = p.gate_bias != nullptr ? p.gate_bias[ch] : 0.f;
        }
      } else {
        src[r] = x + p.v_off + head * DV + slice * kScanColumns + (i - 2 * D);
        dst[r] = 2 * vec + (i - 2 * D);
        kind[r] = 2;
      }
    } else if (PRODUCERS == 0 && MODE == kTokenDecay && i == fetch_per_token) {
      src[r] = x + p.decay_off + head;
      dst[r] = 2 * vec + kScanColumns;
      kind[r] = 3;
    }
  }
  // tokens first .. first + count - 1 of the sequence into a buffer: kBatch tokens' loads at a time, then their
  // activations and gates
  auto stage = [&](float* buffer, int first, int count) {
    for (int tb = 0; tb < count; tb += kBatch) {
      T raw[kRounds][kBatch];
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
#pragma unroll
        for (int t = 0; t < kBatch; ++t)
          if (src[r] != nullptr && tb + t < count) raw[r][t] = src[r][(int64_t)(first + tb + t) * p.x_stride];
      }
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        if (src[r] == nullptr) continue;
#pragma unroll
        for (int t = 0; t < kBatch; ++t) {
          if (tb + t >= count) break;
          const float z = to_float<T>(raw[r][t]);
          float y;
          if (kPrepared) y = z;
          else if (kind[r] == 0) y = silu_f(z);
          else if (kind[r] == 1) y = MODE == kGatedWrite ? low[r] + (1.f - low[r]) * sigmoid_f(z + bias[r]) : silu_f(z);
          else y = MODE == kGatedWrite ? z : silu_f(z);
          buffer[(tb + t) * per_token + dst[r]] = y;
        }
      }
    }
  };
  // the same from the scratch that the preparing kernel filled (prompt form): asynchronous copies of 16 bytes where
  // the widths allow it, of 4 otherwise, all of a chunk in flight at once
  auto stage_copy = [&](float* buffer, int first, int count) {
    const int64_t width = p.act_stride;
    const bool wide_copy = D % 4 == 0 && DV % 4 == 0 && p.act_aligned;
    const int step = wide_copy ? 4 : 1;
    const int per = fetch_per_token / step;
    const float* base = p.act + (int64_t)(t0 + first) * width;
    for (int e = stage_id; e < count * per; e += stagers) {
      const int t = e / per, i = (e % per) * step;
      const float* from = base + (int64_t)t * width;
      float* to = buffer + t * per_token;
      if (i < D) {
        from += p.act_q_off + qk_head * D + i;
        to += i / ROWS * pitch + i % ROWS;
      } else if (i < 2 * D) {
        from += p.act_k_off + qk_head * D + (i - D);
        to += vec + (i - D) / ROWS * pitch + (i - D) % ROWS;
      } else {
        from += p.act_v_off + head * DV + slice * kScanColumns + (i - 2 * D);
        to += 2 * vec + (i - 2 * D);
      }
      if (wide_copy) cp_async_16(to, from);
      else cp_async_4(to, from);
    }
    if (MODE == kTokenDecay) {
      for (int t = stage_id; t < count; t += stagers)
        cp_async_4(buffer + t * per_token + 2 * vec + kScanColumns, base + (int64_t)t * width + p.decay_off + head);
    }
    cp_async_wait_all();
  };
  // a token's q, a and v applied to this thread's rows of S; returns its part of the token's output
  auto apply_loaded = [&](const float4 (&qs)[ROWS / 4], const float4 (&as)[ROWS / 4], float v, float decay) -> float {
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int r4 = 0; r4 < ROWS / 4; ++r4) {
      const float4 q = qs[r4], a = as[r4];
      const int r = r4 * 4;
      if (MODE == kGatedWrite) {
        // f S + (1 - f) v as v + f (S - v): two operations per entry
        S[r] = fmaf(a.x, S[r] - v, v);
        S[r + 1] = fmaf(a.y, S[r + 1] - v, v);
        S[r + 2] = fmaf(a.z, S[r + 2] - v, v);
        S[r + 3] = fmaf(a.w, S[r + 3] - v, v);
      } else {
        S[r] = fmaf(a.x, v, decay * S[r]);
        S[r + 1] = fmaf(a.y, v, decay * S[r + 1]);
        S[r + 2] = fmaf(a.z, v, decay * S[r + 2]);
        S[r + 3] = fmaf(a.w, v, decay * S[r + 3]);
      }
      o0 = fmaf(S[r], q.x, o0);
      o1 = fmaf(S[r + 1], q.y, o1);
      o2 = fmaf(S[r + 2], q.z, o2);
      o3 = fmaf(S[r + 3], q.w, o3);
    }
    return (o0 + o1) + (o2 + o3);
  };
  // a token's row of [q | a | v] in shared memory into registers
  auto fetch = [&](const float* row, float4 (&qs)[ROWS / 4], float4 (&as)[ROWS / 4], float& v, float& d) {
    v = row[2 * vec + col];
    if (MODE == kTokenDecay) d = row[2 * vec + kScanColumns];
    const float4* q4 = reinterpret_cast<const float4*>(row + sub * pitch);
    const float4* a4 = reinterpret_cast<const float4*>(row + vec + sub * pitch);
#pragma unroll
    for (int r4 = 0; r4 < ROWS / 4; ++r4) {
      qs[r4] = q4[r4];
      as[r4] = a4[r4];
    }
  };
  auto apply = [&](const float* row) -> float {
    float4 qs[ROWS / 4], as[ROWS / 4];
    float v, d = decay;
    fetch(row, qs, as, v, d);
    return apply_loaded(qs, as, v, d);
  };
  const int wide = H * DV;
  // count tokens of a buffer in their order, decode form: the lanes that share a column add up their parts of a
  // token's output in three shuffle steps; o_row: this thread's column in the first token's output row
  auto walk = [&](const float* row, int count, float* o_row) {
#pragma unroll 2
    for (int t = 0; t < count; ++t, row += per_token, o_row += wide) {
      float o = apply(row);
#pragma unroll
      for (int w = 4; w > 0; w >>= 1) {                // at most eight lanes share a column
        const float other = __shfl_xor_sync(0xffffffffu, o, w);
        if (w < lanes) o += other;
      }
      if (sub == 0 && j < DV) *o_row = o;
    }
  };
  // the same, prompt form: a warp leaves its rows' part of every token's output in shared memory; when the chunk is
  // walked, the walking warps meet and add the parts up, a thread per (token, column), and store whole rows
  float* parts = smem + 2 * per_buffer;                // [CHUNK][lanes][32]
  auto walk_parts = [&](const float* row, int count, float* o_rows) {
#pragma unroll 2
    for (int t = 0; t < count; ++t, row += per_token) parts[(t * lanes + sub) * kScanColumns + col] = apply(row);
    asm volatile("bar.sync 2, %0;" ::"r"(threads) : "memory");
    for (int i = tid; i < count * kScanColumns; i += threads) {
      const int t = i / kScanColumns, c = i % kScanColumns;
      float o = parts[t * lanes * kScanColumns + c];
      for (int w = 1; w < lanes; ++w) o += parts[(t * lanes + w) * kScanColumns + c];
      if (slice * kScanColumns + c < DV) o_rows[(int64_t)t * wide + c] = o;
    }
  };
  // rows of S beyond the dim never change: q and k stay zero there, a forget gate one; value columns beyond the
  // width stay zero
  for (int i = tid; i < 2 * per_buffer; i += blockDim.x) {
    const int e = i % per_token;
    smem[i] = (MODE == kGatedWrite && e >= vec && e < 2 * vec) ? 1.f : 0.f;
  }
  __syncthreads();
  if (PRODUCERS > 0) {
    if (stager) stage_copy(smem, 0, min(CHUNK, n));
  } else {
    stage(smem, 0, min(CHUNK, n));
  }
  __syncthreads();
  // Every warp of the block meets one barrier per chunk, whatever it does in between.  With staging warps the two
  // roles run loops of their own (neither keeps the other's registers alive) and meet at a named barrier that counts
  // the whole block; a role is whole warps, and both loops have the same number of rounds.
  if (PRODUCERS > 0) {
    const unsigned everyone = blockDim.x;
    if (walker) {
      for (int c0 = 0; c0 < n; c0 += CHUNK) {
        walk_parts(smem + ((c0 / CHUNK) & 1) * per_buffer, min(CHUNK, n - c0),
                   p.out + (int64_t)(t0 + c0) * wide + head * DV + slice * kScanColumns);
        asm volatile("bar.sync 1, %0;" ::"r"(everyone) : "memory");
      }
    } else {
      for (int c0 = 0; c0 < n; c0 += CHUNK) {
        const int next = min(CHUNK, n - c0 - CHUNK);
        if (next > 0) stage_copy(smem + (((c0 / CHUNK) & 1) ^ 1) * per_buffer, c0 + CHUNK, next);
        asm volatile("bar.sync 1, %0;" ::"r"(everyone) : "memory");
      }
    }
  } else {
    for (int c0 = 0; c0 < n; c0 += CHUNK) {
      const int count = min(CHUNK, n - c0), next = min(CHUNK, n - c0 - CHUNK);
      const int cur = (c0 / CHUNK) & 1;
      walk(smem + cur * per_buffer, count, p.out + (int64_t)(t0 + c0) * wide + head * DV + j);
      if (next > 0) stage(smem + (cur ^ 1) * per_buffer, c0 + CHUNK, next);
      __syncthreads();
    }
  }
  if (walker) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) mem[(int64_t)r * threads] = S[r];
  }
}

// v[t, c]   = in[t, c] (+ skip_coef[c / skip_head] * skip[t, skip_off + c])  (* gate(x[t, gate_off + c]), gate_first)
// out[t, c] = v / sqrt(mean over c's group of v^2 + eps) * weight[c % weight_len] * factor
//             (* gate(x[t, gate_off + c]), unless gate_first);   gate: sigmoid or SiLU;   one block per (token, group)
template <typename T>
__global__ void group_norm_gate_kernel(GroupNormGateParams p) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int group = p.group, width = p.width;
  const int groups = width / group;
  const int64_t token = blockIdx.x / groups;
  const int g = blockIdx.x % groups;
  const float* src = p.in + token * width + (int64_t)g * group;
  const T* x = (const T*)p.x;
  auto gate = [&](int c) -> float {
    const float z = to_float<T>(x[token * p.x_stride + p.gate_off + c]);
    return p.gate_kind == 1 ? silu_f(z) : sigmoid_f(z);
  };
  auto value = [&](int i) -> float {
    const int c = g * group + i;
    float v = src[i];
    if (p.skip != nullptr) v = fmaf(p.skip_coef[c / p.skip_head], p.skip[token * p.skip_stride + p.skip_off + c], v);
    if (x != nullptr && p.gate_first) v *= gate(c);
    return v;
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const float v = value(i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = p.factor / sqrtf(ss / (float)group + p.eps);
  T* dst = (T*)p.out + token * width + (int64_t)g * group;
  for (int i = threadIdx.x; i < group; i += blockDim.x) {
    const int c = g * group + i;
    float y = value(i) * inv;
    if (p.weight != nullptr) y *= p.weight[c % p.weight_len];
    if (x != nullptr && !p.gate_first) y *= gate(c);
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

template <typename T, int MODE, int ROWS, int CHUNK, int PRODUCERS>
static int launch_scan_chunk(const LinearScanParams& p, int lanes, cudaStream_t stream) {
  const int slices = (p.v_dim + kScanColumns - 1) / kScanColumns;
  const int64_t blocks = (int64_t)p.num_seqs * p.num_heads * slices;
  const int stagers = PRODUCERS > 0 ? PRODUCERS : kScanColumns * lanes;
  if (blocks > 0x7fffffffLL || 2 * p.head_dim + kScanColumns + 1 > scan_rounds(ROWS, PRODUCERS) * stagers)
    return (int)cudaErrorInvalidValue;
  const size_t smem = (2 * (size_t)CHUNK * (2 * lanes * scan_pitch(ROWS, lanes) + kScanColumns +
                                            (MODE == kTokenDecay ? 4 : 0)) +
                       (PRODUCERS > 0 ? (size_t)CHUNK * lanes * kScanColumns : 0)) * sizeof(float);
  auto kernel = linear_scan_kernel<T, MODE, ROWS, CHUNK, PRODUCERS>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  return (int)launch_chain(kernel, dim3((unsigned)blocks), dim3(kScanColumns * lanes + PRODUCERS), smem, stream,
                           dim3(1, 1, 1), p, lanes, slices);
}

// Steps of about a token per sequence (decoding; the caller gives no scratch) stage two tokens at a time, every
// thread its share: few registers and little shared memory per block, so more blocks share an SM while the memories
// stream through.  Other steps have their activations and gates worked out by a kernel of its own, and the scan
// stages 32 tokens (eight where a lane holds 32 rows) by asynchronous copies in warps of their own.
template <typename T, int MODE, int ROWS>
static int launch_scan(const LinearScanParams& p, int lanes, cudaStream_t stream) {
  if (p.act == nullptr) return launch_scan_chunk<T, MODE, ROWS, 2, 0>(p, lanes, stream);
  if (p.num_tokens > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if constexpr (MODE == kGatedWrite || MODE == kConstantDecay) {
    const int width = 2 * p.num_heads * p.head_dim + p.num_heads * p.v_dim;
    const int across = std::min((width + 255) / 256, 64);
    const int err = (int)launch_chain(linear_prep_kernel<T, MODE>, dim3((unsigned)p.num_tokens, (unsigned)across),
                                      dim3(256), 0, stream, dim3(1, 1, 1), p, width);
    if (err != 0) return err;
  }
  return launch_scan_chunk<T, MODE, ROWS, (ROWS >= 32 ? 8 : 32), kScanProducers>(p, lanes, stream);
}

template <typename T>
static int launch_scan_typed(const LinearScanParams& p, int rows, int lanes, cudaStream_t stream) {
  if (p.mode == kGatedWrite)
    return rows == 16 ? launch_scan<T, kGatedWrite, 16>(p, lanes, stream) : launch_scan<T, kGatedWrite, 32>(p, lanes, stream);
  return rows == 16 ? launch_scan<T, kConstantDecay, 16>(p, lanes, stream)
                    : launch_scan<T, kConstantDecay, 32>(p, lanes, stream);
}

int launch_linear_scan(const LinearScanParams& given, cudaStream_t stream) {
  LinearScanParams p = given;
  if (p.num_tokens == 0 || p.num_seqs == 0) return 0;
  if (p.qk_group == 0) p.qk_group = 1;
  // where the staging warps of the prompt form find a token's q, k and v: in the scratch of the preparing kernel, or,
  // for the prepared modes, in x itself
  if (p.mode == kPlainDecay || p.mode == kTokenDecay) {
    p.act_stride = p.x_stride;
    p.act_q_off = p.q_off;
    p.act_k_off = p.k_off;
    p.act_v_off = p.v_off;
    p.act_aligned = (p.x_stride % 4 == 0 && p.q_off % 4 == 0 && p.k_off % 4 == 0 && p.v_off % 4 == 0 &&
                     reinterpret_cast<uintptr_t>(p.x) % 16 == 0) ? 1 : 0;
  } else {
    const int qk = p.num_heads * p.head_dim;
    p.act_stride = 2 * (int64_t)qk + (int64_t)p.num_heads * p.v_dim;
    p.act_q_off = 0;
    p.act_k_off = qk;
    p.act_v_off = 2 * qk;
    p.act_aligned = 1;
  }
  int rows = 0, lanes = 0;
  if (!linear_scan_shape(p.head_dim, p.v_dim, &rows, &lanes) || p.num_heads < 1 || p.mode < kGatedWrite ||
      p.mode > kTokenDecay || p.qk_group < 1 || p.num_heads % p.qk_group)
    return (int)cudaErrorInvalidValue;
  if (p.mode == kGatedWrite ? p.lower == nullptr : (p.mode != kTokenDecay && p.decay == nullptr))
    return (int)cudaErrorInvalidValue;
  if (p.mode == kPlainDecay || p.mode == kTokenDecay) {
    // prepared input: float32 rows that the staging warps copy from as they are
    if (p.dtype != kFloat32 || (p.act != nullptr && p.act != (const float*)p.x)) return (int)cudaErrorInvalidValue;
    if (p.mode == kPlainDecay)
      return rows == 16 ? launch_scan<float, kPlainDecay, 16>(p, lanes, stream)
                        : launch_scan<float, kPlainDecay, 32>(p, lanes, stream);
    return rows == 16 ? launch_scan<float, kTokenDecay, 16>(p, lanes, stream)
                      : launch_scan<float, kTokenDecay, 32>(p, lanes, stream);
  }
  if (p.qk_group != 1) return (int)cudaErrorInvalidValue;
  return p.dtype == kBFloat16 ? launch_scan_typed<__nv_bfloat16>(p, rows, lanes, stream)
                              : launch_scan_typed<float>(p, rows, lanes, stream);
}

int launch_group_norm_gate(const GroupNormGateParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.group < 1 || p.width % p.group || (p.weight != nullptr && p.weight_len < 1) ||
      (p.skip != nullptr && (p.skip_coef == nullptr || p.skip_head < 1)))
    return (int)cudaErrorInvalidValue;
  const int64_t blocks = p.num_tokens * (p.width / p.group);
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const int group = p.group;
  const int threads = group >= 1024 ? 256 : (group >= 128 ? 128 : (group > 32 ? 64 : 32));
  if (p.dtype == kBFloat16)
    return (int)launch_chain(group_norm_gate_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(group_norm_gate_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1), p);
}

}  // namespace akv
