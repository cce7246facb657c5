// Linear attention with a fixed decay per head ("lightning attention") for a ragged batch of
// portions of sequences, as a recurrence over the tokens of each portion that starts from, and
// leaves, a per-request state. Per head, with q, k [dim] and v [vdim] the SiLU of their projections:
//   S_t = decay S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t
// Everything here is float32: the projections arrive as float32, the activation is applied here,
// the state is float32, held column by column ([vdim][dim] per (request, head)) so that the lanes
// that own a column read and write its `dim` entries as one contiguous run.
//
// `scan`: the columns of S are independent. A group of L lanes owns one column (each lane R of its
// `dim` entries, in runs of four: entry d = 4 (lane + L r4) + e, so that a lane reads its queries
// and keys from shared memory as 16-byte words), a block of 128 threads owns 128 / L columns.
// Queries, keys and values of a few tokens at a time are staged in shared memory (activation
// applied once per block).
//
// Short portions (decode steps, small pieces of prompts) run as one launch, grid (column slices,
// heads, entries): every block walks its entry's tokens in a row. Long portions are cut into
// chunks of `chunk` tokens that run side by side, in three launches:
//   local:  every chunk's own contribution D_c = sum_j decay^(n-1-j) k_j v_j^T, from a zero state;
//   carry:  per entry, chunk after chunk: the state at the chunk's start S_c, with
//           S_(c+1) = decay^n S_c + D_c, put in D_c's place; the last one goes to the request's state;
//   scan:   every chunk again, now from S_c, with queries and outputs.
// Per token and column the recurrence is the same sequence of operations in both forms; only the
// state a chunk starts from is summed in another order, which moves results by rounding alone.
// Chunk c of entry s uses the chunk slot seq_starts[s] / chunk + s + c: these ranges do not meet,
// and tokens / chunk + entries slots hold them all.
// `finish`: per token the heads' outputs together are divided by their root mean square, multiplied
// by the norm's weight and by the sigmoid of the gate's pre-activation.
#include "common.cuh"

namespace pkv {

constexpr int LT_THREADS = 128;
constexpr int LT_STAGE = 16;       // tokens staged in shared memory at a time
constexpr int LT_BATCH = 8;        // loads a thread has in flight per operand while staging

enum { LT_WHOLE = 0, LT_LOCAL = 1, LT_FROM_CARRY = 2 };

__device__ __forceinline__ float lt_silu(float z) { return z / (1.0f + expf(-z)); }

// The entry whose range of chunk slots holds `slot`: the last s with seq_starts[s] / chunk + s <= slot.
__device__ __forceinline__ int lt_entry_of_slot(const int32_t* __restrict__ seq_starts, int seqs, int chunk, int slot) {
  int lo = 0, hi = seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seq_starts[mid] / chunk + mid <= slot) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <int L, int R, int MODE>
__global__ void __launch_bounds__(LT_THREADS)
lightning_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                      const float* __restrict__ decay, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                      const int32_t* __restrict__ state_slots, float* __restrict__ out, int heads, int dim, int vdim,
                      int seqs, int chunk, float* __restrict__ chunk_state) {
  dependents_may_launch();
  wait_for_prior_kernels();
  constexpr int COLS = LT_THREADS / L;
  constexpr int DP = L * R;                       // dim rounded up to what the lanes hold
  constexpr int R4 = R / 4;
  constexpr int PER = LT_STAGE * DP / LT_THREADS; // staged entries per thread and operand
  constexpr int BATCH = PER < LT_BATCH ? PER : LT_BATCH;
  __shared__ __align__(16) float q_s[MODE == LT_LOCAL ? 1 : LT_STAGE][DP];
  __shared__ __align__(16) float k_s[LT_STAGE][DP];
  __shared__ float v_s[LT_STAGE][COLS];
  __shared__ float o_s[MODE == LT_LOCAL ? 1 : LT_STAGE][COLS];
  const int head = blockIdx.y;
  const int c0 = blockIdx.x * COLS;
  const int local = threadIdx.x / L, p = threadIdx.x % L;
  const int column = c0 + local;
  int start, count;
  float* mine;
  if (MODE == LT_WHOLE) {
    const int s = blockIdx.z;
    start = seq_starts[s];
    count = seq_starts[s + 1] - start;
    mine = state + (((size_t)state_slots[s] * heads + head) * vdim + column) * dim;
  } else {
    const int slot = blockIdx.z;
    const int s = lt_entry_of_slot(seq_starts, seqs, chunk, slot);
    const int first = (slot - (seq_starts[s] / chunk + s)) * chunk;
    const int whole = seq_starts[s + 1] - seq_starts[s];
    if (first >= whole) return;                   // a slot no chunk uses
    start = seq_starts[s] + first;
    count = min(chunk, whole - first);
    mine = chunk_state + (((size_t)slot * heads + head) * vdim + column) * dim;
  }
  const float lam = decay[head];
  // a column's entries start on 16-byte boundaries
  const bool wide = (dim & 3) == 0 && (reinterpret_cast<uintptr_t>(MODE == LT_WHOLE ? state : chunk_state) & 15) == 0;
  float S[R];
#pragma unroll
  for (int r4 = 0; r4 < R4; ++r4) {
    const int d = 4 * (p + L * r4);
    if (MODE == LT_LOCAL || column >= vdim || d >= dim) {
      S[4 * r4] = S[4 * r4 + 1] = S[4 * r4 + 2] = S[4 * r4 + 3] = 0.0f;
    } else if (wide) {
      const float4 w = *reinterpret_cast<const float4*>(mine + d);
      S[4 * r4] = w.x; S[4 * r4 + 1] = w.y; S[4 * r4 + 2] = w.z; S[4 * r4 + 3] = w.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) S[4 * r4 + e] = d + e < dim ? mine[d + e] : 0.0f;
    }
  }
  const size_t out_ld = (size_t)heads * vdim;
  for (int base = 0; base < count; base += LT_STAGE) {
    const int n = min(LT_STAGE, count - base);
    __syncthreads();                              // the tokens staged before are consumed and flushed
#pragma unroll 1
    for (int i0 = 0; i0 < PER; i0 += BATCH) {
      float qv[BATCH], kv[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int idx = threadIdx.x + (i0 + i) * LT_THREADS;
        const int j = idx / DP, d = idx - j * DP;
        const bool there = j < n && d < dim;
        const float* row = proj + (size_t)(start + base + (there ? j : 0)) * ld + (size_t)head * dim + (there ? d : 0);
        kv[i] = there ? row[k_off] : 0.0f;
        if (MODE != LT_LOCAL) qv[i] = there ? row[q_off] : 0.0f;
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int idx = threadIdx.x + (i0 + i) * LT_THREADS;
        const int j = idx / DP, d = idx - j * DP;
        k_s[j][d] = lt_silu(kv[i]);
        if (MODE != LT_LOCAL) q_s[j][d] = lt_silu(qv[i]);
      }
    }
    for (int idx = threadIdx.x; idx < n * COLS; idx += LT_THREADS) {
      const int j = idx / COLS, c = idx - j * COLS;
      v_s[j][c] = c0 + c < vdim ? lt_silu(proj[(size_t)(start + base + j) * ld + v_off + (size_t)head * vdim + c0 + c]) : 0.0f;
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float vj = v_s[j][local];
      float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
      for (int r4 = 0; r4 < R4; ++r4) {
        const int d = 4 * (p + L * r4);
        const float4 kk = *reinterpret_cast<const float4*>(&k_s[j][d]);
        S[4 * r4] = fmaf(kk.x, vj, lam * S[4 * r4]);
        S[4 * r4 + 1] = fmaf(kk.y, vj, lam * S[4 * r4 + 1]);
        S[4 * r4 + 2] = fmaf(kk.z, vj, lam * S[4 * r4 + 2]);
        S[4 * r4 + 3] = fmaf(kk.w, vj, lam * S[4 * r4 + 3]);
        if (MODE != LT_LOCAL) {
          const float4 qq = *reinterpret_cast<const float4*>(&q_s[j][d]);
          acc0 = fmaf(S[4 * r4], qq.x, acc0);
          acc1 = fmaf(S[4 * r4 + 1], qq.y, acc1);
          acc0 = fmaf(S[4 * r4 + 2], qq.z, acc0);
          acc1 = fmaf(S[4 * r4 + 3], qq.w, acc1);
        }
      }
      if (MODE != LT_LOCAL) {
        float acc = acc0 + acc1;
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (p == 0) o_s[j][local] = acc;
      }
    }
    if (MODE != LT_LOCAL) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < n * COLS; idx += LT_THREADS) {
        const int j = idx / COLS, c = idx - j * COLS;
        if (c0 + c < vdim) out[(size_t)(start + base + j) * out_ld + (size_t)head * vdim + c0 + c] = o_s[j][c];
      }
    }
  }
  if constexpr (MODE != LT_FROM_CARRY) {
    if (column >= vdim) return;
#pragma unroll
    for (int r4 = 0; r4 < R4; ++r4) {
      const int d = 4 * (p + L * r4);
      if (d >= dim) continue;
      if (wide) {
        *reinterpret_cast<float4*>(mine + d) = make_float4(S[4 * r4], S[4 * r4 + 1], S[4 * r4 + 2], S[4 * r4 + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (d + e < dim) mine[d + e] = S[4 * r4 + e];
      }
    }
  }
}

// Per entry, chunk after chunk: chunk_state[slot] holds the chunk's own contribution and gets the
// state at the chunk's start; the state after the last chunk goes to the request's slot. One
// thread an entry of a head's state; grid (ceil(per_head / 256), heads, entries).
__global__ void __launch_bounds__(256)
lightning_carry_kernel(const float* __restrict__ decay, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                       const int32_t* __restrict__ state_slots, float* __restrict__ chunk_state, int heads, int per_head,
                       int chunk) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int head = blockIdx.y, s = blockIdx.z;
  const int i = blockIdx.x * 256 + threadIdx.x;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  if (i >= per_head || count <= 0) return;
  const float lam = decay[head];
  float full = 1.0f;                               // decay^chunk, by the products the recurrence itself forms
  for (int n = 0; n < chunk; ++n) full *= lam;
  float* request = state + ((size_t)state_slots[s] * heads + head) * per_head + i;
  float S = *request;
  const int slot0 = start / chunk + s;
  for (int first = 0, c = 0; first < count; first += chunk, ++c) {
    float* at = chunk_state + ((size_t)(slot0 + c) * heads + head) * per_head + i;
    const float own = *at;
    *at = S;
    float w = full;
    if (count - first < chunk) {
      w = 1.0f;
      for (int n = 0; n < count - first; ++n) w *= lam;
    }
    S = fmaf(w, S, own);
  }
  *request = S;
}

// o float32 [tokens, n]; gate: pre-activations float32 at proj[t * ld + g_off + i]; out [tokens, n].
template <typename O>
__global__ void __launch_bounds__(256)
lightning_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj, int ld, int g_off,
                        const float* __restrict__ weight, float eps, O* __restrict__ out, int n) {
  dependents_may_launch();
  wait_for_prior_kernels();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * n;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
  const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)n + eps);
  const float* g = proj + (size_t)t * ld + g_off;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[(size_t)t * n + i] = from_float<O>(row[i] * inv * weight[i] / (1.0f + expf(-g[i])));
}

}  // namespace pkv

using namespace pkv;

template <int L, int R>
static int launch_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                       const int32_t* seq_starts, const int32_t* state_slots, float* out, int tokens, int seqs, int heads, int dim,
                       int vdim, int chunk, float* chunk_state, cudaStream_t s) {
  constexpr int COLS = LT_THREADS / L;
  const unsigned slices = (vdim + COLS - 1) / COLS;
  if (chunk <= 0)
    return launch_kernel(lightning_scan_kernel<L, R, LT_WHOLE>, dim3(slices, heads, seqs), dim3(LT_THREADS), 0, s, true, 0, proj, ld,
                         q_off, k_off, v_off, decay, state, seq_starts, state_slots, out, heads, dim, vdim, seqs, 0, chunk_state);
  const int slots = tokens / chunk + seqs;
  if (slots > 65535) return PKV_ERR_LIMIT;
  int rc = launch_kernel(lightning_scan_kernel<L, R, LT_LOCAL>, dim3(slices, heads, slots), dim3(LT_THREADS), 0, s, true, 0, proj, ld,
                         q_off, k_off, v_off, decay, state, seq_starts, state_slots, out, heads, dim, vdim, seqs, chunk, chunk_state);
  if (rc != 0) return rc;
  const int per_head = vdim * dim;
  rc = launch_kernel(lightning_carry_kernel, dim3((per_head + 255) / 256, heads, seqs), dim3(256), 0, s, true, 0, decay, state,
                     seq_starts, state_slots, chunk_state, heads, per_head, chunk);
  if (rc != 0) return rc;
  return launch_kernel(lightning_scan_kernel<L, R, LT_FROM_CARRY>, dim3(slices, heads, slots), dim3(LT_THREADS), 0, s, true, 0, proj,
                       ld, q_off, k_off, v_off, decay, state, seq_starts, state_slots, out, heads, dim, vdim, seqs, chunk, chunk_state);
}

// proj float32 [tokens, ld]: the projections before their activation, q and k [heads, dim] at
// q_off and k_off, v and the gate [heads, vdim] at v_off and g_off. decay float32 [heads]. state
// float32 [slots, heads, vdim, dim], read and brought up to date. scratch float32 [tokens, heads *
// vdim]. out [tokens, heads * vdim] of out_dtype: the normalised, gated outputs. chunk 0: every
// entry's tokens in a row, one launch; chunk > 0: chunks of that many tokens side by side, with
// chunk_state float32 [tokens / chunk + seqs, heads, vdim, dim] as their working memory.
PKV_EXPORT int pkv_lightning(const float* proj, int ld, int q_off, int k_off, int v_off, int g_off, const float* decay,
                             const float* norm_weight, float eps, float* state, const int32_t* seq_starts,
                             const int32_t* state_slots, float* scratch, void* out, int out_dtype, int tokens, int seqs,
                             int heads, int dim, int vdim, int chunk, float* chunk_state, void* stream) {
  if (tokens <= 0 || seqs <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || heads > 65535 || seqs > 65535 || chunk < 0) return PKV_ERR_SIZE;
  if (chunk > 0 && chunk_state == nullptr) return PKV_ERR_SIZE;
  if (dim > 256) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
#define PKV_SCAN(L, R)                                                                                                       \
  rc = launch_scan<L, R>(proj, ld, q_off, k_off, v_off, decay, state, seq_starts, state_slots, scratch, tokens, seqs, heads, dim, \
                         vdim, chunk, chunk_state, s)
  if (dim <= 16) PKV_SCAN(4, 4);
  else if (dim <= 32) PKV_SCAN(4, 8);
  else if (dim <= 64) PKV_SCAN(8, 8);
  else if (dim <= 128) PKV_SCAN(8, 16);
  else PKV_SCAN(16, 16);
#undef PKV_SCAN
  if (rc != 0) return rc;
  const int n = heads * vdim;
  if (out_dtype == PKV_F32)
    return launch_kernel(lightning_finish_kernel<float>, dim3(tokens), dim3(256), 0, s, true, 0, (const float*)scratch, proj, ld,
                         g_off, norm_weight, eps, (float*)out, n);
  if (out_dtype == PKV_BF16)
    return launch_kernel(lightning_finish_kernel<bf16>, dim3(tokens), dim3(256), 0, s, true, 0, (const float*)scratch, proj, ld,
                         g_off, norm_weight, eps, (bf16*)out, n);
  return PKV_ERR_DTYPE;
}
