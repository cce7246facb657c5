// Linear attention with a matrix state per head and a decay that is either a fixed number per head
// (retention) or computed per token and key coordinate (gated linear attention), for a ragged batch
// of portions of sequences. Per head, with q, k [dim], v [vdim] and the decay a [dim]:
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t
// Everything here is float32. The projections arrive as float32 rows `proj [tokens, ld]`; `prepare`
// turns them into the recurrence's inputs in place, once per token:
//   queries and keys: a rotation of the first `rot_dims` coordinates of a head by the token's
//     position (coordinate i pairs with i + rot_dims / 2, angle = position * freq[i]), then a factor;
//   the decay: a_t[d] = sigmoid(z_t[d] + bias[d]) ^ inv_tau = exp(inv_tau * log sigmoid), left as
//     a_t[d] - 1 = expm1(inv_tau * log sigmoid) and applied as S + (a - 1) S: a decay close to 1 would
//     round to 24 bits with an error that a long memory adds up token after token, its small part
//     does not; or the head's fixed number.
// The state is held column by column ([vdim][dim] per (request, head)): the lanes that own a
// column read and write its `dim` entries as one contiguous run.
//
// `scan`: the columns of S are independent. A group of L lanes owns one column (each lane R of its
// `dim` entries, in runs of four), a block of 128 threads owns 128 / L columns.
//
// Short portions (decode steps, small pieces of prompts) run as one launch, grid (column slices,
// heads, entries): every block walks its entry's tokens in a row. Long portions are cut into
// chunks of `chunk` tokens that run side by side, in three launches:
//   local:  every chunk's own contribution D_c from a zero state, and the product P_c of the
//           chunk's decays per key coordinate;
//   carry:  per entry, chunk after chunk: the state at the chunk's start S_c, with
//           S_(c+1) = diag(P_c) S_c + D_c, put in D_c's place; the last one goes to the request's state;
//   scan:   every chunk again, now from S_c, with queries and outputs.
// Per token and column the recurrence is the same sequence of operations in both forms; only the
// state a chunk starts from is summed in another order, which moves results by rounding alone.
// Chunk c of entry s uses the chunk slot seq_starts[s] / chunk + s + c.
// `finish`: per token and head the outputs are divided by their root mean square over vdim,
// multiplied by a weight [vdim] (the same for every head; or none), by the SiLU of the gate's
// pre-activation and by one factor.
#include "common.cuh"

namespace pkv {

constexpr int LA_THREADS = 128;

enum { LA_WHOLE = 0, LA_LOCAL = 1, LA_FROM_CARRY = 2 };

struct LaParams {
  int ld, q_off, k_off, v_off;
  const float* a_pre;        // the decays' pre-activations, rows of [heads][dim] with stride a_ld (GATED only)
  int a_ld;
  const float* a_bias;       // [heads * dim] or null
  float inv_tau;
  const float* head_decay;   // [heads] (fixed decay only)
  float q_scale, k_scale;
  int rot_dims;              // 0: no rotation
  const float* freq;         // [rot_dims / 2]
  const int32_t* positions;  // [tokens]
  int heads, dim, vdim, seqs, chunk;
};

__device__ __forceinline__ int la_entry_of_slot(const int32_t* __restrict__ seq_starts, int seqs, int chunk, int slot) {
  int lo = 0, hi = seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seq_starts[mid] / chunk + mid <= slot) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// log(sigmoid(z)) without overflow: min(z, 0) - log(1 + exp(-|z|))
__device__ __forceinline__ float la_log_sigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// One block a token: queries and keys rotated and scaled in place, the decays' pre-activations replaced
// by the decays minus one.
__global__ void __launch_bounds__(128)
la_prepare_kernel(float* __restrict__ proj, float* __restrict__ a_pre, LaParams p) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x;
  float* row = proj + (size_t)t * p.ld;
  const int n = p.heads * p.dim, half = p.rot_dims >> 1;
  const float pos = p.rot_dims ? (float)p.positions[t] : 0.0f;
  const bool touch = p.rot_dims > 0 || p.q_scale != 1.0f || p.k_scale != 1.0f;
  if (touch) {
    for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
      const int head = idx / p.dim, d = idx - head * p.dim;
      float* q = row + p.q_off + (size_t)head * p.dim;
      float* k = row + p.k_off + (size_t)head * p.dim;
      if (d < half) {                                 // this thread turns the pair (d, d + half) of both
        float sn, cs;
        sincosf(pos * p.freq[d], &sn, &cs);
        const float qu = q[d], qv = q[d + half], ku = k[d], kv = k[d + half];
        q[d] = (qu * cs - qv * sn) * p.q_scale;
        q[d + half] = (qv * cs + qu * sn) * p.q_scale;
        k[d] = (ku * cs - kv * sn) * p.k_scale;
        k[d + half] = (kv * cs + ku * sn) * p.k_scale;
      } else if (d >= p.rot_dims) {
        q[d] *= p.q_scale;
        k[d] *= p.k_scale;
      }
    }
  }
  if (a_pre) {
    float* z = a_pre + (size_t)t * p.a_ld;
    for (int idx = threadIdx.x; idx < n; idx += blockDim.x)
      z[idx] = expm1f(la_log_sigmoid(z[idx] + (p.a_bias ? p.a_bias[idx] : 0.0f)) * p.inv_tau);
  }
}

template <int L, int R, int STAGE, int MODE, bool GATED>
__global__ void __launch_bounds__(LA_THREADS)
la_scan_kernel(const float* __restrict__ proj, LaParams p, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
               const int32_t* __restrict__ state_slots, float* __restrict__ out, float* __restrict__ chunk_state,
               float* __restrict__ chunk_decay) {
  dependents_may_launch();
  wait_for_prior_kernels();
  constexpr int COLS = LA_THREADS / L;
  constexpr int DP = L * R;                       // dim rounded up to what the lanes hold
  constexpr int R4 = R / 4;
  constexpr int PER = STAGE * DP / LA_THREADS;    // staged entries per thread and operand
  constexpr int BATCH = PER < 8 ? PER : 8;
  __shared__ __align__(16) float q_s[MODE == LA_LOCAL ? 1 : STAGE][DP];
  __shared__ __align__(16) float k_s[STAGE][DP];
  __shared__ __align__(16) float a_s[GATED ? STAGE : 1][DP];
  __shared__ float v_s[STAGE][COLS];
  __shared__ float o_s[MODE == LA_LOCAL ? 1 : STAGE][COLS];
  const int heads = p.heads, dim = p.dim, vdim = p.vdim;
  const int head = blockIdx.y;
  const int c0 = blockIdx.x * COLS;
  const int local = threadIdx.x / L, lane = threadIdx.x % L;
  const int column = c0 + local;
  int start, count, slot = 0;
  float* mine;
  if (MODE == LA_WHOLE) {
    const int s = blockIdx.z;
    start = seq_starts[s];
    count = seq_starts[s + 1] - start;
    mine = state + (((size_t)state_slots[s] * heads + head) * vdim + column) * dim;
  } else {
    slot = blockIdx.z;
    const int s = la_entry_of_slot(seq_starts, p.seqs, p.chunk, slot);
    const int first = (slot - (seq_starts[s] / p.chunk + s)) * p.chunk;
    const int whole = seq_starts[s + 1] - seq_starts[s];
    if (first >= whole) return;                   // a slot no chunk uses
    start = seq_starts[s] + first;
    count = min(p.chunk, whole - first);
    mine = chunk_state + (((size_t)slot * heads + head) * vdim + column) * dim;
  }
  const float lam = GATED ? 1.0f : p.head_decay[head];
  const bool wide = (dim & 3) == 0 && (reinterpret_cast<uintptr_t>(MODE == LA_WHOLE ? state : chunk_state) & 15) == 0;
  float S[R];
  float P[(MODE == LA_LOCAL && GATED) ? R : 1];   // the product of the chunk's decays
#pragma unroll
  for (int r4 = 0; r4 < R4; ++r4) {
    const int d = 4 * (lane + L * r4);
    if (MODE == LA_LOCAL || column >= vdim || d >= dim) {
      S[4 * r4] = S[4 * r4 + 1] = S[4 * r4 + 2] = S[4 * r4 + 3] = 0.0f;
    } else if (wide) {
      const float4 w = *reinterpret_cast<const float4*>(mine + d);
      S[4 * r4] = w.x; S[4 * r4 + 1] = w.y; S[4 * r4 + 2] = w.z; S[4 * r4 + 3] = w.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) S[4 * r4 + e] = d + e < dim ? mine[d + e] : 0.0f;
    }
  }
  if (MODE == LA_LOCAL && GATED) {
#pragma unroll
    for (int r = 0; r < R; ++r) P[r] = 1.0f;
  }
  const size_t out_ld = (size_t)heads * vdim;
  for (int base = 0; base < count; base += STAGE) {
    const int n = min(STAGE, count - base);
    __syncthreads();                              // the tokens staged before are consumed and flushed
#pragma unroll 1
    for (int i0 = 0; i0 < PER; i0 += BATCH) {
      float qv[BATCH], kv[BATCH], av[BATCH];          // several loads in flight per operand
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int idx = threadIdx.x + (i0 + i) * LA_THREADS;
        const int j = idx / DP, d = idx - j * DP;
        const bool there = j < n && d < dim;
        const size_t token = (size_t)(start + base + (there ? j : 0));
        const float* row = proj + token * p.ld + (size_t)head * dim + (there ? d : 0);
        kv[i] = there ? row[p.k_off] : 0.0f;
        qv[i] = (MODE != LA_LOCAL && there) ? row[p.q_off] : 0.0f;
        av[i] = (GATED && there) ? p.a_pre[token * p.a_ld + (size_t)head * dim + d] : 0.0f;       // the decay minus one
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int idx = threadIdx.x + (i0 + i) * LA_THREADS;
        const int j = idx / DP, d = idx - j * DP;
        k_s[j][d] = kv[i];
        if (MODE != LA_LOCAL) q_s[j][d] = qv[i];
        if (GATED) a_s[j][d] = av[i];
      }
    }
    for (int idx = threadIdx.x; idx < n * COLS; idx += LA_THREADS) {
      const int j = idx / COLS, c = idx - j * COLS;
      v_s[j][c] = c0 + c < vdim ? proj[(size_t)(start + base + j) * p.ld + p.v_off + (size_t)head * vdim + c0 + c] : 0.0f;
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float vj = v_s[j][local];
      float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
      for (int r4 = 0; r4 < R4; ++r4) {
        const int d = 4 * (lane + L * r4);
        const float4 kk = *reinterpret_cast<const float4*>(&k_s[j][d]);
        if (GATED) {
          const float4 aa = *reinterpret_cast<const float4*>(&a_s[j][d]);      // decays minus one
          S[4 * r4] += fmaf(aa.x, S[4 * r4], kk.x * vj);
          S[4 * r4 + 1] += fmaf(aa.y, S[4 * r4 + 1], kk.y * vj);
          S[4 * r4 + 2] += fmaf(aa.z, S[4 * r4 + 2], kk.z * vj);
          S[4 * r4 + 3] += fmaf(aa.w, S[4 * r4 + 3], kk.w * vj);
          if (MODE == LA_LOCAL) {
            P[4 * r4] = fmaf(aa.x, P[4 * r4], P[4 * r4]);
            P[4 * r4 + 1] = fmaf(aa.y, P[4 * r4 + 1], P[4 * r4 + 1]);
            P[4 * r4 + 2] = fmaf(aa.z, P[4 * r4 + 2], P[4 * r4 + 2]);
            P[4 * r4 + 3] = fmaf(aa.w, P[4 * r4 + 3], P[4 * r4 + 3]);
          }
        } else {
          S[4 * r4] = fmaf(kk.x, vj, lam * S[4 * r4]);
          S[4 * r4 + 1] = fmaf(kk.y, vj, lam * S[4 * r4 + 1]);
          S[4 * r4 + 2] = fmaf(kk.z, vj, lam * S[4 * r4 + 2]);
          S[4 * r4 + 3] = fmaf(kk.w, vj, lam * S[4 * r4 + 3]);
        }
        if (MODE != LA_LOCAL) {
          const float4 qq = *reinterpret_cast<const float4*>(&q_s[j][d]);
          acc0 = fmaf(S[4 * r4], qq.x, acc0);
          acc1 = fmaf(S[4 * r4 + 1], qq.y, acc1);
          acc0 = fmaf(S[4 * r4 + 2], qq.z, acc0);
          acc1 = fmaf(S[4 * r4 + 3], qq.w, acc1);
        }
      }
      if (MODE != LA_LOCAL) {
        float acc = acc0 + acc1;
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) o_s[j][local] = acc;
      }
    }
    if (MODE != LA_LOCAL) {
      __syncthreads();
      for (int idx = threadIdx.x; idx < n * COLS; idx += LA_THREADS) {
        const int j = idx / COLS, c = idx - j * COLS;
        if (c0 + c < vdim) out[(size_t)(start + base + j) * out_ld + (size_t)head * vdim + c0 + c] = o_s[j][c];
      }
    }
  }
  if constexpr (MODE != LA_FROM_CARRY) {
    if (MODE == LA_LOCAL && GATED && blockIdx.x == 0 && local == 0) {
      float* decay_row = chunk_decay + ((size_t)slot * heads + head) * dim;
#pragma unroll
      for (int r4 = 0; r4 < R4; ++r4) {
        const int d = 4 * (lane + L * r4);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (d + e < dim) decay_row[d + e] = P[(MODE == LA_LOCAL && GATED) ? 4 * r4 + e : 0];
      }
    }
    if (column >= vdim) return;
#pragma unroll
    for (int r4 = 0; r4 < R4; ++r4) {
      const int d = 4 * (lane + L * r4);
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
template <bool GATED>
__global__ void __launch_bounds__(256)
la_carry_kernel(const float* __restrict__ head_decay, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                const int32_t* __restrict__ state_slots, float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                int heads, int dim, int per_head, int chunk) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int head = blockIdx.y, s = blockIdx.z;
  const int i = blockIdx.x * 256 + threadIdx.x;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  if (i >= per_head || count <= 0) return;
  const int d = i % dim;
  const float lam = GATED ? 1.0f : head_decay[head];
  float full = 1.0f;                               // decay^chunk, by the products the recurrence itself forms
  if (!GATED)
    for (int n = 0; n < chunk; ++n) full *= lam;
  float* request = state + ((size_t)state_slots[s] * heads + head) * per_head + i;
  float S = *request;
  const int slot0 = start / chunk + s;
  for (int first = 0, c = 0; first < count; first += chunk, ++c) {
    float* at = chunk_state + ((size_t)(slot0 + c) * heads + head) * per_head + i;
    const float own = *at;
    *at = S;
    float w;
    if (GATED) {
      w = chunk_decay[((size_t)(slot0 + c) * heads + head) * dim + d];
    } else {
      w = full;
      if (count - first < chunk) {
        w = 1.0f;
        for (int n = 0; n < count - first; ++n) w *= lam;
      }
    }
    S = fmaf(w, S, own);
  }
  *request = S;
}

// o float32 [tokens, heads * vdim]; gate pre-activations float32 at proj[t * ld + g_off + i]; a warp
// a (token, head): out = o / rms(o over vdim) * weight * silu(gate) * factor.
template <typename O>
__global__ void __launch_bounds__(128)
la_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj, int ld, int g_off, const float* __restrict__ weight,
                 float eps, float factor, O* __restrict__ out, int out_ld, int heads, int vdim) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int head = warp; head < heads; head += 4) {
    const float* row = o + ((size_t)t * heads + head) * vdim;
    float sq = 0.0f;
    for (int i = lane; i < vdim; i += 32) sq = fmaf(row[i], row[i], sq);
    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)vdim + eps);
    const float* g = proj + (size_t)t * ld + g_off + (size_t)head * vdim;
    O* dst = out + (size_t)t * out_ld + (size_t)head * vdim;
    for (int i = lane; i < vdim; i += 32) {
      const float z = g[i];
      dst[i] = from_float<O>(row[i] * inv * (weight ? weight[i] : 1.0f) * (z / (1.0f + expf(-z))) * factor);
    }
  }
}

}  // namespace pkv

using namespace pkv;

template <int L, int R, int STAGE, bool GATED>
static int la_launch(const float* proj, const LaParams& p, float* state, const int32_t* seq_starts, const int32_t* state_slots,
                     float* out, int tokens, float* chunk_state, float* chunk_decay, bool chain_first, cudaStream_t s) {
  constexpr int COLS = LA_THREADS / L;
  const unsigned slices = (p.vdim + COLS - 1) / COLS;
  if (p.chunk <= 0)
    return launch_kernel(la_scan_kernel<L, R, STAGE, LA_WHOLE, GATED>, dim3(slices, p.heads, p.seqs), dim3(LA_THREADS), 0, s, chain_first, 0,
                         proj, p, state, seq_starts, state_slots, out, chunk_state, chunk_decay);
  const int slots = tokens / p.chunk + p.seqs;
  if (slots > 65535) return PKV_ERR_LIMIT;
  int rc = launch_kernel(la_scan_kernel<L, R, STAGE, LA_LOCAL, GATED>, dim3(slices, p.heads, slots), dim3(LA_THREADS), 0, s, chain_first, 0,
                         proj, p, state, seq_starts, state_slots, out, chunk_state, chunk_decay);
  if (rc != 0) return rc;
  const int per_head = p.vdim * p.dim;
  rc = launch_kernel(la_carry_kernel<GATED>, dim3((per_head + 255) / 256, p.heads, p.seqs), dim3(256), 0, s, true, 0, p.head_decay,
                     state, seq_starts, state_slots, chunk_state, (const float*)chunk_decay, p.heads, p.dim, per_head, p.chunk);
  if (rc != 0) return rc;
  return launch_kernel(la_scan_kernel<L, R, STAGE, LA_FROM_CARRY, GATED>, dim3(slices, p.heads, slots), dim3(LA_THREADS), 0, s, true, 0,
                       proj, p, state, seq_starts, state_slots, out, chunk_state, chunk_decay);
}

// proj float32 [tokens, ld]: q and k [heads, dim] at q_off and k_off, v and the output gate's
// pre-activation [heads, vdim] at v_off and g_off; the queries' and keys' columns are overwritten
// (rotated and scaled). With a_pre (overwritten too), float32 rows of [heads, dim] with stride
// a_ld hold the decays' pre-activations (a_bias float32 [heads * dim] or null is added; the decay is
// their sigmoid to the power inv_tau); without, head_decay float32 [heads] holds a fixed decay per head.
// freq float32 [rot_dims / 2] and positions int32 [tokens] when rot_dims > 0. state float32 [slots,
// heads, vdim, dim], read and brought up to date. scratch float32 [tokens, heads * vdim]. out [tokens,
// out_ld] of out_dtype receives the normalised, gated outputs times out_factor in its first heads *
// vdim columns. norm_weight float32 [vdim] or null. chunk 0: every entry's tokens in a row, one
// launch; chunk > 0: chunks of that many tokens side by side, with chunk_state float32 [tokens /
// chunk + seqs, heads, vdim, dim] and (with a_pre) chunk_decay float32 [tokens / chunk + seqs, heads,
// dim] as their working memory.
PKV_EXPORT int pkv_linear_attention(float* proj, int ld, int q_off, int k_off, int v_off, int g_off, float* a_pre,
                                    int a_ld, const float* a_bias, float inv_tau, const float* head_decay, float q_scale, float k_scale,
                                    int rot_dims, const float* freq, const int32_t* positions, const float* norm_weight,
                                    float eps, float out_factor, float* state, const int32_t* seq_starts,
                                    const int32_t* state_slots, float* scratch, void* out, int out_dtype, int out_ld,
                                    int tokens, int seqs, int heads, int dim, int vdim, int chunk, float* chunk_state,
                                    float* chunk_decay, void* stream) {
  if (tokens <= 0 || seqs <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || heads > 65535 || seqs > 65535 || chunk < 0 || out_ld < heads * vdim) return PKV_ERR_SIZE;
  if (rot_dims < 0 || (rot_dims & 1) || rot_dims > dim || (rot_dims && (!freq || !positions))) return PKV_ERR_SIZE;
  const bool gated = a_pre != nullptr;
  if ((!gated && !head_decay) || (gated && a_ld < heads * dim)) return PKV_ERR_SIZE;
  if (chunk > 0 && (chunk_state == nullptr || (gated && chunk_decay == nullptr))) return PKV_ERR_SIZE;
  if (dim > 256) return PKV_ERR_LIMIT;
  LaParams p{ld, q_off, k_off, v_off, a_pre, a_ld, a_bias, inv_tau, head_decay, q_scale, k_scale, rot_dims, freq, positions,
             heads, dim, vdim, seqs, chunk};
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  bool chain_first = true;
  if (gated || rot_dims > 0 || q_scale != 1.0f || k_scale != 1.0f) {
    rc = launch_kernel(la_prepare_kernel, dim3(tokens), dim3(128), 0, s, true, 0, proj, a_pre, p);
    if (rc != 0) return rc;
    // The scan behind it is launched the ordinary way: as a programmatic dependent its blocks arrive on SMs that still
    // run this kernel's (which use no shared memory), keep that division between L1 and shared memory, and an entry
    // walked in a row took 133 us in place of 53.
    chain_first = false;
  }
#define PKV_LA(L, R, STAGE)                                                                                                  \
  rc = gated ? la_launch<L, R, STAGE, true>(proj, p, state, seq_starts, state_slots, scratch, tokens, chunk_state, chunk_decay, chain_first, s) \
             : la_launch<L, R, STAGE, false>(proj, p, state, seq_starts, state_slots, scratch, tokens, chunk_state, chunk_decay, chain_first, s)
  if (dim <= 16) PKV_LA(4, 4, 16);
  else if (dim <= 32) PKV_LA(4, 8, 16);
  else if (dim <= 64) PKV_LA(8, 8, 16);
  else if (dim <= 128) PKV_LA(8, 16, 16);
  else PKV_LA(16, 16, 8);
#undef PKV_LA
  if (rc != 0) return rc;
  if (out_dtype == PKV_F32)
    return launch_kernel(la_finish_kernel<float>, dim3(tokens), dim3(128), 0, s, true, 0, (const float*)scratch, proj, ld, g_off,
                         norm_weight, eps, out_factor, (float*)out, out_ld, heads, vdim);
  if (out_dtype == PKV_BF16)
    return launch_kernel(la_finish_kernel<bf16>, dim3(tokens), dim3(128), 0, s, true, 0, (const float*)scratch, proj, ld, g_off,
                         norm_weight, eps, out_factor, (bf16*)out, out_ld, heads, vdim);
  return PKV_ERR_DTYPE;
}
