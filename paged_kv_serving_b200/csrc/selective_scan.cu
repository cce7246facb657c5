// The selective scan of a Mamba mixer over a ragged batch of portions of sequences.
// Per channel c and state coordinate n, token by token:
//   dt   = softplus(dt_pre[t, c] + dt_bias[c])
//   S[c, n] <- exp(dt * A[c, n]) * S[c, n] + dt * x[t, c] * B[t, n]
//   y[t, c] = sum_n S[c, n] * C[t, n] + D[c] * x[t, c];      out[t, c] = y[t, c] * silu(z[t, c])
// S lives in a per-request state [slots, inner, state] (float32), read when a portion begins and
// written back when it ends, so a sequence may arrive in portions of any size and the result is
// the same operations in the same order however it was cut. With float32 activations the decay
// is applied as S + expm1(dt A) S (a decay close to 1 keeps its small part to full precision).
// Everything that enters the recurrence is float32: the step sizes, the decays, B and C (they arrive as the float32 result
// of their projection), the state. x and z are activations in the compute type.
//
// A team of L lanes (a power of two, at most a warp) owns one channel; each lane keeps R state
// coordinates n = lane_in_team + r * L in registers (R is 2, 4 or 8 by the state's size; L and R
// are template parameters, so every index is a constant). A block of SCAN_THREADS threads takes
// SCAN_THREADS / L channels of one sequence and walks the portion in chunks of SCAN_CHUNK tokens
// staged in shared memory (the softplus is taken while staging). Inside a chunk the token loop is
// unrolled and holds only what depends on the state: the decays exp(dt A) and the inputs dt x B
// of all 16 tokens are independent of it and are scheduled ahead, so the chain through the state
// is one multiply-add a token. Each lane's share of y stays in registers until the chunk ends;
// then the shares of a team are added (shuffles) and left in shared memory, and all threads
// together add D x, apply the gate and store the chunk's outputs. The next chunk's inputs are
// fetched into registers before the current chunk is computed.
// A chunk that the portion does not fill is padded with dt = 0 and x = 0, which leave the state
// as it is (decay 1, input 0); coordinates beyond the state's size are padded with B = C = 0.
// Blocks are small (two warps) so that a prompt's few thousand lanes still spread over all SMs
// and one block's staging overlaps another's arithmetic.
#include "common.cuh"

namespace pkv {

constexpr int SCAN_THREADS = 64;
constexpr int SCAN_CHUNK = 16;
constexpr int SCAN_MAX_REGS = 8;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

struct ScanParams {
  int inner, state;
  int ld_x, ld_z, ld_dt, ld_bc;   // row strides (elements)
  int b_at, c_at;                 // columns of B and C in the float32 projection
};

template <typename X, int L, int R>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const X* __restrict__ x, const X* __restrict__ z, const float* __restrict__ dt_pre,
                      const float* __restrict__ dt_bias, const float* __restrict__ bc, const float* __restrict__ a,
                      const float* __restrict__ d_skip, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                      const int32_t* __restrict__ state_slots, X* __restrict__ out, ScanParams p) {
  dependents_may_launch();
  wait_for_prior_kernels();
  constexpr int CHANNELS = SCAN_THREADS / L;      // channels of this block
  constexpr int PADDED = L * R;                   // state coordinates a team covers (>= state)
  __shared__ float dt_s[SCAN_CHUNK * CHANNELS];   // step sizes (after softplus)
  __shared__ float x_s[SCAN_CHUNK * CHANNELS];
  __shared__ float z_s[SCAN_CHUNK * CHANNELS];
  __shared__ float y_s[SCAN_CHUNK * CHANNELS];
  __shared__ float b_s[SCAN_CHUNK * PADDED];
  __shared__ float c_s[SCAN_CHUNK * PADDED];

  const int s = blockIdx.y;
  const int start = seq_starts[s], n_tokens = seq_starts[s + 1] - start;
  const int slot = state_slots[s];
  const int c0 = blockIdx.x * CHANNELS;
  const int team = threadIdx.x / L, lane = threadIdx.x % L;
  const int c = c0 + team;
  const bool live = c < p.inner;

  float S[R], A[R];                               // the state and the decay rates
  float* mine = state + ((size_t)slot * p.inner + (live ? c : 0)) * p.state;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int n = lane + r * L;
    const bool has = live && n < p.state;
    S[r] = has ? mine[n] : 0.0f;
    A[r] = has ? a[(size_t)c * p.state + n] : 0.0f;
  }

  // What a thread stages of a chunk: ACT_IT elements of dt, x and z and BC_IT of B and C. They are
  // fetched into registers one chunk ahead, so that the loads are in flight while the chunk before
  // is computed (wide states, whose B and C would take too many registers, fetch those when staging).
  constexpr int ACT_IT = (SCAN_CHUNK * CHANNELS + SCAN_THREADS - 1) / SCAN_THREADS;
  constexpr int BC_IT = (SCAN_CHUNK * PADDED + SCAN_THREADS - 1) / SCAN_THREADS;
  constexpr bool BC_AHEAD = BC_IT <= 8;
  float f_dt[ACT_IT], f_x[ACT_IT], f_z[ACT_IT], f_b[BC_AHEAD ? BC_IT : 1], f_c[BC_AHEAD ? BC_IT : 1];
  auto fetch = [&](int t0) {
    const int count = min(SCAN_CHUNK, n_tokens - t0);
#pragma unroll
    for (int it = 0; it < ACT_IT; ++it) {
      const int i = threadIdx.x + it * SCAN_THREADS;
      const int j = i / CHANNELS, ch = c0 + i % CHANNELS;
      const size_t t = (size_t)(start + t0 + j);
      const bool has = i < SCAN_CHUNK * CHANNELS && j < count && ch < p.inner;
      f_dt[it] = has ? dt_pre[t * p.ld_dt + ch] + dt_bias[ch] : -INFINITY;     // softplus(-inf) = 0: a padded step
      f_x[it] = has ? to_float(x[t * p.ld_x + ch]) : 0.0f;
      f_z[it] = has ? to_float(z[t * p.ld_z + ch]) : 0.0f;
    }
    if (BC_AHEAD) {
#pragma unroll
      for (int it = 0; it < BC_IT; ++it) {
        const int i = threadIdx.x + it * SCAN_THREADS;
        const int j = i / PADDED, n = i % PADDED;
        const size_t t = (size_t)(start + t0 + j);
        const bool has = i < SCAN_CHUNK * PADDED && j < count && n < p.state;
        f_b[it] = has ? bc[t * p.ld_bc + p.b_at + n] : 0.0f;
        f_c[it] = has ? bc[t * p.ld_bc + p.c_at + n] : 0.0f;
      }
    }
  };
  if (n_tokens > 0) fetch(0);

  for (int t0 = 0; t0 < n_tokens; t0 += SCAN_CHUNK) {
    const int count = min(SCAN_CHUNK, n_tokens - t0);
    __syncthreads();                               // the chunk before is consumed
#pragma unroll
    for (int it = 0; it < ACT_IT; ++it) {
      const int i = threadIdx.x + it * SCAN_THREADS;
      if (i < SCAN_CHUNK * CHANNELS) {
        dt_s[i] = softplus_f(f_dt[it]);
        x_s[i] = f_x[it];
        z_s[i] = f_z[it];
      }
    }
    if (BC_AHEAD) {
#pragma unroll
      for (int it = 0; it < BC_IT; ++it) {
        const int i = threadIdx.x + it * SCAN_THREADS;
        if (i < SCAN_CHUNK * PADDED) {
          b_s[i] = f_b[it];
          c_s[i] = f_c[it];
        }
      }
    } else {
      for (int i = threadIdx.x; i < SCAN_CHUNK * PADDED; i += SCAN_THREADS) {
        const int j = i / PADDED, n = i % PADDED;
        const size_t t = (size_t)(start + t0 + j);
        const bool has = j < count && n < p.state;
        b_s[i] = has ? bc[t * p.ld_bc + p.b_at + n] : 0.0f;
        c_s[i] = has ? bc[t * p.ld_bc + p.c_at + n] : 0.0f;
      }
    }
    __syncthreads();
    if (t0 + SCAN_CHUNK < n_tokens) fetch(t0 + SCAN_CHUNK);
    float y[SCAN_CHUNK];
#pragma unroll
    for (int j = 0; j < SCAN_CHUNK; ++j) {
      const float dtv = dt_s[j * CHANNELS + team];
      const float dx = dtv * x_s[j * CHANNELS + team];
      float part = 0.0f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if constexpr (sizeof(X) == 4) {
          // true float32: a decay close to 1 rounds to 24 bits with an error that a long memory adds up token
          // after token; exp(a) S = S + expm1(a) S keeps the small part to full precision
          S[r] += fmaf(expm1f(dtv * A[r]), S[r], dx * b_s[j * PADDED + r * L + lane]);
        } else {
          S[r] = fmaf(expf(dtv * A[r]), S[r], dx * b_s[j * PADDED + r * L + lane]);
        }
        part = fmaf(S[r], c_s[j * PADDED + r * L + lane], part);
      }
      y[j] = part;
    }
#pragma unroll
    for (int j = 0; j < SCAN_CHUNK; ++j) {
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1) y[j] += __shfl_xor_sync(0xffffffffu, y[j], o);
      if (lane == 0) y_s[j * CHANNELS + team] = y[j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < count * CHANNELS; i += SCAN_THREADS) {
      const int j = i / CHANNELS, k = i % CHANNELS;
      const int ch = c0 + k;
      if (ch < p.inner) {
        const float zv = z_s[i];
        const float total = fmaf(d_skip[ch], x_s[i], y_s[i]);
        out[(size_t)(start + t0 + j) * p.inner + ch] = from_float<X>(total * (zv / (1.0f + expf(-zv))));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int n = lane + r * L;
      if (n < p.state) mine[n] = S[r];
    }
  }
}

template <typename X, int L, int R>
static int launch_scan(const void* x, const void* z, const float* dt_pre, const float* dt_bias, const float* bc, const float* a,
                       const float* d_skip, float* state, const int32_t* seq_starts, const int32_t* state_slots, void* out,
                       const ScanParams& p, int seqs, cudaStream_t s) {
  constexpr int CHANNELS = SCAN_THREADS / L;
  dim3 grid((p.inner + CHANNELS - 1) / CHANNELS, seqs);
  return launch_kernel(selective_scan_kernel<X, L, R>, grid, dim3(SCAN_THREADS), 0, s, true, 0, (const X*)x, (const X*)z, dt_pre,
                       dt_bias, bc, a, d_skip, state, seq_starts, state_slots, (X*)out, p);
}

template <typename X>
static int launch_scan_for(int n_state, const void* x, const void* z, const float* dt_pre, const float* dt_bias, const float* bc,
                           const float* a, const float* d_skip, float* state, const int32_t* seq_starts,
                           const int32_t* state_slots, void* out, const ScanParams& p, int seqs, cudaStream_t s) {
#define PKV_SCAN(L, R) return launch_scan<X, L, R>(x, z, dt_pre, dt_bias, bc, a, d_skip, state, seq_starts, state_slots, out, p, seqs, s)
  // state coordinates per lane: 2, 4 or 8, the fewest that keep a team within a warp; for the
  // common small states that leaves several lanes (more warps in flight) per channel
  if (n_state <= 2) PKV_SCAN(1, 2);
  if (n_state <= 4) PKV_SCAN(2, 2);
  if (n_state <= 8) PKV_SCAN(4, 2);
  if (n_state <= 16) PKV_SCAN(8, 2);
  if (n_state <= 32) PKV_SCAN(16, 2);
  if (n_state <= 64) PKV_SCAN(32, 2);
  if (n_state <= 128) PKV_SCAN(32, 4);
  PKV_SCAN(32, 8);
#undef PKV_SCAN
}

}  // namespace pkv

using namespace pkv;

// x [tokens, >= inner] (row stride ld_x) and z (ld_z) in the compute type; dt_pre float32 [tokens,
// >= inner] (ld_dt); bc float32 [tokens, ld_bc] with B at column b_at and C at c_at; a [inner,
// state], dt_bias and d_skip [inner] float32; state float32 [slots, inner, state]; out [tokens, inner].
PKV_EXPORT int pkv_selective_scan(const void* x, int ld_x, const void* z, int ld_z, int dtype, const float* dt_pre, int ld_dt,
                                  const float* dt_bias, const float* bc, int ld_bc, int b_at, int c_at, const float* a,
                                  const float* d_skip, float* state, const int32_t* seq_starts, const int32_t* state_slots,
                                  void* out, int tokens, int seqs, int inner, int n_state, void* stream) {
  if (tokens <= 0 || seqs <= 0) return 0;
  if (inner < 1 || n_state < 1 || ld_x < inner || ld_z < inner || ld_dt < inner || b_at < 0 || c_at < 0 ||
      ld_bc < b_at + n_state || ld_bc < c_at + n_state)
    return PKV_ERR_SIZE;
  if (n_state > 32 * SCAN_MAX_REGS || seqs > 65535) return PKV_ERR_LIMIT;
  ScanParams p{inner, n_state, ld_x, ld_z, ld_dt, ld_bc, b_at, c_at};
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32)
    return launch_scan_for<float>(n_state, x, z, dt_pre, dt_bias, bc, a, d_skip, state, seq_starts, state_slots, out, p, seqs, s);
  if (dtype == PKV_BF16)
    return launch_scan_for<bf16>(n_state, x, z, dt_pre, dt_bias, bc, a, d_skip, state, seq_starts, state_slots, out, p, seqs, s);
  return PKV_ERR_DTYPE;
}
