// Linear attention with a fixed decay per head ("lightning attention") for a ragged batch of
// portions of sequences, as a recurrence over the tokens of each portion that starts from, and
// leaves, a per-request state. Per head, with q, k [dim] and v [vdim] the SiLU of their projections:
//   S_t = decay S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t
// Everything here is float32: the projections arrive as float32, the activation is applied here,
// the state is float32, held column by column ([vdim][dim] per (request, head)) so that the lanes
// that own a column read and write its `dim` entries as one contiguous run.
//
// `scan`: the columns of S are independent. A group of L lanes owns one column (each lane R of its
// `dim` entries, entry d = lane + L r), a block of 128 threads owns 128 / L columns, the grid is
// (column slices, heads, entries). Queries, keys and values of a few tokens at a time are staged in
// shared memory (activation applied once per block). The operations per token and column, and
// their order, do not depend on how the sequence was cut into portions.
// `finish`: per token the heads' outputs together are divided by their root mean square, multiplied
// by the norm's weight and by the sigmoid of the gate's pre-activation.
#include "common.cuh"

namespace pkv {

constexpr int LT_THREADS = 128;
constexpr int LT_CHUNK = 16;

__device__ __forceinline__ float lt_silu(float z) { return z / (1.0f + expf(-z)); }

template <int L, int R>
__global__ void __launch_bounds__(LT_THREADS)
lightning_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                      const float* __restrict__ decay, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                      const int32_t* __restrict__ state_slots, float* __restrict__ out, int heads, int dim, int vdim) {
  dependents_may_launch();
  wait_for_prior_kernels();
  constexpr int COLS = LT_THREADS / L;
  constexpr int DP = L * R;                       // dim rounded up to what the lanes hold
  __shared__ float q_s[LT_CHUNK][DP];
  __shared__ float k_s[LT_CHUNK][DP];
  __shared__ float v_s[LT_CHUNK][COLS];
  __shared__ float o_s[LT_CHUNK][COLS];
  const int head = blockIdx.y, s = blockIdx.z;
  const int c0 = blockIdx.x * COLS;
  const int local = threadIdx.x / L, p = threadIdx.x % L;
  const int column = c0 + local;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  const float lam = decay[head];
  float* mine = state + (((size_t)state_slots[s] * heads + head) * vdim + column) * dim;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = p + L * r;
    S[r] = (d < dim && column < vdim) ? mine[d] : 0.0f;
  }
  const size_t out_ld = (size_t)heads * vdim;
  for (int base = 0; base < count; base += LT_CHUNK) {
    const int n = min(LT_CHUNK, count - base);
    __syncthreads();                              // the chunk before is consumed and flushed
    for (int idx = threadIdx.x; idx < n * DP; idx += LT_THREADS) {
      const int j = idx / DP, d = idx - j * DP;
      const float* row = proj + (size_t)(start + base + j) * ld + (size_t)head * dim + d;
      q_s[j][d] = d < dim ? lt_silu(row[q_off]) : 0.0f;
      k_s[j][d] = d < dim ? lt_silu(row[k_off]) : 0.0f;
    }
    for (int idx = threadIdx.x; idx < n * COLS; idx += LT_THREADS) {
      const int j = idx / COLS, c = idx - j * COLS;
      v_s[j][c] = c0 + c < vdim ? lt_silu(proj[(size_t)(start + base + j) * ld + v_off + (size_t)head * vdim + c0 + c]) : 0.0f;
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float vj = v_s[j][local];
      float acc = 0.0f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = p + L * r;
        S[r] = fmaf(k_s[j][d], vj, lam * S[r]);
        acc = fmaf(S[r], q_s[j][d], acc);
      }
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (p == 0) o_s[j][local] = acc;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * COLS; idx += LT_THREADS) {
      const int j = idx / COLS, c = idx - j * COLS;
      if (c0 + c < vdim) out[(size_t)(start + base + j) * out_ld + (size_t)head * vdim + c0 + c] = o_s[j][c];
    }
  }
  if (column < vdim) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p + L * r;
      if (d < dim) mine[d] = S[r];
    }
  }
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
                       const int32_t* seq_starts, const int32_t* state_slots, float* out, int seqs, int heads, int dim, int vdim,
                       cudaStream_t s) {
  constexpr int COLS = LT_THREADS / L;
  dim3 grid((vdim + COLS - 1) / COLS, heads, seqs);
  return launch_kernel(lightning_scan_kernel<L, R>, grid, dim3(LT_THREADS), 0, s, true, 0, proj, ld, q_off, k_off, v_off, decay,
                       state, seq_starts, state_slots, out, heads, dim, vdim);
}

// proj float32 [tokens, ld]: the projections before their activation, q and k [heads, dim] at
// q_off and k_off, v and the gate [heads, vdim] at v_off and g_off. decay float32 [heads]. state
// float32 [slots, heads, vdim, dim], read and brought up to date. scratch float32 [tokens, heads *
// vdim]. out [tokens, heads * vdim] of out_dtype: the normalised, gated outputs.
PKV_EXPORT int pkv_lightning(const float* proj, int ld, int q_off, int k_off, int v_off, int g_off, const float* decay,
                             const float* norm_weight, float eps, float* state, const int32_t* seq_starts,
                             const int32_t* state_slots, float* scratch, void* out, int out_dtype, int tokens, int seqs,
                             int heads, int dim, int vdim, void* stream) {
  if (tokens <= 0 || seqs <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || heads > 65535 || seqs > 65535) return PKV_ERR_SIZE;
  if (dim > 256) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
#define PKV_SCAN(L, R) \
  rc = launch_scan<L, R>(proj, ld, q_off, k_off, v_off, decay, state, seq_starts, state_slots, scratch, seqs, heads, dim, vdim, s)
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
