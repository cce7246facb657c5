// Element-wise and per-row kernels beside those of elementwise.cu: bias + activation, the
// residual add that also hands out the stream in the compute type, an activation times a slice
// of a per-token table, router scores with top-k selection, and the activation of routed experts
// scaled by the router's weights. Arithmetic is float32 throughout; storage is float32 or bfloat16.
#include "common.cuh"

namespace pkv {

enum Activation { ACT_NONE = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_RELU_SQUARED = 3, ACT_SIGMOID = 4, ACT_SILU = 5 };
constexpr int ACT_LAST = ACT_SILU;

__device__ __forceinline__ float activate(float z, int act) {
  switch (act) {
    case ACT_GELU_ERF: return 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    case ACT_GELU_TANH: {
      const float inner = 0.79788456080286535588f * (z + 0.044715f * z * z * z);
      return 0.5f * z * (1.0f + tanhf(inner));
    }
    case ACT_RELU_SQUARED: { const float r = fmaxf(z, 0.0f); return r * r; }
    case ACT_SIGMOID: return 1.0f / (1.0f + expf(-z));
    case ACT_SILU: return z / (1.0f + expf(-z));
    default: return z;
  }
}

// out[r, c] = act(x[r, c] + bias[c])
template <typename X, typename O>
__global__ void bias_act_kernel(const X* __restrict__ x, const float* __restrict__ bias, O* __restrict__ out,
                                long long total, int cols, int act) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float z = to_float(x[i]);
  if (bias) z += bias[i % cols];
  out[i] = from_float<O>(activate(z, act));
}

// hidden[r, c] += delta[r, c] + bias[c]; out[r, c] = hidden[r, c] in the type of out
template <typename D, typename O>
__global__ void residual_add_kernel(float* __restrict__ hidden, const D* __restrict__ delta,
                                    const float* __restrict__ bias, O* __restrict__ out, long long total, int cols) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = hidden[i];
  if (delta) v += to_float(delta[i]);
  if (bias) v += bias[i % cols];
  hidden[i] = v;
  if (out) out[i] = from_float<O>(v);
}

// out[t, j] = act(z[t, j]) * table[ids[t], col0 + j]
template <typename X>
__global__ void act_times_table_kernel(const X* __restrict__ z, const X* __restrict__ table, int table_cols,
                                       int table_rows, const int32_t* __restrict__ ids, int col0, X* __restrict__ out,
                                       int tokens, int n, int act, const int32_t* __restrict__ fed_back,
                                       const int32_t* __restrict__ fed_back_at, int* __restrict__ status) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * n) return;
  const int t = (int)(i / n), j = (int)(i - (long long)t * n);
  int id = ids[t];
  if (fed_back_at && fed_back_at[t] >= 0) id = fed_back[fed_back_at[t]];
  float e = 0.0f;
  if (id >= 0 && id < table_rows) e = to_float(table[(size_t)id * table_cols + col0 + j]);
  else if (status) atomicExch(status, PKV_STATUS_BAD_ID);
  out[i] = from_float<X>(activate(to_float(z[i]), act) * e);
}

// Router: the `top` largest logits of a token are chosen (the lower index wins a tie). Their
// weights are their softmax scores over all experts as they are, or, with `renormalise`, the
// softmax over the chosen logits only; every other expert's weight is zero. `bias` (or none) is
// added to the logits first.
__global__ void route_top_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                 float* __restrict__ weights, int tokens, int experts, int top, int renormalise) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float* z = logits + (size_t)t * ld;
  float* w = weights + (size_t)t * experts;
  float m = -INFINITY;
  for (int e = 0; e < experts; ++e) m = fmaxf(m, z[e] + (bias ? bias[e] : 0.0f));
  float sum = 0.0f;
  if (!renormalise)
    for (int e = 0; e < experts; ++e) sum += expf(z[e] + (bias ? bias[e] : 0.0f) - m);
  for (int e = 0; e < experts; ++e) w[e] = 0.0f;
  // pick `top` times the largest logit not picked yet; a picked expert's weight is > 0
  float last = INFINITY;
  int last_e = -1;
  float chosen_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = -1;
    for (int e = 0; e < experts; ++e) {
      const float v = z[e] + (bias ? bias[e] : 0.0f);
      const bool after_last = v < last || (v == last && e > last_e);   // order: score down, index up
      if (after_last && v > best) { best = v; best_e = e; }
    }
    if (best_e < 0) break;
    const float p = expf(best - m);
    w[best_e] = p;
    chosen_sum += p;
    last = best;
    last_e = best_e;
  }
  const float denom = renormalise ? chosen_sum : sum;
  for (int e = 0; e < experts; ++e)
    if (w[e] != 0.0f) w[e] = w[e] / denom;
}

// up[t, :] holds the up-projections of all routed experts ([experts][ff]) and then of the shared
// expert ([shared_ff]). out = relu(up)^2 scaled by the router's weight of the column's expert, and
// for the shared expert by sigmoid(gate[t]).
template <typename X>
__global__ void expert_act_kernel(const X* __restrict__ up, int ld, const float* __restrict__ weights,
                                  const float* __restrict__ gate, int gate_ld, X* __restrict__ out, int tokens,
                                  int experts, int ff, int shared_ff, int act) {
  const int cols = experts * ff + shared_ff;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * cols) return;
  const int t = (int)(i / cols), c = (int)(i - (long long)t * cols);
  float scale;
  if (c < experts * ff) scale = weights[(size_t)t * experts + c / ff];
  else scale = gate ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_ld])) : 1.0f;
  float v = 0.0f;
  if (scale != 0.0f) v = scale * activate(to_float(up[(size_t)t * ld + c]), act);
  out[(size_t)t * cols + c] = from_float<X>(v);
}


// --- 16-byte forms for bfloat16 rows whose sizes are multiples of 8 -------------------------------

struct Pack8 { float v[8]; };

__device__ __forceinline__ Pack8 load8(const bf16* p) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  Pack8 out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out.v[2 * i] = f.x;
    out.v[2 * i + 1] = f.y;
  }
  return out;
}

__device__ __forceinline__ void store8(bf16* p, const Pack8& x) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x.v[2 * i], x.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

__global__ void bias_act_bf16x8_kernel(const bf16* __restrict__ x, const float* __restrict__ bias, bf16* __restrict__ out,
                                       long long groups, int cols, int act) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  Pack8 v = load8(x + i * 8);
  const int c = (int)((i * 8) % cols);
#pragma unroll
  for (int k = 0; k < 8; ++k) v.v[k] = activate(v.v[k] + (bias ? bias[c + k] : 0.0f), act);
  store8(out + i * 8, v);
}

__global__ void expert_act_bf16x8_kernel(const bf16* __restrict__ up, int ld, const float* __restrict__ weights,
                                         const float* __restrict__ gate, int gate_ld, bf16* __restrict__ out, int tokens,
                                         int experts, int ff, int shared_ff, int act) {
  const int cols = experts * ff + shared_ff;
  const int per_row = cols >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * per_row) return;
  const int t = (int)(i / per_row), c = (int)(i - (long long)t * per_row) << 3;
  float scale;
  if (c < experts * ff) scale = weights[(size_t)t * experts + c / ff];
  else scale = gate ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_ld])) : 1.0f;
  Pack8 v;
  if (scale != 0.0f) {
    v = load8(up + (size_t)t * ld + c);
#pragma unroll
    for (int k = 0; k < 8; ++k) v.v[k] = scale * activate(v.v[k], act);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) v.v[k] = 0.0f;
  }
  store8(out + (size_t)t * cols + c, v);
}


// Gated experts: gu[t, :] holds the gate projections of all routed experts ([experts][ff]) and of
// the shared expert ([shared_ff]) and, `up_at` columns further on, the up projections in the same
// order. out[t, c] = scale * act(gate) * up with the router's weight of the column's expert as
// scale (1 for the shared expert); an expert the token does not use gives exact zeros.
template <typename X>
__global__ void expert_gated_act_kernel(const X* __restrict__ gu, int ld, int up_at, const float* __restrict__ weights,
                                        X* __restrict__ out, int tokens, int experts, int ff, int shared_ff, int act) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int cols = experts * ff + shared_ff;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * cols) return;
  const int t = (int)(i / cols), c = (int)(i - (long long)t * cols);
  const float scale = c < experts * ff ? weights[(size_t)t * experts + c / ff] : 1.0f;
  float v = 0.0f;
  if (scale != 0.0f) {
    const X* row = gu + (size_t)t * ld;
    v = scale * (activate(to_float(row[c]), act) * to_float(row[up_at + c]));
  }
  out[(size_t)t * cols + c] = from_float<X>(v);
}

__global__ void expert_gated_act_bf16x8_kernel(const bf16* __restrict__ gu, int ld, int up_at,
                                               const float* __restrict__ weights, bf16* __restrict__ out, int tokens,
                                               int experts, int ff, int shared_ff, int act) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int cols = experts * ff + shared_ff;
  const int per_row = cols >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * per_row) return;
  const int t = (int)(i / per_row), c = (int)(i - (long long)t * per_row) << 3;
  const float scale = c < experts * ff ? weights[(size_t)t * experts + c / ff] : 1.0f;
  Pack8 v;
  if (scale != 0.0f) {
    v = load8(gu + (size_t)t * ld + c);
    const Pack8 u = load8(gu + (size_t)t * ld + up_at + c);
#pragma unroll
    for (int k = 0; k < 8; ++k) v.v[k] = scale * (activate(v.v[k], act) * u.v[k]);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) v.v[k] = 0.0f;
  }
  store8(out + (size_t)t * cols + c, v);
}

// The residual step of a block that normalises a sublayer's output, not its input:
//   hidden[r] += delta[r] / sqrt(mean(delta[r]^2) + eps) * weight;   out[r] = hidden[r] in the type of out
// One block a row; the row waits in shared memory between the two passes.
template <typename D, typename O>
__global__ void norm_residual_kernel(float* __restrict__ hidden, const D* __restrict__ delta, const float* __restrict__ weight,
                                     float eps, O* __restrict__ out, int d) {
  dependents_may_launch();
  wait_for_prior_kernels();
  extern __shared__ float nr_smem[];   // d floats + 32 scratch
  float* row = nr_smem;
  float* scratch = nr_smem + d;
  const size_t at = (size_t)blockIdx.x * d;
  float sq = 0.0f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = to_float(delta[at + c]);
    row[c] = v;
    sq = fmaf(v, v, sq);
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.0f / sqrtf(sq / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = hidden[at + c] + row[c] * inv * weight[c];
    hidden[at + c] = v;
    if (out) out[at + c] = from_float<O>(v);
  }
}

// Dot product of `n` weights with float values in shared memory; 16-byte loads for bfloat16 rows
// that start on 16-byte boundaries (n a multiple of 8), lane-strided otherwise.
__device__ __forceinline__ float row_dot_strided(const float* w, const float* v, int n, int first, int step) {
  float acc = 0.0f;
  for (int c = first; c < n; c += step) acc = fmaf(w[c], v[c], acc);
  return acc;
}
__device__ __forceinline__ float row_dot_strided(const bf16* w, const float* v, int n, int first, int step) {
  float acc = 0.0f;
  if ((n & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int c = first * 8; c < n; c += step * 8) {
      const Pack8 x = load8(w + c);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc = fmaf(x.v[k], v[c + k], acc);
    }
    return acc;
  }
  for (int c = first; c < n; c += step) acc = fmaf(to_float(w[c]), v[c], acc);
  return acc;
}

// The whole per-token side input for the few rows of a decode step, one block per token:
//   hidden += delta + bias;  x = hidden (rounded to the compute type)
//   z = gate_w x;  g = act(z) * table[id, col0 + j];  y = proj_w g;  out = y / rms(y) * norm_w   (float32)
// with the same roundings between the stages as the separate kernels and library products have.
template <typename W, typename D>
__global__ void __launch_bounds__(256)
token_side_kernel(float* __restrict__ hidden, const D* __restrict__ delta, const float* __restrict__ bias,
                  const W* __restrict__ gate_w, const W* __restrict__ proj_w, const W* __restrict__ table, int table_cols,
                  int table_rows, const int32_t* __restrict__ ids, int col0, const float* __restrict__ norm_w, float eps,
                  float* __restrict__ out, int width, int dim, int act, const int32_t* __restrict__ fed_back,
                  const int32_t* __restrict__ fed_back_at, int* __restrict__ status) {
  extern __shared__ float ts_smem[];
  float* x = ts_smem;             // [width]
  float* y = x + width;           // [width]
  float* g = y + width;           // [dim]
  float* scratch = g + dim;       // [32]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = hidden[(size_t)t * width + c];
    if (delta) v += to_float(delta[(size_t)t * width + c]);
    if (bias) v += bias[c];
    hidden[(size_t)t * width + c] = v;
    x[c] = to_float(from_float<W>(v));
  }
  int id = ids[t];
  if (fed_back_at && fed_back_at[t] >= 0) id = fed_back[fed_back_at[t]];
  const bool known = id >= 0 && id < table_rows;
  if (!known && threadIdx.x == 0 && status) atomicExch(status, PKV_STATUS_BAD_ID);
  __syncthreads();
  for (int j = warp; j < dim; j += (blockDim.x >> 5)) {
    float acc = row_dot_strided(gate_w + (size_t)j * width, x, width, lane, 32);
    acc = warp_sum(acc);
    if (lane == 0) {
      const float z = to_float(from_float<W>(acc));
      const float e = known ? to_float(table[(size_t)id * table_cols + col0 + j]) : 0.0f;
      g[j] = to_float(from_float<W>(activate(z, act) * e));
    }
  }
  __syncthreads();
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float acc = row_dot_strided(proj_w + (size_t)c * dim, g, dim, 0, 1);
    y[c] = acc;
    ss = fmaf(acc, acc, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)t * width + c] = y[c] * inv * norm_w[c];
}

// x <- cap * tanh(x / cap), in place (float32): a soft cap on logits.
__global__ void softcap_kernel(float* __restrict__ x, long long total, float cap) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

// Router with sigmoid scores and groups of experts. score_e = sigmoid(logit_e); an expert is chosen
// by score_e + correction_e (the choice score), its weight comes from score_e alone. The experts
// form `groups` equal groups of neighbours; a group's score is the sum of its two largest choice
// scores (of its one, in groups of one), and only experts of the `keep` best groups can be chosen.
// The `top` allowed experts with the largest choice scores are chosen (the lower index wins a tie);
// their weights are score / (sum of the chosen scores + 1e-20) * scale, every other weight is zero.
// A thread a token; up to 64 groups.
__global__ void route_scored_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction,
                                    float* __restrict__ weights, int tokens, int experts, int top, int groups, int keep,
                                    float scale) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float* z = logits + (size_t)t * ld;
  float* w = weights + (size_t)t * experts;
  const int per_group = experts / groups;
  unsigned long long allowed = ~0ull;
  if (keep < groups) {
    allowed = 0ull;
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int best_g = -1;
      for (int g = 0; g < groups; ++g) {
        if ((allowed >> g) & 1ull) continue;
        float first = -INFINITY, second = -INFINITY;
        for (int e = g * per_group; e < (g + 1) * per_group; ++e) {
          const float c = 1.0f / (1.0f + expf(-z[e])) + (correction ? correction[e] : 0.0f);
          if (c > first) { second = first; first = c; }
          else if (c > second) second = c;
        }
        const float score = per_group > 1 ? first + second : first;
        if (best_g < 0 || score > best) { best = score; best_g = g; }
      }
      if (best_g < 0) break;
      allowed |= 1ull << best_g;
    }
  }
  for (int e = 0; e < experts; ++e) w[e] = 0.0f;
  float last = INFINITY;
  int last_e = -1;
  float chosen_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_s = 0.0f;
    int best_e = -1;
    for (int e = 0; e < experts; ++e) {
      if (!((allowed >> (e / per_group)) & 1ull)) continue;
      const float s = 1.0f / (1.0f + expf(-z[e]));
      const float c = s + (correction ? correction[e] : 0.0f);
      const bool after_last = c < last || (c == last && e > last_e);   // order: choice score down, index up
      if (after_last && (best_e < 0 || c > best)) { best = c; best_e = e; best_s = s; }
    }
    if (best_e < 0) break;
    w[best_e] = -1.0f - best_s;              // marked as chosen (a score may be 0): -1 - score
    chosen_sum += best_s;
    last = best;
    last_e = best_e;
  }
  const float denom = chosen_sum + 1e-20f;
  for (int e = 0; e < experts; ++e)
    if (w[e] < 0.0f) w[e] = (-1.0f - w[e]) / denom * scale;
}

// A gated feed-forward's middle step with biases: gu[t, :] holds the gate columns [n] and, `up_at`
// columns further on, the up columns; out[t, c] = act(gate + gate_bias[c]) * (up + up_bias[c]).
template <typename X>
__global__ void gated_bias_act_kernel(const X* __restrict__ gu, int ld, int up_at, const float* __restrict__ gate_bias,
                                      const float* __restrict__ up_bias, X* __restrict__ out, int tokens, int n, int act) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * n) return;
  const int t = (int)(i / n), c = (int)(i - (long long)t * n);
  const X* row = gu + (size_t)t * ld;
  const float g = to_float(row[c]) + (gate_bias ? gate_bias[c] : 0.0f);
  const float u = to_float(row[up_at + c]) + (up_bias ? up_bias[c] : 0.0f);
  out[(size_t)t * n + c] = from_float<X>(activate(g, act) * u);
}

__global__ void gated_bias_act_bf16x8_kernel(const bf16* __restrict__ gu, int ld, int up_at, const float* __restrict__ gate_bias,
                                             const float* __restrict__ up_bias, bf16* __restrict__ out, int tokens, int n, int act) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int per_row = n >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * per_row) return;
  const int t = (int)(i / per_row), c = (int)(i - (long long)t * per_row) << 3;
  Pack8 g = load8(gu + (size_t)t * ld + c);
  const Pack8 u = load8(gu + (size_t)t * ld + up_at + c);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    g.v[k] = activate(g.v[k] + (gate_bias ? gate_bias[c + k] : 0.0f), act) * (u.v[k] + (up_bias ? up_bias[c + k] : 0.0f));
  store8(out + (size_t)t * n + c, g);
}

// hidden[t] += delta[t] (when given); out[t] = [hidden[t] | other[t]] in the type of out: the
// stream beside a second float32 matrix of the same shape, as the operand of one product.
template <typename D, typename O>
__global__ void pair_rows_kernel(float* __restrict__ hidden, const D* __restrict__ delta, const float* __restrict__ other,
                                 O* __restrict__ out, long long total, int cols) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / cols;
  const int c = (int)(i - t * cols);
  float v = hidden[i];
  if (delta) { v += to_float(delta[i]); hidden[i] = v; }
  out[t * 2 * cols + c] = from_float<O>(v);
  out[t * 2 * cols + cols + c] = from_float<O>(other[i]);
}

// hidden[t, c] = value[t, c] + bias[c]
__global__ void assign_bias_kernel(float* __restrict__ hidden, const float* __restrict__ value, const float* __restrict__ bias,
                                   long long total, int cols) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  hidden[i] = value[i] + (bias ? bias[i % cols] : 0.0f);
}

// Two float32 updates of the same shape become one. With weights: out = fa * a / rms(a) * wa + fb * b /
// rms(b) * wb (each divided by its own root mean square over the row); without: out = fa * a + fb * b.
// One block a row.
__global__ void combine_pair_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                                    const float* __restrict__ wb, float fa, float fb, float eps, float* __restrict__ out, int d) {
  dependents_may_launch();
  wait_for_prior_kernels();
  __shared__ float scratch[32];
  const size_t at = (size_t)blockIdx.x * d;
  float inv_a = 1.0f, inv_b = 1.0f;
  if (wa) {
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      sa = fmaf(a[at + c], a[at + c], sa);
      sb = fmaf(b[at + c], b[at + c], sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    inv_a = 1.0f / sqrtf(sa / (float)d + eps);
    inv_b = 1.0f / sqrtf(sb / (float)d + eps);
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float x = wa ? a[at + c] * inv_a * wa[c] : a[at + c];
    const float y = wb ? b[at + c] * inv_b * wb[c] : b[at + c];
    out[at + c] = fa * x + fb * y;
  }
}

// out[t, h * vdim + j] = x[t, h * vdim + j] * sigmoid(gate[t * gate_ld + h]) * factor: one gate per token and
// head (or none: the factor alone). `out` may be `x` itself, or rows with a stride of their own.
template <typename X>
__global__ void head_gate_kernel(const X* __restrict__ x, const X* __restrict__ gate, int gate_ld, X* __restrict__ out,
                                 int out_ld, long long total, int heads, int vdim, float factor) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / ((long long)heads * vdim);
  const int c = (int)(i - t * heads * vdim);
  float f = factor;
  if (gate) f = factor / (1.0f + expf(-to_float(gate[t * gate_ld + c / vdim])));
  out[t * out_ld + c] = from_float<X>(to_float(x[i]) * f);
}

}  // namespace pkv

using namespace pkv;

static inline unsigned blocks_for(long long total, int threads) { return (unsigned)((total + threads - 1) / threads); }

PKV_EXPORT int pkv_bias_act(const void* x, int x_dtype, const float* bias, void* out, int out_dtype, long long rows,
                            int cols, int act, void* stream) {
  const long long total = rows * cols;
  if (total <= 0) return 0;
  if (act < 0 || act > ACT_LAST) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (x_dtype == PKV_BF16 && out_dtype == PKV_BF16 && cols % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    bias_act_bf16x8_kernel<<<blocks_for(total / 8, 256), 256, 0, s>>>((const bf16*)x, bias, (bf16*)out, total / 8, cols, act);
    return launch_status();
  }
#define PKV_BA(X, O) bias_act_kernel<X, O><<<blocks_for(total, 256), 256, 0, s>>>((const X*)x, bias, (O*)out, total, cols, act); return launch_status()
  if (x_dtype == PKV_F32 && out_dtype == PKV_F32) { PKV_BA(float, float); }
  if (x_dtype == PKV_F32 && out_dtype == PKV_BF16) { PKV_BA(float, bf16); }
  if (x_dtype == PKV_BF16 && out_dtype == PKV_BF16) { PKV_BA(bf16, bf16); }
  if (x_dtype == PKV_BF16 && out_dtype == PKV_F32) { PKV_BA(bf16, float); }
#undef PKV_BA
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_residual_add(float* hidden, const void* delta, int delta_dtype, const float* bias, void* out,
                                int out_dtype, long long rows, int cols, void* stream) {
  const long long total = rows * cols;
  if (total <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_RA(D, O) return launch_kernel(residual_add_kernel<D, O>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, hidden, (const D*)delta, bias, (O*)out, total, cols)
  if (delta_dtype == PKV_F32 && out_dtype == PKV_F32) { PKV_RA(float, float); }
  if (delta_dtype == PKV_F32 && out_dtype == PKV_BF16) { PKV_RA(float, bf16); }
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_BF16) { PKV_RA(bf16, bf16); }
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_F32) { PKV_RA(bf16, float); }
#undef PKV_RA
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_act_times_table(const void* z, const void* table, int dtype, int table_cols, int table_rows,
                                   const int32_t* ids, int col0, void* out, int tokens, int n, int act,
                                   const int32_t* fed_back, const int32_t* fed_back_at, int* status, void* stream) {
  const long long total = (long long)tokens * n;
  if (total <= 0) return 0;
  if (col0 < 0 || col0 + n > table_cols || act < 0 || act > ACT_LAST) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32) {
    act_times_table_kernel<float><<<blocks_for(total, 256), 256, 0, s>>>((const float*)z, (const float*)table, table_cols,
        table_rows, ids, col0, (float*)out, tokens, n, act, fed_back, fed_back_at, status);
  } else if (dtype == PKV_BF16) {
    act_times_table_kernel<bf16><<<blocks_for(total, 256), 256, 0, s>>>((const bf16*)z, (const bf16*)table, table_cols,
        table_rows, ids, col0, (bf16*)out, tokens, n, act, fed_back, fed_back_at, status);
  } else {
    return PKV_ERR_DTYPE;
  }
  return launch_status();
}

PKV_EXPORT int pkv_route_top(const float* logits, int ld, const float* bias, float* weights, int tokens, int experts, int top,
                             int renormalise, void* stream) {
  if (tokens <= 0) return 0;
  if (experts < 1 || top < 1 || top > experts || ld < experts) return PKV_ERR_SIZE;
  // a token a thread, little work each: small blocks spread a prompt's tokens over many SMs
  return launch_kernel(route_top_kernel, dim3(blocks_for(tokens, 32)), dim3(32), 0, (cudaStream_t)stream, true, 0, logits, ld, bias,
                       weights, tokens, experts, top, renormalise);
}

PKV_EXPORT int pkv_expert_gated_act(const void* gu, int dtype, int ld, int up_at, const float* weights, void* out, int tokens,
                                    int experts, int ff, int shared_ff, int act, void* stream) {
  const long long cols = (long long)experts * ff + shared_ff;
  const long long total = (long long)tokens * cols;
  if (total <= 0) return 0;
  if (experts < 0 || ff < 0 || shared_ff < 0 || act < 0 || act > ACT_LAST || up_at < cols || ld < up_at + cols) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32) {
    return launch_kernel(expert_gated_act_kernel<float>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, (const float*)gu, ld,
                         up_at, weights, (float*)out, tokens, experts, ff, shared_ff, act);
  } else if (dtype == PKV_BF16 && ff % 8 == 0 && shared_ff % 8 == 0 && ld % 8 == 0 && up_at % 8 == 0 &&
             ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    return launch_kernel(expert_gated_act_bf16x8_kernel, dim3(blocks_for(total / 8, 256)), dim3(256), 0, s, true, 0, (const bf16*)gu,
                         ld, up_at, weights, (bf16*)out, tokens, experts, ff, shared_ff, act);
  } else if (dtype == PKV_BF16) {
    return launch_kernel(expert_gated_act_kernel<bf16>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, (const bf16*)gu, ld,
                         up_at, weights, (bf16*)out, tokens, experts, ff, shared_ff, act);
  } else {
    return PKV_ERR_DTYPE;
  }
  return launch_status();
}

PKV_EXPORT int pkv_norm_residual(float* hidden, const void* delta, int delta_dtype, const float* weight, float eps, void* out,
                                 int out_dtype, int rows, int d, void* stream) {
  if (rows <= 0) return 0;
  if (d <= 0) return PKV_ERR_SIZE;
  const size_t smem = (size_t)(d + 32) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
#define PKV_NR(D, O)                                                                                                     \
  do {                                                                                                                   \
    if (smem > 48 * 1024) {                                                                                              \
      cudaError_t e = cudaFuncSetAttribute(norm_residual_kernel<D, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                               \
    }                                                                                                                    \
    return launch_kernel(norm_residual_kernel<D, O>, dim3(rows), dim3(threads), smem, s, true, 0, hidden, (const D*)delta,  \
                         weight, eps, (O*)out, d);                                                                        \
  } while (0)
  if (!out) out_dtype = PKV_F32;
  if (delta_dtype == PKV_F32 && out_dtype == PKV_F32) PKV_NR(float, float);
  if (delta_dtype == PKV_F32 && out_dtype == PKV_BF16) PKV_NR(float, bf16);
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_BF16) PKV_NR(bf16, bf16);
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_F32) PKV_NR(bf16, float);
#undef PKV_NR
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_expert_act(const void* up, int dtype, int ld, const float* weights, const float* gate, int gate_ld,
                              void* out, int tokens, int experts, int ff, int shared_ff, int act, void* stream) {
  const long long total = (long long)tokens * ((long long)experts * ff + shared_ff);
  if (total <= 0) return 0;
  if (experts < 0 || ff < 0 || shared_ff < 0 || act < 0 || act > ACT_LAST) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32) {
    expert_act_kernel<float><<<blocks_for(total, 256), 256, 0, s>>>((const float*)up, ld, weights, gate, gate_ld,
                                                                    (float*)out, tokens, experts, ff, shared_ff, act);
  } else if (dtype == PKV_BF16 && ff % 8 == 0 && shared_ff % 8 == 0 && ld % 8 == 0 && ((uintptr_t)up & 15) == 0 &&
             ((uintptr_t)out & 15) == 0) {
    expert_act_bf16x8_kernel<<<blocks_for(total / 8, 256), 256, 0, s>>>((const bf16*)up, ld, weights, gate, gate_ld, (bf16*)out,
                                                                         tokens, experts, ff, shared_ff, act);
  } else if (dtype == PKV_BF16) {
    expert_act_kernel<bf16><<<blocks_for(total, 256), 256, 0, s>>>((const bf16*)up, ld, weights, gate, gate_ld,
                                                                   (bf16*)out, tokens, experts, ff, shared_ff, act);
  } else {
    return PKV_ERR_DTYPE;
  }
  return launch_status();
}

PKV_EXPORT int pkv_token_side(float* hidden, const void* delta, int delta_dtype, const float* bias, const void* gate_w,
                              const void* proj_w, const void* table, int dtype, int table_cols, int table_rows,
                              const int32_t* ids, int col0, const float* norm_w, float eps, float* out, int tokens, int width,
                              int dim, int act, const int32_t* fed_back, const int32_t* fed_back_at, int* status,
                              void* stream) {
  if (tokens <= 0) return 0;
  if (width < 1 || dim < 1 || col0 < 0 || col0 + dim > table_cols || act < 0 || act > ACT_LAST) return PKV_ERR_SIZE;
  const size_t smem = (size_t)(2 * width + dim + 32) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_TS(W, D)                                                                                                    \
  do {                                                                                                                  \
    if (smem > 48 * 1024) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(token_side_kernel<W, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                              \
    }                                                                                                                   \
    token_side_kernel<W, D><<<tokens, 256, smem, s>>>(hidden, (const D*)delta, bias, (const W*)gate_w, (const W*)proj_w,  \
                                                      (const W*)table, table_cols, table_rows, ids, col0, norm_w, eps, out, \
                                                      width, dim, act, fed_back, fed_back_at, status);                  \
    return launch_status();                                                                                             \
  } while (0)
  const int d = delta ? delta_dtype : dtype;
  if (dtype == PKV_F32 && d == PKV_F32) PKV_TS(float, float);
  if (dtype == PKV_BF16 && d == PKV_BF16) PKV_TS(bf16, bf16);
  if (dtype == PKV_BF16 && d == PKV_F32) PKV_TS(bf16, float);
  if (dtype == PKV_F32 && d == PKV_BF16) PKV_TS(float, bf16);
#undef PKV_TS
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_softcap(float* x, long long total, float cap, void* stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.0f)) return PKV_ERR_SIZE;
  return launch_kernel(softcap_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, (cudaStream_t)stream, true, 0, x, total, cap);
}

PKV_EXPORT int pkv_route_scored(const float* logits, int ld, const float* correction, float* weights, int tokens, int experts,
                                int top, int groups, int keep, float scale, void* stream) {
  if (tokens <= 0) return 0;
  if (experts < 1 || top < 1 || top > experts || ld < experts || groups < 1 || groups > 64 || experts % groups || keep < 1 ||
      keep > groups || top > experts / groups * keep)
    return PKV_ERR_SIZE;
  return launch_kernel(route_scored_kernel, dim3(blocks_for(tokens, 32)), dim3(32), 0, (cudaStream_t)stream, true, 0, logits, ld,
                       correction, weights, tokens, experts, top, groups, keep, scale);
}

PKV_EXPORT int pkv_gated_bias_act(const void* gu, int dtype, int ld, int up_at, const float* gate_bias, const float* up_bias,
                                  void* out, int tokens, int n, int act, void* stream) {
  const long long total = (long long)tokens * n;
  if (total <= 0) return 0;
  if (act < 0 || act > ACT_LAST || up_at < n || ld < up_at + n) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32)
    return launch_kernel(gated_bias_act_kernel<float>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, (const float*)gu, ld,
                         up_at, gate_bias, up_bias, (float*)out, tokens, n, act);
  if (dtype == PKV_BF16 && n % 8 == 0 && ld % 8 == 0 && up_at % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0)
    return launch_kernel(gated_bias_act_bf16x8_kernel, dim3(blocks_for(total / 8, 256)), dim3(256), 0, s, true, 0, (const bf16*)gu, ld,
                         up_at, gate_bias, up_bias, (bf16*)out, tokens, n, act);
  if (dtype == PKV_BF16)
    return launch_kernel(gated_bias_act_kernel<bf16>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, (const bf16*)gu, ld,
                         up_at, gate_bias, up_bias, (bf16*)out, tokens, n, act);
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_pair_rows(float* hidden, const void* delta, int delta_dtype, const float* other, void* out, int out_dtype,
                             long long rows, int cols, void* stream) {
  const long long total = rows * cols;
  if (total <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_PR(D, O) return launch_kernel(pair_rows_kernel<D, O>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, hidden, (const D*)delta, other, (O*)out, total, cols)
  if (!delta) delta_dtype = PKV_F32;
  if (delta_dtype == PKV_F32 && out_dtype == PKV_F32) { PKV_PR(float, float); }
  if (delta_dtype == PKV_F32 && out_dtype == PKV_BF16) { PKV_PR(float, bf16); }
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_BF16) { PKV_PR(bf16, bf16); }
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_F32) { PKV_PR(bf16, float); }
#undef PKV_PR
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_assign_bias(float* hidden, const float* value, const float* bias, long long rows, int cols, void* stream) {
  const long long total = rows * cols;
  if (total <= 0) return 0;
  return launch_kernel(assign_bias_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, (cudaStream_t)stream, true, 0, hidden, value,
                       bias, total, cols);
}

PKV_EXPORT int pkv_combine_pair(const float* a, const float* b, const float* wa, const float* wb, float fa, float fb, float eps,
                                float* out, int rows, int d, void* stream) {
  if (rows <= 0) return 0;
  if (d <= 0 || ((wa == nullptr) != (wb == nullptr))) return PKV_ERR_SIZE;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  return launch_kernel(combine_pair_kernel, dim3(rows), dim3(threads), 0, (cudaStream_t)stream, true, 0, a, b, wa, wb, fa, fb, eps,
                       out, d);
}

PKV_EXPORT int pkv_head_gate(const void* x, const void* gate, int dtype, int gate_ld, void* out, int out_ld, int tokens, int heads,
                             int vdim, float factor, void* stream) {
  const long long total = (long long)tokens * heads * vdim;
  if (total <= 0) return 0;
  if ((gate && gate_ld < heads) || out_ld < heads * vdim) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32)
    return launch_kernel(head_gate_kernel<float>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, (const float*)x,
                         (const float*)gate, gate_ld, (float*)out, out_ld, total, heads, vdim, factor);
  if (dtype == PKV_BF16)
    return launch_kernel(head_gate_kernel<bf16>, dim3(blocks_for(total, 256)), dim3(256), 0, s, true, 0, (const bf16*)x,
                         (const bf16*)gate, gate_ld, (bf16*)out, out_ld, total, heads, vdim, factor);
  return PKV_ERR_DTYPE;
}
