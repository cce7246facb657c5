// Layer norm with weight and bias around the sublayers of a residual block, and the token shift
// (a blend of a token's normalised row with that of the token before it). Float32 arithmetic
// throughout: mean first, then the mean of the squared deviations from it.
//
//   layer_norm_step  one block per row, one kernel for what happens to the stream between two
//                    sublayers:
//                        x = hidden[row]
//                        x += mult * (layer_norm(update[row]) * post_w + post_b)     (if update)
//                        x += addend[row]                                            (if addend)
//                        hidden[row] = x                                             (unless `rows` selects)
//                        out[r] = layer_norm(x) * pre_w + pre_b                      (if out)
//                    With `rows` (int32 indices) only those rows are worked on, the stream itself
//                    is left as it is, and out has one row per index.
//   token_shift      out[t] = h[t] + (h[t - 1] - h[t]) * mix, with h[t - 1] taken from the
//                    request's state for the first token of an entry (the state holds the last h
//                    of the request's earlier tokens; zeros at the start of a sequence).
//   token_shift_keep state[slot of entry] = h[last token of the entry], launched behind the
//                    kernel above (which reads the state).
#include "common.cuh"

namespace pkv {

constexpr int LN_THREADS = 256;

// mean and 1 / sqrt(variance + eps) of the `width` floats in shared memory `x`
__device__ __forceinline__ void ln_moments(const float* x, int width, float eps, float* scratch, float& mean, float& inv) {
  float sum = 0.0f;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) sum += x[i];
  mean = block_sum(sum, scratch) / (float)width;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) {
    const float c = x[i] - mean;
    sq = fmaf(c, c, sq);
  }
  inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
}

template <typename U, typename O>
__global__ void __launch_bounds__(LN_THREADS)
layer_norm_step_kernel(float* __restrict__ hidden, const U* __restrict__ update, const float* __restrict__ post_w,
                       const float* __restrict__ post_b, float mult, const float* __restrict__ addend,
                       const float* __restrict__ pre_w, const float* __restrict__ pre_b, O* __restrict__ out,
                       const int32_t* __restrict__ rows, int width, float eps) {
  dependents_may_launch();
  wait_for_prior_kernels();
  extern __shared__ float ln_smem[];        // [width], then 32 floats of scratch
  float* x = ln_smem;
  float* scratch = ln_smem + width;
  const size_t row = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* h = hidden + row * width;
  float mean, inv;
  if (update) {
    const U* u = update + row * width;
    for (int i = threadIdx.x; i < width; i += LN_THREADS) x[i] = to_float(u[i]);
    __syncthreads();
    ln_moments(x, width, eps, scratch, mean, inv);
    for (int i = threadIdx.x; i < width; i += LN_THREADS) {
      float v = fmaf(mult, fmaf((x[i] - mean) * inv, post_w[i], post_b[i]), h[i]);
      if (addend) v += addend[row * width + i];
      x[i] = v;
      if (!rows) h[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += LN_THREADS) {
      float v = h[i];
      if (addend) {
        v += addend[row * width + i];
        if (!rows) h[i] = v;
      }
      x[i] = v;
    }
  }
  if (!out) return;
  __syncthreads();
  ln_moments(x, width, eps, scratch, mean, inv);
  O* o = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) o[i] = from_float<O>(fmaf((x[i] - mean) * inv, pre_w[i], pre_b[i]));
}

template <typename O>
__global__ void __launch_bounds__(LN_THREADS)
token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mix, const float* __restrict__ state,
                   const int32_t* __restrict__ token_seq, const int32_t* __restrict__ seq_starts,
                   const int32_t* __restrict__ state_slots, O* __restrict__ out, int width) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  const float* before = t > seq_starts[s] ? h + (size_t)(t - 1) * width : state + (size_t)state_slots[s] * width;
  const float* mine = h + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += LN_THREADS)
    out[(size_t)t * width + i] = from_float<O>(fmaf(before[i] - mine[i], mix[i], mine[i]));
}

__global__ void __launch_bounds__(LN_THREADS)
token_shift_keep_kernel(const float* __restrict__ h, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                        const int32_t* __restrict__ state_slots, int width) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int s = blockIdx.x;
  const int last = seq_starts[s + 1] - 1;
  if (last < seq_starts[s]) return;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) state[(size_t)state_slots[s] * width + i] = h[(size_t)last * width + i];
}

}  // namespace pkv

using namespace pkv;

template <typename U, typename O>
static int launch_step(float* hidden, const void* update, const float* post_w, const float* post_b, float mult,
                       const float* addend, const float* pre_w, const float* pre_b, void* out, const int32_t* rows, int n_rows,
                       int width, float eps, cudaStream_t s) {
  const size_t smem = ((size_t)width + 32) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(layer_norm_step_kernel<U, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_kernel(layer_norm_step_kernel<U, O>, dim3(n_rows), dim3(LN_THREADS), smem, s, true, 0, hidden, (const U*)update,
                       post_w, post_b, mult, addend, pre_w, pre_b, (O*)out, rows, width, eps);
}

// hidden float32 [n, width] (updated in place unless `rows` is given); update [n, width] of
// `update_dtype` or null (then post_w, post_b and mult are not looked at); addend float32 [n, width]
// or null; out [n_rows, width] of `out_dtype` or null (then pre_w and pre_b are not looked at).
PKV_EXPORT int pkv_layer_norm_step(float* hidden, const void* update, int update_dtype, const float* post_w,
                                   const float* post_b, float mult, const float* addend, const float* pre_w,
                                   const float* pre_b, void* out, int out_dtype, const int32_t* rows, int n_rows, int width,
                                   float eps, void* stream) {
  if (n_rows <= 0) return 0;
  if (width <= 0 || (update && (!post_w || !post_b)) || (out && (!pre_w || !pre_b))) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_LN(U, O) \
  return launch_step<U, O>(hidden, update, post_w, post_b, mult, addend, pre_w, pre_b, out, rows, n_rows, width, eps, s)
  const int u = update ? update_dtype : PKV_F32, o = out ? out_dtype : PKV_F32;
  if (u == PKV_F32 && o == PKV_F32) PKV_LN(float, float);
  if (u == PKV_F32 && o == PKV_BF16) PKV_LN(float, bf16);
  if (u == PKV_BF16 && o == PKV_F32) PKV_LN(bf16, float);
  if (u == PKV_BF16 && o == PKV_BF16) PKV_LN(bf16, bf16);
#undef PKV_LN
  return PKV_ERR_DTYPE;
}

// h float32 [tokens, width]; mix float32 [width]; state float32 [slots, width], read for the first
// token of every entry and then set to the entry's last row of h; out [tokens, width].
PKV_EXPORT int pkv_token_shift(const float* h, const float* mix, float* state, const int32_t* token_seq,
                               const int32_t* seq_starts, const int32_t* state_slots, void* out, int out_dtype, int tokens,
                               int seqs, int width, void* stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || seqs <= 0) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (out_dtype == PKV_F32)
    rc = launch_kernel(token_shift_kernel<float>, dim3(tokens), dim3(LN_THREADS), 0, s, true, 0, h, mix, (const float*)state,
                       token_seq, seq_starts, state_slots, (float*)out, width);
  else if (out_dtype == PKV_BF16)
    rc = launch_kernel(token_shift_kernel<bf16>, dim3(tokens), dim3(LN_THREADS), 0, s, true, 0, h, mix, (const float*)state,
                       token_seq, seq_starts, state_slots, (bf16*)out, width);
  else
    return PKV_ERR_DTYPE;
  if (rc != 0) return rc;
  return launch_kernel(token_shift_keep_kernel, dim3(seqs), dim3(LN_THREADS), 0, s, true, 0, h, state, seq_starts, state_slots,
                       width);
}
