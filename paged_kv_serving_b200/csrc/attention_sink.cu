// Paged causal attention with a sliding window that also keeps the first tokens of a sequence,
// a soft cap on the scores, unit-norm queries and keys, keys and values of different sizes, and
// values that may be blended with those of an earlier layer. Two kernels:
//
//   qkv_prepare     per (token, head): rotates the first `rot_dims` coordinates of a query or key
//                   head (coordinate i pairs with i + rot_dims/2; angle = position * freq[i] in
//                   float32, cos and sin times `rot_factor`), divides the head by its root mean
//                   square, writes queries back in place and keys into the key pool; blends a
//                   value head with the same token's value of another layer,
//                   v <- (1 - lambda) v + lambda v_other, and writes it into the value pool.
//                   A bias per column may be added to the projections first, and the norm may
//                   instead be one over all of a token's query columns (and one over all its key
//                   columns) with a weight per column, applied before the rotation.
//   attention_sink  float32-arithmetic attention for any sizes, float32 or bfloat16 storage:
//                   score = q.k * scale, then cap * tanh(score / cap); query position i sees key
//                   j when j <= i and (i - j < window or j < keep_first); softmax; weighted sum
//                   of the values.
//
// Work decomposition of the attention kernel as in attention_generic.cu: the rows of one
// (sequence, key/value head) are (query token, head in group) pairs, a block of 8 warps takes 8
// consecutive rows, keys are walked in tiles of 32 absolute positions staged in shared memory.
// Tiles are aligned to multiples of 32 from position 0 and folded in ascending order, and a
// masked key adds exactly zero, so a row's result does not depend on how the batch was cut.
#include "common.cuh"

namespace pkv {

constexpr int SK_WARPS = 8;
constexpr int SK_TILE = 32;
constexpr int SK_MAX_ACC = 8;   // value size <= 32 * 8
constexpr int SK_MAX_DIM = 512;

// --- prepare ---------------------------------------------------------------------------------

struct PrepareParams {
  int ld;                 // row stride of qkv: [H * dim | G * dim | G * vdim] and maybe padding
  int n_heads, n_kv, dim, vdim;
  int rot_dims;           // 0: no rotation
  float rot_factor;
  float eps;
  int unit_norm;          // 1: divide query and key heads by their root mean square, after the rotation;
                          // 2: divide all query columns of a token by their joint root mean square (the key
                          //    columns by theirs) and multiply by a weight per column, before the rotation
  int page_size;
  long long pool_slots;   // pages * page_size
  int ld_other;           // row stride of the other layer's values
};

template <typename A, typename C>
__global__ void __launch_bounds__(SK_WARPS * 32)
qkv_prepare_kernel(A* __restrict__ qkv, const int32_t* __restrict__ positions, const float* __restrict__ freq,
                   const float* __restrict__ q_weight, const float* __restrict__ k_weight, const float* __restrict__ bias,
                   const A* __restrict__ v_other, const float* __restrict__ lambda, A* __restrict__ v_keep,
                   C* __restrict__ k_pool, C* __restrict__ v_pool, const int32_t* __restrict__ slots, PrepareParams p,
                   int* __restrict__ status) {
  dependents_may_launch();
  wait_for_prior_kernels();
  extern __shared__ float prep_smem[];                  // [SK_WARPS][dim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  float* buf = prep_smem + warp * p.dim;
  A* row = qkv + (size_t)t * p.ld;
  const float pos = (float)positions[t];
  long long slot = slots ? slots[t] : -1;
  if (slot >= p.pool_slots) {                             // never becomes an address
    if (lane == 0 && status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    slot = -1;
  }
  const long long page = slot >= 0 ? slot / p.page_size : 0;
  const int offset = slot >= 0 ? (int)(slot % p.page_size) : 0;
  const int half = p.rot_dims >> 1;
  const int qk_heads = p.n_heads + p.n_kv;
  const bool joint = p.unit_norm == 2;
  float inv_q = 1.0f, inv_k = 1.0f;
  if (joint) {
    float* scratch = prep_smem + SK_WARPS * p.dim;      // [32]
    const int q_cols = p.n_heads * p.dim, k_cols = p.n_kv * p.dim;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < q_cols; c += blockDim.x) {
      const float v = to_float(row[c]) + (bias ? bias[c] : 0.0f);
      sq = fmaf(v, v, sq);
    }
    inv_q = 1.0f / sqrtf(block_sum(sq, scratch) / (float)q_cols + p.eps);
    sq = 0.0f;
    for (int c = threadIdx.x; c < k_cols; c += blockDim.x) {
      const float v = to_float(row[q_cols + c]) + (bias ? bias[q_cols + c] : 0.0f);
      sq = fmaf(v, v, sq);
    }
    inv_k = 1.0f / sqrtf(block_sum(sq, scratch) / (float)k_cols + p.eps);
    __syncthreads();
  }
  for (int unit = warp; unit < qk_heads + p.n_kv; unit += SK_WARPS) {
    if (unit < qk_heads) {
      // a query head (written back in place) or a key head (written to the pool)
      A* x = row + (size_t)unit * p.dim;
      const float* b = bias ? bias + (size_t)unit * p.dim : nullptr;
      // with the joint norm: the factor of this head's columns before the rotation
      const float pre = joint ? (unit < p.n_heads ? inv_q : inv_k) : 1.0f;
      const float* pre_w = !joint ? nullptr
                                  : (unit < p.n_heads ? (q_weight ? q_weight + (size_t)unit * p.dim : nullptr)
                                                      : (k_weight ? k_weight + (size_t)(unit - p.n_heads) * p.dim : nullptr));
      for (int d = lane; d < p.dim; d += 32) {
        float v = to_float(x[d]) + (b ? b[d] : 0.0f);
        if (joint) v = v * pre * (pre_w ? pre_w[d] : 1.0f);
        buf[d] = v;
      }
      __syncwarp();
      for (int i = lane; i < half; i += 32) {
        const float u = buf[i], v = buf[i + half];
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= p.rot_factor;
        cs *= p.rot_factor;
        buf[i] = u * cs - v * sn;
        buf[i + half] = v * cs + u * sn;
      }
      __syncwarp();
      float inv = 1.0f;
      if (p.unit_norm == 1) {
        float sq = 0.0f;
        for (int d = lane; d < p.dim; d += 32) sq = fmaf(buf[d], buf[d], sq);
        sq = warp_sum(sq);
        inv = 1.0f / sqrtf(sq / (float)p.dim + p.eps);
      }
      const float* q_w = joint ? nullptr : q_weight;
      const float* k_w = joint ? nullptr : k_weight;
      // (the norm's weight, one per coordinate and the same for every head, where the mixer has one)
      if (unit < p.n_heads) {
        for (int d = lane; d < p.dim; d += 32) x[d] = from_float<A>(buf[d] * inv * (q_w ? q_w[d] : 1.0f));
      } else if (slot >= 0) {
        const int kvh = unit - p.n_heads;
        C* dst = k_pool + (((size_t)page * p.n_kv + kvh) * p.page_size + offset) * p.dim;
        for (int d = lane; d < p.dim; d += 32) dst[d] = from_float<C>(buf[d] * inv * (k_w ? k_w[d] : 1.0f));
      }
      __syncwarp();
    } else {
      const int kvh = unit - qk_heads;
      const A* v = row + (size_t)qk_heads * p.dim + (size_t)kvh * p.vdim;
      const A* other = v_other ? v_other + (size_t)t * p.ld_other + (size_t)kvh * p.vdim : nullptr;
      A* keep = v_keep ? v_keep + ((size_t)t * p.n_kv + kvh) * p.vdim : nullptr;
      C* dst = slot >= 0 ? v_pool + (((size_t)page * p.n_kv + kvh) * p.page_size + offset) * p.vdim : nullptr;
      const float lam = other ? lambda[0] : 0.0f;
      const float* b = bias ? bias + (size_t)qk_heads * p.dim + (size_t)kvh * p.vdim : nullptr;
      for (int d = lane; d < p.vdim; d += 32) {
        float val = to_float(v[d]) + (b ? b[d] : 0.0f);
        if (other) val = (1.0f - lam) * val + lam * to_float(other[d]);
        if (keep) keep[d] = from_float<A>(val);
        if (dst) dst[d] = from_float<C>(val);
      }
    }
  }
}

// --- attention -------------------------------------------------------------------------------

struct SinkParams {
  int q_ld, table_stride;
  int n_heads, n_kv, dim, vdim, page_size;
  int window, keep_first;   // window 0: every earlier key is seen
  float scale, softcap;     // softcap 0: none
  int num_pages;
  // per query head, each null or float32 [n_heads]: the score is multiplied by head_scale[h], and
  // bias_a[h] * log(1 + bias_b[h] * (query position - key position)) is taken off it
  const float* head_scale;
  const float* bias_a;
  const float* bias_b;
};

template <typename A, typename C>
__global__ void __launch_bounds__(SK_WARPS * 32)
attention_sink_kernel(const A* __restrict__ q, A* __restrict__ out, const C* __restrict__ k_pool,
                      const C* __restrict__ v_pool, const int32_t* __restrict__ block_table,
                      const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ first_pos,
                      const int32_t* __restrict__ work_seq, const int32_t* __restrict__ work_row0, SinkParams p,
                      int* __restrict__ status) {
  dependents_may_launch();
  wait_for_prior_kernels();
  extern __shared__ float sk_smem[];
  const int dim = p.dim, vdim = p.vdim;
  float* q_s = sk_smem;                            // [SK_WARPS][dim]
  float* k_s = q_s + SK_WARPS * dim;               // [SK_TILE][dim + 1]
  float* v_s = k_s + SK_TILE * (dim + 1);          // [SK_TILE][vdim]

  const int w = blockIdx.x, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = work_seq[w], row0 = work_row0[w];
  const int tok0 = seq_starts[s];
  const int n_q = seq_starts[s + 1] - tok0;
  const int pos0 = first_pos[s];
  const int group = p.n_heads / p.n_kv;
  const int rows_total = n_q * group;

  const int my_row = row0 + warp;
  const bool valid = my_row < rows_total;
  const int q_local = valid ? my_row / group : 0;
  const int head = kvh * group + (valid ? my_row % group : 0);
  const int token = tok0 + q_local;
  const int qpos = pos0 + q_local;

  const int last_row = min(row0 + SK_WARPS - 1, rows_total - 1);
  const int q_lo = pos0 + row0 / group, q_hi = pos0 + last_row / group;
  const int key_hi = q_hi + 1;                                            // exclusive
  const int key_lo = p.window > 0 ? max(0, q_lo - p.window + 1) : 0;      // inclusive
  const int my_lo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
  const int keep = p.window > 0 ? p.keep_first : 0;                       // without a window every key is seen anyway

  if (valid) {
    const A* qr = q + (size_t)token * p.q_ld + (size_t)head * dim;
    for (int d = lane; d < dim; d += 32) q_s[warp * dim + d] = to_float(qr[d]);
  }

  float m = -INFINITY, l = 0.0f;
  float acc[SK_MAX_ACC];
#pragma unroll
  for (int i = 0; i < SK_MAX_ACC; ++i) acc[i] = 0.0f;

  const int32_t* table = block_table + (size_t)s * p.table_stride;
  const int first_window_tile = key_lo / SK_TILE;
  const int kept_tiles = (min(keep, key_hi) + SK_TILE - 1) / SK_TILE;     // tiles that hold kept first tokens
  for (int tile = 0; tile <= (key_hi - 1) / SK_TILE; ++tile) {
    if (tile >= kept_tiles && tile < first_window_tile) continue;         // the same for the whole block
    const int base = tile * SK_TILE;
    __syncthreads();  // previous tile fully consumed (also orders the q_s writes)
    for (int idx = threadIdx.x; idx < SK_TILE * (dim + vdim); idx += SK_WARPS * 32) {
      const bool is_k = idx < SK_TILE * dim;
      const int local = is_k ? idx : idx - SK_TILE * dim;
      const int width = is_k ? dim : vdim;
      const int j = local / width, d = local - j * width;
      const int pos = base + j;
      float val = 0.0f;
      if (pos < key_hi && (pos >= key_lo || pos < keep)) {
        const int page = checked_page(table[pos / p.page_size], p.num_pages, status);
        if (page >= 0) {
          const size_t at = (((size_t)page * p.n_kv + kvh) * p.page_size + (pos % p.page_size)) * width + d;
          val = is_k ? to_float(k_pool[at]) : to_float(v_pool[at]);
        }
      }
      if (is_k) k_s[j * (dim + 1) + d] = val;
      else v_s[j * vdim + d] = val;
    }
    __syncthreads();
    // warp-uniform: no key of this tile is visible to this row
    if (!valid || base > qpos || (base + SK_TILE <= my_lo && base >= keep)) continue;

    const int pos = base + lane;
    float sc = 0.0f;
    const float* qr = q_s + warp * dim;
    const float* kr = k_s + lane * (dim + 1);
    for (int d = 0; d < dim; ++d) sc = fmaf(qr[d], kr[d], sc);
    sc *= p.scale;
    if (p.head_scale) sc *= p.head_scale[head];
    if (p.softcap > 0.0f) sc = p.softcap * tanhf(sc / p.softcap);
    if (p.bias_a) sc -= p.bias_a[head] * log1pf(p.bias_b[head] * (float)max(qpos - pos, 0));
    const bool ok = pos <= qpos && (pos >= my_lo || pos < keep);
    sc = ok ? sc : -INFINITY;
    const float tile_max = warp_max(sc);
    if (tile_max == -INFINITY) continue;  // nothing visible in this tile
    const float new_m = fmaxf(m, tile_max);
    const float rescale = expf(m - new_m);       // m = -inf -> 0
    const float pr = ok ? expf(sc - new_m) : 0.0f;
    l = l * rescale + warp_sum(pr);
#pragma unroll
    for (int i = 0; i < SK_MAX_ACC; ++i) acc[i] *= rescale;
    for (int j = 0; j < SK_TILE; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pr, j);
      const float* vr = v_s + j * vdim;
#pragma unroll
      for (int i = 0; i < SK_MAX_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) acc[i] = fmaf(pj, vr[d], acc[i]);
      }
    }
    m = new_m;
  }

  if (valid) {
    const float denom = l > 0.0f ? l : 1.0f;
    A* o = out + (size_t)token * ((size_t)p.n_heads * vdim) + (size_t)head * vdim;
#pragma unroll
    for (int i = 0; i < SK_MAX_ACC; ++i) {
      const int d = lane + 32 * i;
      if (d < vdim) o[d] = from_float<A>(acc[i] / denom);
    }
  }
}

// --- attention on tensor cores (bfloat16, head sizes that are multiples of 16) -----------------------
//
// The rows of one (entry, key/value head) are (query token, head in group) pairs, row = token *
// group + head in group, so that all query heads of a key/value head share its tiles. One block of
// 4 warps per 64 consecutive rows; each warp owns 16 rows. Keys
// and values are walked in tiles of 64 absolute positions, aligned to multiples of 64 from position
// 0 (first the tiles that hold kept first tokens, then the window's; one range where they meet),
// double-buffered with cp.async from the pages the block table names. Both products run on
// mma.sync m16n8k16 (bfloat16 operands, float32 accumulators); scores, cap, mask, maxima, sums and
// the output accumulator are float32. The key size is a run-time number (it only sets the number
// of k-steps of the first product); the value size is a template parameter (it sizes the
// accumulator). Entries of a few rows (decode) take the same kernel, one block per entry and key/value head;
// for steps that hold nothing else the tile list of every block is cut into up to 8 shares that run
// side by side (blockIdx.z) and a second kernel merges their (maximum, sum, accumulator) states.

constexpr int SM_BM = 64, SM_BN = 64, SM_THREADS = 128, SM_PAD = 8;

struct SinkMmaParams {
  const bf16* q;
  int q_ld;
  bf16* out;
  const bf16* k_pool;
  const bf16* v_pool;
  const int32_t* block_table;
  int table_stride;
  const int32_t* seq_starts;
  const int32_t* first_pos;
  const int32_t* work_seq;
  const int32_t* work_q0;
  int n_heads, n_kv, dk, page_size, window, keep_first;
  float scale_log2, cap_log2, cap_x;   // cap c: c log2(e) and 2 scale / c log2(e); 0: no cap
  int num_pages;
  int* status;
  int num_splits;                      // > 1: blockIdx.z takes a share of the tile list and leaves its state in scratch
  float* part_o;                       // [T * H, splits, DV] unnormalised sums
  float* part_ml;                      // [T * H, splits, 2] maximum (log2 domain) and sum of weights
  const float* head_scale;             // per query head, null or [n_heads]: a factor on the score
  const float* bias_a;                 // per query head, null or [n_heads]: bias_a log(1 + bias_b distance) is taken off
  const float* bias_b;
};

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sm_cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sm_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void sm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void sm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void sm_ldm4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(sm_u32(p)));
}
__device__ __forceinline__ void sm_ldm4t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(sm_u32(p)));
}
__device__ __forceinline__ void sm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 64 rows of keys or values from absolute position `base` into a padded tile [64][d + 8]. Two
// threads share a row (its page is looked up once a thread); rows outside what the block's
// queries can see, and rows whose page was given back, are zero-filled.
__device__ __forceinline__ void sm_load_tile(bf16* tile, const bf16* pool, const int32_t* table, int base, int key_lo,
                                             int key_hi, int keep, int kvh, int n_kv, int page_size, int d, int num_pages,
                                             int* status) {
  const int row = threadIdx.x >> 1, half = threadIdx.x & 1;
  const int pos = base + row;
  const int ld = d + SM_PAD, chunks = d >> 3;
  bf16* dst = tile + row * ld;
  int page = -1;
  if (pos < key_hi && (pos >= key_lo || pos < keep)) page = checked_page(table[pos / page_size], num_pages, status);
  if (page >= 0) {
    const bf16* src = pool + (((size_t)page * n_kv + kvh) * page_size + (pos % page_size)) * d;
    for (int c = half; c < chunks; c += 2) sm_cp16(dst + c * 8, src + c * 8);
  } else {
    for (int c = half; c < chunks; c += 2) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int DV>
__global__ void __launch_bounds__(SM_THREADS) attention_sink_mma_kernel(const SinkMmaParams p) {
  dependents_may_launch();
  wait_for_prior_kernels();
  constexpr int LDV = DV + SM_PAD;
  constexpr int DTILES = DV / 8;
  const int dk = p.dk, ldk = dk + SM_PAD, ksteps = dk >> 4;
  extern __shared__ __align__(16) unsigned char sm_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(sm_raw);        // [64][ldk]
  bf16* k_s = q_s + SM_BM * ldk;                       // [2][64][ldk]
  bf16* v_s = k_s + 2 * SM_BN * ldk;                   // [2][64][LDV]

  const int s = p.work_seq[blockIdx.x], row0 = p.work_q0[blockIdx.x];
  const int kvh = blockIdx.y;
  const int group = p.n_heads / p.n_kv;
  const int tok0 = p.seq_starts[s];
  const int n_q = p.seq_starts[s + 1] - tok0;
  const int pos0 = p.first_pos[s];
  const int rows_valid = min(SM_BM, n_q * group - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  // token (in the step), query head and position of a row of this block
  auto tok_of = [=](int r) { return tok0 + (row0 + r) / group; };
  auto head_of = [=](int r) { return kvh * group + (row0 + r) % group; };
  auto qpos_of = [=](int r) { return pos0 + (row0 + r) / group; };

  const int qpos_first = qpos_of(0);
  const int key_hi = qpos_of(rows_valid - 1) + 1;                               // exclusive
  const int key_lo = p.window > 0 ? max(0, qpos_first - p.window + 1) : 0;
  const int keep = p.window > 0 ? min(p.keep_first, key_hi) : 0;
  const int tile_end = (key_hi - 1) / SM_BN;
  int window_tile = key_lo / SM_BN, kept = (keep + SM_BN - 1) / SM_BN;
  if (kept >= window_tile) {            // the kept tokens' tiles reach the window's: one range
    if (kept > 0) window_tile = 0;
    kept = 0;
  }
  const int tile_begin = window_tile, kept_tiles = kept;
  const int listed = kept_tiles + tile_end - tile_begin + 1;
  auto tile_of = [=](int j) { return j < kept_tiles ? j : tile_begin + (j - kept_tiles); };
  const int32_t* table = p.block_table + (size_t)s * p.table_stride;
  // this block's share of the tile list
  const int per_split = (listed + p.num_splits - 1) / p.num_splits;
  const int j_begin = blockIdx.z * per_split, j_end = min(listed, j_begin + per_split);
  if (j_begin >= j_end) {               // (only with splits) nothing to do: an empty state
    for (int idx = threadIdx.x; idx < rows_valid; idx += SM_THREADS) {
      const size_t at = ((size_t)tok_of(idx) * p.n_heads + head_of(idx)) * p.num_splits + blockIdx.z;
      p.part_ml[2 * at] = -INFINITY;
      p.part_ml[2 * at + 1] = 0.0f;
      for (int d = 0; d < DV; ++d) p.part_o[at * DV + d] = 0.0f;
    }
    return;
  }

  for (int idx = threadIdx.x; idx < SM_BM * (dk >> 3); idx += SM_THREADS) {
    const int row = idx / (dk >> 3), chunk = idx - row * (dk >> 3);
    bf16* dst = q_s + row * ldk + chunk * 8;
    if (row < rows_valid)
      sm_cp16(dst, p.q + (size_t)tok_of(row) * p.q_ld + (size_t)head_of(row) * dk + chunk * 8);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
  sm_load_tile(k_s, p.k_pool, table, tile_of(j_begin) * SM_BN, key_lo, key_hi, keep, kvh, p.n_kv, p.page_size, dk, p.num_pages, p.status);
  sm_load_tile(v_s, p.v_pool, table, tile_of(j_begin) * SM_BN, key_lo, key_hi, keep, kvh, p.n_kv, p.page_size, DV, p.num_pages, p.status);
  sm_commit();

  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int qpos_a = qpos_of(row_a), qpos_b = qpos_of(row_b);
  const int warp_qpos_min = qpos_of(warp * 16);
  const int warp_qpos_max = min(qpos_of(warp * 16 + 15), key_hi - 1);
  const bool warp_active = warp * 16 < rows_valid;
  // the two rows' own factors (log2 domain)
  const int head_a = head_of(row_a), head_b = head_of(row_b);
  const float hs_a = p.head_scale ? p.head_scale[head_a] : 1.0f, hs_b = p.head_scale ? p.head_scale[head_b] : 1.0f;
  const float ba_a = p.bias_a ? p.bias_a[head_a] * 1.4426950408889634f : 0.0f, ba_b = p.bias_a ? p.bias_a[head_b] * 1.4426950408889634f : 0.0f;
  const float bb_a = p.bias_a ? p.bias_b[head_a] : 0.0f, bb_b = p.bias_a ? p.bias_b[head_b] : 0.0f;

  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  for (int j = j_begin; j < j_end; ++j) {
    const int stage = (j - j_begin) & 1;
    const int base = tile_of(j) * SM_BN;
    if (j + 1 < j_end) {
      const int next = tile_of(j + 1) * SM_BN;
      sm_load_tile(k_s + (stage ^ 1) * SM_BN * ldk, p.k_pool, table, next, key_lo, key_hi, keep, kvh, p.n_kv, p.page_size, dk,
                   p.num_pages, p.status);
      sm_load_tile(v_s + (stage ^ 1) * SM_BN * LDV, p.v_pool, table, next, key_lo, key_hi, keep, kvh, p.n_kv, p.page_size, DV,
                   p.num_pages, p.status);
      sm_commit();
      sm_wait<1>();
    } else {
      sm_wait<0>();
    }
    __syncthreads();
    const bf16* kt = k_s + stage * SM_BN * ldk;
    const bf16* vt = v_s + stage * SM_BN * LDV;

    // a warp whose rows all sit before this tile, or after its window with no kept token in the tile, has nothing to do
    const bool skip = !warp_active || base > warp_qpos_max ||
                      (p.window > 0 && base + SM_BN - 1 < warp_qpos_min - p.window + 1 && base >= keep);
    if (!skip) {
      float sc[SM_BN / 8][4];
#pragma unroll
      for (int i = 0; i < SM_BN / 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
      for (int kk = 0; kk < ksteps; ++kk) {
        uint32_t a[4];
        sm_ldm4(a, q_s + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldk + kk * 16 + 8 * (lane >> 4));
#pragma unroll
        for (int jj = 0; jj < SM_BN / 16; ++jj) {
          uint32_t b[4];
          sm_ldm4(b, kt + (jj * 16 + (lane & 7) + 8 * (lane >> 4)) * ldk + kk * 16 + 8 * ((lane >> 3) & 1));
          sm_mma(sc[2 * jj], a, b[0], b[1]);
          sm_mma(sc[2 * jj + 1], a, b[2], b[3]);
        }
      }
      // scale or cap (to the log2 domain) and mask by absolute position
      float tmax_a = -INFINITY, tmax_b = -INFINITY;
#pragma unroll
      for (int i = 0; i < SM_BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float raw = sc[i][e] * ((e < 2) ? hs_a : hs_b);
          float v = raw * p.scale_log2;
          if (p.cap_log2 > 0.0f) v = p.cap_log2 * (1.0f - 2.0f / (1.0f + exp2f(raw * p.cap_x)));
          const int kpos = base + i * 8 + 2 * t4 + (e & 1);
          const int qpos = (e < 2) ? qpos_a : qpos_b;
          if (p.bias_a) v -= ((e < 2) ? ba_a : ba_b) * log1pf(((e < 2) ? bb_a : bb_b) * (float)max(qpos - kpos, 0));
          const bool ok = kpos <= qpos && (p.window == 0 || kpos > qpos - p.window || kpos < keep);
          v = ok ? v : -INFINITY;
          sc[i][e] = v;
          if (e < 2) tmax_a = fmaxf(tmax_a, v); else tmax_b = fmaxf(tmax_b, v);
        }
      }
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
      const float new_a = fmaxf(m_a, tmax_a), new_b = fmaxf(m_b, tmax_b);
      // a row with nothing visible yet keeps shift 0 so that exp2(-inf - 0) = 0
      const float shift_a = new_a == -INFINITY ? 0.0f : new_a, shift_b = new_b == -INFINITY ? 0.0f : new_b;
      const float resc_a = exp2f(m_a - shift_a), resc_b = exp2f(m_b - shift_b);
      m_a = new_a; m_b = new_b;
      float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
      for (int i = 0; i < SM_BN / 8; ++i) {
        sc[i][0] = exp2f(sc[i][0] - shift_a); sc[i][1] = exp2f(sc[i][1] - shift_a);
        sc[i][2] = exp2f(sc[i][2] - shift_b); sc[i][3] = exp2f(sc[i][3] - shift_b);
        sum_a += sc[i][0] + sc[i][1];
        sum_b += sc[i][2] + sc[i][3];
      }
      l_a = l_a * resc_a + sum_a;
      l_b = l_b * resc_b + sum_b;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { o[i][0] *= resc_a; o[i][1] *= resc_a; o[i][2] *= resc_b; o[i][3] *= resc_b; }
#pragma unroll
      for (int kk = 0; kk < SM_BN / 16; ++kk) {
        uint32_t a[4];
        a[0] = sm_pack(sc[2 * kk][0], sc[2 * kk][1]);
        a[1] = sm_pack(sc[2 * kk][2], sc[2 * kk][3]);
        a[2] = sm_pack(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
        a[3] = sm_pack(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int dd = 0; dd < DTILES / 2; ++dd) {
          uint32_t b[4];
          sm_ldm4t(b, vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDV + dd * 16 + 8 * (lane >> 4));
          sm_mma(o[2 * dd], a, b[0], b[1]);
          sm_mma(o[2 * dd + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (p.num_splits > 1) {
    // this share's state: the merge kernel folds the shares of a row in ascending order
    if (row_a < rows_valid) {
      const size_t at = ((size_t)tok_of(row_a) * p.n_heads + head_of(row_a)) * p.num_splits + blockIdx.z;
      if (t4 == 0) { p.part_ml[2 * at] = m_a; p.part_ml[2 * at + 1] = l_a; }
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { p.part_o[at * DV + i * 8 + 2 * t4] = o[i][0]; p.part_o[at * DV + i * 8 + 2 * t4 + 1] = o[i][1]; }
    }
    if (row_b < rows_valid) {
      const size_t at = ((size_t)tok_of(row_b) * p.n_heads + head_of(row_b)) * p.num_splits + blockIdx.z;
      if (t4 == 0) { p.part_ml[2 * at] = m_b; p.part_ml[2 * at + 1] = l_b; }
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { p.part_o[at * DV + i * 8 + 2 * t4] = o[i][2]; p.part_o[at * DV + i * 8 + 2 * t4 + 1] = o[i][3]; }
    }
    return;
  }
  const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
  const size_t out_stride = (size_t)p.n_heads * DV;
  if (row_a < rows_valid) {
    bf16* dst = p.out + (size_t)tok_of(row_a) * out_stride + (size_t)head_of(row_a) * DV;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = sm_pack(o[i][0] * inv_a, o[i][1] * inv_a);
  }
  if (row_b < rows_valid) {
    bf16* dst = p.out + (size_t)tok_of(row_b) * out_stride + (size_t)head_of(row_b) * DV;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = sm_pack(o[i][2] * inv_b, o[i][3] * inv_b);
  }
}

// out[row, d] = sum_z o_z 2^(m_z - M) / sum_z l_z 2^(m_z - M) over the shares z of a row, M their largest maximum.
__global__ void sink_mma_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                      long long rows, int dv, int splits) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * dv) return;
  const long long row = i / dv;
  const int d = (int)(i - row * dv);
  float m = -INFINITY;
  for (int z = 0; z < splits; ++z) m = fmaxf(m, part_ml[2 * (row * splits + z)]);
  float l = 0.0f, acc = 0.0f;
  if (m > -INFINITY) {
    for (int z = 0; z < splits; ++z) {
      const float f = exp2f(part_ml[2 * (row * splits + z)] - m);
      l += part_ml[2 * (row * splits + z) + 1] * f;
      acc += part_o[(row * splits + z) * dv + d] * f;
    }
  }
  out[i] = from_float<bf16>(l > 0.0f ? acc / l : 0.0f);
}

}  // namespace pkv

using namespace pkv;

template <typename A, typename C>
static int launch_prepare(void* qkv, const int32_t* positions, const float* freq, const float* q_weight, const float* k_weight,
                          const float* bias, const void* v_other, const float* lambda,
                          void* v_keep, void* k_pool, void* v_pool, const int32_t* slots, const PrepareParams& p, int tokens,
                          int* status, cudaStream_t s) {
  const size_t smem = ((size_t)SK_WARPS * p.dim + 32) * sizeof(float);
  return launch_kernel(qkv_prepare_kernel<A, C>, dim3(tokens), dim3(SK_WARPS * 32), smem, s, true, 0, (A*)qkv, positions, freq,
                       q_weight, k_weight, bias, (const A*)v_other, lambda, (A*)v_keep, (C*)k_pool, (C*)v_pool, slots, p, status);
}

// qkv [tokens, ld]: H query heads of `dim`, G key heads of `dim`, G value heads of `vdim`.
// freq [rot_dims / 2] float32 (null with rot_dims 0). q_weight, k_weight: float32 [dim] factors on
// the unit-norm query and key heads, or null; with unit_norm 2 (one norm over all query columns, one
// over all key columns, before the rotation) float32 [H * dim] and [G * dim]. bias: float32 [H dim + G
// dim + G vdim] added to the columns first, or null. v_other: the values [tokens, ld_other] of
// another layer to blend with, weight lambda[0] (a float on the device), or null. v_keep: where
// to leave this layer's values [tokens, G * vdim] as they are cached, or null.
// k_pool [pages][G][page_size][dim], v_pool [pages][G][page_size][vdim]; slots: int32 per token,
// negative (or null): nothing is cached for it.
PKV_EXPORT int pkv_qkv_prepare(void* qkv, int act_dtype, int ld, const int32_t* positions, const float* freq, int rot_dims,
                               float rot_factor, float eps, int unit_norm, const float* q_weight, const float* k_weight,
                               const float* bias, const void* v_other, int ld_other,
                               const float* lambda, void* v_keep, void* k_pool, void* v_pool, int cache_dtype,
                               const int32_t* slots, long long pool_slots, int tokens, int n_heads, int n_kv, int dim, int vdim,
                               int page_size, int* status, void* stream) {
  if (tokens <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || dim <= 0 || vdim <= 0 || page_size <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > dim ||
      ld < (n_heads + n_kv) * dim + n_kv * vdim || (v_other && (!lambda || ld_other < n_kv * vdim)) || (rot_dims && !freq))
    return PKV_ERR_SIZE;
  if (dim > SK_MAX_DIM) return PKV_ERR_LIMIT;
  PrepareParams p{ld, n_heads, n_kv, dim, vdim, rot_dims, rot_factor, eps, unit_norm, page_size, pool_slots, ld_other};
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_PREP(A, C) \
  return launch_prepare<A, C>(qkv, positions, freq, q_weight, k_weight, bias, v_other, lambda, v_keep, k_pool, v_pool, slots, p, tokens, status, s)
  if (act_dtype == PKV_F32 && cache_dtype == PKV_F32) PKV_PREP(float, float);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16) PKV_PREP(bf16, bf16);
  if (act_dtype == PKV_F32 && cache_dtype == PKV_BF16) PKV_PREP(float, bf16);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_F32) PKV_PREP(bf16, float);
#undef PKV_PREP
  return PKV_ERR_DTYPE;
}

template <typename A, typename C>
static int launch_sink(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* block_table,
                       const int32_t* seq_starts, const int32_t* first_pos, const int32_t* work_seq,
                       const int32_t* work_row0, int n_work, const SinkParams& p, int* status, cudaStream_t s) {
  const size_t smem = ((size_t)SK_WARPS * p.dim + (size_t)SK_TILE * (p.dim + 1) + (size_t)SK_TILE * p.vdim) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_sink_kernel<A, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_work, p.n_kv);
  return launch_kernel(attention_sink_kernel<A, C>, grid, dim3(SK_WARPS * 32), smem, s, true, 0, (const A*)q, (A*)out,
                       (const C*)k_pool, (const C*)v_pool, block_table, seq_starts, first_pos, work_seq, work_row0, p, status);
}

// Rows per work item, for the host that builds the work list.
PKV_EXPORT int pkv_attention_sink_rows_per_block() { return SK_WARPS; }

PKV_EXPORT int pkv_attention_sink(const void* q, int q_ld, void* out, int act_dtype, const void* k_pool, const void* v_pool,
                                  int cache_dtype, const int32_t* block_table, int table_stride, const int32_t* seq_starts,
                                  const int32_t* first_pos, const int32_t* work_seq, const int32_t* work_row0, int n_work,
                                  int n_heads, int n_kv, int dim, int vdim, int page_size, int window, int keep_first,
                                  float scale, float softcap, const float* head_scale, const float* bias_a,
                                  const float* bias_b, int num_pages, int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || dim <= 0 || vdim <= 0 || page_size <= 0 || window < 0 || keep_first < 0 ||
      num_pages <= 0 || softcap < 0.0f || (bias_a == nullptr) != (bias_b == nullptr))
    return PKV_ERR_SIZE;
  if (vdim > 32 * SK_MAX_ACC || dim > SK_MAX_DIM || n_kv > 65535) return PKV_ERR_LIMIT;
  SinkParams p{q_ld, table_stride, n_heads, n_kv, dim, vdim, page_size, window, keep_first, scale, softcap, num_pages,
               head_scale, bias_a, bias_b};
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_SINK(A, C) \
  return launch_sink<A, C>(q, out, k_pool, v_pool, block_table, seq_starts, first_pos, work_seq, work_row0, n_work, p, status, s)
  if (act_dtype == PKV_F32 && cache_dtype == PKV_F32) PKV_SINK(float, float);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16) PKV_SINK(bf16, bf16);
  if (act_dtype == PKV_F32 && cache_dtype == PKV_BF16) PKV_SINK(float, bf16);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_F32) PKV_SINK(bf16, float);
#undef PKV_SINK
  return PKV_ERR_DTYPE;
}

template <int DV>
static int launch_sink_mma(const SinkMmaParams& p, int n_work, cudaStream_t s) {
  const size_t smem = ((size_t)3 * SM_BM * (p.dk + SM_PAD) + (size_t)2 * SM_BN * (DV + SM_PAD)) * sizeof(bf16);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_sink_mma_kernel<DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int rc = launch_kernel(attention_sink_mma_kernel<DV>, dim3(n_work, p.n_kv, p.num_splits), dim3(SM_THREADS), smem, s,
                               true, 0, p);
  return rc;
}

// 1 when the tensor-core kernel takes these sizes (bfloat16 only): key and value sizes that are
// multiples of 16, values of at most 128, keys of at most 256, query rows on 16-byte boundaries.
PKV_EXPORT int pkv_attention_sink_mma_supports(int dk, int dv, int q_ld) {
  return (dk >= 16 && dk <= 256 && dk % 16 == 0 && dv >= 16 && dv <= 128 && dv % 16 == 0 && q_ld % 8 == 0) ? 1 : 0;
}

PKV_EXPORT int pkv_attention_sink_mma_rows() { return SM_BM; }

// The work list is in blocks of 64 rows of an (entry, key/value head): row = token * (H / G) + head in
// group; work_q0 is the block's first row.
PKV_EXPORT int pkv_attention_sink_mma(const void* q, int q_ld, void* out, const void* k_pool, const void* v_pool,
                                      const int32_t* block_table, int table_stride, const int32_t* seq_starts,
                                      const int32_t* first_pos, const int32_t* work_seq, const int32_t* work_q0, int n_work,
                                      int n_heads, int n_kv, int dk, int dv, int page_size, int window, int keep_first,
                                      float scale, float softcap, const float* head_scale, const float* bias_a,
                                      const float* bias_b, int num_pages, int* status, int num_splits, float* part_o,
                                      float* part_ml, long long tokens, void* stream) {
  if (n_work <= 0) return 0;
  if (!pkv_attention_sink_mma_supports(dk, dv, q_ld)) return PKV_ERR_LIMIT;
  if (num_splits < 1 || num_splits > 8 || (num_splits > 1 && (!part_o || !part_ml))) return PKV_ERR_SIZE;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0 || window < 0 || keep_first < 0 || num_pages <= 0 ||
      softcap < 0.0f || !(scale > 0.0f) || n_kv > 65535 || (bias_a == nullptr) != (bias_b == nullptr))
    return PKV_ERR_SIZE;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)out % 4) return PKV_ERR_ALIGN;
  const float log2e = 1.4426950408889634f;
  SinkMmaParams p{(const bf16*)q, q_ld, (bf16*)out, (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_stride,
                  seq_starts, first_pos, work_seq, work_q0, n_heads, n_kv, dk, page_size, window, keep_first, scale * log2e,
                  softcap * log2e, softcap > 0.0f ? 2.0f * scale / softcap * log2e : 0.0f, num_pages, status, num_splits, part_o,
                  part_ml, head_scale, bias_a, bias_b};
  cudaStream_t s = (cudaStream_t)stream;
  int rc = PKV_ERR_LIMIT;
  switch (dv) {
    case 16: rc = launch_sink_mma<16>(p, n_work, s); break;
    case 32: rc = launch_sink_mma<32>(p, n_work, s); break;
    case 48: rc = launch_sink_mma<48>(p, n_work, s); break;
    case 64: rc = launch_sink_mma<64>(p, n_work, s); break;
    case 80: rc = launch_sink_mma<80>(p, n_work, s); break;
    case 96: rc = launch_sink_mma<96>(p, n_work, s); break;
    case 112: rc = launch_sink_mma<112>(p, n_work, s); break;
    case 128: rc = launch_sink_mma<128>(p, n_work, s); break;
  }
  if (rc != 0 || num_splits == 1) return rc;
  const long long rows = tokens * n_heads;
  return launch_kernel(sink_mma_merge_kernel, dim3((unsigned)((rows * dv + 255) / 256)), dim3(256), 0, s, true, 0,
                       (const float*)part_o, (const float*)part_ml, (bf16*)out, rows, dv, num_splits);
}
