// Attention over a cached latent: every position caches ONE vector [rank + rot] for all heads,
// the RMS-normalised latent c (rank entries) followed by a rotated key part (rot entries). In the
// absorbed form a head's query is [rank + rot] too (its unrotated part already multiplied by the
// head's key up-projection), the score is q . cached * scale, and the value of a position is the
// latent itself; the head's value up-projection is applied to the result by the caller.
//
//   latent_prepare   per token: the query latent and the key/value latent are RMS-normalised
//                    (float32), the shared key part is rotated by the token's position, and the
//                    cache row [c | rotated part] is written at the token's slot.
//   latent_attention rows are (token, head) pairs of an entry, row = token * heads + head; a block
//                    of 8 warps takes 8 consecutive rows and walks the keys in tiles of 32 absolute
//                    positions, staged once in shared memory for all rows. Tiles are aligned to
//                    multiples of 32 from position 0 and folded in ascending order; a masked key
//                    adds exactly zero: a row's result does not depend on how the batch was cut.
//                    The query's rotated part is rotated here, by the query's own position. The
//                    result may be multiplied by sigmoid of a per-(token, head) gate.
// Rotation: coordinate i of the rotated part pairs with i + dims/2 for i < dims/2 (the rest of the
// part passes unchanged); the angle is position * freq[i], computed in float32.
#include "common.cuh"

namespace pkv {

constexpr int LAT_WARPS = 8;
constexpr int LAT_TILE = 32;
constexpr int LAT_MAX_ACC = 16;   // rank <= 32 * 16

__device__ __forceinline__ float rotated(const float* part, int i, int dims, const float* freq, float position) {
  // value of coordinate i of `part` after the rotation (float32 angle)
  const int half = dims >> 1;
  if (i >= dims) return part[i];
  float sn, cs;
  if (i < half) {
    sincosf(position * freq[i], &sn, &cs);
    return part[i] * cs - part[i + half] * sn;
  }
  sincosf(position * freq[i - half], &sn, &cs);
  return part[i] * cs + part[i - half] * sn;
}

// fused: float32 [tokens, ld]: columns [q_off, q_off + q_rank) the query latent before its norm,
// [kv_off, kv_off + rank) the key/value latent before its norm, then rot columns of key part.
template <typename C>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ fused, int ld, int q_off, int q_rank, int kv_off, int rank, int rot,
                      int rot_dims, const float* __restrict__ q_weight, const float* __restrict__ kv_weight,
                      const float* __restrict__ freq, float eps, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ slots, C* __restrict__ c_q, C* __restrict__ pool, long long pool_rows,
                      int* __restrict__ status) {
  extern __shared__ float sh[];        // [rot] the key part, then 32 floats of scratch
  float* part = sh;
  float* scratch = sh + rot;
  const int t = blockIdx.x;
  const float* row = fused + (size_t)t * ld;
  float ss = 0.0f;
  if (q_rank > 0) {                                       // (0: the queries are not low-rank, there is no query latent)
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[q_off + i], row[q_off + i], ss);
    ss = block_sum(ss, scratch);
    const float q_inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      c_q[(size_t)t * q_rank + i] = from_float<C>(row[q_off + i] * q_inv * q_weight[i]);
  }
  const long long slot = slots ? slots[t] : -1;
  if (slot < 0) return;                                   // a stand-in token, or a call that does not write
  if (slot >= pool_rows) {
    if (threadIdx.x == 0) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    return;
  }
  ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(row[kv_off + i], row[kv_off + i], ss);
  for (int i = threadIdx.x; i < rot; i += blockDim.x) part[i] = row[kv_off + rank + i];
  ss = block_sum(ss, scratch);                            // (its barriers also publish `part`)
  const float kv_inv = 1.0f / sqrtf(ss / (float)rank + eps);
  C* dst = pool + (size_t)slot * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<C>(row[kv_off + i] * kv_inv * kv_weight[i]);
  const float position = (float)positions[t];
  for (int i = threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = from_float<C>(rotated(part, i, rot_dims, freq, position));
}

// q_lat: [heads, tokens, rank] (the absorbed unrotated part), Q element type float32 or bfloat16.
// q_rot: rows of the query projection, A element type: the rotated part of head h of token t
//        starts at q_rot + t * q_rot_ld + h * q_rot_head_stride.
// out:   [heads, tokens, rank] in A.
template <typename Q, typename A, typename C>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_attention_kernel(const Q* __restrict__ q_lat, const A* __restrict__ q_rot, int q_rot_ld, int q_rot_head_stride,
                        A* __restrict__ out, const C* __restrict__ pool, const int32_t* __restrict__ block_table,
                        int table_stride, const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ first_pos,
                        const int32_t* __restrict__ work_seq, const int32_t* __restrict__ work_row0,
                        const float* __restrict__ freq, const float* __restrict__ gate, int gate_ld, int tokens, int heads,
                        int rank, int rot, int rot_dims, int page_size, int window, float scale, int num_pages,
                        int* __restrict__ status) {
  extern __shared__ float smem[];
  const int dk = rank + rot;
  float* q_s = smem;                       // [LAT_WARPS][dk]
  float* k_s = q_s + LAT_WARPS * dk;       // [LAT_TILE][dk + 1]

  const int w = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = work_seq[w], row0 = work_row0[w];
  const int tok0 = seq_starts[s];
  const int n_q = seq_starts[s + 1] - tok0;
  const int pos0 = first_pos[s];
  const int rows_total = n_q * heads;

  const int my_row = row0 + warp;
  const bool valid = my_row < rows_total;
  const int q_local = valid ? my_row / heads : 0;
  const int head = valid ? my_row % heads : 0;
  const int token = tok0 + q_local;
  const int qpos = pos0 + q_local;

  const int last_row = min(row0 + LAT_WARPS - 1, rows_total - 1);
  const int q_lo = pos0 + row0 / heads, q_hi = pos0 + last_row / heads;
  const int key_hi = q_hi + 1;                                        // exclusive
  const int key_lo = window > 0 ? max(0, q_lo - window + 1) : 0;      // inclusive
  const int my_lo = window > 0 ? max(0, qpos - window + 1) : 0;

  if (valid) {
    const Q* ql = q_lat + ((size_t)head * tokens + token) * rank;
    for (int d = lane; d < rank; d += 32) q_s[warp * dk + d] = to_float(ql[d]);
    const A* qr = q_rot + (size_t)token * q_rot_ld + (size_t)head * q_rot_head_stride;
    // the unrotated values first (each lane reads what it and its partner lane need from global)
    const int half = rot_dims >> 1;
    const float position = (float)qpos;
    for (int i = lane; i < rot; i += 32) {
      float v = to_float(qr[i]);
      if (i < rot_dims) {
        float sn, cs;
        if (i < half) {
          sincosf(position * freq[i], &sn, &cs);
          v = v * cs - to_float(qr[i + half]) * sn;
        } else {
          sincosf(position * freq[i - half], &sn, &cs);
          v = v * cs + to_float(qr[i - half]) * sn;
        }
      }
      q_s[warp * dk + rank + i] = v;
    }
  }

  float m = -INFINITY, l = 0.0f;
  float acc[LAT_MAX_ACC];
#pragma unroll
  for (int i = 0; i < LAT_MAX_ACC; ++i) acc[i] = 0.0f;

  const int32_t* table = block_table + (size_t)s * table_stride;
  for (int tile = key_lo / LAT_TILE; tile <= (key_hi - 1) / LAT_TILE; ++tile) {
    const int base = tile * LAT_TILE;
    __syncthreads();  // previous tile fully consumed (also orders the q_s writes)
    for (int idx = threadIdx.x; idx < LAT_TILE * dk; idx += LAT_WARPS * 32) {
      const int j = idx / dk, d = idx - j * dk;
      const int pos = base + j;
      float kv = 0.0f;
      if (pos >= key_lo && pos < key_hi) {
        const int page = checked_page(table[pos / page_size], num_pages, status);
        if (page >= 0) kv = to_float(pool[((size_t)page * page_size + (pos % page_size)) * dk + d]);
      }
      k_s[j * (dk + 1) + d] = kv;
    }
    __syncthreads();
    if (!valid || base > qpos || base + LAT_TILE <= my_lo) continue;  // warp-uniform

    const int pos = base + lane;
    float sc = 0.0f;
    const float* qr = q_s + warp * dk;
    const float* kr = k_s + lane * (dk + 1);
    for (int d = 0; d < dk; ++d) sc = fmaf(qr[d], kr[d], sc);
    sc *= scale;
    const bool ok = pos <= qpos && pos >= my_lo;
    sc = ok ? sc : -INFINITY;
    const float tile_max = warp_max(sc);
    if (tile_max == -INFINITY) continue;  // nothing visible in this tile
    const float new_m = fmaxf(m, tile_max);
    const float rescale = expf(m - new_m);       // m = -inf -> 0
    const float p = ok ? expf(sc - new_m) : 0.0f;
    l = l * rescale + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LAT_MAX_ACC; ++i) acc[i] *= rescale;
    for (int j = 0; j < LAT_TILE; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vr = k_s + j * (dk + 1);
#pragma unroll
      for (int i = 0; i < LAT_MAX_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) acc[i] = fmaf(pj, vr[d], acc[i]);
      }
    }
    m = new_m;
  }

  if (valid) {
    float factor = 1.0f / (l > 0.0f ? l : 1.0f);
    if (gate) factor *= 1.0f / (1.0f + expf(-gate[(size_t)token * gate_ld + head]));
    A* o = out + ((size_t)head * tokens + token) * rank;
#pragma unroll
    for (int i = 0; i < LAT_MAX_ACC; ++i) {
      const int d = lane + 32 * i;
      if (d < rank) o[d] = from_float<A>(acc[i] * factor);
    }
  }
}


// ---------------------------------------------------------------------------------------------
// The tensor-core form for bfloat16: one block of 8 warps per 128 consecutive rows of an entry
// (each warp 16 rows; 4 warps and 64 rows where the larger block's shared memory does not fit), keys in tiles of 32 absolute positions aligned to multiples of 32 from
// position 0, double-buffered with cp.async from the pages the block table names. S = Q K^T and
// O += P V run on mma.sync m16n8k16 with float32 accumulators; the values of a tile are the
// first `rank` columns of its keys, read from the same shared-memory tile (transposed loads).
// A block accumulates VT of the `rank` value columns (grid.y blocks share the rows when
// rank > VT and each computes the scores again). Scores, maxima, sums and exponentials are
// float32; queries and probabilities enter the products as bfloat16.
// ---------------------------------------------------------------------------------------------
constexpr int LM_BN = 32;
constexpr int LM_PAD = 8;
constexpr size_t LM_SMEM_LIMIT = 227 * 1024;

__device__ __forceinline__ uint32_t lm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(lm_smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void lm_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lm_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(lm_smem_u32(p)));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(lm_smem_u32(p)));
}
__device__ __forceinline__ void lm_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct LatentParams {
  const void* q_lat;            // [heads, tokens, rank], float32 or bfloat16
  const bf16* q_rot;            // rotated part of head h of token t at q_rot + t * q_rot_ld + h * q_rot_head_stride
  int q_rot_ld, q_rot_head_stride;
  bf16* out;                    // [heads, tokens, rank]
  const bf16* pool;             // [pages, page_size, rank + rot]
  const int32_t* block_table;
  int table_stride;
  const int32_t* seq_starts;
  const int32_t* first_pos;
  const int32_t* work_seq;
  const int32_t* work_row0;
  const float* freq;
  const float* gate;
  int gate_ld, tokens, heads, rank, rot, rot_dims, page_size, window;
  float scale_log2;
  int num_pages;
  int* status;
  // With num_splits > 1 the key range of a block is cut into that many parts (blockIdx.z); every part
  // leaves its unnormalised sums [split][heads * tokens][rank] and (maximum, sum) [split][heads * tokens][2],
  // and a second kernel merges them.
  int num_splits;
  float* part_o;
  float* part_ml;
};

template <int LM_THREADS>
__device__ __forceinline__ void lm_load_tile(bf16* tile, const LatentParams& p, const int32_t* table, int base, int key_lo,
                                             int key_hi, int dk, int ld) {
  const int chunks = dk >> 3;
  for (int idx = threadIdx.x; idx < LM_BN * chunks; idx += LM_THREADS) {
    const int row = idx / chunks, chunk = idx - row * chunks;
    const int pos = base + row;
    bf16* dst = tile + row * ld + chunk * 8;
    int page = -1;
    if (pos >= key_lo && pos < key_hi) page = checked_page(table[pos / p.page_size], p.num_pages, p.status);
    if (page >= 0)
      lm_cp_async16(dst, p.pool + ((size_t)page * p.page_size + (pos % p.page_size)) * dk + chunk * 8);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int VT, typename Q, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) latent_attention_mma_kernel(const LatentParams p) {
  constexpr int DTILES = VT / 8;
  constexpr int LM_BM = WARPS * 16;
  constexpr int LM_THREADS = WARPS * 32;
  extern __shared__ __align__(16) unsigned char lm_smem[];
  const int dk = p.rank + p.rot;
  const int ld = dk + LM_PAD;
  bf16* q_s = reinterpret_cast<bf16*>(lm_smem);     // [LM_BM][ld]
  bf16* k_s = q_s + LM_BM * ld;                      // [2][LM_BN][ld]

  const int s = p.work_seq[blockIdx.x], row0 = p.work_row0[blockIdx.x];
  const int v0 = blockIdx.y * VT;                    // first value column of this block
  const int tok0 = p.seq_starts[s];
  const int n_q = p.seq_starts[s + 1] - tok0;
  const int pos0 = p.first_pos[s];
  const int heads = p.heads;
  const int rows_total = n_q * heads;
  const int rows_valid = min(LM_BM, rows_total - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int q_first = pos0 + row0 / heads;
  const int q_last = pos0 + (row0 + rows_valid - 1) / heads;
  const int key_hi = q_last + 1;                                              // exclusive
  const int key_lo = p.window > 0 ? max(0, q_first - p.window + 1) : 0;
  int tile_begin = key_lo / LM_BN, tile_end = (key_hi - 1) / LM_BN;           // inclusive
  if (p.num_splits > 1) {
    const int per_split = (tile_end - tile_begin + p.num_splits) / p.num_splits;
    tile_begin += (int)blockIdx.z * per_split;
    tile_end = min(tile_end, tile_begin + per_split - 1);                     // may leave no tile at all
  }
  const int32_t* table = p.block_table + (size_t)s * p.table_stride;

  if (tile_begin <= tile_end) lm_load_tile<LM_THREADS>(k_s, p, table, tile_begin * LM_BN, key_lo, key_hi, dk, ld);
  lm_cp_async_commit();

  // the queries of this block: absorbed part as it is, rotated part rotated by the row's position
  {
    const Q* q_lat = reinterpret_cast<const Q*>(p.q_lat);
    const int half = p.rot_dims >> 1;
    // (only the 16-row tiles that hold a valid row are ever read: a decode entry stages one tile, not the block's all)
    const int rows_staged = min(LM_BM, (rows_valid + 15) & ~15);
    for (int idx = threadIdx.x; idx < rows_staged * dk; idx += LM_THREADS) {
      const int row = idx / dk, d = idx - row * dk;
      float v = 0.0f;
      if (row < rows_valid) {
        const int r = row0 + row;
        const int token = tok0 + r / heads, head = r % heads;
        if (d < p.rank) {
          v = to_float(q_lat[((size_t)head * p.tokens + token) * p.rank + d]);
        } else {
          const int i = d - p.rank;
          const bf16* qr = p.q_rot + (size_t)token * p.q_rot_ld + (size_t)head * p.q_rot_head_stride;
          v = to_float(qr[i]);
          if (i < p.rot_dims) {
            const float position = (float)(pos0 + r / heads);
            float sn, cs;
            if (i < half) {
              sincosf(position * p.freq[i], &sn, &cs);
              v = v * cs - to_float(qr[i + half]) * sn;
            } else {
              sincosf(position * p.freq[i - half], &sn, &cs);
              v = v * cs + to_float(qr[i - half]) * sn;
            }
          }
        }
      }
      q_s[row * ld + d] = __float2bfloat16_rn(v);
    }
  }

  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int qpos_a = pos0 + (row0 + row_a) / heads, qpos_b = pos0 + (row0 + row_b) / heads;
  const int warp_qpos_min = pos0 + (row0 + warp * 16) / heads;
  const int warp_qpos_max = pos0 + min(row0 + warp * 16 + 15, rows_total - 1) / heads;
  const bool warp_active = warp * 16 < rows_valid;
  const int ksteps = dk >> 4;

  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  for (int tile = tile_begin; tile <= tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    const int base = tile * LM_BN;
    if (tile < tile_end) {
      lm_load_tile<LM_THREADS>(k_s + (stage ^ 1) * LM_BN * ld, p, table, base + LM_BN, key_lo, key_hi, dk, ld);
      lm_cp_async_commit();
      lm_cp_async_wait<1>();
    } else {
      lm_cp_async_wait<0>();
    }
    __syncthreads();            // the tile (and, the first time, the queries) are in shared memory
    const bf16* kt = k_s + stage * LM_BN * ld;

    const bool skip = !warp_active || base > warp_qpos_max ||
                      (p.window > 0 && base + LM_BN - 1 < warp_qpos_min - p.window + 1);
    if (!skip) {
      float sc[LM_BN / 8][4];
#pragma unroll
      for (int j = 0; j < LM_BN / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
      for (int kk = 0; kk < ksteps; ++kk) {
        uint32_t a[4];
        lm_ldmatrix_x4(a, q_s + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ld + kk * 16 + 8 * (lane >> 4));
#pragma unroll
        for (int jj = 0; jj < LM_BN / 16; ++jj) {
          uint32_t b[4];
          lm_ldmatrix_x4(b, kt + (jj * 16 + (lane & 7) + 8 * (lane >> 4)) * ld + kk * 16 + 8 * ((lane >> 3) & 1));
          lm_mma_bf16(sc[2 * jj], a, b[0], b[1]);
          lm_mma_bf16(sc[2 * jj + 1], a, b[2], b[3]);
        }
      }
      const bool need_mask = base + LM_BN - 1 > warp_qpos_min || (p.window > 0 && base < warp_qpos_max - p.window + 1);
      float tmax_a = -INFINITY, tmax_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < LM_BN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sc[j][e] * p.scale_log2;
          if (need_mask) {
            const int kpos = base + j * 8 + 2 * t4 + (e & 1);
            const int qpos = (e < 2) ? qpos_a : qpos_b;
            const bool ok = kpos <= qpos && (p.window == 0 || kpos > qpos - p.window);
            v = ok ? v : -INFINITY;
          }
          sc[j][e] = v;
          if (e < 2) tmax_a = fmaxf(tmax_a, v); else tmax_b = fmaxf(tmax_b, v);
        }
      }
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
      const float new_a = fmaxf(m_a, tmax_a), new_b = fmaxf(m_b, tmax_b);
      const float shift_a = new_a == -INFINITY ? 0.0f : new_a, shift_b = new_b == -INFINITY ? 0.0f : new_b;
      const float resc_a = exp2f(m_a - shift_a), resc_b = exp2f(m_b - shift_b);
      m_a = new_a; m_b = new_b;
      float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
      for (int j = 0; j < LM_BN / 8; ++j) {
        sc[j][0] = exp2f(sc[j][0] - shift_a); sc[j][1] = exp2f(sc[j][1] - shift_a);
        sc[j][2] = exp2f(sc[j][2] - shift_b); sc[j][3] = exp2f(sc[j][3] - shift_b);
        sum_a += sc[j][0] + sc[j][1];
        sum_b += sc[j][2] + sc[j][3];
      }
      l_a = l_a * resc_a + sum_a;
      l_b = l_b * resc_b + sum_b;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { o[i][0] *= resc_a; o[i][1] *= resc_a; o[i][2] *= resc_b; o[i][3] *= resc_b; }
#pragma unroll
      for (int kk = 0; kk < LM_BN / 16; ++kk) {
        uint32_t a[4];
        a[0] = lm_pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
        a[1] = lm_pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
        a[2] = lm_pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
        a[3] = lm_pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int dd = 0; dd < DTILES / 2; ++dd) {
          if (v0 + dd * 16 < p.rank) {             // (rank is a multiple of 16: whole groups of columns)
            uint32_t b[4];
            lm_ldmatrix_x4_trans(b, kt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ld + v0 + dd * 16 + 8 * (lane >> 4));
            lm_mma_bf16(o[2 * dd], a, b[0], b[1]);
            lm_mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
  }

  lm_cp_async_wait<0>();
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (p.num_splits > 1) {
    const size_t all_rows = (size_t)heads * p.tokens;
#pragma unroll
    for (int half_rows = 0; half_rows < 2; ++half_rows) {
      const int row = half_rows ? row_b : row_a;
      if (row >= rows_valid) continue;
      const int r = row0 + row;
      const size_t at = (size_t)(r % heads) * p.tokens + (tok0 + r / heads);
      float* dst = p.part_o + ((size_t)blockIdx.z * all_rows + at) * p.rank + v0;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        if (v0 + i * 8 < p.rank) {
          dst[i * 8 + 2 * t4] = half_rows ? o[i][2] : o[i][0];
          dst[i * 8 + 2 * t4 + 1] = half_rows ? o[i][3] : o[i][1];
        }
      }
      if (t4 == 0 && blockIdx.y == 0) {
        float* ml = p.part_ml + ((size_t)blockIdx.z * all_rows + at) * 2;
        ml[0] = half_rows ? m_b : m_a;
        ml[1] = half_rows ? l_b : l_a;
      }
    }
    return;
  }
  float f_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, f_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
#pragma unroll
  for (int half_rows = 0; half_rows < 2; ++half_rows) {
    const int row = half_rows ? row_b : row_a;
    if (row >= rows_valid) continue;
    const int r = row0 + row;
    const int token = tok0 + r / heads, head = r % heads;
    float f = half_rows ? f_b : f_a;
    if (p.gate) f *= 1.0f / (1.0f + expf(-p.gate[(size_t)token * p.gate_ld + head]));
    bf16* dst = p.out + ((size_t)head * p.tokens + token) * p.rank + v0;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      if (v0 + i * 8 < p.rank) {
        const float x = half_rows ? o[i][2] : o[i][0], y = half_rows ? o[i][3] : o[i][1];
        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = lm_pack_bf16(x * f, y * f);
      }
    }
  }
}


// Merges the parts of a split launch: out[row] = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s, times
// sigmoid of the row's gate. One block per (head, token) row.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                    const float* __restrict__ gate, int gate_ld, int tokens, int heads, int rank, int splits) {
  const size_t row = blockIdx.x;                     // head * tokens + token
  const size_t all_rows = (size_t)heads * tokens;
  float m = -INFINITY;
  for (int z = 0; z < splits; ++z) m = fmaxf(m, part_ml[((size_t)z * all_rows + row) * 2]);
  float l = 0.0f;
  for (int z = 0; z < splits; ++z) {
    const float* ml = part_ml + ((size_t)z * all_rows + row) * 2;
    if (ml[0] != -INFINITY) l += exp2f(ml[0] - m) * ml[1];
  }
  float f = l > 0.0f ? 1.0f / l : 0.0f;
  if (gate) {
    const int head = (int)(row / tokens), token = (int)(row % tokens);
    f *= 1.0f / (1.0f + expf(-gate[(size_t)token * gate_ld + head]));
  }
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.0f;
    for (int z = 0; z < splits; ++z) {
      const float mz = part_ml[((size_t)z * all_rows + row) * 2];
      if (mz != -INFINITY) acc += exp2f(mz - m) * part_o[((size_t)z * all_rows + row) * rank + d];
    }
    out[row * rank + d] = __float2bfloat16_rn(acc * f);
  }
}

}  // namespace pkv

using namespace pkv;

PKV_EXPORT int pkv_latent_rows_per_block() { return LAT_WARPS; }

PKV_EXPORT int pkv_latent_prepare(const float* fused, int ld, int q_off, int q_rank, int kv_off, int rank, int rot,
                                  int rot_dims, const float* q_weight, const float* kv_weight, const float* freq, float eps,
                                  const int32_t* positions, const int32_t* slots, void* c_q, void* pool, int cache_dtype,
                                  long long pool_rows, int tokens, int* status, void* stream) {
  if (tokens <= 0) return 0;
  if (q_rank < 0 || (q_rank > 0 && !q_weight) || rank < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return PKV_ERR_SIZE;
  const size_t smem = (size_t)(rot + 32) * sizeof(float);
  if (smem > 48 * 1024) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
  if (cache_dtype == PKV_F32)
    latent_prepare_kernel<float><<<tokens, 256, smem, s>>>(fused, ld, q_off, q_rank, kv_off, rank, rot, rot_dims, q_weight,
        kv_weight, freq, eps, positions, slots, (float*)c_q, (float*)pool, pool_rows, status);
  else if (cache_dtype == PKV_BF16)
    latent_prepare_kernel<bf16><<<tokens, 256, smem, s>>>(fused, ld, q_off, q_rank, kv_off, rank, rot, rot_dims, q_weight,
        kv_weight, freq, eps, positions, slots, (bf16*)c_q, (bf16*)pool, pool_rows, status);
  else
    return PKV_ERR_DTYPE;
  return launch_status();
}

template <typename Q, typename A, typename C>
static int launch_latent(const void* q_lat, const void* q_rot, int q_rot_ld, int q_rot_head_stride, void* out,
                         const void* pool, const int32_t* block_table, int table_stride, const int32_t* seq_starts,
                         const int32_t* first_pos, const int32_t* work_seq, const int32_t* work_row0, int n_work,
                         const float* freq, const float* gate, int gate_ld, int tokens, int heads, int rank, int rot,
                         int rot_dims, int page_size, int window, float scale, int num_pages, int* status, cudaStream_t s) {
  const int dk = rank + rot;
  const size_t smem = ((size_t)LAT_WARPS * dk + (size_t)LAT_TILE * (dk + 1)) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<Q, A, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  latent_attention_kernel<Q, A, C><<<n_work, LAT_WARPS * 32, smem, s>>>(
      (const Q*)q_lat, (const A*)q_rot, q_rot_ld, q_rot_head_stride, (A*)out, (const C*)pool, block_table, table_stride,
      seq_starts, first_pos, work_seq, work_row0, freq, gate, gate_ld, tokens, heads, rank, rot, rot_dims, page_size,
      window, scale, num_pages, status);
  return launch_status();
}

PKV_EXPORT int pkv_latent_attention(const void* q_lat, int q_lat_dtype, const void* q_rot, int q_rot_ld,
                                    int q_rot_head_stride, void* out, int act_dtype, const void* pool, int cache_dtype,
                                    const int32_t* block_table, int table_stride, const int32_t* seq_starts,
                                    const int32_t* first_pos, const int32_t* work_seq, const int32_t* work_row0,
                                    int n_work, const float* freq, const float* gate, int gate_ld, int tokens, int heads,
                                    int rank, int rot, int rot_dims, int page_size, int window, float scale,
                                    int num_pages, int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (heads < 1 || rank < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || page_size < 1 ||
      window < 0 || num_pages < 1)
    return PKV_ERR_SIZE;
  if (rank > 32 * LAT_MAX_ACC) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_LAT(Q, A, C)                                                                                            \
  return launch_latent<Q, A, C>(q_lat, q_rot, q_rot_ld, q_rot_head_stride, out, pool, block_table, table_stride,    \
                                seq_starts, first_pos, work_seq, work_row0, n_work, freq, gate, gate_ld, tokens,    \
                                heads, rank, rot, rot_dims, page_size, window, scale, num_pages, status, s)
  if (act_dtype == PKV_F32 && cache_dtype == PKV_F32 && q_lat_dtype == PKV_F32) PKV_LAT(float, float, float);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16 && q_lat_dtype == PKV_F32) PKV_LAT(float, bf16, bf16);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16 && q_lat_dtype == PKV_BF16) PKV_LAT(bf16, bf16, bf16);
#undef PKV_LAT
  return PKV_ERR_DTYPE;
}

static size_t lm_smem_bytes(int rank, int rot, int warps) {
  return (size_t)(warps * 16 + 2 * LM_BN) * (rank + rot + LM_PAD) * sizeof(bf16);
}

// Whether the tensor-core kernel takes these sizes (else the general kernel above serves them).
PKV_EXPORT int pkv_latent_mma_supports(int rank, int rot) {
  if (rank < 16 || (rank & 15) || ((rank + rot) & 15)) return 0;
  return lm_smem_bytes(rank, rot, 4) <= LM_SMEM_LIMIT ? 1 : 0;
}

// Rows of a block for these sizes (the host's work list is cut to it).
PKV_EXPORT int pkv_latent_mma_rows_per_block(int rank, int rot) {
  return lm_smem_bytes(rank, rot, 8) <= LM_SMEM_LIMIT ? 128 : 64;
}

template <int VT, typename Q, int WARPS>
static int launch_latent_mma(const LatentParams& p, int n_work, cudaStream_t s) {
  const size_t smem = lm_smem_bytes(p.rank, p.rot, WARPS);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<VT, Q, WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_work, (p.rank + VT - 1) / VT, p.num_splits);
  latent_attention_mma_kernel<VT, Q, WARPS><<<grid, WARPS * 32, smem, s>>>(p);
  if (p.num_splits > 1)
    latent_merge_kernel<<<(unsigned)(p.heads * p.tokens), 128, 0, s>>>(p.part_o, p.part_ml, p.out, p.gate, p.gate_ld, p.tokens,
                                                                     p.heads, p.rank, p.num_splits);
  return launch_status();
}

PKV_EXPORT int pkv_latent_attention_mma(const void* q_lat, int q_lat_dtype, const void* q_rot, int q_rot_ld,
                                        int q_rot_head_stride, void* out, const void* pool, const int32_t* block_table,
                                        int table_stride, const int32_t* seq_starts, const int32_t* first_pos,
                                        const int32_t* work_seq, const int32_t* work_row0, int n_work, const float* freq,
                                        const float* gate, int gate_ld, int tokens, int heads, int rank, int rot,
                                        int rot_dims, int page_size, int window, float scale, int num_pages, int* status,
                                        int num_splits, float* part_o, float* part_ml, void* stream) {
  if (n_work <= 0) return 0;
  if (num_splits < 1 || num_splits > 64 || (num_splits > 1 && (!part_o || !part_ml))) return PKV_ERR_SIZE;
  if (heads < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || page_size < 1 || window < 0 || num_pages < 1)
    return PKV_ERR_SIZE;
  if (!pkv_latent_mma_supports(rank, rot)) return PKV_ERR_SIZE;
  LatentParams p;
  p.q_lat = q_lat; p.q_rot = (const bf16*)q_rot; p.q_rot_ld = q_rot_ld; p.q_rot_head_stride = q_rot_head_stride;
  p.out = (bf16*)out; p.pool = (const bf16*)pool; p.block_table = block_table; p.table_stride = table_stride;
  p.seq_starts = seq_starts; p.first_pos = first_pos; p.work_seq = work_seq; p.work_row0 = work_row0; p.freq = freq;
  p.gate = gate; p.gate_ld = gate_ld; p.tokens = tokens; p.heads = heads; p.rank = rank; p.rot = rot; p.rot_dims = rot_dims;
  p.page_size = page_size; p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.num_pages = num_pages;
  p.status = status;
  p.num_splits = num_splits; p.part_o = part_o; p.part_ml = part_ml;
  cudaStream_t s = (cudaStream_t)stream;
  const bool wide = pkv_latent_mma_rows_per_block(rank, rot) == 128;
#define PKV_LM(VT)                                                                                  \
  do {                                                                                              \
    if (q_lat_dtype == PKV_F32 && wide) return launch_latent_mma<VT, float, 8>(p, n_work, s);      \
    if (q_lat_dtype == PKV_F32) return launch_latent_mma<VT, float, 4>(p, n_work, s);              \
    if (q_lat_dtype == PKV_BF16 && wide) return launch_latent_mma<VT, bf16, 8>(p, n_work, s);      \
    if (q_lat_dtype == PKV_BF16) return launch_latent_mma<VT, bf16, 4>(p, n_work, s);              \
    return PKV_ERR_DTYPE;                                                                           \
  } while (0)
  if (rank <= 64) PKV_LM(64);
  if (rank <= 128) PKV_LM(128);
  PKV_LM(256);
#undef PKV_LM
}
