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
  int unit_norm;          // divide query and key heads by their root mean square
  int page_size;
  long long pool_slots;   // pages * page_size
  int ld_other;           // row stride of the other layer's values
};

template <typename A, typename C>
__global__ void __launch_bounds__(SK_WARPS * 32)
qkv_prepare_kernel(A* __restrict__ qkv, const int32_t* __restrict__ positions, const float* __restrict__ freq,
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
  for (int unit = warp; unit < qk_heads + p.n_kv; unit += SK_WARPS) {
    if (unit < qk_heads) {
      // a query head (written back in place) or a key head (written to the pool)
      A* x = row + (size_t)unit * p.dim;
      for (int i = lane; i < half; i += 32) {
        const float u = to_float(x[i]), v = to_float(x[i + half]);
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= p.rot_factor;
        cs *= p.rot_factor;
        buf[i] = u * cs - v * sn;
        buf[i + half] = v * cs + u * sn;
      }
      for (int d = p.rot_dims + lane; d < p.dim; d += 32) buf[d] = to_float(x[d]);
      __syncwarp();
      float inv = 1.0f;
      if (p.unit_norm) {
        float sq = 0.0f;
        for (int d = lane; d < p.dim; d += 32) sq = fmaf(buf[d], buf[d], sq);
        sq = warp_sum(sq);
        inv = 1.0f / sqrtf(sq / (float)p.dim + p.eps);
      }
      if (unit < p.n_heads) {
        for (int d = lane; d < p.dim; d += 32) x[d] = from_float<A>(buf[d] * inv);
      } else if (slot >= 0) {
        const int kvh = unit - p.n_heads;
        C* dst = k_pool + (((size_t)page * p.n_kv + kvh) * p.page_size + offset) * p.dim;
        for (int d = lane; d < p.dim; d += 32) dst[d] = from_float<C>(buf[d] * inv);
      }
      __syncwarp();
    } else {
      const int kvh = unit - qk_heads;
      const A* v = row + (size_t)qk_heads * p.dim + (size_t)kvh * p.vdim;
      const A* other = v_other ? v_other + (size_t)t * p.ld_other + (size_t)kvh * p.vdim : nullptr;
      A* keep = v_keep ? v_keep + ((size_t)t * p.n_kv + kvh) * p.vdim : nullptr;
      C* dst = slot >= 0 ? v_pool + (((size_t)page * p.n_kv + kvh) * p.page_size + offset) * p.vdim : nullptr;
      const float lam = other ? lambda[0] : 0.0f;
      for (int d = lane; d < p.vdim; d += 32) {
        float val = to_float(v[d]);
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
    if (p.softcap > 0.0f) sc = p.softcap * tanhf(sc / p.softcap);
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

}  // namespace pkv

using namespace pkv;

template <typename A, typename C>
static int launch_prepare(void* qkv, const int32_t* positions, const float* freq, const void* v_other, const float* lambda,
                          void* v_keep, void* k_pool, void* v_pool, const int32_t* slots, const PrepareParams& p, int tokens,
                          int* status, cudaStream_t s) {
  const size_t smem = (size_t)SK_WARPS * p.dim * sizeof(float);
  return launch_kernel(qkv_prepare_kernel<A, C>, dim3(tokens), dim3(SK_WARPS * 32), smem, s, true, 0, (A*)qkv, positions, freq,
                       (const A*)v_other, lambda, (A*)v_keep, (C*)k_pool, (C*)v_pool, slots, p, status);
}

// qkv [tokens, ld]: H query heads of `dim`, G key heads of `dim`, G value heads of `vdim`.
// freq [rot_dims / 2] float32 (null with rot_dims 0). v_other: the values [tokens, ld_other] of
// another layer to blend with, weight lambda[0] (a float on the device), or null. v_keep: where
// to leave this layer's values [tokens, G * vdim] as they are cached, or null.
// k_pool [pages][G][page_size][dim], v_pool [pages][G][page_size][vdim]; slots: int32 per token,
// negative (or null): nothing is cached for it.
PKV_EXPORT int pkv_qkv_prepare(void* qkv, int act_dtype, int ld, const int32_t* positions, const float* freq, int rot_dims,
                               float rot_factor, float eps, int unit_norm, const void* v_other, int ld_other,
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
  return launch_prepare<A, C>(qkv, positions, freq, v_other, lambda, v_keep, k_pool, v_pool, slots, p, tokens, status, s)
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
                                  float scale, float softcap, int num_pages, int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || dim <= 0 || vdim <= 0 || page_size <= 0 || window < 0 || keep_first < 0 ||
      num_pages <= 0 || softcap < 0.0f)
    return PKV_ERR_SIZE;
  if (vdim > 32 * SK_MAX_ACC || dim > SK_MAX_DIM || n_kv > 65535) return PKV_ERR_LIMIT;
  SinkParams p{q_ld, table_stride, n_heads, n_kv, dim, vdim, page_size, window, keep_first, scale, softcap, num_pages};
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
