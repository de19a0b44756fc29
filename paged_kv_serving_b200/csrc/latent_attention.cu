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
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[q_off + i], row[q_off + i], ss);
  ss = block_sum(ss, scratch);
  const float q_inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    c_q[(size_t)t * q_rank + i] = from_float<C>(row[q_off + i] * q_inv * q_weight[i]);
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

}  // namespace pkv

using namespace pkv;

PKV_EXPORT int pkv_latent_rows_per_block() { return LAT_WARPS; }

PKV_EXPORT int pkv_latent_prepare(const float* fused, int ld, int q_off, int q_rank, int kv_off, int rank, int rot,
                                  int rot_dims, const float* q_weight, const float* kv_weight, const float* freq, float eps,
                                  const int32_t* positions, const int32_t* slots, void* c_q, void* pool, int cache_dtype,
                                  long long pool_rows, int tokens, int* status, void* stream) {
  if (tokens <= 0) return 0;
  if (q_rank < 1 || rank < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return PKV_ERR_SIZE;
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
