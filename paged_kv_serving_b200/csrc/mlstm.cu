// The matrix memory of xLSTM (mLSTM) for a ragged batch of portions of sequences, as a
// recurrence over the tokens of each portion that starts from, and leaves, a per-request state.
// Per head, with log gates i_t and f_t (float32, from capped pre-activations):
//   m_t = max(f_t + m_{t-1}, i_t)                       (m starts at 0)
//   a_t = exp(f_t + m_{t-1} - m_t),  b_t = exp(i_t - m_t)
//   S_t = a_t S_{t-1} + b_t k_t v_t^T,   n_t = a_t n_{t-1} + b_t k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// Everything here is float32: the projections arrive as float32, the state is float32. S is held
// column by column, [vdim][dim] per (request, head): the lanes that own a column read and write its
// `dim` entries as one contiguous run.
//
// Three kernels.
// `gates`: one warp per (entry, head). The recurrence of m is a chain of maps x -> max(x + f, i),
// which compose associatively ((f1, i1) then (f2, i2) is (f1 + f2, max(i1 + f2, i2))): the warp
// takes 32 tokens at a time, one per lane (the gates' transcendentals run side by side), scans the
// maps with shuffles, and leaves a_t, b_t and m_t per (token, head).
// `scan`: given a_t and b_t the columns of S are independent, and n is one more column whose
// value is always 1. A group of P lanes owns one column (each lane R of its `dim` entries), a
// block of 128 threads owns 128 / P columns, the grid is (column slices, heads, entries). Keys,
// queries, values and coefficients of a few tokens at a time arrive in shared memory by cp.async,
// the next chunk while this one is walked. The order of operations per token and column does not
// depend on how the sequence was cut into portions.
// `finish`: per (token, head) the numerators are divided by the denominator, then by their root
// mean square, multiplied by the norm's weight and by sigmoid of the output gate's pre-activation.
#include "common.cuh"

namespace pkv {

__device__ __forceinline__ float log_sigmoid(float z) {
  // log(1 / (1 + exp(-z))) without overflow on either side
  return fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
}

__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const float* __restrict__ proj, int ld, int i_off, int f_off, const float* __restrict__ i_bias,
                   const float* __restrict__ f_bias, float cap, float* __restrict__ m_state,
                   const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ state_slots,
                   float* __restrict__ coef, int heads) {
  const int head = blockIdx.x, s = blockIdx.y, lane = threadIdx.x;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  float* m_mine = m_state + (size_t)state_slots[s] * heads + head;
  float m_in = *m_mine;
  const float bi = i_bias[head], bf = f_bias[head];
  for (int base = 0; base < count; base += 32) {
    const int j = base + lane;
    const bool live = j < count;
    float log_i = -INFINITY, log_f = 0.0f;              // the identity map for lanes past the end
    if (live) {
      const float* row = proj + (size_t)(start + j) * ld;
      log_i = cap * tanhf((row[i_off + head] + bi) / cap);
      log_f = log_sigmoid(cap * tanhf((row[f_off + head] + bf) / cap));
    }
    // inclusive scan of the maps x -> max(x + F, M)
    float F = log_f, M = log_i;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float f_before = __shfl_up_sync(0xffffffffu, F, d), m_before = __shfl_up_sync(0xffffffffu, M, d);
      if (lane >= d) {
        M = fmaxf(m_before + F, M);
        F = f_before + F;
      }
    }
    const float m_t = fmaxf(m_in + F, M);
    float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
    if (lane == 0) m_prev = m_in;
    if (live) {
      float* c = coef + ((size_t)(start + j) * heads + head) * 4;
      c[0] = expf(log_f + m_prev - m_t);
      c[1] = expf(log_i - m_t);
      c[2] = m_t;
    }
    m_in = __shfl_sync(0xffffffffu, m_t, 31);
  }
  if (lane == 0) *m_mine = m_in;
}

__device__ __forceinline__ void ml_cp_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ml_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void ml_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ml_cp_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}

// A group of P lanes owns ML_C columns, each lane R entries of every one of them: P * R >= dim,
// P a power of two <= 32. Column `vdim` is the normaliser n (its value is 1 for every token; its
// state lives in n_state and its readout n . q goes to `dots`).
// EXACT: dim == P * R, so no entry of a lane lies beyond the column and the inner loops carry no guards.
template <int R, int ML_C, bool EXACT>
__global__ void __launch_bounds__(128)
mlstm_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, float q_scale,
                  const float* __restrict__ coef, float* __restrict__ s_state, float* __restrict__ n_state,
                  const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ state_slots,
                  float* __restrict__ out, float* __restrict__ dots, int heads, int dim, int vdim, int P, int chunk,
                  int vec4) {
  extern __shared__ __align__(16) float ml_smem[];
  const int head = blockIdx.y, s = blockIdx.z;
  const int per_block = (128 / P) * ML_C;
  const int c0 = blockIdx.x * per_block;
  const int local0 = (threadIdx.x / P) * ML_C;        // first of this group's columns, inside the block
  const int p = threadIdx.x % P;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  const int slot = state_slots[s];
  // one stage of shared memory: k [chunk][dim], q [chunk][dim], v [chunk][per_block], (a, b) [chunk][2]
  const int stage_floats = chunk * (2 * dim + per_block + 2);
  float* s_mine = s_state + ((size_t)slot * heads + head) * dim * vdim;
  float* n_mine = n_state + ((size_t)slot * heads + head) * dim;
  float sv[ML_C][R];
#pragma unroll
  for (int c = 0; c < ML_C; ++c) {
    const int column = c0 + local0 + c;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p + P * r;
      float v = 0.0f;
      if (d < dim && column < vdim) v = s_mine[(size_t)column * dim + d];
      else if (d < dim && column == vdim) v = n_mine[d];
      sv[c][r] = v;
    }
  }

  auto load = [&](int stage, int first) {
    float* ks = ml_smem + stage * stage_floats;
    float* qs = ks + chunk * dim;
    float* vs = qs + chunk * dim;
    float* cs = vs + chunk * per_block;
    const int n = min(chunk, count - first);
    if (vec4) {
      const int quarter = dim >> 2;
      for (int idx = threadIdx.x; idx < n * quarter; idx += 128) {
        const int t = idx / quarter, d = (idx - t * quarter) << 2;
        const float* row = proj + (size_t)(start + first + t) * ld;
        ml_cp_async16(ks + t * dim + d, row + k_off + head * dim + d);
        ml_cp_async16(qs + t * dim + d, row + q_off + head * dim + d);
      }
    } else {
      for (int idx = threadIdx.x; idx < n * dim; idx += 128) {
        const int t = idx / dim, d = idx - t * dim;
        const float* row = proj + (size_t)(start + first + t) * ld;
        ml_cp_async4(ks + idx, row + k_off + head * dim + d);
        ml_cp_async4(qs + idx, row + q_off + head * dim + d);
      }
    }
    for (int idx = threadIdx.x; idx < n * per_block; idx += 128) {
      const int t = idx / per_block, c = idx - t * per_block;
      if (c0 + c < vdim) ml_cp_async4(vs + idx, proj + (size_t)(start + first + t) * ld + v_off + head * vdim + c0 + c);
    }
    for (int idx = threadIdx.x; idx < n * 2; idx += 128)
      ml_cp_async4(cs + idx, coef + ((size_t)(start + first + (idx >> 1)) * heads + head) * 4 + (idx & 1));
  };

  if (count > 0) load(0, 0);
  ml_cp_async_commit();
  int stage = 0;
  for (int first = 0; first < count; first += chunk, stage ^= 1) {
    if (first + chunk < count) load(stage ^ 1, first + chunk);
    ml_cp_async_commit();
    ml_cp_async_wait<1>();
    __syncthreads();
    const float* ks = ml_smem + stage * stage_floats;
    const float* qs = ks + chunk * dim;
    const float* vs = qs + chunk * dim;
    const float* cs = vs + chunk * per_block;
    const int n = min(chunk, count - first);
    const float* kt = ks + p;
    const float* qt = qs + p;
    for (int t = 0; t < n; ++t, kt += dim, qt += dim) {
      const float a = cs[2 * t], b = cs[2 * t + 1];
      float kk[R], qq[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const bool in = EXACT || p + P * r < dim;
        kk[r] = in ? kt[P * r] : 0.0f;
        qq[r] = in ? qt[P * r] : 0.0f;
      }
      float num[ML_C];
#pragma unroll
      for (int c = 0; c < ML_C; ++c) {
        const int column = c0 + local0 + c;
        const float bv = column < vdim ? b * vs[t * per_block + local0 + c] : (column == vdim ? b : 0.0f);
        float acc = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          sv[c][r] = fmaf(bv, kk[r], a * sv[c][r]);
          acc = fmaf(sv[c][r], qq[r], acc);
        }
        num[c] = acc;
      }
      for (int o = P >> 1; o > 0; o >>= 1) {
#pragma unroll
        for (int c = 0; c < ML_C; ++c) num[c] += __shfl_xor_sync(0xffffffffu, num[c], o);
      }
      if (p == 0) {
        const size_t token = (size_t)(start + first + t);
#pragma unroll
        for (int c = 0; c < ML_C; ++c) {
          const int column = c0 + local0 + c;
          if (column < vdim) out[token * heads * vdim + head * vdim + column] = num[c] * q_scale;
          else if (column == vdim) dots[token * heads + head] = num[c] * q_scale;
        }
      }
    }
    __syncthreads();        // the stage is free for the load after next
  }
  ml_cp_async_wait<0>();
#pragma unroll
  for (int c = 0; c < ML_C; ++c) {
    const int column = c0 + local0 + c;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p + P * r;
      if (d < dim && column < vdim) s_mine[(size_t)column * dim + d] = sv[c][r];
      else if (d < dim && column == vdim) n_mine[d] = sv[c][r];
    }
  }
}

// One warp per (token, head): o / rms(o) * weight * sigmoid(gate)
template <typename O>
__global__ void mlstm_finish_kernel(const float* __restrict__ o, const float* __restrict__ dots,
                                    const float* __restrict__ coef, const float* __restrict__ weight,
                                    const float* __restrict__ proj, int ld, int g_off, O* __restrict__ out,
                                    long long rows, int heads, int vdim, float eps) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int head = (int)(row - t * heads);
  const float* mine = o + (size_t)row * vdim;
  const float denom = fmaxf(fabsf(dots[row]), expf(-coef[(size_t)row * 4 + 2])) + 1e-6f;
  float ss = 0.0f;
  for (int c = lane; c < vdim; c += 32) {
    const float v = mine[c] / denom;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    const float gate = proj[(size_t)t * ld + g_off + head * vdim + c];
    const float v = mine[c] / denom * inv * weight[head * vdim + c] * (1.0f / (1.0f + expf(-gate)));
    out[(size_t)row * vdim + c] = from_float<O>(v);
  }
}

}  // namespace pkv

using namespace pkv;

// proj: float32 [tokens, ld] with the columns of q, k ([heads][dim]), v, g ([heads][vdim]) and of
// the two gates ([heads]) at the given offsets. coef: float32 scratch [tokens, heads, 4].
// o: float32 scratch [tokens, heads * vdim + heads] (numerators, then n . q per (token, head)).
// out: [tokens, heads * vdim] in out_dtype.
PKV_EXPORT int pkv_mlstm(const float* proj, int ld, int q_off, int k_off, int v_off, int g_off, int i_off, int f_off,
                         const float* i_bias, const float* f_bias, const float* norm_weight, float cap, float q_scale,
                         float eps, float* s_state, float* n_state, float* m_state, const int32_t* seq_starts,
                         const int32_t* state_slots, float* coef, float* o, void* out, int out_dtype, int tokens,
                         int seqs, int heads, int dim, int vdim, void* stream) {
  if (tokens <= 0 || seqs <= 0) return 0;
  if (heads < 1 || dim < 1 || vdim < 1 || !(cap > 0.0f)) return PKV_ERR_SIZE;
  if (dim > 1024 || seqs > 65535 || heads > 65535) return PKV_ERR_LIMIT;
  if (out_dtype != PKV_F32 && out_dtype != PKV_BF16) return PKV_ERR_DTYPE;
  cudaStream_t s = (cudaStream_t)stream;
  mlstm_gates_kernel<<<dim3(heads, seqs), 32, 0, s>>>(proj, ld, i_off, f_off, i_bias, f_bias, cap, m_state, seq_starts,
                                                     state_slots, coef, heads);
  // lanes per column: enough that a lane holds at most R entries of it
  const int R = dim <= 256 ? 8 : 32;
  // columns per group of lanes (registers: ML_C * R state entries a lane). Two columns a group, which doubles
  // the blocks of a single long prompt, measured slower than four (keys and queries are staged twice as often).
  const int ML_C = dim <= 256 ? 4 : 1;
  int P = 1;
  while (P * R < dim) P <<= 1;
  const int per_block = (128 / P) * ML_C;
  // tokens per stage of shared memory: as many as fit in about 40 KB a stage, 16 at most
  int chunk = 16;
  while (chunk > 1 && (size_t)chunk * (2 * dim + per_block + 2) * sizeof(float) > 40 * 1024) chunk >>= 1;
  const size_t smem = 2 * (size_t)chunk * (2 * dim + per_block + 2) * sizeof(float);
  float* dots = o + (size_t)tokens * heads * vdim;
  const int vec4 = (dim % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && chunk % 2 == 0) ? 1 : 0;
  dim3 grid((vdim + 1 + per_block - 1) / per_block, heads, seqs);
  if (R == 8 && P * R == dim) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_scan_kernel<8, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mlstm_scan_kernel<8, 4, true><<<grid, 128, smem, s>>>(proj, ld, q_off, k_off, v_off, q_scale, coef, s_state, n_state, seq_starts,
                                                       state_slots, o, dots, heads, dim, vdim, P, chunk, vec4);
  } else if (R == 8) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_scan_kernel<8, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mlstm_scan_kernel<8, 4, false><<<grid, 128, smem, s>>>(proj, ld, q_off, k_off, v_off, q_scale, coef, s_state, n_state, seq_starts,
                                                 state_slots, o, dots, heads, dim, vdim, P, chunk, vec4);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mlstm_scan_kernel<32, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mlstm_scan_kernel<32, 1, false><<<grid, 128, smem, s>>>(proj, ld, q_off, k_off, v_off, q_scale, coef, s_state, n_state, seq_starts,
                                                  state_slots, o, dots, heads, dim, vdim, P, chunk, vec4);
  }
  const long long rows = (long long)tokens * heads;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  if (out_dtype == PKV_F32)
    mlstm_finish_kernel<float><<<blocks, 128, 0, s>>>(o, dots, coef, norm_weight, proj, ld, g_off, (float*)out, rows, heads,
                                                      vdim, eps);
  else
    mlstm_finish_kernel<bf16><<<blocks, 128, 0, s>>>(o, dots, coef, norm_weight, proj, ld, g_off, (bf16*)out, rows, heads,
                                                     vdim, eps);
  return launch_status();
}
