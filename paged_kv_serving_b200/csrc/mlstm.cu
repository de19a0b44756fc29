// The matrix memory of xLSTM (mLSTM) for a ragged batch of portions of sequences, as a
// recurrence over the tokens of each portion that starts from, and leaves, a per-request state.
// Per head, with log gates i_t and f_t (float32, from capped pre-activations):
//   m_t = max(f_t + m_{t-1}, i_t)                       (m starts at 0)
//   a_t = exp(f_t + m_{t-1} - m_t),  b_t = exp(i_t - m_t)
//   S_t = a_t S_{t-1} + b_t k_t v_t^T,   n_t = a_t n_{t-1} + b_t k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// Everything here is float32: the projections arrive as float32, the state is float32.
//
// Three kernels. `gates`: one warp per (entry, head) walks the tokens, keeps n in registers
// (dimension d on lane d % 32) and m, and leaves a_t, b_t and the denominator per (token, head).
// `scan`: the columns of S are independent given those three numbers; a group of P lanes owns
// one column (each lane R of its `dim` entries), so a block of 128 threads owns 128 / P columns
// and the grid is (column slices, heads, entries). The order of operations per token does not
// depend on how the sequence was cut into portions, so a portion boundary changes nothing.
// `finish`: per (token, head) the output is divided by its root mean square, multiplied by the
// norm's weight and by sigmoid of the output gate's pre-activation.
#include "common.cuh"

namespace pkv {

constexpr int MLSTM_MAX_N = 32;     // dim <= 32 * MLSTM_MAX_N for the gates kernel

__device__ __forceinline__ float log_sigmoid(float z) {
  // log(1 / (1 + exp(-z))) without overflow on either side
  return fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
}

__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int i_off, int f_off,
                   const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                   float* __restrict__ n_state, float* __restrict__ m_state, const int32_t* __restrict__ seq_starts,
                   const int32_t* __restrict__ state_slots, float* __restrict__ coef, int heads, int dim) {
  const int head = blockIdx.x, s = blockIdx.y, lane = threadIdx.x;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  const int slot = state_slots[s];
  float* n_mine = n_state + ((size_t)slot * heads + head) * dim;
  float* m_mine = m_state + (size_t)slot * heads + head;
  float n[MLSTM_MAX_N];
#pragma unroll
  for (int r = 0; r < MLSTM_MAX_N; ++r) {
    const int d = lane + 32 * r;
    n[r] = d < dim ? n_mine[d] : 0.0f;
  }
  float m = *m_mine;
  const float bi = i_bias[head], bf = f_bias[head];
  for (int j = 0; j < count; ++j) {
    const float* row = proj + (size_t)(start + j) * ld;
    const float log_i = cap * tanhf((row[i_off + head] + bi) / cap);
    const float log_f = log_sigmoid(cap * tanhf((row[f_off + head] + bf) / cap));
    const float m_new = fmaxf(log_f + m, log_i);
    const float a = expf(log_f + m - m_new), b = expf(log_i - m_new);
    float dot = 0.0f;
#pragma unroll
    for (int r = 0; r < MLSTM_MAX_N; ++r) {
      const int d = lane + 32 * r;
      if (d < dim) {
        n[r] = a * n[r] + b * row[k_off + head * dim + d];
        dot = fmaf(n[r], row[q_off + head * dim + d] * q_scale, dot);
      }
    }
    dot = warp_sum(dot);
    m = m_new;
    if (lane == 0) {
      float* c = coef + ((size_t)(start + j) * heads + head) * 4;
      c[0] = a;
      c[1] = b;
      c[2] = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
    }
  }
#pragma unroll
  for (int r = 0; r < MLSTM_MAX_N; ++r) {
    const int d = lane + 32 * r;
    if (d < dim) n_mine[d] = n[r];
  }
  if (lane == 0) *m_mine = m;
}

// P lanes per column, R entries of the column per lane: P * R >= dim, P a power of two <= 32.
template <int R>
__global__ void __launch_bounds__(128)
mlstm_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, float q_scale,
                  const float* __restrict__ coef, float* __restrict__ s_state, const int32_t* __restrict__ seq_starts,
                  const int32_t* __restrict__ state_slots, float* __restrict__ out, int heads, int dim, int vdim, int P) {
  const int head = blockIdx.y, s = blockIdx.z;
  const int per_block = 128 / P;
  const int column = blockIdx.x * per_block + threadIdx.x / P;
  const int p = threadIdx.x % P;
  const bool live = column < vdim;
  const int start = seq_starts[s], count = seq_starts[s + 1] - start;
  const int slot = state_slots[s];
  // S is [dim][vdim] per (slot, head)
  float* s_mine = s_state + ((size_t)slot * heads + head) * dim * vdim + (live ? column : 0);
  float sv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = p + P * r;
    sv[r] = (live && d < dim) ? s_mine[(size_t)d * vdim] : 0.0f;
  }
  for (int j = 0; j < count; ++j) {
    const float* row = proj + (size_t)(start + j) * ld;
    const float* c = coef + ((size_t)(start + j) * heads + head) * 4;
    const float a = c[0], b = c[1], denom = c[2];
    const float bv = live ? b * row[v_off + head * vdim + column] : 0.0f;
    float num = 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = p + P * r;
      if (d < dim) {
        sv[r] = fmaf(bv, row[k_off + head * dim + d], a * sv[r]);
        num = fmaf(sv[r], row[q_off + head * dim + d] * q_scale, num);
      }
    }
    for (int o = P >> 1; o > 0; o >>= 1) num += __shfl_xor_sync(0xffffffffu, num, o);
    if (live && p == 0) out[(size_t)(start + j) * heads * vdim + head * vdim + column] = num / denom;
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = p + P * r;
    if (live && d < dim) s_mine[(size_t)d * vdim] = sv[r];
  }
}

// One warp per (token, head): o / rms(o) * weight * sigmoid(gate)
template <typename O>
__global__ void mlstm_finish_kernel(const float* __restrict__ o, const float* __restrict__ weight,
                                    const float* __restrict__ proj, int ld, int g_off, O* __restrict__ out,
                                    long long rows, int heads, int vdim, float eps) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int head = (int)(row - t * heads);
  const float* mine = o + (size_t)row * vdim;
  float ss = 0.0f;
  for (int c = lane; c < vdim; c += 32) ss = fmaf(mine[c], mine[c], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    const float gate = proj[(size_t)t * ld + g_off + head * vdim + c];
    const float v = mine[c] * inv * weight[head * vdim + c] * (1.0f / (1.0f + expf(-gate)));
    out[(size_t)row * vdim + c] = from_float<O>(v);
  }
}

}  // namespace pkv

using namespace pkv;

// proj: float32 [tokens, ld] with the columns of q, k ([heads][dim]), v, g ([heads][vdim]) and of
// the two gates ([heads]) at the given offsets. coef: float32 scratch [tokens, heads, 4].
// o: float32 scratch [tokens, heads * vdim]. out: [tokens, heads * vdim] in out_dtype.
PKV_EXPORT int pkv_mlstm(const float* proj, int ld, int q_off, int k_off, int v_off, int g_off, int i_off, int f_off,
                         const float* i_bias, const float* f_bias, const float* norm_weight, float cap, float q_scale,
                         float eps, float* s_state, float* n_state, float* m_state, const int32_t* seq_starts,
                         const int32_t* state_slots, float* coef, float* o, void* out, int out_dtype, int tokens,
                         int seqs, int heads, int dim, int vdim, void* stream) {
  if (tokens <= 0 || seqs <= 0) return 0;
  if (heads < 1 || dim < 1 || vdim < 1 || !(cap > 0.0f)) return PKV_ERR_SIZE;
  if (dim > 32 * MLSTM_MAX_N || seqs > 65535 || heads > 65535) return PKV_ERR_LIMIT;
  if (out_dtype != PKV_F32 && out_dtype != PKV_BF16) return PKV_ERR_DTYPE;
  cudaStream_t s = (cudaStream_t)stream;
  mlstm_gates_kernel<<<dim3(heads, seqs), 32, 0, s>>>(proj, ld, q_off, k_off, i_off, f_off, i_bias, f_bias, cap, q_scale,
                                                     n_state, m_state, seq_starts, state_slots, coef, heads, dim);
  // lanes per column: enough that a lane holds at most R entries of it
  int R = dim <= 256 ? 8 : 32;
  int P = 1;
  while (P * R < dim) P <<= 1;
  const int per_block = 128 / P;
  dim3 grid((vdim + per_block - 1) / per_block, heads, seqs);
  if (R == 8)
    mlstm_scan_kernel<8><<<grid, 128, 0, s>>>(proj, ld, q_off, k_off, v_off, q_scale, coef, s_state, seq_starts, state_slots,
                                              o, heads, dim, vdim, P);
  else
    mlstm_scan_kernel<32><<<grid, 128, 0, s>>>(proj, ld, q_off, k_off, v_off, q_scale, coef, s_state, seq_starts,
                                               state_slots, o, heads, dim, vdim, P);
  const long long rows = (long long)tokens * heads;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  if (out_dtype == PKV_F32)
    mlstm_finish_kernel<float><<<blocks, 128, 0, s>>>(o, norm_weight, proj, ld, g_off, (float*)out, rows, heads, vdim, eps);
  else
    mlstm_finish_kernel<bf16><<<blocks, 128, 0, s>>>(o, norm_weight, proj, ld, g_off, (bf16*)out, rows, heads, vdim, eps);
  return launch_status();
}
