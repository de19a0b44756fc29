// The selective scan of a Mamba mixer over a ragged batch of portions of sequences.
// Per channel c and state coordinate n, token by token:
//   dt   = softplus(dt_pre[t, c] + dt_bias[c])
//   S[c, n] <- exp(dt * A[c, n]) * S[c, n] + dt * x[t, c] * B[t, n]
//   y[t, c] = sum_n S[c, n] * C[t, n] + D[c] * x[t, c];      out[t, c] = y[t, c] * silu(z[t, c])
// S lives in a per-request state [slots, inner, state] (float32), read when a portion begins and
// written back when it ends, so a sequence may arrive in portions of any size and the result is
// the same operations in the same order however it was cut. Everything that enters the
// recurrence is float32: the step sizes, the decays, B and C (they arrive as the float32 result
// of their projection), the state. x and z are activations in the compute type.
//
// A team of L lanes (a power of two, at most a warp) owns one channel; each lane keeps up to
// SCAN_REGS state coordinates n = lane_in_team + r * L in registers. A block of SCAN_THREADS
// threads takes SCAN_THREADS / L channels of one sequence and walks the portion in chunks of
// SCAN_CHUNK tokens staged in shared memory (coalesced loads of dt, x, z, B and C).
#include "common.cuh"

namespace pkv {

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_REGS = 8;
constexpr int SCAN_CHUNK = 16;

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

struct ScanParams {
  int inner, state;
  int ld_x, ld_z, ld_dt, ld_bc;   // row strides (elements)
  int b_at, c_at;                 // columns of B and C in the float32 projection
  int lanes;                      // L
};

template <typename X>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const X* __restrict__ x, const X* __restrict__ z, const float* __restrict__ dt_pre,
                      const float* __restrict__ dt_bias, const float* __restrict__ bc, const float* __restrict__ a,
                      const float* __restrict__ d_skip, float* __restrict__ state, const int32_t* __restrict__ seq_starts,
                      const int32_t* __restrict__ state_slots, X* __restrict__ out, ScanParams p) {
  extern __shared__ float scan_smem[];
  const int L = p.lanes;
  const int channels = SCAN_THREADS / L;          // channels of this block
  float* dt_s = scan_smem;                        // [SCAN_CHUNK][channels]   step sizes (after softplus)
  float* x_s = dt_s + SCAN_CHUNK * channels;      // [SCAN_CHUNK][channels]
  float* z_s = x_s + SCAN_CHUNK * channels;       // [SCAN_CHUNK][channels]
  float* b_s = z_s + SCAN_CHUNK * channels;       // [SCAN_CHUNK][state]
  float* c_s = b_s + SCAN_CHUNK * p.state;        // [SCAN_CHUNK][state]

  const int s = blockIdx.y;
  const int start = seq_starts[s], n_tokens = seq_starts[s + 1] - start;
  const int slot = state_slots[s];
  const int c0 = blockIdx.x * channels;
  const int team = threadIdx.x / L, lane = threadIdx.x - team * L;
  const int c = c0 + team;
  const bool live = c < p.inner;

  float S[SCAN_REGS], A[SCAN_REGS];
  float* mine = state + ((size_t)slot * p.inner + (live ? c : 0)) * p.state;
#pragma unroll
  for (int r = 0; r < SCAN_REGS; ++r) {
    const int n = lane + r * L;
    const bool has = live && n < p.state;
    S[r] = has ? mine[n] : 0.0f;
    A[r] = has ? a[(size_t)c * p.state + n] : 0.0f;
  }
  const float skip = live ? d_skip[c] : 0.0f;

  for (int t0 = 0; t0 < n_tokens; t0 += SCAN_CHUNK) {
    const int count = min(SCAN_CHUNK, n_tokens - t0);
    __syncthreads();                               // the chunk before is consumed
    for (int i = threadIdx.x; i < count * channels; i += SCAN_THREADS) {
      const int j = i / channels, k = i - j * channels;
      const int ch = c0 + k;
      const size_t t = (size_t)(start + t0 + j);
      float dtv = 0.0f, xv = 0.0f, zv = 0.0f;
      if (ch < p.inner) {
        dtv = softplus_f(dt_pre[t * p.ld_dt + ch] + dt_bias[ch]);
        xv = to_float(x[t * p.ld_x + ch]);
        zv = to_float(z[t * p.ld_z + ch]);
      }
      dt_s[j * channels + k] = dtv;
      x_s[j * channels + k] = xv;
      z_s[j * channels + k] = zv;
    }
    for (int i = threadIdx.x; i < count * p.state; i += SCAN_THREADS) {
      const int j = i / p.state, n = i - j * p.state;
      const size_t t = (size_t)(start + t0 + j);
      b_s[j * p.state + n] = bc[t * p.ld_bc + p.b_at + n];
      c_s[j * p.state + n] = bc[t * p.ld_bc + p.c_at + n];
    }
    __syncthreads();
    for (int j = 0; j < count; ++j) {
      const float dtv = dt_s[j * channels + team], xv = x_s[j * channels + team];
      const float dx = dtv * xv;
      const float* bj = b_s + j * p.state;
      const float* cj = c_s + j * p.state;
      float y = 0.0f;
#pragma unroll
      for (int r = 0; r < SCAN_REGS; ++r) {
        const int n = lane + r * L;
        if (n < p.state) {
          S[r] = fmaf(expf(dtv * A[r]), S[r], dx * bj[n]);
          y = fmaf(S[r], cj[n], y);
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (lane == 0 && live) {
        const float zv = z_s[j * channels + team];
        y = fmaf(skip, xv, y);
        out[(size_t)(start + t0 + j) * p.inner + c] = from_float<X>(y * (zv / (1.0f + expf(-zv))));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < SCAN_REGS; ++r) {
      const int n = lane + r * L;
      if (n < p.state) mine[n] = S[r];
    }
  }
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
  if (n_state > 32 * SCAN_REGS || seqs > 65535) return PKV_ERR_LIMIT;
  int lanes = 1;
  while (lanes * SCAN_REGS < n_state) lanes <<= 1;
  const int channels = SCAN_THREADS / lanes;
  ScanParams p{inner, n_state, ld_x, ld_z, ld_dt, ld_bc, b_at, c_at, lanes};
  const size_t smem = (size_t)SCAN_CHUNK * (3 * channels + 2 * n_state) * sizeof(float);
  dim3 grid((inner + channels - 1) / channels, seqs);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PKV_F32)
    selective_scan_kernel<float><<<grid, SCAN_THREADS, smem, s>>>((const float*)x, (const float*)z, dt_pre, dt_bias, bc, a,
                                                                  d_skip, state, seq_starts, state_slots, (float*)out, p);
  else if (dtype == PKV_BF16)
    selective_scan_kernel<bf16><<<grid, SCAN_THREADS, smem, s>>>((const bf16*)x, (const bf16*)z, dt_pre, dt_bias, bc, a, d_skip,
                                                                 state, seq_starts, state_slots, (bf16*)out, p);
  else
    return PKV_ERR_DTYPE;
  return launch_status();
}
