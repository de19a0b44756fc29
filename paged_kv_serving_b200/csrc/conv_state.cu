// A short causal convolution over time on every channel for a ragged batch of portions of
// sequences, in two forms that share the kernels:
//   out[t] = x[t] + sum_{j < taps} w[:, j] * x[t - taps + 1 + j]              (added to its own input)
//   out[t] = act(bias + sum_{j < taps} w[:, j] * x[t - taps + 1 + j])         (bias and activation)
// with zeros before position 0. The input rows may be a column range of a wider matrix (a row
// stride of their own).
// The last taps - 1 inputs of every sequence live in a per-request state [slots, taps - 1, width]
// (oldest first), so that a sequence can be fed in portions of any size: a token near the start
// of its portion reads what the portion before left there. Two kernels: the first computes every
// output of the step and only reads the state, the second (one thread per entry and channel)
// writes the state the step leaves. Arithmetic is float32; storage float32 or bfloat16.
#include "common.cuh"

namespace pkv {

constexpr int CONV_MAX_TAPS = 16;

__device__ __forceinline__ float conv_finish(float own, float acc, float bias, int residual, int act) {
  float v = acc + bias;
  if (act == 1) v = v / (1.0f + expf(-v));     // SiLU
  return residual ? own + v : v;
}

template <typename X>
__global__ void conv_residual_kernel(const X* __restrict__ x, int ld, const float* __restrict__ w, const float* __restrict__ bias,
                                     const X* __restrict__ state,
                                     const int32_t* __restrict__ token_seq, const int32_t* __restrict__ seq_starts,
                                     const int32_t* __restrict__ state_slots, X* __restrict__ out, int tokens, int width,
                                     int taps, int residual, int act) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * width) return;
  const int t = (int)(i / width), c = (int)(i - (long long)t * width);
  const int s = token_seq[t];
  const int local = t - seq_starts[s];
  const int slot = state_slots[s];
  const int tail = taps - 1;
  const float own = to_float(x[(size_t)t * ld + c]);
  float acc = own * w[(size_t)c * taps + tail];
  for (int j = 0; j < tail; ++j) {
    const int src = local - tail + j;              // place inside this portion; negative: before it
    float v;
    if (src >= 0) v = to_float(x[(size_t)(t - tail + j) * ld + c]);
    else v = to_float(state[((size_t)slot * tail + (tail + src)) * width + c]);
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  out[i] = from_float<X>(conv_finish(own, acc, bias ? bias[c] : 0.0f, residual, act));
}

// The same for bfloat16 rows whose width is a multiple of 8: a thread takes 8 channels of a token
// with 16-byte loads and stores; the weights arrive transposed, w_t [taps][width], so that the 8
// channels' weights of a tap are two 16-byte loads as well.
__global__ void conv_residual_bf16x8_kernel(const bf16* __restrict__ x, int ld, const float* __restrict__ w_t,
                                            const float* __restrict__ bias,
                                            const bf16* __restrict__ state, const int32_t* __restrict__ token_seq,
                                            const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ state_slots,
                                            bf16* __restrict__ out, int tokens, int width, int taps, int residual, int act) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int per_row = width >> 3;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * per_row) return;
  const int t = i / per_row, c = (i - t * per_row) << 3;
  const int s = token_seq[t];
  const int local = t - seq_starts[s];
  const int slot = state_slots[s];
  const int tail = taps - 1;
  float own[8], acc[8];
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)t * ld + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      own[2 * k] = f.x;
      own[2 * k + 1] = f.y;
    }
  }
  {
    const float4 lo = *reinterpret_cast<const float4*>(w_t + (size_t)tail * width + c);
    const float4 hi = *reinterpret_cast<const float4*>(w_t + (size_t)tail * width + c + 4);
    const float wk[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = own[k] * wk[k];
  }
  for (int j = 0; j < tail; ++j) {
    const int src = local - tail + j;
    const bf16* from = src >= 0 ? x + (size_t)(t - tail + j) * ld + c
                                : state + ((size_t)slot * tail + (tail + src)) * width + c;
    const uint4 raw = *reinterpret_cast<const uint4*>(from);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float4 lo = *reinterpret_cast<const float4*>(w_t + (size_t)j * width + c);
    const float4 hi = *reinterpret_cast<const float4*>(w_t + (size_t)j * width + c + 4);
    const float wk[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      acc[2 * k] = fmaf(wk[2 * k], f.x, acc[2 * k]);
      acc[2 * k + 1] = fmaf(wk[2 * k + 1], f.y, acc[2 * k + 1]);
    }
  }
  uint4 packed;
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = conv_finish(own[k], acc[k], bias ? bias[c + k] : 0.0f, residual, act);
#pragma unroll
  for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
  *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = packed;
}

template <typename X>
__global__ void conv_state_update_kernel(const X* __restrict__ x, int ld, X* __restrict__ state,
                                         const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ state_slots,
                                         int seqs, int width, int taps) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)seqs * width) return;
  const int s = (int)(i / width), c = (int)(i - (long long)s * width);
  const int start = seq_starts[s], n = seq_starts[s + 1] - start;
  const int tail = taps - 1;
  X* mine = state + (size_t)state_slots[s] * tail * width + c;
  // new[k] = the input at place n - tail + k of this portion, or (before the portion) old[n + k];
  // ascending k reads old places that have not been written yet
  for (int k = 0; k < tail; ++k) {
    const int src = n - tail + k;
    mine[(size_t)k * width] = src >= 0 ? x[(size_t)(start + src) * ld + c] : mine[(size_t)(n + k) * width];
  }
}

}  // namespace pkv

using namespace pkv;

// w: [width][taps]; w_t: the same weights as [taps][width], or null (the 16-byte form needs it).
// ld: row stride of x in elements (>= width); bias [width] or null; residual: add the input itself;
// act: 0 none, 1 SiLU.
PKV_EXPORT int pkv_conv_residual(const void* x, int dtype, int ld, const float* w, const float* w_t, const float* bias, void* state,
                                 const int32_t* token_seq, const int32_t* seq_starts, const int32_t* state_slots, void* out,
                                 int tokens, int seqs, int width, int taps, int residual, int act, void* stream) {
  if (tokens <= 0) return 0;
  if (width < 1 || taps < 1 || taps > CONV_MAX_TAPS || seqs < 1 || ld < width || act < 0 || act > 1) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const long long total = (long long)tokens * width;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  const unsigned state_blocks = (unsigned)(((long long)seqs * width + 255) / 256);
  // (the tail's update waits at its top for the kernel that reads the tail to finish)
  int rc = 0;
  if (dtype == PKV_F32) {
    rc = launch_kernel(conv_residual_kernel<float>, dim3(blocks), dim3(256), 0, s, true, 0, (const float*)x, ld, w, bias,
                       (const float*)state, token_seq, seq_starts, state_slots, (float*)out, tokens, width, taps, residual, act);
    if (rc == 0 && taps > 1)
      rc = launch_kernel(conv_state_update_kernel<float>, dim3(state_blocks), dim3(256), 0, s, true, 0, (const float*)x, ld,
                         (float*)state, seq_starts, state_slots, seqs, width, taps);
  } else if (dtype == PKV_BF16) {
    const bool wide = w_t != nullptr && ((uintptr_t)w_t & 15) == 0 && width % 8 == 0 && ld % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
                      ((uintptr_t)out & 15) == 0 && (taps == 1 || ((uintptr_t)state & 15) == 0) && total / 8 < (1ll << 31);
    if (wide)
      rc = launch_kernel(conv_residual_bf16x8_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, s, true, 0,
                         (const bf16*)x, ld, w_t, bias, (const bf16*)state, token_seq, seq_starts, state_slots, (bf16*)out, tokens,
                         width, taps, residual, act);
    else
      rc = launch_kernel(conv_residual_kernel<bf16>, dim3(blocks), dim3(256), 0, s, true, 0, (const bf16*)x, ld, w, bias,
                         (const bf16*)state, token_seq, seq_starts, state_slots, (bf16*)out, tokens, width, taps, residual, act);
    if (rc == 0 && taps > 1)
      rc = launch_kernel(conv_state_update_kernel<bf16>, dim3(state_blocks), dim3(256), 0, s, true, 0, (const bf16*)x, ld,
                         (bf16*)state, seq_starts, state_slots, seqs, width, taps);
  } else {
    return PKV_ERR_DTYPE;
  }
  return rc;
}
