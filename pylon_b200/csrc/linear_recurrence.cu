// A gated linear recurrence over channels (the recurrent block of Griffin, with its real-gated linear recurrent unit).
//
// Per token, from one product of the layer's input, columns [y | x] of C channels each (biases b_y, b_x):
//
//     gate  = gelu_tanh(y + b_y)
//     u     = conv(x + b_x)                  causal, per channel, `taps` wide, the last tap on the current token, zeros before
//                                            the sequence starts; conv_w [C, taps], conv_b [C]
//     r, i  = sigmoid(R u_b + b_r), sigmoid(I u_b + b_i)     R, I: block-diagonal maps of `blocks` equal parts of the channels
//     log a = -factor * r * softplus(lam)    a = exp(log a)
//     S     = a * S + sqrt(1 - a^2) * i * u  from S = 0, the first token like every other
//     out   = S * gate
//
// What a request carries from token to token is one float32 slot [C + (taps - 1) * C]: S, then the convolution's last taps - 1
// inputs (x + b_x), oldest first.  Three kernels with the gates' product behind the first:
//
//   linear_recurrence_conv    a thread per (token, channel): u in float32 and in the compute dtype (the product's operand)
//   linear_recurrence_gates   a thread per (token, channel): everything of a token that does not need the state - a - 1, the term
//                             sqrt(1 - a^2) * i * u and the gelu branch - so that the walk is left with two multiply-adds a token
//   linear_recurrence_scan    a thread per (request row, channel) walks the row's tokens: S, out = S * gate; then it writes S and the
//                             last inputs back
// Long rows (a prompt) are walked in segments side by side instead: the recurrence is linear in S, so a segment walked from S = 0
// gives its own share L and, as the sum of its log a, the factor on what entered it: S_out = S_in + S_in expm1(sum log a) + L (again
// without rounding a product of decays close to one).  `segment_local` (a thread per row, segment and channel), `segment_carry` (a
// thread per row and channel: the segments' entering states in order, the slot's new state and kept inputs), `segment_walk` (every
// segment again from its entering state, writing out).
//
// Everything but the operands of the products is float32: the sigmoids, softplus, decay and its logarithm, the state.
// sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)), which keeps its digits when a is close to one, and a * S as S + S * expm1(log a):
// a channel that hardly decays has an a whose distance from one is a few units in its last place, and rounding a itself would change
// that distance, the same way at every token, by a share that shows after a thousand tokens.
#include "common.cuh"

namespace pylon {

constexpr int RECURRENCE_MAX_TAPS = 16;

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float x) { return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x))); }

// proj [T, ld] in T, the x branch at column x_offset; bias_x float32 [C]; state float32 [slots, state_floats].
// u32 float32 [T, C]; u16 [T, C] in T (may be null when T is float: u32 serves).
template <typename T>
__global__ void linear_recurrence_conv_kernel(const T* __restrict__ proj, long long ld, int x_offset, const float* __restrict__ bias_x,
                                              const float* __restrict__ conv_w, const float* __restrict__ conv_b, int taps,
                                              const float* __restrict__ state, long long state_floats, const int* __restrict__ token_row,
                                              const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ u32,
                                              T* __restrict__ u16, int channels, long long total) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const int t = (int)(item / channels), c = (int)(item % channels);
  const int row = token_row[t];
  if (row < 0) return;   // a padding token: it belongs to no request
  const int first = q_start[row];
  const int i = t - first;
  const float* history = state + (long long)slots[row] * state_floats + channels;   // [taps - 1, C], oldest first
  float acc = conv_b[c];
  for (int j = 0; j < taps; ++j) {
    const int n = i - (taps - 1) + j;   // which of the row's tokens this tap weighs; negative: before this step
    const float x = n >= 0 ? to_float<T>(proj[(long long)(first + n) * ld + x_offset + c]) + bias_x[c] : history[(long long)(taps - 1 + n) * channels + c];
    acc = fmaf(conv_w[(long long)c * taps + j], x, acc);
  }
  u32[item] = acc;
  if (u16 != nullptr) u16[item] = from_float<T>(acc);
}

// gates float32 [T, blocks, 2 * part]: per block the r logits, then the i logits.  decay_less_one, branch float32 [T, C] out; term: u in,
// sqrt(1 - a^2) * i * u out, float32 [T, C] in place.
template <typename T>
__global__ void linear_recurrence_gates_kernel(const T* __restrict__ proj, long long ld, int y_offset, const float* __restrict__ bias_y,
                                               const float* __restrict__ gates, const float* __restrict__ bias_r, const float* __restrict__ bias_i,
                                               const float* __restrict__ lam, float factor, const int* __restrict__ token_row,
                                               float* __restrict__ term, float* __restrict__ decay_less_one, float* __restrict__ branch, int channels,
                                               int part, long long total) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const long long t = item / channels;
  const int c = (int)(item % channels);
  if (token_row[t] < 0) return;   // a padding token: it belongs to no request
  const long long gate_column = t * 2 * channels + (long long)(c / part) * 2 * part + c % part;
  const float r = sigmoid_f(gates[gate_column] + bias_r[c]);
  const float i = sigmoid_f(gates[gate_column + part] + bias_i[c]);
  const float log_a = -factor * softplus_f(lam[c]) * r;
  decay_less_one[item] = expm1f(log_a);
  term[item] = sqrtf(-expm1f(2.f * log_a)) * i * term[item];
  branch[item] = gelu_tanh_f(to_float<T>(proj[t * ld + y_offset + c]) + bias_y[c]);
}

// out [T, C] in T.
template <typename T>
__global__ void linear_recurrence_scan_kernel(const T* __restrict__ proj, long long ld, int x_offset, const float* __restrict__ bias_x,
                                              const float* __restrict__ term, const float* __restrict__ decay_less_one,
                                              const float* __restrict__ branch, int taps, float* __restrict__ state, long long state_floats,
                                              const int* __restrict__ q_start, const int* __restrict__ slots, T* __restrict__ out, int channels) {
  grid_dependency_wait();
  allow_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  if (c >= channels) return;
  const int first = q_start[row], count = q_start[row + 1] - first;
  if (count <= 0) return;   // a row without tokens (a padded step): its state stays as it is
  float* mine = state + (long long)slots[row] * state_floats;
  float s = mine[c];
#pragma unroll 8
  for (int n = 0; n < count; ++n) {
    const long long at = (long long)(first + n) * channels + c;
    s += fmaf(s, decay_less_one[at], term[at]);
    out[at] = from_float<T>(s * branch[at]);
  }
  mine[c] = s;
  // the last taps - 1 inputs, oldest first: from this step's tokens, and from the old ones where the step is shorter
  float keep[RECURRENCE_MAX_TAPS];
  float* history = mine + channels;
  const float bx = bias_x[c];
  for (int k = 0; k < taps - 1; ++k) {
    const int n = count - (taps - 1) + k;
    keep[k] = n >= 0 ? to_float<T>(proj[(long long)(first + n) * ld + x_offset + c]) + bx : history[(long long)(taps - 1 + n) * channels + c];
  }
  for (int k = 0; k < taps - 1; ++k) history[(long long)k * channels + c] = keep[k];
}

// local, log_sum float32 [rows, segments, C] out.
__global__ void linear_recurrence_segment_local_kernel(const float* __restrict__ term, const float* __restrict__ decay_less_one,
                                                       const int* __restrict__ q_start, float* __restrict__ local, float* __restrict__ log_sum,
                                                       int channels, int segments) {
  grid_dependency_wait();
  allow_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int segment = blockIdx.y, row = blockIdx.z;
  if (c >= channels) return;
  const int first = q_start[row], count = q_start[row + 1] - first;
  if (count <= 0) return;
  const int each = (count + segments - 1) / segments;
  const int begin = segment * each, end = begin + each < count ? begin + each : count;
  float s = 0.f, logs = 0.f;
#pragma unroll 8
  for (int n = begin; n < end; ++n) {
    const long long at = (long long)(first + n) * channels + c;
    const float less = decay_less_one[at];
    s += fmaf(s, less, term[at]);
    logs += log1pf(less);
  }
  const long long where = ((long long)row * segments + segment) * channels + c;
  local[where] = s;
  log_sum[where] = logs;
}

// carry float32 [rows, segments, C] out: the state that enters each segment.
template <typename T>
__global__ void linear_recurrence_segment_carry_kernel(const T* __restrict__ proj, long long ld, int x_offset, const float* __restrict__ bias_x,
                                                       const float* __restrict__ local, const float* __restrict__ log_sum, float* __restrict__ carry,
                                                       int taps, float* __restrict__ state, long long state_floats, const int* __restrict__ q_start,
                                                       const int* __restrict__ slots, int channels, int segments) {
  grid_dependency_wait();
  allow_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  if (c >= channels) return;
  const int first = q_start[row], count = q_start[row + 1] - first;
  if (count <= 0) return;
  float* mine = state + (long long)slots[row] * state_floats;
  float s = mine[c];
  for (int segment = 0; segment < segments; ++segment) {
    const long long where = ((long long)row * segments + segment) * channels + c;
    carry[where] = s;
    s += fmaf(s, expm1f(log_sum[where]), local[where]);
  }
  mine[c] = s;
  float keep[RECURRENCE_MAX_TAPS];
  float* history = mine + channels;
  const float bx = bias_x[c];
  for (int k = 0; k < taps - 1; ++k) {
    const int n = count - (taps - 1) + k;
    keep[k] = n >= 0 ? to_float<T>(proj[(long long)(first + n) * ld + x_offset + c]) + bx : history[(long long)(taps - 1 + n) * channels + c];
  }
  for (int k = 0; k < taps - 1; ++k) history[(long long)k * channels + c] = keep[k];
}

template <typename T>
__global__ void linear_recurrence_segment_walk_kernel(const float* __restrict__ term, const float* __restrict__ decay_less_one,
                                                      const float* __restrict__ branch, const float* __restrict__ carry,
                                                      const int* __restrict__ q_start, T* __restrict__ out, int channels, int segments) {
  grid_dependency_wait();
  allow_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int segment = blockIdx.y, row = blockIdx.z;
  if (c >= channels) return;
  const int first = q_start[row], count = q_start[row + 1] - first;
  if (count <= 0) return;
  const int each = (count + segments - 1) / segments;
  const int begin = segment * each, end = begin + each < count ? begin + each : count;
  float s = carry[((long long)row * segments + segment) * channels + c];
#pragma unroll 8
  for (int n = begin; n < end; ++n) {
    const long long at = (long long)(first + n) * channels + c;
    s += fmaf(s, decay_less_one[at], term[at]);
    out[at] = from_float<T>(s * branch[at]);
  }
}

}  // namespace pylon

using namespace pylon;

// u16 null with dtype float32 (u32 is the operand then).
extern "C" int pylon_linear_recurrence_conv(const void* proj, long long ld, int x_offset, const float* bias_x, const float* conv_w, const float* conv_b,
                                            int taps, const float* state, long long state_floats, const int* token_row, const int* q_start,
                                            const int* slots, float* u32, void* u16, int channels, int num_tokens, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (channels < 1 || taps < 1 || taps > RECURRENCE_MAX_TAPS || state_floats < (long long)channels * taps)
    PYLON_REFUSE("linear_recurrence_conv: %d channels, %d taps (at most %d), a slot of %lld floats", channels, taps, RECURRENCE_MAX_TAPS, state_floats);
  const long long total = (long long)num_tokens * channels;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == PYLON_DTYPE_F32)
    launch_dependent(linear_recurrence_conv_kernel<float>, grid, dim3(256), 0, stream, (const float*)proj, ld, x_offset, bias_x, conv_w, conv_b, taps, state,
                     state_floats, token_row, q_start, slots, u32, (float*)nullptr, channels, total);
  else if (dtype == PYLON_DTYPE_BF16)
    launch_dependent(linear_recurrence_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)proj, ld, x_offset, bias_x, conv_w, conv_b,
                     taps, state, state_floats, token_row, q_start, slots, u32, (__nv_bfloat16*)u16, channels, total);
  else PYLON_REFUSE("linear_recurrence_conv: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("linear_recurrence_conv");
}

// term: float32 [T, C], u on entry and the recurrence's input term on return; decay_less_one, branch: float32 [T, C] scratch.
// segments > 1: every row is walked in so many segments side by side, with segment_scratch float32 [3, num_rows, segments, C].
extern "C" int pylon_linear_recurrence_scan(const void* proj, long long ld, int y_offset, int x_offset, const float* bias_y, const float* bias_x,
                                            float* term, const float* gates, const float* bias_r, const float* bias_i, const float* lam, float factor,
                                            int taps, float* state, long long state_floats, const int* token_row, const int* q_start, const int* slots,
                                            float* decay_less_one, float* branch, void* out, int channels, int blocks, int num_rows, int num_tokens,
                                            int segments, float* segment_scratch, int dtype, cudaStream_t stream) {
  if (num_rows <= 0 || num_tokens <= 0) return 0;
  if (channels < 1 || blocks < 1 || channels % blocks || taps < 1 || taps > RECURRENCE_MAX_TAPS || state_floats < (long long)channels * taps || num_rows > 65535)
    PYLON_REFUSE("linear_recurrence_scan: %d channels in %d blocks, %d taps, %d rows", channels, blocks, taps, num_rows);
  if (segments < 1 || segments > 1024 || (segments > 1 && !segment_scratch)) PYLON_REFUSE("linear_recurrence_scan: %d segments", segments);
  const int threads = 128;
  const dim3 grid((unsigned)((channels + threads - 1) / threads), (unsigned)num_rows);
  const dim3 by_segment((unsigned)((channels + threads - 1) / threads), (unsigned)segments, (unsigned)num_rows);
  const long long one = (long long)num_rows * segments * channels;
  float* local = segment_scratch;
  float* log_sum = segment_scratch ? segment_scratch + one : nullptr;
  float* carry = segment_scratch ? segment_scratch + 2 * one : nullptr;
  const int part = channels / blocks;
  const long long total = (long long)num_tokens * channels;
  const dim3 flat((unsigned)((total + 255) / 256));
  if (dtype == PYLON_DTYPE_F32) {
    launch_dependent(linear_recurrence_gates_kernel<float>, flat, dim3(256), 0, stream, (const float*)proj, ld, y_offset, bias_y, gates, bias_r, bias_i, lam,
                     factor, token_row, term, decay_less_one, branch, channels, part, total);
    if (segments > 1) {
      launch_dependent(linear_recurrence_segment_local_kernel, by_segment, dim3(threads), 0, stream, (const float*)term, (const float*)decay_less_one, q_start,
                       local, log_sum, channels, segments);
      launch_dependent(linear_recurrence_segment_carry_kernel<float>, grid, dim3(threads), 0, stream, (const float*)proj, ld, x_offset, bias_x,
                       (const float*)local, (const float*)log_sum, carry, taps, state, state_floats, q_start, slots, channels, segments);
      launch_dependent(linear_recurrence_segment_walk_kernel<float>, by_segment, dim3(threads), 0, stream, (const float*)term, (const float*)decay_less_one,
                       (const float*)branch, (const float*)carry, q_start, (float*)out, channels, segments);
    } else
    launch_dependent(linear_recurrence_scan_kernel<float>, grid, dim3(threads), 0, stream, (const float*)proj, ld, x_offset, bias_x, (const float*)term,
                     (const float*)decay_less_one, (const float*)branch, taps, state, state_floats, q_start, slots, (float*)out, channels);
  } else if (dtype == PYLON_DTYPE_BF16) {
    launch_dependent(linear_recurrence_gates_kernel<__nv_bfloat16>, flat, dim3(256), 0, stream, (const __nv_bfloat16*)proj, ld, y_offset, bias_y, gates, bias_r,
                     bias_i, lam, factor, token_row, term, decay_less_one, branch, channels, part, total);
    if (segments > 1) {
      launch_dependent(linear_recurrence_segment_local_kernel, by_segment, dim3(threads), 0, stream, (const float*)term, (const float*)decay_less_one, q_start,
                       local, log_sum, channels, segments);
      launch_dependent(linear_recurrence_segment_carry_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)proj, ld, x_offset, bias_x,
                       (const float*)local, (const float*)log_sum, carry, taps, state, state_floats, q_start, slots, channels, segments);
      launch_dependent(linear_recurrence_segment_walk_kernel<__nv_bfloat16>, by_segment, dim3(threads), 0, stream, (const float*)term,
                       (const float*)decay_less_one, (const float*)branch, (const float*)carry, q_start, (__nv_bfloat16*)out, channels, segments);
    } else
    launch_dependent(linear_recurrence_scan_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)proj, ld, x_offset, bias_x,
                     (const float*)term, (const float*)decay_less_one, (const float*)branch, taps, state, state_floats, q_start, slots, (__nv_bfloat16*)out,
                     channels);
  } else PYLON_REFUSE("linear_recurrence_scan: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("linear_recurrence_scan");
}
