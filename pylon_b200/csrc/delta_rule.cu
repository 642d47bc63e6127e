// The gated delta rule: a recurrent mixer whose state is one matrix S [dim, vdim] per head.
//
// Per token, from projections of the layer's input (query and key heads may be shared by
// several value heads):
//
//     q, k, v   <- silu(short causal convolution over time, per channel)
//     q, k      <- unit vectors per head (x / sqrt(sum x^2 + unit_eps)); q also times dim^-1/2
//     beta      =  sigmoid(b),   g = exp(-exp(A_log) * softplus(a + dt_bias))        (per head)
//     S <- g S;  w = beta (v - S^T k);  S <- S + k w^T;  o = S^T q                 (in this order)
//     out       =  o / rms(o) * norm_weight * silu(gate)                             (per head)
//
// Two options.  A decay per head and key channel (`decay_in` given): g [dim] = exp(-exp(A_log_head) * softplus(decay_in + dt_bias)),
// dt_bias then [heads, dim], and `S <- g S` scales the rows of S, each by its channel's factor.  And the output gate from a
// float32 tensor of its own, through a sigmoid instead of silu.
//
// What is carried from token to token per request lies in one float32 slot: the heads' matrices
// [heads, dim, vdim] followed by the last (taps - 1) inputs of the convolution [taps - 1, channels].
// All of the recurrence is float32: unit norms, decay, beta, the state, the read-out and its norm.
//
// Four kernels:
//   delta_prepare       one warp per (token, q/k/v head): convolution + silu (+ unit norm), and per
//                       token the heads' decay and beta, into float32 buffers
//   delta_conv_advance  per (row, channel): the slot's convolution inputs move on by the row's tokens
//   delta_recurrence    per (row, head, slice of vdim): walks the row's tokens in order; the columns
//                       of S are independent of each other, so a block owns COLS of them, a column's
//                       dim entries spread over P lanes that add up by shuffles
//   delta_gated_norm    one warp per (token, head): RMS norm of the read-out, weight, gate
// The order of every sum depends on the sizes only, so a token's result does not depend on how the
// step was cut or what else is in the batch.
#include "common.cuh"

namespace pylon {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// proj: [T, ld] projections in T (columns [q | k | v | ...] from column 0; gate_a / gate_b name the columns of a and b).
// conv_w: float32 [taps, channels] in the same channel order (tap by tap, so that a warp's channels lie side by side).  state: float32 [slots, slot_floats]; the convolution
// inputs start at conv_offset.  qkv: float32 [T, channels] out.  gates: float32 [T, 2, heads] out (decay, beta).
template <typename T, int MAX_TAPS>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ conv_w, int taps,
                                     const float* __restrict__ state, long long slot_floats, long long conv_offset,
                                     const int* __restrict__ token_row, const int* __restrict__ q_start, const int* __restrict__ slots,
                                     float* __restrict__ qkv, float* __restrict__ gates, const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias, int col_a, int col_b, int heads, int kv_heads, int dim, int vdim,
                                     float unit_eps, int num_tokens, const float* __restrict__ decay_in, long long ld_decay,
                                     float* __restrict__ decays) {
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int plain_units = 2 * kv_heads + heads + 1;   // q heads, k heads, v heads, and one unit for the token's gates
  const int units = plain_units + (decay_in != nullptr ? heads : 0);   // with a decay per channel: one more unit per head
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * units) return;
  const int t = (int)(item / units), unit = (int)(item % units);
  const int row = token_row[t];
  if (row < 0) return;
  const T* mine = proj + (long long)t * ld;
  if (unit >= plain_units) {
    const int h = unit - plain_units;
    const float rate = expf(a_log[h]);
    for (int e = lane; e < dim; e += 32)
      decays[((long long)t * heads + h) * dim + e] = expf(-rate * softplus_f(decay_in[(long long)t * ld_decay + h * dim + e] + dt_bias[h * dim + e]));
    return;
  }
  if (unit == plain_units - 1) {
    for (int h = lane; h < heads; h += 32) {
      const float b = to_float<T>(mine[col_b + h]);
      if (decay_in == nullptr) gates[(long long)t * 2 * heads + h] = expf(-expf(a_log[h]) * softplus_f(to_float<T>(mine[col_a + h]) + dt_bias[h]));
      else gates[(long long)t * 2 * heads + h] = 1.f;
      gates[(long long)t * 2 * heads + heads + h] = 1.f / (1.f + expf(-b));
    }
    return;
  }
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const bool is_value = unit >= 2 * kv_heads;
  const int size = is_value ? vdim : dim;
  const int first = is_value ? 2 * kv_heads * dim + (unit - 2 * kv_heads) * vdim : unit * dim;
  const int index = t - q_start[row];        // the token's place among the row's tokens of this step
  const float* old = state + (long long)slots[row] * slot_floats + conv_offset;   // [taps - 1, channels]
  auto convolved = [&](int c) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;       // how many tokens before this one
      float input;
      if (back <= index) input = to_float<T>(proj[(long long)(t - back) * ld + c]);
      else input = old[(long long)(taps - 1 - (back - index)) * channels + c];
      acc = fmaf(conv_w[(long long)j * channels + c], input, acc);
    }
    return silu_f(acc);
  };
  constexpr int KEPT = 8;   // heads of up to 256 channels stay in registers between the convolution and the scaling
  float sumsq = 0.f;
  if (size <= 32 * KEPT) {
    float kept[KEPT];
#pragma unroll
    for (int n = 0; n < KEPT; ++n) {
      const int e = lane + 32 * n;
      kept[n] = e < size ? convolved(first + e) : 0.f;
      sumsq = fmaf(kept[n], kept[n], sumsq);
    }
    float factor = 1.f;
    if (!is_value) {
      factor = rsqrtf(warp_sum(sumsq) + unit_eps);
      if (unit < kv_heads) factor *= rsqrtf((float)dim);
    }
#pragma unroll
    for (int n = 0; n < KEPT; ++n) {
      const int e = lane + 32 * n;
      if (e < size) qkv[(long long)t * channels + first + e] = is_value ? kept[n] : kept[n] * factor;
    }
    return;
  }
  for (int e = lane; e < size; e += 32) {
    const float value = convolved(first + e);
    qkv[(long long)t * channels + first + e] = value;   // values are done; queries and keys are scaled below
    sumsq = fmaf(value, value, sumsq);
  }
  if (is_value) return;
  sumsq = warp_sum(sumsq);
  float factor = rsqrtf(sumsq + unit_eps);
  if (unit < kv_heads) factor *= rsqrtf((float)dim);
  __syncwarp();
  for (int e = lane; e < size; e += 32) qkv[(long long)t * channels + first + e] *= factor;
}

// The last (taps - 1) convolution inputs of every row move on by the tokens the row brought.
template <typename T, int MAX_TAPS>
__global__ void delta_conv_advance_kernel(const T* __restrict__ proj, long long ld, int taps, float* __restrict__ state,
                                          long long slot_floats, long long conv_offset, const int* __restrict__ q_start,
                                          const int* __restrict__ slots, int channels, int num_rows) {
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)num_rows * channels) return;
  const int row = (int)(item / channels), c = (int)(item % channels);
  const int begin = q_start[row], count = q_start[row + 1] - begin;
  if (count <= 0) return;
  float* mine = state + (long long)slots[row] * slot_floats + conv_offset;
  float kept[MAX_TAPS];
#pragma unroll
  for (int m = 0; m < MAX_TAPS; ++m) {
    if (m < taps - 1) {
      const int rel = count - (taps - 1) + m;   // place among the row's tokens; negative: from the old inputs
      kept[m] = rel >= 0 ? to_float<T>(proj[(long long)(begin + rel) * ld + c]) : mine[(long long)(m + count) * channels + c];
    }
  }
#pragma unroll
  for (int m = 0; m < MAX_TAPS; ++m)
    if (m < taps - 1) mine[(long long)m * channels + c] = kept[m];
}

__device__ __forceinline__ void delta_copy_async(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void delta_copy_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void delta_copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void delta_copy_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// grid (slices of vdim, heads, rows); block = cols columns x P lanes (padded to a whole warp).  PER >= ceil(dim / P).
// The walk over a row's tokens is a chain of dependent steps, so what a step waits for must be near: the tokens' keys,
// queries, values, decay and beta come into shared memory `stage_tokens` tokens at a time by asynchronous copies, two
// stages in turn, while the tokens of the stage before are walked.  Shared memory: 2 * stage_tokens * per_token floats, per_token
// = 2 dim + cols + 2 rounded up to a multiple of 4.  `wide`: dim, vdim, cols and the buffers' addresses allow 16-byte copies (copies of
// 4 bytes go through one by one: with them alone a token took 1,400 cycles).
template <int PER, bool CHANNEL>
__global__ void delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ gates, float* __restrict__ state,
                                        long long slot_floats, const int* __restrict__ q_start, const int* __restrict__ slots,
                                        float* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int lanes, int cols,
                                        int stage_tokens, int wide, const float* __restrict__ decays) {
  extern __shared__ __align__(16) float stages[];
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int P = lanes;
  const int p = threadIdx.x % P;
  const int column = threadIdx.x / P;                  // among the block's columns
  const int j = blockIdx.x * cols + column;            // my column of the head's matrix
  const int head = blockIdx.y, row = blockIdx.z;
  const int begin = q_start[row], end = q_start[row + 1];
  if (end <= begin) return;
  const bool live = j < vdim && column < cols;   // a block is padded to a whole warp: the lanes beyond its columns only keep the shuffles whole
  const int kv = head / (heads / kv_heads);
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const int q_col = kv * dim, k_col = kv_heads * dim + kv * dim, v_col = 2 * kv_heads * dim + head * vdim + blockIdx.x * cols;
  const int base = (CHANNEL ? 3 : 2) * dim;              // keys | queries | with a decay per channel: the head's decays
  const int per_token = (base + cols + 2 + 3) & ~3;      // ... | the block's values | decay | beta | padding
  float* mine = state + (long long)slots[row] * slot_floats + ((long long)head * dim) * vdim + j;   // S[i, j] at mine[i * vdim]
  float s[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = p + n * P;
    s[n] = (live && i < dim) ? mine[(long long)i * vdim] : 0.f;
  }
  auto fetch = [&](int first, int buffer) {
    const int count = min(stage_tokens, end - first);
    if (wide) {
      const int units = (base + cols) >> 2;   // 16-byte units of a token: keys, queries, (decays,) values
      for (int x = threadIdx.x; x < count * units; x += blockDim.x) {
        const int token = x / units, e = (x - token * units) << 2;
        float* dst = stages + ((long long)buffer * stage_tokens + token) * per_token + e;
        const float* src = qkv + (long long)(first + token) * channels;
        if (e < dim) delta_copy_async_16(dst, src + k_col + e);
        else if (e < 2 * dim) delta_copy_async_16(dst, src + q_col + (e - dim));
        else if (CHANNEL && e < base) delta_copy_async_16(dst, decays + ((long long)(first + token) * heads + head) * dim + (e - 2 * dim));
        else if (blockIdx.x * cols + (e - base) < vdim) delta_copy_async_16(dst, src + v_col + (e - base));   // vdim is a multiple of 4: a unit is inside or outside
        else dst[0] = dst[1] = dst[2] = dst[3] = 0.f;
      }
      for (int x = threadIdx.x; x < count * 2; x += blockDim.x) {
        const int token = x >> 1;
        delta_copy_async(stages + ((long long)buffer * stage_tokens + token) * per_token + base + cols + (x & 1),
                         gates + (long long)(first + token) * 2 * heads + ((x & 1) ? heads + head : head));
      }
      delta_copy_commit();
      return;
    }
    for (int token = 0; token < count; ++token) {
      float* dst = stages + ((long long)buffer * stage_tokens + token) * per_token;
      const float* src = qkv + (long long)(first + token) * channels;
      const float* gate = gates + (long long)(first + token) * 2 * heads;
      for (int e = threadIdx.x; e < base + cols + 2; e += blockDim.x) {
        if (e < dim) delta_copy_async(dst + e, src + k_col + e);
        else if (e < 2 * dim) delta_copy_async(dst + e, src + q_col + (e - dim));
        else if (CHANNEL && e < base) delta_copy_async(dst + e, decays + ((long long)(first + token) * heads + head) * dim + (e - 2 * dim));
        else if (e < base + cols) {
          const int c = e - base;
          if (blockIdx.x * cols + c < vdim) delta_copy_async(dst + e, src + v_col + c); else dst[e] = 0.f;
        } else delta_copy_async(dst + e, gate + (e == base + cols ? head : heads + head));
      }
    }
    delta_copy_commit();
  };
  int buffer = 0;
  fetch(begin, 0);
  for (int first = begin; first < end; first += stage_tokens) {
    if (first + stage_tokens < end) {
      fetch(first + stage_tokens, buffer ^ 1);
      delta_copy_wait<1>();
    } else {
      delta_copy_wait<0>();
    }
    __syncthreads();
    const int count = min(stage_tokens, end - first);
    const float* staged = stages + (long long)buffer * stage_tokens * per_token;
#pragma unroll 2
    for (int token = 0; token < count; ++token) {
      const float* here = staged + token * per_token;
      float k[PER], q[PER], gk[CHANNEL ? PER : 1];
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        const int i = p + n * P;
        k[n] = i < dim ? here[i] : 0.f;
        q[n] = i < dim ? here[dim + i] : 0.f;
        if (CHANNEL) gk[n] = i < dim ? here[2 * dim + i] : 0.f;
      }
      const float v = column < cols ? here[base + column] : 0.f;
      const float g = here[base + cols], beta = here[base + cols + 1];
      float dot[2] = {0.f, 0.f};   // two chains: the sums are chains of dependent steps
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        s[n] *= CHANNEL ? gk[n] : g;
        dot[n & 1] = fmaf(s[n], k[n], dot[n & 1]);
      }
      float sum = dot[0] + dot[1];
      for (int offset = P >> 1; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      const float w = beta * (v - sum);
      float read[2] = {0.f, 0.f};
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        s[n] = fmaf(k[n], w, s[n]);
        read[n & 1] = fmaf(s[n], q[n], read[n & 1]);
      }
      float o = read[0] + read[1];
      for (int offset = P >> 1; offset > 0; offset >>= 1) o += __shfl_xor_sync(0xffffffffu, o, offset);
      if (live && p == 0) out[((long long)(first + token) * heads + head) * vdim + j] = o;
    }
    __syncthreads();   // the stage is free to be filled again
    buffer ^= 1;
  }
  if (live) {
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = p + n * P;
      if (i < dim) mine[(long long)i * vdim] = s[n];
    }
  }
}

// The same walk for the sizes models have, with everything that shapes the inner loop known to the compiler: dim = PER * P
// exactly, P lanes to a column (4 to 32), PER a multiple of 4, 16-byte copies.  A lane holds entries (4 (m P + p) + c) of its column, c < 4,
// m < PER / 4, so that the lanes of a column read a token's keys and queries as neighbouring 16-byte units (no bank conflicts, a
// quarter of the loads), the shuffles unroll and no access needs a bound.  A token costs some 100 instructions this way; the
// general kernel above, with its sizes at run time, took 341 (measured at dim 128: 0.33 us a token against 0.48 us).
template <int PER, int P, bool CHANNEL>
__global__ void __launch_bounds__(128) delta_recurrence_exact_kernel(const float* __restrict__ qkv, const float* __restrict__ gates,
                                                                     float* __restrict__ state, long long slot_floats,
                                                                     const int* __restrict__ q_start, const int* __restrict__ slots,
                                                                     float* __restrict__ out, int heads, int kv_heads, int vdim, int stage_tokens,
                                                                     const float* __restrict__ decays) {
  constexpr int DIM = PER * P, COLS = 128 / P, BASE = (CHANNEL ? 3 : 2) * DIM, PER_TOKEN = BASE + COLS + 4;   // keys | queries | (the head's decays per channel) | the block's values | decay, beta, padding
  extern __shared__ __align__(16) float stages[];
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int p = threadIdx.x % P, column = threadIdx.x / P;
  const int j = blockIdx.x * COLS + column;
  const int head = blockIdx.y, row = blockIdx.z;
  const int begin = q_start[row], end = q_start[row + 1];
  if (end <= begin) return;
  const bool live = j < vdim;
  const int kv = head / (heads / kv_heads);
  const int channels = 2 * kv_heads * DIM + heads * vdim;
  const int q_col = kv * DIM, k_col = kv_heads * DIM + kv * DIM, v_col = 2 * kv_heads * DIM + head * vdim + blockIdx.x * COLS;
  float* mine = state + (long long)slots[row] * slot_floats + ((long long)head * DIM) * vdim + j;   // S[i, j] at mine[i * vdim]
  float s[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = 4 * ((n >> 2) * P + p) + (n & 3);
    s[n] = live ? mine[(long long)i * vdim] : 0.f;
  }
  auto fetch = [&](int first, int buffer) {
    const int count = min(stage_tokens, end - first);
    constexpr int UNITS = (BASE + COLS) / 4;
    for (int x = threadIdx.x; x < count * UNITS; x += 128) {
      const int token = x / UNITS, e = (x - token * UNITS) << 2;
      float* dst = stages + (buffer * stage_tokens + token) * PER_TOKEN + e;
      const float* src = qkv + (long long)(first + token) * channels;
      if (e < DIM) delta_copy_async_16(dst, src + k_col + e);
      else if (e < 2 * DIM) delta_copy_async_16(dst, src + q_col + (e - DIM));
      else if (CHANNEL && e < BASE) delta_copy_async_16(dst, decays + ((long long)(first + token) * heads + head) * DIM + (e - 2 * DIM));
      else if (blockIdx.x * COLS + (e - BASE) < vdim) delta_copy_async_16(dst, src + v_col + (e - BASE));
      else dst[0] = dst[1] = dst[2] = dst[3] = 0.f;
    }
    for (int x = threadIdx.x; x < count * 2; x += 128) {
      const int token = x >> 1;
      delta_copy_async(stages + (buffer * stage_tokens + token) * PER_TOKEN + BASE + COLS + (x & 1),
                       gates + (long long)(first + token) * 2 * heads + ((x & 1) ? heads + head : head));
    }
    delta_copy_commit();
  };
  // A warp issues in order, so the two sums of a token - S^T k, which the next token waits for, and the read-out S^T q, which
  // nothing waits for - are not left one behind the other: the read-out of token t is added up lane by lane beside the first sum
  // of token t + 1 (from the state as token t left it, before the next decay), and both go through one round of shuffles.
  float q_before[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) q_before[n] = 0.f;
  float* o_before = nullptr;   // where the pending read-out goes
  int buffer = 0;
  fetch(begin, 0);
  for (int first = begin; first < end; first += stage_tokens) {
    if (first + stage_tokens < end) {
      fetch(first + stage_tokens, buffer ^ 1);
      delta_copy_wait<1>();
    } else {
      delta_copy_wait<0>();
    }
    __syncthreads();
    const int count = min(stage_tokens, end - first);
    const float* staged = stages + buffer * stage_tokens * PER_TOKEN;
    float* o_row = out + ((long long)first * heads + head) * vdim + j;
#pragma unroll 2
    for (int token = 0; token < count; ++token) {
      const float* here = staged + token * PER_TOKEN;
      float k[PER], q[PER], gk[CHANNEL ? PER : 1];
#pragma unroll
      for (int m = 0; m < PER / 4; ++m) {
        const float4 k4 = *reinterpret_cast<const float4*>(here + 4 * (m * P + p));
        const float4 q4 = *reinterpret_cast<const float4*>(here + DIM + 4 * (m * P + p));
        k[4 * m] = k4.x; k[4 * m + 1] = k4.y; k[4 * m + 2] = k4.z; k[4 * m + 3] = k4.w;
        q[4 * m] = q4.x; q[4 * m + 1] = q4.y; q[4 * m + 2] = q4.z; q[4 * m + 3] = q4.w;
        if (CHANNEL) {
          const float4 g4 = *reinterpret_cast<const float4*>(here + 2 * DIM + 4 * (m * P + p));
          gk[4 * m] = g4.x; gk[4 * m + 1] = g4.y; gk[4 * m + 2] = g4.z; gk[4 * m + 3] = g4.w;
        }
      }
      const float v = here[BASE + column];
      const float g = here[BASE + COLS], beta = here[BASE + COLS + 1];
      constexpr int CHAINS = PER >= 16 ? 4 : 2;   // the sums are chains of dependent steps: several side by side
      float dot[CHAINS], read[CHAINS];
#pragma unroll
      for (int c = 0; c < CHAINS; ++c) dot[c] = read[c] = 0.f;
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        read[n % CHAINS] = fmaf(s[n], q_before[n], read[n % CHAINS]);
        s[n] *= CHANNEL ? gk[n] : g;
        dot[n % CHAINS] = fmaf(s[n], k[n], dot[n % CHAINS]);
      }
      float sum = dot[0] + dot[1], o = read[0] + read[1];
      if (CHAINS == 4) { sum += dot[2] + dot[3]; o += read[2] + read[3]; }
#pragma unroll
      for (int offset = P >> 1; offset > 0; offset >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        o += __shfl_xor_sync(0xffffffffu, o, offset);
      }
      if (o_before != nullptr && live && p == 0) *o_before = o;
      const float w = beta * (v - sum);
#pragma unroll
      for (int n = 0; n < PER; ++n) {
        s[n] = fmaf(k[n], w, s[n]);
        q_before[n] = q[n];
      }
      o_before = o_row + (long long)token * heads * vdim;
    }
    __syncthreads();   // the stage is free to be filled again
    buffer ^= 1;
  }
  {   // the last token's read-out
    float read[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < PER; ++n) read[n & 1] = fmaf(s[n], q_before[n], read[n & 1]);
    float o = read[0] + read[1];
#pragma unroll
    for (int offset = P >> 1; offset > 0; offset >>= 1) o += __shfl_xor_sync(0xffffffffu, o, offset);
    if (o_before != nullptr && live && p == 0) *o_before = o;
  }
  if (live) {
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = 4 * ((n >> 2) * P + p) + (n & 3);
      mine[(long long)i * vdim] = s[n];
    }
  }
}

// o: float32 [T, heads, vdim]; gate: columns of proj from col_gate, [heads, vdim], through silu - or, if given, the float32 tensor
// gate_own [T, ld_gate] through a sigmoid; out [T, heads * vdim] in T.
template <typename T>
__global__ void delta_gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, long long ld, int col_gate,
                                        const float* __restrict__ weight, T* __restrict__ out, int heads, int vdim, float eps,
                                        int num_tokens, const float* __restrict__ gate_own, long long ld_gate) {
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), head = (int)(item % heads);
  const float* mine = o + item * vdim;
  float sumsq = 0.f;
  for (int e = lane; e < vdim; e += 32) sumsq = fmaf(mine[e], mine[e], sumsq);
  sumsq = warp_sum(sumsq);
  const float inv = rsqrtf(sumsq / (float)vdim + eps);
  const T* gate = proj + (long long)t * ld + col_gate + head * vdim;
  T* dst = out + item * vdim;
  if (gate_own != nullptr) {
    const float* own = gate_own + (long long)t * ld_gate + head * vdim;
    for (int e = lane; e < vdim; e += 32) dst[e] = from_float<T>(mine[e] * inv * weight[e] * (1.f / (1.f + expf(-own[e]))));
    return;
  }
  for (int e = lane; e < vdim; e += 32) dst[e] = from_float<T>(mine[e] * inv * weight[e] * silu_f(to_float<T>(gate[e])));
}

}  // namespace pylon

using namespace pylon;

constexpr int DELTA_MAX_TAPS = 16;

template <typename T>
static int launch_delta(const void* proj_v, long long ld, const float* conv_w, int taps, float* state, long long slot_floats,
                        const int* token_row, const int* q_start, const int* slots, float* qkv, float* gates, float* o, void* out_v,
                        const float* a_log, const float* dt_bias, const float* norm_weight, int col_a, int col_b, int col_gate,
                        int heads, int kv_heads, int dim, int vdim, float unit_eps, float norm_eps, int num_tokens, int num_rows,
                        const float* decay_in, long long ld_decay, float* decays, const float* gate_own, long long ld_gate,
                        cudaStream_t stream) {
  const T* proj = (const T*)proj_v;
  const bool channel = decay_in != nullptr;
  T* out = (T*)out_v;
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const long long conv_offset = (long long)heads * dim * vdim;
  {
    const int warps = 4;
    const long long items = (long long)num_tokens * (2 * kv_heads + heads + 1 + (channel ? heads : 0));
    launch_dependent(delta_prepare_kernel<T, DELTA_MAX_TAPS>, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream,
        proj, ld, conv_w, taps, state, slot_floats, conv_offset, token_row, q_start, slots, qkv, gates, a_log, dt_bias, col_a, col_b,
        heads, kv_heads, dim, vdim, unit_eps, num_tokens, decay_in, ld_decay, decays);
  }
  if (taps > 1) {
    const long long items = (long long)num_rows * channels;
    launch_dependent(delta_conv_advance_kernel<T, DELTA_MAX_TAPS>, dim3((unsigned)((items + 127) / 128)), dim3(128), 0, stream,
        proj, ld, taps, state, slot_floats, conv_offset, q_start, slots, channels, num_rows);
  }
  bool walked = false;
  if (dim % 4 == 0 && vdim % 4 == 0 && (uintptr_t)qkv % 16 == 0) {
    // the sizes models have: the kernel whose inner loop is fixed when it is compiled
#define PYLON_DELTA_EXACT(PER_, P_)                                                                                                   \
    if (!walked && dim == PER_ * P_) {                                                                                                 \
      constexpr int COLS_ = 128 / P_;                                                                                                  \
      const int per_token_ = (channel ? 3 : 2) * PER_ * P_ + COLS_ + 4;                                                                \
      int stage_tokens = 16;                                                                                                           \
      while (stage_tokens > 1 && 2LL * stage_tokens * per_token_ * (long long)sizeof(float) > 48 * 1024) stage_tokens /= 2;            \
      if (channel)                                                                                                                     \
        launch_dependent(delta_recurrence_exact_kernel<PER_, P_, true>, dim3((vdim + COLS_ - 1) / COLS_, heads, num_rows), dim3(128),  \
                         2ull * stage_tokens * per_token_ * sizeof(float), stream, qkv, gates, state, slot_floats, q_start, slots, o,  \
                         heads, kv_heads, vdim, stage_tokens, (const float*)decays);                                                   \
      else                                                                                                                             \
        launch_dependent(delta_recurrence_exact_kernel<PER_, P_, false>, dim3((vdim + COLS_ - 1) / COLS_, heads, num_rows), dim3(128), \
                         2ull * stage_tokens * per_token_ * sizeof(float), stream, qkv, gates, state, slot_floats, q_start, slots, o,  \
                         heads, kv_heads, vdim, stage_tokens, (const float*)decays);                                                   \
      walked = true;                                                                                                                   \
    }
    // lanes to a column: as few as leave a lane 32 entries at most (fewer rounds of shuffles, longer sums per lane: at dim 128 four
    // lanes of 32 entries took 445 us for 2,048 tokens where eight of 16 took 540)
    PYLON_DELTA_EXACT(8, 4) PYLON_DELTA_EXACT(16, 4) PYLON_DELTA_EXACT(24, 4) PYLON_DELTA_EXACT(32, 4) PYLON_DELTA_EXACT(20, 8) PYLON_DELTA_EXACT(24, 8)
    PYLON_DELTA_EXACT(28, 8) PYLON_DELTA_EXACT(32, 8) PYLON_DELTA_EXACT(24, 16) PYLON_DELTA_EXACT(32, 16) PYLON_DELTA_EXACT(32, 32)
#undef PYLON_DELTA_EXACT
  }
  if (!walked) {
    // P lanes share a column: the fewest (a power of two, at least 4) that leave a lane at most 16 entries, so a block of
    // 128 threads owns 32 columns at most and the slices of vdim fill the device also with few heads.
    int lanes = 4;
    while (lanes < 32 && (dim + lanes - 1) / lanes > 16) lanes *= 2;
    const int per = (dim + lanes - 1) / lanes;
    int cols = 128 / lanes;
    while (cols > 1 && cols / 2 >= vdim) cols /= 2;
    dim3 grid((vdim + cols - 1) / cols, heads, num_rows);
    const int threads = cols * lanes;   // a multiple of 32 unless one warp holds all columns; shuffles stay inside groups of P lanes
    // tokens per stage: 16, or as many as two stages of leave under 48 KB (at least 2 for every dim this entry takes)
    const int per_token = ((channel ? 3 : 2) * dim + cols + 2 + 3) & ~3;
    const int wide = dim % 4 == 0 && vdim % 4 == 0 && cols % 4 == 0 && (uintptr_t)qkv % 16 == 0;
    int stage_tokens = 16;
    while (stage_tokens > 1 && 2LL * stage_tokens * per_token * (long long)sizeof(float) > 48 * 1024) stage_tokens /= 2;
    const size_t smem = 2ull * stage_tokens * per_token * sizeof(float);
#define PYLON_DELTA_RECURRENCE(N) \
    if (channel) launch_dependent(delta_recurrence_kernel<N, true>, grid, dim3(threads < 32 ? 32 : threads), smem, stream, qkv, gates, state, slot_floats, q_start, slots, o, heads, kv_heads, dim, vdim, lanes, cols, stage_tokens, wide, (const float*)decays); \
    else launch_dependent(delta_recurrence_kernel<N, false>, grid, dim3(threads < 32 ? 32 : threads), smem, stream, qkv, gates, state, slot_floats, q_start, slots, o, heads, kv_heads, dim, vdim, lanes, cols, stage_tokens, wide, (const float*)decays)
    if (per <= 4) PYLON_DELTA_RECURRENCE(4);
    else if (per <= 8) PYLON_DELTA_RECURRENCE(8);
    else if (per <= 16) PYLON_DELTA_RECURRENCE(16);
    else PYLON_DELTA_RECURRENCE(32);
#undef PYLON_DELTA_RECURRENCE
  }
  {
    const int warps = 4;
    const long long items = (long long)num_tokens * heads;
    launch_dependent(delta_gated_norm_kernel<T>, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream,
        o, proj, ld, col_gate, norm_weight, out, heads, vdim, norm_eps, num_tokens, gate_own, ld_gate);
  }
  PYLON_CHECK_LAUNCH("gated_delta_rule");
}

// proj: [num_tokens, ld] with columns [q (kv_heads * dim) | k (kv_heads * dim) | v (heads * vdim) | ...] and the gate
// (heads * vdim), a and b (heads each) at the columns named.  state: float32 [slots, slot_floats], slot_floats >=
// heads * dim * vdim + (taps - 1) * channels.  qkv [T, channels], gates [T, 2 * heads], o [T, heads * vdim]: float32 work
// buffers.  out: [T, heads * vdim] in dtype.  Rows without tokens leave their slot as it is.  decay_in (or null): float32 [T, ld_decay],
// heads * dim columns, the decay's input per head and key channel; dt_bias is then [heads * dim], decays a float32 work buffer
// [T, heads * dim], and col_a is not read.  gate_own (or null): float32 [T, ld_gate], heads * vdim columns, the output gate's input, through a
// sigmoid; col_gate is then not read.
extern "C" int pylon_gated_delta_rule(const void* proj, long long ld, const float* conv_w, int taps, float* state,
                                      long long slot_floats, const int* token_row, const int* q_start, const int* slots, float* qkv,
                                      float* gates, float* o, void* out, const float* a_log, const float* dt_bias,
                                      const float* norm_weight, int col_a, int col_b, int col_gate, int heads, int kv_heads, int dim,
                                      int vdim, float unit_eps, float norm_eps, int num_tokens, int num_rows, int dtype,
                                      const float* decay_in, long long ld_decay, float* decays, const float* gate_own, long long ld_gate,
                                      cudaStream_t stream) {
  if (num_tokens <= 0 || num_rows <= 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads) PYLON_REFUSE("gated_delta_rule: %d heads over %d query/key heads", heads, kv_heads);
  if (dim < 1 || dim > 1024 || vdim < 1) PYLON_REFUSE("gated_delta_rule: dim %d (1 to 1024), vdim %d", dim, vdim);
  if (taps < 1 || taps > DELTA_MAX_TAPS) PYLON_REFUSE("gated_delta_rule: %d taps (1 to %d)", taps, DELTA_MAX_TAPS);
  if (heads > 65535 || num_rows > 65535) PYLON_REFUSE("gated_delta_rule: %d heads, %d rows", heads, num_rows);
  const long long needed = (long long)heads * dim * vdim + (long long)(taps - 1) * (2 * kv_heads * dim + heads * vdim);
  if (decay_in != nullptr && decays == nullptr) PYLON_REFUSE("gated_delta_rule: a decay per channel needs its work buffer");
  if (slot_floats < needed) PYLON_REFUSE("gated_delta_rule: a slot of %lld floats, %lld needed", slot_floats, needed);
#define PYLON_DELTA_ARGS proj, ld, conv_w, taps, state, slot_floats, token_row, q_start, slots, qkv, gates, o, out, a_log, dt_bias, \
    norm_weight, col_a, col_b, col_gate, heads, kv_heads, dim, vdim, unit_eps, norm_eps, num_tokens, num_rows, decay_in, ld_decay, decays, \
    gate_own, ld_gate, stream
  if (dtype == PYLON_DTYPE_F32) return launch_delta<float>(PYLON_DELTA_ARGS);
  if (dtype == PYLON_DTYPE_BF16) return launch_delta<__nv_bfloat16>(PYLON_DELTA_ARGS);
#undef PYLON_DELTA_ARGS
  PYLON_REFUSE("gated_delta_rule: unknown dtype %d", dtype);
}
