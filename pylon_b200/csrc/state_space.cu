// A state-space mixer with one decay per head and step (the scalar-decay form of a selective state-space layer).
//
// Per token, from one projection of the layer's input with columns [z | x | B | C | dt] (z, x: heads * vdim; B, C:
// groups * N; dt: heads; head h uses the B and C of group h / (heads / groups)):
//
//     x, B, C  <- silu(short causal convolution over time, per channel, with a bias)
//     dt       <- softplus(dt + dt_bias),   a = exp(-exp(A_log) * dt)                       (per head)
//     S <- a S + dt B x^T   (S is [N, vdim] per head),   y = S^T C + D x                    (the read-out sees the token's write)
//     out      =  rmsnorm_in_groups(y * silu(z)) * norm_weight                              (the gate comes before the norm)
//
// What is carried from token to token per request lies in one float32 slot: the heads' matrices [heads, N, vdim]
// followed by the last (taps - 1) inputs of the convolution [taps - 1, channels], channels = heads * vdim + 2 groups N.
// Everything behind the projection is float32.
//
// Four kernels:
//   ssm_prepare        a thread per (token, channel): convolution + bias + silu; per (token, head) the step and the decay
//   ssm_conv_advance   per (row, channel): the slot's convolution inputs move on by the row's tokens
//   ssm_recurrence     per (row, head, slice of vdim): walks the row's tokens in order; the columns of S do not depend on
//                      each other, so a block owns `cols` of them, a column's N entries spread over P lanes whose
//                      read-outs add up by shuffles.  The state's update is elementwise: nothing in the walk waits for a sum.
//   ssm_gated_norm     a block per (token, norm group): gate, RMS norm of the group, weight
// The order of every sum depends on the sizes only, so a token's result does not depend on how the step was cut or what
// else is in the batch.
#include "common.cuh"

namespace pylon {

__device__ __forceinline__ float ssm_silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float ssm_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// proj: [T, ld]; the convolved columns start at col_conv, the steps at col_dt.  conv_w: float32 [taps, channels], conv_b [channels].
// xbc: float32 [T, channels] out.  gates: float32 [T, 2, heads] out (decay, step).
template <typename T>
__global__ void ssm_prepare_kernel(const T* __restrict__ proj, long long ld, int col_conv, int col_dt, const float* __restrict__ conv_w,
                                   const float* __restrict__ conv_b, int taps, const float* __restrict__ state, long long slot_floats,
                                   long long conv_offset, const int* __restrict__ token_row, const int* __restrict__ q_start,
                                   const int* __restrict__ slots, float* __restrict__ xbc, float* __restrict__ gates,
                                   const float* __restrict__ a_log, const float* __restrict__ dt_bias, int heads, int channels, int num_tokens) {
  grid_dependency_wait();
  allow_dependents();
  const int per_token = channels + heads;
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)num_tokens * per_token) return;
  const int t = (int)(item / per_token), c = (int)(item % per_token);
  const int row = token_row[t];
  if (row < 0) return;
  if (c >= channels) {
    const int h = c - channels;
    const float dt = ssm_softplus(to_float<T>(proj[(long long)t * ld + col_dt + h]) + dt_bias[h]);
    gates[(long long)t * 2 * heads + h] = expf(-expf(a_log[h]) * dt);
    gates[(long long)t * 2 * heads + heads + h] = dt;
    return;
  }
  const int index = t - q_start[row];        // the token's place among the row's tokens of this step
  const float* old = state + (long long)slots[row] * slot_floats + conv_offset;   // [taps - 1, channels]
  float acc = conv_b[c];
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;           // how many tokens before this one
    float input;
    if (back <= index) input = to_float<T>(proj[(long long)(t - back) * ld + col_conv + c]);
    else input = old[(long long)(taps - 1 - (back - index)) * channels + c];
    acc = fmaf(conv_w[(long long)j * channels + c], input, acc);
  }
  xbc[(long long)t * channels + c] = ssm_silu(acc);
}

template <typename T, int MAX_TAPS>
__global__ void ssm_conv_advance_kernel(const T* __restrict__ proj, long long ld, int col_conv, int taps, float* __restrict__ state,
                                        long long slot_floats, long long conv_offset, const int* __restrict__ q_start,
                                        const int* __restrict__ slots, int channels, int num_rows) {
  grid_dependency_wait();
  allow_dependents();
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
      kept[m] = rel >= 0 ? to_float<T>(proj[(long long)(begin + rel) * ld + col_conv + c]) : mine[(long long)(m + count) * channels + c];
    }
  }
#pragma unroll
  for (int m = 0; m < MAX_TAPS; ++m)
    if (m < taps - 1) mine[(long long)m * channels + c] = kept[m];
}

__device__ __forceinline__ void ssm_copy_async(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void ssm_copy_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void ssm_copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void ssm_copy_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// grid (slices of vdim, heads, rows); block = cols columns x P lanes (padded to a whole warp).  PER >= ceil(N / P), a multiple of 4.
// A lane holds PER neighbouring entries of its column: p * PER, p * PER + 1, ...  The tokens' B, C, the block's x, decay and step
// come into shared memory `stage_tokens` tokens at a time by asynchronous copies, two stages in turn.  In a stage a token's B (and C)
// lies lane by lane, PER entries and 4 floats of padding each, so that a lane reads its entries as 16-byte words and the eight lanes
// that read in one go do not meet in a bank (four entries need no padding); entries past N are zeros, written once.  Shared memory: 2 * stage_tokens * per_token
// floats, per_token = 2 P ssm_lane_floats(PER) + cols + 2 rounded up to a multiple of 4.  `wide`: N, cols and the buffers' addresses allow
// 16-byte copies.
__host__ __device__ constexpr int ssm_lane_floats(int per) { return per == 4 ? 4 : per + 4; }

template <int PER, int P>
__global__ void ssm_recurrence_kernel(const float* __restrict__ xbc, const float* __restrict__ gates, float* __restrict__ state,
                                      long long slot_floats, const int* __restrict__ q_start, const int* __restrict__ slots,
                                      const float* __restrict__ skip, float* __restrict__ out, int heads, int groups, int n_state, int vdim,
                                      int cols, int stage_tokens, int wide) {
  extern __shared__ __align__(16) float stages[];
  constexpr int LANE_FLOATS = ssm_lane_floats(PER);
  grid_dependency_wait();
  allow_dependents();
  const int p = threadIdx.x % P;
  const int column = threadIdx.x / P;
  const int j = blockIdx.x * cols + column;
  const int head = blockIdx.y, row = blockIdx.z;
  const int begin = q_start[row], end = q_start[row + 1];
  if (end <= begin) return;
  const bool live = j < vdim && column < cols;
  const int group = head / (heads / groups);
  const int inner = heads * vdim, channels = inner + 2 * groups * n_state;
  const int x_col = head * vdim + blockIdx.x * cols, b_col = inner + group * n_state, c_col = inner + groups * n_state + group * n_state;
  const int c_at = P * LANE_FLOATS, x_at = 2 * c_at, gate_at = x_at + cols;   // where C, x and the two gates lie in a token's stage
  const int per_token = (gate_at + 2 + 3) & ~3;
  float* mine = state + (long long)slots[row] * slot_floats + ((long long)head * n_state) * vdim + j;   // S[n, j] at mine[n * vdim]
  const float d_skip = skip[head];
  float s[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = p * PER + n;
    s[n] = (live && i < n_state) ? mine[(long long)i * vdim] : 0.f;
  }
  if (P * PER > n_state) {   // the entries past N are zeros and stay so: no copy writes them
    for (int x = threadIdx.x; x < 2 * stage_tokens * per_token; x += blockDim.x) stages[x] = 0.f;
    __syncthreads();
  }
  auto place = [&](int e) { return (e / PER) * LANE_FLOATS + e % PER; };   // where entry e of B or C lies
  auto fetch = [&](int first, int buffer) {
    const int count = min(stage_tokens, end - first);
    if (wide) {
      const int units = (2 * n_state + cols) >> 2;
      for (int x = threadIdx.x; x < count * units; x += blockDim.x) {
        const int token = x / units, e = (x - token * units) << 2;
        float* dst = stages + ((long long)buffer * stage_tokens + token) * per_token;
        const float* src = xbc + (long long)(first + token) * channels;
        if (e < n_state) ssm_copy_async_16(dst + place(e), src + b_col + e);
        else if (e < 2 * n_state) ssm_copy_async_16(dst + c_at + place(e - n_state), src + c_col + (e - n_state));
        else if (blockIdx.x * cols + (e - 2 * n_state) < vdim) ssm_copy_async_16(dst + x_at + (e - 2 * n_state), src + x_col + (e - 2 * n_state));   // vdim is a multiple of 4 here
        else { float* z = dst + x_at + (e - 2 * n_state); z[0] = z[1] = z[2] = z[3] = 0.f; }
      }
      for (int x = threadIdx.x; x < count * 2; x += blockDim.x) {
        const int token = x >> 1;
        ssm_copy_async(stages + ((long long)buffer * stage_tokens + token) * per_token + gate_at + (x & 1),
                       gates + (long long)(first + token) * 2 * heads + ((x & 1) ? heads + head : head));
      }
      ssm_copy_commit();
      return;
    }
    for (int token = 0; token < count; ++token) {
      float* dst = stages + ((long long)buffer * stage_tokens + token) * per_token;
      const float* src = xbc + (long long)(first + token) * channels;
      const float* gate = gates + (long long)(first + token) * 2 * heads;
      for (int e = threadIdx.x; e < 2 * n_state + cols + 2; e += blockDim.x) {
        if (e < n_state) ssm_copy_async(dst + place(e), src + b_col + e);
        else if (e < 2 * n_state) ssm_copy_async(dst + c_at + place(e - n_state), src + c_col + (e - n_state));
        else if (e < 2 * n_state + cols) {
          const int c = e - 2 * n_state;
          if (blockIdx.x * cols + c < vdim) ssm_copy_async(dst + x_at + c, src + x_col + c); else dst[x_at + c] = 0.f;
        } else ssm_copy_async(dst + gate_at + (e - 2 * n_state - cols), gate + (e == 2 * n_state + cols ? head : heads + head));
      }
    }
    ssm_copy_commit();
  };
  int buffer = 0;
  fetch(begin, 0);
  for (int first = begin; first < end; first += stage_tokens) {
    if (first + stage_tokens < end) {
      fetch(first + stage_tokens, buffer ^ 1);
      ssm_copy_wait<1>();
    } else {
      ssm_copy_wait<0>();
    }
    __syncthreads();
    const int count = min(stage_tokens, end - first);
    const float* staged = stages + (long long)buffer * stage_tokens * per_token;
    float* y_at = out + ((long long)first * heads + head) * vdim + j;
#pragma unroll 4
    for (int token = 0; token < count; ++token) {
      const float* here = staged + token * per_token;
      const float x = column < cols ? here[x_at + column] : 0.f;
      const float a = here[gate_at], dt = here[gate_at + 1];
      const float write = dt * x;
      const float4* b4 = reinterpret_cast<const float4*>(here + p * LANE_FLOATS);
      const float4* c4 = reinterpret_cast<const float4*>(here + c_at + p * LANE_FLOATS);
      float read[2] = {0.f, 0.f};
#pragma unroll
      for (int n = 0; n < PER; n += 4) {
        const float4 b = b4[n >> 2], c = c4[n >> 2];
        s[n] = fmaf(s[n], a, b.x * write);
        s[n + 1] = fmaf(s[n + 1], a, b.y * write);
        s[n + 2] = fmaf(s[n + 2], a, b.z * write);
        s[n + 3] = fmaf(s[n + 3], a, b.w * write);
        read[0] = fmaf(s[n], c.x, read[0]);
        read[1] = fmaf(s[n + 1], c.y, read[1]);
        read[0] = fmaf(s[n + 2], c.z, read[0]);
        read[1] = fmaf(s[n + 3], c.w, read[1]);
      }
      float y = read[0] + read[1];
#pragma unroll
      for (int offset = P >> 1; offset > 0; offset >>= 1) y += __shfl_xor_sync(0xffffffffu, y, offset);
      if (live && p == 0) y_at[(long long)token * heads * vdim] = fmaf(d_skip, x, y);
    }
    __syncthreads();   // the stage is free to be filled again
    buffer ^= 1;
  }
  if (live) {
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = p * PER + n;
      if (i < n_state) mine[(long long)i * vdim] = s[n];
    }
  }
}

// y: float32 [T, inner]; z: columns of proj from col_gate; out [T, inner] in T.  A block per (token, norm group).  HELD: a thread
// keeps its (at most SSM_NORM_HELD) gated values between the sum of squares and the result: y and z are read and silu taken once.
constexpr int SSM_NORM_HELD = 8;
template <typename T, bool HELD>
__global__ void ssm_gated_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, long long ld, int col_gate,
                                      const float* __restrict__ weight, T* __restrict__ out, int inner, int norm_groups, float eps) {
  __shared__ float scratch[33];
  grid_dependency_wait();
  allow_dependents();
  const int t = blockIdx.x / norm_groups, part = blockIdx.x % norm_groups;
  const int size = inner / norm_groups, first = part * size;
  const float* mine = y + (long long)t * inner + first;
  const T* gate = proj + (long long)t * ld + col_gate + first;
  T* dst = out + (long long)t * inner + first;
  float sumsq = 0.f;
  if (HELD) {
    float held[SSM_NORM_HELD];
#pragma unroll
    for (int k = 0; k < SSM_NORM_HELD; ++k) {
      const int e = threadIdx.x + k * blockDim.x;
      held[k] = e < size ? mine[e] * ssm_silu(to_float<T>(gate[e])) : 0.f;
      sumsq = fmaf(held[k], held[k], sumsq);
    }
    sumsq = block_sum(sumsq, scratch);
    const float inv = rsqrtf(sumsq / (float)size + eps);
#pragma unroll
    for (int k = 0; k < SSM_NORM_HELD; ++k) {
      const int e = threadIdx.x + k * blockDim.x;
      if (e < size) dst[e] = from_float<T>(held[k] * inv * weight[first + e]);
    }
  } else {
    for (int e = threadIdx.x; e < size; e += blockDim.x) {
      const float g = mine[e] * ssm_silu(to_float<T>(gate[e]));
      sumsq = fmaf(g, g, sumsq);
    }
    sumsq = block_sum(sumsq, scratch);
    const float inv = rsqrtf(sumsq / (float)size + eps);
    for (int e = threadIdx.x; e < size; e += blockDim.x)
      dst[e] = from_float<T>(mine[e] * ssm_silu(to_float<T>(gate[e])) * inv * weight[first + e]);
  }
}

}  // namespace pylon

using namespace pylon;

constexpr int SSM_MAX_TAPS = 16;

template <typename T>
static int launch_state_space(const void* proj_v, long long ld, const float* conv_w, const float* conv_b, int taps, float* state,
                              long long slot_floats, const int* token_row, const int* q_start, const int* slots, float* xbc, float* gates,
                              float* y, void* out_v, const float* a_log, const float* dt_bias, const float* skip, const float* norm_weight,
                              int heads, int groups, int n_state, int vdim, int norm_groups, float norm_eps, int num_tokens, int num_rows,
                              cudaStream_t stream) {
  const T* proj = (const T*)proj_v;
  T* out = (T*)out_v;
  const int inner = heads * vdim, channels = inner + 2 * groups * n_state;
  const int col_conv = inner, col_dt = inner + channels;
  const long long conv_offset = (long long)heads * n_state * vdim;
  {
    const long long items = (long long)num_tokens * (channels + heads);
    launch_dependent(ssm_prepare_kernel<T>, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, stream, proj, ld, col_conv, col_dt, conv_w,
                     conv_b, taps, state, slot_floats, conv_offset, token_row, q_start, slots, xbc, gates, a_log, dt_bias, heads, channels,
                     num_tokens);
  }
  if (taps > 1) {
    const long long items = (long long)num_rows * channels;
    launch_dependent(ssm_conv_advance_kernel<T, SSM_MAX_TAPS>, dim3((unsigned)((items + 127) / 128)), dim3(128), 0, stream, proj, ld,
                     col_conv, taps, state, slot_floats, conv_offset, q_start, slots, channels, num_rows);
  }
  {
    // P lanes share a column: the fewest (a power of two) that leave a lane at most 16 entries.  (More lanes with fewer entries
    // each put more warps on a scheduler, but a warp's work per token is mostly what does not shrink with its entries - staging,
    // shuffles, the store - so 32 lanes of 4 entries took as long as 8 lanes of 16 at 32 heads of 128 x 64.)
    int lanes = 1;
    while (lanes < 32 && (n_state + lanes - 1) / lanes > 16) lanes *= 2;
    const int per = (n_state + lanes - 1) / lanes;
    int cols = 128 / lanes;
    while (cols > 1 && cols / 2 >= vdim) cols /= 2;
    dim3 grid((vdim + cols - 1) / cols, heads, num_rows);
    const int threads = cols * lanes;
    const int per_slot = lanes > 1 ? (per <= 16 ? 16 : 32) : per <= 4 ? 4 : per <= 8 ? 8 : 16;   // the kernel's PER
    const int per_token = (2 * lanes * ssm_lane_floats(per_slot) + cols + 2 + 3) & ~3;
    const int wide = n_state % 4 == 0 && vdim % 4 == 0 && cols % 4 == 0 && (uintptr_t)xbc % 16 == 0;
    int stage_tokens = 16;
    while (stage_tokens > 1 && 2LL * stage_tokens * per_token * (long long)sizeof(float) > 48 * 1024) stage_tokens /= 2;
    const size_t smem = 2ull * stage_tokens * per_token * sizeof(float);
#define PYLON_SSM_RECURRENCE(N, L) \
    launch_dependent(ssm_recurrence_kernel<N, L>, grid, dim3(threads < 32 ? 32 : threads), smem, stream, xbc, gates, state, slot_floats, q_start, slots, skip, y, heads, groups, n_state, vdim, cols, stage_tokens, wide)
    // the lanes and entries that the rule above can give: one lane up to 16 entries, then 16 entries up to 32 lanes, then 32 entries
    if (lanes == 1) { if (per <= 4) PYLON_SSM_RECURRENCE(4, 1); else if (per <= 8) PYLON_SSM_RECURRENCE(8, 1); else PYLON_SSM_RECURRENCE(16, 1); }
    else if (lanes == 2) PYLON_SSM_RECURRENCE(16, 2);
    else if (lanes == 4) PYLON_SSM_RECURRENCE(16, 4);
    else if (lanes == 8) PYLON_SSM_RECURRENCE(16, 8);
    else if (lanes == 16) PYLON_SSM_RECURRENCE(16, 16);
    else if (per <= 16) PYLON_SSM_RECURRENCE(16, 32);
    else PYLON_SSM_RECURRENCE(32, 32);
#undef PYLON_SSM_RECURRENCE
  }
  {
    // as many threads as leave each at most SSM_NORM_HELD values of a norm group (by the sizes alone)
    const int size = inner / norm_groups;
    int threads = 128;
    while (threads < 1024 && threads * SSM_NORM_HELD < size) threads *= 2;
    if (threads * SSM_NORM_HELD >= size)
      launch_dependent(ssm_gated_norm_kernel<T, true>, dim3((unsigned)num_tokens * norm_groups), dim3(threads), 0, stream, y, proj, ld, 0, norm_weight,
                       out, inner, norm_groups, norm_eps);
    else
      launch_dependent(ssm_gated_norm_kernel<T, false>, dim3((unsigned)num_tokens * norm_groups), dim3(threads), 0, stream, y, proj, ld, 0, norm_weight,
                       out, inner, norm_groups, norm_eps);
  }
  PYLON_CHECK_LAUNCH("state_space");
}

// proj: [num_tokens, ld] with columns [z (heads * vdim) | x (heads * vdim) | B (groups * N) | C (groups * N) | dt (heads)].
// state: float32 [slots, slot_floats], slot_floats >= heads * N * vdim + (taps - 1) * channels.  xbc [T, channels], gates
// [T, 2 * heads], y [T, heads * vdim]: float32 work buffers.  out: [T, heads * vdim] in dtype.  Rows without tokens leave their slot
// as it is; tokens without a row are skipped.
extern "C" int pylon_state_space(const void* proj, long long ld, const float* conv_w, const float* conv_b, int taps, float* state,
                                 long long slot_floats, const int* token_row, const int* q_start, const int* slots, float* xbc, float* gates,
                                 float* y, void* out, const float* a_log, const float* dt_bias, const float* skip, const float* norm_weight,
                                 int heads, int groups, int n_state, int vdim, int norm_groups, float norm_eps, int num_tokens, int num_rows,
                                 int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || num_rows <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups) PYLON_REFUSE("state_space: %d heads over %d groups", heads, groups);
  if (n_state < 1 || n_state > 1024 || vdim < 1) PYLON_REFUSE("state_space: state %d (1 to 1024), vdim %d", n_state, vdim);
  if (norm_groups < 1 || (heads * vdim) % norm_groups) PYLON_REFUSE("state_space: %d channels in %d norm groups", heads * vdim, norm_groups);
  if (taps < 1 || taps > SSM_MAX_TAPS) PYLON_REFUSE("state_space: %d taps (1 to %d)", taps, SSM_MAX_TAPS);
  if (heads > 65535 || num_rows > 65535) PYLON_REFUSE("state_space: %d heads, %d rows", heads, num_rows);
  const long long needed = (long long)heads * n_state * vdim + (long long)(taps - 1) * (heads * vdim + 2 * groups * n_state);
  if (slot_floats < needed) PYLON_REFUSE("state_space: a slot of %lld floats, %lld needed", slot_floats, needed);
#define PYLON_SSM_ARGS proj, ld, conv_w, conv_b, taps, state, slot_floats, token_row, q_start, slots, xbc, gates, y, out, a_log, dt_bias, skip, \
    norm_weight, heads, groups, n_state, vdim, norm_groups, norm_eps, num_tokens, num_rows, stream
  if (dtype == PYLON_DTYPE_F32) return launch_state_space<float>(PYLON_SSM_ARGS);
  if (dtype == PYLON_DTYPE_BF16) return launch_state_space<__nv_bfloat16>(PYLON_SSM_ARGS);
#undef PYLON_SSM_ARGS
  PYLON_REFUSE("state_space: unknown dtype %d", dtype);
}
