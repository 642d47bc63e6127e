// A matrix of memory per head with exponential gates (the mLSTM cell of xLSTM), walked token by token.
//
// Per token and head, from one product of the layer's input, columns [q | k | v | g] (q, k: heads x dim; v, g: heads x vdim), and
// float32 gate logits [i | f] (heads each) with biases:
//
//     q = q * dim^-1/2
//     i = cap * tanh((i + b_i) / cap)                      the log of the input gate
//     f = logsigmoid(cap * tanh((f + b_f) / cap))          the log of the forget gate
//     m' = max(f + m, i)                                   a running maximum that starts at 0
//     S = exp(f + m - m') S + exp(i - m') k v^T            S [dim, vdim] and n [dim] start at zero
//     n = exp(f + m - m') n + exp(i - m') k
//     o = S^T q / (max(|n . q|, exp(-m')) + read_eps)
//
// and then, in a second kernel, each head's o divided by its root mean square (eps inside the root), times a weight [heads * vdim],
// times sigmoid(g), in the compute dtype: ready for the output projection.
//
// What a request carries from token to token is one float32 slot, per head [S (dim x vdim) | n (dim) | m].  The columns of S do not
// see each other, so a block takes (request row, head, 16 columns): warp w of four owns four neighbouring columns, lane l the rows
// l, l + 32, ... of them (up to MEMORY_MAX_DIM rows), and a read-out is a sum over the lanes.  n and m are kept by every warp (the
// same arithmetic in the same order from the gates' logarithms, which a kernel ahead of the walk forms for every token and head - the
// walk is left with three exponentials a token); the four read-outs of a warp are summed over its lanes together, each round of
// exchanges halving what a lane holds (6 exchanges instead of 20); the first warp leaves their new values in a buffer beside the state, and a small kernel behind
// the walk puts them into the slot (a block that starts late must still find the old ones there).  Everything is float32.
#include "common.cuh"

namespace pylon {

constexpr int MEMORY_COLUMNS = 4;        // columns of S a warp owns
constexpr int MEMORY_WARPS = 4;
constexpr int MEMORY_MAX_DIM = 256;      // rows of S: up to 8 a lane

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// In place on gate logits float32 [T, 2 heads] (the input gates', then the forget gates'): i = cap tanh((i + b_i) / cap),
// f = logsigmoid(cap tanh((f + b_f) / cap)).
__global__ void matrix_memory_gates_kernel(float* __restrict__ gates, const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, int heads,
                                           long long total) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const int column = (int)(item % (2 * heads));
  const float x = gates[item];
  gates[item] = column < heads ? cap * tanhf((x + bias_i[column]) / cap) : log_sigmoid_f(cap * tanhf((x + bias_f[column - heads]) / cap));
}

// Sums of four values over the 32 lanes of a warp: every lane l returns the sum of value 2 (l / 16) + l / 8 % 2.
__device__ __forceinline__ float warp_sum_of_four(const float (&v)[4], int lane) {
  float two[2];
  const bool high16 = lane & 16, high8 = lane & 8;
#pragma unroll
  for (int c = 0; c < 2; ++c) two[c] = (high16 ? v[c + 2] : v[c]) + __shfl_xor_sync(0xffffffffu, high16 ? v[c] : v[c + 2], 16);
  float one = (high8 ? two[1] : two[0]) + __shfl_xor_sync(0xffffffffu, high8 ? two[0] : two[1], 8);
  one += __shfl_xor_sync(0xffffffffu, one, 4);
  one += __shfl_xor_sync(0xffffffffu, one, 2);
  one += __shfl_xor_sync(0xffffffffu, one, 1);
  return one;
}
static_assert(MEMORY_COLUMNS == 4, "the read-outs of a warp are summed four at a time");

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(MEMORY_WARPS * 32) matrix_memory_scan_kernel(
    const T* __restrict__ proj, long long ld, const float* __restrict__ gate_logits,
    float read_eps, float* __restrict__ state, long long state_floats, const int* __restrict__ q_start, const int* __restrict__ slots,
    float* __restrict__ read, float* __restrict__ fresh, int heads, int dim, int vdim) {
  grid_dependency_wait();
  allow_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y, row = blockIdx.z;
  const int j0 = (blockIdx.x * MEMORY_WARPS + warp) * MEMORY_COLUMNS;
  const int first = q_start[row], count = q_start[row + 1] - first;
  if (count <= 0 || j0 >= vdim) return;   // a row without tokens (a padded step) keeps its state; a warp beyond the last column has nothing
  float* mine = state + (long long)slots[row] * state_floats + (long long)head * ((long long)dim * vdim + dim + 1);
  float* n_state = mine + (long long)dim * vdim;
  float s[PER_LANE][MEMORY_COLUMNS], n[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int d = lane + 32 * i;
    n[i] = d < dim ? n_state[d] : 0.f;
#pragma unroll
    for (int c = 0; c < MEMORY_COLUMNS; ++c) s[i][c] = (d < dim && j0 + c < vdim) ? mine[(long long)d * vdim + j0 + c] : 0.f;
  }
  float m = n_state[dim];
  const float q_scale = rsqrtf((float)dim);
  const long long q_column = (long long)head * dim, k_column = (long long)heads * dim + q_column;
  const long long v_column = 2LL * heads * dim + (long long)head * vdim + j0;
  // what the next token brings is asked for while this token's arithmetic runs: the walk is a chain over tokens, and a load that
  // starts only when its token's turn comes would put the memory's latency into every link
  float k_next[PER_LANE], q_next[PER_LANE], v_next[MEMORY_COLUMNS], gi_next, gf_next;
  auto fetch = [&](int t) {
    const T* x = proj + (long long)t * ld;
    gi_next = gate_logits[(long long)t * 2 * heads + head];            // the gates' logarithms, formed ahead of the walk
    gf_next = gate_logits[(long long)t * 2 * heads + heads + head];
#pragma unroll
    for (int c = 0; c < MEMORY_COLUMNS; ++c) v_next[c] = j0 + c < vdim ? to_float<T>(x[v_column + c]) : 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int d = lane + 32 * i;
      k_next[i] = d < dim ? to_float<T>(x[k_column + d]) : 0.f;
      q_next[i] = d < dim ? to_float<T>(x[q_column + d]) * q_scale : 0.f;
    }
  };
  fetch(first);
#pragma unroll 2
  for (int t = first; t < first + count; ++t) {
    float k_now[PER_LANE], q_now[PER_LANE], v[MEMORY_COLUMNS], o[MEMORY_COLUMNS];
    const float gi = gi_next, gf = gf_next;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) { k_now[i] = k_next[i]; q_now[i] = q_next[i]; }
#pragma unroll
    for (int c = 0; c < MEMORY_COLUMNS; ++c) { v[c] = v_next[c]; o[c] = 0.f; }
    if (t + 1 < first + count) fetch(t + 1);
    // the sum f + m with what its rounding drops (two-sum): where it becomes the new maximum, the old content is kept times
    // exp(-dropped), not times one - else every token would leave a factor of a few units in the last place of m behind
    const float sum = gf + m;
    const float part = sum - gf;
    const float dropped = (gf - (sum - part)) + (m - part);
    const float m_new = fmaxf(sum, gi);
    const float keep = expf((sum - m_new) + dropped), take = expf(gi - m_new);
    m = m_new;
    float nq = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const float k = k_now[i] * take, q = q_now[i];
      n[i] = fmaf(keep, n[i], k);
      nq = fmaf(n[i], q, nq);
#pragma unroll
      for (int c = 0; c < MEMORY_COLUMNS; ++c) {
        s[i][c] = fmaf(keep, s[i][c], k * v[c]);
        o[c] = fmaf(s[i][c], q, o[c]);
      }
    }
    nq = warp_sum(nq);
    const float below = fmaxf(fabsf(nq), expf(-m)) + read_eps;
    const float result = warp_sum_of_four(o, lane);
    const int column = ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1);
    if ((lane & 7) == 0 && j0 + column < vdim) read[(long long)t * heads * vdim + (long long)head * vdim + j0 + column] = result / below;
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d >= dim) continue;
    if (j0 == 0) fresh[((long long)row * heads + head) * (dim + 1) + d] = n[i];
#pragma unroll
    for (int c = 0; c < MEMORY_COLUMNS; ++c)
      if (j0 + c < vdim) mine[(long long)d * vdim + j0 + c] = s[i][c];
  }
  if (j0 == 0 && lane == 0) fresh[((long long)row * heads + head) * (dim + 1) + dim] = m;
}

// The same walk for bfloat16 rows of whole 16-byte pieces, fed through shared memory: what 8 tokens bring (k and q of the head, the
// block's 16 columns of v, the gates' logarithms) comes by cp.async into one of two stages while the 8 tokens before are walked, once
// for the block's four warps.  The walk is a chain over tokens; a load that starts a token ahead does not cover the way to the far
// half of the L2 (measured: 2,280 cycles a token with loads one token ahead, of which the arithmetic is some 600).
constexpr int MEMORY_CHUNK = 8;

__device__ __forceinline__ void memory_copy_or_zeros(void* shared, const void* global, bool real, int bytes) {
  const unsigned target = (unsigned)__cvta_generic_to_shared(shared);
  const int taken = real ? bytes : 0;   // what is not copied is written as zeros
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(target), "l"(global), "r"(taken) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(target), "l"(global), "r"(taken) : "memory");
}

template <int PER_LANE>
__global__ void __launch_bounds__(MEMORY_WARPS * 32) matrix_memory_scan_staged_kernel(
    const __nv_bfloat16* __restrict__ proj, long long ld, const float* __restrict__ gate_logits, float read_eps, float* __restrict__ state,
    long long state_floats, const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ read, float* __restrict__ fresh,
    int heads, int dim, int vdim) {
  extern __shared__ __align__(16) unsigned char memory_stages[];
  constexpr int BLOCK_COLUMNS = MEMORY_WARPS * MEMORY_COLUMNS;
  const int stage_bytes = MEMORY_CHUNK * (2 * dim * 2 + BLOCK_COLUMNS * 2 + 8);   // k, q, the block's v columns, two gates per token
  grid_dependency_wait();
  allow_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y, row = blockIdx.z;
  const int jb = blockIdx.x * BLOCK_COLUMNS, j0 = jb + warp * MEMORY_COLUMNS;
  const int first = q_start[row], count = q_start[row + 1] - first;
  if (count <= 0) return;   // a row without tokens (a padded step) keeps its state; the same for every thread of the block
  const bool active = j0 < vdim;   // a warp beyond the last column still helps to copy
  float* mine = state + (long long)slots[row] * state_floats + (long long)head * ((long long)dim * vdim + dim + 1);
  float* n_state = mine + (long long)dim * vdim;
  float s[PER_LANE][MEMORY_COLUMNS], n[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int d = lane + 32 * i;
    n[i] = d < dim ? n_state[d] : 0.f;
#pragma unroll
    for (int c = 0; c < MEMORY_COLUMNS; ++c) s[i][c] = (active && d < dim && j0 + c < vdim) ? mine[(long long)d * vdim + j0 + c] : 0.f;
  }
  float m = n_state[dim];
  const float q_scale = rsqrtf((float)dim);
  const long long q_column = (long long)head * dim, k_column = (long long)heads * dim + q_column;
  const long long v_column = 2LL * heads * dim + (long long)head * vdim + jb;
  const int row_pieces = dim / 8, token_pieces = 2 * row_pieces + BLOCK_COLUMNS / 8;
  auto issue = [&](int chunk) {
    unsigned char* base = memory_stages + (size_t)(chunk & 1) * stage_bytes;
    __nv_bfloat16* k_stage = reinterpret_cast<__nv_bfloat16*>(base);
    __nv_bfloat16* q_stage = k_stage + MEMORY_CHUNK * dim;
    __nv_bfloat16* v_stage = q_stage + MEMORY_CHUNK * dim;
    float* gate_stage = reinterpret_cast<float*>(v_stage + MEMORY_CHUNK * BLOCK_COLUMNS);
    for (int x = threadIdx.x; x < MEMORY_CHUNK * token_pieces; x += blockDim.x) {
      const int token = x / token_pieces, piece = x % token_pieces;
      const bool there = chunk * MEMORY_CHUNK + token < count;
      const __nv_bfloat16* from = proj + (long long)(first + chunk * MEMORY_CHUNK + token) * ld;
      if (piece < row_pieces) memory_copy_or_zeros(k_stage + token * dim + piece * 8, there ? from + k_column + piece * 8 : proj, there, 16);
      else if (piece < 2 * row_pieces) memory_copy_or_zeros(q_stage + token * dim + (piece - row_pieces) * 8, there ? from + q_column + (piece - row_pieces) * 8 : proj, there, 16);
      else {
        const int column = (piece - 2 * row_pieces) * 8;
        const bool real = there && jb + column < vdim;
        memory_copy_or_zeros(v_stage + token * BLOCK_COLUMNS + column, real ? from + v_column + column : proj, real, 16);
      }
    }
    if (threadIdx.x < MEMORY_CHUNK * 2) {
      const int token = threadIdx.x >> 1, which = threadIdx.x & 1;
      const bool there = chunk * MEMORY_CHUNK + token < count;
      memory_copy_or_zeros(gate_stage + threadIdx.x, there ? gate_logits + (long long)(first + chunk * MEMORY_CHUNK + token) * 2 * heads + which * heads + head : gate_logits,
                           there, 4);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  const int chunks = (count + MEMORY_CHUNK - 1) / MEMORY_CHUNK;
  issue(0);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    if (chunk + 1 < chunks) issue(chunk + 1);
    else asm volatile("cp.async.commit_group;\n" ::: "memory");   // an empty group, so that the groups count the chunks
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");        // this chunk has arrived (for this thread's copies)
    __syncthreads();                                               // ... for everyone's
    const unsigned char* base = memory_stages + (size_t)(chunk & 1) * stage_bytes;
    const __nv_bfloat16* k_stage = reinterpret_cast<const __nv_bfloat16*>(base);
    const __nv_bfloat16* q_stage = k_stage + MEMORY_CHUNK * dim;
    const __nv_bfloat16* v_stage = q_stage + MEMORY_CHUNK * dim;
    const float* gate_stage = reinterpret_cast<const float*>(v_stage + MEMORY_CHUNK * BLOCK_COLUMNS);
    const int here = count - chunk * MEMORY_CHUNK < MEMORY_CHUNK ? count - chunk * MEMORY_CHUNK : MEMORY_CHUNK;
    if (active) {
      for (int token = 0; token < here; ++token) {
        const int t = first + chunk * MEMORY_CHUNK + token;
        const float gi = gate_stage[2 * token], gf = gate_stage[2 * token + 1];
        float v[MEMORY_COLUMNS], o[MEMORY_COLUMNS];
#pragma unroll
        for (int c = 0; c < MEMORY_COLUMNS; ++c) {
          v[c] = __bfloat162float(v_stage[token * BLOCK_COLUMNS + warp * MEMORY_COLUMNS + c]);   // zeros beyond the last column
          o[c] = 0.f;
        }
        const float sum = gf + m;                                   // two-sum: see the kernel above
        const float part = sum - gf;
        const float dropped = (gf - (sum - part)) + (m - part);
        const float m_new = fmaxf(sum, gi);
        const float keep = expf((sum - m_new) + dropped), take = expf(gi - m_new);
        m = m_new;
        float nq = 0.f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
          const int d = lane + 32 * i;
          const float k = d < dim ? __bfloat162float(k_stage[token * dim + d]) * take : 0.f;
          const float q = d < dim ? __bfloat162float(q_stage[token * dim + d]) * q_scale : 0.f;
          n[i] = fmaf(keep, n[i], k);
          nq = fmaf(n[i], q, nq);
#pragma unroll
          for (int c = 0; c < MEMORY_COLUMNS; ++c) {
            s[i][c] = fmaf(keep, s[i][c], k * v[c]);
            o[c] = fmaf(s[i][c], q, o[c]);
          }
        }
        nq = warp_sum(nq);
        const float below = fmaxf(fabsf(nq), expf(-m)) + read_eps;
        const float result = warp_sum_of_four(o, lane);
        const int column = ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1);
        if ((lane & 7) == 0 && j0 + column < vdim) read[(long long)t * heads * vdim + (long long)head * vdim + j0 + column] = result / below;
      }
    }
    __syncthreads();   // the stage is free for the chunk after the next
  }
  if (!active) return;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d >= dim) continue;
    if (j0 == 0) fresh[((long long)row * heads + head) * (dim + 1) + d] = n[i];
#pragma unroll
    for (int c = 0; c < MEMORY_COLUMNS; ++c)
      if (j0 + c < vdim) mine[(long long)d * vdim + j0 + c] = s[i][c];
  }
  if (j0 == 0 && lane == 0) fresh[((long long)row * heads + head) * (dim + 1) + dim] = m;
}

// fresh [rows, heads, dim + 1] -> the n and m of every head in the rows' slots; rows without tokens keep theirs.
__global__ void matrix_memory_commit_kernel(const float* __restrict__ fresh, float* __restrict__ state, long long state_floats, const int* __restrict__ q_start,
                                            const int* __restrict__ slots, int heads, int dim, int vdim) {
  grid_dependency_wait();
  allow_dependents();
  const int head = blockIdx.x, row = blockIdx.y;
  if (q_start[row + 1] - q_start[row] <= 0) return;
  float* n_state = state + (long long)slots[row] * state_floats + (long long)head * ((long long)dim * vdim + dim + 1) + (long long)dim * vdim;
  const float* from = fresh + ((long long)row * heads + head) * (dim + 1);
  for (int e = threadIdx.x; e <= dim; e += blockDim.x) n_state[e] = from[e];
}

// One warp per (token, head): read [T, heads * vdim] float32 -> out in T = read / rms(read over the head) * weight * sigmoid(g).
template <typename T>
__global__ void matrix_memory_out_kernel(const float* __restrict__ read, const T* __restrict__ proj, long long ld, long long g_column,
                                         const float* __restrict__ weight, float eps, T* __restrict__ out, int heads, int vdim, long long items) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long long t = item / heads;
  const int head = (int)(item % heads);
  const float* o = read + t * heads * vdim + (long long)head * vdim;
  float squares = 0.f;
  for (int j = lane; j < vdim; j += 32) squares = fmaf(o[j], o[j], squares);
  const float inv = rsqrtf(warp_sum(squares) / (float)vdim + eps);
  const T* g = proj + t * ld + g_column + (long long)head * vdim;
  T* dst = out + t * heads * vdim + (long long)head * vdim;
  for (int j = lane; j < vdim; j += 32) dst[j] = from_float<T>(o[j] * inv * weight[head * vdim + j] / (1.f + expf(-to_float<T>(g[j]))));
}

}  // namespace pylon

using namespace pylon;

// proj [T, ld] in dtype, columns [q | k | v | g]; gate_logits float32 [T, 2 heads], replaced by the gates' logarithms; state float32 [slots, state_floats]; read float32
// [T, heads * vdim] out; fresh float32 [num_rows, heads, dim + 1]: scratch.
extern "C" int pylon_matrix_memory_scan(const void* proj, long long ld, float* gate_logits, const float* bias_i, const float* bias_f, float cap,
                                        float read_eps, float* state, long long state_floats, const int* q_start, const int* slots, float* read, float* fresh,
                                        int heads, int dim, int vdim, int num_rows, int num_tokens, int dtype, cudaStream_t stream) {
  if (num_rows <= 0 || num_tokens <= 0) return 0;
  if (heads < 1 || dim < 1 || dim > MEMORY_MAX_DIM || vdim < 1 || !(cap > 0.f) || num_rows > 65535 || heads > 65535 ||
      state_floats < (long long)heads * ((long long)dim * vdim + dim + 1))
    PYLON_REFUSE("matrix_memory_scan: %d heads of %d x %d (at most %d rows), cap %f, %d request rows", heads, dim, vdim, MEMORY_MAX_DIM, cap, num_rows);
  const int per_block = MEMORY_WARPS * MEMORY_COLUMNS;
  const dim3 grid((unsigned)((vdim + per_block - 1) / per_block), (unsigned)heads, (unsigned)num_rows);
  const dim3 block(MEMORY_WARPS * 32);
  const int per_lane = (dim + 31) / 32;
  const long long gate_items = (long long)num_tokens * 2 * heads;
  launch_dependent(matrix_memory_gates_kernel, dim3((unsigned)((gate_items + 255) / 256)), dim3(256), 0, stream, gate_logits, bias_i, bias_f, cap, heads, gate_items);
#define PYLON_MEMORY(T, P)                                                                                                                          \
  launch_dependent(matrix_memory_scan_kernel<T, P>, grid, block, 0, stream, (const T*)proj, ld, (const float*)gate_logits, read_eps, state,          \
                   state_floats, q_start, slots, read, fresh, heads, dim, vdim)
#define PYLON_MEMORY_T(T)                                                                          \
  do {                                                                                             \
    if (per_lane <= 1) PYLON_MEMORY(T, 1); else if (per_lane <= 2) PYLON_MEMORY(T, 2);             \
    else if (per_lane <= 4) PYLON_MEMORY(T, 4); else PYLON_MEMORY(T, 8);                           \
  } while (0)
  const bool pieces = dim % 8 == 0 && vdim % 8 == 0 && ld % 8 == 0 && (uintptr_t)proj % 16 == 0;   // rows of whole 16-byte pieces: through shared memory
  const size_t staged_bytes = 2 * (size_t)MEMORY_CHUNK * (2 * dim * 2 + per_block * 2 + 8);
#define PYLON_MEMORY_STAGED(P)                                                                                                                        \
  launch_dependent(matrix_memory_scan_staged_kernel<P>, grid, block, staged_bytes, stream, (const __nv_bfloat16*)proj, ld, (const float*)gate_logits, \
                   read_eps, state, state_floats, q_start, slots, read, fresh, heads, dim, vdim)
  if (dtype == PYLON_DTYPE_F32) PYLON_MEMORY_T(float);
  else if (dtype == PYLON_DTYPE_BF16 && pieces) {
    if (per_lane <= 1) PYLON_MEMORY_STAGED(1); else if (per_lane <= 2) PYLON_MEMORY_STAGED(2);
    else if (per_lane <= 4) PYLON_MEMORY_STAGED(4); else PYLON_MEMORY_STAGED(8);
  }
  else if (dtype == PYLON_DTYPE_BF16) PYLON_MEMORY_T(__nv_bfloat16);
  else PYLON_REFUSE("matrix_memory_scan: unknown dtype %d", dtype);
#undef PYLON_MEMORY_STAGED
#undef PYLON_MEMORY_T
#undef PYLON_MEMORY
  launch_dependent(matrix_memory_commit_kernel, dim3((unsigned)heads, (unsigned)num_rows), dim3(64), 0, stream, (const float*)fresh, state, state_floats, q_start,
                   slots, heads, dim, vdim);
  PYLON_CHECK_LAUNCH("matrix_memory_scan");
}

extern "C" int pylon_matrix_memory_out(const float* read, const void* proj, long long ld, long long g_column, const float* weight, float eps, void* out,
                                       int heads, int vdim, int num_tokens, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (heads < 1 || vdim < 1) PYLON_REFUSE("matrix_memory_out: %d heads of %d", heads, vdim);
  const long long items = (long long)num_tokens * heads;
  const int warps = 4;
  const dim3 grid((unsigned)((items + warps - 1) / warps));
  if (dtype == PYLON_DTYPE_F32)
    launch_dependent(matrix_memory_out_kernel<float>, grid, dim3(warps * 32), 0, stream, read, (const float*)proj, ld, g_column, weight, eps, (float*)out, heads, vdim, items);
  else if (dtype == PYLON_DTYPE_BF16)
    launch_dependent(matrix_memory_out_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, stream, read, (const __nv_bfloat16*)proj, ld, g_column, weight, eps,
                     (__nv_bfloat16*)out, heads, vdim, items);
  else PYLON_REFUSE("matrix_memory_out: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("matrix_memory_out");
}
