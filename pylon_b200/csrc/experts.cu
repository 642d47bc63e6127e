// A mixture of experts: every token goes through `top` of `experts` small gated feed-forwards, chosen by a router.
//
//     z       = W_r h + b_r                       (float32, whatever the compute dtype)
//     chosen  = the `top` largest z (the lower index wins a tie),   share = softmax over the chosen z only
//     out     = sum over chosen e of share_e * W_down,e (act(W_gate,e h) * (W_up,e h))
//
// A second way of routing (RouteScored): the scores are s = sigmoid(z); the choice goes by s + correction (a learnt vector), and only
// among the experts of the `keep` best of `groups` equal groups of neighbours, a group's worth being the sum of its two largest choice
// scores (of its one, if it has one expert); share = s of the chosen (without the correction), divided by their sum plus share_eps.  The
// router matrix may have `extra` rows behind the experts': their logits leave as sigmoid(z) in extra_out [T, extra] (the gate of an
// expert that every token goes through, say).  An ungated expert is W_down act(W_up h): the first product applies act itself.
//
// Nothing here needs the host to know how many tokens an expert got, so the step stays one sequence of launches (and
// can be captured): the (token, choice) pairs are sorted by expert into row tiles of ROWS slots, every expert's span
// padded to whole tiles, and the grouped products run over the most tiles there can be; a tile beyond the last one, and
// a slot of padding inside a tile, is skipped.
//
//   experts_route     router logits, the top choices, their shares: a block per token in a step of few tokens, else a warp per four
//   experts_plan      one block: tokens per expert, the experts' first tiles, a slot for every pair
//   experts_product   a block per (row tile, column tile): rows gathered by slot, the expert's matrix, float32 sums in a
//                     fixed order of k; with GLU the gate and up tiles side by side and act(gate) * up written
//   experts_product_mma   the same on tensor cores (bfloat16, mma.sync m16n8k16), the matrices through a ring of cp.async stages:
//                     the products of a step of few tokens
//   experts_sort_rows the tokens' rows copied into the order of their slots, for a step of many tokens: its products are the
//                     grouped form of the tcgen05 kernel (gemm_tcgen05.cu) over row tiles of 128 slots
//   experts_gather    out[t] = sum_k share[t, k] * y[slot(t, k)], float32
// A row's sums do not depend on where in a tile it lies or what else is in the batch.
#include "common.cuh"
#include <mma.h>

namespace pylon {

constexpr int EXPERT_ROWS = 32;   // slots to a row tile

__device__ __forceinline__ float expert_activation(float x, int kind) {
  if (kind == 0) return x / (1.f + expf(-x));
  if (kind == 1) return fmaxf(x, 0.f);
  if (kind == 3) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));   // gelu, exact form
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// The row of w that holds column n of the gate (half 0) or of the up projection (half 1): the two halves one after the other, or
// (interleaved) alternating in groups of 8 rows, the layout the tcgen05 product's gated epilogue takes.
__device__ __forceinline__ long long glu_row(int n, int half, int n_out, int interleaved) {
  return interleaved ? ((long long)(n >> 3) << 4) + (half << 3) + (n & 7) : (long long)half * n_out + n;
}

// The `top` largest of a token's logits (the lower index wins a tie) and the softmax over just those; one warp.  logits is spoilt.
__device__ __forceinline__ void route_choose(float* logits, int* __restrict__ chosen, float* __restrict__ share, long long t, int experts, int top,
                                             int lane) {
  float first = 0.f, total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int where = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float z = logits[e];
      if (z > best) { best = z; where = e; }   // strictly larger: a lane keeps its lowest index
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
      if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
    }
    if (where == 0x7fffffff) where = 0;   // every logit was NaN or -inf: still a valid expert
    if (k == 0) first = best;
    const float weight = expf(best - first);
    total += weight;
    if (lane == 0) {
      chosen[t * top + k] = where;
      share[t * top + k] = weight;
      logits[where] = -INFINITY;
    }
    __syncwarp();
  }
  const float inv = 1.f / total;
  if (lane < top) share[t * top + lane] *= inv;
  for (int k = 32 + lane; k < top; k += 32) share[t * top + k] *= inv;
}

// How the scores are made and the choice is restricted; correction null: none; groups 0: no groups.
struct RouteScored {
  int on;                    // 0: the softmax form above; the rest is unused then
  const float* correction;   // [experts] or null
  int groups, keep;
  float share_eps;
  int extra;                 // rows of the router behind the experts'
  float* extra_out;          // [T, extra]
};

// One warp.  logits [experts + extra] holds z; choice [experts] and worth [groups] are scratch.
__device__ __forceinline__ void route_choose_scored(float* logits, float* choice, float* worth, int* __restrict__ chosen, float* __restrict__ share,
                                                    long long t, int experts, int top, int lane, const RouteScored& mode) {
  for (int x = lane; x < mode.extra; x += 32) mode.extra_out[t * mode.extra + x] = 1.f / (1.f + expf(-logits[experts + x]));
  for (int e = lane; e < experts; e += 32) {
    const float s = 1.f / (1.f + expf(-logits[e]));
    logits[e] = s;
    choice[e] = s + (mode.correction != nullptr ? mode.correction[e] : 0.f);
  }
  __syncwarp();
  if (mode.groups > 0) {
    const int size = experts / mode.groups;
    for (int g = lane; g < mode.groups; g += 32) {
      float first = -INFINITY, second = -INFINITY;
      for (int i = 0; i < size; ++i) {
        const float c = choice[g * size + i];
        if (c > first) { second = first; first = c; }
        else if (c > second) second = c;
      }
      worth[g] = size > 1 ? first + second : first;
    }
    __syncwarp();
    for (int k = 0; k < mode.keep; ++k) {   // the best group not yet kept, the lower index on a tie; a kept group's worth becomes +inf
      float best = -INFINITY;
      int where = 0x7fffffff;
      for (int g = lane; g < mode.groups; g += 32) {
        const float w = worth[g];
        if (w != INFINITY && (w > best || where == 0x7fffffff)) { best = w; where = g; }
      }
      for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
        if (other_where != 0x7fffffff && (where == 0x7fffffff || other > best || (other == best && other_where < where))) { best = other; where = other_where; }
      }
      if (lane == 0 && where != 0x7fffffff) worth[where] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (worth[e / size] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int where = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float c = choice[e];
      if (c > best) { best = c; where = e; }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
      if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
    }
    if (where == 0x7fffffff) where = 0;
    const float s = logits[where];
    total += s;
    if (lane == 0) {
      chosen[t * top + k] = where;
      share[t * top + k] = s;
      choice[where] = -INFINITY;
    }
    __syncwarp();
  }
  const float inv = 1.f / (total + mode.share_eps);
  if (lane < top) share[t * top + lane] *= inv;
  for (int k = 32 + lane; k < top; k += 32) share[t * top + k] *= inv;
}

// h [T, width] in T; router float32 [experts, width]; bias float32 [experts] or null.  chosen int32 [T, top], share float32 [T, top].
// A logit is summed in one order whatever the kernel form: the columns fall into four classes by (c mod 128) / 32; within class k
// lane l adds the columns 128 i + 32 k + l in order of i, the 32 lanes' sums are added up by the same butterfly, and the four class
// sums are added in order of k.  So a token's choice does not depend on how many tokens the step has.
//
// Many tokens: a warp takes TOKENS tokens side by side, so that a router value it has loaded serves all of them, and walks the four
// classes one after the other.  Shared memory: warps * TOKENS * experts floats.
template <typename T, int TOKENS>
__global__ void experts_route_kernel(const T* __restrict__ h, long long ld, const float* __restrict__ router, const float* __restrict__ bias,
                                     int* __restrict__ chosen, float* __restrict__ share, int width, int experts, int top, int num_tokens,
                                     RouteScored mode) {
  extern __shared__ float logits_all[];
  const int rows = experts + mode.extra;                                        // rows of the router
  const int per_token = rows + (mode.on ? experts + mode.groups : 0);           // floats of shared memory a token takes
  grid_dependency_wait();
  allow_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = (blockIdx.x * (blockDim.x >> 5) + warp) * TOKENS;
  if (t0 >= num_tokens) return;
  constexpr int SIDE = 8;   // experts side by side: the tokens' rows are read once per eight experts
  for (int e0 = 0; e0 < rows; e0 += SIDE) {
    float total[TOKENS][SIDE];
    for (int k = 0; k < 4; ++k) {
      float acc[TOKENS][SIDE];
#pragma unroll
      for (int i = 0; i < TOKENS; ++i)
#pragma unroll
        for (int j = 0; j < SIDE; ++j) acc[i][j] = 0.f;
#pragma unroll 4
      for (int c = 32 * k + lane; c < width; c += 128) {   // unrolled, so that several columns' loads are on their way at once
        float x[TOKENS], r[SIDE];
#pragma unroll
        for (int i = 0; i < TOKENS; ++i) x[i] = t0 + i < num_tokens ? to_float<T>(h[(long long)(t0 + i) * ld + c]) : 0.f;
#pragma unroll
        for (int j = 0; j < SIDE; ++j) r[j] = e0 + j < rows ? router[(long long)(e0 + j) * width + c] : 0.f;
#pragma unroll
        for (int i = 0; i < TOKENS; ++i)
#pragma unroll
          for (int j = 0; j < SIDE; ++j) acc[i][j] = fmaf(x[i], r[j], acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < TOKENS; ++i)
#pragma unroll
        for (int j = 0; j < SIDE; ++j) {
          const float z = warp_sum(acc[i][j]);
          total[i][j] = k == 0 ? z : total[i][j] + z;
        }
    }
#pragma unroll
    for (int i = 0; i < TOKENS; ++i)
#pragma unroll
      for (int j = 0; j < SIDE; ++j)
        if (lane == 0 && e0 + j < rows)
          logits_all[(warp * TOKENS + i) * per_token + e0 + j] = total[i][j] + (bias != nullptr && e0 + j < experts ? bias[e0 + j] : 0.f);
  }
  __syncwarp();
  for (int i = 0; i < TOKENS && t0 + i < num_tokens; ++i) {
    float* mine = logits_all + (warp * TOKENS + i) * per_token;
    if (mode.on) route_choose_scored(mine, mine + rows, mine + rows + experts, chosen, share, t0 + i, experts, top, lane, mode);
    else route_choose(mine, chosen, share, t0 + i, experts, top, lane);
  }
}

// Few tokens: a block of four warps per token, warp k takes class k.  Shared memory: (4 * 8 + experts) floats.
template <typename T>
__global__ void __launch_bounds__(128) experts_route_block_kernel(const T* __restrict__ h, long long ld, const float* __restrict__ router,
                                                                  const float* __restrict__ bias, int* __restrict__ chosen, float* __restrict__ share,
                                                                  int width, int experts, int top, RouteScored mode) {
  extern __shared__ float route_shared[];
  constexpr int SIDE = 8;
  float* parts = route_shared;               // [4][SIDE]
  float* logits = route_shared + 4 * SIDE;   // [experts + extra], then with mode.on [experts] choice scores and [groups] groups' worths
  const int rows = experts + mode.extra;
  grid_dependency_wait();
  allow_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = blockIdx.x;
  for (int e0 = 0; e0 < rows; e0 += SIDE) {
    float acc[SIDE];
#pragma unroll
    for (int j = 0; j < SIDE; ++j) acc[j] = 0.f;
#pragma unroll 4
    for (int c = threadIdx.x; c < width; c += 128) {
      const float x = to_float<T>(h[t * ld + c]);
#pragma unroll
      for (int j = 0; j < SIDE; ++j) acc[j] = fmaf(x, e0 + j < rows ? router[(long long)(e0 + j) * width + c] : 0.f, acc[j]);
    }
#pragma unroll
    for (int j = 0; j < SIDE; ++j) {
      const float z = warp_sum(acc[j]);
      if (lane == 0) parts[warp * SIDE + j] = z;
    }
    __syncthreads();
    if (threadIdx.x < SIDE && e0 + threadIdx.x < rows) {
      const int j = threadIdx.x;
      logits[e0 + j] = ((parts[j] + parts[SIDE + j]) + parts[2 * SIDE + j]) + parts[3 * SIDE + j] + (bias != nullptr && e0 + j < experts ? bias[e0 + j] : 0.f);
    }
    __syncthreads();
  }
  if (warp == 0) {
    if (mode.on) route_choose_scored(logits, logits + rows, logits + rows + experts, chosen, share, t, experts, top, lane, mode);
    else route_choose(logits, chosen, share, t, experts, top, lane);
  }
}

// One block.  chosen [pairs]; slot_of [pairs] out; source [max_slots] out: the pair in a slot, or -1; tile_expert [max_tiles] out:
// the expert of a row tile of tile_rows slots, or -1.  Shared memory: 2 * experts + 1 ints.
__global__ void experts_plan_kernel(const int* __restrict__ chosen, int* __restrict__ slot_of, int* __restrict__ source,
                                    int* __restrict__ tile_expert, int pairs, int experts, int max_slots, int max_tiles, int tile_rows) {
  extern __shared__ int plan[];
  grid_dependency_wait();
  allow_dependents();
  int* count = plan;                 // tokens per expert, then the next free slot of each
  int* first = plan + experts;       // first slot of each expert, [experts + 1]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  for (int s = threadIdx.x; s < max_slots; s += blockDim.x) source[s] = -1;
  for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) tile_expert[tile] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&count[chosen[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = at;
      at += (count[e] + tile_rows - 1) / tile_rows * tile_rows;
    }
    first[experts] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    for (int tile = first[e] / tile_rows; tile < first[e + 1] / tile_rows; ++tile) tile_expert[tile] = e;
    count[e] = first[e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int slot = atomicAdd(&count[chosen[i]], 1);   // the order inside an expert's span does not matter: rows do not see each other
    slot_of[i] = slot;
    source[slot] = i;
  }
}

// out[slot, n] = sum_k a[row(slot), k] * w[expert, n, k].  row(slot) = source[slot] / divide when `gathered`, else slot.
// GLU: w is [experts, 2 * n_out, k] (gate rows, then up rows) and out[slot, n] = act(gate) * up in T; else out is float32.
// Block 256 threads = 16 x 16; tile EXPERT_ROWS x 64; a thread owns 2 rows x 4 columns.
template <typename T, bool GLU>
__global__ void __launch_bounds__(256) experts_product_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ w,
                                                              const int* __restrict__ source, const int* __restrict__ tile_expert,
                                                              int gathered, int divide, void* __restrict__ out_v, int n_out, int k_size,
                                                              int kind, int interleaved, int act_out) {
  constexpr int TN = 64, TK = 16;
  __shared__ float a_tile[EXPERT_ROWS][TK + 1];
  __shared__ float b_tile[GLU ? 2 : 1][TN][TK + 1];
  __shared__ int rows[EXPERT_ROWS];
  grid_dependency_wait();
  allow_dependents();
  const int tile = blockIdx.y;
  const int expert = tile_expert[tile];
  if (expert < 0) return;
  const int n0 = blockIdx.x * TN;
  if (threadIdx.x < EXPERT_ROWS) {
    const int pair = source[tile * EXPERT_ROWS + threadIdx.x];
    rows[threadIdx.x] = pair < 0 ? -1 : (gathered ? pair / divide : tile * EXPERT_ROWS + threadIdx.x);
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const long long w_rows = GLU ? 2LL * n_out : n_out;
  const T* w_mine = w + (long long)expert * w_rows * k_size;
  float acc[GLU ? 2 : 1][2][4];
#pragma unroll
  for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;
  for (int k0 = 0; k0 < k_size; k0 += TK) {
    for (int x = threadIdx.x; x < EXPERT_ROWS * TK; x += 256) {
      const int r = x / TK, c = x % TK;
      const int row = rows[r];
      a_tile[r][c] = (row >= 0 && k0 + c < k_size) ? to_float<T>(a[(long long)row * lda + k0 + c]) : 0.f;
    }
    for (int x = threadIdx.x; x < TN * TK; x += 256) {
      const int r = x / TK, c = x % TK;
      const bool inside = n0 + r < n_out && k0 + c < k_size;
      b_tile[0][r][c] = inside ? to_float<T>(w_mine[glu_row(n0 + r, 0, n_out, GLU && interleaved) * k_size + k0 + c]) : 0.f;
      if (GLU) b_tile[1][r][c] = inside ? to_float<T>(w_mine[glu_row(n0 + r, 1, n_out, interleaved) * k_size + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < TK; ++c) {
      float av[2], bv[GLU ? 2 : 1][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) av[i] = a_tile[ty * 2 + i][c];
#pragma unroll
      for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[g][j] = b_tile[g][tx * 4 + j][c];
#pragma unroll
      for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(av[i], bv[g][j], acc[g][i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (rows[r] < 0) continue;
    const long long slot = (long long)tile * EXPERT_ROWS + r;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= n_out) continue;
      if (GLU) ((T*)out_v)[slot * n_out + n] = from_float<T>(expert_activation(acc[0][i][j], kind) * acc[GLU ? 1 : 0][i][j]);
      else if (act_out) ((T*)out_v)[slot * n_out + n] = from_float<T>(expert_activation(acc[0][i][j], kind));   // an ungated expert's first product
      else ((float*)out_v)[slot * n_out + n] = acc[0][i][j];
    }
  }
}

// The same product on tensor cores for bfloat16: a block of four warps takes a row tile of 32 slots x 64 columns (with GLU: 64 gate and
// the 64 matching up columns); warp w owns columns 16 w .. 16 w + 15 of the tile, both 16-row halves.  Steps of 64 along k through a ring
// of four shared-memory stages that cp.async fills ahead of the products (a step of few tokens is bound by the experts' matrices
// coming from memory, so several steps' loads are kept in flight); rows padded by 8 elements so that fragment loads do not collide;
// k_size is a multiple of 8, the rest of a step and the rows of empty slots are filled with zeros.
constexpr int MMA_TN = 64, MMA_TK = 64, MMA_PAD = 8;
__host__ __device__ constexpr int mma_stages(bool) { return 4; }   // (six stages for the plain product, whose stages are half as large, were faster at width 2,048 and slower at 4,096)
__host__ __device__ constexpr int mma_stage_elements(bool glu) { return (EXPERT_ROWS + (glu ? 2 : 1) * MMA_TN) * (MMA_TK + MMA_PAD); }
constexpr size_t mma_shared_bytes(bool glu) { return (size_t)mma_stages(glu) * mma_stage_elements(glu) * sizeof(__nv_bfloat16); }

__device__ __forceinline__ void copy_16_or_zeros(void* shared, const void* global, bool real) {
  const unsigned target = (unsigned)__cvta_generic_to_shared(shared);
  const int bytes = real ? 16 : 0;   // what is not copied is written as zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(target), "l"(global), "r"(bytes) : "memory");
}

template <bool GLU>
__global__ void __launch_bounds__(128) experts_product_mma_kernel(const __nv_bfloat16* __restrict__ a, long long lda,
                                                                  const __nv_bfloat16* __restrict__ w, const int* __restrict__ source,
                                                                  const int* __restrict__ tile_expert, int gathered, int divide,
                                                                  void* __restrict__ out_v, int n_out, int k_size, int kind, int interleaved, int act_out) {
  constexpr int TN = MMA_TN, TK = MMA_TK, LD = MMA_TK + MMA_PAD, G = GLU ? 2 : 1, MMA_STAGES = mma_stages(GLU);
  constexpr int A_ELEMENTS = EXPERT_ROWS * LD, STAGE_ELEMENTS = mma_stage_elements(GLU);
  extern __shared__ __align__(16) unsigned char mma_shared[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(mma_shared);
  __shared__ int rows[EXPERT_ROWS];
  grid_dependency_wait();
  allow_dependents();
  const int tile = blockIdx.y;
  const int expert = tile_expert[tile];
  if (expert < 0) return;
  const int n0 = blockIdx.x * TN;
  if (threadIdx.x < EXPERT_ROWS) {
    const int pair = source[tile * EXPERT_ROWS + threadIdx.x];
    rows[threadIdx.x] = pair < 0 ? -1 : (gathered ? pair / divide : tile * EXPERT_ROWS + threadIdx.x);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = lane >> 2, quad = lane & 3;
  const long long w_rows = GLU ? 2LL * n_out : n_out;
  const __nv_bfloat16* w_mine = w + (long long)expert * w_rows * k_size;
  float acc[G][2][2][4];   // [gate | up][row half][column eighth][fragment]
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int f = 0; f < 4; ++f) acc[g][i][j][f] = 0.f;
  const int steps = (k_size + TK - 1) / TK;
  auto fill = [&](int step) {   // every thread commits one group a call, also an empty one, so that the groups count the steps
    if (step < steps) {
      const int k0 = step * TK;
      __nv_bfloat16* a_stage = ring + (size_t)(step % MMA_STAGES) * STAGE_ELEMENTS;
      __nv_bfloat16* b_stage = a_stage + A_ELEMENTS;
      for (int x = threadIdx.x; x < EXPERT_ROWS * (TK / 8); x += 128) {
        const int r = x / (TK / 8), c = (x % (TK / 8)) * 8;
        const int row = rows[r];
        const bool real = row >= 0 && k0 + c < k_size;
        copy_16_or_zeros(a_stage + r * LD + c, real ? a + (long long)row * lda + k0 + c : a, real);
      }
      for (int x = threadIdx.x; x < G * TN * (TK / 8); x += 128) {
        const int g = x / (TN * (TK / 8)), y = x % (TN * (TK / 8));
        const int r = y / (TK / 8), c = (y % (TK / 8)) * 8;
        const bool real = n0 + r < n_out && k0 + c < k_size;
        copy_16_or_zeros(b_stage + (g * TN + r) * LD + c, real ? w_mine + glu_row(n0 + r, g, n_out, GLU && interleaved) * k_size + k0 + c : w_mine, real);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
#pragma unroll
  for (int step = 0; step < MMA_STAGES - 1; ++step) fill(step);
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(MMA_STAGES - 2) : "memory");   // this step's stage has arrived (for this thread's copies)
    __syncthreads();                                                               // ... for everyone's; and the stage of the step before is free
    fill(step + MMA_STAGES - 1);
    const __nv_bfloat16* a_stage = ring + (size_t)(step % MMA_STAGES) * STAGE_ELEMENTS;
    const __nv_bfloat16* b_stage = a_stage + A_ELEMENTS;
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      unsigned af[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        af[i][0] = *reinterpret_cast<const unsigned*>(a_stage + (16 * i + group) * LD + kk + 2 * quad);
        af[i][1] = *reinterpret_cast<const unsigned*>(a_stage + (16 * i + group + 8) * LD + kk + 2 * quad);
        af[i][2] = *reinterpret_cast<const unsigned*>(a_stage + (16 * i + group) * LD + kk + 2 * quad + 8);
        af[i][3] = *reinterpret_cast<const unsigned*>(a_stage + (16 * i + group + 8) * LD + kk + 2 * quad + 8);
      }
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = 16 * warp + 8 * j + group;
          const unsigned b0 = *reinterpret_cast<const unsigned*>(b_stage + (g * TN + n) * LD + kk + 2 * quad);
          const unsigned b1 = *reinterpret_cast<const unsigned*>(b_stage + (g * TN + n) * LD + kk + 2 * quad + 8);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                         : "+f"(acc[g][i][j][0]), "+f"(acc[g][i][j][1]), "+f"(acc[g][i][j][2]), "+f"(acc[g][i][j][3])
                         : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(b0), "r"(b1));
        }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = 16 * i + group + 8 * half;
      if (rows[r] < 0) continue;
      const long long slot = (long long)tile * EXPERT_ROWS + r;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int n = n0 + 16 * warp + 8 * j + 2 * quad + e;
          if (n >= n_out) continue;
          const float value = acc[0][i][j][2 * half + e];
          if (GLU) ((__nv_bfloat16*)out_v)[slot * n_out + n] = __float2bfloat16_rn(expert_activation(value, kind) * acc[G - 1][i][j][2 * half + e]);
          else if (act_out) ((__nv_bfloat16*)out_v)[slot * n_out + n] = __float2bfloat16_rn(expert_activation(value, kind));
          else ((float*)out_v)[slot * n_out + n] = value;
        }
    }
}

// out[t, c] = sum_k share[t, k] * y[slot_of[t * top + k], c], the choices in their order; y in float32 or in the compute dtype.
// With `common` ([T, width] in C, an expert that every token goes through) and `gate` (float32 [T]): + gate[t] * common[t, c].
template <typename Y, typename C>
__global__ void experts_gather_kernel(const Y* __restrict__ y, const int* __restrict__ slot_of, const float* __restrict__ share,
                                      float* __restrict__ out, int width, int top, long long total, const C* __restrict__ common,
                                      const float* __restrict__ gate) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const long long t = item / width;
  const int c = (int)(item % width);
  float acc = 0.f;
  for (int k = 0; k < top; ++k) acc = fmaf(share[t * top + k], to_float<Y>(y[(long long)slot_of[t * top + k] * width + c]), acc);
  if (common != nullptr) acc = fmaf(gate[t], to_float<C>(common[item]), acc);
  out[item] = acc;
}

// sorted[slot, :] = h[source[slot] / top, :], zeros in an empty slot: the tokens' rows in the order of their experts, for a product
// that takes whole row tiles from memory.  A thread moves 16 bytes; chunks = 16-byte pieces of a row.
__global__ void experts_sort_rows_kernel(const uint4* __restrict__ h, long long ld_chunks, const int* __restrict__ source, uint4* __restrict__ sorted,
                                         int chunks, int top, long long total) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const long long slot = item / chunks;
  const int c = (int)(item % chunks);
  const int pair = source[slot];
  sorted[item] = pair < 0 ? make_uint4(0, 0, 0, 0) : h[(long long)(pair / top) * ld_chunks + c];
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_experts_row_tile() { return EXPERT_ROWS; }

// scored != 0: the sigmoid form (see RouteScored); router is then float32 [experts + extra, width].
extern "C" int pylon_experts_route(const void* h, long long ld, const float* router, const float* bias, int* chosen, float* share, int width,
                                   int experts, int top, int num_tokens, int dtype, int scored, const float* correction, int groups, int keep,
                                   float share_eps, int extra, float* extra_out, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (experts < 1 || top < 1 || top > experts || experts > 2048) PYLON_REFUSE("experts_route: %d of %d experts (at most 2048)", top, experts);
  if (!scored && (correction || groups || extra)) PYLON_REFUSE("experts_route: a correction, groups and extra rows go with the sigmoid form");
  if (scored && (groups < 0 || (groups > 0 && (experts % groups || keep < 1 || keep > groups || top > keep * (experts / groups))) || extra < 0 || extra > 64 ||
                 (extra > 0 && !extra_out)))
    PYLON_REFUSE("experts_route: %d groups of which %d are kept for %d of %d experts, %d extra rows", groups, keep, top, experts, extra);
  const RouteScored mode{scored ? 1 : 0, correction, groups, keep, share_eps, extra, extra_out};
  const int per_token = experts + extra + (scored ? experts + groups : 0);
  if (num_tokens < 512) {   // a step of few tokens wants many threads a token
    const size_t smem = (size_t)(4 * 8 + per_token) * sizeof(float);
    if (dtype == PYLON_DTYPE_F32)
      launch_dependent(experts_route_block_kernel<float>, dim3((unsigned)num_tokens), dim3(128), smem, stream, (const float*)h, ld, router, bias, chosen, share, width, experts, top, mode);
    else if (dtype == PYLON_DTYPE_BF16)
      launch_dependent(experts_route_block_kernel<__nv_bfloat16>, dim3((unsigned)num_tokens), dim3(128), smem, stream, (const __nv_bfloat16*)h, ld, router, bias, chosen, share, width, experts, top, mode);
    else PYLON_REFUSE("experts_route: unknown dtype %d", dtype);
  } else {
    constexpr int warps = 4, side = 4;   // tokens a warp takes side by side (57 us for 2,048 tokens of 2,048 columns and 8 experts; two a warp took 73 us)
    const dim3 grid((unsigned)((num_tokens + warps * side - 1) / (warps * side)));
    const size_t smem = (size_t)warps * side * per_token * sizeof(float);
    if (dtype == PYLON_DTYPE_F32)
      launch_dependent(experts_route_kernel<float, side>, grid, dim3(warps * 32), smem, stream, (const float*)h, ld, router, bias, chosen, share, width, experts, top, num_tokens, mode);
    else if (dtype == PYLON_DTYPE_BF16)
      launch_dependent(experts_route_kernel<__nv_bfloat16, side>, grid, dim3(warps * 32), smem, stream, (const __nv_bfloat16*)h, ld, router, bias, chosen, share, width, experts, top, num_tokens, mode);
    else PYLON_REFUSE("experts_route: unknown dtype %d", dtype);
  }
  PYLON_CHECK_LAUNCH("experts_route");
}

// tile_rows: the slots of a row tile (pylon_experts_row_tile() for the products of this file, 128 for the grouped tcgen05 product).
extern "C" int pylon_experts_plan(const int* chosen, int* slot_of, int* source, int* tile_expert, int pairs, int experts, int max_slots,
                                  int max_tiles, int tile_rows, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (tile_rows < 1 || max_slots < pairs || (long long)max_tiles * tile_rows < max_slots)
    PYLON_REFUSE("experts_plan: %d slots in %d tiles of %d for %d pairs", max_slots, max_tiles, tile_rows, pairs);
  launch_dependent(experts_plan_kernel, dim3(1), dim3(1024), (size_t)(2 * experts + 1) * sizeof(int), stream, chosen, slot_of, source, tile_expert,
                   pairs, experts, max_slots, max_tiles, tile_rows);
  PYLON_CHECK_LAUNCH("experts_plan");
}

template <bool GLU>
static void allow_mma_shared_memory() {
  static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
  if (configured) return;
  cudaFuncSetAttribute(experts_product_mma_kernel<GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_shared_bytes(GLU));
  configured = true;
}

// a: [rows, lda] in dtype; w: [experts, (glu ? 2 : 1) * n_out, k] in dtype, contiguous (with glu an expert's gate rows, then its up rows;
// or, interleaved != 0, alternating in groups of 8); out: [max_tiles * EXPERT_ROWS, n_out], in dtype with glu, else float32.
// glu == 2: no gate, but the activation on the product itself, out in dtype (the first product of an ungated expert).
extern "C" int pylon_experts_product(const void* a, long long lda, const void* w, const int* source, const int* tile_expert, int gathered,
                                     int divide, void* out, int n_out, int k_size, int max_tiles, int glu, int kind, int interleaved, int dtype,
                                     cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  const int act_out = glu == 2 ? 1 : 0;
  if (act_out) glu = 0;
  if (n_out <= 0 || k_size <= 0 || divide < 1 || kind < 0 || kind > 3) PYLON_REFUSE("experts_product: n %d, k %d, divide %d, activation %d", n_out, k_size, divide, kind);
  if (max_tiles > 65535) PYLON_REFUSE("experts_product: %d row tiles", max_tiles);
  if (interleaved && (!glu || n_out % 8)) PYLON_REFUSE("experts_product: interleaved rows need a gated product of a multiple of 8 columns, got %d", n_out);
  const dim3 grid((unsigned)((n_out + 63) / 64), (unsigned)max_tiles);
  if (dtype == PYLON_DTYPE_F32) {
    if (glu) launch_dependent(experts_product_kernel<float, true>, grid, dim3(256), 0, stream, (const float*)a, lda, (const float*)w, source, tile_expert, gathered, divide, out, n_out, k_size, kind, interleaved, act_out);
    else launch_dependent(experts_product_kernel<float, false>, grid, dim3(256), 0, stream, (const float*)a, lda, (const float*)w, source, tile_expert, gathered, divide, out, n_out, k_size, kind, interleaved, act_out);
  } else if (dtype == PYLON_DTYPE_BF16) {
    const __nv_bfloat16* ab = (const __nv_bfloat16*)a;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    const bool vectors = k_size % 8 == 0 && lda % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0;
    if (vectors) {
      if (glu) {
        allow_mma_shared_memory<true>();
        launch_dependent(experts_product_mma_kernel<true>, grid, dim3(128), mma_shared_bytes(true), stream, ab, lda, wb, source, tile_expert, gathered, divide, out, n_out, k_size, kind, interleaved, act_out);
      } else {
        allow_mma_shared_memory<false>();
        launch_dependent(experts_product_mma_kernel<false>, grid, dim3(128), mma_shared_bytes(false), stream, ab, lda, wb, source, tile_expert, gathered, divide, out, n_out, k_size, kind, interleaved, act_out);
      }
    } else {
      if (glu) launch_dependent(experts_product_kernel<__nv_bfloat16, true>, grid, dim3(256), 0, stream, ab, lda, wb, source, tile_expert, gathered, divide, out, n_out, k_size, kind, interleaved, act_out);
      else launch_dependent(experts_product_kernel<__nv_bfloat16, false>, grid, dim3(256), 0, stream, ab, lda, wb, source, tile_expert, gathered, divide, out, n_out, k_size, kind, interleaved, act_out);
    }
  } else PYLON_REFUSE("experts_product: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("experts_product");
}

// h [T, ld] and sorted [max_slots, width] in a 16-bit or 32-bit dtype; rows of whole 16-byte pieces at 16-byte addresses.
extern "C" int pylon_experts_sort_rows(const void* h, long long ld, const int* source, void* sorted, int width, int top, int max_slots, int dtype,
                                       cudaStream_t stream) {
  if (max_slots <= 0) return 0;
  const int per_chunk = dtype == PYLON_DTYPE_F32 ? 4 : 8;
  if (top < 1 || width % per_chunk || ld % per_chunk || (uintptr_t)h % 16 || (uintptr_t)sorted % 16)
    PYLON_REFUSE("experts_sort_rows: rows of %d (stride %lld) are not whole 16-byte pieces at 16-byte addresses", width, ld);
  const int chunks = width / per_chunk;
  const long long total = (long long)max_slots * chunks;
  launch_dependent(experts_sort_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const uint4*)h, ld / per_chunk, source, (uint4*)sorted,
                   chunks, top, total);
  PYLON_CHECK_LAUNCH("experts_sort_rows");
}

// y: [slots, width] in float32 (y_dtype PYLON_DTYPE_F32) or bfloat16; out float32 [num_tokens, width].
// common ([num_tokens, width] in common_dtype) and gate (float32 [num_tokens]), both or neither: out += gate[t] * common[t].
extern "C" int pylon_experts_gather(const void* y, const int* slot_of, const float* share, float* out, int num_tokens, int width, int top, int y_dtype,
                                    const void* common, const float* gate, int common_dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if ((common == nullptr) != (gate == nullptr)) PYLON_REFUSE("experts_gather: a common expert's output and its gate go together");
  const long long total = (long long)num_tokens * width;
  const dim3 grid((unsigned)((total + 255) / 256));
  const bool common_f32 = common == nullptr || common_dtype == PYLON_DTYPE_F32;
#define PYLON_GATHER(Y, C) launch_dependent(experts_gather_kernel<Y, C>, grid, dim3(256), 0, stream, (const Y*)y, slot_of, share, out, width, top, total, (const C*)common, gate)
  if (y_dtype == PYLON_DTYPE_F32) { if (common_f32) PYLON_GATHER(float, float); else PYLON_GATHER(float, __nv_bfloat16); }
  else if (y_dtype == PYLON_DTYPE_BF16) { if (common_f32) PYLON_GATHER(__nv_bfloat16, float); else PYLON_GATHER(__nv_bfloat16, __nv_bfloat16); }
  else PYLON_REFUSE("experts_gather: unknown dtype %d", y_dtype);
#undef PYLON_GATHER
  PYLON_CHECK_LAUNCH("experts_gather");
}
