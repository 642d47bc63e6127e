// Paged causal attention on the tensor cores (bfloat16, mma.sync m16n8k16 with float32 sums) for scores and masks that the other
// tensor-core kernels do not take: a window that keeps the first keys of the sequence, a bias by distance, a sink, values of
// another width than the keys.
//
// A token at position p of its request sees the keys j <= p with p - j < window (window 0: all of them) or j < keep_first.  Its
// score for key j is (q . k_j) * scale + bias[min(p - j, bias_rows - 1), h] (bias null: none); with sinks the softmax's
// denominator of head h also holds exp(sinks[h]), a key without a value.  Query head h reads KV head h / (nq / nkv).
//
// A block takes 16 neighbouring tokens of one request and one KV head; its warps are the query heads of that KV head (at most 8),
// so a tile of 32 keys and their values is fetched from the pages once for the whole group, by cp.async into one of two stages while
// the tile before is worked on (where the tile's keys lie in the pages is looked up a tile further ahead); rows padded so that the
// first product's 32-bit fragment loads and the second's ldmatrix (transposing: the values lie row by row as they came) meet no bank
// twice.  Tiles: the kept first keys, then from the first key the block's first token sees to its last token; what a token does not
// see inside a tile is masked.
// Softmax online in float32.  The weights enter the second product as two bfloat16 numbers each, the rounded weight and what
// the rounding dropped, so that they count with 16 bits of their 24: the sum of weights and the weighted sum agree to float32's
// own rounding of the products.  Built per (key size, value size); both are multiples of 16 and 8 up to 256.
//
// A step of few tokens (decoding) has few blocks, each with a whole window of keys to walk: the key tiles of a block are then dealt
// out to `splits` blocks in turn, each leaves its normalised part, its maximum and its sum in scratch, and a second kernel adds the
// parts up with their weights (the sink is met by the first split alone).
#include "common.cuh"

#ifndef PYLON_HEAD_DIM
#define PYLON_HEAD_DIM 64
#endif
#ifndef PYLON_VALUE_DIM
#define PYLON_VALUE_DIM PYLON_HEAD_DIM
#endif

namespace pylon {

constexpr int D = PYLON_HEAD_DIM, DV = PYLON_VALUE_DIM;
static_assert(D % 16 == 0 && D <= 256 && DV % 8 == 0 && DV <= 256, "key rows of a multiple of 16 and value rows of a multiple of 8, up to 256");
constexpr int WINDOW_TOKENS = 16;   // tokens of a block
constexpr int WINDOW_KEYS = 32;     // keys of a tile
constexpr int WINDOW_MAX_GROUP = 8; // query heads per KV head: the warps of a block
constexpr int K_LD = D + 8;         // 16-bit elements between the rows of the key tile: 32-bit fragment loads fall into 32 banks
constexpr int V_LD = DV + 8;         // likewise between the rows of the value tile: the eight 16-byte rows of an ldmatrix fall into different banks

struct WindowParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const __nv_bfloat16* k_pages;
  const __nv_bfloat16* v_pages;
  __nv_bfloat16* out;
  const int* q_start;
  const int* kv_len;
  const int* block_table;
  int table_width, page_size, num_pages, nq, nkv, window, keep_first, bias_rows;
  float scale;
  const float* bias;
  const float* sinks;
  int* error;
  int splits, total_tokens;
  float* scratch;   // splits > 1: parts [splits, tokens, nq, DV] float32, then (maximum, sum) [splits, tokens, nq, 2]
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_bf16(float low, float high) {
  const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
  return *reinterpret_cast<const unsigned*>(&pair);
}

__device__ __forceinline__ void window_copy_or_zeros(void* shared, const void* global, bool real) {
  const unsigned target = (unsigned)__cvta_generic_to_shared(shared);
  const int bytes = real ? 16 : 0;   // what is not copied is written as zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(target), "l"(global), "r"(bytes) : "memory");
}

__global__ void __launch_bounds__(WINDOW_MAX_GROUP * 32) window_attention_kernel(WindowParams p) {
  extern __shared__ __align__(16) unsigned char window_stages[];   // two stages of [keys K_LD | values V_LD] rows
  __shared__ long long key_row[2][WINDOW_KEYS];   // the cache row (page, KV head, slot) of every key of a tile, -1: none
  constexpr int STAGE_ELEMENTS = WINDOW_KEYS * (K_LD + V_LD);
  grid_dependency_wait();
  allow_dependents();
  const int row = blockIdx.z, kv_head = blockIdx.y;
  const int first = p.q_start[row], count = p.q_start[row + 1] - first;
  const int split = blockIdx.x % p.splits;
  const int t0 = blockIdx.x / p.splits * WINDOW_TOKENS;
  if (t0 >= count) return;   // the row has fewer tokens than the longest (or none: a padded step)
  const int valid_tokens = count - t0 < WINDOW_TOKENS ? count - t0 : WINDOW_TOKENS;
  const int p0 = p.kv_len[row] - count + t0, p_last = p0 + valid_tokens - 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, quad = lane & 3;
  const int group = p.nq / p.nkv;
  const int head = kv_head * group + warp;
  const int* table = p.block_table + (size_t)row * p.table_width;
  const float* bias_of_head = p.bias ? p.bias + head : nullptr;

  // the queries of the warp's head: 16 tokens x D as A fragments (rows group_id and group_id + 8), zeros for tokens the row does not have
  unsigned qa[D / 16][4];
  {
    const __nv_bfloat16* q_low = p.q + (size_t)(first + t0 + group_id) * p.q_stride + (size_t)head * D;
    const __nv_bfloat16* q_high = q_low + 8 * p.q_stride;
    const bool low = group_id < valid_tokens, high = group_id + 8 < valid_tokens;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = low ? *reinterpret_cast<const unsigned*>(q_low + 16 * ks + 2 * quad) : 0u;
      qa[ks][1] = high ? *reinterpret_cast<const unsigned*>(q_high + 16 * ks + 2 * quad) : 0u;
      qa[ks][2] = low ? *reinterpret_cast<const unsigned*>(q_low + 16 * ks + 2 * quad + 8) : 0u;
      qa[ks][3] = high ? *reinterpret_cast<const unsigned*>(q_high + 16 * ks + 2 * quad + 8) : 0u;
    }
  }
  float o[DV / 8][4];
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
  // a sink is a key of score sinks[h] and value zero, met before all others (its one in the sum is held by one lane of the four)
  float top[2], sum[2];
  top[0] = top[1] = (p.sinks && split == 0) ? p.sinks[head] : -INFINITY;
  sum[0] = sum[1] = (p.sinks && split == 0 && quad == 0) ? 1.f : 0.f;

  const int lo_first = p.window > 0 ? (p0 - p.window + 1 > 0 ? p0 - p.window + 1 : 0) : 0;   // the first key of the window of the block's first token
  const int kept = p.keep_first < lo_first ? p.keep_first : lo_first;                        // the keys before it that stay visible: [0, kept)
  const int kept_end = (kept + WINDOW_KEYS - 1) / WINDOW_KEYS * WINDOW_KEYS;
  // the block's tiles in order: every `splits`-th tile of the kept keys' tiles and then the window's; beyond p_last: none left
  auto after = [&](int tile_start) {
    for (int turn = 0; turn < p.splits && tile_start <= p_last; ++turn) {
      tile_start += WINDOW_KEYS;
      if (tile_start == kept_end && kept > 0) {   // behind the kept keys' tiles: on to the window's first tile, if that lies further on
        const int window_start = lo_first / WINDOW_KEYS * WINDOW_KEYS;
        if (window_start > tile_start) tile_start = window_start;
      }
    }
    return tile_start;
  };
  auto look_up = [&](int stage, int tile_start) {   // where every key of the tile lies: looked up once, a tile ahead of its copies
    if (threadIdx.x < WINDOW_KEYS) {
      const int j = tile_start + threadIdx.x;
      long long where = -1;
      if (j <= p_last && (j >= lo_first || j < kept)) {
        const int page = table[j / p.page_size];
        if (page >= 0 && page < p.num_pages) where = ((long long)page * p.nkv + kv_head) * p.page_size + j % p.page_size;
        else if (p.error) atomicExch(p.error, PYLON_ERROR_BAD_PAGE);   // a key that is seen has a page
      }
      key_row[stage][threadIdx.x] = where;
    }
  };
  auto issue = [&](int stage, int tile_start) {   // the tile's keys and values on their way into the stage (an empty group behind the last tile)
    if (tile_start <= p_last) {
      __nv_bfloat16* k_tile = reinterpret_cast<__nv_bfloat16*>(window_stages) + (size_t)stage * STAGE_ELEMENTS;
      __nv_bfloat16* v_tile = k_tile + WINDOW_KEYS * K_LD;
      for (int x = threadIdx.x; x < WINDOW_KEYS * (D / 8); x += blockDim.x) {
        const int key = x / (D / 8), piece = x % (D / 8);
        const long long where = key_row[stage][key];
        window_copy_or_zeros(k_tile + key * K_LD + piece * 8, where >= 0 ? p.k_pages + where * D + piece * 8 : p.k_pages, where >= 0);
      }
      for (int x = threadIdx.x; x < WINDOW_KEYS * (DV / 8); x += blockDim.x) {
        const int key = x / (DV / 8), piece = x % (DV / 8);
        const long long where = key_row[stage][key];
        window_copy_or_zeros(v_tile + key * V_LD + piece * 8, where >= 0 ? p.v_pages + where * DV + piece * 8 : p.v_pages, where >= 0);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  int tile_start = kept > 0 ? 0 : lo_first / WINDOW_KEYS * WINDOW_KEYS;
  for (int turn = 0; turn < split && tile_start <= p_last; ++turn) {   // this split's first tile
    tile_start += WINDOW_KEYS;
    if (tile_start == kept_end && kept > 0) {
      const int window_start = lo_first / WINDOW_KEYS * WINDOW_KEYS;
      if (window_start > tile_start) tile_start = window_start;
    }
  }
  int next_start = after(tile_start);
  look_up(0, tile_start);
  look_up(1, next_start);
  __syncthreads();
  issue(0, tile_start);
  for (int stage = 0; tile_start <= p_last; stage ^= 1) {
    issue(stage ^ 1, next_start);                       // the next tile's copies run while this tile is worked on
    const int third_start = after(next_start);
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");   // this tile has arrived (for this thread's copies)
    __syncthreads();                                          // ... for everyone's; and this stage's look-ups are used up
    look_up(stage, third_start);                              // read when the tile after the next is issued, two barriers on
    const __nv_bfloat16* k_tile = reinterpret_cast<const __nv_bfloat16*>(window_stages) + (size_t)stage * STAGE_ELEMENTS;
    const __nv_bfloat16* v_tile = k_tile + WINDOW_KEYS * K_LD;
    {
      float s[WINDOW_KEYS / 8][4];
#pragma unroll
      for (int nt = 0; nt < WINDOW_KEYS / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const __nv_bfloat16* from = k_tile + (8 * nt + group_id) * K_LD + 16 * ks + 2 * quad;
          mma_bf16(s[nt], qa[ks], *reinterpret_cast<const unsigned*>(from), *reinterpret_cast<const unsigned*>(from + 8));
        }
      }
      float tile_top[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < WINDOW_KEYS / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int token = group_id + 8 * r, pos = p0 + token, j = tile_start + 8 * nt + 2 * quad + (e & 1);
          const bool seen = token < valid_tokens && j <= pos && (p.window == 0 || pos - j < p.window || j < p.keep_first);
          float score = -INFINITY;
          if (seen) {
            score = s[nt][e] * p.scale;
            if (p.bias) score += bias_of_head[(pos - j < p.bias_rows ? pos - j : p.bias_rows - 1) * p.nq];
          }
          s[nt][e] = score;
          tile_top[r] = fmaxf(tile_top[r], score);
        }
      float rescale[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_top[r] = fmaxf(tile_top[r], __shfl_xor_sync(0xffffffffu, tile_top[r], 1));
        tile_top[r] = fmaxf(tile_top[r], __shfl_xor_sync(0xffffffffu, tile_top[r], 2));
        const float new_top = fmaxf(top[r], tile_top[r]);
        rescale[r] = (top[r] == -INFINITY || new_top == -INFINITY) ? (new_top == -INFINITY ? 1.f : 0.f) : __expf(top[r] - new_top);
        top[r] = new_top;
        sum[r] *= rescale[r];
      }
      unsigned weights[WINDOW_KEYS / 16][4], dropped[WINDOW_KEYS / 16][4];
#pragma unroll
      for (int nt = 0; nt < WINDOW_KEYS / 8; ++nt) {
        float w[4], rest[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          w[e] = s[nt][e] == -INFINITY ? 0.f : __expf(s[nt][e] - top[r]);   // the hardware's exponential: a relative 2^-21, below what the weights carry on
          sum[r] += w[e];
          rest[e] = w[e] - __bfloat162float(__float2bfloat16_rn(w[e]));
        }
        weights[nt >> 1][(nt & 1) * 2] = pack_bf16(w[0], w[1]);
        weights[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(w[2], w[3]);
        dropped[nt >> 1][(nt & 1) * 2] = pack_bf16(rest[0], rest[1]);
        dropped[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(rest[2], rest[3]);
      }
      // the values lie row by row as they came; ldmatrix with .trans hands each lane its two keys of one column: rows 16 ks + (lane % 16)
      const unsigned v_from = (unsigned)__cvta_generic_to_shared(v_tile + (lane & 15) * V_LD);
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt) {
        o[nt][0] *= rescale[0]; o[nt][1] *= rescale[0];
        o[nt][2] *= rescale[1]; o[nt][3] *= rescale[1];
#pragma unroll
        for (int ks = 0; ks < WINDOW_KEYS / 16; ++ks) {
          unsigned b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];\n"
                       : "=r"(b0), "=r"(b1)
                       : "r"(v_from + (unsigned)((16 * ks * V_LD + 8 * nt) * sizeof(__nv_bfloat16))));
          mma_bf16(o[nt], weights[ks], b0, b1);
          mma_bf16(o[nt], dropped[ks], b0, b1);
        }
      }
    }
    __syncthreads();   // the stage is free for the tile after the next
    tile_start = next_start;
    next_start = third_start;
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
    const int token = group_id + 8 * r;
    if (token >= valid_tokens) continue;
    const float inv = sum[r] > 0.f ? 1.f / sum[r] : 0.f;
    if (p.splits == 1) {
      __nv_bfloat16* to = p.out + ((size_t)(first + t0 + token) * p.nq + head) * DV + 2 * quad;
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt)
        *reinterpret_cast<__nv_bfloat162*>(to + 8 * nt) = __floats2bfloat162_rn(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
    } else {
      const size_t index = ((size_t)split * p.total_tokens + first + t0 + token) * p.nq + head;
      float* to = p.scratch + index * DV + 2 * quad;
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt) *reinterpret_cast<float2*>(to + 8 * nt) = make_float2(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
      if (quad == 0) {
        float* stats = p.scratch + (size_t)p.splits * p.total_tokens * p.nq * DV + index * 2;
        stats[0] = top[r];
        stats[1] = sum[r];
      }
    }
  }
}

// out[token, head] = sum_s w_s part_s / sum_s w_s with w_s = sum_s * exp(top_s - max top): one warp per (token, head).
__global__ void window_attention_combine_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out, const int* __restrict__ token_row,
                                                int splits, int total_tokens, int nq) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)total_tokens * nq) return;
  if (token_row[item / nq] < 0) return;   // a padding token: no block wrote parts for it
  const size_t rows = (size_t)total_tokens * nq;
  const float* stats = scratch + (size_t)splits * rows * DV;
  float top = -INFINITY;
  for (int s = 0; s < splits; ++s)
    if (stats[((size_t)s * rows + item) * 2 + 1] > 0.f) top = fmaxf(top, stats[((size_t)s * rows + item) * 2]);
  float total = 0.f;
  float acc[(DV + 31) / 32];
#pragma unroll
  for (int k = 0; k < (DV + 31) / 32; ++k) acc[k] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* st = stats + ((size_t)s * rows + item) * 2;
    if (!(st[1] > 0.f)) continue;
    const float w = st[1] * expf(st[0] - top);
    total += w;
    const float* part = scratch + ((size_t)s * rows + item) * DV;
#pragma unroll
    for (int k = 0; k < (DV + 31) / 32; ++k)
      if (lane + 32 * k < DV) acc[k] = fmaf(w, part[lane + 32 * k], acc[k]);
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
  for (int k = 0; k < (DV + 31) / 32; ++k)
    if (lane + 32 * k < DV) out[item * DV + lane + 32 * k] = __float2bfloat16_rn(acc[k] * inv);
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_window_attention_max_group() { return WINDOW_MAX_GROUP; }

// Floats of scratch for `splits` > 1 (0 for one split).
extern "C" long long pylon_window_attention_scratch_floats(int splits, int total_tokens, int nq) {
  return splits > 1 ? (long long)splits * total_tokens * nq * (DV + 2) : 0;
}

// q [T, >= nq * D] bfloat16 with a row stride; pages [P, nkv, page_size, D] and [P, nkv, page_size, DV]; out [T, nq * DV]; q_start int32
// [rows + 1]; kv_len int32 [rows]; block_table int32 [rows, table_width]; bias float32 [bias_rows, nq] or null; sinks float32 [nq] or null.
// max_q: the most tokens a row brings (an upper bound is fine).  splits > 1: the key tiles of every block dealt out to so many blocks, with
// scratch of pylon_window_attention_scratch_floats floats and token_row int32 [total_tokens] (-1: a padding token).
extern "C" int pylon_window_attention(const void* q, long long q_stride, const void* k_pages, const void* v_pages, void* out, const int* q_start,
                                      const int* kv_len, const int* block_table, int table_width, int page_size, int num_pages, int nq, int nkv,
                                      int window, int keep_first, float scale, const float* bias, int bias_rows, const float* sinks, int num_rows,
                                      int max_q, int splits, float* scratch, const int* token_row, int total_tokens, int* error, cudaStream_t stream) {
  if (num_rows <= 0 || max_q <= 0) return 0;
  if (nkv < 1 || nq < 1 || nq % nkv || nq / nkv > WINDOW_MAX_GROUP) PYLON_REFUSE("window_attention: %d query heads over %d KV heads (at most %d each)", nq, nkv, WINDOW_MAX_GROUP);
  if (page_size < 1 || table_width < 1 || window < 0 || keep_first < 0 || (bias && bias_rows < 1) || num_rows > 65535 || nkv > 65535)
    PYLON_REFUSE("window_attention: page size %d, table width %d, window %d, %d kept, %d bias rows, %d rows", page_size, table_width, window, keep_first, bias_rows, num_rows);
  if (splits < 1 || splits > 64 || (splits > 1 && (!scratch || !token_row || total_tokens < 1))) PYLON_REFUSE("window_attention: %d splits", splits);
  if (q_stride % 2 || (uintptr_t)q % 4 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)out % 4)
    PYLON_REFUSE("window_attention: rows must start at even elements, pages at 16-byte addresses");
  WindowParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
  p.out = (__nv_bfloat16*)out; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table; p.table_width = table_width;
  p.page_size = page_size; p.num_pages = num_pages; p.nq = nq; p.nkv = nkv; p.window = window; p.keep_first = keep_first; p.bias_rows = bias_rows;
  p.scale = scale; p.bias = bias; p.sinks = sinks; p.error = error; p.splits = splits; p.total_tokens = total_tokens; p.scratch = scratch;
  const int group = nq / nkv;
  const dim3 grid((unsigned)((max_q + WINDOW_TOKENS - 1) / WINDOW_TOKENS * splits), (unsigned)nkv, (unsigned)num_rows);
  const size_t stages = 2 * (size_t)WINDOW_KEYS * (K_LD + V_LD) * sizeof(__nv_bfloat16);
  if (stages > 48 * 1024) {
    static bool raised[MAX_DEVICES] = {};   // function attributes belong to a device
    if (!raised[current_device_slot()]) {
      cudaFuncSetAttribute(window_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stages);
      raised[current_device_slot()] = true;
    }
  }
  launch_dependent(window_attention_kernel, grid, dim3(group * 32), stages, stream, p);
  if (splits > 1) {
    const long long items = (long long)total_tokens * nq;
    launch_dependent(window_attention_combine_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const float*)scratch, (__nv_bfloat16*)out,
                     token_row, splits, total_tokens, nq);
  }
  PYLON_CHECK_LAUNCH("window_attention");
}
