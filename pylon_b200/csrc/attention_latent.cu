// Paged causal attention over one shared row per token, on the tensor cores (bfloat16, mma.sync m16n8k16).
//
// Every query head reads the same cache row of D numbers per token (nkv = 1); the keys are the whole rows, the values their
// first DV columns.  That is the attention of a mixer that caches a latent per token and applies its per-head key and
// value matrices on the query's side and behind the attention.  Because the heads share their keys, the heads of a token
// are packed beside tokens into the M dimension of the products: a block takes 64 packed rows (token-major, then head) of
// one request - for a decoded token its H heads, for a prompt portion 64 / H tokens - and walks the keys those rows can
// see in tiles of 32, each tile loaded once for all of them (cp.async, two buffers).
//
// Eight warps, 4 along the rows x 2: the two warps of a row pair each compute the scores of the pair's 16 rows against half
// of the tile's 32 keys, hand each other the rows' maxima and their halves of the softmax weights (float32, online, base 2;
// through shared memory, behind a barrier of the pair's own), and each adds P V for its half of the value columns, V read
// from the key tile itself through transposed ldmatrix.  The output accumulator, 16 x DV / 2 per warp, stays in registers.
//
// Options: a window (a token at position p sees keys j with p - window < j <= p), sinks (one float32 per head: the
// softmax's denominator also holds exp(sink), unscaled), and a split of the keys over `splits` blocks per tile for steps
// with few packed rows (decoded tokens): every block leaves its normalised part, its maximum and its sum in scratch, and
// a second kernel combines them.  D and DV are compile-time sizes (D a multiple of 16 up to 832, DV a multiple of 32 up to 512).
#include "common.cuh"

#ifndef PYLON_LATENT_DIM
#define PYLON_LATENT_DIM 576
#endif
// PYLON_LATENT_SPLIT_WEIGHTS 1: a softmax weight enters the second product as two bfloat16 numbers, the rounded weight and what the
// rounding dropped (twice the products over the values), so that it counts with 16 of its 24 bits: for designs that ask for the
// attention's weights in 32-bit.
#ifndef PYLON_LATENT_SPLIT_WEIGHTS
#define PYLON_LATENT_SPLIT_WEIGHTS 0
#endif
#ifndef PYLON_LATENT_VALUE_DIM
#define PYLON_LATENT_VALUE_DIM 512
#endif

namespace pylon {

constexpr int LD = PYLON_LATENT_DIM, LDV = PYLON_LATENT_VALUE_DIM;
constexpr int LAT_BM = 64, LAT_BN = 32, LAT_THREADS = 256;
constexpr int LAT_PITCH = LD + 8;                 // elements between rows in shared memory: 16 bytes of padding, ldmatrix without bank conflicts
constexpr int LAT_NV = LDV / 2;                   // value columns of a warp
constexpr int LAT_NV_TILES = LAT_NV / 8;
constexpr int LAT_CHUNKS = LD / 8;                // 16-byte chunks of a row
static_assert(LD % 16 == 0 && LDV % 32 == 0 && LDV <= LD && LDV <= 512 && LD <= 832, "latent attention: rows a multiple of 16 up to 832, values a multiple of 32 up to 512");

__device__ __forceinline__ void cp_async_16(void* smem, const void* global, bool valid) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(address), "l"(global), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&pair);
}

// scratch, when the keys are split: parts [splits, packed rows, LDV] float32, then (maximum, sum) [splits, packed rows, 2];
// packed row of (token t of the step, head h) = t * nq + h.
__global__ void __launch_bounds__(LAT_THREADS, 1) latent_attention_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ pages, __nv_bfloat16* __restrict__ out,
    float* __restrict__ scratch, const int* __restrict__ q_start, const int* __restrict__ kv_len, const int* __restrict__ block_table,
    int table_width, int page_size, int num_pages, int nq, int window, float scale_log2, const float* __restrict__ sinks, int splits,
    int total_tokens) {
  extern __shared__ __align__(16) unsigned char latent_shared[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(latent_shared);       // [64][PITCH]
  __nv_bfloat16* ks = qs + LAT_BM * LAT_PITCH;                                // [2][32][PITCH]
  const int row = blockIdx.y, tile = blockIdx.x, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
  const int t0 = q_start[row], tokens = q_start[row + 1] - t0;
  const int packed = tokens * nq;
  if (tile * LAT_BM >= packed) return;   // also a row without tokens
  const int first_pos = kv_len[row] - tokens;
  const int* table = block_table + (size_t)row * table_width;

  // the keys the tile's rows can see, in tiles of 32 aligned at position 0
  const int tok_a = (tile * LAT_BM) / nq;
  int tok_b = (tile * LAT_BM + LAT_BM - 1) / nq;
  if (tok_b > tokens - 1) tok_b = tokens - 1;
  int key_lo = window > 0 ? first_pos + tok_a - window + 1 : 0;
  if (key_lo < 0) key_lo = 0;
  const int key_hi = first_pos + tok_b;
  const int tile_first = key_lo / LAT_BN, tile_last = key_hi / LAT_BN;
  const int all_tiles = tile_last - tile_first + 1;
  const int per_split = (all_tiles + splits - 1) / splits;
  const int my_first = tile_first + split * per_split;
  int my_last = my_first + per_split - 1;
  if (my_last > tile_last) my_last = tile_last;

  // the tile's queries
  for (int c = tid; c < LAT_BM * LAT_CHUNKS; c += LAT_THREADS) {
    const int m = c / LAT_CHUNKS, part = c % LAT_CHUNKS;
    const int p = tile * LAT_BM + m;
    const bool valid = p < packed;
    const int tok = valid ? p / nq : 0, h = valid ? p % nq : 0;
    cp_async_16(qs + m * LAT_PITCH + part * 8, q + (size_t)(t0 + tok) * q_stride + (size_t)h * LD + part * 8, valid);
  }
  // where a tile's 32 keys lie in the pool (element offsets, -1: no such key), looked up once per key by the first threads
  // a tile ahead of its copy, so that the copy itself is address arithmetic only
  __shared__ long long key_base[2][LAT_BN];
  // what the two warps of a row pair hand each other: their rows' maxima (and, at the end, sums), and their halves of a tile's weights
  __shared__ float pair_row[4][2][16];
  __shared__ __align__(16) __nv_bfloat16 pair_weights[4][16][LAT_BN + 8];
#if PYLON_LATENT_SPLIT_WEIGHTS
  __shared__ __align__(16) __nv_bfloat16 pair_dropped[4][16][LAT_BN + 8];   // what rounding the weights to bfloat16 dropped
#endif
  auto pair_barrier = [](int pair) { asm volatile("bar.sync %0, 64;\n" ::"r"(pair + 1) : "memory"); };
  auto find_keys = [&](int key_tile, int which, int n) {
    const int j = key_tile * LAT_BN + n;
    int page = -1;
    if (j <= key_hi && j / page_size < table_width) page = table[j / page_size];
    key_base[which][n] = page >= 0 && page < num_pages ? ((long long)page * page_size + j % page_size) * LD : -1;
  };
  auto load_keys = [&](int key_tile, int buffer) {
    __nv_bfloat16* dst = ks + (size_t)buffer * LAT_BN * LAT_PITCH;
    const long long* base = key_base[key_tile & 1];
    for (int c = tid; c < LAT_BN * LAT_CHUNKS; c += LAT_THREADS) {
      const int n = c / LAT_CHUNKS, part = c % LAT_CHUNKS;
      const long long from = base[n];
      cp_async_16(dst + n * LAT_PITCH + part * 8, pages + (from >= 0 ? from : 0) + part * 8, from >= 0);
    }
  };
  if (tid < 2 * LAT_BN) find_keys(my_first + tid / LAT_BN, (my_first + tid / LAT_BN) & 1, tid % LAT_BN);
  __syncthreads();
  if (my_first <= my_last) load_keys(my_first, 0);
  cp_async_commit();

  // the two rows of the warp's 16 that this thread holds scores of
  const int r_lo = wm * 16 + (lane >> 2), r_hi = r_lo + 8;
  int pos[2], head[2];
  bool live[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int p = tile * LAT_BM + (i ? r_hi : r_lo);
    live[i] = p < packed;
    pos[i] = live[i] ? first_pos + p / nq : -1;
    head[i] = live[i] ? p % nq : 0;
  }
  float top[2], sum[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool sink = sinks != nullptr && split == 0 && live[i];   // the sink counts once: in the first part
    top[i] = sink ? sinks[head[i]] * 1.4426950408889634f : -INFINITY;
    sum[i] = sink && wn == 0 ? 1.f : 0.f;   // a row's sum is kept in two halves, one per warp of the pair; the sink's one is in the first
  }
  float o[LAT_NV_TILES][4];
#pragma unroll
  for (int n = 0; n < LAT_NV_TILES; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int key_tile = my_first; key_tile <= my_last; ++key_tile) {
    const int buffer = (key_tile - my_first) & 1;
    cp_async_wait<0>();
    __syncthreads();   // the tile is here; every warp is done with the tile before, whose buffer the next copy fills
    if (key_tile < my_last) load_keys(key_tile + 1, buffer ^ 1);
    cp_async_commit();
    if (tid < LAT_BN && key_tile + 2 <= my_last) find_keys(key_tile + 2, key_tile & 1, tid);   // read by the copy that the next round issues, behind its barrier
    const __nv_bfloat16* kt = ks + (size_t)buffer * LAT_BN * LAT_PITCH;
    // a warp whose 16 rows lie behind the tile's last packed row (a decoded token of 16 heads fills one warp pair of four) only
    // helps with the copies and keeps the barriers
    if (tile * LAT_BM + wm * 16 >= packed) continue;

    // scores of the warp's 16 rows against its half of the tile's 32 keys (the other warp of the pair does the other half); the
    // fragments of step k + 1 are asked for before the products of step k are issued (the compiler keeps the order as written)
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    {
      const __nv_bfloat16* a_from = qs + (wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LAT_PITCH + (lane >> 4) * 8;
      const __nv_bfloat16* b_from = kt + (wn * 16 + (lane & 7) + (lane >> 4) * 8) * LAT_PITCH + ((lane >> 3) & 1) * 8;
      unsigned a[2][4], b[2][4];
      ldmatrix_x4(a[0], a_from);
      ldmatrix_x4(b[0], b_from);
#pragma unroll
      for (int k = 0; k < LD / 16; ++k) {
        const int now = k & 1, next = now ^ 1;
        if (k + 1 < LD / 16) {
          ldmatrix_x4(a[next], a_from + (k + 1) * 16);
          ldmatrix_x4(b[next], b_from + (k + 1) * 16);
        }
        mma_bf16(s[0], a[now], b[now][0], b[now][1]);
        mma_bf16(s[1], a[now], b[now][2], b[now][3]);
      }
    }
    // scale and mask; the rows' maxima over the warp's keys go to the pair's other warp and its come here
    float tile_top[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = key_tile * LAT_BN + wn * 16 + n * 8 + (lane & 3) * 2 + (e & 1);
        const bool seen = live[i] && j <= pos[i] && (window <= 0 || j > pos[i] - window);
        s[n][e] = seen ? s[n][e] * scale_log2 : -INFINITY;
        tile_top[i] = fmaxf(tile_top[i], s[n][e]);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tile_top[i] = fmaxf(tile_top[i], __shfl_xor_sync(0xffffffffu, tile_top[i], 1));
      tile_top[i] = fmaxf(tile_top[i], __shfl_xor_sync(0xffffffffu, tile_top[i], 2));
      if ((lane & 3) == 0) pair_row[wm][wn][(lane >> 2) + 8 * i] = tile_top[i];
    }
    pair_barrier(wm);
    float rescale[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tile_top[i] = fmaxf(tile_top[i], pair_row[wm][wn ^ 1][(lane >> 2) + 8 * i]);
      const float new_top = fmaxf(top[i], tile_top[i]);
      rescale[i] = new_top == -INFINITY ? 1.f : exp2f(top[i] - new_top);   // top -inf: nothing was added yet, 0 * anything
      top[i] = new_top;
    }
    // softmax weights of the warp's keys (float32, base 2): into the pair's tile of weights as bfloat16; the sums stay apart, each warp
    // adding up its own keys, until the end
    float tile_sum[2] = {0.f, 0.f};
    const float use_top[2] = {top[0] == -INFINITY ? 0.f : top[0], top[1] == -INFINITY ? 0.f : top[1]};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0 = exp2f(s[n][0] - use_top[0]), p1 = exp2f(s[n][1] - use_top[0]);
      const float p2 = exp2f(s[n][2] - use_top[1]), p3 = exp2f(s[n][3] - use_top[1]);
      tile_sum[0] += p0 + p1;
      tile_sum[1] += p2 + p3;
      const int column = wn * 16 + n * 8 + (lane & 3) * 2;
      *reinterpret_cast<unsigned*>(&pair_weights[wm][lane >> 2][column]) = pack_bf16(p0, p1);
      *reinterpret_cast<unsigned*>(&pair_weights[wm][(lane >> 2) + 8][column]) = pack_bf16(p2, p3);
#if PYLON_LATENT_SPLIT_WEIGHTS
      *reinterpret_cast<unsigned*>(&pair_dropped[wm][lane >> 2][column]) =
          pack_bf16(p0 - __bfloat162float(__float2bfloat16_rn(p0)), p1 - __bfloat162float(__float2bfloat16_rn(p1)));
      *reinterpret_cast<unsigned*>(&pair_dropped[wm][(lane >> 2) + 8][column]) =
          pack_bf16(p2 - __bfloat162float(__float2bfloat16_rn(p2)), p3 - __bfloat162float(__float2bfloat16_rn(p3)));
#endif
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tile_sum[i] += __shfl_xor_sync(0xffffffffu, tile_sum[i], 1);
      tile_sum[i] += __shfl_xor_sync(0xffffffffu, tile_sum[i], 2);
      sum[i] = sum[i] * rescale[i] + tile_sum[i];
    }
#pragma unroll
    for (int n = 0; n < LAT_NV_TILES; ++n) {
      o[n][0] *= rescale[0];
      o[n][1] *= rescale[0];
      o[n][2] *= rescale[1];
      o[n][3] *= rescale[1];
    }
    pair_barrier(wm);   // both halves of the weights are there; the maxima are read (they are written again only behind this barrier)
    // O += P V for the warp's half of the value columns, the next pair of value fragments asked for ahead of the products
    {
      const __nv_bfloat16* v_from = kt + ((lane & 7) + ((lane >> 3) & 1) * 8) * LAT_PITCH + wn * LAT_NV + (lane >> 4) * 8;
      const __nv_bfloat16* p_from = &pair_weights[wm][(lane & 7) + ((lane >> 3) & 1) * 8][(lane >> 4) * 8];
      unsigned b[2][4];
      ldmatrix_x4_trans(b[0], v_from);
#pragma unroll
      for (int step = 0; step < 2; ++step) {
        unsigned a[4];
        ldmatrix_x4(a, p_from + step * 16);
#if PYLON_LATENT_SPLIT_WEIGHTS
        unsigned rest[4];
        ldmatrix_x4(rest, &pair_dropped[wm][(lane & 7) + ((lane >> 3) & 1) * 8][(lane >> 4) * 8] + step * 16);
#endif
#pragma unroll
        for (int n = 0; n < LAT_NV_TILES; n += 2) {
          const int now = (step * (LAT_NV_TILES / 2) + (n >> 1)) & 1, next = now ^ 1;   // the fragments' buffers take turns across both steps
          if (n + 2 < LAT_NV_TILES)
            ldmatrix_x4_trans(b[next], v_from + step * 16 * LAT_PITCH + (n + 2) * 8);
          else if (step == 0)
            ldmatrix_x4_trans(b[next], v_from + 16 * LAT_PITCH);
          mma_bf16(o[n], a, b[now][0], b[now][1]);
          mma_bf16(o[n + 1], a, b[now][2], b[now][3]);
#if PYLON_LATENT_SPLIT_WEIGHTS
          mma_bf16(o[n], rest, b[now][0], b[now][1]);
          mma_bf16(o[n + 1], rest, b[now][2], b[now][3]);
#endif
        }
      }
    }
    // the weights are written again only behind the next tile's first pair barrier, which the other warp reaches with these reads done
  }
  // a row's sum is the sum of the pair's two halves
  if (tile * LAT_BM + wm * 16 < packed) {
    pair_barrier(wm);
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if ((lane & 3) == 0) pair_row[wm][wn][(lane >> 2) + 8 * i] = sum[i];
    pair_barrier(wm);
#pragma unroll
    for (int i = 0; i < 2; ++i) sum[i] += pair_row[wm][wn ^ 1][(lane >> 2) + 8 * i];
  }
  cp_async_wait<0>();

  // results: straight to the output, or this part to scratch
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!live[i]) continue;
    const int p = tile * LAT_BM + (i ? r_hi : r_lo);
    const int token = t0 + p / nq;
    if (splits == 1) {
      const float inv = sum[i] > 0.f ? 1.f / sum[i] : 0.f;
      __nv_bfloat16* dst = out + ((size_t)token * nq + head[i]) * LDV + wn * LAT_NV + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < LAT_NV_TILES; ++n)
        *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    } else {
      const size_t packed_rows = (size_t)total_tokens * nq;
      const size_t index = (size_t)split * packed_rows + (size_t)token * nq + head[i];
      const float inv = sum[i] > 0.f ? 1.f / sum[i] : 0.f;
      float* dst = scratch + index * LDV + wn * LAT_NV + (lane & 3) * 2;
#pragma unroll
      for (int n = 0; n < LAT_NV_TILES; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
      if (wn == 0 && (lane & 3) == 0) {
        float* stats = scratch + (size_t)splits * packed_rows * LDV + index * 2;
        stats[0] = top[i];
        stats[1] = sum[i];
      }
    }
  }
}

// out[row] = sum_s w_s part_s[row] / sum_s w_s with w_s = sum_s * 2^(top_s - max top): one block per packed row.
__global__ void __launch_bounds__(128) latent_attention_combine_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out,
                                                                      const int* __restrict__ token_row, int nq, int splits, int total_tokens) {
  __shared__ float weight[65536 / 1024];   // at most 64 splits
  __shared__ float total_shared;
  const int packed_row = blockIdx.x;
  if (token_row[packed_row / nq] < 0) return;   // a padding token: no block wrote parts for it
  const size_t packed_rows = (size_t)total_tokens * nq;
  const float* stats = scratch + (size_t)splits * packed_rows * LDV;
  if (threadIdx.x < 32) {   // the parts' weights once, by the first warp
    float top = -INFINITY, sum = 0.f;
    for (int s = threadIdx.x; s < splits; s += 32) top = fmaxf(top, stats[((size_t)s * packed_rows + packed_row) * 2]);
    top = warp_max(top);
    for (int s = threadIdx.x; s < splits; s += 32) {
      const float* st = stats + ((size_t)s * packed_rows + packed_row) * 2;
      const float w = st[1] > 0.f ? st[1] * exp2f(st[0] - top) : 0.f;
      weight[s] = w;
      sum += w;
    }
    sum = warp_sum(sum);
    if (threadIdx.x == 0) total_shared = sum;
  }
  __syncthreads();
  const float inv = total_shared > 0.f ? 1.f / total_shared : 0.f;
  // a thread's (up to four) elements of all parts: the loads of several parts are in flight together
  constexpr int PER_THREAD = (LDV + 127) / 128;
  float acc[PER_THREAD];
#pragma unroll
  for (int k = 0; k < PER_THREAD; ++k) acc[k] = 0.f;
#pragma unroll 4
  for (int s = 0; s < splits; ++s) {
    const float* part = scratch + ((size_t)s * packed_rows + packed_row) * LDV;
#pragma unroll
    for (int k = 0; k < PER_THREAD; ++k) {
      const int e = threadIdx.x + k * 128;
      if (e < LDV) acc[k] = fmaf(weight[s], part[e], acc[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < PER_THREAD; ++k) {
    const int e = threadIdx.x + k * 128;
    if (e < LDV) out[(size_t)packed_row * LDV + e] = __float2bfloat16_rn(acc[k] * inv);
  }
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_latent_attention_dims(int* d, int* dv) {
  *d = LD;
  *dv = LDV;
  return 0;
}

// float32 numbers of scratch a call with `splits` > 1 needs.
extern "C" long long pylon_latent_attention_scratch_floats(int splits, int total_tokens, int nq) {
  return splits > 1 ? (long long)splits * total_tokens * nq * (LDV + 2) : 0;
}

extern "C" int pylon_latent_attention(const void* q, long long q_stride, const void* pages, void* out, float* scratch, const int* q_start,
                                      const int* kv_len, const int* token_row, const int* block_table, int table_width, int page_size, int num_pages,
                                      int nq, int window, float scale, const float* sinks, int rows, int total_tokens, int max_q, int splits,
                                      cudaStream_t stream) {
  if (rows <= 0 || total_tokens <= 0 || max_q <= 0) return 0;
  if (nq < 1 || page_size < 1 || table_width < 1 || window < 0 || splits < 1 || splits > 64 || rows > 65535)
    PYLON_REFUSE("latent_attention: %d heads, page size %d, table width %d, window %d, %d splits, %d rows", nq, page_size, table_width, window, splits, rows);
  if (q_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)pages & 15)) PYLON_REFUSE("latent_attention: queries and pages must lie on 16-byte boundaries");
  if (splits > 1 && !scratch) PYLON_REFUSE("latent_attention: %d splits need scratch", splits);
  const size_t smem = (size_t)(LAT_BM + 2 * LAT_BN) * LAT_PITCH * sizeof(__nv_bfloat16);
  static bool configured[MAX_DEVICES] = {};
  bool& done = configured[current_device_slot()];
  if (!done) {
    if (cudaFuncSetAttribute(latent_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      PYLON_REFUSE("latent_attention: %zu bytes of shared memory are not to be had", smem);
    done = true;
  }
  const long long tiles = ((long long)max_q * nq + LAT_BM - 1) / LAT_BM;
  if (tiles > 0x7fffffffLL) PYLON_REFUSE("latent_attention: too many tiles");
  dim3 grid((unsigned)tiles, rows, splits);
  latent_attention_kernel<<<grid, LAT_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, (__nv_bfloat16*)out, scratch, q_start, kv_len, block_table, table_width, page_size,
      num_pages, nq, window, scale * 1.4426950408889634f, sinks, splits, total_tokens);
  if (splits > 1)
    latent_attention_combine_kernel<<<(unsigned)((long long)total_tokens * nq), 128, 0, stream>>>(scratch, (__nv_bfloat16*)out, token_row, nq, splits, total_tokens);
  PYLON_CHECK_LAUNCH("latent_attention");
}
