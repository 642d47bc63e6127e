// Small kernels that stand between products:
//   side_by_side     out[t] = [a[t] | b[t]] in the compute dtype, from two float32 blocks (the input of a map over both)
//   gated_unit       out = act(gate + b_gate) * (up + b_up) from a product with columns [gate | up]; act = silu, relu or
//                    the tanh form of gelu; the biases may be absent
//   add_bias         float32 rows += a bias, in place
//   mean_of_normed   out[t] = (1 / n) sum_i rmsnorm(y_i[t]) * w_i over n mixers' outputs of one token (each output either a
//                    block in the compute dtype or float32 partial sums of a product cut along k), float32 out
// All arithmetic is float32.
#include "common.cuh"

namespace pylon {

template <typename T>
__global__ void side_by_side_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int width, long long total) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const long long t = item / (2 * width);
  const int c = (int)(item % (2 * width));
  out[item] = from_float<T>(c < width ? a[t * width + c] : b[t * width + (c - width)]);
}

__device__ __forceinline__ float unit_activation(float x, int kind) {
  if (kind == 0) return x / (1.f + expf(-x));                                       // silu
  if (kind == 1) return fmaxf(x, 0.f);                                              // relu
  if (kind == 3) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));           // gelu, exact (erf) form
  return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));   // gelu, tanh form
}

// The same for bfloat16 in whole 16-byte pieces: a thread takes eight neighbouring elements.
__global__ void activation_vec_kernel(uint4* __restrict__ x, long long pieces, int kind) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= pieces) return;
  uint4 eight = x[item];
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&eight);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(pairs[i]);
    pairs[i] = __floats2bfloat162_rn(unit_activation(v.x, kind), unit_activation(v.y, kind));
  }
  x[item] = eight;
}

// In place: x <- act(x), element by element.
template <typename T>
__global__ void activation_kernel(T* __restrict__ x, long long total, int kind) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item < total) x[item] = from_float<T>(unit_activation(to_float<T>(x[item]), kind));
}

template <typename T>
__global__ void gated_unit_kernel(const T* __restrict__ gate_up, long long ld, const float* __restrict__ bias, T* __restrict__ out,
                                  int inner, long long total, int kind) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= total) return;
  const long long t = item / inner;
  const int c = (int)(item % inner);
  float g = to_float<T>(gate_up[t * ld + c]), u = to_float<T>(gate_up[t * ld + inner + c]);
  if (bias != nullptr) { g += bias[c]; u += bias[inner + c]; }
  out[item] = from_float<T>(unit_activation(g, kind) * u);
}

// The same for bfloat16 rows of whole 16-byte pieces: a thread takes eight neighbouring columns.
__global__ void gated_unit_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, long long ld, const float* __restrict__ bias,
                                      __nv_bfloat16* __restrict__ out, int inner, long long total, int kind) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (item >= total) return;
  const long long t = item / inner;
  const int c = (int)(item % inner);
  const uint4 g8 = *reinterpret_cast<const uint4*>(gate_up + t * ld + c), u8 = *reinterpret_cast<const uint4*>(gate_up + t * ld + inner + c);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g8);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u8);
  uint4 packed;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
    if (bias != nullptr) {
      g.x += bias[c + 2 * i]; g.y += bias[c + 2 * i + 1];
      u.x += bias[inner + c + 2 * i]; u.y += bias[inner + c + 2 * i + 1];
    }
    o2[i] = __floats2bfloat162_rn(unit_activation(g.x, kind) * u.x, unit_activation(g.y, kind) * u.y);
  }
  *reinterpret_cast<uint4*>(out + item) = packed;
}

__global__ void add_bias_kernel(float* __restrict__ rows, const float* __restrict__ bias, int width, long long total) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item < total) rows[item] += bias[item % width];
}

struct NormedInput {
  const void* data;     // [parts, T, width]
  const float* weight;  // [width]
  int parts;            // 1 for a plain block
  int is_float;         // partial sums are float32; a plain block has the compute dtype
};
constexpr int MEAN_OF_NORMED_MAX = 4;
struct NormedInputs { NormedInput of[MEAN_OF_NORMED_MAX]; };

// A block per token.  Per input: the row is added up over its parts, its sum of squares reduced over the block, and the
// normed row joins the mean.  HELD: a thread keeps its (at most MEAN_HELD) columns of every input in registers between the
// sum of squares and the result, so a row is read once; otherwise it is read twice.
constexpr int MEAN_HELD = 8;
template <typename T, bool HELD>
__global__ void mean_of_normed_kernel(NormedInputs inputs, int count, float* __restrict__ out, int width, long long tokens, float eps) {
  __shared__ float scratch[33];
  grid_dependency_wait();
  allow_dependents();
  const long long t = blockIdx.x;
  float inv[MEAN_OF_NORMED_MAX];
  auto value = [&](const NormedInput& in, int c) {
    float v = 0.f;
    if (in.is_float) {
      const float* p = (const float*)in.data + t * width + c;
      for (int part = 0; part < in.parts; ++part) v += p[(long long)part * tokens * width];
    } else {
      v = to_float<T>(((const T*)in.data)[t * width + c]);
    }
    return v;
  };
  const float share = 1.f / (float)count;
  if (HELD) {
    float held[MEAN_OF_NORMED_MAX][MEAN_HELD];
#pragma unroll
    for (int i = 0; i < MEAN_OF_NORMED_MAX; ++i) {
      if (i >= count) break;
      float sumsq = 0.f;
#pragma unroll
      for (int k = 0; k < MEAN_HELD; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        held[i][k] = c < width ? value(inputs.of[i], c) : 0.f;
        sumsq = fmaf(held[i][k], held[i][k], sumsq);
      }
      inv[i] = rsqrtf(block_sum(sumsq, scratch) / (float)width + eps);
    }
#pragma unroll
    for (int k = 0; k < MEAN_HELD; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      if (c >= width) break;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < MEAN_OF_NORMED_MAX; ++i)
        if (i < count) acc += held[i][k] * inv[i] * inputs.of[i].weight[c];
      out[t * width + c] = acc * share;
    }
  } else {
    for (int i = 0; i < count; ++i) {
      float sumsq = 0.f;
      for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = value(inputs.of[i], c);
        sumsq = fmaf(v, v, sumsq);
      }
      inv[i] = rsqrtf(block_sum(sumsq, scratch) / (float)width + eps);
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float acc = 0.f;
      for (int i = 0; i < count; ++i) acc += value(inputs.of[i], c) * inv[i] * inputs.of[i].weight[c];
      out[t * width + c] = acc * share;
    }
  }
}

// The same for rows of whole 16-byte pieces that a block holds in registers: a thread takes two groups of four neighbouring columns
// of every input (16-byte loads of float32 partial sums, 8-byte loads of bfloat16 rows), and the inputs' sums of squares are reduced
// over the block together, behind one pair of barriers.  Shared memory: MEAN_OF_NORMED_MAX * 33 floats (static).
template <typename T>
__global__ void mean_of_normed_vec_kernel(NormedInputs inputs, int count, float* __restrict__ out, int width, long long tokens, float eps) {
  __shared__ float scratch[MEAN_OF_NORMED_MAX][33];
  grid_dependency_wait();
  allow_dependents();
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  auto value4 = [&](const NormedInput& in, int c) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (in.is_float) {
      const float* p = (const float*)in.data + t * width + c;
      for (int part = 0; part < in.parts; ++part) {
        const float4 x = *reinterpret_cast<const float4*>(p + (long long)part * tokens * width);
        v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
      }
    } else {
      T x[4];
      *reinterpret_cast<uint2*>(x) = *reinterpret_cast<const uint2*>((const T*)in.data + t * width + c);   // only taken for 16-bit T
      v = make_float4(to_float<T>(x[0]), to_float<T>(x[1]), to_float<T>(x[2]), to_float<T>(x[3]));
    }
    return v;
  };
  float4 held[MEAN_OF_NORMED_MAX][2];
  float sumsq[MEAN_OF_NORMED_MAX];
#pragma unroll
  for (int i = 0; i < MEAN_OF_NORMED_MAX; ++i) {
    sumsq[i] = 0.f;
    if (i < count) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int c = 4 * (threadIdx.x + k * blockDim.x);
        held[i][k] = c < width ? value4(inputs.of[i], c) : make_float4(0.f, 0.f, 0.f, 0.f);
        sumsq[i] = fmaf(held[i][k].x, held[i][k].x, sumsq[i]);
        sumsq[i] = fmaf(held[i][k].y, held[i][k].y, sumsq[i]);
        sumsq[i] = fmaf(held[i][k].z, held[i][k].z, sumsq[i]);
        sumsq[i] = fmaf(held[i][k].w, held[i][k].w, sumsq[i]);
      }
      sumsq[i] = warp_sum(sumsq[i]);
      if (lane == 0) scratch[i][warp] = sumsq[i];
    }
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < MEAN_OF_NORMED_MAX; ++i)
      if (i < count) {
        const float w = warp_sum(lane < warps ? scratch[i][lane] : 0.f);
        if (lane == 0) scratch[i][32] = w;
      }
  }
  __syncthreads();
  const float share = 1.f / (float)count;
  float inv[MEAN_OF_NORMED_MAX];
#pragma unroll
  for (int i = 0; i < MEAN_OF_NORMED_MAX; ++i) inv[i] = i < count ? rsqrtf(scratch[i][32] / (float)width + eps) : 0.f;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int c = 4 * (threadIdx.x + k * blockDim.x);
    if (c >= width) break;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < MEAN_OF_NORMED_MAX; ++i)
      if (i < count) {
        const float4 w = *reinterpret_cast<const float4*>(inputs.of[i].weight + c);
        acc.x += held[i][k].x * inv[i] * w.x; acc.y += held[i][k].y * inv[i] * w.y;
        acc.z += held[i][k].z * inv[i] * w.z; acc.w += held[i][k].w * inv[i] * w.w;
      }
    *reinterpret_cast<float4*>(out + t * width + c) = make_float4(acc.x * share, acc.y * share, acc.z * share, acc.w * share);
  }
}

// out[t, c] = sum_i scale_i * y_i[t, c] over up to four inputs, each a block in the compute dtype or float32 partial sums.
template <typename T>
__global__ void weighted_sum_kernel(NormedInputs inputs, float4 scales, int count, float* __restrict__ out, long long per_part) {
  grid_dependency_wait();
  allow_dependents();
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= per_part) return;
  const float scale[4] = {scales.x, scales.y, scales.z, scales.w};
  float acc = 0.f;
  for (int i = 0; i < count; ++i) {
    const NormedInput& in = inputs.of[i];
    float v = 0.f;
    if (in.is_float) {
      for (int part = 0; part < in.parts; ++part) v += ((const float*)in.data)[(long long)part * per_part + item];
    } else {
      v = to_float<T>(((const T*)in.data)[item]);
    }
    acc = fmaf(scale[i], v, acc);
  }
  out[item] = acc;
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_side_by_side(const float* a, const float* b, void* out, int tokens, int width, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0) PYLON_REFUSE("side_by_side: width %d", width);
  const long long total = (long long)tokens * 2 * width;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == PYLON_DTYPE_F32) launch_dependent(side_by_side_kernel<float>, grid, dim3(256), 0, stream, a, b, (float*)out, width, total);
  else if (dtype == PYLON_DTYPE_BF16) launch_dependent(side_by_side_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, a, b, (__nv_bfloat16*)out, width, total);
  else PYLON_REFUSE("side_by_side: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("side_by_side");
}

extern "C" int pylon_gated_unit(const void* gate_up, long long ld, const float* bias, void* out, int tokens, int inner, int kind, int dtype,
                                cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (inner <= 0 || kind < 0 || kind > 3) PYLON_REFUSE("gated_unit: inner width %d, activation %d", inner, kind);
  const long long total = (long long)tokens * inner;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == PYLON_DTYPE_F32) launch_dependent(gated_unit_kernel<float>, grid, dim3(256), 0, stream, (const float*)gate_up, ld, bias, (float*)out, inner, total, kind);
  else if (dtype == PYLON_DTYPE_BF16 && inner % 8 == 0 && ld % 8 == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)out % 16 == 0)
    launch_dependent(gated_unit_vec_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, ld, bias, (__nv_bfloat16*)out, inner,
                     total, kind);
  else if (dtype == PYLON_DTYPE_BF16)
    launch_dependent(gated_unit_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, ld, bias, (__nv_bfloat16*)out, inner, total, kind);
  else PYLON_REFUSE("gated_unit: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("gated_unit");
}

extern "C" int pylon_add_bias(float* rows, const float* bias, long long count, int width, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (width <= 0) PYLON_REFUSE("add_bias: width %d", width);
  const long long total = count * width;
  launch_dependent(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, rows, bias, width, total);
  PYLON_CHECK_LAUNCH("add_bias");
}

// data[i]: [parts[i], tokens, width] - float32 where is_float[i], else in dtype (parts 1); weights[i]: float32 [width]; out float32 [tokens, width].
extern "C" int pylon_mean_of_normed(const void* const* data, const float* const* weights, const int* parts, const int* is_float, int count,
                                    float* out, int tokens, int width, float eps, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (count < 1 || count > MEAN_OF_NORMED_MAX || width <= 0) PYLON_REFUSE("mean_of_normed: %d inputs (1 to %d), width %d", count, MEAN_OF_NORMED_MAX, width);
  NormedInputs inputs;
  for (int i = 0; i < count; ++i) inputs.of[i] = NormedInput{data[i], weights[i], parts[i], is_float[i]};
  // as many threads as leave each at most MEAN_HELD columns (by the width alone, so that a token's sums do not depend on the step)
  int threads = 128;
  while (threads < 1024 && threads * MEAN_HELD < width) threads *= 2;
  const bool held = threads * MEAN_HELD >= width;
  bool pieces = held && dtype == PYLON_DTYPE_BF16 && width % 4 == 0 && (uintptr_t)out % 16 == 0;   // rows of whole 16-byte pieces, blocks of a 16-bit dtype
  for (int i = 0; i < count && pieces; ++i) pieces = (uintptr_t)data[i] % 16 == 0 && (uintptr_t)weights[i] % 16 == 0;
  if (pieces) {
    launch_dependent(mean_of_normed_vec_kernel<__nv_bfloat16>, dim3((unsigned)tokens), dim3(threads), 0, stream, inputs, count, out, width, (long long)tokens, eps);
    PYLON_CHECK_LAUNCH("mean_of_normed");
  }
#define PYLON_MEAN(T, HELD) launch_dependent(mean_of_normed_kernel<T, HELD>, dim3((unsigned)tokens), dim3(threads), 0, stream, inputs, count, out, width, (long long)tokens, eps)
  if (dtype == PYLON_DTYPE_F32) { if (held) PYLON_MEAN(float, true); else PYLON_MEAN(float, false); }
  else if (dtype == PYLON_DTYPE_BF16) { if (held) PYLON_MEAN(__nv_bfloat16, true); else PYLON_MEAN(__nv_bfloat16, false); }
  else PYLON_REFUSE("mean_of_normed: unknown dtype %d", dtype);
#undef PYLON_MEAN
  PYLON_CHECK_LAUNCH("mean_of_normed");
}

// outputs[i]: [parts_i, T, width] float32 partial sums (is_float_i) or [T, width] in dtype; out float32 [T, width] = sum_i scales[i] * outputs[i].
extern "C" int pylon_weighted_sum(const void* const* outputs, const int* parts, const int* is_float, const float* scales, int count, float* out,
                                  long long total, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (count < 1 || count > MEAN_OF_NORMED_MAX) PYLON_REFUSE("weighted_sum: %d inputs (1 to %d)", count, MEAN_OF_NORMED_MAX);
  NormedInputs inputs;
  float factor[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < count; ++i) {
    inputs.of[i].data = outputs[i];
    inputs.of[i].weight = nullptr;
    inputs.of[i].parts = parts[i];
    inputs.of[i].is_float = is_float[i];
    factor[i] = scales[i];
  }
  const float4 packed = make_float4(factor[0], factor[1], factor[2], factor[3]);
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == PYLON_DTYPE_F32) launch_dependent(weighted_sum_kernel<float>, grid, dim3(256), 0, stream, inputs, packed, count, out, total);
  else if (dtype == PYLON_DTYPE_BF16) launch_dependent(weighted_sum_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, inputs, packed, count, out, total);
  else PYLON_REFUSE("weighted_sum: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("weighted_sum");
}

// x: [total] in dtype, in place.
extern "C" int pylon_activation(void* x, long long total, int kind, int dtype, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (kind < 0 || kind > 3) PYLON_REFUSE("activation: kind %d", kind);
  const dim3 grid((unsigned)((total + 255) / 256));
  if (dtype == PYLON_DTYPE_F32) launch_dependent(activation_kernel<float>, grid, dim3(256), 0, stream, (float*)x, total, kind);
  else if (dtype == PYLON_DTYPE_BF16 && total % 8 == 0 && (uintptr_t)x % 16 == 0)
    launch_dependent(activation_vec_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, stream, (uint4*)x, total / 8, kind);
  else if (dtype == PYLON_DTYPE_BF16) launch_dependent(activation_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)x, total, kind);
  else PYLON_REFUSE("activation: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("activation");
}
