// The residual stream kept as several copies ("hyper-connections"), and the norms that read it.
//
// A model may carry S >= 1 streams x_1 .. x_S per token, float32 [T, S, W].  A sublayer reads one
// combination of them, u = sum_s read[s] * x_s, through a norm, and its output y goes back into all
// of them at once, computed from the old ones:
//
//     x_t <- sum_s mix[s, t] * x_s + scale * out[t] * y            (mix is indexed [from, to])
//
// The plain residual sum is the case S = 1 with mix = out = read = 1, optionally with a factor on
// the sublayer's output.  One kernel does the pending update of the sublayer before and the read
// and norm of the sublayer after, so the streams are read and written once per sublayer:
//
//     update (optional)  ->  u = sum_s read[s] x_s  ->  norm(u) * weight  ->  out
//
// Norm kinds: 0 = layer norm without bias, (u - mean) / sqrt(var + eps) * w with var the mean of
// the squared deviations (two passes over the row, which lies in shared memory); 1 = RMS norm,
// u / sqrt(mean(u^2) + eps) * w; 2 = dynamic tanh, tanh(alpha u) * w + b with alpha one learnt number and b a
// vector (no statistics of the row, no eps).  Everything is float32 but the sublayer's output as it comes in
// and the normalised row as it goes out.  With a row selection the streams are not written: the
// selected rows are normalised from the updated values computed on the fly (final norm at the
// rows whose logits are wanted).
#include "common.cuh"

namespace pylon {

constexpr int MAX_STREAMS = 8;

template <typename TD, int V>
__device__ __forceinline__ void load_delta(const TD* src, float (&dst)[V]) {
  if constexpr (V == 4 && sizeof(TD) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
  } else if constexpr (V == 4) {
    const float4 raw = *reinterpret_cast<const float4*>(src);
    dst[0] = raw.x; dst[1] = raw.y; dst[2] = raw.z; dst[3] = raw.w;
  } else {
    dst[0] = to_float<TD>(src[0]);
  }
}

// V: columns a thread handles at once (4: 16-byte accesses, for widths that are multiples of 4 and aligned rows; else 1).
template <typename TD, typename TO, int V>
__global__ void streams_update_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int delta_parts, long long part_stride,
                                           float scale, const float* __restrict__ mix, const float* __restrict__ outw,
                                           const float* __restrict__ read, const float* __restrict__ weight, const int* __restrict__ rows,
                                           TO* __restrict__ out, int streams, int width, float eps, int kind,
                                           const float* __restrict__ bias, const float* __restrict__ alpha) {
  extern __shared__ __align__(16) float shared[];
  float* u_row = shared;                 // [width]
  float* scratch = u_row + width;        // [34]
  float* coef = scratch + 34;            // mix [S * S], out [S], read [S]
  const int S = streams;
  // the routes are weights of the model: they are read while the kernel ahead is still running
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) coef[i] = mix ? mix[i] : (i / S == i % S ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    coef[S * S + i] = (outw ? outw[i] : 1.f) * scale;
    coef[S * S + S + i] = read ? read[i] : 1.f;
  }
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  __syncthreads();
  const float* c_mix = coef;
  const float* c_out = coef + S * S;
  const float* c_read = c_out + S;
  const int n = blockIdx.x;
  const long long t = rows ? rows[n] : n;
  float* xt = x + t * (long long)S * width;
  const bool update = delta != nullptr || mix != nullptr;
  float local_sum = 0.f;
  for (int e = threadIdx.x * V; e < width; e += blockDim.x * V) {
    float old[MAX_STREAMS][V];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) {
      if (s < S) {
        if constexpr (V == 4) {
          const float4 raw = *reinterpret_cast<const float4*>(xt + (long long)s * width + e);
          old[s][0] = raw.x; old[s][1] = raw.y; old[s][2] = raw.z; old[s][3] = raw.w;
        } else {
          old[s][0] = xt[(long long)s * width + e];
        }
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) old[s][v] = 0.f;
      }
    }
    float y[V];
#pragma unroll
    for (int v = 0; v < V; ++v) y[v] = 0.f;
    if (delta) {
      for (int part = 0; part < delta_parts; ++part) {
        float piece[V];
        load_delta<TD, V>(delta + part * part_stride + t * width + e, piece);
#pragma unroll
        for (int v = 0; v < V; ++v) y[v] += piece[v];
      }
    }
    float u[V];
#pragma unroll
    for (int v = 0; v < V; ++v) u[v] = 0.f;
#pragma unroll
    for (int to = 0; to < MAX_STREAMS; ++to) {
      if (to < S) {
        float value[V];
#pragma unroll
        for (int v = 0; v < V; ++v) value[v] = old[to][v];
        if (update) {
#pragma unroll
          for (int v = 0; v < V; ++v) value[v] = 0.f;
#pragma unroll
          for (int from = 0; from < MAX_STREAMS; ++from)
            if (from < S) {
#pragma unroll
              for (int v = 0; v < V; ++v) value[v] = fmaf(c_mix[from * S + to], old[from][v], value[v]);
            }
#pragma unroll
          for (int v = 0; v < V; ++v) value[v] = fmaf(c_out[to], y[v], value[v]);
          if (!rows) {
            if constexpr (V == 4) *reinterpret_cast<float4*>(xt + (long long)to * width + e) = make_float4(value[0], value[1], value[2], value[3]);
            else xt[(long long)to * width + e] = value[0];
          }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) u[v] = fmaf(c_read[to], value[v], u[v]);
      }
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      u_row[e + v] = u[v];
      local_sum += u[v];
    }
  }
  if (!out) return;
  float mean = 0.f, inv = 1.f;
  if (kind == 0) mean = block_sum(local_sum, scratch) / (float)width;
  if (kind != 2) {
    float local_sq = 0.f;
    for (int e = threadIdx.x * V; e < width; e += blockDim.x * V) {   // each thread reads back what it wrote itself
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const float c = u_row[e + v] - mean;
        local_sq = fmaf(c, c, local_sq);
      }
    }
    inv = rsqrtf(block_sum(local_sq, scratch) / (float)width + eps);
  }
  const float slope = kind == 2 ? alpha[0] : 0.f;
  TO* orow = out + (long long)n * width;
  for (int e = threadIdx.x * V; e < width; e += blockDim.x * V) {
    float result[V];
#pragma unroll
    for (int v = 0; v < V; ++v)
      result[v] = kind == 2 ? fmaf(tanhf(slope * u_row[e + v]), weight[e + v], bias[e + v]) : (u_row[e + v] - mean) * inv * weight[e + v];
    if constexpr (V == 4 && sizeof(TO) == 2) {
      const __nv_bfloat162 a = __floats2bfloat162_rn(result[0], result[1]), b = __floats2bfloat162_rn(result[2], result[3]);
      uint2 packed;
      packed.x = *reinterpret_cast<const unsigned*>(&a);
      packed.y = *reinterpret_cast<const unsigned*>(&b);
      *reinterpret_cast<uint2*>(orow + e) = packed;
    } else if constexpr (V == 4) {
      *reinterpret_cast<float4*>(orow + e) = make_float4(result[0], result[1], result[2], result[3]);
    } else {
      orow[e] = from_float<TO>(result[0]);
    }
  }
}

}  // namespace pylon

using namespace pylon;

// x: float32 [tokens, streams, width], updated in place unless `rows` selects.  delta: the sublayer's output [tokens, width] in
// delta_dtype, or float32 partial sums [delta_parts, tokens, width] whose sum it is, or null (nothing pending).  mix [S, S], outw [S],
// read [S]: float32 on the device, null = identity / ones / ones.  weight null: only the update (out is not written).
// out: [n_rows, width] in out_dtype.  n_rows: the selected rows, or all tokens.
extern "C" int pylon_streams_update_norm(float* x, const void* delta, int delta_parts, int delta_dtype, float scale, const float* mix,
                                         const float* outw, const float* read, const float* weight, const int* rows, void* out,
                                         int out_dtype, int n_rows, int tokens, int streams, int width, float eps, int kind,
                                         const float* bias, const float* alpha, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (streams < 1 || streams > MAX_STREAMS) PYLON_REFUSE("streams_update_norm: %d streams (1 to %d)", streams, MAX_STREAMS);
  if (width < 1 || width > 32768) PYLON_REFUSE("streams_update_norm: width %d", width);
  if (kind < 0 || kind > 2) PYLON_REFUSE("streams_update_norm: norm kind %d", kind);
  if (kind == 2 && out && (!bias || !alpha)) PYLON_REFUSE("streams_update_norm: a dynamic tanh needs its bias and its alpha");
  if ((weight == nullptr) != (out == nullptr)) PYLON_REFUSE("streams_update_norm: a norm weight and an output go together");
  if (!out && rows) PYLON_REFUSE("streams_update_norm: a row selection without an output does nothing");
  if (delta && delta_parts < 1) PYLON_REFUSE("streams_update_norm: %d parts", delta_parts);
  if (delta && delta_parts > 1 && delta_dtype != PYLON_DTYPE_F32) PYLON_REFUSE("streams_update_norm: partial sums are float32");
  int threads = width >= 8192 ? 512 : (width >= 1024 ? 256 : 128);
  // A step of few tokens is a few blocks: each gets as many threads as its row has 16-byte units (up to 512), so that a row is one
  // round or two of loads, not eight one behind the other (7.4 us a call at 8 tokens and width 2,048 with 256 threads).  Only where the result is
  // bfloat16: the order of the row's sums follows the threads, and in float32 mode it must not depend on how many tokens a step has.
  if (out_dtype == PYLON_DTYPE_BF16 && n_rows <= 256 && width % 4 == 0) {
    const int wanted = ((width / 4 + 31) / 32) * 32;
    if (wanted > threads) threads = wanted < 512 ? wanted : 512;   // 512 threads of up to 96 registers fit a block's register file
  }
  const size_t smem = (size_t)(width + 34 + streams * streams + 2 * streams) * sizeof(float);
  const long long part_stride = (long long)tokens * width;
  const bool vector = width % 4 == 0 && ((uintptr_t)x % 16 == 0) && (!delta || (uintptr_t)delta % 16 == 0) && (!out || (uintptr_t)out % 16 == 0);
#define PYLON_STREAMS_LAUNCH_V(TD, TO, V)                                                                                        \
  do {                                                                                                                           \
    static bool raised[MAX_DEVICES] = {};                                                                                        \
    if (smem > 48 * 1024 && !raised[current_device_slot()]) {                                                                    \
      cudaFuncSetAttribute(streams_update_norm_kernel<TD, TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);      \
      raised[current_device_slot()] = true;                                                                                      \
    }                                                                                                                            \
    launch_dependent(streams_update_norm_kernel<TD, TO, V>, dim3(n_rows), dim3(threads), smem, stream, x, (const TD*)delta,      \
                     delta_parts, part_stride, scale, mix, outw, read, weight, rows, (TO*)out, streams, width, eps, kind, bias,  \
                     alpha);                                                                                                     \
  } while (0)
#define PYLON_STREAMS_LAUNCH(TD, TO)                                                      \
  do {                                                                                    \
    if (vector) PYLON_STREAMS_LAUNCH_V(TD, TO, 4); else PYLON_STREAMS_LAUNCH_V(TD, TO, 1); \
  } while (0)
  const bool delta_f32 = !delta || delta_dtype == PYLON_DTYPE_F32;
  if (!delta_f32 && delta_dtype != PYLON_DTYPE_BF16) PYLON_REFUSE("streams_update_norm: unknown delta dtype %d", delta_dtype);
  if (out_dtype == PYLON_DTYPE_F32) {
    if (delta_f32) PYLON_STREAMS_LAUNCH(float, float); else PYLON_STREAMS_LAUNCH(__nv_bfloat16, float);
  } else if (out_dtype == PYLON_DTYPE_BF16) {
    if (delta_f32) PYLON_STREAMS_LAUNCH(float, __nv_bfloat16); else PYLON_STREAMS_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else {
    PYLON_REFUSE("streams_update_norm: unknown output dtype %d", out_dtype);
  }
#undef PYLON_STREAMS_LAUNCH
#undef PYLON_STREAMS_LAUNCH_V
  PYLON_CHECK_LAUNCH("streams_update_norm");
}
