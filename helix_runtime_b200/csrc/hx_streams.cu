// Residual streams (hyper-connections), the sums around them, and the biased activation of a
// plain feed-forward.
//
// A model with S residual streams keeps, per token, S rows of the model's width next to each
// other: X[token][s][c], float32.  A sublayer reads a weighted sum of them,
//
//     u[c] = sum_s a[s] X[s][c],        h = u / sqrt(mean(u^2) + eps) * w[c],
//
// and, once it has produced y (float32, the sublayer's output before any sum), all streams
// are rewritten at once from the old ones:
//
//     X'[r][c] = sum_s M[s][r] X[s][c] + b[r] * scale[c] * y[c].
//
// S = 1 with a = M = b = 1 is the ordinary residual sum with a per-channel layer scale.  All
// of it is float32; only h is rounded to the compute type.
#include "hx_common.cuh"

namespace {

constexpr int MAX_STREAMS = 16;

// ------------------------------------------------------------------ spread the embedding

__global__ void streams_spread_kernel(const float* __restrict__ x, float* __restrict__ streams,
                                      int hidden, int count, size_t total) {
  hx_pdl_prologue();
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t token = i / hidden;
  const int c = static_cast<int>(i - token * hidden);
  const float v = x[i];
  float* row = streams + token * static_cast<size_t>(count) * hidden + c;
  for (int s = 0; s < count; ++s) row[static_cast<size_t>(s) * hidden] = v;
}

// ------------------------------------------------------------- weighted read, RMS norm

// One block per output row.  `rows` gathers (the final norm runs on the wanted rows only);
// `clear`, when given, is the float32 row [hidden] that the sublayer will sum its output into:
// it is zeroed here, or set to `initial` [hidden] (a bias the sublayer's output starts from);
// row index = the token, not the gathered one.  COUNT > 0: the number of
// streams is known to the compiler; VECTORS > 0: the width is a multiple of four and a thread
// keeps up to VECTORS float4 of the weighted sum, so the streams are read once.
template <typename TOut, int COUNT, int VECTORS>
__global__ __launch_bounds__(256) void streams_read_norm_kernel(
    const float* __restrict__ streams, const float* __restrict__ read, int count_arg,
    const float* __restrict__ weight, TOut* __restrict__ out, float* __restrict__ clear,
    const float* __restrict__ initial, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  __shared__ float a[MAX_STREAMS];
  const int count = COUNT > 0 ? COUNT : count_arg;
  if (threadIdx.x < count) a[threadIdx.x] = read != nullptr ? read[threadIdx.x] : 1.0f;
  hx_pdl_prologue();
  __syncthreads();
  const int out_row = blockIdx.x;
  const int in_row = rows != nullptr ? rows[out_row] : out_row;
  const float* base = streams + static_cast<size_t>(in_row) * count * hidden;
  TOut* yr = out + static_cast<size_t>(out_row) * hidden;
  float sum = 0.0f;
  if constexpr (VECTORS > 0) {
    const int vectors = hidden >> 2;
    float4 u[VECTORS > 0 ? VECTORS : 1];
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
      const int v = threadIdx.x + i * 256;
      u[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (v < vectors) {
#pragma unroll
        for (int s = 0; s < (COUNT > 0 ? COUNT : MAX_STREAMS); ++s) {
          if (s < count) {
            const float4 x = reinterpret_cast<const float4*>(base + static_cast<size_t>(s) * hidden)[v];
            u[i].x = fmaf(a[s], x.x, u[i].x);
            u[i].y = fmaf(a[s], x.y, u[i].y);
            u[i].z = fmaf(a[s], x.z, u[i].z);
            u[i].w = fmaf(a[s], x.w, u[i].w);
          }
        }
        sum = fmaf(u[i].x, u[i].x, sum);
        sum = fmaf(u[i].y, u[i].y, sum);
        sum = fmaf(u[i].z, u[i].z, sum);
        sum = fmaf(u[i].w, u[i].w, sum);
      }
    }
    const float total = hx_block_sum(sum, scratch);
    const float inverse = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int i = 0; i < VECTORS; ++i) {
      const int v = threadIdx.x + i * 256;
      if (v < vectors) {
        const float4 w = reinterpret_cast<const float4*>(weight)[v];
        const int c = v << 2;
        yr[c + 0] = hx_from_float<TOut>(u[i].x * inverse * w.x);
        yr[c + 1] = hx_from_float<TOut>(u[i].y * inverse * w.y);
        yr[c + 2] = hx_from_float<TOut>(u[i].z * inverse * w.z);
        yr[c + 3] = hx_from_float<TOut>(u[i].w * inverse * w.w);
        if (clear != nullptr)
          reinterpret_cast<float4*>(clear + static_cast<size_t>(out_row) * hidden)[v] =
              initial != nullptr ? reinterpret_cast<const float4*>(initial)[v]
                                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float u = 0.0f;
      for (int s = 0; s < count; ++s) u = fmaf(a[s], base[static_cast<size_t>(s) * hidden + c], u);
      sum = fmaf(u, u, sum);
    }
    const float total = hx_block_sum(sum, scratch);
    const float inverse = 1.0f / sqrtf(total / static_cast<float>(hidden) + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float u = 0.0f;
      for (int s = 0; s < count; ++s) u = fmaf(a[s], base[static_cast<size_t>(s) * hidden + c], u);
      yr[c] = hx_from_float<TOut>(u * inverse * weight[c]);
      if (clear != nullptr)
        clear[static_cast<size_t>(out_row) * hidden + c] = initial != nullptr ? initial[c] : 0.0f;
    }
  }
}

// ---------------------------------------------------------------- rewrite all streams
// COUNT > 0: the number of streams is known to the compiler (the loops over them unroll to
// what is needed); 0: any number up to MAX_STREAMS.  blockIdx.y is the token.
template <int COUNT>
__global__ __launch_bounds__(256) void streams_write_kernel(
    float* __restrict__ streams, const float* __restrict__ y, const float* __restrict__ mixing,
    const float* __restrict__ write, const float* __restrict__ scale, int count_arg, int hidden) {
  constexpr int LIMIT = COUNT > 0 ? COUNT : MAX_STREAMS;
  __shared__ float m[MAX_STREAMS * MAX_STREAMS];
  __shared__ float b[MAX_STREAMS];
  const int count = COUNT > 0 ? COUNT : count_arg;
  for (int i = threadIdx.x; i < count * count; i += blockDim.x)
    m[i] = mixing != nullptr ? mixing[i] : 1.0f;
  if (threadIdx.x < count) b[threadIdx.x] = write != nullptr ? write[threadIdx.x] : 1.0f;
  hx_pdl_prologue();
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= hidden) return;
  const size_t token = blockIdx.y;
  float* row = streams + token * static_cast<size_t>(count) * hidden + c;
  float old[LIMIT];
#pragma unroll
  for (int s = 0; s < LIMIT; ++s)
    if (s < count) old[s] = row[static_cast<size_t>(s) * hidden];
  const float add = (scale != nullptr ? scale[c] : 1.0f) * y[token * hidden + c];
#pragma unroll
  for (int r = 0; r < LIMIT; ++r) {
    if (r < count) {
      float v = 0.0f;
#pragma unroll
      for (int s = 0; s < LIMIT; ++s)
        if (s < count) v = fmaf(m[s * count + r], old[s], v);
      row[static_cast<size_t>(r) * hidden] = fmaf(b[r], add, v);
    }
  }
}

// ------------------------------------------------- sums of scaled rows, bias, activation

// x[t][c] += sum_i scale[i] * source_i[t][c]; the sources (float32 accumulators of the
// sublayers that ran side by side) are zeroed as they are read.
struct ScaledSources {
  float* source[4];
  float scale[4];
  int count;
};

// One float4 per thread where the buffers allow it (VEC = 4), else single floats.
template <int VEC>
__global__ __launch_bounds__(256) void scaled_sum_kernel(float* __restrict__ x,
                                                         const __grid_constant__ ScaledSources sources,
                                                         size_t total) {
  hx_pdl_prologue();
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
  if (i >= total) return;
  if constexpr (VEC == 4) {
    float4 v = *reinterpret_cast<float4*>(x + i);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k < sources.count) {
        float4* source = reinterpret_cast<float4*>(sources.source[k] + i);
        const float4 s = *source;
        const float scale = sources.scale[k];
        v.x = fmaf(scale, s.x, v.x);
        v.y = fmaf(scale, s.y, v.y);
        v.z = fmaf(scale, s.z, v.z);
        v.w = fmaf(scale, s.w, v.w);
        *source = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
    *reinterpret_cast<float4*>(x + i) = v;
  } else {
    float v = x[i];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k < sources.count) {
        v = fmaf(sources.scale[k], sources.source[k][i], v);
        sources.source[k][i] = 0.0f;
      }
    }
    x[i] = v;
  }
}

// x[t][c] += bias[c]; blockIdx.y is the token.
__global__ __launch_bounds__(256) void add_bias_kernel(float* __restrict__ x,
                                                       const float* __restrict__ bias, int width) {
  hx_pdl_prologue();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  x[static_cast<size_t>(blockIdx.y) * width + c] += bias[c];
}

enum BiasedActivation : int { ACT_XIELU = 0, ACT_TANH = 1 };

// xIELU with its two constants already passed through softplus (ap = softplus(p),
// aq = 1/2 + softplus(q)): z > 0: ap z^2 + z/2; z <= 0: aq (exp(z) - 1 - z) + z/2.
__device__ __forceinline__ float xielu(float z, float ap, float aq) {
  if (z > 0.0f) return fmaf(ap * z, z, 0.5f * z);
  return fmaf(aq, expm1f(z) - z, 0.5f * z);
}

// out[t][c] = f(in[t][c] + bias[c]); `in` float32 (a product's sums), `out` the compute type.
// blockIdx.y is the token; a thread takes four neighbouring channels.
template <typename TOut>
__global__ __launch_bounds__(256) void biased_activation_kernel(
    const float* __restrict__ in, int ld_in, const float* __restrict__ bias, TOut* __restrict__ out,
    int ld_out, int width, int activation, float p0, float p1) {
  hx_pdl_prologue();
  const size_t token = blockIdx.y;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c0 >= width) return;
  const float* source = in + token * ld_in + c0;
  TOut* target = out + token * ld_out + c0;
  float z[4];
  const bool whole = c0 + 4 <= width && (ld_in & 3) == 0 &&
                     (reinterpret_cast<uintptr_t>(in) & 15) == 0;
  if (whole) {
    const float4 v = *reinterpret_cast<const float4*>(source);
    z[0] = v.x; z[1] = v.y; z[2] = v.z; z[3] = v.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) z[j] = c0 + j < width ? source[j] : 0.0f;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (c0 + j < width) {
      const float v = z[j] + (bias != nullptr ? bias[c0 + j] : 0.0f);
      target[j] = hx_from_float<TOut>(activation == ACT_TANH ? tanhf(v) : xielu(v, p0, p1));
    }
  }
}

inline unsigned blocks_for(size_t total, int threads) {
  return static_cast<unsigned>((total + threads - 1) / threads);
}

}  // namespace

HX_API int hx_streams_spread(const float* x, float* streams, int tokens, int hidden, int count,
                             cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && hidden > 0 && count >= 1, "hx_streams_spread: bad sizes");
  if (tokens == 0) return HX_OK;
  const size_t total = static_cast<size_t>(tokens) * hidden;
  hx_launch(streams_spread_kernel, blocks_for(total, 256), 256, 0, stream, x, streams, hidden,
            count, total);
  HX_CHECK_LAUNCH("hx_streams_spread");
  return HX_OK;
}

HX_API int hx_streams_read_norm(const float* streams, const float* read, int count,
                                const float* weight, void* out, int out_dtype, float* clear,
                                const float* initial, const int* rows, int n_rows, int hidden,
                                float eps, cudaStream_t stream) {
  HX_REQUIRE(n_rows >= 0 && hidden > 0, "hx_streams_read_norm: bad sizes");
  HX_REQUIRE(count >= 1 && count <= MAX_STREAMS, "hx_streams_read_norm: 1 to %d streams",
             MAX_STREAMS);
  HX_REQUIRE(eps > 0.0f, "hx_streams_read_norm: eps must be positive");
  if (n_rows == 0) return HX_OK;
  HX_REQUIRE(out_dtype == HX_F32 || out_dtype == HX_BF16,
             "hx_streams_read_norm: unknown dtype %d", out_dtype);
  const bool aligned = ((reinterpret_cast<uintptr_t>(streams) | reinterpret_cast<uintptr_t>(weight) |
                         reinterpret_cast<uintptr_t>(clear) | reinterpret_cast<uintptr_t>(initial)) &
                        15) == 0;
  const bool vector = hidden % 4 == 0 && hidden <= 4 * 256 * 8 && aligned;
#define HX_READ_NORM(T, COUNT, VECTORS)                                                        \
  hx_launch(streams_read_norm_kernel<T, COUNT, VECTORS>, n_rows, 256, 0, stream, streams, read, \
            count, weight, static_cast<T*>(out), clear, initial, rows, hidden, eps)
#define HX_READ_NORM_COUNT(T, VECTORS)                   \
  switch (count) {                                       \
    case 1: HX_READ_NORM(T, 1, VECTORS); break;          \
    case 2: HX_READ_NORM(T, 2, VECTORS); break;          \
    case 4: HX_READ_NORM(T, 4, VECTORS); break;          \
    default: HX_READ_NORM(T, 0, VECTORS);                \
  }
#define HX_READ_NORM_ALL(T)                                            \
  if (vector && hidden <= 4 * 256 * 4) { HX_READ_NORM_COUNT(T, 4) }     \
  else if (vector) { HX_READ_NORM_COUNT(T, 8) }                         \
  else { HX_READ_NORM(T, 0, 0); }
  if (out_dtype == HX_F32) {
    HX_READ_NORM_ALL(float)
  } else {
    HX_READ_NORM_ALL(__nv_bfloat16)
  }
#undef HX_READ_NORM_ALL
#undef HX_READ_NORM_COUNT
#undef HX_READ_NORM
  HX_CHECK_LAUNCH("hx_streams_read_norm");
  return HX_OK;
}

HX_API int hx_streams_write(float* streams, const float* y, const float* mixing,
                            const float* write, const float* scale, int count, int tokens,
                            int hidden, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && hidden > 0, "hx_streams_write: bad sizes");
  HX_REQUIRE(count >= 1 && count <= MAX_STREAMS, "hx_streams_write: 1 to %d streams", MAX_STREAMS);
  if (tokens == 0) return HX_OK;
  const dim3 grid((hidden + 255) / 256, tokens);
  switch (count) {
    case 1: hx_launch(streams_write_kernel<1>, grid, 256, 0, stream, streams, y, mixing, write, scale, count, hidden); break;
    case 2: hx_launch(streams_write_kernel<2>, grid, 256, 0, stream, streams, y, mixing, write, scale, count, hidden); break;
    case 3: hx_launch(streams_write_kernel<3>, grid, 256, 0, stream, streams, y, mixing, write, scale, count, hidden); break;
    case 4: hx_launch(streams_write_kernel<4>, grid, 256, 0, stream, streams, y, mixing, write, scale, count, hidden); break;
    case 8: hx_launch(streams_write_kernel<8>, grid, 256, 0, stream, streams, y, mixing, write, scale, count, hidden); break;
    default: hx_launch(streams_write_kernel<0>, grid, 256, 0, stream, streams, y, mixing, write, scale, count, hidden);
  }
  HX_CHECK_LAUNCH("hx_streams_write");
  return HX_OK;
}

HX_API int hx_scaled_sum(float* x, float* const* sources, const float* scales, int count,
                         int tokens, int width, cudaStream_t stream) {
  HX_REQUIRE(count >= 1 && count <= 4, "hx_scaled_sum: 1 to 4 sources");
  HX_REQUIRE(tokens >= 0 && width > 0, "hx_scaled_sum: bad sizes");
  if (tokens == 0) return HX_OK;
  ScaledSources packed;
  packed.count = count;
  for (int i = 0; i < count; ++i) {
    packed.source[i] = sources[i];
    packed.scale[i] = scales[i];
  }
  const size_t total = static_cast<size_t>(tokens) * width;
  uintptr_t addresses = reinterpret_cast<uintptr_t>(x);
  for (int i = 0; i < count; ++i) addresses |= reinterpret_cast<uintptr_t>(sources[i]);
  if (width % 4 == 0 && (addresses & 15) == 0) {
    hx_launch(scaled_sum_kernel<4>, blocks_for(total / 4, 256), 256, 0, stream, x, packed, total);
  } else {
    hx_launch(scaled_sum_kernel<1>, blocks_for(total, 256), 256, 0, stream, x, packed, total);
  }
  HX_CHECK_LAUNCH("hx_scaled_sum");
  return HX_OK;
}

HX_API int hx_add_bias(float* x, const float* bias, int tokens, int width, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && width > 0, "hx_add_bias: bad sizes");
  if (tokens == 0) return HX_OK;
  hx_launch(add_bias_kernel, dim3((width + 255) / 256, tokens), 256, 0, stream, x, bias, width);
  HX_CHECK_LAUNCH("hx_add_bias");
  return HX_OK;
}

HX_API int hx_biased_activation(const float* in, int ld_in, const float* bias, void* out,
                                int ld_out, int out_dtype, int tokens, int width, int activation,
                                float p0, float p1, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && width > 0 && ld_in >= width && ld_out >= width,
             "hx_biased_activation: bad sizes");
  HX_REQUIRE(activation == ACT_XIELU || activation == ACT_TANH,
             "hx_biased_activation: unknown activation %d", activation);
  if (tokens == 0) return HX_OK;
  const dim3 grid((width + 1023) / 1024, tokens);
  if (out_dtype == HX_F32) {
    hx_launch(biased_activation_kernel<float>, grid, 256, 0, stream, in, ld_in, bias,
              static_cast<float*>(out), ld_out, width, activation, p0, p1);
  } else if (out_dtype == HX_BF16) {
    hx_launch(biased_activation_kernel<__nv_bfloat16>, grid, 256, 0, stream, in, ld_in, bias,
              static_cast<__nv_bfloat16*>(out), ld_out, width, activation, p0, p1);
  } else {
    HX_REQUIRE(false, "hx_biased_activation: unknown dtype %d", out_dtype);
  }
  HX_CHECK_LAUNCH("hx_biased_activation");
  return HX_OK;
}
