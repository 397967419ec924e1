// Recurrent mixers: what runs between their matrix products.
//
//   * a causal per-channel filter over time with bias and silu (the short convolution in
//     front of a state-space recurrence);
//   * the selective state-space recurrence, one [state x width] matrix per head,
//         S_t = exp(-exp(A) d_t) S_(t-1) + d_t B_t x_t',   y_t = S_t' C_t + D x_t,
//         d_t = softplus(dt_t + bias);
//   * the token shift of a time-mixing layer (each projection reads its own blend of the
//     token's input and the previous token's);
//   * the decayed outer-product recurrence with a bonus on the current token,
//         o_t = (S_(t-1) + diag(u) k_t v_t')' r_t,   S_t = diag(w_t) S_(t-1) + k_t v_t',
//         w_t = exp(-exp(l_t + w0));
//   * a gated RMS norm over equal groups of channels.
//
// A step brings a portion of every sequence (cut anywhere, one token when decoding); what a
// recurrence carries from portion to portion lives in a per-request state row of float32
// (`state + slot * state_stride`), zero at admission: the filter's last taps - 1 inputs, the
// previous token's input, the matrices S.  Decays, step sizes, their exponentials and
// logarithms, the matrices and the sums over them are float32 throughout; projections arrive
// in the compute type, as their products stored them.
//
// Both recurrences run one CTA per (request, head).  A thread owns a column of S (one value
// coordinate) and a share of its rows: the rows are dealt to `parts` neighbouring lanes, which
// add their partial sums with shuffles.  The tokens' vectors are staged through shared memory
// a tile at a time, with the exponentials taken once per tile, not once per thread.
#include "hx_common.cuh"

namespace {

__device__ __forceinline__ float softplus(float x) {
  return x > 20.0f ? x : log1pf(expf(x));
}

// ---------------------------------------------------------------- filter, bias, silu

template <typename T>
struct FilterArgs {
  const T* raw;             // [tokens, ld_raw], already offset to the first filtered column
  int ld_raw;
  T* out;                   // [tokens, ld_out]
  int ld_out;
  const float* taps_weight; // [channels, taps], the last tap on the token itself
  const float* bias;        // [channels] or null
  float* state;             // per slot: [taps - 1, channels]
  long long state_stride;
  int taps;
  int channels;
  int silu;
  const int* token_request;
  const int* request_slot;
  const int* request_start;
};

__device__ __forceinline__ float filter_finish(float y, int silu) {
  return silu ? hx_silu(y) : y;
}

// The first taps - 1 tokens of a portion reach behind it, into the state.  The thread of the
// portion's first token (per channel) computes all of them and then writes the new state;
// the threads of the others among them do nothing; later tokens read the step's rows only.
// So one thread per (request, channel) touches the state and nothing races.
template <typename T>
__global__ __launch_bounds__(256) void causal_filter_kernel(const FilterArgs<T> a) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.channels) return;
  const int request = a.token_request[token];
  const int start = a.request_start[request];
  const int index = token - start;
  const int reach = a.taps - 1;
  const float* w = a.taps_weight + static_cast<size_t>(c) * a.taps;
  const float b = a.bias != nullptr ? a.bias[c] : 0.0f;
  if (index >= reach) {
    float y = b;
    for (int j = 0; j < a.taps; ++j)
      y = fmaf(w[j], hx_to_float<T>(a.raw[static_cast<size_t>(token - reach + j) * a.ld_raw + c]), y);
    a.out[static_cast<size_t>(token) * a.ld_out + c] = hx_from_float<T>(filter_finish(y, a.silu));
    return;
  }
  if (index != 0) return;
  const int count = a.request_start[request + 1] - start;
  float* state = a.state + static_cast<size_t>(a.request_slot[request]) * a.state_stride + c;
  const int behind = count < reach ? count : reach;
  for (int i = 0; i < behind; ++i) {
    float y = b;
    for (int j = 0; j < a.taps; ++j) {
      const int place = i - reach + j;       // relative to the portion's start
      const float u = place >= 0
                          ? hx_to_float<T>(a.raw[static_cast<size_t>(start + place) * a.ld_raw + c])
                          : state[static_cast<size_t>(place + reach) * a.channels];
      y = fmaf(w[j], u, y);
    }
    a.out[static_cast<size_t>(start + i) * a.ld_out + c] = hx_from_float<T>(filter_finish(y, a.silu));
  }
  // new state: the last `reach` inputs up to the portion's end; what the portion does not
  // cover moves up from the old state (ascending rows read ahead of where they write)
  for (int r = 0; r < reach; ++r) {
    const int place = count - reach + r;
    state[static_cast<size_t>(r) * a.channels] =
        place >= 0 ? hx_to_float<T>(a.raw[static_cast<size_t>(start + place) * a.ld_raw + c])
                   : state[static_cast<size_t>(place + reach) * a.channels];
  }
}

// ------------------------------------------------------------ state-space recurrence

constexpr int ROWS_PER_THREAD = 16;

template <typename T>
struct ScanArgs {
  const T* x;        // [tokens, ld]: x at column 0 (heads * width)
  const T* b;        // [tokens, ld]: groups * state
  const T* c;
  int ld;
  const T* dt;       // [tokens, ld_dt], column = head
  int ld_dt;
  const float* dt_bias;   // [heads]
  const float* a_log;     // [heads]
  const float* skip;      // [heads]
  float* state;           // per slot: [heads, state, width]
  long long state_stride;
  float* y;               // [tokens, heads * width]
  const int* request_start;
  const int* request_slot;
  int heads, width, rows, groups;   // rows = state size N
  int parts;                        // lanes that share a column
  int tile;                         // tokens staged at once
};

template <typename T>
__global__ void state_space_scan_kernel(const ScanArgs<T> a) {
  extern __shared__ float shared[];
  hx_pdl_prologue();
  const int request = blockIdx.x;
  const int head = blockIdx.y;
  const int group = head / (a.heads / a.groups);
  const int start = a.request_start[request];
  const int count = a.request_start[request + 1] - start;
  const int parts = a.parts;
  const int column = threadIdx.x / parts;
  const int part = threadIdx.x - column * parts;
  const bool live = column < a.width;
  // staged per token: B [rows], C [rows], x [width], step size, decay
  const int per_token = 2 * a.rows + a.width + 2;
  float* s_state = a.state + static_cast<size_t>(a.request_slot[request]) * a.state_stride +
                   static_cast<size_t>(head) * a.rows * a.width;
  float S[ROWS_PER_THREAD];
#pragma unroll
  for (int k = 0; k < ROWS_PER_THREAD; ++k) {
    const int n = part + k * parts;
    S[k] = (live && n < a.rows) ? s_state[static_cast<size_t>(n) * a.width + column] : 0.0f;
  }
  const float rate = expf(a.a_log[head]);
  const float bias = a.dt_bias[head];
  const float skip = a.skip[head];
  for (int base = 0; base < count; base += a.tile) {
    const int here = min(a.tile, count - base);
    __syncthreads();
    for (int i = threadIdx.x; i < here * per_token; i += blockDim.x) {
      const int t = i / per_token;
      const int e = i - t * per_token;
      const size_t token = static_cast<size_t>(start + base + t);
      float v;
      if (e < a.rows) {
        v = hx_to_float<T>(a.b[token * a.ld + group * a.rows + e]);
      } else if (e < 2 * a.rows) {
        v = hx_to_float<T>(a.c[token * a.ld + group * a.rows + (e - a.rows)]);
      } else if (e < 2 * a.rows + a.width) {
        v = hx_to_float<T>(a.x[token * a.ld + head * a.width + (e - 2 * a.rows)]);
      } else {
        const float step = softplus(hx_to_float<T>(a.dt[token * a.ld_dt + head]) + bias);
        v = e == 2 * a.rows + a.width ? step : expf(-rate * step);
      }
      shared[i] = v;
    }
    __syncthreads();
    for (int t = 0; t < here; ++t) {
      const float* row = shared + t * per_token;
      const float step = row[2 * a.rows + a.width];
      const float decay = row[2 * a.rows + a.width + 1];
      const float xv = live ? row[2 * a.rows + column] : 0.0f;
      const float push = step * xv;
      float sum = 0.0f;
#pragma unroll
      for (int k = 0; k < ROWS_PER_THREAD; ++k) {
        const int n = part + k * parts;
        if (n < a.rows) {
          S[k] = fmaf(decay, S[k], row[n] * push);
          sum = fmaf(S[k], row[a.rows + n], sum);
        }
      }
      for (int offset = parts >> 1; offset > 0; offset >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0)
        a.y[static_cast<size_t>(start + base + t) * (a.heads * a.width) + head * a.width + column] =
            fmaf(skip, xv, sum);
    }
  }
  if (live) {
#pragma unroll
    for (int k = 0; k < ROWS_PER_THREAD; ++k) {
      const int n = part + k * parts;
      if (n < a.rows) s_state[static_cast<size_t>(n) * a.width + column] = S[k];
    }
  }
}

// -------------------------------------------------------------------------- token shift

// out[s][t][c] = h[t][c] + (h[t-1][c] - h[t][c]) * mu[s][c], the previous row of a portion's
// first token being the request's state row (zero at admission); the state becomes the
// portion's last row.  The thread of the first token reads the old state before it writes.
template <typename T>
__global__ __launch_bounds__(256) void token_shift_kernel(
    const T* __restrict__ h, int ld, const float* __restrict__ mu, int mixes, T* __restrict__ out,
    long long mix_stride, float* __restrict__ state, long long state_stride, int hidden,
    const int* __restrict__ token_request, const int* __restrict__ request_slot,
    const int* __restrict__ request_start) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= hidden) return;
  const int request = token_request[token];
  const int start = request_start[request];
  const float own = hx_to_float<T>(h[static_cast<size_t>(token) * ld + c]);
  float before;
  if (token > start) {
    before = hx_to_float<T>(h[static_cast<size_t>(token - 1) * ld + c]);
  } else {
    float* kept = state + static_cast<size_t>(request_slot[request]) * state_stride + c;
    before = *kept;
    const int last = request_start[request + 1] - 1;
    *kept = hx_to_float<T>(h[static_cast<size_t>(last) * ld + c]);
  }
  const float delta = before - own;
  for (int s = 0; s < mixes; ++s)
    out[static_cast<size_t>(s) * mix_stride + static_cast<size_t>(token) * hidden + c] =
        hx_from_float<T>(fmaf(delta, mu[static_cast<size_t>(s) * hidden + c], own));
}

// ------------------------------------------------- decayed outer-product recurrence

template <typename T>
struct OuterScanArgs {
  const T* r;
  const T* k;
  const T* v;
  int ld_r, ld_k, ld_v;
  const float* decay_log;   // [tokens, heads * dim]: the decay's inner sum, before w0
  int ld_decay;
  const float* w0;          // [heads * dim]
  const float* bonus;       // [heads, dim]
  float* state;             // per slot: [heads, dim (key), dim (value)]
  long long state_stride;
  float* o;                 // [tokens, heads * dim]
  const int* request_start;
  const int* request_slot;
  int heads, dim;
  int parts, tile;
};

template <typename T>
__global__ void outer_product_scan_kernel(const OuterScanArgs<T> a) {
  extern __shared__ float shared[];
  hx_pdl_prologue();
  const int request = blockIdx.x;
  const int head = blockIdx.y;
  const int start = a.request_start[request];
  const int count = a.request_start[request + 1] - start;
  const int parts = a.parts;
  const int dim = a.dim;
  const int column = threadIdx.x / parts;
  const int part = threadIdx.x - column * parts;
  const bool live = column < dim;
  const int per_token = 4 * dim;   // r, k, w, v
  float* s_state = a.state + static_cast<size_t>(a.request_slot[request]) * a.state_stride +
                   static_cast<size_t>(head) * dim * dim;
  float S[ROWS_PER_THREAD];
  float u[ROWS_PER_THREAD];
#pragma unroll
  for (int i = 0; i < ROWS_PER_THREAD; ++i) {
    const int n = part + i * parts;
    const bool have = live && n < dim;
    S[i] = have ? s_state[static_cast<size_t>(n) * dim + column] : 0.0f;
    u[i] = n < dim ? a.bonus[head * dim + n] : 0.0f;
  }
  for (int base = 0; base < count; base += a.tile) {
    const int here = min(a.tile, count - base);
    __syncthreads();
    for (int i = threadIdx.x; i < here * per_token; i += blockDim.x) {
      const int t = i / per_token;
      const int e = i - t * per_token;
      const int which = e / dim;
      const int d = e - which * dim;
      const size_t token = static_cast<size_t>(start + base + t);
      const int channel = head * dim + d;
      float value;
      if (which == 0) {
        value = hx_to_float<T>(a.r[token * a.ld_r + channel]);
      } else if (which == 1) {
        value = hx_to_float<T>(a.k[token * a.ld_k + channel]);
      } else if (which == 2) {
        value = expf(-expf(a.decay_log[token * a.ld_decay + channel] + a.w0[channel]));
      } else {
        value = hx_to_float<T>(a.v[token * a.ld_v + channel]);
      }
      shared[i] = value;
    }
    __syncthreads();
    for (int t = 0; t < here; ++t) {
      const float* row = shared + t * per_token;
      const float vj = live ? row[3 * dim + column] : 0.0f;
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < ROWS_PER_THREAD; ++i) {
        const int n = part + i * parts;
        if (n < dim) {
          const float pair = row[dim + n] * vj;
          sum = fmaf(row[n], fmaf(u[i], pair, S[i]), sum);
          S[i] = fmaf(row[2 * dim + n], S[i], pair);
        }
      }
      for (int offset = parts >> 1; offset > 0; offset >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0)
        a.o[static_cast<size_t>(start + base + t) * (a.heads * dim) + head * dim + column] = sum;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < ROWS_PER_THREAD; ++i) {
      const int n = part + i * parts;
      if (n < dim) s_state[static_cast<size_t>(n) * dim + column] = S[i];
    }
  }
}

// ----------------------------------------------------------------- gated group norm

// Channels in `groups` equal parts, each divided by its own root mean square (eps inside the
// root), times a weight.  gate_after = 0: the gate silu(g) multiplies BEFORE the norm
// (v = y silu(g); out = v / rms(v) * w); 1: after it (out = y / rms(y) * w * silu(g)).
template <typename T>
__global__ __launch_bounds__(128) void gated_group_norm_kernel(
    const float* __restrict__ y, int ld_y, const T* __restrict__ gate, int ld_gate,
    const float* __restrict__ weight, T* __restrict__ out, int ld_out, int width, float eps,
    int gate_after) {
  __shared__ float scratch[32];
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int first = blockIdx.y * width;
  const float* yr = y + static_cast<size_t>(token) * ld_y + first;
  const T* gr = gate + static_cast<size_t>(token) * ld_gate + first;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = yr[c];
    if (!gate_after) v *= hx_silu(hx_to_float<T>(gr[c]));
    sum = fmaf(v, v, sum);
  }
  const float total = hx_block_sum(sum, scratch);
  const float inverse = 1.0f / sqrtf(total / static_cast<float>(width) + eps);
  T* o = out + static_cast<size_t>(token) * ld_out + first;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float g = hx_silu(hx_to_float<T>(gr[c]));
    float v = yr[c];
    if (!gate_after) v *= g;
    v = v * inverse * weight[first + c];
    if (gate_after) v *= g;
    o[c] = hx_from_float<T>(v);
  }
}

// lanes that share a column: the smallest power of two that leaves a thread at most
// ROWS_PER_THREAD rows; 0 when even a whole warp would not do
int parts_for(int rows) {
  for (int parts = 1; parts <= 32; parts <<= 1)
    if (parts * ROWS_PER_THREAD >= rows) return parts;
  return 0;
}

// tokens staged per tile so that the tile fits the shared memory a CTA gets without asking
int tile_for(int floats_per_token) {
  const int budget = 40 * 1024 / 4;
  int tile = budget / floats_per_token;
  if (tile > 32) tile = 32;
  return tile;
}

}  // namespace

HX_API int hx_causal_filter(const void* raw, int ld_raw, void* out, int ld_out, int dtype,
                            const float* taps_weight, const float* bias, float* state,
                            long long state_stride, int taps, int channels, int silu, int tokens,
                            const int* token_request, const int* request_slot,
                            const int* request_start, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && channels > 0 && taps >= 1, "hx_causal_filter: bad sizes");
  HX_REQUIRE(taps == 1 || state != nullptr, "hx_causal_filter: a filter of %d taps needs state", taps);
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens, (channels + 255) / 256);
  if (dtype == HX_F32) {
    FilterArgs<float> a{static_cast<const float*>(raw), ld_raw, static_cast<float*>(out), ld_out,
                        taps_weight, bias, state, state_stride, taps, channels, silu,
                        token_request, request_slot, request_start};
    hx_launch(causal_filter_kernel<float>, grid, 256, 0, stream, a);
  } else if (dtype == HX_BF16) {
    FilterArgs<__nv_bfloat16> a{static_cast<const __nv_bfloat16*>(raw), ld_raw,
                                static_cast<__nv_bfloat16*>(out), ld_out, taps_weight, bias, state,
                                state_stride, taps, channels, silu, token_request, request_slot,
                                request_start};
    hx_launch(causal_filter_kernel<__nv_bfloat16>, grid, 256, 0, stream, a);
  } else {
    HX_REQUIRE(false, "hx_causal_filter: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_causal_filter");
  return HX_OK;
}

HX_API int hx_state_space_scan(const void* x, const void* b, const void* c, int ld, const void* dt,
                               int ld_dt, int dtype, const float* dt_bias, const float* a_log,
                               const float* skip, float* state, long long state_stride, float* y,
                               const int* request_start, const int* request_slot, int requests,
                               int heads, int width, int rows, int groups, cudaStream_t stream) {
  HX_REQUIRE(requests >= 0 && heads > 0 && width > 0 && rows > 0 && groups > 0,
             "hx_state_space_scan: bad sizes");
  HX_REQUIRE(heads % groups == 0, "hx_state_space_scan: heads must be a multiple of groups");
  const int parts = parts_for(rows);
  HX_REQUIRE(parts > 0, "hx_state_space_scan: a state of %d rows is more than %d", rows,
             32 * ROWS_PER_THREAD);
  const int threads = (width * parts + 31) / 32 * 32;
  HX_REQUIRE(threads <= 1024, "hx_state_space_scan: heads of %d with a state of %d need %d threads",
             width, rows, threads);
  const int per_token = 2 * rows + width + 2;
  const int tile = tile_for(per_token);
  HX_REQUIRE(tile >= 1, "hx_state_space_scan: a token's vectors do not fit shared memory");
  if (requests == 0) return HX_OK;
  const dim3 grid(requests, heads);
  const size_t shared_bytes = static_cast<size_t>(tile) * per_token * sizeof(float);
  if (dtype == HX_F32) {
    ScanArgs<float> a{static_cast<const float*>(x), static_cast<const float*>(b),
                      static_cast<const float*>(c), ld, static_cast<const float*>(dt), ld_dt,
                      dt_bias, a_log, skip, state, state_stride, y, request_start, request_slot,
                      heads, width, rows, groups, parts, tile};
    hx_launch(state_space_scan_kernel<float>, grid, threads, shared_bytes, stream, a);
  } else if (dtype == HX_BF16) {
    ScanArgs<__nv_bfloat16> a{static_cast<const __nv_bfloat16*>(x),
                              static_cast<const __nv_bfloat16*>(b),
                              static_cast<const __nv_bfloat16*>(c), ld,
                              static_cast<const __nv_bfloat16*>(dt), ld_dt, dt_bias, a_log, skip,
                              state, state_stride, y, request_start, request_slot, heads, width,
                              rows, groups, parts, tile};
    hx_launch(state_space_scan_kernel<__nv_bfloat16>, grid, threads, shared_bytes, stream, a);
  } else {
    HX_REQUIRE(false, "hx_state_space_scan: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_state_space_scan");
  return HX_OK;
}

HX_API int hx_token_shift(const void* h, int ld, int dtype, const float* mu, int mixes, void* out,
                          long long mix_stride, float* state, long long state_stride, int tokens,
                          int hidden, const int* token_request, const int* request_slot,
                          const int* request_start, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && hidden > 0 && mixes >= 1, "hx_token_shift: bad sizes");
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens, (hidden + 255) / 256);
  if (dtype == HX_F32) {
    hx_launch(token_shift_kernel<float>, grid, 256, 0, stream, static_cast<const float*>(h), ld, mu,
              mixes, static_cast<float*>(out), mix_stride, state, state_stride, hidden,
              token_request, request_slot, request_start);
  } else if (dtype == HX_BF16) {
    hx_launch(token_shift_kernel<__nv_bfloat16>, grid, 256, 0, stream,
              static_cast<const __nv_bfloat16*>(h), ld, mu, mixes, static_cast<__nv_bfloat16*>(out),
              mix_stride, state, state_stride, hidden, token_request, request_slot, request_start);
  } else {
    HX_REQUIRE(false, "hx_token_shift: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_token_shift");
  return HX_OK;
}

HX_API int hx_outer_product_scan(const void* r, int ld_r, const void* k, int ld_k, const void* v,
                                 int ld_v, int dtype, const float* decay_log, int ld_decay,
                                 const float* w0, const float* bonus, float* state,
                                 long long state_stride, float* o, const int* request_start,
                                 const int* request_slot, int requests, int heads, int dim,
                                 cudaStream_t stream) {
  HX_REQUIRE(requests >= 0 && heads > 0 && dim > 0, "hx_outer_product_scan: bad sizes");
  const int parts = parts_for(dim);
  HX_REQUIRE(parts > 0, "hx_outer_product_scan: heads of %d are more than %d", dim,
             32 * ROWS_PER_THREAD);
  const int threads = (dim * parts + 31) / 32 * 32;
  HX_REQUIRE(threads <= 1024, "hx_outer_product_scan: heads of %d need %d threads", dim, threads);
  const int tile = tile_for(4 * dim);
  HX_REQUIRE(tile >= 1, "hx_outer_product_scan: a token's vectors do not fit shared memory");
  if (requests == 0) return HX_OK;
  const dim3 grid(requests, heads);
  const size_t shared_bytes = static_cast<size_t>(tile) * 4 * dim * sizeof(float);
  if (dtype == HX_F32) {
    OuterScanArgs<float> a{static_cast<const float*>(r), static_cast<const float*>(k),
                           static_cast<const float*>(v), ld_r, ld_k, ld_v, decay_log, ld_decay, w0,
                           bonus, state, state_stride, o, request_start, request_slot, heads, dim,
                           parts, tile};
    hx_launch(outer_product_scan_kernel<float>, grid, threads, shared_bytes, stream, a);
  } else if (dtype == HX_BF16) {
    OuterScanArgs<__nv_bfloat16> a{static_cast<const __nv_bfloat16*>(r),
                                   static_cast<const __nv_bfloat16*>(k),
                                   static_cast<const __nv_bfloat16*>(v), ld_r, ld_k, ld_v,
                                   decay_log, ld_decay, w0, bonus, state, state_stride, o,
                                   request_start, request_slot, heads, dim, parts, tile};
    hx_launch(outer_product_scan_kernel<__nv_bfloat16>, grid, threads, shared_bytes, stream, a);
  } else {
    HX_REQUIRE(false, "hx_outer_product_scan: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_outer_product_scan");
  return HX_OK;
}

HX_API int hx_gated_group_norm(const float* y, int ld_y, const void* gate, int ld_gate, int dtype,
                               const float* weight, void* out, int ld_out, int tokens, int channels,
                               int groups, float eps, int gate_after, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && channels > 0 && groups > 0 && channels % groups == 0,
             "hx_gated_group_norm: bad sizes");
  HX_REQUIRE(eps > 0.0f, "hx_gated_group_norm: eps must be positive");
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens, groups);
  const int width = channels / groups;
  if (dtype == HX_F32) {
    hx_launch(gated_group_norm_kernel<float>, grid, 128, 0, stream, y, ld_y,
              static_cast<const float*>(gate), ld_gate, weight, static_cast<float*>(out), ld_out,
              width, eps, gate_after);
  } else if (dtype == HX_BF16) {
    hx_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, 128, 0, stream, y, ld_y,
              static_cast<const __nv_bfloat16*>(gate), ld_gate, weight,
              static_cast<__nv_bfloat16*>(out), ld_out, width, eps, gate_after);
  } else {
    HX_REQUIRE(false, "hx_gated_group_norm: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_gated_group_norm");
  return HX_OK;
}
