// Short causal convolution over time on the projected rows of a mixer, with the cache append
// fused in, and the sigmoid output gate.
//
// Convolution.  Every channel c of the projected queries, keys and values is filtered along
// the sequence with `taps` weights of its own:
//
//     y[t, c] = sum_{j < taps} w[c, j] * u[t - (taps - 1) + j, c],      u = 0 before the sequence
//
// so w[c, taps - 1] multiplies the token's own value.  A step brings a portion of a sequence
// (cut anywhere), so the last taps - 1 projected values of every sequence are kept in a state
// row per request, `state[slot, i, c]` = u at position (length - (taps - 1) + i), zero at
// admission.  Products and the sum are float32 (ascending j), one rounding into the storage
// type; projected values are used as the projection's own store rounds them.
//
// Who touches the state.  The first taps - 1 tokens of a request's portion are the only ones
// whose filter reaches behind the portion.  The thread of a request's FIRST token (per
// channel) computes all of them, then writes the new state; the threads of tokens 1 .. taps - 2
// do nothing, and every later token reads the step's own rows only.  One thread per (request,
// channel) reads and writes the state, so nothing races, whatever the portion's length.
//
// Columns.  A row is [q heads | k heads | v heads | passthrough]: the first three (heads of
// `head_dim`) are filtered; queries go to `out`, keys and values to their pages (or to `out`
// when the caller appends them itself); passthrough columns (an output gate's projection that
// shares the product) are copied, rounded, to `out`.  With `accum` the projection is read
// from that float32 accumulator, which is NOT cleared here: neighbouring tokens read each
// other's sums, so whoever runs next clears it (hx_sigmoid_gate does).
#include "hx_common.cuh"

namespace {

template <typename T>
struct ConvArgs {
  const T* raw;
  int ld_raw;
  const float* accum;
  int ld_accum;
  T* out;
  int ld_out;
  const float* filter;      // [conv channels, taps]
  T* state;                 // [slots, taps - 1, conv channels]
  int taps;
  const int* positions;
  const int* token_request;
  const int* request_slot;
  const int* request_start;
  const int* block_tables;
  int table_stride;
  T* k_cache;
  T* v_cache;
  int write_cache;
  int heads, kv_heads, head_dim;
  int total;                // columns of a row in all
  int page_size, num_pages;
  int* status;
};

template <typename T>
__device__ __forceinline__ float projected(const ConvArgs<T>& a, int token, int c) {
  if (a.accum != nullptr)
    return hx_to_float<T>(hx_from_float<T>(a.accum[static_cast<size_t>(token) * a.ld_accum + c]));
  return hx_to_float<T>(a.raw[static_cast<size_t>(token) * a.ld_raw + c]);
}

template <typename T>
__device__ __forceinline__ void emit(const ConvArgs<T>& a, int token, int position, int table_row,
                                     int c, float y) {
  const int q_size = a.heads * a.head_dim;
  if (c < q_size || !a.write_cache) {
    a.out[static_cast<size_t>(token) * a.ld_out + c] = hx_from_float<T>(y);
    return;
  }
  const int kv_size = a.kv_heads * a.head_dim;
  const bool is_key = c < q_size + kv_size;
  const int within = c - q_size - (is_key ? 0 : kv_size);
  const int kv_head = within / a.head_dim;
  const int d = within - kv_head * a.head_dim;
  const int page =
      a.block_tables[static_cast<size_t>(table_row) * a.table_stride + position / a.page_size];
  if (page < 0 || page >= a.num_pages) {
    if (a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
    return;
  }
  T* cache = is_key ? a.k_cache : a.v_cache;
  const int chunk = hx_cache_chunk(sizeof(T), a.head_dim);
  cache[hx_cache_offset(page, kv_head, position % a.page_size, d, a.kv_heads, a.page_size,
                        a.head_dim, chunk)] = hx_from_float<T>(y);
}

template <typename T>
__global__ __launch_bounds__(256) void short_conv_append_kernel(const ConvArgs<T> a) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.total) return;
  const int channels = (a.heads + 2 * a.kv_heads) * a.head_dim;
  if (c >= channels) {      // passthrough: rounded and copied
    a.out[static_cast<size_t>(token) * a.ld_out + c] = hx_from_float<T>(projected(a, token, c));
    return;
  }
  const int request = a.token_request[token];
  const int start = a.request_start[request];
  const int index = token - start;                 // place of the token in its portion
  const int reach = a.taps - 1;
  const int table_row = a.request_slot[request];
  const float* w = a.filter + static_cast<size_t>(c) * a.taps;
  if (index >= reach) {
    // the filter stays inside the portion
    float y = 0.0f;
    for (int j = 0; j < a.taps; ++j) y = fmaf(w[j], projected(a, token - reach + j, c), y);
    emit(a, token, a.positions[token], table_row, c, y);
    return;
  }
  if (index != 0) return;      // computed by the thread of the portion's first token
  const int count = a.request_start[request + 1] - start;
  const int first_position = a.positions[token];
  T* state = a.state + static_cast<size_t>(table_row) * reach * channels + c;
  const int behind = count < reach ? count : reach;
  for (int i = 0; i < behind; ++i) {
    // token start + i: taps j reach position i - reach + j of the portion; negative ones are
    // state rows (row r of the state is position r - reach relative to the portion's start)
    float y = 0.0f;
    for (int j = 0; j < a.taps; ++j) {
      const int place = i - reach + j;
      const float u = place >= 0 ? projected(a, start + place, c)
                                 : hx_to_float<T>(state[static_cast<size_t>(place + reach) * channels]);
      y = fmaf(w[j], u, y);
    }
    emit(a, start + i, first_position + i, table_row, c, y);
  }
  // the new state: the last `reach` values up to the portion's end; what the portion does not
  // cover moves up from the old state (ascending rows read ahead of where they write)
  for (int r = 0; r < reach; ++r) {
    const int place = count - reach + r;
    const T value = place >= 0 ? hx_from_float<T>(projected(a, start + place, c))
                               : state[static_cast<size_t>(place + reach) * channels];
    state[static_cast<size_t>(r) * channels] = value;
  }
}

// The same for bfloat16 rows made of whole 16-byte pieces (8 channels): one thread per piece,
// every access 16 bytes wide (32 for the float32 accumulator), and a piece of a key or value
// is exactly one 16-byte chunk of the cache layout.  Up to CONV_FAST_TAPS taps, whose weights
// (and the token's place, its request and its page: the step's own description) are looked
// up BEFORE the wait for the projection, while the projection still runs.
constexpr int CONV_FAST_TAPS = 4;

__device__ __forceinline__ void unpack8(const uint4& packed, float (&x)[8]) {
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(pairs[i]);
    x[2 * i] = v.x;
    x[2 * i + 1] = v.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  uint4 packed;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
  return packed;
}

// eight projected values of `token` from column c, as the projection's store rounds them
__device__ __forceinline__ uint4 projected8(const ConvArgs<__nv_bfloat16>& a, int token, int c) {
  if (a.accum != nullptr) {
    const float4* source =
        reinterpret_cast<const float4*>(a.accum + static_cast<size_t>(token) * a.ld_accum + c);
    const float4 lo = source[0], hi = source[1];
    const float raw[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    return pack8(raw);
  }
  return *reinterpret_cast<const uint4*>(a.raw + static_cast<size_t>(token) * a.ld_raw + c);
}

__device__ __forceinline__ void emit8(const ConvArgs<__nv_bfloat16>& a, int token, int position,
                                      int table_row, int c, const uint4& packed) {
  const int q_size = a.heads * a.head_dim;
  if (c < q_size || !a.write_cache) {
    *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(token) * a.ld_out + c) = packed;
    return;
  }
  const int kv_size = a.kv_heads * a.head_dim;
  const bool is_key = c < q_size + kv_size;
  const int within = c - q_size - (is_key ? 0 : kv_size);
  const int kv_head = within / a.head_dim;
  const int d = within - kv_head * a.head_dim;
  const int page =
      a.block_tables[static_cast<size_t>(table_row) * a.table_stride + position / a.page_size];
  if (page < 0 || page >= a.num_pages) {
    if (a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
    return;
  }
  __nv_bfloat16* cache = is_key ? a.k_cache : a.v_cache;
  *reinterpret_cast<uint4*>(cache + hx_cache_offset(page, kv_head, position % a.page_size, d,
                                                    a.kv_heads, a.page_size, a.head_dim, 8)) = packed;
}

// A thread takes one piece (8 channels) of `run` consecutive tokens of the batch: the filter's
// weights are fetched once (16 bytes a load), and a row of projected values is fetched once
// and kept for the tokens behind it.
template <int TAPS>
__global__ __launch_bounds__(256) void short_conv_append_pieces_kernel(
    const ConvArgs<__nv_bfloat16> a, int tokens, int run) {
  hx_pdl_trigger();
  constexpr int REACH = TAPS - 1;
  const int first = blockIdx.x * run;
  const int last = min(first + run, tokens);      // exclusive
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const int channels = (a.heads + 2 * a.kv_heads) * a.head_dim;
  if (c >= a.total) {
    hx_pdl_wait();      // a grid must not be seen complete before its predecessor is
    return;
  }
  if (c >= channels) {      // passthrough: rounded and copied
    hx_pdl_wait();
    for (int token = first; token < last; ++token)
      *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(token) * a.ld_out + c) =
          projected8(a, token, c);
    return;
  }
  // w[j][i]: tap j of channel c + i; the 8 * TAPS weights of the piece are contiguous
  float w[TAPS][8];
  {
    float flat[8 * TAPS];
    const float4* source = reinterpret_cast<const float4*>(a.filter + static_cast<size_t>(c) * TAPS);
#pragma unroll
    for (int v = 0; v < 2 * TAPS; ++v) {
      const float4 x = source[v];
      flat[4 * v] = x.x; flat[4 * v + 1] = x.y; flat[4 * v + 2] = x.z; flat[4 * v + 3] = x.w;
    }
#pragma unroll
    for (int j = 0; j < TAPS; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) w[j][i] = flat[i * TAPS + j];
  }
  // the run's first token (in decoding the only one): its request, place and position are
  // the step's own description and are looked up while the projection still runs
  const int first_request = a.token_request[first];
  const int first_start = a.request_start[first_request];
  const int first_slot = a.request_slot[first_request];
  const int first_position = a.positions[first];
  hx_pdl_wait();

  // rows[j]: the projected values of batch row (token - REACH + j); they are used only by a
  // token that lies at least REACH tokens into its request's portion
  uint4 rows[TAPS];
#pragma unroll
  for (int j = 0; j < REACH; ++j) {
    const int row = first - REACH + j;
    // (rows of another request are never used: not fetched)
    rows[j] = row >= first_start ? projected8(a, row, c) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int token = first; token < last; ++token) {
    rows[REACH] = projected8(a, token, c);
    const bool head = token == first;
    const int request = head ? first_request : a.token_request[token];
    const int start = head ? first_start : a.request_start[request];
    const int index = token - start;
    const int table_row = head ? first_slot : a.request_slot[request];
    if (index >= REACH) {
      float y[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        float u[8];
        unpack8(rows[j], u);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = fmaf(w[j][i], u[i], y[i]);
      }
      emit8(a, token, head ? first_position : a.positions[token], table_row, c, pack8(y));
    } else if (index == 0) {
      // the portion's first token: the tokens whose filter reaches behind the portion, then
      // the new state (see the scalar kernel)
      const int count = a.request_start[request + 1] - start;
      const int position = head ? first_position : a.positions[token];
      __nv_bfloat16* state = a.state + static_cast<size_t>(table_row) * REACH * channels + c;
      const int behind = count < REACH ? count : REACH;
      for (int t = 0; t < behind; ++t) {
        float y[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
          const int place = t - REACH + j;
          float u[8];
          unpack8(place >= 0 ? projected8(a, start + place, c)
                             : *reinterpret_cast<const uint4*>(
                                   state + static_cast<size_t>(place + REACH) * channels), u);
#pragma unroll
          for (int i = 0; i < 8; ++i) y[i] = fmaf(w[j][i], u[i], y[i]);
        }
        emit8(a, start + t, position + t, table_row, c, pack8(y));
      }
      for (int r = 0; r < REACH; ++r) {
        const int place = count - REACH + r;
        const uint4 value = place >= 0 ? projected8(a, start + place, c)
                                       : *reinterpret_cast<const uint4*>(
                                             state + static_cast<size_t>(place + REACH) * channels);
        *reinterpret_cast<uint4*>(state + static_cast<size_t>(r) * channels) = value;
      }
    }
#pragma unroll
    for (int j = 0; j < REACH; ++j) rows[j] = rows[j + 1];
  }
}

bool pieces_apply(const ConvArgs<__nv_bfloat16>& a) {
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return a.taps <= CONV_FAST_TAPS && a.head_dim % 8 == 0 && a.total % 8 == 0 &&
         a.ld_out % 8 == 0 && aligned(a.out) && aligned(a.state) &&
         (a.raw == nullptr || (a.ld_raw % 8 == 0 && aligned(a.raw))) &&
         (a.accum == nullptr || (a.ld_accum % 4 == 0 && aligned(a.accum))) &&
         (!a.write_cache || (aligned(a.k_cache) && aligned(a.v_cache)));
}

int launch_conv(const ConvArgs<__nv_bfloat16>& a, int tokens, cudaStream_t stream) {
  if (!pieces_apply(a)) {
    const dim3 grid(tokens, (a.total + 255) / 256);
    HX_REQUIRE(grid.y <= 65535, "hx_short_conv_append: rows too wide");
    hx_launch(short_conv_append_kernel<__nv_bfloat16>, grid, 256, 0, stream, a);
    return HX_OK;
  }
  const int run = tokens >= 1024 ? 8 : (tokens >= 256 ? 2 : 1);
  const int pieces = a.total / 8;
  const int block = pieces >= 256 ? 256 : ((pieces + 31) / 32) * 32;
  const dim3 grid((tokens + run - 1) / run, (pieces + block - 1) / block);
  HX_REQUIRE(grid.y <= 65535, "hx_short_conv_append: rows too wide");
  switch (a.taps) {
    case 1: hx_launch(short_conv_append_pieces_kernel<1>, grid, block, 0, stream, a, tokens, run); break;
    case 2: hx_launch(short_conv_append_pieces_kernel<2>, grid, block, 0, stream, a, tokens, run); break;
    case 3: hx_launch(short_conv_append_pieces_kernel<3>, grid, block, 0, stream, a, tokens, run); break;
    default: hx_launch(short_conv_append_pieces_kernel<4>, grid, block, 0, stream, a, tokens, run); break;
  }
  return HX_OK;
}

template <typename T>
int launch_conv(const ConvArgs<T>& a, int tokens, cudaStream_t stream) {
  const dim3 grid(tokens, (a.total + 255) / 256);
  HX_REQUIRE(grid.y <= 65535, "hx_short_conv_append: rows too wide");
  hx_launch(short_conv_append_kernel<T>, grid, 256, 0, stream, a);
  return HX_OK;
}

// context[t, c] *= sigmoid(gate[t, c]) in float32, one rounding; then the rows of `clear`
// (a float32 accumulator the step's projection summed into) are zeroed.
template <typename T>
__global__ __launch_bounds__(256) void sigmoid_gate_kernel(T* __restrict__ context, int ld_context,
                                                           const T* __restrict__ gate, int ld_gate,
                                                           int tokens, int width,
                                                           float* __restrict__ clear, int ld_clear,
                                                           int clear_width) {
  hx_pdl_prologue();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t first = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t total = static_cast<size_t>(tokens) * width;
  for (size_t index = first; index < total; index += stride) {
    const size_t t = index / width;
    const int c = static_cast<int>(index - t * width);
    T* value = context + t * ld_context + c;
    const float g = hx_to_float<T>(gate[t * ld_gate + c]);
    *value = hx_from_float<T>(hx_to_float<T>(*value) * hx_sigmoid(g));
  }
  if (clear != nullptr) {
    const size_t cells = static_cast<size_t>(tokens) * clear_width;
    for (size_t index = first; index < cells; index += stride) {
      const size_t t = index / clear_width;
      clear[t * ld_clear + (index - t * clear_width)] = 0.0f;
    }
  }
}

}  // namespace

// See the head of this file.  raw or accum is given (the other null); `state` may be null
// when taps == 1.  request_slot[r] is the request's state row and its block-table row.
HX_API int hx_short_conv_append(const void* raw, int ld_raw, const float* accum, int ld_accum,
                                void* out, int ld_out, int dtype, const float* filter, void* state,
                                int taps, const int* positions, const int* token_request,
                                const int* request_slot, const int* request_start,
                                const int* block_tables, int table_stride, void* k_cache,
                                void* v_cache, int write_cache, int tokens, int heads,
                                int kv_heads, int head_dim, int total, int page_size,
                                int num_pages, int* status, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0,
             "hx_short_conv_append: bad sizes");
  const int channels = (heads + 2 * kv_heads) * head_dim;
  HX_REQUIRE(taps >= 1 && taps <= 64, "hx_short_conv_append: taps %d outside 1..64", taps);
  HX_REQUIRE(total >= channels, "hx_short_conv_append: a row holds %d columns, fewer than its "
             "%d filtered ones", total, channels);
  HX_REQUIRE((raw != nullptr) != (accum != nullptr),
             "hx_short_conv_append: give the projected rows or their accumulator");
  HX_REQUIRE(raw == nullptr || ld_raw >= total, "hx_short_conv_append: row stride too small");
  HX_REQUIRE(accum == nullptr || ld_accum >= total,
             "hx_short_conv_append: accumulator stride too small");
  HX_REQUIRE(out != nullptr && ld_out >= total, "hx_short_conv_append: output stride too small");
  HX_REQUIRE(out != raw, "hx_short_conv_append: the filter cannot run in place");
  HX_REQUIRE(filter != nullptr && (taps == 1 || state != nullptr),
             "hx_short_conv_append: filter or state missing");
  HX_REQUIRE(!write_cache || (page_size > 0 && num_pages > 0 && k_cache && v_cache && block_tables),
             "hx_short_conv_append: cache arguments missing");
  if (tokens == 0) return HX_OK;
  int rc;
  if (dtype == HX_F32) {
    ConvArgs<float> a{static_cast<const float*>(raw), ld_raw, accum, ld_accum,
                      static_cast<float*>(out), ld_out, filter, static_cast<float*>(state), taps,
                      positions, token_request, request_slot, request_start, block_tables,
                      table_stride, static_cast<float*>(k_cache), static_cast<float*>(v_cache),
                      write_cache, heads, kv_heads, head_dim, total, page_size, num_pages, status};
    rc = launch_conv(a, tokens, stream);
  } else if (dtype == HX_BF16) {
    ConvArgs<__nv_bfloat16> a{static_cast<const __nv_bfloat16*>(raw), ld_raw, accum, ld_accum,
                              static_cast<__nv_bfloat16*>(out), ld_out, filter,
                              static_cast<__nv_bfloat16*>(state), taps, positions, token_request,
                              request_slot, request_start, block_tables, table_stride,
                              static_cast<__nv_bfloat16*>(k_cache),
                              static_cast<__nv_bfloat16*>(v_cache), write_cache, heads, kv_heads,
                              head_dim, total, page_size, num_pages, status};
    rc = launch_conv(a, tokens, stream);
  } else {
    HX_REQUIRE(false, "hx_short_conv_append: unknown dtype %d", dtype);
  }
  if (rc != HX_OK) return rc;
  HX_CHECK_LAUNCH("hx_short_conv_append");
  return HX_OK;
}

// context[t, :width] *= sigmoid(gate[t, :width]); `clear` (may be null): float32 rows
// [tokens, clear_width] to zero afterwards.
HX_API int hx_sigmoid_gate(void* context, int ld_context, const void* gate, int ld_gate, int dtype,
                           int tokens, int width, float* clear, int ld_clear, int clear_width,
                           cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && width > 0 && ld_context >= width && ld_gate >= width,
             "hx_sigmoid_gate: bad sizes");
  HX_REQUIRE(clear == nullptr || (clear_width > 0 && ld_clear >= clear_width),
             "hx_sigmoid_gate: bad accumulator sizes");
  if (tokens == 0) return HX_OK;
  const size_t cells = static_cast<size_t>(tokens) * (clear != nullptr && clear_width > width ? clear_width : width);
  const size_t resident = static_cast<size_t>(hx_device_sm_count() > 0 ? hx_device_sm_count() : 1) * 16;
  const size_t wanted = (cells + 255) / 256;
  const int blocks = static_cast<int>(wanted < resident ? wanted : resident);
  if (dtype == HX_F32) {
    hx_launch(sigmoid_gate_kernel<float>, blocks, 256, 0, stream, static_cast<float*>(context),
              ld_context, static_cast<const float*>(gate), ld_gate, tokens, width, clear, ld_clear,
              clear_width);
  } else if (dtype == HX_BF16) {
    hx_launch(sigmoid_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream,
              static_cast<__nv_bfloat16*>(context), ld_context,
              static_cast<const __nv_bfloat16*>(gate), ld_gate, tokens, width, clear, ld_clear,
              clear_width);
  } else {
    HX_REQUIRE(false, "hx_sigmoid_gate: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_sigmoid_gate");
  return HX_OK;
}
