// Rotary encoding with angles taken from the position itself, a per-head RMS norm of queries
// and keys in front of it, rotated values, and the cache append, in one kernel; and the
// rotation that turns an attention output back.
//
// A projected row is [q heads | k heads | v heads], every head `row_dim` wide of which the
// first `head_dim` (values: `value_dim`) coordinates are real and the rest exact zeros.
//
//   * norm (optional): a head x becomes x / sqrt(mean(x^2) + eps) * g with one weight g
//     [head_dim] for all query heads and one for all key heads; before the rotation.
//   * rotation of q and k: the first `rotary_dim` coordinates turn in pairs by the angle
//     position * f[m], f[m] = base^(-2m / rotary_dim) (the table `freq`, float32); pairs are
//     (m, m + rotary_dim/2) (layout 1, halves) or (2m, 2m + 1) (layout 0, interleaved).  The
//     angle is the float32 product, sine and cosine are float32.
//   * rotated values (optional): the value of position j turns by j over all `value_dim`
//     coordinates with its own table `value_freq` and layout, and is cached so.  A head's
//     attention output at position i, a weighted sum of such values, is turned back by -i
//     (hx_rotate_back), which leaves every value turned by its distance to the query.
//
// One warp per head: the lanes hold the head's pairs in registers between the sum of squares
// and the rotation.  Keys and values go to their pages, queries back into the row.
#include "hx_common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_PAIRS_PER_LANE = 4;     // heads up to 256 wide

__device__ __forceinline__ void pair_of(int p, int dims, int layout, int& i0, int& i1,
                                        bool& rotate) {
  const int half = dims >> 1;
  if (layout == 0) {
    i0 = 2 * p;
    i1 = i0 + 1;
    rotate = i1 < dims;
  } else if (p < half) {
    i0 = p;
    i1 = p + half;
    rotate = true;
  } else {
    i0 = dims + 2 * (p - half);
    i1 = i0 + 1;
    rotate = false;
  }
}

template <typename T>
struct RotaryArgs {
  T* qkv;
  int ld;
  float* accum;             // float32 sums of the projection (then qkv's k/v columns are unused)
  int ld_accum;
  const int* positions;
  const int* token_request;
  const int* request_table_row;
  const int* block_tables;
  int table_stride;
  T* k_cache;
  T* v_cache;
  int write_cache;
  const float* freq;        // [rotary_dim / 2]
  const float* value_freq;  // [value_dim / 2] or null: values are stored as projected
  const float* q_norm;      // [head_dim] or null
  const float* k_norm;
  float eps;
  int heads, kv_heads, head_dim, value_dim, row_dim, rotary_dim, layout, value_layout;
  int page_size, num_pages;
  int* status;
};

template <typename T>
__global__ __launch_bounds__(WARPS * 32) void norm_rotary_append_kernel(const RotaryArgs<T> a) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y * WARPS + (threadIdx.x >> 5);
  if (head >= a.heads + 2 * a.kv_heads) return;
  const int position = a.positions[token];
  const bool is_query = head < a.heads;
  const bool is_key = !is_query && head < a.heads + a.kv_heads;
  T* vec = a.qkv + static_cast<size_t>(token) * a.ld + static_cast<size_t>(head) * a.row_dim;
  float* sums = a.accum != nullptr
                    ? a.accum + static_cast<size_t>(token) * a.ld_accum +
                          static_cast<size_t>(head) * a.row_dim
                    : nullptr;

  int page = -1;
  const int slot = position % a.page_size;
  if (!is_query && a.write_cache) {
    const int table_row = a.request_table_row[a.token_request[token]];
    page = a.block_tables[static_cast<size_t>(table_row) * a.table_stride + position / a.page_size];
    if (page < 0 || page >= a.num_pages) {
      if (lane == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
      page = -1;
    }
  }

  const int real = (is_query || is_key) ? a.head_dim : a.value_dim;
  const int dims = (is_query || is_key) ? a.rotary_dim : (a.value_freq != nullptr ? a.value_dim : 0);
  const int layout = (is_query || is_key) ? a.layout : a.value_layout;
  const float* freq = (is_query || is_key) ? a.freq : a.value_freq;
  const float* weight = is_query ? a.q_norm : (is_key ? a.k_norm : nullptr);
  const int pairs = a.row_dim >> 1;

  float x0[MAX_PAIRS_PER_LANE], x1[MAX_PAIRS_PER_LANE];
  float squares = 0.0f;
#pragma unroll
  for (int i = 0; i < MAX_PAIRS_PER_LANE; ++i) {
    const int p = lane + i * 32;
    if (p >= pairs) continue;
    int i0, i1;
    bool rotate;
    pair_of(p, dims, layout, i0, i1, rotate);
    if (sums != nullptr) {
      // rounded as the projection's own store would have rounded them; cleared for the next use
      x0[i] = hx_to_float<T>(hx_from_float<T>(sums[i0]));
      x1[i] = hx_to_float<T>(hx_from_float<T>(sums[i1]));
      sums[i0] = 0.0f;
      sums[i1] = 0.0f;
    } else {
      x0[i] = hx_to_float<T>(vec[i0]);
      x1[i] = hx_to_float<T>(vec[i1]);
    }
    squares = fmaf(x0[i], x0[i], squares);
    squares = fmaf(x1[i], x1[i], squares);
  }
  float inverse = 1.0f;
  if (weight != nullptr) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      squares += __shfl_xor_sync(0xffffffffu, squares, offset);
    inverse = 1.0f / sqrtf(squares / static_cast<float>(real) + a.eps);
  }
  const float place = static_cast<float>(position);
  const int chunk = hx_cache_chunk(sizeof(T), a.row_dim);
  T* cache = is_key ? a.k_cache : a.v_cache;
  const int kv_head = is_key ? head - a.heads : head - a.heads - a.kv_heads;
#pragma unroll
  for (int i = 0; i < MAX_PAIRS_PER_LANE; ++i) {
    const int p = lane + i * 32;
    if (p >= pairs) continue;
    int i0, i1;
    bool rotate;
    pair_of(p, dims, layout, i0, i1, rotate);
    float u = x0[i], v = x1[i];
    if (weight != nullptr) {
      u = i0 < real ? u * inverse * weight[i0] : 0.0f;
      v = i1 < real ? v * inverse * weight[i1] : 0.0f;
    }
    if (rotate) {
      float s, c;
      sincosf(place * freq[p], &s, &c);
      const float ru = u * c - v * s;
      const float rv = v * c + u * s;
      u = ru;
      v = rv;
    }
    const T tu = hx_from_float<T>(u);
    const T tv = hx_from_float<T>(v);
    if (is_query) {
      vec[i0] = tu;
      vec[i1] = tv;
    } else if (page >= 0) {
      cache[hx_cache_offset(page, kv_head, slot, i0, a.kv_heads, a.page_size, a.row_dim, chunk)] = tu;
      cache[hx_cache_offset(page, kv_head, slot, i1, a.kv_heads, a.page_size, a.row_dim, chunk)] = tv;
    } else if (!a.write_cache) {
      vec[i0] = tu;
      vec[i1] = tv;
    }
  }
}

// out[t][head] turned by -position over its first `dims` coordinates, in place.
template <typename T>
__global__ __launch_bounds__(WARPS * 32) void rotate_back_kernel(
    T* __restrict__ rows, int ld, const int* __restrict__ positions,
    const float* __restrict__ freq, int heads, int row_dim, int dims, int layout) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y * WARPS + (threadIdx.x >> 5);
  if (head >= heads) return;
  T* vec = rows + static_cast<size_t>(token) * ld + static_cast<size_t>(head) * row_dim;
  const float place = -static_cast<float>(positions[token]);
  for (int p = lane; p < (dims >> 1); p += 32) {
    int i0, i1;
    bool rotate;
    pair_of(p, dims, layout, i0, i1, rotate);
    if (!rotate) continue;
    const float u = hx_to_float<T>(vec[i0]);
    const float v = hx_to_float<T>(vec[i1]);
    float s, c;
    sincosf(place * freq[p], &s, &c);
    vec[i0] = hx_from_float<T>(u * c - v * s);
    vec[i1] = hx_from_float<T>(v * c + u * s);
  }
}

}  // namespace

HX_API int hx_norm_rotary_append(void* qkv, int dtype, int ld, float* accum, int ld_accum,
                                 const int* positions, const int* token_request,
                                 const int* request_table_row, const int* block_tables,
                                 int table_stride, void* k_cache, void* v_cache, int write_cache,
                                 const float* freq, const float* value_freq, const float* q_norm,
                                 const float* k_norm, float eps, int tokens, int heads,
                                 int kv_heads, int head_dim, int value_dim, int row_dim,
                                 int rotary_dim, int layout, int value_layout, int page_size,
                                 int num_pages, int* status, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0, "hx_norm_rotary_append: bad sizes");
  HX_REQUIRE(row_dim % 2 == 0 && row_dim <= 64 * MAX_PAIRS_PER_LANE,
             "hx_norm_rotary_append: heads are even and at most %d wide", 64 * MAX_PAIRS_PER_LANE);
  HX_REQUIRE(head_dim <= row_dim && value_dim <= row_dim && value_dim % 2 == 0,
             "hx_norm_rotary_append: head sizes exceed the row width");
  HX_REQUIRE(rotary_dim % 2 == 0 && rotary_dim >= 0 && rotary_dim <= head_dim,
             "hx_norm_rotary_append: rotary_dim must be even and at most head_dim");
  HX_REQUIRE((q_norm == nullptr) == (k_norm == nullptr) && (q_norm == nullptr || eps > 0.0f),
             "hx_norm_rotary_append: the norm has both weights and a positive eps, or neither");
  HX_REQUIRE(!write_cache || (k_cache != nullptr && v_cache != nullptr && block_tables != nullptr),
             "hx_norm_rotary_append: no cache to write to");
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens, (heads + 2 * kv_heads + WARPS - 1) / WARPS);
  if (dtype == HX_F32) {
    RotaryArgs<float> a{static_cast<float*>(qkv), ld, accum, ld_accum, positions, token_request,
                        request_table_row, block_tables, table_stride,
                        static_cast<float*>(k_cache), static_cast<float*>(v_cache), write_cache,
                        freq, value_freq, q_norm, k_norm, eps, heads, kv_heads, head_dim,
                        value_dim, row_dim, rotary_dim, layout, value_layout, page_size, num_pages,
                        status};
    hx_launch(norm_rotary_append_kernel<float>, grid, WARPS * 32, 0, stream, a);
  } else if (dtype == HX_BF16) {
    RotaryArgs<__nv_bfloat16> a{static_cast<__nv_bfloat16*>(qkv), ld, accum, ld_accum, positions,
                                token_request, request_table_row, block_tables, table_stride,
                                static_cast<__nv_bfloat16*>(k_cache),
                                static_cast<__nv_bfloat16*>(v_cache), write_cache, freq,
                                value_freq, q_norm, k_norm, eps, heads, kv_heads, head_dim,
                                value_dim, row_dim, rotary_dim, layout, value_layout, page_size,
                                num_pages, status};
    hx_launch(norm_rotary_append_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, stream, a);
  } else {
    HX_REQUIRE(false, "hx_norm_rotary_append: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_norm_rotary_append");
  return HX_OK;
}

HX_API int hx_rotate_back(void* rows, int dtype, int ld, const int* positions, const float* freq,
                          int tokens, int heads, int row_dim, int dims, int layout,
                          cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && dims % 2 == 0 && dims <= row_dim,
             "hx_rotate_back: bad sizes");
  if (tokens == 0 || dims == 0) return HX_OK;
  const dim3 grid(tokens, (heads + WARPS - 1) / WARPS);
  if (dtype == HX_F32) {
    hx_launch(rotate_back_kernel<float>, grid, WARPS * 32, 0, stream, static_cast<float*>(rows), ld,
              positions, freq, heads, row_dim, dims, layout);
  } else if (dtype == HX_BF16) {
    hx_launch(rotate_back_kernel<__nv_bfloat16>, grid, WARPS * 32, 0, stream,
              static_cast<__nv_bfloat16*>(rows), ld, positions, freq, heads, row_dim, dims, layout);
  } else {
    HX_REQUIRE(false, "hx_rotate_back: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_rotate_back");
  return HX_OK;
}
