// Norms that sit between a product and what follows it, one CTA per token, float32 throughout:
//
//   * hx_norm_residual_add: a sublayer whose output passes an RMS norm BEFORE it joins the
//     residual, x += mult * y / sqrt(mean(y^2) + eps) * w; optionally the updated row is also
//     written in the compute type (the input of a product that reads the residual itself);
//   * hx_biased_normed_rows: what an attention layer does to its fused projection
//     [q | k | v | head gates] before the cache append: biases, ONE RMS norm over all of a
//     token's query coordinates and one over all of its key coordinates (not per head), a
//     factor on the query that grows with the logarithm of the position, values blended with
//     the values an earlier layer computed for the same token, and the sigmoid of the head
//     gates' sums; queries, keys and values leave in rows of row_dim per head (zeros behind
//     the head's own coordinates), keys and values straight into the cache pages;
//   * hx_head_gate: every head of the attention's result times its token's gate;
//   * hx_token_gate: g = gelu_tanh(s) * table[token][offset + c], the gate of a per-token
//     input that is looked up in a table by the token's id.
#include "hx_common.cuh"

namespace {

// A thread holds its share of the row in registers between the two passes (up to
// NORM_ADD_QUADS float4 pieces; wider rows read the rest again), and all of its loads are in
// flight together: with a few dozen tokens the kernel is a handful of round trips to memory.
constexpr int NORM_ADD_THREADS = 256;
constexpr int NORM_ADD_QUADS = 8;       // 256 threads x 8 x 4 floats: rows up to 8,192 wide

template <typename T>
__global__ __launch_bounds__(NORM_ADD_THREADS) void norm_residual_add_kernel(
    float* __restrict__ residual, const float* __restrict__ y, const float* __restrict__ weight,
    float eps, float mult, T* __restrict__ cast_out, int ld_cast, int width) {
  __shared__ float scratch[32];
  hx_pdl_prologue();
  const size_t row = static_cast<size_t>(blockIdx.x) * width;
  T* cast = cast_out == nullptr ? nullptr : cast_out + static_cast<size_t>(blockIdx.x) * ld_cast;
  const bool wide = (width & 3) == 0 &&
                    ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(y) |
                      reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
  if (wide && width <= NORM_ADD_THREADS * NORM_ADD_QUADS * 4) {
    const int quads = width >> 2;
    float4 held[NORM_ADD_QUADS];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NORM_ADD_QUADS; ++i) {
      const int q = threadIdx.x + i * NORM_ADD_THREADS;
      held[i] = q < quads ? *reinterpret_cast<const float4*>(y + row + 4 * q)
                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int i = 0; i < NORM_ADD_QUADS; ++i) {
      sum = fmaf(held[i].x, held[i].x, sum); sum = fmaf(held[i].y, held[i].y, sum);
      sum = fmaf(held[i].z, held[i].z, sum); sum = fmaf(held[i].w, held[i].w, sum);
    }
    const float inverse =
        mult / sqrtf(hx_block_sum(sum, scratch) / static_cast<float>(width) + eps);
    float4 w[NORM_ADD_QUADS], x[NORM_ADD_QUADS];
#pragma unroll
    for (int i = 0; i < NORM_ADD_QUADS; ++i) {
      const int q = threadIdx.x + i * NORM_ADD_THREADS;
      if (q < quads) {
        w[i] = *reinterpret_cast<const float4*>(weight + 4 * q);
        x[i] = *reinterpret_cast<const float4*>(residual + row + 4 * q);
      }
    }
#pragma unroll
    for (int i = 0; i < NORM_ADD_QUADS; ++i) {
      const int q = threadIdx.x + i * NORM_ADD_THREADS;
      if (q >= quads) continue;
      x[i].x = fmaf(held[i].x * inverse, w[i].x, x[i].x);
      x[i].y = fmaf(held[i].y * inverse, w[i].y, x[i].y);
      x[i].z = fmaf(held[i].z * inverse, w[i].z, x[i].z);
      x[i].w = fmaf(held[i].w * inverse, w[i].w, x[i].w);
      *reinterpret_cast<float4*>(residual + row + 4 * q) = x[i];
      if (cast != nullptr) {
        cast[4 * q] = hx_from_float<T>(x[i].x);
        cast[4 * q + 1] = hx_from_float<T>(x[i].y);
        cast[4 * q + 2] = hx_from_float<T>(x[i].z);
        cast[4 * q + 3] = hx_from_float<T>(x[i].w);
      }
    }
    return;
  }
  float sum = 0.0f;
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += blockDim.x) sum = fmaf(y[row + c], y[row + c], sum);
  const float inverse =
      mult / sqrtf(hx_block_sum(sum, scratch) / static_cast<float>(width) + eps);
#pragma unroll 4
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = fmaf(y[row + c] * inverse, weight[c], residual[row + c]);
    residual[row + c] = x;
    if (cast != nullptr) cast[c] = hx_from_float<T>(x);
  }
}

template <typename T>
struct NormedRowsArgs {
  float* projected;            // [tokens, ld_projected]: q | k | v | head gates
  int ld_projected;
  int clear;                   // 1: the buffer is an accumulator, leave it zero
  const float* q_bias;         // [heads * head_dim] or null
  const float* k_bias;         // [kv_heads * head_dim] or null
  const float* v_bias;         // [kv_heads * value_dim] or null
  const float* q_weight;       // [heads * head_dim] or null: no norm
  const float* k_weight;       // [kv_heads * head_dim] or null
  float eps;
  const int* positions;
  float temp_coef;             // query factor 1 + coef * ln(floor((p + 1) / every) + 1)
  int temp_every;              // 0: none
  int value_mix;               // 0: none; 1: this layer's values are kept as the source;
                               // 2: v <- (1 - lambda) v + lambda source
  float lambda;
  float* value_source;         // [tokens, kv_heads * value_dim]
  T* rows;                     // [tokens, ld_rows]: heads | kv_heads | kv_heads rows of row_dim
  int ld_rows;
  float* gates;                // [tokens, heads]: sigmoid of the gate sums; null: none
  int heads, kv_heads, head_dim, value_dim, row_dim;
  // The cache append (k_cache null: keys and values go to `rows` instead): the token's keys
  // and values are written to slot position % page_size of the page its request's block table
  // names for position / page_size, in the cache's layout (hx_cache_offset).
  const int* token_request;
  const int* request_table_row;
  const int* block_tables;
  int table_stride;
  T* k_cache;
  T* v_cache;
  int page_size, num_pages;
  int* status;
};

// floor(n / d) for n * d < 2^32 as one multiplication: m = ceil(2^32 / d) (d > 1).
struct FastDivisor {
  unsigned d, m;
  __device__ __forceinline__ int quotient(int n) const {
    return d == 1u ? n : static_cast<int>(__umulhi(static_cast<unsigned>(n), m));
  }
};
inline FastDivisor fast_divisor(int d) {
  FastDivisor f;
  f.d = static_cast<unsigned>(d);
  f.m = d > 1 ? static_cast<unsigned>(((1ull << 32) + d - 1) / d) : 0u;
  return f;
}

// A thread keeps its share of the token's queries and keys in registers between the pass that
// sums their squares and the pass that writes them (NORMED_Q_HELD and NORMED_K_HELD numbers a
// thread; wider projections read the sums again), so all of its loads of a pass are in flight
// together and a token costs a handful of round trips.
constexpr int NORMED_ROWS_THREADS = 512;
constexpr int NORMED_Q_HELD = 16;       // 512 threads: queries up to 8,192 numbers a token
constexpr int NORMED_K_HELD = 8;        // keys up to 4,096

template <typename T>
__global__ __launch_bounds__(NORMED_ROWS_THREADS) void biased_normed_rows_kernel(
    const NormedRowsArgs<T> a, const FastDivisor by_dim, const FastDivisor by_value_dim) {
  __shared__ float scratch[32];
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int tid = threadIdx.x, threads = blockDim.x;
  float* in = a.projected + static_cast<size_t>(token) * a.ld_projected;
  T* out = a.rows + static_cast<size_t>(token) * a.ld_rows;
  const int D = a.head_dim, R = a.row_dim, E = a.value_dim;
  const int q_size = a.heads * D;
  const int k_size = a.kv_heads * D;
  const int v_size = a.kv_heads * E;
  const float* k_in = in + q_size;
  const float* v_in = k_in + k_size;
  const bool held = q_size <= NORMED_Q_HELD * threads && k_size <= NORMED_K_HELD * threads;

  // ---- where keys and values go: the token's slot of its page, or behind the queries (a
  // chain of four dependent loads, started first so that it runs beside the row's own loads)
  const bool append = a.k_cache != nullptr;
  int page = -1, slot = 0;
  if (append) {
    const int position = a.positions[token];
    const int table_row = a.request_table_row[a.token_request[token]];
    page = a.block_tables[static_cast<size_t>(table_row) * a.table_stride + position / a.page_size];
    slot = position % a.page_size;
    if (page < 0 || page >= a.num_pages) {
      if (tid == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
      page = -1;
    }
  }
  // ---- biased sums, and the sums of their squares
  float q[NORMED_Q_HELD], k[NORMED_K_HELD];
  float q_sum = 0.0f, k_sum = 0.0f;
  if (held) {
#pragma unroll
    for (int i = 0; i < NORMED_Q_HELD; ++i) {
      const int c = tid + i * threads;
      q[i] = c < q_size ? in[c] + (a.q_bias != nullptr ? a.q_bias[c] : 0.0f) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < NORMED_K_HELD; ++i) {
      const int c = tid + i * threads;
      k[i] = c < k_size ? k_in[c] + (a.k_bias != nullptr ? a.k_bias[c] : 0.0f) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < NORMED_Q_HELD; ++i) q_sum = fmaf(q[i], q[i], q_sum);
#pragma unroll
    for (int i = 0; i < NORMED_K_HELD; ++i) k_sum = fmaf(k[i], k[i], k_sum);
  } else {
#pragma unroll 4
    for (int c = tid; c < q_size; c += threads) {
      const float v = in[c] + (a.q_bias != nullptr ? a.q_bias[c] : 0.0f);
      q_sum = fmaf(v, v, q_sum);
    }
#pragma unroll 4
    for (int c = tid; c < k_size; c += threads) {
      const float v = k_in[c] + (a.k_bias != nullptr ? a.k_bias[c] : 0.0f);
      k_sum = fmaf(v, v, k_sum);
    }
  }
  float q_factor = 1.0f, k_factor = 1.0f;
  if (a.q_weight != nullptr)
    q_factor = 1.0f / sqrtf(hx_block_sum(q_sum, scratch) / static_cast<float>(q_size) + a.eps);
  if (a.k_weight != nullptr)
    k_factor = 1.0f / sqrtf(hx_block_sum(k_sum, scratch) / static_cast<float>(k_size) + a.eps);
  if (a.temp_every > 0)
    q_factor *= 1.0f + a.temp_coef *
        logf(static_cast<float>((a.positions[token] + 1) / a.temp_every) + 1.0f);

  const int chunk = hx_cache_chunk(sizeof(T), R);
  T* key_rows = out + a.heads * R;
  T* value_rows = key_rows + a.kv_heads * R;
  auto put = [&](T* cache, T* rows, int head, int d, float value) {
    if (!append) {
      rows[head * R + d] = hx_from_float<T>(value);
    } else if (page >= 0) {
      cache[hx_cache_offset(page, head, slot, d, a.kv_heads, a.page_size, R, chunk)] =
          hx_from_float<T>(value);
    }
  };

  // ---- queries and keys: element c of the projection is coordinate c % D of head c / D
  auto write_q = [&](int c, float value) {
    const int head = by_dim.quotient(c);
    if (a.q_weight != nullptr) value *= a.q_weight[c];
    out[head * R + (c - head * D)] = hx_from_float<T>(value * q_factor);
  };
  auto write_k = [&](int c, float value) {
    const int head = by_dim.quotient(c);
    if (a.k_weight != nullptr) value *= a.k_weight[c];
    put(a.k_cache, key_rows, head, c - head * D, value * k_factor);
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < NORMED_Q_HELD; ++i) {
      const int c = tid + i * threads;
      if (c < q_size) write_q(c, q[i]);
    }
#pragma unroll
    for (int i = 0; i < NORMED_K_HELD; ++i) {
      const int c = tid + i * threads;
      if (c < k_size) write_k(c, k[i]);
    }
  } else {
#pragma unroll 4
    for (int c = tid; c < q_size; c += threads)
      write_q(c, in[c] + (a.q_bias != nullptr ? a.q_bias[c] : 0.0f));
#pragma unroll 4
    for (int c = tid; c < k_size; c += threads)
      write_k(c, k_in[c] + (a.k_bias != nullptr ? a.k_bias[c] : 0.0f));
  }
  // ---- values, kept for or blended with another layer's
  float* source = a.value_source == nullptr ? nullptr
                                            : a.value_source + static_cast<size_t>(token) * v_size;
#pragma unroll 4
  for (int c = tid; c < v_size; c += threads) {
    float v = v_in[c] + (a.v_bias != nullptr ? a.v_bias[c] : 0.0f);
    if (a.value_mix == 1) {
      source[c] = v;
    } else if (a.value_mix == 2) {
      v = (1.0f - a.lambda) * v + a.lambda * source[c];
    }
    const int head = by_value_dim.quotient(c);
    put(a.v_cache, value_rows, head, c - head * E, v);
  }
  // ---- zeros behind a head's own coordinates
  if (R > D) {
    const int pad = R - D;
    for (int p = tid; p < (a.heads + a.kv_heads) * pad; p += threads) {
      const int head = p / pad, d = D + p - head * pad;
      if (head < a.heads) {
        out[head * R + d] = hx_from_float<T>(0.0f);
      } else {
        put(a.k_cache, key_rows, head - a.heads, d, 0.0f);
      }
    }
  }
  if (R > E) {
    const int pad = R - E;
    for (int p = tid; p < a.kv_heads * pad; p += threads) {
      const int head = p / pad;
      put(a.v_cache, value_rows, head, E + p - head * pad, 0.0f);
    }
  }
  if (a.gates != nullptr)
    for (int h = tid; h < a.heads; h += threads)
      a.gates[static_cast<size_t>(token) * a.heads + h] =
          hx_sigmoid(in[q_size + k_size + v_size + h]);
  if (a.clear) {
    __syncthreads();
    const int used = q_size + k_size + v_size + (a.gates != nullptr ? a.heads : 0);
    for (int c = tid; c < used; c += threads) in[c] = 0.0f;
  }
}

// The same four numbers at a time, for projections whose heads, rows and strides are multiples of
// four and whose buffers are 16-byte aligned (the host checks): a load, a bias, a weight and a
// store serve four numbers, and their head is worked out once.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ float4 scale4(float4 a, float4 w, float f) {
  return make_float4(a.x * w.x * f, a.y * w.y * f, a.z * w.z * f, a.w * w.w * f);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  uint2 packed;
  *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = packed;
}

template <typename T>
__global__ __launch_bounds__(NORMED_ROWS_THREADS) void biased_normed_rows_quads_kernel(
    const NormedRowsArgs<T> a, const FastDivisor by_dim, const FastDivisor by_value_dim) {
  constexpr int Q_QUADS = NORMED_Q_HELD / 4, K_QUADS = NORMED_K_HELD / 4;
  __shared__ float scratch[32];
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int tid = threadIdx.x, threads = blockDim.x;
  float* in = a.projected + static_cast<size_t>(token) * a.ld_projected;
  T* out = a.rows + static_cast<size_t>(token) * a.ld_rows;
  const int D = a.head_dim, R = a.row_dim, E = a.value_dim;
  const int q_size = a.heads * D;
  const int k_size = a.kv_heads * D;
  const int v_size = a.kv_heads * E;
  float* k_in = in + q_size;
  float* v_in = k_in + k_size;
  const bool held = q_size <= NORMED_Q_HELD * threads && k_size <= NORMED_K_HELD * threads;
  const float4 ones = make_float4(1.0f, 1.0f, 1.0f, 1.0f);

  // where keys and values go (see biased_normed_rows_kernel)
  const bool append = a.k_cache != nullptr;
  int page = -1, slot = 0;
  if (append) {
    const int position = a.positions[token];
    const int table_row = a.request_table_row[a.token_request[token]];
    page = a.block_tables[static_cast<size_t>(table_row) * a.table_stride + position / a.page_size];
    slot = position % a.page_size;
    if (page < 0 || page >= a.num_pages) {
      if (tid == 0 && a.status != nullptr) atomicOr(a.status, HX_FLAG_BAD_PAGE);
      page = -1;
    }
  }
  auto biased_q = [&](int c) {
    const float4 v = load4(in + c);
    return a.q_bias != nullptr ? add4(v, load4(a.q_bias + c)) : v;
  };
  auto biased_k = [&](int c) {
    const float4 v = load4(k_in + c);
    return a.k_bias != nullptr ? add4(v, load4(a.k_bias + c)) : v;
  };
  auto squares = [](float4 v, float sum) {
    sum = fmaf(v.x, v.x, sum); sum = fmaf(v.y, v.y, sum);
    sum = fmaf(v.z, v.z, sum); return fmaf(v.w, v.w, sum);
  };
  float4 q[Q_QUADS], k[K_QUADS];
  float q_sum = 0.0f, k_sum = 0.0f;
  if (held) {
#pragma unroll
    for (int i = 0; i < Q_QUADS; ++i) {
      const int c = 4 * (tid + i * threads);
      q[i] = c < q_size ? biased_q(c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int i = 0; i < K_QUADS; ++i) {
      const int c = 4 * (tid + i * threads);
      k[i] = c < k_size ? biased_k(c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int i = 0; i < Q_QUADS; ++i) q_sum = squares(q[i], q_sum);
#pragma unroll
    for (int i = 0; i < K_QUADS; ++i) k_sum = squares(k[i], k_sum);
  } else {
    for (int c = 4 * tid; c < q_size; c += 4 * threads) q_sum = squares(biased_q(c), q_sum);
    for (int c = 4 * tid; c < k_size; c += 4 * threads) k_sum = squares(biased_k(c), k_sum);
  }
  float q_factor = 1.0f, k_factor = 1.0f;
  if (a.q_weight != nullptr)
    q_factor = 1.0f / sqrtf(hx_block_sum(q_sum, scratch) / static_cast<float>(q_size) + a.eps);
  if (a.k_weight != nullptr)
    k_factor = 1.0f / sqrtf(hx_block_sum(k_sum, scratch) / static_cast<float>(k_size) + a.eps);
  if (a.temp_every > 0)
    q_factor *= 1.0f + a.temp_coef *
        logf(static_cast<float>((a.positions[token] + 1) / a.temp_every) + 1.0f);

  const int chunk = hx_cache_chunk(sizeof(T), R);      // a multiple of four here
  T* key_rows = out + a.heads * R;
  T* value_rows = key_rows + a.kv_heads * R;
  auto put4 = [&](T* cache, T* rows, int head, int d, float4 value) {
    if (!append) {
      store4(rows + head * R + d, value);
    } else if (page >= 0) {
      store4(cache + hx_cache_offset(page, head, slot, d, a.kv_heads, a.page_size, R, chunk), value);
    }
  };
  auto write_q = [&](int c, float4 value) {
    const int head = by_dim.quotient(c);
    store4(out + head * R + (c - head * D),
           scale4(value, a.q_weight != nullptr ? load4(a.q_weight + c) : ones, q_factor));
  };
  auto write_k = [&](int c, float4 value) {
    const int head = by_dim.quotient(c);
    put4(a.k_cache, key_rows, head, c - head * D,
         scale4(value, a.k_weight != nullptr ? load4(a.k_weight + c) : ones, k_factor));
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < Q_QUADS; ++i) {
      const int c = 4 * (tid + i * threads);
      if (c < q_size) write_q(c, q[i]);
    }
#pragma unroll
    for (int i = 0; i < K_QUADS; ++i) {
      const int c = 4 * (tid + i * threads);
      if (c < k_size) write_k(c, k[i]);
    }
  } else {
    for (int c = 4 * tid; c < q_size; c += 4 * threads) write_q(c, biased_q(c));
    for (int c = 4 * tid; c < k_size; c += 4 * threads) write_k(c, biased_k(c));
  }
  float* source = a.value_source == nullptr ? nullptr
                                            : a.value_source + static_cast<size_t>(token) * v_size;
  for (int c = 4 * tid; c < v_size; c += 4 * threads) {
    float4 v = load4(v_in + c);
    if (a.v_bias != nullptr) v = add4(v, load4(a.v_bias + c));
    if (a.value_mix == 1) {
      store4(source + c, v);
    } else if (a.value_mix == 2) {
      const float4 s = load4(source + c);
      const float keep = 1.0f - a.lambda;
      v = make_float4(keep * v.x + a.lambda * s.x, keep * v.y + a.lambda * s.y,
                      keep * v.z + a.lambda * s.z, keep * v.w + a.lambda * s.w);
    }
    const int head = by_value_dim.quotient(c);
    put4(a.v_cache, value_rows, head, c - head * E, v);
  }
  // zeros behind a head's own coordinates, four at a time
  const float4 zeros = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  if (R > D) {
    const int pad = (R - D) >> 2;
    for (int p = tid; p < (a.heads + a.kv_heads) * pad; p += threads) {
      const int head = p / pad, d = D + 4 * (p - head * pad);
      if (head < a.heads) {
        store4(out + head * R + d, zeros);
      } else {
        put4(a.k_cache, key_rows, head - a.heads, d, zeros);
      }
    }
  }
  if (R > E) {
    const int pad = (R - E) >> 2;
    for (int p = tid; p < a.kv_heads * pad; p += threads) {
      const int head = p / pad;
      put4(a.v_cache, value_rows, head, E + 4 * (p - head * pad), zeros);
    }
  }
  if (a.gates != nullptr)
    for (int h = tid; h < a.heads; h += threads)
      a.gates[static_cast<size_t>(token) * a.heads + h] =
          hx_sigmoid(in[q_size + k_size + v_size + h]);
  if (a.clear) {
    __syncthreads();
    const int used = q_size + k_size + v_size + (a.gates != nullptr ? a.heads : 0);
    for (int c = tid; c < used; c += threads) in[c] = 0.0f;
  }
}

// grid (tokens, ceil(heads / 8)): a warp takes a head
constexpr int HEAD_GATE_WARPS = 8;

template <typename T>
__global__ __launch_bounds__(HEAD_GATE_WARPS * 32) void head_gate_kernel(
    T* __restrict__ context, int ld_context, const float* __restrict__ gates, int heads,
    int row_dim) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int head = blockIdx.y * HEAD_GATE_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (head >= heads) return;
  const float gate = gates[static_cast<size_t>(token) * heads + head];
  T* row = context + static_cast<size_t>(token) * ld_context + head * row_dim;
#pragma unroll 4
  for (int c = lane; c < row_dim; c += 32) row[c] = hx_from_float<T>(hx_to_float<T>(row[c]) * gate);
}

// grid (tokens)
template <typename T>
__global__ __launch_bounds__(128) void token_gate_kernel(
    float* __restrict__ sums, int ld_sums, int clear, const T* __restrict__ table, int ld_table,
    int offset, int vocab, const int* __restrict__ token_ids, T* __restrict__ out, int ld_out,
    int dim, int* __restrict__ status) {
  hx_pdl_prologue();
  const int token = blockIdx.x;
  int id = token_ids[token];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, HX_FLAG_BAD_TOKEN);
    id = 0;
  }
  float* s = sums + static_cast<size_t>(token) * ld_sums;
  const T* e = table + static_cast<size_t>(id) * ld_table + offset;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    out[static_cast<size_t>(token) * ld_out + c] =
        hx_from_float<T>(hx_gelu_tanh(s[c]) * hx_to_float<T>(e[c]));
    if (clear) s[c] = 0.0f;
  }
}

}  // namespace

// residual[:tokens] += mult * y / sqrt(mean(y^2) + eps) * weight, float32 rows [tokens, width]
// contiguous; cast_out (may be null): the updated rows in `dtype`, row stride ld_cast.
HX_API int hx_norm_residual_add(float* residual, const float* y, const float* weight, float eps,
                                float mult, void* cast_out, int ld_cast, int dtype, int tokens,
                                int width, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && width > 0 && eps > 0.0f, "hx_norm_residual_add: bad sizes");
  HX_REQUIRE(cast_out == nullptr || ld_cast >= width, "hx_norm_residual_add: bad stride");
  if (tokens == 0) return HX_OK;
  if (dtype == HX_F32) {
    hx_launch(norm_residual_add_kernel<float>, dim3(tokens), NORM_ADD_THREADS, 0, stream, residual, y, weight,
              eps, mult, static_cast<float*>(cast_out), ld_cast, width);
  } else if (dtype == HX_BF16) {
    hx_launch(norm_residual_add_kernel<__nv_bfloat16>, dim3(tokens), NORM_ADD_THREADS, 0, stream, residual, y,
              weight, eps, mult, static_cast<__nv_bfloat16*>(cast_out), ld_cast, width);
  } else {
    HX_REQUIRE(false, "hx_norm_residual_add: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_norm_residual_add");
  return HX_OK;
}

// projected float32 [tokens, ld_projected] = [heads * head_dim | kv_heads * head_dim | kv_heads *
// value_dim | heads gate sums (when gates is not null)]; rows [tokens, ld_rows] in `dtype` =
// [heads | kv_heads | kv_heads] rows of row_dim; with k_cache the keys and values go to the
// token's slot of its request's pages instead (the cache append of the other position
// kernels) and only the queries to `rows`.  See NormedRowsArgs for the rest.
HX_API int hx_biased_normed_rows(float* projected, int ld_projected, int clear,
                                 const float* q_bias, const float* k_bias, const float* v_bias,
                                 const float* q_weight, const float* k_weight, float eps,
                                 const int* positions, float temp_coef, int temp_every,
                                 int value_mix, float lambda, float* value_source, void* rows,
                                 int ld_rows, float* gates, int dtype, int tokens, int heads,
                                 int kv_heads, int head_dim, int value_dim, int row_dim,
                                 const int* token_request, const int* request_table_row,
                                 const int* block_tables, int table_stride, void* k_cache,
                                 void* v_cache, int page_size, int num_pages, int* status,
                                 cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && value_dim > 0 &&
                 row_dim >= head_dim && row_dim >= value_dim,
             "hx_biased_normed_rows: bad sizes");
  HX_REQUIRE(ld_projected >= heads * head_dim + kv_heads * (head_dim + value_dim) +
                                 (gates != nullptr ? heads : 0) &&
                 ld_rows >= (heads + (k_cache == nullptr ? 2 * kv_heads : 0)) * row_dim,
             "hx_biased_normed_rows: bad strides");
  HX_REQUIRE(k_cache == nullptr ||
                 (v_cache != nullptr && token_request != nullptr && request_table_row != nullptr &&
                  block_tables != nullptr && positions != nullptr && page_size > 0 &&
                  num_pages > 0 && table_stride > 0),
             "hx_biased_normed_rows: the cache append needs the step's description");
  HX_REQUIRE(value_mix >= 0 && value_mix <= 2 && (value_mix == 0 || value_source != nullptr),
             "hx_biased_normed_rows: value mixing needs its source buffer");
  HX_REQUIRE(temp_every >= 0 && (temp_every == 0 || positions != nullptr) &&
                 ((q_weight == nullptr && k_weight == nullptr) || eps > 0.0f),
             "hx_biased_normed_rows: bad constants");
  if (tokens == 0) return HX_OK;
  HX_REQUIRE(static_cast<long long>(heads) * head_dim < 65536 &&
                 static_cast<long long>(kv_heads) * value_dim < 65536 && row_dim < 65536,
             "hx_biased_normed_rows: projections of 65,536 numbers and more are not supported");
  const FastDivisor by_dim = fast_divisor(head_dim), by_value_dim = fast_divisor(value_dim);
  // four numbers at a time where every piece starts on a 16-byte boundary (8 for bfloat16 rows)
  auto aligned = [](const void* p, uintptr_t to) {
    return p == nullptr || (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0;
  };
  const uintptr_t row_bytes = dtype == HX_F32 ? 16 : 8;
  const bool quads =
      head_dim % 4 == 0 && value_dim % 4 == 0 && row_dim % 4 == 0 && ld_projected % 4 == 0 &&
      ld_rows % 4 == 0 && aligned(projected, 16) && aligned(q_bias, 16) && aligned(k_bias, 16) &&
      aligned(v_bias, 16) && aligned(q_weight, 16) && aligned(k_weight, 16) &&
      aligned(value_source, 16) && aligned(rows, row_bytes) && aligned(k_cache, 16) &&
      aligned(v_cache, 16);
  if (dtype == HX_F32) {
    NormedRowsArgs<float> a{projected, ld_projected, clear, q_bias, k_bias, v_bias, q_weight,
                            k_weight, eps, positions, temp_coef, temp_every, value_mix, lambda,
                            value_source, static_cast<float*>(rows), ld_rows, gates, heads,
                            kv_heads, head_dim, value_dim, row_dim, token_request,
                            request_table_row, block_tables, table_stride,
                            static_cast<float*>(k_cache), static_cast<float*>(v_cache), page_size,
                            num_pages, status};
    hx_launch(quads ? biased_normed_rows_quads_kernel<float> : biased_normed_rows_kernel<float>,
              dim3(tokens), NORMED_ROWS_THREADS, 0, stream, a, by_dim, by_value_dim);
  } else if (dtype == HX_BF16) {
    NormedRowsArgs<__nv_bfloat16> a{projected, ld_projected, clear, q_bias, k_bias, v_bias,
                                    q_weight, k_weight, eps, positions, temp_coef, temp_every,
                                    value_mix, lambda, value_source,
                                    static_cast<__nv_bfloat16*>(rows), ld_rows, gates, heads,
                                    kv_heads, head_dim, value_dim, row_dim, token_request,
                                    request_table_row, block_tables, table_stride,
                                    static_cast<__nv_bfloat16*>(k_cache),
                                    static_cast<__nv_bfloat16*>(v_cache), page_size, num_pages,
                                    status};
    hx_launch(quads ? biased_normed_rows_quads_kernel<__nv_bfloat16>
                    : biased_normed_rows_kernel<__nv_bfloat16>,
              dim3(tokens), NORMED_ROWS_THREADS, 0, stream, a, by_dim, by_value_dim);
  } else {
    HX_REQUIRE(false, "hx_biased_normed_rows: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_biased_normed_rows");
  return HX_OK;
}

// context[t][h * row_dim + c] *= gates[t][h]; context in `dtype`, gates float32 [tokens, heads].
HX_API int hx_head_gate(void* context, int ld_context, const float* gates, int dtype, int tokens,
                        int heads, int row_dim, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && heads <= 65535 * HEAD_GATE_WARPS && row_dim > 0 &&
                 ld_context >= heads * row_dim, "hx_head_gate: bad sizes");
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens, (heads + HEAD_GATE_WARPS - 1) / HEAD_GATE_WARPS);
  if (dtype == HX_F32) {
    hx_launch(head_gate_kernel<float>, grid, HEAD_GATE_WARPS * 32, 0, stream,
              static_cast<float*>(context), ld_context, gates, heads, row_dim);
  } else if (dtype == HX_BF16) {
    hx_launch(head_gate_kernel<__nv_bfloat16>, grid, HEAD_GATE_WARPS * 32, 0, stream,
              static_cast<__nv_bfloat16*>(context), ld_context, gates, heads, row_dim);
  } else {
    HX_REQUIRE(false, "hx_head_gate: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_head_gate");
  return HX_OK;
}

// out[t][c] = gelu_tanh(sums[t][c]) * table[token_ids[t]][offset + c] for c < dim; sums float32
// (cleared when `clear`), table and out in `dtype`.
HX_API int hx_token_gate(float* sums, int ld_sums, int clear, const void* table, int ld_table,
                         int offset, int vocab, const int* token_ids, void* out, int ld_out,
                         int dtype, int tokens, int dim, int* status, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && dim > 0 && ld_sums >= dim && ld_out >= dim && offset >= 0 &&
                 ld_table >= offset + dim && vocab > 0, "hx_token_gate: bad sizes");
  if (tokens == 0) return HX_OK;
  if (dtype == HX_F32) {
    hx_launch(token_gate_kernel<float>, dim3(tokens), 128, 0, stream, sums, ld_sums, clear,
              static_cast<const float*>(table), ld_table, offset, vocab, token_ids,
              static_cast<float*>(out), ld_out, dim, status);
  } else if (dtype == HX_BF16) {
    hx_launch(token_gate_kernel<__nv_bfloat16>, dim3(tokens), 128, 0, stream, sums, ld_sums,
              clear, static_cast<const __nv_bfloat16*>(table), ld_table, offset, vocab, token_ids,
              static_cast<__nv_bfloat16*>(out), ld_out, dim, status);
  } else {
    HX_REQUIRE(false, "hx_token_gate: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_token_gate");
  return HX_OK;
}
