// Attention over a cached latent: what runs between the products of a latent-attention mixer.
//
// A token's down-projection holds [query latent | key/value latent | shared rotated key part].
// Both latents are RMS-normed with a weight; keys and values of all heads are functions of the
// one key/value latent c, so only c and the rotated part are cached: every head attends to the
// one cached row [c | rot(kr)] with the query [Wuk_h' q_h | rot(qr_h)] (the up-projection of
// the keys moved to the query's side) and reads the value row [c]; the head's value
// up-projection follows the weighted sum.  Scores are the same numbers as with per-head keys.
//
//   * hx_latent_prepare: both norms; the query latent goes to its own buffer in the compute
//     type; the key row [c | rot(kr) | 0...] and the value row [c | 0...] go to the token's row
//     of the attention's buffer (width row_dim each);
//   * hx_latent_queries: the rotated part of every head's query, turned by the position, behind
//     the head's latent part in that buffer, zeros to the row's end.
//
// Norms, angles and rotations are float32 (the float32 engine takes the angle in double).
// `amplitude` multiplies sine and cosine (1 unless the frequencies are stretched for contexts
// beyond the trained length; the stretched frequencies themselves come from the host).
#include "hx_common.cuh"

namespace {

template <bool EXACT>
__device__ __forceinline__ void angle_of(int position, int pair, const float* freq,
                                         const double* freq_exact, float& sine, float& cosine) {
  if (EXACT) {
    double s, c;
    sincos(static_cast<double>(position) * freq_exact[pair], &s, &c);
    sine = static_cast<float>(s);
    cosine = static_cast<float>(c);
  } else {
    sincosf(static_cast<float>(position) * freq[pair], &sine, &cosine);
  }
}

// coordinate e of `rot` coordinates, of which the first `dims` are rotated in pairs
template <bool EXACT, typename Load>
__device__ __forceinline__ float rotated(Load load, int e, int dims, int layout, int position,
                                         const float* freq, const double* freq_exact,
                                         float amplitude) {
  const float x = load(e);
  if (e >= dims) return x;
  int pair, partner;
  bool leads;
  if (layout == 0) {
    pair = e >> 1; partner = e ^ 1; leads = (e & 1) == 0;
  } else {
    const int half = dims >> 1;
    leads = e < half;
    pair = leads ? e : e - half;
    partner = leads ? e + half : e - half;
  }
  float sine, cosine;
  angle_of<EXACT>(position, pair, freq, freq_exact, sine, cosine);
  sine *= amplitude;        // 1 unless the frequencies are stretched
  cosine *= amplitude;
  const float y = load(partner);
  return leads ? x * cosine - y * sine : x * cosine + y * sine;
}

template <typename T>
struct LatentPrepareArgs {
  const float* down;        // [tokens, ld_down]: q_rank | kv_rank | rot
  int ld_down;
  const float* q_weight;    // [q_rank]
  const float* kv_weight;   // [kv_rank]
  float eps;
  const int* positions;
  const float* freq;
  const double* freq_exact;
  int rotary_dims, layout;
  T* query_latent;          // [tokens, ld_latent]
  int ld_latent;
  T* rows;                  // [tokens, ld_rows]: the key row at key_offset, the value row behind it
  int ld_rows, key_offset;
  int q_rank, kv_rank, rot, row_dim;
  float amplitude;          // factor on sine and cosine
};

template <typename T>
__global__ __launch_bounds__(128) void latent_prepare_kernel(const LatentPrepareArgs<T> a) {
  constexpr bool EXACT = sizeof(T) == 4;
  __shared__ float scratch[32];
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const float* down = a.down + static_cast<size_t>(token) * a.ld_down;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < a.q_rank; c += blockDim.x) sum = fmaf(down[c], down[c], sum);
  const float q_inverse =
      1.0f / sqrtf(hx_block_sum(sum, scratch) / static_cast<float>(a.q_rank) + a.eps);
  T* latent = a.query_latent + static_cast<size_t>(token) * a.ld_latent;
  for (int c = threadIdx.x; c < a.q_rank; c += blockDim.x)
    latent[c] = hx_from_float<T>(down[c] * q_inverse * a.q_weight[c]);
  const float* kv = down + a.q_rank;
  sum = 0.0f;
  for (int c = threadIdx.x; c < a.kv_rank; c += blockDim.x) sum = fmaf(kv[c], kv[c], sum);
  const float kv_inverse =
      1.0f / sqrtf(hx_block_sum(sum, scratch) / static_cast<float>(a.kv_rank) + a.eps);
  T* key = a.rows + static_cast<size_t>(token) * a.ld_rows + a.key_offset;
  T* value = key + a.row_dim;
  const float* shared_part = kv + a.kv_rank;
  const int position = a.positions[token];
  for (int c = threadIdx.x; c < a.row_dim; c += blockDim.x) {
    float k = 0.0f, v = 0.0f;
    if (c < a.kv_rank) {
      // keys and values read the latent as it is cached: one rounding
      k = v = hx_to_float<T>(hx_from_float<T>(kv[c] * kv_inverse * a.kv_weight[c]));
    } else if (c < a.kv_rank + a.rot) {
      k = rotated<EXACT>([&](int e) { return shared_part[e]; }, c - a.kv_rank, a.rotary_dims,
                         a.layout, position, a.freq, a.freq_exact, a.amplitude);
    }
    key[c] = hx_from_float<T>(k);
    value[c] = hx_from_float<T>(v);
  }
}

// grid (tokens, heads): q_rot [tokens, ld_q] holds heads * rot rotated-part coordinates from
// column rot_offset on
template <typename T>
__global__ __launch_bounds__(64) void latent_queries_kernel(
    const T* __restrict__ q, int ld_q, int rot_offset, T* __restrict__ rows, int ld_rows,
    const int* __restrict__ positions, const float* __restrict__ freq,
    const double* __restrict__ freq_exact, int rotary_dims, int layout, int kv_rank, int rot,
    int row_dim, float amplitude) {
  constexpr bool EXACT = sizeof(T) == 4;
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int head = blockIdx.y;
  const T* part = q + static_cast<size_t>(token) * ld_q + rot_offset + head * rot;
  T* row = rows + static_cast<size_t>(token) * ld_rows + head * row_dim;
  const int position = positions[token];
  for (int c = kv_rank + threadIdx.x; c < row_dim; c += blockDim.x) {
    float v = 0.0f;
    if (c < kv_rank + rot)
      v = rotated<EXACT>([&](int e) { return hx_to_float<T>(part[e]); }, c - kv_rank, rotary_dims,
                         layout, position, freq, freq_exact, amplitude);
    row[c] = hx_from_float<T>(v);
  }
}

}  // namespace

HX_API int hx_latent_prepare(const float* down, int ld_down, const float* q_weight,
                             const float* kv_weight, float eps, const int* positions,
                             const float* freq, const double* freq_exact, int rotary_dims,
                             int layout, void* query_latent, int ld_latent, void* rows, int ld_rows,
                             int key_offset, int dtype, int tokens, int q_rank, int kv_rank, int rot,
                             int row_dim, float amplitude, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && q_rank > 0 && kv_rank > 0 && rot >= 0 && row_dim >= kv_rank + rot,
             "hx_latent_prepare: bad sizes");
  HX_REQUIRE(ld_down >= q_rank + kv_rank + rot && ld_latent >= q_rank &&
                 ld_rows >= key_offset + 2 * row_dim,
             "hx_latent_prepare: bad strides");
  HX_REQUIRE(rotary_dims >= 0 && rotary_dims <= rot && rotary_dims % 2 == 0 && eps > 0.0f,
             "hx_latent_prepare: %d of %d coordinates rotated", rotary_dims, rot);
  HX_REQUIRE(rotary_dims == 0 || (freq != nullptr && (dtype != HX_F32 || freq_exact != nullptr)),
             "hx_latent_prepare: frequencies missing");
  if (tokens == 0) return HX_OK;
  if (dtype == HX_F32) {
    LatentPrepareArgs<float> a{down, ld_down, q_weight, kv_weight, eps, positions, freq, freq_exact,
                               rotary_dims, layout, static_cast<float*>(query_latent), ld_latent,
                               static_cast<float*>(rows), ld_rows, key_offset, q_rank, kv_rank, rot,
                               row_dim, amplitude};
    hx_launch(latent_prepare_kernel<float>, dim3(tokens), 128, 0, stream, a);
  } else if (dtype == HX_BF16) {
    LatentPrepareArgs<__nv_bfloat16> a{down, ld_down, q_weight, kv_weight, eps, positions, freq,
                                       freq_exact, rotary_dims, layout,
                                       static_cast<__nv_bfloat16*>(query_latent), ld_latent,
                                       static_cast<__nv_bfloat16*>(rows), ld_rows, key_offset,
                                       q_rank, kv_rank, rot, row_dim, amplitude};
    hx_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens), 128, 0, stream, a);
  } else {
    HX_REQUIRE(false, "hx_latent_prepare: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_latent_prepare");
  return HX_OK;
}

HX_API int hx_latent_queries(const void* q, int ld_q, int rot_offset, void* rows, int ld_rows,
                             const int* positions, const float* freq, const double* freq_exact,
                             int rotary_dims, int layout, int dtype, int tokens, int heads,
                             int kv_rank, int rot, int row_dim, float amplitude,
                             cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && kv_rank > 0 && rot >= 0 && row_dim >= kv_rank + rot,
             "hx_latent_queries: bad sizes");
  HX_REQUIRE(ld_q >= rot_offset + heads * rot && ld_rows >= heads * row_dim,
             "hx_latent_queries: bad strides");
  HX_REQUIRE(rotary_dims >= 0 && rotary_dims <= rot && rotary_dims % 2 == 0,
             "hx_latent_queries: %d of %d coordinates rotated", rotary_dims, rot);
  if (tokens == 0 || row_dim == kv_rank) return HX_OK;
  const dim3 grid(tokens, heads);
  if (dtype == HX_F32) {
    hx_launch(latent_queries_kernel<float>, grid, 64, 0, stream, static_cast<const float*>(q), ld_q,
              rot_offset, static_cast<float*>(rows), ld_rows, positions, freq, freq_exact,
              rotary_dims, layout, kv_rank, rot, row_dim, amplitude);
  } else if (dtype == HX_BF16) {
    hx_launch(latent_queries_kernel<__nv_bfloat16>, grid, 64, 0, stream,
              static_cast<const __nv_bfloat16*>(q), ld_q, rot_offset,
              static_cast<__nv_bfloat16*>(rows), ld_rows, positions, freq, freq_exact, rotary_dims,
              layout, kv_rank, rot, row_dim, amplitude);
  } else {
    HX_REQUIRE(false, "hx_latent_queries: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_latent_queries");
  return HX_OK;
}

// ------------------------------------------------------------- one small product per head
//
// out[t, h * out_stride + o] = sum_i w[h][o][i] * x[t, h * x_stride + i]: every head has its
// own [out_dim x in_dim] matrix (the up-projection of the keys moved to the queries, the
// up-projection of the values behind the weighted sum).  A CTA computes a [64 tokens x 64
// outputs] tile of one head with float32 sums, 4 x 4 per thread, the operands staged through
// shared memory sixteen reduction steps at a time.
namespace {

constexpr int HP_TILE = 64;
constexpr int HP_DEPTH = 16;

template <typename T>
__global__ __launch_bounds__(256) void head_products_kernel(
    const T* __restrict__ x, int ld_x, int x_stride, const T* __restrict__ w,
    T* __restrict__ out, int ld_out, int out_stride, int tokens, int out_dim, int in_dim) {
  __shared__ float xs[HP_DEPTH][HP_TILE + 4];
  __shared__ float ws[HP_DEPTH][HP_TILE + 4];
  hx_pdl_prologue();
  const int head = blockIdx.z;
  const int token0 = blockIdx.x * HP_TILE;
  const int out0 = blockIdx.y * HP_TILE;
  const T* xh = x + static_cast<size_t>(head) * x_stride;
  const T* wh = w + static_cast<size_t>(head) * out_dim * in_dim;
  const int tx = threadIdx.x & 15;      // outputs tx * 4 ..
  const int ty = threadIdx.x >> 4;      // tokens ty * 4 ..
  float sums[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) sums[i][j] = 0.0f;
  for (int k0 = 0; k0 < in_dim; k0 += HP_DEPTH) {
    __syncthreads();
    for (int e = threadIdx.x; e < HP_TILE * HP_DEPTH; e += 256) {
      const int row = e / HP_DEPTH, k = e - row * HP_DEPTH;
      const int token = token0 + row, o = out0 + row, i = k0 + k;
      xs[k][row] = (token < tokens && i < in_dim)
                       ? hx_to_float<T>(xh[static_cast<size_t>(token) * ld_x + i]) : 0.0f;
      ws[k][row] = (o < out_dim && i < in_dim)
                       ? hx_to_float<T>(wh[static_cast<size_t>(o) * in_dim + i]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HP_DEPTH; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w};
      const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sums[i][j] = fmaf(av[i], bv[j], sums[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int token = token0 + ty * 4 + i;
    if (token >= tokens) continue;
    T* row = out + static_cast<size_t>(token) * ld_out + static_cast<size_t>(head) * out_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int o = out0 + tx * 4 + j;
      if (o < out_dim) row[o] = hx_from_float<T>(sums[i][j]);
    }
  }
}

}  // namespace

// x [tokens, ld_x] with head h's input at column h * x_stride; w [heads, out_dim, in_dim];
// out [tokens, ld_out] with head h's result at column h * out_stride; all in the compute dtype.
HX_API int hx_head_products(const void* x, int ld_x, int x_stride, const void* w, void* out,
                            int ld_out, int out_stride, int dtype, int tokens, int heads,
                            int out_dim, int in_dim, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && heads > 0 && out_dim > 0 && in_dim > 0, "hx_head_products: bad sizes");
  HX_REQUIRE(ld_x >= (heads - 1) * x_stride + in_dim && ld_out >= (heads - 1) * out_stride + out_dim,
             "hx_head_products: bad strides");
  if (tokens == 0) return HX_OK;
  const dim3 grid((tokens + HP_TILE - 1) / HP_TILE, (out_dim + HP_TILE - 1) / HP_TILE, heads);
  if (dtype == HX_F32) {
    hx_launch(head_products_kernel<float>, grid, 256, 0, stream, static_cast<const float*>(x), ld_x,
              x_stride, static_cast<const float*>(w), static_cast<float*>(out), ld_out, out_stride,
              tokens, out_dim, in_dim);
  } else if (dtype == HX_BF16) {
    hx_launch(head_products_kernel<__nv_bfloat16>, grid, 256, 0, stream,
              static_cast<const __nv_bfloat16*>(x), ld_x, x_stride,
              static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out), ld_out,
              out_stride, tokens, out_dim, in_dim);
  } else {
    HX_REQUIRE(false, "hx_head_products: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_head_products");
  return HX_OK;
}
