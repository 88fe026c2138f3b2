// A feed-forward of routed experts: every token goes through `top` of `experts` small gated
// feed-forwards, chosen by a router, and their outputs are summed with the router's weights.
//
//   * hx_route_top: scores s = sigmoid(z) of the router's float32 sums z, the `top` largest
//     (the lowest index among equals), weights s / (sum of the chosen + 1e-20) * scale;
//   * hx_expert_gate_up: act[pair] = f(Wg[e] x) * (Wu[e] x) for every (token, choice) pair;
//   * hx_expert_down: out[token] += sum_k weight_k * Wd[e_k] act[pair_k], the choices in
//     ascending order, one writer per output (no atomics: the sum's order is fixed).
//
// The two products read the expert's matrices through the chosen index, a row per warp: with
// few tokens (decoding) that is the stream of the chosen experts' weights, which is all such a
// step has to move.  Nothing here looks at device values on the host, so a step can be
// recorded into a CUDA graph.
#include "hx_common.cuh"

namespace {

constexpr int ROUTE_MAX_PER_LANE = 32;      // experts a lane can mark as taken: 1,024 in all

// What the router's sums become, and what is chosen by and weighted with.
struct RouteRule {
  int softmax;                // 0: s = sigmoid(z); 1: s = softmax(z) over all outputs
  const float* correction;    // [experts] added to s for the CHOICE only; may be null
  int normalize;              // 1: weights s / (sum of the chosen + 1e-20) * scale; 0: s * scale
};

__global__ __launch_bounds__(128) void route_top_kernel(const float* __restrict__ sums, int ld,
                                                        int tokens, int experts, int top,
                                                        float scale, RouteRule rule,
                                                        int* __restrict__ chosen,
                                                        float* __restrict__ weights) {
  hx_pdl_prologue();
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const int lane = threadIdx.x & 31;
  const float* z = sums + static_cast<size_t>(token) * ld;
  // softmax: the row's maximum and the sum of exp(z - max), in ascending order per lane
  float row_max = 0.0f, inverse_sum = 1.0f;
  if (rule.softmax) {
    row_max = -INFINITY;
    for (int e = lane; e < experts; e += 32) row_max = fmaxf(row_max, z[e]);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, offset));
    float sum = 0.0f;
    for (int e = lane; e < experts; e += 32) sum += expf(z[e] - row_max);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
      sum += __shfl_xor_sync(0xffffffffu, sum, offset);
    inverse_sum = 1.0f / sum;
  }
  auto score_of = [&](int e) {
    return rule.softmax ? expf(z[e] - row_max) * inverse_sum : hx_sigmoid(z[e]);
  };
  unsigned taken = 0u;          // bit i: expert lane + 32 i is chosen already
  float total = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, best_score = 0.0f;
    int best_index = 0x7fffffff;
    for (int i = 0, e = lane; e < experts; ++i, e += 32) {
      if (taken & (1u << i)) continue;
      const float s = score_of(e);
      const float c = rule.correction != nullptr ? s + rule.correction[e] : s;
      if (c > best) { best = c; best_score = s; best_index = e; }   // the first of equals stays
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const float other_score = __shfl_xor_sync(0xffffffffu, best_score, offset);
      const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
      if (other > best || (other == best && other_index < best_index)) {
        best = other;
        best_score = other_score;
        best_index = other_index;
      }
    }
    if ((best_index & 31) == lane && best_index < experts) taken |= 1u << (best_index >> 5);
    total += best_score;
    if (lane == 0) {
      chosen[static_cast<size_t>(token) * top + k] = best_index;
      weights[static_cast<size_t>(token) * top + k] = best_score;
    }
  }
  __syncwarp();
  if (lane < top) {
    float* w = weights + static_cast<size_t>(token) * top + lane;
    *w = rule.normalize ? *w / (total + 1e-20f) * scale : *w * scale;
  }
}

// sum over a lane's share of w[0..width) * x[0..width), x float32 in shared memory
template <typename T>
__device__ __forceinline__ float lane_dot(const T* __restrict__ w, const float* x, int width,
                                          int lane);

template <>
__device__ __forceinline__ float lane_dot<float>(const float* __restrict__ w, const float* x,
                                                 int width, int lane) {
  float sum = 0.0f;
  if ((width & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    for (int c = lane * 4; c < width; c += 128) {
      const float4 a = *reinterpret_cast<const float4*>(w + c);
      const float4 b = *reinterpret_cast<const float4*>(x + c);
      sum = fmaf(a.x, b.x, sum); sum = fmaf(a.y, b.y, sum);
      sum = fmaf(a.z, b.z, sum); sum = fmaf(a.w, b.w, sum);
    }
  } else {
    for (int c = lane; c < width; c += 32) sum = fmaf(w[c], x[c], sum);
  }
  return sum;
}

template <>
__device__ __forceinline__ float lane_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w,
                                                         const float* x, int width, int lane) {
  float sum = 0.0f;
  if ((width & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    for (int c = lane * 8; c < width; c += 256) {
      const uint4 packed = *reinterpret_cast<const uint4*>(w + c);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&packed);
      const float4 x0 = *reinterpret_cast<const float4*>(x + c);
      const float4 x1 = *reinterpret_cast<const float4*>(x + c + 4);
      const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]);
      const float2 d = __bfloat1622float2(pairs[2]), e = __bfloat1622float2(pairs[3]);
      sum = fmaf(a.x, x0.x, sum); sum = fmaf(a.y, x0.y, sum);
      sum = fmaf(b.x, x0.z, sum); sum = fmaf(b.y, x0.w, sum);
      sum = fmaf(d.x, x1.x, sum); sum = fmaf(d.y, x1.y, sum);
      sum = fmaf(e.x, x1.z, sum); sum = fmaf(e.y, x1.w, sum);
    }
  } else {
    for (int c = lane; c < width; c += 32) sum = fmaf(__bfloat162float(w[c]), x[c], sum);
  }
  return sum;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

constexpr int EXPERT_WARPS = 4;
constexpr int GATE_UP_ROWS = 32;      // activation rows a CTA of the first product computes
constexpr int DOWN_ROWS = 32;         // output rows a CTA of the second product computes

// grid (pairs, ceil(ff / GATE_UP_ROWS)); shared: the token's input row in float32
template <typename T>
__global__ __launch_bounds__(EXPERT_WARPS * 32) void expert_gate_up_kernel(
    const T* __restrict__ x, int ld_x, const T* __restrict__ gate_up, const int* __restrict__ chosen,
    T* __restrict__ act, int top, int ff, int width, int experts, int activation, float limit) {
  extern __shared__ float4 shared4[];
  float* xs = reinterpret_cast<float*>(shared4);
  hx_pdl_prologue();
  const int pair = blockIdx.x;
  const int token = pair / top;
  const int expert = chosen[pair];
  if (expert < 0 || expert >= experts) return;
  const T* xr = x + static_cast<size_t>(token) * ld_x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = hx_to_float<T>(xr[c]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* w = gate_up + static_cast<size_t>(expert) * 2 * ff * width;
  const int first = blockIdx.y * GATE_UP_ROWS;
  for (int j = first + warp; j < first + GATE_UP_ROWS && j < ff; j += EXPERT_WARPS) {
    const float g = warp_sum(lane_dot<T>(w + static_cast<size_t>(j) * width, xs, width, lane));
    const float u = warp_sum(lane_dot<T>(w + static_cast<size_t>(ff + j) * width, xs, width, lane));
    if (lane == 0)
      act[static_cast<size_t>(pair) * ff + j] = hx_from_float<T>(hx_gated(g, u, activation, limit));
  }
}

// grid (tokens, ceil(width / DOWN_ROWS)); shared: one activation row in float32 at a time
template <typename T>
__global__ __launch_bounds__(EXPERT_WARPS * 32) void expert_down_kernel(
    const T* __restrict__ act, const T* __restrict__ down, const int* __restrict__ chosen,
    const float* __restrict__ weights, float* __restrict__ out, int ld_out, int top, int ff,
    int width, int experts) {
  extern __shared__ float4 shared4[];
  float* as = reinterpret_cast<float*>(shared4);
  hx_pdl_prologue();
  const int token = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = blockIdx.y * DOWN_ROWS;
  constexpr int PER_WARP = DOWN_ROWS / EXPERT_WARPS;
  float sums[PER_WARP];
#pragma unroll
  for (int r = 0; r < PER_WARP; ++r) sums[r] = 0.0f;
  for (int k = 0; k < top; ++k) {
    const int pair = token * top + k;
    const int expert = chosen[pair];
    const float weight = weights[pair];
    __syncthreads();
    for (int c = threadIdx.x; c < ff; c += blockDim.x)
      as[c] = hx_to_float<T>(act[static_cast<size_t>(pair) * ff + c]);
    __syncthreads();
    if (expert < 0 || expert >= experts) continue;
    const T* w = down + static_cast<size_t>(expert) * width * ff;
#pragma unroll
    for (int r = 0; r < PER_WARP; ++r) {
      const int i = first + warp + r * EXPERT_WARPS;
      if (i < width)
        sums[r] = fmaf(weight, warp_sum(lane_dot<T>(w + static_cast<size_t>(i) * ff, as, ff, lane)),
                       sums[r]);
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < PER_WARP; ++r) {
      const int i = first + warp + r * EXPERT_WARPS;
      if (i < width) out[static_cast<size_t>(token) * ld_out + i] += sums[r];
    }
  }
}

// ---- the pairs of a step sorted by expert, for one grouped product per projection ----------
//
// With many tokens an expert's matrices should be read once for all of its tokens, not once
// per token.  The (token, choice) pairs are laid out expert by expert, every expert's rows
// rounded up to a whole tile of the product's token side, the tokens' inputs are copied into
// that order, two grouped tensor-core products run over the tiles (each tile names its
// expert), and the outputs are summed back per token in the order of its choices.  A row's
// result does not depend on where in a tile it lies, so pairs take their rows by atomic
// counters; rows of padding hold whatever the buffer held and are never read back.

constexpr int ROWS_THREADS = 1024;

// One CTA.  pair_row[pair]: the pair's row in the grouped order (-1: no valid expert);
// tile_group[t], t < max_tiles: the expert of tile t, -1 behind the last tile in use.
__global__ __launch_bounds__(ROWS_THREADS) void expert_rows_kernel(
    const int* __restrict__ chosen, int pairs, int experts, int tile, int max_tiles,
    int* __restrict__ pair_row, int* __restrict__ tile_group) {
  extern __shared__ int shared_counts[];
  int* counts = shared_counts;              // pairs of the expert, then its fill cursor
  int* first_row = shared_counts + experts; // the expert's first row
  __shared__ int tiles_in_use;
  hx_pdl_prologue();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
    const int e = chosen[pair];
    if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0;
    for (int e = 0; e < experts; ++e) {
      first_row[e] = row;
      row += (counts[e] + tile - 1) / tile * tile;
    }
    tiles_in_use = row / tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int begin = first_row[e] / tile;
    const int end = begin + (counts[e] + tile - 1) / tile;
    for (int t = begin; t < end && t < max_tiles; ++t) tile_group[t] = e;
  }
  for (int t = tiles_in_use + threadIdx.x; t < max_tiles; t += blockDim.x) tile_group[t] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
    const int e = chosen[pair];
    pair_row[pair] = (e >= 0 && e < experts) ? first_row[e] + atomicAdd(&counts[e], 1) : -1;
  }
}

// grid (pairs): grouped[pair_row[pair]] = x[pair / top]
template <typename T>
__global__ __launch_bounds__(128) void expert_gather_kernel(
    const T* __restrict__ x, int ld_x, const int* __restrict__ pair_row, T* __restrict__ grouped,
    int ld_grouped, int top, int width) {
  hx_pdl_prologue();
  const int pair = blockIdx.x;
  const int row = pair_row[pair];
  if (row < 0) return;
  const T* from = x + static_cast<size_t>(pair / top) * ld_x;
  T* to = grouped + static_cast<size_t>(row) * ld_grouped;
  constexpr int PER = 16 / sizeof(T);
  if (width % PER == 0 && ld_x % PER == 0 && ld_grouped % PER == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(grouped)) & 15) == 0) {
    for (int c = threadIdx.x; c < width / PER; c += blockDim.x)
      reinterpret_cast<uint4*>(to)[c] = reinterpret_cast<const uint4*>(from)[c];
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) to[c] = from[c];
  }
}

// grid (ceil(width / 512), tokens): out[t][c] += sum_k weights[t][k] * y[pair_row[t top + k]][c]
__global__ __launch_bounds__(128) void expert_combine_kernel(
    const float* __restrict__ y, int ld_y, const int* __restrict__ pair_row,
    const float* __restrict__ weights, float* __restrict__ out, int ld_out, int top, int width) {
  hx_pdl_prologue();
  const int token = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= width) return;
  float* o = out + static_cast<size_t>(token) * ld_out;
  const bool wide = c + 4 <= width && ld_y % 4 == 0 && ld_out % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int k = 0; k < top; ++k) {
    const int row = pair_row[token * top + k];
    if (row < 0) continue;
    const float weight = weights[token * top + k];
    const float* from = y + static_cast<size_t>(row) * ld_y + c;
    if (wide) {
      const float4 v = *reinterpret_cast<const float4*>(from);
      sums[0] = fmaf(weight, v.x, sums[0]); sums[1] = fmaf(weight, v.y, sums[1]);
      sums[2] = fmaf(weight, v.z, sums[2]); sums[3] = fmaf(weight, v.w, sums[3]);
    } else {
      for (int i = 0; i < 4 && c + i < width; ++i) sums[i] = fmaf(weight, from[i], sums[i]);
    }
  }
  if (wide) {
    float4 v = *reinterpret_cast<float4*>(o + c);
    v.x += sums[0]; v.y += sums[1]; v.z += sums[2]; v.w += sums[3];
    *reinterpret_cast<float4*>(o + c) = v;
  } else {
    for (int i = 0; i < 4 && c + i < width; ++i) o[c + i] += sums[i];
  }
}

// grid (ceil(width / 512), tokens): out[t][c] += x[t][c] * (sum of the weights of the token's
// choices that name no expert with matrices: index >= experts is an identity output)
template <typename T>
__global__ __launch_bounds__(128) void expert_identity_kernel(
    const T* __restrict__ x, int ld_x, const int* __restrict__ chosen,
    const float* __restrict__ weights, float* __restrict__ out, int ld_out, int top, int width,
    int experts) {
  hx_pdl_prologue();
  const int token = blockIdx.y;
  float weight = 0.0f;
  for (int k = 0; k < top; ++k)
    if (chosen[token * top + k] >= experts) weight += weights[token * top + k];
  if (weight == 0.0f) return;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  for (int c = c0; c < c0 + 4 && c < width; ++c)
    out[static_cast<size_t>(token) * ld_out + c] =
        fmaf(weight, hx_to_float<T>(x[static_cast<size_t>(token) * ld_x + c]),
             out[static_cast<size_t>(token) * ld_out + c]);
}

}  // namespace

// sums float32 [tokens, ld] (the router's products); chosen int32 and weights float32
// [tokens, top].  softmax: scores are softmax(z) over all `experts` outputs instead of
// sigmoid(z); correction [experts] (may be null) is added to the scores for the choice only;
// normalize 0: the weights are the chosen scores times scale, not divided by their sum.
HX_API int hx_route_top_ruled(const float* sums, int ld, int tokens, int experts, int top,
                              float scale, int softmax, const float* correction, int normalize,
                              int* chosen, float* weights, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts && ld >= experts,
             "hx_route_top: bad sizes");
  HX_REQUIRE(experts <= 32 * ROUTE_MAX_PER_LANE && top <= 32,
             "hx_route_top: at most %d experts and 32 choices", 32 * ROUTE_MAX_PER_LANE);
  if (tokens == 0) return HX_OK;
  const RouteRule rule{softmax, correction, normalize};
  hx_launch(route_top_kernel, dim3((tokens + 3) / 4), 128, 0, stream, sums, ld, tokens, experts,
            top, scale, rule, chosen, weights);
  HX_CHECK_LAUNCH("hx_route_top");
  return HX_OK;
}

// s = sigmoid(z), the `top` largest, weights s / (sum of the chosen + 1e-20) * scale.
HX_API int hx_route_top(const float* sums, int ld, int tokens, int experts, int top, float scale,
                        int* chosen, float* weights, cudaStream_t stream) {
  return hx_route_top_ruled(sums, ld, tokens, experts, top, scale, 0, nullptr, 1, chosen, weights,
                            stream);
}

// x [tokens, ld_x], gate_up [experts, 2 * ff, width] (gate rows, then up rows), act
// [tokens * top, ff], all in the compute dtype; chosen int32 [tokens, top].
HX_API int hx_expert_gate_up_limited(const void* x, int ld_x, const void* gate_up, const int* chosen,
                             void* act, int dtype, int tokens, int top, int ff, int width,
                             int experts, int activation, float limit, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && top > 0 && ff > 0 && width > 0 && experts > 0 && ld_x >= width,
             "hx_expert_gate_up: bad sizes");
  HX_REQUIRE(width * sizeof(float) <= 48 * 1024, "hx_expert_gate_up: rows of %d are too wide",
             width);
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens * top, (ff + GATE_UP_ROWS - 1) / GATE_UP_ROWS);
  const size_t shared = (static_cast<size_t>(width) * sizeof(float) + 15) / 16 * 16;
  if (dtype == HX_F32) {
    hx_launch(expert_gate_up_kernel<float>, grid, EXPERT_WARPS * 32, shared, stream,
              static_cast<const float*>(x), ld_x, static_cast<const float*>(gate_up), chosen,
              static_cast<float*>(act), top, ff, width, experts, activation, limit);
  } else if (dtype == HX_BF16) {
    hx_launch(expert_gate_up_kernel<__nv_bfloat16>, grid, EXPERT_WARPS * 32, shared, stream,
              static_cast<const __nv_bfloat16*>(x), ld_x,
              static_cast<const __nv_bfloat16*>(gate_up), chosen, static_cast<__nv_bfloat16*>(act),
              top, ff, width, experts, activation, limit);
  } else {
    HX_REQUIRE(false, "hx_expert_gate_up: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_expert_gate_up");
  return HX_OK;
}

HX_API int hx_expert_gate_up(const void* x, int ld_x, const void* gate_up, const int* chosen,
                             void* act, int dtype, int tokens, int top, int ff, int width,
                             int experts, int activation, cudaStream_t stream) {
  return hx_expert_gate_up_limited(x, ld_x, gate_up, chosen, act, dtype, tokens, top, ff, width,
                                   experts, activation, 0.0f, stream);
}

// act [tokens * top, ff] and down [experts, width, ff] in the compute dtype; out float32
// [tokens, ld_out] is summed into.
HX_API int hx_expert_down(const void* act, const void* down, const int* chosen,
                          const float* weights, float* out, int ld_out, int dtype, int tokens,
                          int top, int ff, int width, int experts, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && top > 0 && ff > 0 && width > 0 && experts > 0 && ld_out >= width,
             "hx_expert_down: bad sizes");
  HX_REQUIRE(ff * sizeof(float) <= 48 * 1024, "hx_expert_down: experts of %d are too wide", ff);
  if (tokens == 0) return HX_OK;
  const dim3 grid(tokens, (width + DOWN_ROWS - 1) / DOWN_ROWS);
  const size_t shared = (static_cast<size_t>(ff) * sizeof(float) + 15) / 16 * 16;
  if (dtype == HX_F32) {
    hx_launch(expert_down_kernel<float>, grid, EXPERT_WARPS * 32, shared, stream,
              static_cast<const float*>(act), static_cast<const float*>(down), chosen, weights,
              out, ld_out, top, ff, width, experts);
  } else if (dtype == HX_BF16) {
    hx_launch(expert_down_kernel<__nv_bfloat16>, grid, EXPERT_WARPS * 32, shared, stream,
              static_cast<const __nv_bfloat16*>(act), static_cast<const __nv_bfloat16*>(down),
              chosen, weights, out, ld_out, top, ff, width, experts);
  } else {
    HX_REQUIRE(false, "hx_expert_down: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_expert_down");
  return HX_OK;
}

// Tiles the grouped order of `pairs` pairs over `experts` experts can take with this tile.
HX_API int hx_expert_tile_bound(int pairs, int experts, int tile) {
  if (pairs < 0 || experts <= 0 || tile <= 0) return 0;
  return static_cast<int>((static_cast<long long>(pairs) + static_cast<long long>(experts) * (tile - 1) +
                           tile - 1) / tile);
}

// chosen int32 [pairs]; pair_row int32 [pairs]; tile_group int32 [max_tiles] with max_tiles at
// least hx_expert_tile_bound(pairs, experts, tile).
HX_API int hx_expert_rows(const int* chosen, int pairs, int experts, int tile, int max_tiles,
                          int* pair_row, int* tile_group, cudaStream_t stream) {
  HX_REQUIRE(pairs >= 0 && experts > 0 && tile > 0, "hx_expert_rows: bad sizes");
  HX_REQUIRE(experts <= 4096, "hx_expert_rows: at most 4096 experts");
  HX_REQUIRE(max_tiles >= hx_expert_tile_bound(pairs, experts, tile),
             "hx_expert_rows: %d tiles do not hold %d pairs of %d experts", max_tiles, pairs,
             experts);
  if (pairs == 0) return HX_OK;
  hx_launch(expert_rows_kernel, dim3(1), ROWS_THREADS, 2 * experts * sizeof(int), stream, chosen,
            pairs, experts, tile, max_tiles, pair_row, tile_group);
  HX_CHECK_LAUNCH("hx_expert_rows");
  return HX_OK;
}

// x [tokens, ld_x] and grouped [rows, ld_grouped] in the compute dtype.
HX_API int hx_expert_gather(const void* x, int ld_x, const int* pair_row, void* grouped,
                            int ld_grouped, int dtype, int tokens, int top, int width,
                            cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && top > 0 && width > 0 && ld_x >= width && ld_grouped >= width,
             "hx_expert_gather: bad sizes");
  if (tokens == 0) return HX_OK;
  if (dtype == HX_F32) {
    hx_launch(expert_gather_kernel<float>, dim3(tokens * top), 128, 0, stream,
              static_cast<const float*>(x), ld_x, pair_row, static_cast<float*>(grouped),
              ld_grouped, top, width);
  } else if (dtype == HX_BF16) {
    hx_launch(expert_gather_kernel<__nv_bfloat16>, dim3(tokens * top), 128, 0, stream,
              static_cast<const __nv_bfloat16*>(x), ld_x, pair_row,
              static_cast<__nv_bfloat16*>(grouped), ld_grouped, top, width);
  } else {
    HX_REQUIRE(false, "hx_expert_gather: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_expert_gather");
  return HX_OK;
}

// y float32 [rows, ld_y] (an expert's output per grouped row); out float32 [tokens, ld_out] is
// summed into, a token's choices in ascending order, one writer per element.
HX_API int hx_expert_combine(const float* y, int ld_y, const int* pair_row, const float* weights,
                             float* out, int ld_out, int tokens, int top, int width,
                             cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && top > 0 && width > 0 && ld_y >= width && ld_out >= width,
             "hx_expert_combine: bad sizes");
  HX_REQUIRE(tokens <= 65535, "hx_expert_combine: at most 65535 tokens a step");
  if (tokens == 0) return HX_OK;
  hx_launch(expert_combine_kernel, dim3((width + 511) / 512, tokens), 128, 0, stream, y, ld_y,
            pair_row, weights, out, ld_out, top, width);
  HX_CHECK_LAUNCH("hx_expert_combine");
  return HX_OK;
}

// out float32 [tokens, ld_out] += x[token] * (sum of the weights of the token's choices with an
// index >= experts): outputs of the router behind the experts return their input.
HX_API int hx_expert_identity_add(const void* x, int ld_x, const int* chosen, const float* weights,
                                  float* out, int ld_out, int dtype, int tokens, int top,
                                  int width, int experts, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && top > 0 && width > 0 && ld_x >= width && ld_out >= width &&
                 experts >= 0, "hx_expert_identity_add: bad sizes");
  HX_REQUIRE(tokens <= 65535, "hx_expert_identity_add: at most 65535 tokens a step");
  if (tokens == 0) return HX_OK;
  const dim3 grid((width + 511) / 512, tokens);
  if (dtype == HX_F32) {
    hx_launch(expert_identity_kernel<float>, grid, 128, 0, stream, static_cast<const float*>(x),
              ld_x, chosen, weights, out, ld_out, top, width, experts);
  } else if (dtype == HX_BF16) {
    hx_launch(expert_identity_kernel<__nv_bfloat16>, grid, 128, 0, stream,
              static_cast<const __nv_bfloat16*>(x), ld_x, chosen, weights, out, ld_out, top, width,
              experts);
  } else {
    HX_REQUIRE(false, "hx_expert_identity_add: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_expert_identity_add");
  return HX_OK;
}
