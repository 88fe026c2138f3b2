// A sublayer joined to the residual through a gate: x += y * sigmoid(g + b), with g the sums of
// a product of the sublayer's input and b a bias per channel; and the rows of two float32
// streams laid side by side in the compute type, as the input of a product over both.
// Everything is float32 but the joined rows' store.
#include "hx_common.cuh"

namespace {

// residual[t][c] += output[t][c] * sigmoid(gate[t][c] + bias[c])
__global__ __launch_bounds__(256) void gated_residual_add_kernel(
    float* __restrict__ residual, const float* __restrict__ output, const float* __restrict__ gate,
    int ld_gate, const float* __restrict__ bias, int width) {
  hx_pdl_prologue();
  const int token = blockIdx.y;
  const size_t row = static_cast<size_t>(token) * width;
  const float* g = gate + static_cast<size_t>(token) * ld_gate;
  if ((width & 3) == 0 && (ld_gate & 3) == 0) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= width) return;
    const float4 y = *reinterpret_cast<const float4*>(output + row + c);
    const float4 s = *reinterpret_cast<const float4*>(g + c);
    const float4 b = *reinterpret_cast<const float4*>(bias + c);
    float4 x = *reinterpret_cast<float4*>(residual + row + c);
    x.x = fmaf(y.x, hx_sigmoid(s.x + b.x), x.x);
    x.y = fmaf(y.y, hx_sigmoid(s.y + b.y), x.y);
    x.z = fmaf(y.z, hx_sigmoid(s.z + b.z), x.z);
    x.w = fmaf(y.w, hx_sigmoid(s.w + b.w), x.w);
    *reinterpret_cast<float4*>(residual + row + c) = x;
    return;
  }
  for (int c = blockIdx.x * blockDim.x * 4 + threadIdx.x; c < width && c < (blockIdx.x + 1) * blockDim.x * 4;
       c += blockDim.x)
    residual[row + c] = fmaf(output[row + c], hx_sigmoid(g[c] + bias[c]), residual[row + c]);
}

// out[t] = [a[t] | b[t]] rounded to T
template <typename T>
__global__ __launch_bounds__(256) void join_rows_kernel(const float* __restrict__ a,
                                                        const float* __restrict__ b,
                                                        T* __restrict__ out, int ld_out, int width) {
  hx_pdl_prologue();
  const int token = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * width) return;
  const float v = c < width ? a[static_cast<size_t>(token) * width + c]
                            : b[static_cast<size_t>(token) * width + c - width];
  out[static_cast<size_t>(token) * ld_out + c] = hx_from_float<T>(v);
}

}  // namespace

// residual[:tokens] += output[:tokens] * sigmoid(gate[:tokens] + bias), all float32;
// residual and output [tokens, width] contiguous, gate with row stride ld_gate.
HX_API int hx_gated_residual_add(float* residual, const float* output, const float* gate,
                                 int ld_gate, const float* bias, int tokens, int width,
                                 cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && width > 0 && ld_gate >= width, "hx_gated_residual_add: bad sizes");
  if (tokens == 0) return HX_OK;
  hx_launch(gated_residual_add_kernel, dim3((width + 1023) / 1024, tokens), 256, 0, stream,
            residual, output, gate, ld_gate, bias, width);
  HX_CHECK_LAUNCH("hx_gated_residual_add");
  return HX_OK;
}

// out[:tokens] = [a | b] in the compute dtype; a, b float32 [tokens, width] contiguous.
HX_API int hx_join_rows(const float* a, const float* b, void* out, int ld_out, int dtype,
                        int tokens, int width, cudaStream_t stream) {
  HX_REQUIRE(tokens >= 0 && width > 0 && ld_out >= 2 * width, "hx_join_rows: bad sizes");
  if (tokens == 0) return HX_OK;
  const dim3 grid((2 * width + 255) / 256, tokens);
  if (dtype == HX_F32) {
    hx_launch(join_rows_kernel<float>, grid, 256, 0, stream, a, b, static_cast<float*>(out),
              ld_out, width);
  } else if (dtype == HX_BF16) {
    hx_launch(join_rows_kernel<__nv_bfloat16>, grid, 256, 0, stream, a, b,
              static_cast<__nv_bfloat16*>(out), ld_out, width);
  } else {
    HX_REQUIRE(false, "hx_join_rows: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_join_rows");
  return HX_OK;
}
