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
// Both recurrences run CTAs per (request, head, block of columns).  A thread owns a column of S
// (one value coordinate) and a run of consecutive rows of it (4, 8 or 16, by the matrix's size):
// `parts` neighbouring lanes share a
// column and add their partial sums with shuffles.  The tokens' vectors are staged through
// shared memory a tile at a time (loads issued four at a time, the exponentials taken once
// per token and channel, not once per thread), each lane's rows of a vector lying together
// (padded against bank conflicts) so that 16-byte loads fetch them.  CTAs are
// small (128 threads) so that several share an SM and one's staging hides behind another's
// arithmetic.  In memory a head's matrix is laid out for exactly this dealing,
// [row % run][column][row / run]: the k-th value of every thread is one contiguous run, so that
// loading and storing the state (all a decode step does here) are full-width transactions.
// Rows beyond the matrix (when the run does not divide them) are padding;
// hx_scan_state_floats() gives the size.
#include "hx_common.cuh"

namespace {

__device__ __forceinline__ float softplus(float x) {
  return x > 20.0f ? x : log1pf(expf(x));
}

// One step S <- decay * S + add of a recurrence in the float32 engine.  A decay close to one
// cannot be told from its neighbours in float32 (their spacing is 6e-8), and a head that hardly
// forgets multiplies a thousand such decays over a long prompt: the roundings add up like a
// random walk and show in the logits of late positions.  So the decay arrives as d = decay - 1
// (taken with expm1f, which keeps its digits), the step is S + (d S + add), and the rounding of
// that sum (a two-sum recovers it) is carried beside S in `carry`, which decays like S.  What
// reads the state reads S + carry; the state row holds S + carry rounded once.
__device__ __forceinline__ void decayed_add_exact(float& S, float& carry, float d, float add) {
  const float t = fmaf(d, S, add);
  const float sum = S + t;
  const float shadow = sum - S;
  const float error = (S - (sum - shadow)) + (t - shadow);
  carry = fmaf(d, carry, carry) + error;
  S = sum;
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

// Rows of a column that one lane keeps.  A pure function of the row count, because the state's
// order in memory follows from it.  Sixteen for every size: runs of 4 and 8 (more lanes and
// CTAs per head, each staging the tokens' vectors again) were measured at the sizes of a 7B
// model's layers and lost, 2.0 against 1.26 ms for 2,048 tokens of a state-space layer and
// 190 against 68 us for a decode step of 64 requests of a time-mixing layer.
__host__ __device__ constexpr int rows_per_thread(int rows) { return rows > 0 ? 16 : 16; }
// Threads of a CTA at most.  A head whose columns need more is cut into blocks of columns
// (blockIdx.z), each a CTA of its own with the same tokens staged.
constexpr int SCAN_THREADS = 256;
// CTAs the compiler makes room for on an SM (it bounds the registers of a thread).
#ifndef HX_SCAN_CTAS
#define HX_SCAN_CTAS 2
#endif
#ifndef HX_SCAN_TILE_KB
#define HX_SCAN_TILE_KB 24
#endif

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
  float* state;           // per slot: heads x head_stride, see the layout above
  long long state_stride;
  int head_stride;
  float* y;               // [tokens, heads * width]
  const int* request_start;
  const int* request_slot;
  int heads, width, rows, groups;   // rows = state size N
  int parts;                        // lanes that share a column
  int block_lanes;                  // lanes (columns x parts) of one CTA
  int tile;                         // tokens staged at once
  int per_token;                    // floats staged per token
};

// Rows of a staged vector are kept in runs of RPT (one lane's share); runs of eight and more
// have four floats of padding behind them, so that the lanes of a warp, which read different
// runs with 16-byte loads, fall on different banks.
template <int RPT> constexpr int run_stride() { return RPT + (RPT >= 8 ? 4 : 0); }
template <int RPT>
__device__ __forceinline__ int padded(int n) { return n + (n / RPT) * (RPT >= 8 ? 4 : 0); }

// One vector of `length` elements for each of `tokens` tokens: dst[t * stride + place(e)] =
// load(t, e).  Warps take tokens, lanes take elements (consecutive addresses), four loads in
// flight per lane; nothing divides.
template <bool ONE_TOKEN, typename Load, typename Place>
__device__ __forceinline__ void stage(float* dst, int stride, int tokens, int length, Load load,
                                      Place place) {
  if (ONE_TOKEN) {      // a decode step: one vector, one load per thread and round
    for (int e = threadIdx.x; e < length; e += blockDim.x) dst[place(e)] = load(0, e);
    return;
  }
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = warp; t < tokens; t += warps) {
    float* row = dst + t * stride;
    for (int first = lane; first < length; first += 128) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (first + 32 * u < length) v[u] = load(t, first + 32 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (first + 32 * u < length) row[place(first + 32 * u)] = v[u];
    }
  }
}

// ONE_TOKEN: every request of the step brings exactly one token (a decode step).  The kernel
// then only loads a matrix, touches it once and stores it: its time is the state's bytes over
// what the SM keeps in flight, so the compiler is held to fewer registers (three CTAs an SM).
template <typename T, int ROWS_PER_THREAD, bool ONE_TOKEN>
__global__ __launch_bounds__(SCAN_THREADS, ONE_TOKEN ? 3 : HX_SCAN_CTAS)
void state_space_scan_kernel(const ScanArgs<T> a) {
  constexpr int STRIDE = run_stride<ROWS_PER_THREAD>();
  constexpr bool EXACT = sizeof(T) == 4;      // the float32 engine, see decayed_add_exact
  extern __shared__ float4 shared4[];
  float* shared = reinterpret_cast<float*>(shared4);
  hx_pdl_prologue();
  const int request = blockIdx.x;
  const int head = blockIdx.y;
  const int group = head / (a.heads / a.groups);
  const int start = a.request_start[request];
  const int count = ONE_TOKEN ? 1 : a.request_start[request + 1] - start;
  const int parts = a.parts;
  const int rows = a.rows;
  const int width = a.width;
  const int lane = blockIdx.z * a.block_lanes + threadIdx.x;    // among the head's lanes
  const int column = lane / parts;
  const int part = lane - column * parts;
  const bool live = column < width && threadIdx.x < a.block_lanes;
  // staged per token: B and C (parts runs each), x [width], step size, decay
  const int run = parts * STRIDE;
  const int per_token = a.per_token;
  const int lanes = width * parts;       // threads of a head that own state
  float* s_state = a.state + static_cast<size_t>(a.request_slot[request]) * a.state_stride +
                   static_cast<size_t>(head) * a.head_stride;
  float S[ROWS_PER_THREAD];
  float carry[EXACT ? ROWS_PER_THREAD : 1];
#pragma unroll
  for (int k = 0; k < ROWS_PER_THREAD; ++k) {
    const int n = part * ROWS_PER_THREAD + k;
    S[k] = (live && n < rows) ? s_state[static_cast<size_t>(k) * lanes + lane] : 0.0f;
    carry[EXACT ? k : 0] = 0.0f;
  }
  // rows the matrix does not have stay zero in the staged vectors: nothing is guarded below
  for (int i = threadIdx.x; i < (ONE_TOKEN ? 1 : a.tile) * per_token; i += blockDim.x)
    shared[i] = 0.0f;
  const float rate = expf(a.a_log[head]);
  const float bias = a.dt_bias[head];
  const float skip = a.skip[head];
  const size_t ld = a.ld;
  for (int base = 0; base < count; base += a.tile) {
    const int here = min(a.tile, count - base);
    const size_t first = static_cast<size_t>(start + base);
    __syncthreads();
    const T* b = a.b + first * ld + group * rows;
    const T* c = a.c + first * ld + group * rows;
    const T* x = a.x + first * ld + head * width;
    stage<ONE_TOKEN>(shared, per_token, here, rows,
          [&](int t, int e) { return hx_to_float<T>(b[t * ld + e]); }, padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + run, per_token, here, rows,
          [&](int t, int e) { return hx_to_float<T>(c[t * ld + e]); }, padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + 2 * run, per_token, here, width,
          [&](int t, int e) { return hx_to_float<T>(x[t * ld + e]); }, [](int e) { return e; });
    for (int t = threadIdx.x; t < here; t += blockDim.x) {
      const float step = softplus(hx_to_float<T>(a.dt[(first + t) * a.ld_dt + head]) + bias);
      shared[t * per_token + 2 * run + width] = step;
      shared[t * per_token + 2 * run + width + 1] = EXACT ? expm1f(-rate * step) : expf(-rate * step);
    }
    __syncthreads();
    float* y_out = a.y + first * (a.heads * width) + head * width + column;
#pragma unroll 1
    for (int t = 0; t < here; ++t) {
      const float* row = shared + t * per_token;
      const float4* b4 = reinterpret_cast<const float4*>(row + part * STRIDE);
      const float4* c4 = reinterpret_cast<const float4*>(row + run + part * STRIDE);
      const float step = row[2 * run + width];
      const float decay = row[2 * run + width + 1];
      const float xv = live ? row[2 * run + column] : 0.0f;
      const float push = step * xv;
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int q = 0; q < ROWS_PER_THREAD / 4; ++q) {
        const float4 bv = b4[q];
        const float4 cv = c4[q];
        if constexpr (EXACT) {       // `decay` holds decay - 1 here
          decayed_add_exact(S[4 * q + 0], carry[4 * q + 0], decay, bv.x * push);
          decayed_add_exact(S[4 * q + 1], carry[4 * q + 1], decay, bv.y * push);
          decayed_add_exact(S[4 * q + 2], carry[4 * q + 2], decay, bv.z * push);
          decayed_add_exact(S[4 * q + 3], carry[4 * q + 3], decay, bv.w * push);
          sum0 = fmaf(S[4 * q + 0] + carry[4 * q + 0], cv.x, sum0);
          sum1 = fmaf(S[4 * q + 1] + carry[4 * q + 1], cv.y, sum1);
          sum0 = fmaf(S[4 * q + 2] + carry[4 * q + 2], cv.z, sum0);
          sum1 = fmaf(S[4 * q + 3] + carry[4 * q + 3], cv.w, sum1);
        } else {
          S[4 * q + 0] = fmaf(decay, S[4 * q + 0], bv.x * push);
          S[4 * q + 1] = fmaf(decay, S[4 * q + 1], bv.y * push);
          S[4 * q + 2] = fmaf(decay, S[4 * q + 2], bv.z * push);
          S[4 * q + 3] = fmaf(decay, S[4 * q + 3], bv.w * push);
          sum0 = fmaf(S[4 * q + 0], cv.x, sum0);
          sum1 = fmaf(S[4 * q + 1], cv.y, sum1);
          sum0 = fmaf(S[4 * q + 2], cv.z, sum0);
          sum1 = fmaf(S[4 * q + 3], cv.w, sum1);
        }
      }
      float sum = sum0 + sum1;
      for (int offset = parts >> 1; offset > 0; offset >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0) y_out[static_cast<size_t>(t) * (a.heads * width)] = fmaf(skip, xv, sum);
    }
  }
  if (live) {
#pragma unroll
    for (int k = 0; k < ROWS_PER_THREAD; ++k) {
      const int n = part * ROWS_PER_THREAD + k;
      if (n < rows)
        s_state[static_cast<size_t>(k) * lanes + lane] = EXACT ? S[k] + carry[EXACT ? k : 0] : S[k];
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
  float* state;             // per slot: heads x head_stride, see the layout above
  long long state_stride;
  int head_stride;
  float* o;                 // [tokens, heads * dim]
  const int* request_start;
  const int* request_slot;
  int heads, dim;
  int parts, block_lanes, tile, per_token;
};

template <typename T, int ROWS_PER_THREAD, bool ONE_TOKEN>
__global__ __launch_bounds__(SCAN_THREADS, ONE_TOKEN ? 3 : HX_SCAN_CTAS)
void outer_product_scan_kernel(const OuterScanArgs<T> a) {
  constexpr int STRIDE = run_stride<ROWS_PER_THREAD>();
  constexpr bool EXACT = sizeof(T) == 4;      // the float32 engine, see decayed_add_exact
  extern __shared__ float4 shared4[];
  float* shared = reinterpret_cast<float*>(shared4);
  hx_pdl_prologue();
  const int request = blockIdx.x;
  const int head = blockIdx.y;
  const int start = a.request_start[request];
  const int count = ONE_TOKEN ? 1 : a.request_start[request + 1] - start;
  const int parts = a.parts;
  const int dim = a.dim;
  const int lane = blockIdx.z * a.block_lanes + threadIdx.x;
  const int column = lane / parts;
  const int part = lane - column * parts;
  const bool live = column < dim && threadIdx.x < a.block_lanes;
  // staged per token: r, k, w, bonus * k (parts runs each), v [dim]
  const int run = parts * STRIDE;
  const int per_token = a.per_token;
  const int lanes = dim * parts;
  float* s_state = a.state + static_cast<size_t>(a.request_slot[request]) * a.state_stride +
                   static_cast<size_t>(head) * a.head_stride;
  float S[ROWS_PER_THREAD];
  float carry[EXACT ? ROWS_PER_THREAD : 1];
#pragma unroll
  for (int i = 0; i < ROWS_PER_THREAD; ++i) {
    const int n = part * ROWS_PER_THREAD + i;
    S[i] = (live && n < dim) ? s_state[static_cast<size_t>(i) * lanes + lane] : 0.0f;
    carry[EXACT ? i : 0] = 0.0f;
  }
  for (int i = threadIdx.x; i < (ONE_TOKEN ? 1 : a.tile) * per_token; i += blockDim.x)
    shared[i] = 0.0f;
  const int channel0 = head * dim;
  for (int base = 0; base < count; base += a.tile) {
    const int here = min(a.tile, count - base);
    const size_t first = static_cast<size_t>(start + base);
    __syncthreads();
    const T* r = a.r + first * a.ld_r + channel0;
    const T* k = a.k + first * a.ld_k + channel0;
    const T* v = a.v + first * a.ld_v + channel0;
    const float* decay_log = a.decay_log + first * a.ld_decay + channel0;
    const float* w0 = a.w0 + channel0;
    const float* bonus = a.bonus + channel0;
    stage<ONE_TOKEN>(shared, per_token, here, dim,
          [&](int t, int e) { return hx_to_float<T>(r[static_cast<size_t>(t) * a.ld_r + e]); }, padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + run, per_token, here, dim,
          [&](int t, int e) { return hx_to_float<T>(k[static_cast<size_t>(t) * a.ld_k + e]); }, padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + 2 * run, per_token, here, dim,
          [&](int t, int e) {
            const float rate = expf(decay_log[static_cast<size_t>(t) * a.ld_decay + e] + w0[e]);
            return EXACT ? expm1f(-rate) : expf(-rate);
          },
          padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + 3 * run, per_token, here, dim,
          [&](int t, int e) {
            return bonus[e] * hx_to_float<T>(k[static_cast<size_t>(t) * a.ld_k + e]);
          },
          padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + 4 * run, per_token, here, dim,
          [&](int t, int e) { return hx_to_float<T>(v[static_cast<size_t>(t) * a.ld_v + e]); },
          [](int e) { return e; });
    __syncthreads();
    float* o_out = a.o + first * (a.heads * dim) + channel0 + column;
#pragma unroll 1
    for (int t = 0; t < here; ++t) {
      const float* row = shared + t * per_token;
      const float4* r4 = reinterpret_cast<const float4*>(row + part * STRIDE);
      const float4* k4 = reinterpret_cast<const float4*>(row + run + part * STRIDE);
      const float4* w4 = reinterpret_cast<const float4*>(row + 2 * run + part * STRIDE);
      const float4* u4 = reinterpret_cast<const float4*>(row + 3 * run + part * STRIDE);
      const float vj = live ? row[4 * run + column] : 0.0f;
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int q = 0; q < ROWS_PER_THREAD / 4; ++q) {
        const float4 rv = r4[q];
        const float4 kv = k4[q];
        const float4 wv = w4[q];
        const float4 uv = u4[q];          // bonus * k
        const float p0 = kv.x * vj, p1 = kv.y * vj, p2 = kv.z * vj, p3 = kv.w * vj;
        if constexpr (EXACT) {       // `wv` holds the decays minus one here
          sum0 = fmaf(rv.x, fmaf(uv.x, vj, S[4 * q + 0] + carry[4 * q + 0]), sum0);
          sum1 = fmaf(rv.y, fmaf(uv.y, vj, S[4 * q + 1] + carry[4 * q + 1]), sum1);
          sum0 = fmaf(rv.z, fmaf(uv.z, vj, S[4 * q + 2] + carry[4 * q + 2]), sum0);
          sum1 = fmaf(rv.w, fmaf(uv.w, vj, S[4 * q + 3] + carry[4 * q + 3]), sum1);
          decayed_add_exact(S[4 * q + 0], carry[4 * q + 0], wv.x, p0);
          decayed_add_exact(S[4 * q + 1], carry[4 * q + 1], wv.y, p1);
          decayed_add_exact(S[4 * q + 2], carry[4 * q + 2], wv.z, p2);
          decayed_add_exact(S[4 * q + 3], carry[4 * q + 3], wv.w, p3);
        } else {
          sum0 = fmaf(rv.x, fmaf(uv.x, vj, S[4 * q + 0]), sum0);
          sum1 = fmaf(rv.y, fmaf(uv.y, vj, S[4 * q + 1]), sum1);
          sum0 = fmaf(rv.z, fmaf(uv.z, vj, S[4 * q + 2]), sum0);
          sum1 = fmaf(rv.w, fmaf(uv.w, vj, S[4 * q + 3]), sum1);
          S[4 * q + 0] = fmaf(wv.x, S[4 * q + 0], p0);
          S[4 * q + 1] = fmaf(wv.y, S[4 * q + 1], p1);
          S[4 * q + 2] = fmaf(wv.z, S[4 * q + 2], p2);
          S[4 * q + 3] = fmaf(wv.w, S[4 * q + 3], p3);
        }
      }
      float sum = sum0 + sum1;
      for (int offset = parts >> 1; offset > 0; offset >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0) o_out[static_cast<size_t>(t) * (a.heads * dim)] = sum;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < ROWS_PER_THREAD; ++i) {
      const int n = part * ROWS_PER_THREAD + i;
      if (n < dim)
        s_state[static_cast<size_t>(i) * lanes + lane] = EXACT ? S[i] + carry[EXACT ? i : 0] : S[i];
    }
  }
}

// ------------------------------------------------- linear attention with a matrix state

// One [dim x vdim] matrix S per head, walked token by token, in two rules:
//   plain decay:  S <- g S + k v',                          o = S' q
//   delta rule:   S <- g S;  u = beta (v - S' k);  S <- S + k u';  o = S' q
// (the read-out sees the token's own write).  g is a constant of the head, or
// g = exp(-exp(A_h) softplus(a + bias_h)) from a projected column a; beta = sigmoid(b) from a
// projected column b.  Queries and keys arrive as projected (or filtered) rows and are made
// ready in float32 while a tile is staged: either turned into unit vectors per head
// (x / sqrt(sum x^2 + eps)) or rotated by their position over their first `rotary_dim`
// coordinates, then scaled by a constant each.  Several value heads may read one query/key
// head (head h reads h / (heads / qk_heads)).
template <typename T>
struct LinearStateArgs {
  const T* q;
  const T* k;
  const T* v;
  int ld_q, ld_k, ld_v;
  const T* decay_in;        // [tokens, ld_gates], column = head; null: the head's constant
  const T* beta_in;         // [tokens, ld_gates], column = head; null with the plain rule
  int ld_gates;
  const float* a_log;       // [heads]
  const float* dt_bias;     // [heads]
  const float* fixed_decay;     // [heads]: g, and
  const float* fixed_decay_m1;  // g - 1 rounded from double
  const int* positions;     // [tokens]; null: no rotation
  const float* freq;        // [rotary_dim / 2]
  const double* freq_exact; // the same in double (float32 engine)
  int rotary_dim, rotary_layout;   // layout 0: pairs (2i, 2i+1); 1: pairs (i, i + rotary_dim/2)
  int unit_norm;
  float unit_eps, q_scale, k_scale;
  float* state;
  long long state_stride;
  int head_stride;
  float* o;                 // [tokens, heads * vdim]
  const int* request_start;
  const int* request_slot;
  int heads, qk_heads, dim, vdim;
  int parts, block_lanes, tile, per_token;
};

template <typename T, bool DELTA, bool ONE_TOKEN>
__global__ __launch_bounds__(SCAN_THREADS, ONE_TOKEN ? 3 : HX_SCAN_CTAS)
void linear_state_scan_kernel(const LinearStateArgs<T> a) {
  constexpr int ROWS_PER_THREAD = 16;
  constexpr int STRIDE = run_stride<ROWS_PER_THREAD>();
  constexpr bool EXACT = sizeof(T) == 4;      // the float32 engine, see decayed_add_exact
  extern __shared__ float4 shared4[];
  float* shared = reinterpret_cast<float*>(shared4);
  hx_pdl_prologue();
  const int request = blockIdx.x;
  const int head = blockIdx.y;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int start = a.request_start[request];
  const int count = ONE_TOKEN ? 1 : a.request_start[request + 1] - start;
  const int parts = a.parts;
  const int dim = a.dim;
  const int vdim = a.vdim;
  const int lane = blockIdx.z * a.block_lanes + threadIdx.x;
  const int column = lane / parts;
  const int part = lane - column * parts;
  const bool live = column < vdim && threadIdx.x < a.block_lanes;
  // staged per token: q, k (parts runs each), v [vdim], decay, beta
  const int run = parts * STRIDE;
  const int per_token = a.per_token;
  const int lanes = vdim * parts;
  float* s_state = a.state + static_cast<size_t>(a.request_slot[request]) * a.state_stride +
                   static_cast<size_t>(head) * a.head_stride;
  float S[ROWS_PER_THREAD];
  float carry[EXACT ? ROWS_PER_THREAD : 1];
#pragma unroll
  for (int i = 0; i < ROWS_PER_THREAD; ++i) {
    const int n = part * ROWS_PER_THREAD + i;
    S[i] = (live && n < dim) ? s_state[static_cast<size_t>(i) * lanes + lane] : 0.0f;
    carry[EXACT ? i : 0] = 0.0f;
  }
  for (int i = threadIdx.x; i < (ONE_TOKEN ? 1 : a.tile) * per_token; i += blockDim.x)
    shared[i] = 0.0f;
  const float rate = a.decay_in != nullptr ? expf(a.a_log[head]) : 0.0f;
  const float bias = a.decay_in != nullptr ? a.dt_bias[head] : 0.0f;
  const float constant = a.decay_in != nullptr
                             ? 0.0f
                             : (EXACT ? a.fixed_decay_m1[head] : a.fixed_decay[head]);
  const bool rotate = a.positions != nullptr && a.rotary_dim > 0;
  const float load_q_scale = a.unit_norm ? 1.0f : a.q_scale;
  const float load_k_scale = a.unit_norm ? 1.0f : a.k_scale;
  for (int base = 0; base < count; base += a.tile) {
    const int here = min(a.tile, count - base);
    const size_t first = static_cast<size_t>(start + base);
    __syncthreads();
    const T* q = a.q + first * a.ld_q + qk_head * dim;
    const T* k = a.k + first * a.ld_k + qk_head * dim;
    const T* v = a.v + first * a.ld_v + head * vdim;
    auto prepared = [&](const T* rows, int ld, float scale) {
      return [=](int t, int e) -> float {
        float x = hx_to_float<T>(rows[static_cast<size_t>(t) * ld + e]);
        if (rotate && e < a.rotary_dim) {
          int pair, partner;
          bool leads;
          if (a.rotary_layout == 0) {
            pair = e >> 1; partner = e ^ 1; leads = (e & 1) == 0;
          } else {
            const int half = a.rotary_dim >> 1;
            leads = e < half;
            pair = leads ? e : e - half;
            partner = leads ? e + half : e - half;
          }
          const float y = hx_to_float<T>(rows[static_cast<size_t>(t) * ld + partner]);
          const int position = a.positions[first + t];
          float sine, cosine;
          if (EXACT) {
            double s, c;
            sincos(static_cast<double>(position) * a.freq_exact[pair], &s, &c);
            sine = static_cast<float>(s); cosine = static_cast<float>(c);
          } else {
            sincosf(static_cast<float>(position) * a.freq[pair], &sine, &cosine);
          }
          x = leads ? x * cosine - y * sine : x * cosine + y * sine;
        }
        return x * scale;
      };
    };
    stage<ONE_TOKEN>(shared, per_token, here, dim, prepared(q, a.ld_q, load_q_scale),
                     padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + run, per_token, here, dim, prepared(k, a.ld_k, load_k_scale),
                     padded<ROWS_PER_THREAD>);
    stage<ONE_TOKEN>(shared + 2 * run, per_token, here, vdim,
          [&](int t, int e) { return hx_to_float<T>(v[static_cast<size_t>(t) * a.ld_v + e]); },
          [](int e) { return e; });
    for (int t = threadIdx.x; t < here; t += blockDim.x) {
      float decay = constant, beta = 1.0f;
      if (a.decay_in != nullptr) {
        const float step =
            softplus(hx_to_float<T>(a.decay_in[(first + t) * a.ld_gates + head]) + bias);
        decay = EXACT ? expm1f(-rate * step) : expf(-rate * step);
      }
      if (DELTA) beta = hx_sigmoid(hx_to_float<T>(a.beta_in[(first + t) * a.ld_gates + head]));
      shared[t * per_token + 2 * run + vdim] = decay;
      shared[t * per_token + 2 * run + vdim + 1] = beta;
    }
    if (a.unit_norm) {
      // the padding between and behind the runs is zero, so the sums may run over all of it
      __syncthreads();
      const int warp = threadIdx.x >> 5, warps = blockDim.x >> 5, in_warp = threadIdx.x & 31;
      for (int t = warp; t < here; t += warps) {
        float* qrow = shared + t * per_token;
        float* krow = qrow + run;
        float sq = 0.0f, sk = 0.0f;
        for (int e = in_warp; e < run; e += 32) {
          sq = fmaf(qrow[e], qrow[e], sq);
          sk = fmaf(krow[e], krow[e], sk);
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
          sq += __shfl_xor_sync(0xffffffffu, sq, offset);
          sk += __shfl_xor_sync(0xffffffffu, sk, offset);
        }
        const float fq = a.q_scale / sqrtf(sq + a.unit_eps);
        const float fk = a.k_scale / sqrtf(sk + a.unit_eps);
        for (int e = in_warp; e < run; e += 32) {
          qrow[e] *= fq;
          krow[e] *= fk;
        }
      }
    }
    __syncthreads();
    float* o_out = a.o + first * (a.heads * vdim) + head * vdim + column;
#pragma unroll 1
    for (int t = 0; t < here; ++t) {
      const float* row = shared + t * per_token;
      const float4* q4 = reinterpret_cast<const float4*>(row + part * STRIDE);
      const float4* k4 = reinterpret_cast<const float4*>(row + run + part * STRIDE);
      const float vj = live ? row[2 * run + column] : 0.0f;
      const float decay = row[2 * run + vdim];     // EXACT: the decay minus one
      float u = vj;
      if (DELTA) {
        const float beta = row[2 * run + vdim + 1];
        float dot0 = 0.0f, dot1 = 0.0f;
#pragma unroll
        for (int c = 0; c < ROWS_PER_THREAD / 4; ++c) {
          const float4 kv = k4[c];
          if constexpr (EXACT) {
            dot0 = fmaf(S[4 * c + 0] + carry[4 * c + 0], kv.x, dot0);
            dot1 = fmaf(S[4 * c + 1] + carry[4 * c + 1], kv.y, dot1);
            dot0 = fmaf(S[4 * c + 2] + carry[4 * c + 2], kv.z, dot0);
            dot1 = fmaf(S[4 * c + 3] + carry[4 * c + 3], kv.w, dot1);
          } else {
            dot0 = fmaf(S[4 * c + 0], kv.x, dot0);
            dot1 = fmaf(S[4 * c + 1], kv.y, dot1);
            dot0 = fmaf(S[4 * c + 2], kv.z, dot0);
            dot1 = fmaf(S[4 * c + 3], kv.w, dot1);
          }
        }
        float dot = dot0 + dot1;
        for (int offset = parts >> 1; offset > 0; offset >>= 1)
          dot += __shfl_xor_sync(0xffffffffu, dot, offset);
        // what the decayed matrix holds for this key
        const float held = EXACT ? fmaf(decay, dot, dot) : decay * dot;
        u = beta * (vj - held);
      }
      float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
      for (int c = 0; c < ROWS_PER_THREAD / 4; ++c) {
        const float4 qv = q4[c];
        const float4 kv = k4[c];
        if constexpr (EXACT) {
          decayed_add_exact(S[4 * c + 0], carry[4 * c + 0], decay, kv.x * u);
          decayed_add_exact(S[4 * c + 1], carry[4 * c + 1], decay, kv.y * u);
          decayed_add_exact(S[4 * c + 2], carry[4 * c + 2], decay, kv.z * u);
          decayed_add_exact(S[4 * c + 3], carry[4 * c + 3], decay, kv.w * u);
          sum0 = fmaf(S[4 * c + 0] + carry[4 * c + 0], qv.x, sum0);
          sum1 = fmaf(S[4 * c + 1] + carry[4 * c + 1], qv.y, sum1);
          sum0 = fmaf(S[4 * c + 2] + carry[4 * c + 2], qv.z, sum0);
          sum1 = fmaf(S[4 * c + 3] + carry[4 * c + 3], qv.w, sum1);
        } else {
          S[4 * c + 0] = fmaf(decay, S[4 * c + 0], kv.x * u);
          S[4 * c + 1] = fmaf(decay, S[4 * c + 1], kv.y * u);
          S[4 * c + 2] = fmaf(decay, S[4 * c + 2], kv.z * u);
          S[4 * c + 3] = fmaf(decay, S[4 * c + 3], kv.w * u);
          sum0 = fmaf(S[4 * c + 0], qv.x, sum0);
          sum1 = fmaf(S[4 * c + 1], qv.y, sum1);
          sum0 = fmaf(S[4 * c + 2], qv.z, sum0);
          sum1 = fmaf(S[4 * c + 3], qv.w, sum1);
        }
      }
      float sum = sum0 + sum1;
      for (int offset = parts >> 1; offset > 0; offset >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0) o_out[static_cast<size_t>(t) * (a.heads * vdim)] = sum;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < ROWS_PER_THREAD; ++i) {
      const int n = part * ROWS_PER_THREAD + i;
      if (n < dim)
        s_state[static_cast<size_t>(i) * lanes + lane] = EXACT ? S[i] + carry[EXACT ? i : 0] : S[i];
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

// lanes that share a column: the smallest power of two that leaves a lane at most
// rows_per_thread(rows) rows; 0 when even a whole warp would not do
int parts_for(int rows) {
  for (int parts = 1; parts <= 32; parts <<= 1)
    if (parts * rows_per_thread(rows) >= rows) return parts;
  return 0;
}

int state_floats(int columns, int rows) {
  const int parts = parts_for(rows);
  return parts * rows_per_thread(rows) * columns;
}

// floats staged per token: `vectors` vectors of `rows` rows in padded runs, and `plain` more;
// a multiple of four, so that every token's runs start on 16 bytes
int staged_floats(int vectors, int rows, int plain) {
  const int rpt = rows_per_thread(rows);
  return (vectors * parts_for(rows) * (rpt + (rpt >= 8 ? 4 : 0)) + plain + 3) / 4 * 4;
}

// tokens staged per tile: a tile of at most HX_SCAN_TILE_KB kilobytes (below the 48 KB a CTA gets
// without asking), so that several CTAs share an SM
int tile_for(int floats_per_token) {
  const int budget = HX_SCAN_TILE_KB * 1024 / 4;
  int tile = budget / floats_per_token;
  if (tile > 32) tile = 32;
  return tile;
}

}  // namespace

// Floats a head's matrix of `rows` x `columns` takes in a request's state row.
HX_API int hx_scan_state_floats(int columns, int rows) { return state_floats(columns, rows); }

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
                               const float* skip, float* state, long long state_stride,
                               int head_stride, float* y, const int* request_start,
                               const int* request_slot, int requests, int tokens, int heads,
                               int width, int rows, int groups, cudaStream_t stream) {
  HX_REQUIRE(requests >= 0 && heads > 0 && width > 0 && rows > 0 && groups > 0,
             "hx_state_space_scan: bad sizes");
  HX_REQUIRE(heads % groups == 0, "hx_state_space_scan: heads must be a multiple of groups");
  const int parts = parts_for(rows);
  HX_REQUIRE(parts > 0, "hx_state_space_scan: a state of %d rows is more than %d", rows, 32 * 16);
  const int block_lanes = min(width, SCAN_THREADS / parts) * parts;
  const int threads = (block_lanes + 31) / 32 * 32;
  const int column_blocks = (width * parts + block_lanes - 1) / block_lanes;
  HX_REQUIRE(head_stride >= state_floats(width, rows),
             "hx_state_space_scan: a head's state takes %d floats, not %d", state_floats(width, rows),
             head_stride);
  const int per_token = staged_floats(2, rows, width + 2);
  const int tile = tile_for(per_token);
  HX_REQUIRE(tile >= 1, "hx_state_space_scan: a token's vectors do not fit shared memory");
  if (requests == 0) return HX_OK;
  const dim3 grid(requests, heads, column_blocks);
  const size_t shared_bytes = static_cast<size_t>(tile) * per_token * sizeof(float);
  const bool one_token = tokens == requests;      // every request brings at least one
  const size_t one_bytes = static_cast<size_t>(per_token) * sizeof(float);
  if (dtype == HX_F32) {
    ScanArgs<float> a{static_cast<const float*>(x), static_cast<const float*>(b),
                      static_cast<const float*>(c), ld, static_cast<const float*>(dt), ld_dt,
                      dt_bias, a_log, skip, state, state_stride, head_stride, y, request_start,
                      request_slot, heads, width, rows, groups, parts, block_lanes, tile, per_token};
    if (one_token) {
      switch (rows_per_thread(rows)) {
        case 4: hx_launch(state_space_scan_kernel<float, 4, true>, grid, threads, one_bytes, stream, a); break;
        case 8: hx_launch(state_space_scan_kernel<float, 8, true>, grid, threads, one_bytes, stream, a); break;
        default: hx_launch(state_space_scan_kernel<float, 16, true>, grid, threads, one_bytes, stream, a);
      }
    } else {
      switch (rows_per_thread(rows)) {
        case 4: hx_launch(state_space_scan_kernel<float, 4, false>, grid, threads, shared_bytes, stream, a); break;
        case 8: hx_launch(state_space_scan_kernel<float, 8, false>, grid, threads, shared_bytes, stream, a); break;
        default: hx_launch(state_space_scan_kernel<float, 16, false>, grid, threads, shared_bytes, stream, a);
      }
    }
  } else if (dtype == HX_BF16) {
    ScanArgs<__nv_bfloat16> a{static_cast<const __nv_bfloat16*>(x),
                              static_cast<const __nv_bfloat16*>(b),
                              static_cast<const __nv_bfloat16*>(c), ld,
                              static_cast<const __nv_bfloat16*>(dt), ld_dt, dt_bias, a_log, skip,
                              state, state_stride, head_stride, y, request_start, request_slot,
                              heads, width, rows, groups, parts, block_lanes, tile, per_token};
    if (one_token) {
      switch (rows_per_thread(rows)) {
        case 4: hx_launch(state_space_scan_kernel<__nv_bfloat16, 4, true>, grid, threads, one_bytes, stream, a); break;
        case 8: hx_launch(state_space_scan_kernel<__nv_bfloat16, 8, true>, grid, threads, one_bytes, stream, a); break;
        default: hx_launch(state_space_scan_kernel<__nv_bfloat16, 16, true>, grid, threads, one_bytes, stream, a);
      }
    } else {
      switch (rows_per_thread(rows)) {
        case 4: hx_launch(state_space_scan_kernel<__nv_bfloat16, 4, false>, grid, threads, shared_bytes, stream, a); break;
        case 8: hx_launch(state_space_scan_kernel<__nv_bfloat16, 8, false>, grid, threads, shared_bytes, stream, a); break;
        default: hx_launch(state_space_scan_kernel<__nv_bfloat16, 16, false>, grid, threads, shared_bytes, stream, a);
      }
    }
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
                                 long long state_stride, int head_stride, float* o,
                                 const int* request_start, const int* request_slot, int requests,
                                 int tokens, int heads, int dim, cudaStream_t stream) {
  HX_REQUIRE(requests >= 0 && heads > 0 && dim > 0, "hx_outer_product_scan: bad sizes");
  const int parts = parts_for(dim);
  HX_REQUIRE(parts > 0, "hx_outer_product_scan: heads of %d are more than %d", dim, 32 * 16);
  const int block_lanes = min(dim, SCAN_THREADS / parts) * parts;
  const int threads = (block_lanes + 31) / 32 * 32;
  const int column_blocks = (dim * parts + block_lanes - 1) / block_lanes;
  HX_REQUIRE(head_stride >= state_floats(dim, dim),
             "hx_outer_product_scan: a head's state takes %d floats, not %d", state_floats(dim, dim),
             head_stride);
  const int per_token = staged_floats(4, dim, dim);
  const int tile = tile_for(per_token);
  HX_REQUIRE(tile >= 1, "hx_outer_product_scan: a token's vectors do not fit shared memory");
  if (requests == 0) return HX_OK;
  const dim3 grid(requests, heads, column_blocks);
  const size_t shared_bytes = static_cast<size_t>(tile) * per_token * sizeof(float);
  const bool one_token = tokens == requests;
  const size_t one_bytes = static_cast<size_t>(per_token) * sizeof(float);
  if (dtype == HX_F32) {
    OuterScanArgs<float> a{static_cast<const float*>(r), static_cast<const float*>(k),
                           static_cast<const float*>(v), ld_r, ld_k, ld_v, decay_log, ld_decay, w0,
                           bonus, state, state_stride, head_stride, o, request_start, request_slot,
                           heads, dim, parts, block_lanes, tile, per_token};
    if (one_token) {
      switch (rows_per_thread(dim)) {
        case 4: hx_launch(outer_product_scan_kernel<float, 4, true>, grid, threads, one_bytes, stream, a); break;
        case 8: hx_launch(outer_product_scan_kernel<float, 8, true>, grid, threads, one_bytes, stream, a); break;
        default: hx_launch(outer_product_scan_kernel<float, 16, true>, grid, threads, one_bytes, stream, a);
      }
    } else {
      switch (rows_per_thread(dim)) {
        case 4: hx_launch(outer_product_scan_kernel<float, 4, false>, grid, threads, shared_bytes, stream, a); break;
        case 8: hx_launch(outer_product_scan_kernel<float, 8, false>, grid, threads, shared_bytes, stream, a); break;
        default: hx_launch(outer_product_scan_kernel<float, 16, false>, grid, threads, shared_bytes, stream, a);
      }
    }
  } else if (dtype == HX_BF16) {
    OuterScanArgs<__nv_bfloat16> a{static_cast<const __nv_bfloat16*>(r),
                                   static_cast<const __nv_bfloat16*>(k),
                                   static_cast<const __nv_bfloat16*>(v), ld_r, ld_k, ld_v,
                                   decay_log, ld_decay, w0, bonus, state, state_stride,
                                   head_stride, o, request_start, request_slot, heads, dim, parts,
                                   block_lanes, tile, per_token};
    if (one_token) {
      switch (rows_per_thread(dim)) {
        case 4: hx_launch(outer_product_scan_kernel<__nv_bfloat16, 4, true>, grid, threads, one_bytes, stream, a); break;
        case 8: hx_launch(outer_product_scan_kernel<__nv_bfloat16, 8, true>, grid, threads, one_bytes, stream, a); break;
        default: hx_launch(outer_product_scan_kernel<__nv_bfloat16, 16, true>, grid, threads, one_bytes, stream, a);
      }
    } else {
      switch (rows_per_thread(dim)) {
        case 4: hx_launch(outer_product_scan_kernel<__nv_bfloat16, 4, false>, grid, threads, shared_bytes, stream, a); break;
        case 8: hx_launch(outer_product_scan_kernel<__nv_bfloat16, 8, false>, grid, threads, shared_bytes, stream, a); break;
        default: hx_launch(outer_product_scan_kernel<__nv_bfloat16, 16, false>, grid, threads, shared_bytes, stream, a);
      }
    }
  } else {
    HX_REQUIRE(false, "hx_outer_product_scan: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_outer_product_scan");
  return HX_OK;
}

namespace {
template <typename T>
void launch_linear_state(const LinearStateArgs<T>& a, bool delta, bool one_token, dim3 grid,
                         int threads, size_t shared_bytes, size_t one_bytes, cudaStream_t stream) {
  if (delta) {
    if (one_token) hx_launch(linear_state_scan_kernel<T, true, true>, grid, threads, one_bytes, stream, a);
    else hx_launch(linear_state_scan_kernel<T, true, false>, grid, threads, shared_bytes, stream, a);
  } else {
    if (one_token) hx_launch(linear_state_scan_kernel<T, false, true>, grid, threads, one_bytes, stream, a);
    else hx_launch(linear_state_scan_kernel<T, false, false>, grid, threads, shared_bytes, stream, a);
  }
}
}  // namespace

// Linear attention with a [dim x vdim] matrix per head (see LinearStateArgs).  q, k
// [tokens, qk_heads * dim] and v [tokens, heads * vdim] in the compute dtype; `decay_in` and
// `beta_in` are columns of projected rows (one per head) or null (then `fixed_decay` and
// `fixed_decay_m1` [heads] give the head's constant decay and the same minus one);
// delta != 0 needs `beta_in`.  Rotation: `positions` with `freq` (and `freq_exact` in the
// float32 engine), or null.  o [tokens, heads * vdim] float32.
HX_API int hx_linear_state_scan(const void* q, int ld_q, const void* k, int ld_k, const void* v,
                                int ld_v, int dtype, int delta, const void* decay_in,
                                const void* beta_in, int ld_gates, const float* a_log,
                                const float* dt_bias, const float* fixed_decay,
                                const float* fixed_decay_m1, const int* positions,
                                const float* freq, const double* freq_exact, int rotary_dim,
                                int rotary_layout, int unit_norm, float unit_eps, float q_scale,
                                float k_scale, float* state, long long state_stride,
                                int head_stride, float* o, const int* request_start,
                                const int* request_slot, int requests, int tokens, int heads,
                                int qk_heads, int dim, int vdim, cudaStream_t stream) {
  HX_REQUIRE(requests >= 0 && heads > 0 && qk_heads > 0 && dim > 0 && vdim > 0,
             "hx_linear_state_scan: bad sizes");
  HX_REQUIRE(heads % qk_heads == 0,
             "hx_linear_state_scan: heads must be a multiple of the query/key heads");
  HX_REQUIRE(!delta || beta_in != nullptr, "hx_linear_state_scan: the delta rule needs beta");
  HX_REQUIRE(decay_in != nullptr ? (a_log != nullptr && dt_bias != nullptr)
                                 : (fixed_decay != nullptr && fixed_decay_m1 != nullptr),
             "hx_linear_state_scan: a decay needs its rate and bias, or the heads' constants");
  HX_REQUIRE(positions == nullptr || rotary_dim == 0 ||
                 (rotary_dim % 2 == 0 && rotary_dim <= dim && freq != nullptr &&
                  (dtype != HX_F32 || freq_exact != nullptr)),
             "hx_linear_state_scan: rotation over %d of %d coordinates", rotary_dim, dim);
  const int parts = parts_for(dim);
  HX_REQUIRE(parts > 0, "hx_linear_state_scan: heads of %d are more than %d", dim, 32 * 16);
  const int block_lanes = min(vdim, SCAN_THREADS / parts) * parts;
  const int threads = (block_lanes + 31) / 32 * 32;
  const int column_blocks = (vdim * parts + block_lanes - 1) / block_lanes;
  HX_REQUIRE(head_stride >= state_floats(vdim, dim),
             "hx_linear_state_scan: a head's state takes %d floats, not %d", state_floats(vdim, dim),
             head_stride);
  const int per_token = staged_floats(2, dim, vdim + 2);
  const int tile = tile_for(per_token);
  HX_REQUIRE(tile >= 1, "hx_linear_state_scan: a token's vectors do not fit shared memory");
  if (requests == 0) return HX_OK;
  const dim3 grid(requests, heads, column_blocks);
  const size_t shared_bytes = static_cast<size_t>(tile) * per_token * sizeof(float);
  const bool one_token = tokens == requests;
  const size_t one_bytes = static_cast<size_t>(per_token) * sizeof(float);
  if (dtype == HX_F32) {
    LinearStateArgs<float> a{static_cast<const float*>(q), static_cast<const float*>(k),
                             static_cast<const float*>(v), ld_q, ld_k, ld_v,
                             static_cast<const float*>(decay_in), static_cast<const float*>(beta_in),
                             ld_gates, a_log, dt_bias, fixed_decay, fixed_decay_m1, positions, freq,
                             freq_exact, rotary_dim, rotary_layout, unit_norm, unit_eps, q_scale,
                             k_scale, state, state_stride, head_stride, o, request_start,
                             request_slot, heads, qk_heads, dim, vdim, parts, block_lanes, tile,
                             per_token};
    launch_linear_state(a, delta != 0, one_token, grid, threads, shared_bytes, one_bytes, stream);
  } else if (dtype == HX_BF16) {
    LinearStateArgs<__nv_bfloat16> a{
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
        static_cast<const __nv_bfloat16*>(v), ld_q, ld_k, ld_v,
        static_cast<const __nv_bfloat16*>(decay_in), static_cast<const __nv_bfloat16*>(beta_in),
        ld_gates, a_log, dt_bias, fixed_decay, fixed_decay_m1, positions, freq, freq_exact,
        rotary_dim, rotary_layout, unit_norm, unit_eps, q_scale, k_scale, state, state_stride,
        head_stride, o, request_start, request_slot, heads, qk_heads, dim, vdim, parts,
        block_lanes, tile, per_token};
    launch_linear_state(a, delta != 0, one_token, grid, threads, shared_bytes, one_bytes, stream);
  } else {
    HX_REQUIRE(false, "hx_linear_state_scan: unknown dtype %d", dtype);
  }
  HX_CHECK_LAUNCH("hx_linear_state_scan");
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
