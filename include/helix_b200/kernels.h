/* helix_b200/kernels.h: the C interface of the sm_100a kernel library.
 *
 * The engine's entry points for users are the Python package (helix_runtime_b200.Engine) and
 * the command line (bin/helix_generate); the reference exposes its engine to C++ through
 * include/helix (README.md:199-209).  What this project offers to C and C++ callers is the
 * layer below: every kernel the engine runs, as a plain C function of the shared library the
 * package builds (helix_runtime_b200/csrc/_build/libhelix_b200_<hash>.so; CUDA runtime linked
 * statically).  The Python side calls exactly these symbols through ctypes.
 *
 * Conventions.  Every function takes raw device pointers, sizes and the stream to launch on;
 * it allocates nothing (scratch is the caller's; see hx_paged_attention_no_alloc for the one
 * exception that brings its own) and never synchronises.  It returns 0, or a negative code
 * (HX_RC_*) and leaves a message for hx_last_error().  Sizes a kernel cannot run are refused
 * on the host, before any launch: never a wrong result.  Kernels that can detect a bad input
 * on the device (a token id outside the vocabulary, a page number outside the pool, a bounded
 * wait that ran out, a non-finite logit, a position beyond the rotary table) OR a bit into the caller's `status` word
 * (HX_STATUS_*), which the host reads after the step.
 *
 * dtype codes: HX_F32 = 0, HX_BF16 = 1.  Matrices are [rows, row stride] row-major; weights
 * are [out_features, in_features] ("K-major").  Epilogues of the products: 0 store in the
 * activation dtype, 1 store float32, 2 add into float32, 3 SwiGLU (tensor cores only).
 *
 * Cache layout of one layer, keys and values alike:
 *   [page][kv_head][head_dim / c][slot][c]   with c = hx_cache_chunk_elements(dtype, head_dim)
 * (16 bytes of elements when the head size allows), so the keys of a (page, head) are one
 * contiguous block.  Block tables are int32 [rows, table_stride], -1 = no page.
 */
#ifndef HELIX_B200_KERNELS_H
#define HELIX_B200_KERNELS_H

#ifdef __CUDACC__
#include <cuda_runtime.h>
#else
typedef struct CUstream_st* cudaStream_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define HX_RC_ARGUMENT (-1)
#define HX_RC_LAUNCH (-2)
#define HX_RC_UNSUPPORTED (-3)

#define HX_DTYPE_F32 0
#define HX_DTYPE_BF16 1

#define HX_STATUS_BAD_TOKEN 1
#define HX_STATUS_BAD_PAGE 2
#define HX_STATUS_WAIT_TIMEOUT 4
#define HX_STATUS_NONFINITE 8
#define HX_STATUS_BAD_POSITION 16

/* ---- library ---------------------------------------------------------------------------- */
int hx_abi_version(void);
int hx_sm_count(void);                     /* multiprocessors of the current device, 0 on error */
const char* hx_last_error(void);          /* message of this thread's last failed call */
long long hx_launch_count(void);          /* kernels launched by this library so far */
void hx_set_dependent_launch(int enabled); /* programmatic dependent launch between kernels */
/* the kernels' bounded mbarrier wait on a barrier of its own, limited to `polls` polls
   (1..1,000,000): with arrive = 0 it runs out, sets HX_STATUS_WAIT_TIMEOUT in *status and the
   kernel returns; *succeeded (may be null) receives 1 or 0 */
int hx_bounded_wait_check(int polls, int arrive, int* status, int* succeeded, cudaStream_t stream);

/* ---- embedding, norm, activation ------------------------------------------------------- */
/* out[t, :] = table[ids[t], :] as float32 (the residual stream) */
int hx_embed(const void* table, int dtype, const int* ids, float* out, int tokens, int hidden,
             int vocab, int* status, cudaStream_t stream);
/* the same times a constant: out[t, :] = table[ids[t], :] * scale, the product in float32 */
int hx_embed_scaled(const void* table, int dtype, const int* ids, float* out, int tokens,
                    int hidden, int vocab, float scale, int* status, cudaStream_t stream);
/* x[t, :] += y[t, :], float32 rows of `hidden` */
int hx_add_rows(float* x, const float* y, int tokens, int hidden, cudaStream_t stream);
/* y[r, :] = (x[r', :] - mean) / sqrt(var + eps) * weight + bias, r' = rows ? rows[r] : r, var the
   mean of the squared deviations, float32 inside; bias may be null */
int hx_layernorm(const float* x, const float* weight, const float* bias, void* y, int out_dtype,
                 const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream);
/* y[r, :] = x[rows ? rows[r] : r, :] * rsqrt(mean(x^2) + eps) * weight, float32 inside */
int hx_rmsnorm(const float* x, const float* weight, void* y, int out_dtype, const int* rows,
               int n_rows, int hidden, float eps, cudaStream_t stream);
/* act[t, f] = silu(gate_up[t, f]) * gate_up[t, intermediate + f]; zero_input clears gate_up */
int hx_swiglu(float* gate_up, void* act, int out_dtype, int tokens, int intermediate, int ld_in,
              int zero_input, cudaStream_t stream);

/* act[t, f] = g(gate_up[t, f]) * gate_up[t, intermediate + f]; activation 0: g = silu,
   1: g = the tanh approximation of GELU, z * sigmoid(2 c (z + a z^3)) with c = sqrt(2/pi),
   a = 0.044715 */
int hx_gated_activation(float* gate_up, void* act, int out_dtype, int tokens, int intermediate,
                        int ld_in, int zero_input, int activation, cudaStream_t stream);
/* the same with biases on gate and up (either may be null) and two more activations: 2: g =
   relu; 3: the clamped form with its limit L, min(gate, L) * sigmoid(1.702 min(gate, L)) *
   (clamp(up, -L, L) + 1) */
int hx_biased_gated_activation(float* gate_up, const float* gate_bias, const float* up_bias,
                               void* act, int out_dtype, int tokens, int intermediate, int ld_in,
                               int zero_input, int activation, float limit, cudaStream_t stream);
/* context[t, :width] *= sigmoid(gate[t, :width]); clear (may be null): float32 rows
   [tokens, clear_width] that are zeroed afterwards */
int hx_sigmoid_gate(void* context, int ld_context, const void* gate, int ld_gate, int dtype,
                    int tokens, int width, float* clear, int ld_clear, int clear_width,
                    cudaStream_t stream);

/* ---- short causal filter over time + cache append --------------------------------------- */
/* row = [q heads | k heads | v heads | passthrough], `total` columns; every q/k/v channel c is
 * filtered along its sequence, y[t] = sum_j filter[c, j] * u[t - (taps - 1) + j], zeros before
 * the sequence; state[slot, taps - 1, channels] carries each request's last projected values
 * from step to step.  raw (storage dtype) or accum (float32 sums, left uncleared) is given.
 * Queries and passthrough columns go to `out`, keys and values to their pages when
 * write_cache, else to `out` as well. */
int hx_short_conv_append(const void* raw, int ld_raw, const float* accum, int ld_accum, void* out,
                         int ld_out, int dtype, const float* filter, void* state, int taps,
                         const int* positions, const int* token_request, const int* request_slot,
                         const int* request_start, const int* block_tables, int table_stride,
                         void* k_cache, void* v_cache, int write_cache, int tokens, int heads,
                         int kv_heads, int head_dim, int total, int page_size, int num_pages,
                         int* status, cudaStream_t stream);

/* ---- residual streams, sums around them, biased activation ------------------------------ */
/* A token's `count` residual streams lie side by side: streams[token][s][hidden], float32. */
int hx_streams_spread(const float* x, float* streams, int tokens, int hidden, int count,
                      cudaStream_t stream);
/* out[r] = rmsnorm(sum_s read[s] * streams[rows ? rows[r] : r][s]) * weight (read NULL: ones);
 * clear (may be NULL): float32 rows [n_rows, hidden] that are zeroed, or set to initial [hidden]
 * when that is given */
int hx_streams_read_norm(const float* streams, const float* read, int count, const float* weight,
                         void* out, int out_dtype, float* clear, const float* initial,
                         const int* rows, int n_rows, int hidden, float eps, cudaStream_t stream);
/* streams[t][r] = sum_s mixing[s][r] * streams[t][s] + write[r] * scale[c] * y[t][c], all r at
 * once from the old streams (mixing, write, scale NULL: ones) */
int hx_streams_write(float* streams, const float* y, const float* mixing, const float* write,
                     const float* scale, int count, int tokens, int hidden, cudaStream_t stream);
/* x += sum_i scales[i] * sources[i] (host arrays of `count` <= 4); the sources are zeroed */
int hx_scaled_sum(float* x, float* const* sources, const float* scales, int count, int tokens,
                  int width, cudaStream_t stream);
int hx_add_bias(float* x, const float* bias, int tokens, int width, cudaStream_t stream);
/* out = f(in + bias); activation 0: xIELU with p0 = softplus(p), p1 = 1/2 + softplus(q)
 * (z > 0: p0 z^2 + z/2; else p1 (exp(z) - 1 - z) + z/2); 1: tanh */
int hx_biased_activation(const float* in, int ld_in, const float* bias, void* out, int ld_out,
                         int out_dtype, int tokens, int width, int activation, float p0, float p1,
                         cudaStream_t stream);

/* ---- recurrent mixers ------------------------------------------------------------------ */
/* Per-request state is float32, `state + slot * state_stride`, zero at admission. */
/* out[t][c] = f(bias[c] + sum_j taps[c][j] * raw[t - (n - 1) + j][c]) along each request; the
 * state holds the last n - 1 inputs [n - 1][channels]; silu != 0: f = silu */
int hx_causal_filter(const void* raw, int ld_raw, void* out, int ld_out, int dtype,
                     const float* taps_weight, const float* bias, float* state,
                     long long state_stride, int taps, int channels, int silu, int tokens,
                     const int* token_request, const int* request_slot, const int* request_start,
                     cudaStream_t stream);
/* floats that a head's rows x columns matrix takes in a state row (the kernels' own order) */
int hx_scan_state_floats(int columns, int rows);
/* per head: S = exp(-exp(a_log) d) S + d B x', y = S' C + skip x, d = softplus(dt + dt_bias);
 * state: heads x head_stride floats; y float32 [tokens][heads * width]; tokens == requests
 * (a decode step) takes the kernel built for one token per request */
int hx_state_space_scan(const void* x, const void* b, const void* c, int ld, const void* dt,
                        int ld_dt, int dtype, const float* dt_bias, const float* a_log,
                        const float* skip, float* state, long long state_stride, int head_stride,
                        float* y, const int* request_start, const int* request_slot, int requests,
                        int tokens, int heads, int width, int rows, int groups,
                        cudaStream_t stream);
/* out[s][t] = h[t] + (h[t-1] - h[t]) * mu[s]; the state row [hidden] is the previous step's
 * last row and becomes this step's */
int hx_token_shift(const void* h, int ld, int dtype, const float* mu, int mixes, void* out,
                   long long mix_stride, float* state, long long state_stride, int tokens,
                   int hidden, const int* token_request, const int* request_slot,
                   const int* request_start, cudaStream_t stream);
/* per head: o = (S + diag(bonus) k v')' r, then S = diag(w) S + k v', w = exp(-exp(decay_log +
 * w0)); state: heads x head_stride floats; o float32 */
int hx_outer_product_scan(const void* r, int ld_r, const void* k, int ld_k, const void* v,
                          int ld_v, int dtype, const float* decay_log, int ld_decay,
                          const float* w0, const float* bonus, float* state,
                          long long state_stride, int head_stride, float* o,
                          const int* request_start,
                          const int* request_slot, int requests, int tokens, int heads, int dim,
                          cudaStream_t stream);
/* linear attention with a dim x vdim matrix per head.  delta == 0: S = g S + k v', o = S' q;
 * delta != 0: S = g S, u = beta (v - S' k), S += k u', o = S' q.  g: exp(-exp(a_log) *
 * softplus(decay_in + dt_bias)) from a projected column per head, or the constants fixed_decay
 * (with fixed_decay_m1 = fixed_decay - 1) when decay_in is null; beta = sigmoid(beta_in).
 * Before the recurrence q and k may be rotated by the position (positions + freq, freq_exact
 * in the float32 engine; layout 0 interleaved, 1 halves), made unit vectors (unit_norm:
 * x / sqrt(sum x^2 + unit_eps)) and scaled.  Head h reads q/k head h / (heads / qk_heads);
 * o float32 [tokens][heads * vdim] */
int hx_linear_state_scan(const void* q, int ld_q, const void* k, int ld_k, const void* v,
                         int ld_v, int dtype, int delta, const void* decay_in,
                         const void* beta_in, int ld_gates, const float* a_log,
                         const float* dt_bias, const float* fixed_decay,
                         const float* fixed_decay_m1, const int* positions, const float* freq,
                         const double* freq_exact, int rotary_dim, int rotary_layout,
                         int unit_norm, float unit_eps, float q_scale, float k_scale,
                         float* state, long long state_stride, int head_stride, float* o,
                         const int* request_start, const int* request_slot, int requests,
                         int tokens, int heads, int qk_heads, int dim, int vdim,
                         cudaStream_t stream);
/* channels in `groups` equal parts, each over its root mean square, times weight; the gate
 * silu(gate) multiplies before the norm (gate_after 0) or after it (1) */
int hx_gated_group_norm(const float* y, int ld_y, const void* gate, int ld_gate, int dtype,
                        const float* weight, void* out, int ld_out, int tokens, int channels,
                        int groups, float eps, int gate_after, cudaStream_t stream);

/* ---- gated connection, joined streams --------------------------------------------------- */
/* residual[t][c] += output[t][c] * sigmoid(gate[t][c] + bias[c]), all float32 */
int hx_gated_residual_add(float* residual, const float* output, const float* gate, int ld_gate,
                          const float* bias, int tokens, int width, cudaStream_t stream);
/* out[t] = [a[t] | b[t]] in the compute dtype (a, b float32 [tokens][width]) */
int hx_join_rows(const float* a, const float* b, void* out, int ld_out, int dtype, int tokens,
                 int width, cudaStream_t stream);

/* ---- norms between a product and what follows it ---------------------------------------- */
/* residual[t] += mult * y[t] / sqrt(mean(y[t]^2) + eps) * weight (float32 [tokens][width]);
 * cast_out (may be null): the updated rows in `dtype` */
int hx_norm_residual_add(float* residual, const float* y, const float* weight, float eps,
                         float mult, void* cast_out, int ld_cast, int dtype, int tokens, int width,
                         cudaStream_t stream);
/* projected float32 = [heads * head_dim q | kv_heads * head_dim k | kv_heads * value_dim v |
 * heads gate sums (with gates)]: biases (may be null), one RMS norm over ALL of a token's q
 * and one over all of its k (weights null: none), q times 1 + temp_coef * ln(floor((p + 1) /
 * temp_every) + 1) (temp_every 0: none), value_mix 1: v is stored in value_source, 2: v <- (1 -
 * lambda) v + lambda value_source; rows = [heads | kv_heads | kv_heads] rows of row_dim in
 * `dtype`; gates (may be null) [tokens][heads] = sigmoid of the gate sums; clear: projected is
 * left zero; with k_cache the keys and values are appended to the token's pages (as
 * hx_rope_append does) instead of written to `rows` */
int hx_biased_normed_rows(float* projected, int ld_projected, int clear, const float* q_bias,
                          const float* k_bias, const float* v_bias, const float* q_weight,
                          const float* k_weight, float eps, const int* positions, float temp_coef,
                          int temp_every, int value_mix, float lambda, float* value_source,
                          void* rows, int ld_rows, float* gates, int dtype, int tokens, int heads,
                          int kv_heads, int head_dim, int value_dim, int row_dim,
                          const int* token_request, const int* request_table_row,
                          const int* block_tables, int table_stride, void* k_cache, void* v_cache,
                          int page_size, int num_pages, int* status, cudaStream_t stream);
/* context[t][h * row_dim + c] *= gates[t][h] */
int hx_head_gate(void* context, int ld_context, const float* gates, int dtype, int tokens,
                 int heads, int row_dim, cudaStream_t stream);
/* out[t][c] = gelu_tanh(sums[t][c]) * table[token_ids[t]][offset + c], c < dim */
int hx_token_gate(float* sums, int ld_sums, int clear, const void* table, int ld_table, int offset,
                  int vocab, const int* token_ids, void* out, int ld_out, int dtype, int tokens,
                  int dim, int* status, cudaStream_t stream);

/* ---- routed experts --------------------------------------------------------------------- */
/* s = sigmoid(sums); the `top` largest (lowest index among equals); weights s / (sum of the
 * chosen + 1e-20) * scale; chosen and weights [tokens][top] */
int hx_route_top(const float* sums, int ld, int tokens, int experts, int top, float scale,
                 int* chosen, float* weights, cudaStream_t stream);
/* the same by a rule: softmax != 0: s = softmax(sums) over all `experts` outputs; correction
 * [experts] (may be null) is added to s for the choice only; normalize 0: weights s * scale */
int hx_route_top_ruled(const float* sums, int ld, int tokens, int experts, int top, float scale,
                       int softmax, const float* correction, int normalize, int* chosen,
                       float* weights, cudaStream_t stream);
/* act[t * top + k] = f(Wg[e] x[t]) * (Wu[e] x[t]), e = chosen[t][k]; gate_up [experts][2 ff]
 * [width] (gate rows first) */
int hx_expert_gate_up(const void* x, int ld_x, const void* gate_up, const int* chosen, void* act,
                      int dtype, int tokens, int top, int ff, int width, int experts,
                      int activation, cudaStream_t stream);
/* the same for every gate activation of hx_biased_gated_activation, with the clamped form's limit */
int hx_expert_gate_up_limited(const void* x, int ld_x, const void* gate_up, const int* chosen,
                              void* act, int dtype, int tokens, int top, int ff, int width,
                              int experts, int activation, float limit, cudaStream_t stream);
/* out[t] += sum_k weights[t][k] * Wd[chosen[t][k]] act[t * top + k], k ascending; out float32 */
int hx_expert_down(const void* act, const void* down, const int* chosen, const float* weights,
                   float* out, int ld_out, int dtype, int tokens, int top, int ff, int width,
                   int experts, cudaStream_t stream);

/* The pairs (token, choice) of a step sorted by expert, every expert's rows a whole number of
 * tiles: pair_row[pair] (-1: no valid expert), tile_group[t] the expert of tile t (-1 behind
 * the last in use); max_tiles >= hx_expert_tile_bound(pairs, experts, tile) */
int hx_expert_tile_bound(int pairs, int experts, int tile);
int hx_expert_rows(const int* chosen, int pairs, int experts, int tile, int max_tiles,
                   int* pair_row, int* tile_group, cudaStream_t stream);
/* grouped[pair_row[t * top + k]] = x[t] */
int hx_expert_gather(const void* x, int ld_x, const int* pair_row, void* grouped, int ld_grouped,
                     int dtype, int tokens, int top, int width, cudaStream_t stream);
/* out[t] += sum_k weights[t][k] * y[pair_row[t * top + k]], k ascending; y, out float32 */
int hx_expert_combine(const float* y, int ld_y, const int* pair_row, const float* weights,
                      float* out, int ld_out, int tokens, int top, int width,
                      cudaStream_t stream);
/* out[t] += x[t] * (sum of weights[t][k] over the choices with chosen[t][k] >= experts): router
 * outputs behind the experts return their input */
int hx_expert_identity_add(const void* x, int ld_x, const int* chosen, const float* weights,
                           float* out, int ld_out, int dtype, int tokens, int top, int width,
                           int experts, cudaStream_t stream);

/* ---- attention over a cached latent ----------------------------------------------------- */
/* down [tokens][q_rank + kv_rank + rot] float32: both latents RMS-normed with a weight; the
 * query latent goes to query_latent; the key row [c | rot(kr) | 0..] and the value row
 * [c | 0..] (row_dim wide each) go to `rows` at key_offset and behind it */
int hx_latent_prepare(const float* down, int ld_down, const float* q_weight,
                      const float* kv_weight, float eps, const int* positions, const float* freq,
                      const double* freq_exact, int rotary_dims, int layout, void* query_latent,
                      int ld_latent, void* rows, int ld_rows, int key_offset, int dtype,
                      int tokens, int q_rank, int kv_rank, int rot, int row_dim, float amplitude,
                      cudaStream_t stream);
/* (amplitude: a factor on sine and cosine, 1 unless the frequencies are stretched) */
/* every head's rotated query part (q at rot_offset inside a head), turned by the position,
 * behind the head's kv_rank latent coordinates in `rows`, zeros to row_dim */
int hx_latent_queries(const void* q, int ld_q, int rot_offset, void* rows, int ld_rows,
                      const int* positions, const float* freq, const double* freq_exact,
                      int rotary_dims, int layout, int dtype, int tokens, int heads, int kv_rank,
                      int rot, int row_dim, float amplitude, cudaStream_t stream);
/* out[t][h * out_stride + o] = sum_i w[h][o][i] * x[t][h * x_stride + i] */
int hx_head_products(const void* x, int ld_x, int x_stride, const void* w, void* out, int ld_out,
                     int out_stride, int dtype, int tokens, int heads, int out_dim, int in_dim,
                     cudaStream_t stream);

/* ---- rotation from positions, normed heads, rotated values + cache append --------------- */
/* heads are row_dim wide (head_dim / value_dim real coordinates); q_norm, k_norm (both or
 * neither): per-head RMS norm before the rotation; freq [rotary_dim / 2]; value_freq
 * [value_dim / 2] or NULL (values stored as projected); layout 0: pairs (2m, 2m+1), 1:
 * (m, m + dims/2); accum as for hx_rope_append */
int hx_norm_rotary_append(void* qkv, int dtype, int ld, float* accum, int ld_accum,
                          const int* positions, const int* token_request,
                          const int* request_table_row, const int* block_tables, int table_stride,
                          void* k_cache, void* v_cache, int write_cache, const float* freq,
                          const float* value_freq, const float* q_norm, const float* k_norm,
                          float eps, int tokens, int heads, int kv_heads, int head_dim,
                          int value_dim, int row_dim, int rotary_dim, int layout, int value_layout,
                          int page_size, int num_pages, int* status, cudaStream_t stream);
/* every head of rows[t] turned by minus positions[t] over its first `dims` coordinates */
int hx_rotate_back(void* rows, int dtype, int ld, const int* positions, const float* freq,
                   int tokens, int heads, int row_dim, int dims, int layout, cudaStream_t stream);

/* ---- rotary encoding + cache append ---------------------------------------------------- */
/* qkv row = [q heads | k heads | v heads]; pairing 0: pairs (2p, 2p+1), 1: (p, p + rotary/2).
 * accum != NULL: take the row from this float32 accumulator instead and clear it. */
int hx_rope_append(void* qkv, int dtype, int ld, const int* positions, const int* token_request,
                   const int* request_table_row, const int* block_tables, int table_stride,
                   void* k_cache, void* v_cache, int write_cache, const float* cos_table,
                   const float* sin_table, int table_positions, int tokens, int heads, int kv_heads,
                   int head_dim, int rotary_dim, int pairing, int page_size, int num_pages,
                   int* status, float* accum, int ld_accum, cudaStream_t stream);
/* token_ids[i] = max(sampled[rows[i]], 0): a step takes its tokens from the output of the
 * step before it without a round trip to the host */
int hx_feed_tokens(int* token_ids, const int* sampled, const int* rows, int count,
                   int sampled_rows, cudaStream_t stream);

/* ---- matrix products: out[t, f] (+)= sum_k x[t, k] * w[f, k] ---------------------------- */
/* CUDA cores, float32 accumulate in a fixed order; both dtypes; the true 32-bit path */
int hx_gemm_simt(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int dtype,
                 int tokens, int features, int depth, int epilogue, cudaStream_t stream);
/* tcgen05 tensor cores, bfloat16 operands, float32 accumulate in tensor memory.
 * weight_tiles != 0: w holds the matrix as [ceil(rows / 128)][ceil(depth / 64)] tiles of
 * [128][64] elements, zero padded, each tile 16 contiguous kilobytes (ldw is ignored). */
int hx_gemm_tc_supports(int tokens, int features, int depth, int ldx, int ldw);
int hx_gemm_tc_token_tile(int tokens);
int hx_gemm_tc(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
               int weight_rows, void* out, int ldo, int tokens, int features, int depth,
               int epilogue, int up_row_offset, int k_splits, int weight_tiles, int* status,
               cudaStream_t stream);
/* the fused QKV product of a prompt portion (more than 64 tokens) with rotary encoding and
   cache append as its epilogue: rotated queries to `out`, keys and values to their pages */
int hx_gemm_tc_rope_append_min_tokens(void);
int hx_gemm_tc_rope_append(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
                           int weight_rows, void* out, int ldo, int tokens, int depth,
                           int weight_tiles, const int* positions, const int* token_request,
                           const int* request_table_row, const int* block_tables,
                           int table_stride, void* k_cache, void* v_cache, const float* cos_table,
                           const float* sin_table, int table_positions, int heads, int kv_heads,
                           int head_dim, int rotary_dim, int page_size, int num_pages, int* status,
                           cudaStream_t stream);

/* hx_gemm_tc with the gated epilogue for every gate activation (see hx_biased_gated_activation)
 * and float32 biases on the gate and the up rows ([features] each, either may be null) */
int hx_gemm_tc_gated(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
                     int weight_rows, void* out, int ldo, int tokens, int features, int depth,
                     int activation, float gate_limit, const float* gate_bias, const float* up_bias,
                     int up_row_offset, int weight_tiles, int* status, cudaStream_t stream);
/* grouped product: rows of x come in tiles of token_tile (16..256), tile t multiplies with
 * group tile_group[t] of w (`groups` matrices of group_rows rows one below the other); a
 * negative entry skips the tile; tile_group is device memory, written on the stream before */
int hx_gemm_tc_grouped(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
                       int group_rows, int groups, void* out, int ldo, int tokens, int features,
                       int depth, int epilogue, int up_row_offset, int token_tile,
                       const int* tile_group, int* status, cudaStream_t stream);
/* the grouped product with the gated epilogue for every gate activation (see
 * hx_biased_gated_activation); gate_limit: the clamped form's limit */
int hx_gemm_tc_grouped_gated(const void* x, int ldx, int x_capacity_rows, const void* w, int ldw,
                             int group_rows, int groups, void* out, int ldo, int tokens,
                             int features, int depth, int activation, float gate_limit,
                             int up_row_offset, int token_tile, const int* tile_group,
                             int* status, cudaStream_t stream);

/* ---- attention over the paged cache ----------------------------------------------------- */
int hx_cache_chunk_elements(int dtype, int head_dim);
long long hx_paged_attention_scratch_floats(int tokens, int heads, int head_dim, int max_splits);
/* the same when the caller says which case it has (the streaming kernel needs less) */
long long hx_paged_attention_scratch_floats_for(int dtype, int tokens, int heads, int head_dim,
                                                int page_size, int window, int max_splits);
/* every query token over the keys [position - window + 1 (or 0), position] of its request */
int hx_paged_attention(const void* q, int ldq, const void* k_cache, const void* v_cache, int dtype,
                       const int* positions, const int* token_request,
                       const int* request_table_row, const int* block_tables, int table_stride,
                       const int* request_start, int skip_query_len, void* out, int ldo,
                       float* partial, int* arrivals, int tokens, int heads, int kv_heads,
                       int head_dim, int page_size, int num_pages, int window, float scale,
                       int split_keys, int max_splits, int* status, cudaStream_t stream);
/* the same with kept first keys: the query at position p sees key j <= p when p - j < window or
   j < keep_first */
int hx_paged_attention_kept(const void* q, int ldq, const void* k_cache, const void* v_cache,
                            int dtype, const int* positions, const int* token_request,
                            const int* request_table_row, const int* block_tables,
                            int table_stride, const int* request_start, int skip_query_len,
                            void* out, int ldo, float* partial, int* arrivals, int tokens,
                            int heads, int kv_heads, int head_dim, int page_size, int num_pages,
                            int window, int keep_first, float scale, int split_keys,
                            int max_splits, int* status, cudaStream_t stream);
/* the same with two optional float32 arrays per query head (null: absent): sinks: the softmax's
   denominator also holds exp(sinks[h]), a term without key or value; slopes: the score of key j
   for the query at position i is lowered by slopes[h] * (i - j) */
int hx_paged_attention_biased(const void* q, int ldq, const void* k_cache, const void* v_cache,
                              int dtype, const int* positions, const int* token_request,
                              const int* request_table_row, const int* block_tables,
                              int table_stride, const int* request_start, int skip_query_len,
                              void* out, int ldo, float* partial, int* arrivals, int tokens,
                              int heads, int kv_heads, int head_dim, int page_size, int num_pages,
                              int window, int keep_first, float scale, int split_keys,
                              int max_splits, const float* sinks, const float* slopes,
                              int* status, cudaStream_t stream);
/* the same with scratch built into the library: see hx_no_alloc.h beside the sources */
int hx_paged_attention_no_alloc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                int dtype, const int* positions, const int* token_request,
                                const int* request_table_row, const int* block_tables,
                                int table_stride, const int* request_start, int skip_query_len,
                                void* out, int ldo, int tokens, int heads, int kv_heads,
                                int head_dim, int page_size, int num_pages, int window, float scale,
                                int split_keys, int max_splits, int* status, cudaStream_t stream);
/* prompt portions on the tensor cores (bfloat16, head sizes in steps of 16 up to 128 and of
   32 up to 256) */
int hx_prefill_attention_supports(int head_dim, int page_size);
int hx_prefill_attention(const void* q, int ldq, const void* k_cache, const void* v_cache,
                         const int* request_start, const int* request_context,
                         const int* request_table_row, const int* block_tables, int table_stride,
                         void* out, int ldo, int requests, int tile_bound, int heads, int kv_heads,
                         int head_dim, int page_size, int num_pages, float scale, int min_query_len,
                         int* status, cudaStream_t stream);
/* the same with a window: the query at position p sees key j <= p when p - j < window or
   j < keep_first; tiles of keys that no row of a query tile sees are not read */
int hx_prefill_attention_windowed(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                  const int* request_start, const int* request_context,
                                  const int* request_table_row, const int* block_tables,
                                  int table_stride, void* out, int ldo, int requests,
                                  int tile_bound, int heads, int kv_heads, int head_dim,
                                  int page_size, int num_pages, float scale, int min_query_len,
                                  int window, int keep_first, int* status, cudaStream_t stream);

/* the same with the heads of a key/value head side by side in a tile's rows (2 to 64 heads
 * per key/value head): keys and values are read once for all of them; requests of any length
 * from min_query_len on; tile_bound counts tiles of hx_prefill_attention_packed_tokens tokens */
int hx_prefill_attention_packed_tokens(int heads, int kv_heads);
int hx_prefill_attention_packed(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                const int* request_start, const int* request_context,
                                const int* request_table_row, const int* block_tables,
                                int table_stride, void* out, int ldo, int requests,
                                int tile_bound, int heads, int kv_heads, int head_dim,
                                int page_size, int num_pages, float scale, int min_query_len,
                                int window, int keep_first, int* status, cudaStream_t stream);
/* hx_prefill_attention_windowed (pack_heads 0) or hx_prefill_attention_packed (pack_heads != 0)
 * with the optional sinks and slopes of hx_paged_attention_biased */
int hx_prefill_attention_biased(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                const int* request_start, const int* request_context,
                                const int* request_table_row, const int* block_tables,
                                int table_stride, void* out, int ldo, int requests,
                                int tile_bound, int heads, int kv_heads, int head_dim,
                                int page_size, int num_pages, float scale, int min_query_len,
                                int window, int keep_first, int pack_heads, const float* sinks,
                                const float* slopes, int* status, cudaStream_t stream);

/* the same on tcgen05, scores and partial outputs in tensor memory (pages of 16, 32, 64) */
int hx_prefill_attention_tc_supports(int head_dim, int page_size);
int hx_prefill_attention_tc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                            const int* request_start, const int* request_context,
                            const int* request_table_row, const int* block_tables,
                            int table_stride, void* out, int ldo, int requests, int tile_bound,
                            int heads, int kv_heads, int head_dim, int page_size, int num_pages,
                            float scale, int min_query_len, int* status, cudaStream_t stream);
/* hx_prefill_attention_tc_windowed with the optional sinks and slopes of
 * hx_paged_attention_biased */
int hx_prefill_attention_tc_biased(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                   const int* request_start, const int* request_context,
                                   const int* request_table_row, const int* block_tables,
                                   int table_stride, void* out, int ldo, int requests,
                                   int tile_bound, int heads, int kv_heads, int head_dim,
                                   int page_size, int num_pages, float scale, int min_query_len,
                                   int window, int keep_first, const float* sinks,
                                   const float* slopes, int* status, cudaStream_t stream);
/* the tcgen05 kernel with a window and kept first keys (see hx_prefill_attention_windowed) */
int hx_prefill_attention_tc_windowed(const void* q, int ldq, const void* k_cache,
                                     const void* v_cache, const int* request_start,
                                     const int* request_context, const int* request_table_row,
                                     const int* block_tables, int table_stride, void* out, int ldo,
                                     int requests, int tile_bound, int heads, int kv_heads,
                                     int head_dim, int page_size, int num_pages, float scale,
                                     int min_query_len, int window, int keep_first, int* status,
                                     cudaStream_t stream);

/* ---- sampling --------------------------------------------------------------------------- */
/* lowest id among the maxima; -1 and HX_STATUS_NONFINITE for a row with a non-finite logit */
int hx_argmax(const float* logits, int ld, int rows, int vocab, int* tokens, int* status,
              cudaStream_t stream);
/* inverse-CDF draw from softmax(logits / temperature) with the caller's uniform numbers;
 * temperature 0 is the greedy rule */
int hx_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
              const float* uniform, int* tokens, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HELIX_B200_KERNELS_H */
