/* hfb200.h - C entry points of the CUDA library (sm_100a).
 *
 * Every function takes device pointers, sizes and the CUDA stream to launch on, returns HFB_OK or
 * an error code, and allocates nothing unless its comment says so.  `hfb_last_error()` gives the
 * message of the last failure on the calling thread.  Element types are passed as HFB_F32 /
 * HFB_BF16 codes.  Matrices are row-major with the inner dimension contiguous: activations
 * [rows, features], weights [out, in] (the reference's layout, src/model.h:14-21).
 */
#ifndef HFB200_H
#define HFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { HFB_F32 = 0, HFB_BF16 = 1 };

/* status codes, named after the reference's (src/hfc.h:12-22) */
enum { HFB_OK = 0, HFB_EINVAL = 1, HFB_ENOTSUP = 2, HFB_ECUDA = 3, HFB_ERANGE = 4, HFB_EIO = 5 };

typedef void *hfb_stream;     /* a cudaStream_t */

const char *hfb_last_error(void);
int hfb_version(void);

/* x[t, :] = table[ids[t], :] as float32.  ids outside [0, V) raise the device error word. */
int hfb_embed(const int32_t *ids, const void *table, int table_dt, float *out, int T, int V, int E, hfb_stream s);

/* x[t, :] = table[ids[t], :] * scale + pair[row(t), :] as float32, where row(t) hashes the token with the one before it
 * in its request: (previous * mul_prev + ids[t] * mul_cur) mod buckets, and row `buckets` (the table's last) for a
 * request's first token.  The previous token of a request's first token in this step comes from prev_state[slot of the
 * request] (token + 1; 0 = the request has no token yet), which the kernel then sets to the request's last token of
 * the step.  token_seq [T], cu_tokens [S + 1], seq_slots [S] as the step function builds them.  pair == NULL: no pair
 * term and no state. */
int hfb_embed_pair(const int32_t *ids, const void *table, int table_dt, float scale, const void *pair, int pair_dt,
                   int buckets, int64_t mul_prev, int64_t mul_cur, const int32_t *token_seq, const int32_t *cu_tokens,
                   const int32_t *seq_slots, int32_t *prev_state, int n_slots, float *out, int T, int V, int E,
                   hfb_stream s);

/* out[m, :] = x[rows ? rows[m] : m, :] * rsqrt(mean(x^2) + eps) * w, sums in float32. */
int hfb_rmsnorm(const float *x, const void *w, int w_dt, float eps, void *out, int out_dt,
                const int32_t *rows, int M, int E, hfb_stream s);

/* out[M,N] (=|+=) a[M,K] . w[N,K]^T (+ bias[N]); plain float32-accumulating kernel for any sizes and
 * any mix of element types.  accumulate != 0 requires a float32 `out`. */
int hfb_linear_plain(const void *a, int a_dt, const void *w, int w_dt, const void *bias, int bias_dt,
                     void *out, int out_dt, int accumulate, int M, int N, int K, hfb_stream s);

/* The same product for bfloat16 a and w on the tensor cores (tcgen05, TMA, TMEM).  K must be a multiple of 8
 * and the operands 16-byte aligned, else HFB_ENOTSUP.  Where there are fewer output tiles than SMs (few rows; or a
 * few hundred rows, few output features and a long K) the kernel may split K over more CTAs and sum float32
 * partials kept in `workspace`; hfb_linear_tc_workspace gives the bytes that takes (0 = none); with a smaller or
 * null workspace it runs unsplit.  The kernels are launched so that they may start while the kernel in front of them
 * on the stream still runs (programmatic dependent launch), and they read `w`, the weights, before they wait for
 * that kernel: `w` must be complete before the kernel in front is launched (weights are; an operand that the
 * kernel in front computes belongs in `a`).  HFB_PDL=0 in the environment turns the early start off. */
size_t hfb_linear_tc_workspace(int M, int N, int K);
int hfb_linear_tc(const void *a, const void *w, const void *bias, int bias_dt, void *out, int out_dt,
                  int accumulate, int M, int N, int K, void *workspace, size_t workspace_bytes, hfb_stream s);

/* The product with a SwiGLU epilogue: w holds gate row i at 2i and up row i at 2i+1; out[M, N/2]. */
int hfb_linear_tc_swiglu(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, hfb_stream s);

/* The gated product with another activation of the gate (HFB_ACT_* code), and out = act(a . w^T) with the activation in
 * the epilogue (act other than silu; K is never split). */
int hfb_linear_tc_glu(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, int act, hfb_stream s);
int hfb_linear_tc_act(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, int act, hfb_stream s);

/* q|k|v of 256 tokens and more with the rest of the step in the product's epilogue: bias, rounding to bfloat16,
 * rotation of the query and key heads by cos_sin [n_positions, d / 2, 2] at the tokens' positions, queries to q_out
 * [M, H d], keys and values to cache slot slots[t] (null: nothing is cached).  bfloat16 throughout, head sizes 64 and
 * 128, the whole head rotated.  HFB_ENOTSUP, with nothing launched, for other sizes. */
int hfb_linear_tc_rope_kv(const void *a, const void *w, const void *bias, const float *cos_sin, int n_positions,
                          const int32_t *positions, const int32_t *slots, void *q_out, void *k_cache, void *v_cache,
                          int64_t cache_slots, int M, int K, int H, int G, int d, hfb_stream s);

/* Only the split-K partial sums partial[*splits, M, N] (float32) of a product, for a fused reduction to finish;
 * `workspace` must hold hfb_linear_tc_partials_workspace bytes.  Above 128 rows that size is 0 for a product that
 * would not be split, and this entry refuses it (HFB_ENOTSUP). */
size_t hfb_linear_tc_partials_workspace(int M, int N, int K);
int hfb_linear_tc_partials(const void *a, const void *w, int M, int N, int K, void *workspace, size_t workspace_bytes,
                           int *splits, hfb_stream s);

/* residual[M,N] += sum_s partial[s] (+ bias); if xn: xn = rmsnorm(residual) * w (the next product's input). */
int hfb_reduce_residual_norm(const float *partial, int splits, int M, int N, const void *bias, int bias_dt,
                             float *residual, const void *w, int w_dt, float eps, void *xn, int xn_dt, hfb_stream s);

/* hfb_rope_kv_write reading sum_s partial[s] + bias instead of a finished q|k|v row. */
int hfb_reduce_rope_kv(const float *partial, int splits, int dt, const void *bias, int bias_dt, const float *cos_sin,
                       int n_rot, int n_positions, const int32_t *positions, const int32_t *slots, void *q_out,
                       void *k_cache, void *v_cache, int64_t cache_slots, int T, int H, int G, int d, hfb_stream s);

/* arg-max with many blocks per row (two passes; scratch of hfb_argmax2_scratch bytes). */
size_t hfb_argmax2_scratch(int M, int V);
int hfb_argmax2(const float *logits, int32_t *out, int M, int V, void *scratch, size_t scratch_bytes, hfb_stream s);

/* Splits qkv[T, (H+2G)*d] into rotated queries q_out[T, H*d], rotated keys and plain values written
 * to the paged cache at slots[t] (page * block_size + offset; < 0 or slots == NULL: not written).
 * cos_sin is float32 [positions, n_rot/2, 2]; n_rot == 0 means no rotation. */
int hfb_rope_kv_write(const void *qkv, int dt, const float *cos_sin, int n_rot, int n_positions,
                      const int32_t *positions, const int32_t *slots, void *q_out, void *k_cache, void *v_cache,
                      int64_t cache_slots, int T, int H, int G, int d, hfb_stream s);

/* Attention of every token over its request's cached keys lo..pos, plain kernel: one block per (token, head), float32
 * softmax.  `window` names the mask, here and in every attention entry point below: > 0, lo = max(0, pos - window + 1)
 * (a sliding window); < 0, lo = pos - pos % (-window) (chunks of -window positions counted from position 0: a query
 * sees the keys of its own chunk); 0, lo = 0.  Keys [.., G, d], values [.., G, dv] with rows v_row elements apart
 * (dv; or d with v_cache == k_cache, when a value is the first dv elements of its key), out [T, H dv].  Head sizes up
 * to 640. */
/* Options of the score that the plain kernel, the two-tile tensor-core kernel and the decode kernel take: `head_scales`
 * (float32 [H], or NULL): the scaled score of head h is multiplied by head_scales[h]; `softcap` > 0: the score becomes
 * softcap * tanh(score / softcap), after the factors and before any bias and the softmax. */
int hfb_attention_plain(const void *q, const void *k_cache, const void *v_cache, int dt,
                        const int32_t *block_table, int max_blocks, const int32_t *token_seq,
                        const int32_t *positions, int block_size, int64_t num_pages, int window, float scale,
                        void *out, int T, int H, int G, int d, int dv, int v_row, const float *sinks, int zero_sink,
                        const float *slopes, const float *head_scales, float softcap, hfb_stream s);

/* The same for bfloat16 with head_dim 64 or 128 and a block size that divides 64, tiled, on tensor cores.
 * Tiles (tile_seq, tile_t0 = first token index, tile_nt = tokens) cover the step's tokens; a tile holds at
 * most hfb_attention_fast_tile_tokens(H, G, warps) tokens of one request.  warps = 4 for prompt portions and
 * mixed batches (splits must be 1), warps = 1 for decode, where `splits` > 1 cuts each request's keys into
 * that many ranges whose partial results are merged in order; they live in `scratch`
 * (stages = 4 with warps = 4 selects a deeper load pipeline for CTAs that have an SM to themselves)
 * (hfb_attention_fast_scratch bytes). */
int hfb_attention_fast_tile_tokens(int H, int G, int warps);
size_t hfb_attention_fast_scratch(int T, int H, int d, int splits);
int hfb_attention_fast(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                       int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                       const int32_t *tile_nt, int n_tiles, int warps, int stages, int splits, int block_size,
                       int64_t num_pages, int window, float scale, void *out, void *scratch, size_t scratch_bytes,
                       int T, int H, int G, int d, hfb_stream s);

/* Decode attention with the keys and values fetched by TMA: tiles as hfb_attention_fast's 16-row form takes them
 * (one or two tokens of one request), bfloat16, head_dim 64 or 128, block sizes 8..64 dividing 64.  `stages` (2..4)
 * tiles of 64 keys are in flight per CTA; `splits` > 1 needs hfb_attention_fast_scratch bytes of scratch, and is
 * merged by the CTA that stores a tile's last split when `counters` (n_tiles * G ints, zero before the first launch
 * and after every launch) is given, else by a second kernel. */
int hfb_attention_decode(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                         int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                         const int32_t *tile_nt, int n_tiles, int stages, int splits, int block_size, int64_t num_pages,
                         int window, float scale, void *out, void *scratch, size_t scratch_bytes, int T, int H, int G,
                         int d, int *counters, int counters_len, hfb_stream s);

/* The same with options of the softmax: `sinks` (float32 [H], or `zero_sink` for a score of zero), a score per head
 * without key or value that joins the denominator once, and `slopes` (float32 [H]): slope * (query position - key
 * position) is taken off every score. */
int hfb_attention_decode_opt(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                             int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                             const int32_t *tile_nt, int n_tiles, int stages, int splits, int block_size, int64_t num_pages,
                             int window, float scale, void *out, void *scratch, size_t scratch_bytes, int T, int H, int G,
                             int d, int *counters, int counters_len, const float *sinks, int zero_sink, const float *slopes,
                             const float *head_scales, float softcap, hfb_stream s);

/* Attention of prompt portions on tcgen05 (S and PV accumulators in TMEM, K and V gathered page by page with
 * TMA): bfloat16, head_dim 128, block sizes 8..128 that divide 128.  Tiles hold at most 128 / (H/G) tokens. */
int hfb_attention_tc(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                     int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                     const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window,
                     float scale, void *out, int T, int H, int G, int d, hfb_stream s);

/* The same with two 128-row tiles per CTA (tiles hold at most 2 * (128 / (H/G)) tokens): the softmax of one tile
 * runs while the tensor core works on the other; the running output stays in TMEM.  head_dim 64 or 128. */
int hfb_attention_tc2(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                      int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                      const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window, float scale,
                      void *out, int T, int H, int G, int d, hfb_stream s);

/* ... with the options of hfb_attention_decode_opt. */
int hfb_attention_tc2_opt(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                          int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                          const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window, float scale,
                          void *out, int T, int H, int G, int d, const float *sinks, int zero_sink, const float *slopes,
                          const float *head_scales, float softcap, hfb_stream s);

/* Launches may overlap with the kernel in front (programmatic dependent launch): on by default, off with HFB_PDL=0. */
void hfb_set_launch_overlap(int on);

/* out[t, f] = silu(g) * u with g = gu[t, f], u = gu[t, F + f], or, interleaved, g = gu[t, 2f], u = gu[t, 2f + 1] */
int hfb_swiglu(const void *gu, void *out, int dt, int T, int F, int interleaved, hfb_stream s);

/* Activations: codes for hfb_glu / hfb_act / the expert products. */
enum { HFB_ACT_SILU = 0, HFB_ACT_RELU = 1, HFB_ACT_GELU_TANH = 2, HFB_ACT_RELU2 = 3, HFB_ACT_NONE = 4 };
/* added to the activation of hfb_moe_gemm: rows of w alternate gate, up, and out [.., N / 2] = act(gate) * up */
enum { HFB_ACT_GLU = 256 };

/* out[t, f] = act(g) * u, gate and up laid out as for hfb_swiglu */
int hfb_glu(const void *gu, void *out, int dt, int T, int F, int interleaved, int act, hfb_stream s);

/* out[i] = act(x[i]) (in place when out == x) */
int hfb_act(const void *x, void *out, int dt, int64_t total, int act, hfb_stream s);

/* x[i] *= scale */
int hfb_scale(float *x, int64_t total, float scale, hfb_stream s);

/* Dynamic Tanh norm: out[m, :] = tanh(alpha * x[rows ? rows[m] : m, :]) * w + b (alpha a scalar on the device). */
int hfb_dyt(const void *x, int x_dt, const int32_t *rows, const void *alpha, const void *w, const void *b,
            int p_dt, void *out, int out_dt, int M, int E, hfb_stream s);

/* residual += dyt(y); with out != NULL also out = dyt2(residual) (the next sublayer's input).  y is the sum, in this
 * order, of: y [splits, M, E], the partial sums of a product (a finished y has splits = 1; none: splits = 0), the
 * product's bias (null: none), and sum_j mix_w[m, j] * mix_y[m * top + j, :] (float32; null: none). */
int hfb_dyt_residual(const void *y, int y_dt, int splits, const void *bias, int bias_dt, const float *mix_y,
                     const float *mix_w, int top, const void *alpha, const void *w, const void *b, int p_dt,
                     float *residual, const void *alpha2, const void *w2, const void *b2, int p2_dt,
                     void *out, int out_dt, int M, int E, hfb_stream s);

/* The tail of a q|k|v product: src [splits, T, H d + G d + G dv] float32 partial sums (+ bias) -> rotation of the first
 * n_rot dimensions of query and key heads -> with norm != 0, x / sqrt(mean(x^2) + eps) per head, times q_w / k_w
 * (float32 [d], shared by the heads; null: no weight) -> q_out [T, H d], keys [.., G, d] and values [.., G, dv] at cache
 * slot slots[t].  G == 0: the row holds queries only.  Values mixed across layers: v_mode 1 copies the row's values to
 * v_first [T, G dv] (float32) as they are; v_mode 2 replaces them by (1 - v_lambda) v + v_lambda v_first before they
 * are stored; 0: neither.  pairing 0 rotates the pairs (i, i + n_rot/2), 1 the pairs (2i, 2i + 1).  dv == 0: the row has
 * no value heads (src [splits, T, H d + G d]) and v_cache is not written. */
int hfb_rope_norm_kv_write(const float *src, int splits, const void *bias, int bias_dt, const float *cos_sin,
                           int n_rot, int n_positions, const int32_t *positions, const int32_t *slots,
                           void *q_out, void *k_cache, void *v_cache, int out_dt, int64_t cache_slots, int T,
                           int H, int G, int d, int dv, int norm, float eps, const float *q_w, const float *k_w,
                           float *v_first, int v_mode, float v_lambda, int pairing, hfb_stream s);

/* Latent attention, the tail of the down product: src [splits, T, q_rank + kv_rank + rot] float32 partial sums ->
 * query latent = rmsnorm(src[:q_rank]) * q_w -> cq_out [T, q_rank]; key/value latent = rmsnorm(next kv_rank) * kv_w ->
 * cache row [0, kv_rank); the last `rot` values rotated (pairs (2i, 2i+1), cos_sin [n_positions, rot / 2, 2]) -> cache
 * row [kv_rank, kv_rank + rot).  The cache holds one row of kv_rank + rot per slot.  Norm weights float32. */
int hfb_latent_split(const float *src, int splits, const float *q_w, const float *kv_w, float eps, const float *cos_sin,
                     int n_positions, const int32_t *positions, const int32_t *slots, void *cq_out, void *cache,
                     int out_dt, int64_t cache_slots, int T, int q_rank, int kv_rank, int rot, hfb_stream s);

/* Latent attention, the tail of the query product: src [splits, T, H (d + rot)] float32 partial sums; per head the
 * first d values go to q_plain [T, H, d] as they are, the last `rot` rotated (pairs (2i, 2i+1)) to
 * q_att [T, H, att_row] at column att_col. */
int hfb_latent_query_rope(const float *src, int splits, const float *cos_sin, int n_positions, const int32_t *positions,
                          void *q_plain, void *q_att, int out_dt, int T, int H, int d, int rot, int att_row, int att_col,
                          hfb_stream s);

/* The two steps above and the per-head product below in one kernel, bfloat16: q_att [T, H, kv_rank + rot] receives, per
 * head, w_ukt[h] (bfloat16 [kv_rank, d]) times the head's plain part (rounded to bfloat16) in its first kv_rank columns and
 * the rotated part behind them. */
int hfb_latent_query_absorb(const float *src, int splits, const float *cos_sin, int n_positions, const int32_t *positions,
                            const void *w_ukt, void *q_att, int T, int H, int d, int rot, int kv_rank, hfb_stream s);

/* A product per head: out[t, h, n] = sum_k w[h, n, k] * in[t, h, k], n < N, k < K; rows of `in` hold H heads in_row
 * apart from column 0, rows of `out` H heads out_row apart (in_row >= K, out_row >= N: a head's result may land in the
 * first N columns of a wider row).  float32 sums; operands all bfloat16 (tensor cores) or all float32. */
int hfb_headwise_linear(const void *in, int in_dt, const void *w, int w_dt, void *out, int out_dt, int T, int H, int N,
                        int K, int in_row, int out_row, hfb_stream s);

/* The choice of a mixture of experts' router from its float32 logits z [splits, T, E] (partial sums of the router's
 * product, summed in order, plus its bias; finished logits: splits = 1, bias null): the `top` largest (lowest index first
 * among equals) go to ids [T, top], their softmax over the chosen logits only to weights [T, top]. */
int hfb_moe_topk(const float *z, int splits, const void *bias, int bias_dt, int T, int E, int top, int32_t *ids,
                 float *weights, hfb_stream s);

/* Groups the T * top (token, choice) pairs by expert: order[p] = pair at sorted place p; tiles of at most `tile`
 * places of one expert in tile_expert / tile_p0 / tile_n (room for hfb_moe_max_tiles entries); *n_tiles on the device.
 * Steps of few tokens ask for tiles of 16 places (more, smaller blocks for the product behind). */
int hfb_moe_max_tiles(int pairs, int E, int tile);
int hfb_moe_sort(const int32_t *ids, int pairs, int E, int tile, int32_t *order, int32_t *tile_expert, int32_t *tile_p0,
                 int32_t *tile_n, int32_t *n_tiles, hfb_stream s);

/* Grouped product over the sorted places: out[dst(p), :] = act(a[src(p), :] . w[expert(p)]^T), w [E, N, K].
 * src(p) = order[p] / src_div when src_div > 0, else p; dst(p) = order[p] when scatter != 0, else p.  `tile`: the most
 * places a tile of the lists holds, up to 128; with 16 and less the form for steps of a few tokens runs. */
int hfb_moe_gemm(const void *a, int a_dt, const void *w, int w_dt, void *out, int out_dt, int act, int N, int K,
                 const int32_t *order, int src_div, int scatter, const int32_t *tile_expert, const int32_t *tile_p0,
                 const int32_t *tile_n, const int32_t *n_tiles, int max_tiles, int tile, hfb_stream s);

/* out[t, :] = sum_j weights[t, j] * y[t * top + j, :] in float32, j in order */
int hfb_moe_combine(const void *y, int y_dt, const float *weights, float *out, int T, int top, int N, hfb_stream s);

/* The router of a mixture whose scores are a softmax over all router outputs: z [splits, T, E] float32 partial sums;
 * s = softmax(z); choice score = s + correction (null: none); the outputs form n_groups equal groups of neighbours and
 * only those of the `keep` groups with the largest choice score can be chosen; ids [T, top] = the `top` largest choice
 * scores (largest first, the lower index among equals), weights = s[ids] * scale. */
int hfb_moe_route_softmax(const float *z, int splits, const void *correction, int corr_dt, int T, int E, int top,
                          int n_groups, int keep, float scale, int32_t *ids, float *weights, hfb_stream s);

/* Hyper-connections: the residual stream in S copies, x [T, S, E] float32.
 * hc_spread: every copy = emb [T, E].
 * hc_in_norm: out[m, :] = norm(sum_s in_w[s] x[rows ? rows[m] : m, s, :]) with the Dynamic Tanh norm (alpha, w, b) of type
 *   p_dt; in_w == NULL: the plain sum; alpha == NULL: no norm.
 * hc_update: y = scale .* (factor_a * sum of ya's splits_a planes + factor_b * sum of yb's planes + sum_j mix_w[t, j] *
 *   (mix_ids[t, j] >= n_real ? mix_h[t, :] : mix_y[t * top + j, :])), any of the three terms absent when its pointer is
 *   null; then x'[t, d, :] = sum_s hc_mix[s, d] x[t, s, :] + hc_out[d] y for every copy d from the old copies, and, with
 *   out != NULL, out[t, :] = norm(sum_d next_in[d] x'[t, d, :]) (next_in NULL: plain sum; alpha NULL: no norm). */
int hfb_hc_spread(const float *emb, float *x, int S, int T, int E, hfb_stream s);
int hfb_hc_in_norm(const float *x, int S, const float *in_w, const int32_t *rows, const void *alpha, const void *w,
                   const void *b, int p_dt, void *out, int out_dt, int M, int E, hfb_stream s);
int hfb_hc_update(float *x, int S, const float *ya, int splits_a, float factor_a, const float *yb, int splits_b,
                  float factor_b, const float *mix_y, const float *mix_w, const int32_t *mix_ids, int top, int n_real,
                  const void *mix_h, int mix_h_dt, const void *scale, int scale_dt, const float *hc_mix,
                  const float *hc_out, const float *next_in, const void *alpha, const void *w, const void *b,
                  int p_dt, void *out, int out_dt, int T, int E, hfb_stream s);

/* Recurrent mixers (float32 throughout; a request's state lives in row seq_slots[seq] of a [n_slots, slot_stride] array).
 * decay: out[t, h, i] = exp(-rate[h] * softplus(sign * (z[t, h, i] + bias[h, i]))), z the sum of `splits` planes
 *   [T, z_stride] read from column z_col0 on.
 * short_conv: causal convolution over time per channel (w [C, taps], last column = current token), silu, then unit
 *   length for the first n_unit heads of a row made of n_a heads of d_a and n_b heads of d_b channels (the first n_scaled
 *   of them also times `scale`); `carried` holds each request's last taps - 1 inputs and is brought up to date.
 * linear_scan: per head S <- diag(a) S + k u^T, o = S^T q * q_scale with u = v, or, with beta_logit, u = sigmoid(beta)
 *   (v - (diag(a) S)^T k); state [H, dv, d] per slot; rows of q, k (Hq heads), a, v, o (H heads) with their strides.
 * gate_norm: out = o / sqrt(mean(o^2) + eps) * w * gate(g) per head; gate 0 silu, 1 sigmoid. */
int hfb_decay(const float *z, int splits, int z_stride, int z_col0, const void *bias, int bias_dt, const float *rate,
              float sign, float *out, int T, int H, int d, hfb_stream s);
int hfb_short_conv(const float *x, int splits, const void *w, int w_dt, int taps, float *carried, int64_t slot_stride,
                   const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, int S,
                   float *out, int T, int n_a, int d_a, int n_b, int d_b, int n_unit, int n_scaled, float scale,
                   float unit_eps, hfb_stream s);
int hfb_linear_scan(const float *q, int q_stride, const float *k, int k_stride, const float *v, int v_stride,
                    const float *a, int a_stride, const float *beta_logit, int beta_stride, float q_scale,
                    float *state, int64_t slot_stride, const int32_t *cu_tokens, const int32_t *seq_slots,
                    int n_slots, int S, float *o, int o_stride, int H, int Hq, int d, int dv, hfb_stream s);
int hfb_gate_norm(const float *o, const void *w, int w_dt, float eps, const float *g, int g_splits, int g_stride,
                  int g_col0, int gate, void *out, int out_dt, int T, int H, int dv, hfb_stream s);

/* minGRU over a step's tokens: row = `splits` float32 planes [T, 3 W] of [update gate | candidate | output gate] sums;
 * z = sigmoid(a + bz), u = b + bx, cand = u >= 0 ? u + 1/2 : sigmoid(u), S <- (1 - z) S + z cand, out = S silu(g); S [W]
 * float32 per request in its slot of `state` (rows slot_stride apart). */
int hfb_mingru_scan(const float *row, int splits, const void *bz, const void *bx, int b_dt, float *state, int64_t slot_stride,
                    const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, int S, void *out, int out_dt, int T, int W,
                    hfb_stream s);

/* Layer norm of rows of the float32 stream: (x - mean) / sqrt(var + eps) * w (center = 1) or x / sqrt(mean(x^2) + eps) * w
 * (center = 0), w float32 [E]; out[r] = norm(x[rows ? rows[r] : r]) for N rows, x having n_src rows. */
int hfb_layernorm(const float *x, const float *w, float eps, int center, const int32_t *rows, int n_src, void *out, int out_dt,
                  int N, int E, hfb_stream s);
/* The same norm with the token shift behind it: out[t] = h_t + (h_(t-1) - h_t) * mu, h = norm(x), h_(t-1) from the step's
 * previous row or, for a request's first token of the step, from its slot of `state` (float32, rows slot_stride apart),
 * which then receives the h of the request's last token of the step. */
int hfb_layernorm_shift(const float *x, const float *w, const float *mu, float eps, int center, float *state, int64_t slot_stride,
                        const int32_t *token_seq, const int32_t *cu_tokens, const int32_t *seq_slots, int n_slots, void *out,
                        int out_dt, int T, int E, hfb_stream s);
/* The tail of a sublayer's last product for such norms: residual[m] += sum of `splits` partial sums [splits, M, N] (+ bias),
 * then, if xn is given, xn[m] = norm(residual[m]) (w float32 [N]); splits = 0: only the norm.  With `mu` (float32 [N]) the
 * token shift of a step of single tokens: row m is request m, slot seq_slots[m] of `state` gives the previous h and
 * receives this one.  Rows of up to 16,384 values. */
int hfb_reduce_residual_layernorm(const float *partial, int splits, int M, int N, const void *bias, int bias_dt, float *residual,
                                  const float *w, float eps, int center, const float *mu, float *state, int64_t slot_stride,
                                  const int32_t *seq_slots, int n_slots, void *xn, int xn_dt, hfb_stream s);
/* out = a * sigmoid(g) (gate 1) or a * silu(g) (gate 0); g: `splits` float32 planes [T, g_stride] from column g_col0 on,
 * plus `bias` (float32 [C]) where given; a and out [T, C] of type dt. */
int hfb_gate_mul(const void *a, int dt, const float *g, int splits, int g_stride, int g_col0, const float *bias, int gate, void *out,
                 int T, int C, hfb_stream s);

/* out[m] = index of the first maximum of logits[m, :] */
int hfb_argmax(const float *logits, int32_t *out, int M, int V, hfb_stream s);

/* One token per row: greedy where temps[m] <= 0, else temperature sampling with top-k (0 = off), min-p
 * (0 = off) and top-p (1 = off) in the reference's order of operations (src/sample.c:66-116);
 * uniforms[m] in [0, 1) is the row's draw. */
int hfb_sample(const float *logits, int M, int V, const float *temps, const int32_t *top_ks,
               const float *top_ps, const float *min_ps, const float *uniforms, int32_t *out, hfb_stream s);

/* Device error word: kernels set bits instead of touching memory out of range.  Reading syncs the stream. */
enum { HFB_ERR_TOKEN_ID = 1, HFB_ERR_PAGE = 2, HFB_ERR_SLOT = 4, HFB_ERR_WAIT = 8, HFB_ERR_POSITION = 16 };
int hfb_error_word_take(int32_t *word, hfb_stream s);
/* Queues a copy of the word into pinned host memory and returns; read it after your own wait on the stream. */
int hfb_error_word_peek_async(int32_t *host_word, hfb_stream s);

#ifdef __cplusplus
}
#endif
#endif
