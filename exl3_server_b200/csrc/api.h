// C entry points of the kernel library.  Every function launches on the given
// stream and returns 0, a cudaError_t (> 0) or a negative code from
// common.cuh; exl3_last_error() gives the message of the calling thread's
// last failure.  Element type codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

extern "C" {

const char* exl3_last_error();
int exl3_abi_version();
long long exl3_launch_count();

int exl3_embed(const int* ids, const void* table, int table_dtype, float* h, int T, int H, int V,
               float scale, cudaStream_t stream);
int exl3_add_rmsnorm(float* h, const void* y, int y_dtype, float y_scale, const void* w, int w_dtype,
                     float eps, void* out, int out_dtype, float out_scale, const int* rows, int n_rows,
                     int H, cudaStream_t stream);
// interleave 0: gu = [gate (I) | up (I)]; 8: eight gate columns, then the eight up columns of the same features.
int exl3_silu_mul(const void* gu, void* out, int dtype, int T, int I, int interleave, cudaStream_t stream);
// The same with another activation on the gate: kind 0 silu, 1 gelu (exact), 2 gelu by the tanh formula.
int exl3_act_mul(const void* gu, void* out, int dtype, int T, int I, int interleave, int kind, cudaStream_t stream);
// inv_freq: rot / 2 frequencies; inv_freq_lo: what float32 lost of them, or null (see rope_sincos in common.cuh).
int exl3_rope_kv_write(void* qkv, int dtype, const float* inv_freq, const float* inv_freq_lo, int rot,
                       float pos_scale, const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride,
                       void* k_pool, void* v_pool, int T, int nh, int nkv, int hd, int page, int write_kv,
                       cudaStream_t stream);

// y[M,N] = x[M,K] . w[N,K]^T (+ bias[N]); any sizes; float32 accumulation in a
// fixed order over K.  in_dtype covers x, w and bias; out_dtype covers y.
int exl3_gemm_simt(const void* x, const void* w, const void* bias, void* y, int in_dtype, int out_dtype,
                   int M, int N, int K, cudaStream_t stream);
// bfloat16 weights streamed once for M <= 16 rows of x (tensor-core mma, K % 8 == 0).
// epilogue 1: rows of w are 8 gate rows then 8 up rows, repeated; y[M, N/2] = silu(gate) * up.
int exl3_gemv_bf16(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N,
                   int K, int epilogue, cudaStream_t stream);

// exl3_gemv_bf16 (epilogue 0) with the xIELU activation on its results: act_p z^2 + z / 2 for z > 0, act_n (exp(z) - 1 - z)
// + z / 2 otherwise, with act_p = softplus(p) and act_n = 1/2 + softplus(q) given by the caller.
int exl3_gemv_bf16_gelu(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                        int kind, cudaStream_t stream);
int exl3_gemv_bf16_act(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                       float act_p, float act_n, cudaStream_t stream);

// bfloat16 GEMM on tcgen05 tensor cores with TMA loads (K and N multiples of 8); epilogue 1 as in
// exl3_gemv_bf16 (N a multiple of 16, output N/2 wide).  exl3_gemm_tc_status() returns and clears the
// code a kernel left when one of its bounded waits ran out (0: none).
int exl3_gemm_tc(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int epilogue,
                 cudaStream_t stream);
int exl3_gemm_tc_status();
// Launches a kernel whose only wait can never be satisfied (short limit): status becomes 9.
int exl3_gemm_tc_wait_selftest(cudaStream_t stream);

// Attention of single query tokens over the paged cache.  Token t belongs to
// batch row tok_seq[t] and sits at position tok_pos[t]; it sees keys
// max(0, pos - window + 1) .. pos (window 0: from 0).  n_splits > 1 cuts the
// keys into chunks of split_keys and needs scratch; see attention_simt.cu.
int exl3_attn_tokens(const void* q, int64_t q_row_stride, void* out, int dtype, const void* k_pool,
                     const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                     const int* tok_seq, int T, int nh, int nkv, int hd, int page, int window, float scale,
                     int split_keys, int max_splits, float* scratch, size_t scratch_bytes,
                     cudaStream_t stream);
size_t exl3_attn_tokens_scratch_bytes(int T, int nh, int hd, int max_splits);
// The same with values narrower than keys and rows of both pools kv_row elements apart (hdv <= hd <= kv_row, all
// multiples of 16): out is [T, nh, hdv] and the scratch is sized with hdv.  With v_pool == k_pool the values are the
// first hdv features of the keys (one latent row per token that every head reads).
int exl3_attn_tokens_kv(const void* q, int64_t q_row_stride, void* out, int dtype, const void* k_pool,
                        const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                        const int* tok_seq, int T, int nh, int nkv, int hd, int hdv, int kv_row, int page, int window,
                        float scale, int split_keys, int max_splits, float* scratch, size_t scratch_bytes,
                        cudaStream_t stream);

// The general form: the value pool has a row pitch of its own (v_row >= hdv; hd, hdv and both pitches multiples of 8,
// values may be wider than keys); chunk > 0 also hides every key before floor(pos / chunk) * chunk; sink != 0 adds
// one to the softmax's denominator (a key of score 0 without a value).
int exl3_attn_tokens_ex(const void* q, int64_t q_row_stride, void* out, int dtype, const void* k_pool,
                        const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                        const int* tok_seq, int T, int nh, int nkv, int hd, int hdv, int kv_row, int v_row, int page,
                        int window, int chunk, int sink, float scale, int split_keys, int max_splits, float* scratch,
                        size_t scratch_bytes, cudaStream_t stream);
// The same with the output as float32 [T, heads, value_dim] when out_f32 is set (whatever the cache's type).
int exl3_attn_tokens_wide(const void* q, int64_t q_row_stride, void* out, int out_f32, int dtype, const void* k_pool,
                        const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                        const int* tok_seq, int T, int nh, int nkv, int hd, int hdv, int kv_row, int v_row, int page,
                        int window, int chunk, int sink, float scale, int split_keys, int max_splits, float* scratch,
                        size_t scratch_bytes, cudaStream_t stream);

// Token embedding plus a row of a second table picked by a hash of (previous token, token):
//   h[t] = table[id_t] + extra[(prev_t * mul_prev + id_t * mul_cur) mod buckets],  extra[buckets] for position 0.
// The previous token of a row's first token in this step comes from last_token[slot] (int32 per slot), which the
// kernel then sets to the row's last token of the step.  Sums are float32.
int exl3_embed_hashed(const int* ids, const int* tok_pos, const int* tok_seq, const int* row_start,
                      const int* slot_ids, const void* table, const void* extra, int dtype, int buckets,
                      long long mul_prev, long long mul_cur, int* last_token, float* h, int T, int H, int V,
                      cudaStream_t stream);

// The step between an attention's joint input projection and the attention itself (see qk_prep.cu).
//   x [T, ld] holds per token nh query heads (at q_off), nkv key heads (k_off) of hd features and nkv value heads
//   (v_off, or < 0 for none) of hdv features.  norm: 0 none, 1 divide a query/key head by its root mean square,
//   2 the same times q_w / k_w [hd].  rot > 0: rotary encoding of the first rot features (layout 0: feature i with
//   i + rot / 2; 1: feature 2i with 2i + 1), sines and cosines times mscale.  Keys are then multiplied by k_mul.
//   mix_lambda != null: v <- (1 - lambda) v + lambda v_src[t] (v_src [T, v_src_ld], its own type).
//   Queries go to q_out [T, nh * hd_pad]; keys and values to the paged cache (k_pool / v_pool, rows of hd_pad /
//   hdv_pad features, pad features zero), or, when k_pool is null, keys to k_out [T, nkv * hd_pad].
int exl3_qk_prep(const void* x, int x_dtype, int64_t ld, int q_off, int k_off, int v_off, int T, int nh, int nkv,
                 int hd, int hdv, int hd_pad, int hdv_pad, int norm, const void* q_w, const void* k_w, int w_dtype,
                 float eps, int rot, int layout, const float* inv_freq, const float* inv_freq_lo, float mscale,
                 float k_mul, const void* mix_lambda, int lambda_dtype, const void* v_src, int v_src_dtype,
                 int64_t v_src_ld, const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride,
                 int page, void* q_out, int q_out_dtype, void* k_out, int k_out_dtype, void* k_pool, void* v_pool,
                 int pool_dtype, cudaStream_t stream);

// Token shift: for s < n_mix, out[s][t] = h[t] + (h[t - 1] - h[t]) * mu[s]; the row before a row's first token of
// this step comes from prev[slot] (float32 [slots, H], zero for a new sequence), which is then set to the row's last
// h of the step.
int exl3_token_shift(const void* h, int h_dtype, const void* mu, int mu_dtype, int n_mix, float* prev,
                     const int* tok_seq, const int* row_start, const int* slot_ids, void* out, int out_dtype, int T,
                     int H, cudaStream_t stream);

// A linear recurrence with a matrix state per head (float32 [slots, heads, dk, dv]); see linear_scan.cu.
//   mode 0 (decay per token and key channel, bonus for the current token):
//     o_t = S^T r_t + (sum_i r_ti u_i k_ti) v_t,   S <- diag(w_t) S + k_t v_t^T,  w_t = exp(-exp(wraw_t + w0))
//   mode 1 (one decay per head): S <- decay_h S + k_t v_t^T,  o_t = S^T r_t
// r, k [T, *] of rk_dtype with row pitches r_ld, k_ld; v of v_dtype; wraw of w_dtype; out float32 [T, heads * dv].
size_t exl3_linear_scan_scratch_bytes(int B, int T, int heads, int dk, int dv, int max_new);
int exl3_linear_scan(int mode, const void* r, int64_t r_ld, const void* k, int64_t k_ld, int rk_dtype, const void* v,
                     int64_t v_ld, int v_dtype, const void* wraw, int64_t w_ld, int w_dtype, const void* w0,
                     const void* u, int wu_dtype, const float* decay, float* state, const int* slot_ids,
                     const int* row_start, float* out, int B, int T, int heads, int dk, int dv, int max_new,
                     int in_act, float* scratch, size_t scratch_bytes, cudaStream_t stream);
// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w[h, :] (w null: 1) * silu(gate[t, h, :]) (gate null: 1; gate_kind 1:
// sigmoid instead of silu).  in_act of exl3_linear_scan: 1 applies silu to r, k and v as they are read.
int exl3_head_norm_gate(const float* o, const void* w, int w_dtype, const void* gate, int gate_dtype, int64_t gate_ld,
                        int gate_kind, float eps, void* out, int out_dtype, int T, int heads, int dv, cudaStream_t stream);
// out[t] = coef * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb), float32 out
int exl3_normed_sum2(const void* a, const void* b, int ab_dtype, const void* wa, const void* wb, int w_dtype, float eps,
                     float coef, float* out, int T, int H, cudaStream_t stream);
// h += y / rms(y) * w (as exl3_norm_add) and, over the new residual, x = h / rms(h) * w2 in x's type: the norm on
// a sublayer's output, the residual sum and the next sublayer's input norm in one kernel.
int exl3_norm_add_norm(float* h, const void* y, int y_dtype, const void* w, int w_dtype, float eps, const void* w2,
                       int w2_dtype, float eps2, void* x, int x_dtype, int T, int H, cudaStream_t stream);
// kind 0: z/2 (1 + erf(z / sqrt 2)); 1: z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); 2: tanh(z)
int exl3_activation(const void* z, int z_dtype, void* out, int out_dtype, int64_t n, int kind, cudaStream_t stream);
// x <- cap * tanh(x / cap) in place
int exl3_softcap(float* x, int64_t n, float cap, cudaStream_t stream);

// Attention over latent rows on the tensor cores (bfloat16; see attention_latent.cu).  q [T * H, dk] and out
// [T * H, dv] hold the rows of each sequence's tokens of this step head by head; the pool holds one row of dk
// features per key, page = 64 keys, whose first dv features are the values.  Batch row b has the tokens
// row_start[b] .. row_start[b + 1], the first of them at position row_pos0[b]; max_new is the most tokens of any row.
// n_splits > 1: chunks of pages_per_chunk pages, merged through scratch (exl3_attn_latent_scratch_bytes).
// exl3_attn_latent_row_tile: sixteens of rows a block takes for these sizes (0: dk does not fit shared memory).
int exl3_attn_latent_row_tile(int dk, int max_rows);
size_t exl3_attn_latent_scratch_bytes(int T, int H, int dv, int n_splits);
// gate (float32 [T * H], or null): a factor per row on the output.
// pool_pages: pages in the pool (its rows are pool_pages * 64).  exl3_attn_latent_status() returns and clears the flag a
// block left when a bounded wait for a page's copies ran out.
int exl3_attn_latent(const void* q, void* out, const void* pool, int64_t pool_pages, const int* block_table, int bt_stride,
                     const int* row_start, const int* row_pos0, int B, int T, int max_new, int H, int dk, int dv, int page,
                     float scale, int pages_per_chunk, int n_splits, float* scratch, size_t scratch_bytes,
                     const float* gate, cudaStream_t stream);
int exl3_attn_latent_status();

// Residual update with the norm on the sublayer's output: h[t,:] += y[t,:] * rsqrt(mean(y[t,:]^2) + eps) * w (skipped
// when y is null), then x[t,:] = h[t,:] in x_dtype (skipped when x is null).  Statistics and the sum are float32.
int exl3_norm_add(float* h, const void* y, int y_dtype, const void* w, int w_dtype, float eps, void* x, int x_dtype,
                  int T, int H, cudaStream_t stream);
// xIELU, element by element, with the two raw parameters pq (any float type): for z > 0, softplus(p) z^2 + z / 2;
// else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
int exl3_xielu(const void* z, int z_dtype, const void* pq, int pq_dtype, void* out, int out_dtype, int64_t n,
               cudaStream_t stream);

// minGRU over the packed tokens of a step.  zug [T, 3 * width]: the gate, candidate and output-gate projections
// (biases added).  Per batch row b (tokens row_start[b] .. row_start[b + 1]) and channel, from state[slot_ids[b]]:
// S = (1 - z) S + z c with z = sigmoid(zug[., 0:width]), c = u + 1/2 for u >= 0 else sigmoid(u), u = zug[., width:2 width];
// y = S * silu(zug[., 2 width:]).  The last S goes back to the state.  All in float32.  max_new: the most tokens of
// any row; rows of many tokens run as chunks side by side and need scratch (exl3_mingru_scratch_bytes; 0: none).
size_t exl3_mingru_scratch_bytes(int B, int T, int width, int max_new);
int exl3_mingru_scan(const void* zug, int zug_dtype, void* y, int y_dtype, float* state, const int* slot_ids,
                     const int* row_start, int B, int T, int width, int max_new, float* scratch, size_t scratch_bytes,
                     cudaStream_t stream);

// Latent attention, step 1, per token, from the joint projection a [T, lda] (float32 or bfloat16):
//   cq [T, q_rank]      = rmsnorm(a[:, q_off : q_off + q_rank]) * wq
//   cache row of token  = [ rmsnorm(a[:, kv_off : kv_off + kv_rank]) * wkv | 0 .. | rope(a[:, kv_off + kv_rank : + rot_dim]) | 0 .. ]
//                         (the rotated part starts at rank_pad; the row is kv_row wide; skipped when pool is null)
//   gate [T, heads]     = sigmoid(a[:, g_off : g_off + heads])  (float32)
// The rotation takes the first rot features of the rot_dim part in half-split pairs at the token's position.
int exl3_latent_prep(const void* a, int a_dtype, int lda, int T, int q_off, int q_rank, const void* wq, int wq_dtype,
                     int kv_off, int kv_rank, int rot_dim, const void* wkv, int wkv_dtype, int g_off, int heads, float eps,
                     const float* inv_freq, const float* inv_freq_lo, int rot, const int* tok_pos, const int* tok_seq,
                     const int* block_table, int bt_stride, int page, void* pool, int pool_dtype, int kv_row,
                     int rank_pad, void* cq, int cq_dtype, float* gate, cudaStream_t stream);
// Products per head: out[t, h, n] = mul[t, h] * sum_k x[t, h, k] * w[h, k, n]  (n < N, k < K; mul null: 1), with
// x[t, h, k] at x + t * x_row + h * x_head + k and out likewise; float32 sums in the order of k.  With rot_dim > 0 the
// rot_dim features of x that follow a head's K are rotated (first rot of them, half-split pairs, at the token's
// position) and written behind the head's outputs at out[t, h, tail_off ..]; what lies between N and tail_off and
// behind the tail up to out_head is set to zero.  x, w and out have one element type.  With w null only the tails are
// written (the products come from elsewhere).
int exl3_head_gemm(const void* x, int64_t x_row, int x_head, const void* w, void* out, int64_t out_row, int out_head,
                   int dtype, int T, int heads, int K, int N, const float* mul, int rot_dim, int rot,
                   const float* inv_freq, const float* inv_freq_lo, const int* tok_pos, int tail_off,
                   cudaStream_t stream);

size_t exl3_argmax_scratch_bytes(int R, int V);
// Whole prompts on tcgen05 tensor cores with TMA loads from the paged cache (bfloat16, heads of 64 or 128, pages
// of 64, tiles of 128 queries); variant 0: chosen by the number of blocks, 1: a tile a block, 2: four blocks an SM
// (heads of 64), 3: two tiles a block (the first of the list with the last, and so on); see attention_prefill_tc.cu.
// chunk > 0: a query also sees nothing before its own block of chunk positions; sink != 0: one more in the softmax's
// denominator (both as in exl3_attn_tokens_ex; the decode kernel below takes the same two).
int exl3_attn_prefill_tc_supported(int dtype, int hd, int page);
int exl3_attn_prefill_tc_status();
int exl3_attn_prefill_tc(const void* q, int64_t q_row_stride, int T, void* out, const void* k_pool,
                         const void* v_pool, int64_t n_pool_rows, const int* block_table, int bt_stride,
                         const int* row_start, const int* row_pos0, const int* tile_seq, const int* tile_q0,
                         int n_tiles, int nh, int nkv, int hd, int page, int window, int chunk, int sink, float scale,
                         int variant, cudaStream_t stream);

// exl3_gemv_bf16 as the two sides of a norm that is no kernel of its own.  With ss_in the input is the x_raw of a
// producing call and the results are multiplied by rsqrt(sum of ss_in's blocks / width + eps) per batch row.
// With epilogue 2 no y is written: h[M, N] += result * rho, x_raw = h * norm_w, ss_out[16, ceil(N / 16)] = sums of
// squares per batch row and block.  See gemv_bf16.cuh.
int exl3_gemv_bf16_normed(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N,
                          int K, int epilogue, const float* ss_in, int ss_blocks, float eps, float width, float* h,
                          float rho, const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out,
                          cudaStream_t stream);

// The same projection and epilogues for up to 128 rows on tcgen05 tensor cores: the weights are the 128-row operand
// and stream once by TMA, K is cut over the blocks of a cluster and summed through distributed shared memory (no
// scratch, no atomics).  ss_in / ss_out are [rows >= M, blocks].  split: cuts of K, 0 = chosen from N and K; tiles:
// 128-row tiles of w per block (1 or 2), 0 = chosen.
// exl3_gemm_skinny_status() returns and clears the code a kernel left when one of its bounded waits ran out.
int exl3_gemm_skinny(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                     int epilogue, const float* ss_in, int ss_blocks, float eps, float width, float* h, float rho,
                     const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out, int split, int tiles,
                     cudaStream_t stream);
int exl3_gemm_skinny_status();
int exl3_gemm_skinny_max_rows();
int exl3_gemm_skinny_split(int N, int K);
int exl3_gemm_skinny_max_clusters(int s);

// Projections of many rows with two blocks of a cluster as one tensor core (tcgen05.mma.cta_group::2, tiles of
// 256 x 256): input and epilogues as exl3_gemm_skinny's (0 plain, 1 gated, 2 residual and the next norm's pieces),
// y bfloat16; ss_out is [M, exl3_gemm_pair_ss_blocks(N)].  exl3_gemm_pair_status() returns and clears the code a
// kernel left when one of its bounded waits ran out.
int exl3_gemm_pair(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int epilogue,
                   const float* ss_in, int ss_blocks, float eps, float width, float* h, float rho,
                   const void* norm_w, int norm_w_dtype, void* x_raw, float* ss_out, cudaStream_t stream);
// The q/k/v projection of heads of 64 with the half-split rotary encoding (rot 64, or 0 for none) and the cache
// write in its epilogue: of y [M, (nh + 2 nkv) * 64] only the queries' columns are written; rotated keys and
// values go to each token's place in the paged pools (write_kv).
int exl3_gemm_pair_rope(const void* x, const void* w, const void* bias, void* y, int M, int K, const float* ss_in,
                        int ss_blocks, float eps, float width, const int* tok_pos, const int* tok_seq,
                        const int* block_table, int bt_stride, const float* inv_freq, const float* inv_freq_lo, int rot,
                        float pos_scale, int nh, int nkv, int hd, int page, void* k_pool, void* v_pool,
                        int64_t pool_rows, int write_kv, cudaStream_t stream);
int exl3_gemm_pair_status();
int exl3_gemm_pair_ss_blocks(int N);

// Decoded tokens on the tensor cores with TMA loads from the paged cache (bfloat16, head_dim 64 or 128, pages of 64, up
// to 16 query heads per kv head, 1024 tokens, 256 chunks); arguments and scratch as exl3_attn_tokens; optionally
// it applies the rotary encoding and takes each token's own key and value from the projection's output, writing
// them to the cache itself.  head_split n (a divisor of the query heads per kv head): the query heads of a kv head
// as n groups of work.  in_block 1: a block per (token, group of heads), whose warps take the item's chunks (at most
// 4) and merge them in shared memory; 2: a cluster of two blocks (at most 8 chunks, the first block merging, the
// second one's records read out of its shared memory); no scratch in either.  twins 2 (with in_block 1 or 2, an even
// head_split and groups of up to 8 heads): two groups of query heads of a kv head per block, walking the same pages
// out of the same rings, 8 computing warps.  See attention_decode.cu.
int exl3_attn_decode_supported(int dtype, int T, int nh, int nkv, int hd, int page, int split_keys, int max_splits);
int exl3_attn_decode_status();
int exl3_attn_decode(const void* q, int64_t q_row_stride, void* out, void* k_pool, void* v_pool,
                     int64_t n_pool_rows, const int* block_table, int bt_stride, const int* tok_pos,
                     const int* tok_seq, int T, int nh, int nkv, int hd, int page, int window, int chunk, int sink,
                     float scale, int split_keys, int max_splits, float* scratch, size_t scratch_bytes, const float* inv_freq,
                     const float* inv_freq_lo, int rot, float pos_scale, int write_new, int head_split, int in_block,
                     int twins, cudaStream_t stream);

int exl3_argmax(const float* logits, int* out, int R, int V, void* scratch, size_t scratch_bytes,
                cudaStream_t stream);
// The reference's sampler on the device (see sampling_filtered.cu).  rows: float64 [R, 5] = temperature (<= 0:
// greedy), top_k (0: off; at most exl3_sample_filtered_cap()), top_p, min_p, uniform number in [0, 1).
int exl3_sample_filtered(const float* logits, const double* rows, int* out, int R, int V, cudaStream_t stream);
int exl3_sample_filtered_cap();
// counts: R device pointers (null: none) to int32 [V] token counts of the rows' contexts; params: float32 [R, 3] =
// repetition, presence and frequency penalty.  Changes logits in place.  exl3_sample_count adds the chosen tokens.
int exl3_sample_penalties(float* logits, int R, int V, const int* const* counts, const float* params,
                          cudaStream_t stream);
int exl3_sample_count(int* const* counts, const int* ids, int R, int V, cudaStream_t stream);

// A norm without statistics, y = tanh(alpha x) w + b, and the residual step of layers whose sublayers run side by
// side (see tanh_norm.cu): when a is given, h += m * (sa * a + sb * b) in place (b may be null); then up to two
// norms of the residual rows (out1, out2 null: skipped).  rows (no a then): only those rows of h are normed, into
// [n_rows, H].  Vectors and alphas are float32.
int exl3_tanh_norm_add(float* h, const void* a, int a_dtype, const void* b, int b_dtype, const float* sa, const float* sb,
                       float m, const int* rows, int n_rows, const float* w1, const float* b1, const float* alpha1,
                       void* out1, const float* w2, const float* b2, const float* alpha2, void* out2, int out_dtype,
                       int T, int H, cudaStream_t stream);

// A routed feed-forward (see moe.cu).  exl3_moe_route: wr float32 [E + extra, W]; idx int32 and wt float32 [T, top];
// gate_out float32 [T] = sigmoid of the extra row.  exl3_moe_plan: order int32 [P], plan int32 [4 + 3 * max tiles].
// exl3_moe_gemm: out[p] = act(W[e(p)] A[p / a_div]) for the planned pairs, W [n_experts, N, K]; act 0 none, 1 gelu
// (exact), 2 gelu by the tanh formula, 3 silu.  exl3_moe_combine: the weighted sum, float32 [T, H]; picks from
// n_experts on stand for the input x itself; shared (any type) is added times gate (null: as it is).
// exl3_moe_gemv: the same product for plans of tiles of at most exl3_moe_gemv_rows() rows (decode), bfloat16 A and W.
// exl3_moe_gather + exl3_moe_gemm_tc (moe_tc.cu): rows of x in the plan's order, and the product on tcgen05 tensor
// cores for plans of tiles of at most exl3_moe_tc_rows() rows; out bfloat16 in the plan's order or float32 at the
// pairs' own places.  plan[1] holds the number of planned pairs.
int exl3_moe_tile_rows();
int exl3_moe_gemv_rows();
int exl3_moe_tc_rows();
int exl3_moe_tc_status();
int exl3_moe_tc_supported(int N, int K);
int exl3_moe_max_tiles(int P, int n_experts, int tile_rows);
int exl3_moe_gemv(const void* A, int64_t lda, int a_div, const void* W, const int* order, const int* plan, void* out,
                  int out_dtype, int P, int n_experts, int N, int K, int act, cudaStream_t stream);
int exl3_moe_gather(const void* x, int64_t ldx, int top, const int* order, const int* plan, void* xs, int P, int K,
                    cudaStream_t stream);
int exl3_moe_gemm_tc(const void* A, const void* W, const int* order, const int* plan, void* out, int out_dtype, int P,
                     int n_experts, int N, int K, int act, cudaStream_t stream);
int exl3_moe_route(const void* x, int x_dtype, int64_t ldx, const float* wr, const float* corr, int T, int W, int E,
                   int extra, int groups, int keep, int top, float scale, int score_kind, int* idx, float* wt,
                   float* gate_out, cudaStream_t stream);
int exl3_moe_plan(const int* idx, int P, int n_experts, int tile_rows, int* order, int* plan, cudaStream_t stream);
int exl3_moe_gemm(const void* A, int a_dtype, int64_t lda, int a_div, const void* W, int w_dtype, const int* order,
                  const int* plan, void* out, int out_dtype, int P, int n_experts, int N, int K, int act,
                  cudaStream_t stream);
int exl3_moe_combine(const float* y, const int* idx, const float* wt, const void* x, int x_dtype, int64_t ldx,
                     const void* shared, int shared_dtype, const float* gate, float* out, int T, int H, int top,
                     int n_experts, cudaStream_t stream);

// Heads of several maps (see diff_attn.cu): rotation, widened queries and the cache write; and the combination of
// two maps' outputs.
int exl3_maps_prep(const void* x, int x_dtype, int64_t ld, int q_off, int k_off, int v_off, int T, int nh, int nkv,
                   int maps, int d, int dv, int row, int v_row, int rot, const float* f_hi, const float* f_lo,
                   const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride, int page, void* q_out,
                   int q_dtype, void* k_pool, void* v_pool, int pool_dtype, cudaStream_t stream);
int exl3_diff_combine(const void* a, int a_dtype, int a_row, const void* gate, int gate_dtype, int64_t gate_ld,
                      float lambda, float eps, float mult, void* out, int out_dtype, int out_row, int T, int heads,
                      int dv, cudaStream_t stream);

// exl3_attn_tokens_wide with three more options: with a window, keys at positions below keep_first stay visible; softcap > 0
// replaces a score s (after the scale) by softcap * tanh(s / softcap); sink_vals [heads] (float32, with sink) are the
// sink's scores per query head instead of 0.  max_splits must count the chunks of the kept keys too.
int exl3_attn_tokens_opt(const void* q, int64_t q_row_stride, void* out, int out_f32, int dtype, const void* k_pool,
                         const void* v_pool, const int* block_table, int bt_stride, const int* tok_pos,
                         const int* tok_seq, int T, int nh, int nkv, int hd, int hdv, int kv_row, int v_row, int page,
                         int window, int chunk, int sink, float scale, int split_keys, int max_splits, float* scratch,
                         size_t scratch_bytes, int keep_first, float softcap, const float* sink_vals, cudaStream_t stream);

// rows of gu are [gate (I) | up (I)], ld elements apart: out = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit)
// and u = clamp(up, -limit, limit).
int exl3_clamped_glu(const void* gu, int in_dtype, int64_t ld, void* out, int out_dtype, int T, int I, float limit,
                     float alpha, cudaStream_t stream);

// Hyper-connections (see hyper.cu): the write of a sublayer's output y into all S streams of x (mix [S, S] indexed
// [from, to], w_out [S]) and/or the read r = rmsnorm(sum_s w_in[s] x_s) * norm_w that follows it.  xin is [T, s_in, W]
// with s_in 1 (one row stands for S equal streams) or S; xout [T, S, W] may be xin.  rows (reads only): the tokens read.
int exl3_hyper_max_streams();
int exl3_hyper_step(const float* xin, int s_in, float* xout, int S, const void* y, int y_dtype, const float* mix,
                    const float* w_out, const float* w_in, const void* norm_w, int norm_w_dtype, float eps, void* r,
                    int r_dtype, const int* rows, int n_rows, int T, int W, cudaStream_t stream);

// Recurrences with a matrix state per head (see matrix_memory.cu).  q, k, v: rows of a step's packed tokens with their own
// pitches; states float32 per slot; out float32 [T, heads * dv].
int exl3_mlstm_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, int qkv_dtype,
                    const void* zi, const void* zf, int gate_dtype, int64_t ld_gate, float cap, float q_scale,
                    float* s_state, float* n_state, float* m_state, const int* slot_ids, const int* row_start,
                    float* out, int rows, int T, int heads, int dk, int dv, int max_new, float* scratch,
                    size_t scratch_bytes, cudaStream_t stream);
// Bytes of scratch that exl3_mlstm_scan needs for a step (0 for steps of short rows).
size_t exl3_mlstm_scan_scratch_bytes(int rows, int T, int heads, int dk, int dv, int max_new);
int exl3_delta_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, int qkv_dtype,
                    const void* zb, int zb_dtype, int64_t ld_zb, const void* za, int za_dtype, int64_t ld_za,
                    const float* a_log, const float* dt_bias, float* s_state, const int* slot_ids, const int* row_start,
                    float* out, int rows, int T, int heads, int qk_heads, int dk, int dv, int max_new, float* scratch,
                    size_t scratch_bytes, cudaStream_t stream);
size_t exl3_delta_scan_scratch_bytes(int rows, int T, int heads, int dk, int dv, int max_new);
// Short causal convolution per channel, SiLU, unit q and k heads (see matrix_memory.cu).  out float32 [T, 2 qk_heads dk +
// v_heads dv]; state float32 [slots, channels, n_taps - 1].
int exl3_conv_prep_max_taps();
int exl3_conv_prep(const void* x, int x_dtype, int64_t ldx, int q_off, int k_off, int v_off, const float* q_taps,
                   const float* k_taps, const float* v_taps, int qk_heads, int dk, int v_heads, int dv, int n_taps,
                   float eps, float q_scale, float* state, const int* slot_ids, const int* row_start, float* out,
                   int rows, int T, int max_new, cudaStream_t stream);
// out = sa * a + sb * b element by element, float32 out.
int exl3_scaled_sum2(const void* a, const void* b, int ab_dtype, float sa, float sb, float* out, int64_t n,
                     cudaStream_t stream);
int exl3_attn_prefill_tc_opt(const void* q, int64_t q_row_stride, int T, void* out, const void* k_pool, const void* v_pool,
                             int64_t n_pool_rows, const int* block_table, int bt_stride, const int* row_start,
                             const int* row_pos0, const int* tile_seq, const int* tile_q0, int n_tiles, int nh, int nkv,
                             int hd, int page, int window, int chunk, int sink, float scale, int variant, int keep_first,
                             float softcap, const float* sink_vals, cudaStream_t stream);
// y[M, N] (float32) = x[M, K] . w[N, K]^T (+ bias) for a handful of output features and many rows; x, w and bias of one
// type, K and the pitch of x multiples of 16 bytes.
int exl3_gemm_few_out(const void* x, int64_t ldx, const void* w, const void* bias, float* y, int in_dtype, int M, int N,
                      int K, cudaStream_t stream);
}
