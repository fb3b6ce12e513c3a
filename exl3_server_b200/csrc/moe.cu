// A routed feed-forward (mixture of experts): the router, the plan of a step's (token, expert) pairs, the experts'
// two projections as grouped matrix products, and the weighted sum.
//
//   router   z = Wr x (float32), s = softmax(z) or sigmoid(z) over all router outputs, choice c = s + correction;
//            the outputs form equal groups of neighbours, a group's score is its largest c, only the outputs of the
//            `keep` best groups can be chosen; the `top` largest c among those are the token's picks, each with the
//            weight s * scale (no renormalisation).  One more row of Wr may follow the router's: its sigmoid is a
//            gate per token (for a shared expert) that the same kernel leaves beside the picks.
//   plan     the pairs (token, pick) whose pick is an expert with weights, ordered by expert and cut into tiles of
//            at most a given number of rows of one expert; everything stays on the device (no count reaches the host), so the
//            step can be part of a recorded graph.
//   experts  mid[p] = act(W_up[e] x[token(p)]),  y[p] = W_down[e] mid[p], a block per (tile, 64 output features);
//            a row's sum walks K in order with one float32 accumulator, so it does not depend on the row's tile mates.
//   sum      out[t] = sum_k weight[t, k] * (y[t, k], or x[t] itself when pick k is an identity output: those are the
//            router outputs from n_experts on, which have no weights) + gate[t] * shared[t].
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int RT_TOK = 4;        // tokens a block of the router takes (one a warp for the choice)
constexpr int RT_WARPS = 16;     // warps of a block: router outputs are dealt out to them in turn
constexpr int RT_KC = 512;       // columns of x staged at a time
constexpr int RT_FEW_TOKENS = 64; // steps of up to so many tokens take the router's few-token form
constexpr int MOE_TM = 32;       // rows of a tile
constexpr int MOE_TN = 64;       // output features of a block
constexpr int MOE_TK = 32;

__device__ inline float moe_ld(const float* p) { return __ldcg(p); }
__device__ inline float moe_ld(const __nv_bfloat16* p) { return __bfloat162float(__ldcg(p)); }
__device__ inline void moe_st(float* p, float v) { *p = v; }
__device__ inline void moe_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// (value, index) of the larger; equal values: the lower index
__device__ inline void arg_better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
__device__ inline void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    arg_better(v, i, ov, oi);
  }
}

// The choice of one token by one warp: zt [E (+ S)] logits (scores on return), ct [E], gst and gkt [groups] scratch.
__device__ inline void route_choice(int t, int lane, float* zt, float* ct, float* gst, float* gkt,
                                    const float* __restrict__ corr, int E, int S, int groups, int keep, int top,
                                    float scale, int score_kind, int* idx, float* wt, float* gate_out) {
  // score_kind: bit 0 set: sigmoid scores (else softmax); bit 1 set: a group's score is the sum of its two largest
  // choice scores (else its largest)
  const bool group_pair = (score_kind & 2) != 0;
  score_kind &= 1;
  if (S && lane == 0) gate_out[t] = 1.0f / (1.0f + expf(-zt[E]));
  if (score_kind == 0) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zt[e]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(zt[e] - mx);
      ct[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
      const float s = ct[e] / sum;
      zt[e] = s;
      ct[e] = s + corr[e];
    }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float s = 1.0f / (1.0f + expf(-zt[e]));
      zt[e] = s;
      ct[e] = s + corr[e];
    }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float m = -INFINITY, m2 = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = ct[e];
        if (v > m) { m2 = m; m = v; } else if (v > m2) m2 = v;
      }
      gst[g] = (group_pair && per > 1) ? m + m2 : m;
      gkt[g] = 0.0f;
    }
    __syncwarp();
    for (int r = 0; r < keep; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gkt[g] == 0.0f) arg_better(bv, bi, gst[g], g);
      warp_argmax(bv, bi);
      if (lane == 0 && bi < groups) gkt[bi] = 1.0f;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gkt[e / per] == 0.0f) ct[e] = -INFINITY;   // not 0: choice scores may be negative
    __syncwarp();
  }
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (ct[e] > -INFINITY) arg_better(bv, bi, ct[e], e);
    warp_argmax(bv, bi);
    if (lane == 0) {
      if (bi < E) {
        idx[(int64_t)t * top + r] = bi;
        wt[(int64_t)t * top + r] = zt[bi] * scale;
        ct[bi] = -INFINITY;
      } else {
        idx[(int64_t)t * top + r] = -1;
        wt[(int64_t)t * top + r] = 0.0f;
      }
    }
    __syncwarp();
  }
}

template <typename TX>
__global__ void __launch_bounds__(RT_WARPS * 32)
moe_route_kernel(const TX* x, int64_t ldx, const float* __restrict__ wr, const float* __restrict__ corr, int T, int W,
                 int E, int S, int groups, int keep, int top, float scale, int score_kind, int* idx, float* wt,
                 float* gate_out) {
  extern __shared__ float rs[];
  const int R = E + S;
  float* xs = rs;                                  // [RT_TOK][RT_KC]
  float* z = xs + RT_TOK * RT_KC;                  // [RT_TOK][R]   logits, then scores
  float* c = z + RT_TOK * R;                       // [RT_TOK][E]   choice scores
  float* gs = c + RT_TOK * E;                      // [RT_TOK][groups] group scores
  float* gk = gs + RT_TOK * groups;                // [RT_TOK][groups] 1: the group is kept
  pdl_wait();
  pdl_trigger();
  const int t0 = blockIdx.x * RT_TOK;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < RT_TOK * R; i += blockDim.x) z[i] = 0.0f;
  for (int k0 = 0; k0 < W; k0 += RT_KC) {
    const int kc = min(RT_KC, W - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < RT_TOK * RT_KC; i += blockDim.x) {
      const int tok = i / RT_KC, col = i - tok * RT_KC;
      xs[i] = (t0 + tok < T && col < kc) ? moe_ld(x + (int64_t)(t0 + tok) * ldx + k0 + col) : 0.0f;
    }
    __syncthreads();
    for (int e = warp; e < R; e += RT_WARPS) {
      const float* wrow = wr + (int64_t)e * W + k0;
      float part[RT_TOK];
#pragma unroll
      for (int tok = 0; tok < RT_TOK; ++tok) part[tok] = 0.0f;
      // a fixed number of passes, so that the row's loads are all under way before the first is used
      float wv[RT_KC / 32];
#pragma unroll
      for (int i = 0; i < RT_KC / 32; ++i) wv[i] = lane + 32 * i < kc ? wrow[lane + 32 * i] : 0.0f;
#pragma unroll
      for (int i = 0; i < RT_KC / 32; ++i) {
#pragma unroll
        for (int tok = 0; tok < RT_TOK; ++tok) part[tok] = fmaf(wv[i], xs[tok * RT_KC + lane + 32 * i], part[tok]);
      }
#pragma unroll
      for (int tok = 0; tok < RT_TOK; ++tok) {
        const float s = warp_sum(part[tok]);
        if (lane == 0) z[tok * R + e] += s;
      }
    }
  }
  __syncthreads();
  const int t = t0 + warp;                         // this warp's token
  if (warp >= RT_TOK || t >= T) return;
  float* zt = z + warp * R;
  float* ct = c + warp * E;
  float* gst = gs + warp * groups;
  float* gkt = gk + warp * groups;
  route_choice(t, lane, zt, ct, gst, gkt, corr, E, S, groups, keep, top, scale, score_kind, idx, wt, gate_out);
}

// The router for steps of few tokens (decode), where the chain of dependent loads is what costs: a token a block,
// all of its input in shared memory at once, and the (output, piece of RT_KC columns) pairs spread over 32 warps, each
// of which has the next pair's piece of the router's row under way while it works on the present one.  The pieces'
// sums are added in their order, so the logits are those of a fixed order whatever the step holds.
constexpr int RS_WARPS = 32;

__device__ inline void rs_load(float (&wv)[RT_KC / 32], const float* __restrict__ wr, int W, int pieces, int item, int lane) {
  const int e = item / pieces, c0 = (item - e * pieces) * RT_KC;
  const float* wrow = wr + (int64_t)e * W + c0;
#pragma unroll
  for (int i = 0; i < RT_KC / 32; ++i) wv[i] = c0 + lane + 32 * i < W ? wrow[lane + 32 * i] : 0.0f;
}

template <typename TX>
__global__ void __launch_bounds__(RS_WARPS * 32)
moe_route_few_kernel(const TX* x, int64_t ldx, const float* __restrict__ wr, const float* __restrict__ corr, int T, int W,
                     int E, int S, int groups, int keep, int top, float scale, int score_kind, int* idx, float* wt,
                     float* gate_out) {
  extern __shared__ float rs[];
  const int R = E + S;
  const int pieces = (W + RT_KC - 1) / RT_KC;
  const int cols = pieces * RT_KC;
  float* xs = rs;                                  // [cols], zeros beyond W
  float* zp = xs + cols;                           // [pieces][R] sums of the pieces
  float* z = zp + pieces * R;                      // [R] logits, then scores
  float* c = z + R;                                // [E] choice scores
  float* gs = c + E;                               // [groups]
  float* gk = gs + groups;                         // [groups]
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_items = R * pieces;
  // the router's rows do not depend on the kernel before: the first piece is asked for before waiting for it
  float cur[RT_KC / 32], nxt[RT_KC / 32];
  if (warp < n_items) rs_load(cur, wr, W, pieces, warp, lane);
  pdl_wait();
  pdl_trigger();
  for (int i = threadIdx.x; i < cols; i += blockDim.x) xs[i] = i < W ? moe_ld(x + (int64_t)t * ldx + i) : 0.0f;
  __syncthreads();
  for (int item = warp; item < n_items; item += RS_WARPS) {
    const bool more = item + RS_WARPS < n_items;
    if (more) rs_load(nxt, wr, W, pieces, item + RS_WARPS, lane);
    const int e = item / pieces, pc = item - e * pieces;
    float part = 0.0f;
#pragma unroll
    for (int i = 0; i < RT_KC / 32; ++i) part = fmaf(cur[i], xs[pc * RT_KC + lane + 32 * i], part);
    part = warp_sum(part);
    if (lane == 0) zp[pc * R + e] = part;
    if (more) {
#pragma unroll
      for (int i = 0; i < RT_KC / 32; ++i) cur[i] = nxt[i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    float sum = 0.0f;
    for (int pc = 0; pc < pieces; ++pc) sum += zp[pc * R + i];
    z[i] = sum;
  }
  __syncthreads();
  if (warp == 0) route_choice(t, lane, z, c, gs, gk, corr, E, S, groups, keep, top, scale, score_kind, idx, wt, gate_out);
}

// One block.  plan[0]: number of tiles; plan[1]: planned pairs (places of `order` in use); then per tile (expert,
// first place in `order`, rows), from plan[4] on.  Tiles hold at most tile_rows rows.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* idx, int P, int n_experts, int tile_rows, int* order, int* plan) {
  extern __shared__ int ps[];                      // counts, offsets, cursors
  int* counts = ps;
  int* offs = ps + n_experts;
  int* cursor = offs + n_experts;
  pdl_wait();
  pdl_trigger();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = __ldcg(idx + p);
    if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < n_experts; ++e) {
      offs[e] = off;
      for (int r = 0; r < counts[e]; r += tile_rows) {
        plan[4 + 3 * nt] = e;
        plan[5 + 3 * nt] = off + r;
        plan[6 + 3 * nt] = min(tile_rows, counts[e] - r);
        ++nt;
      }
      off += counts[e];
    }
    plan[0] = nt;
    plan[1] = off;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = __ldcg(idx + p);
    if (e >= 0 && e < n_experts) order[offs[e] + atomicAdd(&cursor[e], 1)] = p;
  }
}

__device__ inline float moe_act(float v, int act) {
  if (act == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
  if (act == 2) return 0.5f * v * (1.0f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v)));
  if (act == 3) return v / (1.0f + expf(-v));
  return v;
}

// out[p, n] = act(sum_k A[p / a_div, k] * W[e(p), n, k]) for the pairs p of the block's tile.
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* A, int64_t lda, int a_div, const TW* __restrict__ Wt, const int* order, const int* plan,
                TO* out, int N, int K, int act) {
  __shared__ float As[MOE_TK][MOE_TM + 1];
  __shared__ float Ws[MOE_TK][MOE_TN + 1];
  __shared__ int rows[MOE_TM];
  pdl_wait();
  pdl_trigger();
  const int tile = blockIdx.x;
  if (tile >= __ldcg(plan)) return;
  const int e = __ldcg(plan + 4 + 3 * tile), start = __ldcg(plan + 5 + 3 * tile), nrows = __ldcg(plan + 6 + 3 * tile);
  const int n0 = blockIdx.y * MOE_TN;
  if (threadIdx.x < MOE_TM) rows[threadIdx.x] = threadIdx.x < nrows ? __ldcg(order + start + threadIdx.x) : -1;
  __syncthreads();
  const TW* Wexp = Wt + (int64_t)e * N * K;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;       // rows ty * 2 .. + 1, columns tx * 4 .. + 3
  float acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  const int lk = threadIdx.x & 31, lr = threadIdx.x >> 5;       // loads: 32 consecutive k, 8 rows a pass
  for (int k0 = 0; k0 < K; k0 += MOE_TK) {
#pragma unroll
    for (int r = lr; r < MOE_TM; r += 8) {
      const int p = rows[r];
      As[lk][r] = (p >= 0 && k0 + lk < K) ? moe_ld(A + (int64_t)(p / a_div) * lda + k0 + lk) : 0.0f;
    }
#pragma unroll
    for (int r = lr; r < MOE_TN; r += 8) {
      const int n = n0 + r;
      Ws[lk][r] = (n < N && k0 + lk < K) ? moe_ld(Wexp + (int64_t)n * K + k0 + lk) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_TK; ++k) {
      const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = Ws[k][tx * 4 + j];
        acc[0][j] = fmaf(a0, w, acc[0][j]);
        acc[1][j] = fmaf(a1, w, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int p = rows[ty * 2 + i];
    if (p < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) moe_st(out + (int64_t)p * N + n, moe_act(acc[i][j], act));
    }
  }
}


// ---- a few rows per expert (decode): the experts' matrices are read once, a warp per output feature ---------------
//
// out[p, n] = act(sum_k A[p / a_div, k] * W[e(p), n, k]) for tiles of at most MV_ROWS pairs.  K is walked in pieces
// of MV_KC columns: the block puts the tile's rows of A for the piece into shared memory, and every warp takes
// MV_FEAT output features, whose rows of W it reads in 16-byte pieces, all of a piece's loads under way before the
// first is used.  One float32 sum per (feature, pair) and lane; the lanes' sums meet in a fixed order, so a pair's
// result does not depend on its tile mates.
constexpr int MV_ROWS = 4, MV_FEAT = 4, MV_WARPS = 8, MV_KC = 1024, MV_IT = MV_KC / 256;

template <typename TO>
__global__ void __launch_bounds__(MV_WARPS * 32, 2)
moe_gemv_kernel(const __nv_bfloat16* A, int64_t lda, int a_div, const __nv_bfloat16* __restrict__ Wt, const int* order,
                const int* plan, TO* out, int N, int K, int act) {
  __shared__ int rows[MV_ROWS];
  __shared__ uint4 xs[MV_ROWS][MV_KC / 8];
  pdl_wait();
  pdl_trigger();
  const int tile = blockIdx.x;
  if (tile >= __ldcg(plan)) return;
  const int e = __ldcg(plan + 4 + 3 * tile), start = __ldcg(plan + 5 + 3 * tile), nrows = __ldcg(plan + 6 + 3 * tile);
  if (threadIdx.x < MV_ROWS) rows[threadIdx.x] = threadIdx.x < nrows ? __ldcg(order + start + threadIdx.x) : -1;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.y * MV_WARPS + warp) * MV_FEAT;
  const __nv_bfloat16* Wexp = Wt + (int64_t)e * N * K;
  float acc[MV_FEAT][MV_ROWS];
#pragma unroll
  for (int f = 0; f < MV_FEAT; ++f)
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) acc[f][r] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += MV_KC) {
    // this warp's pieces of W first: they come from DRAM
    uint4 wv[MV_FEAT][MV_IT];
#pragma unroll
    for (int f = 0; f < MV_FEAT; ++f) {
      const int n = min(n0 + f, N - 1);
#pragma unroll
      for (int it = 0; it < MV_IT; ++it) {
        const int k = k0 + it * 256 + lane * 8;
        wv[f][it] = k < K ? __ldg(reinterpret_cast<const uint4*>(Wexp + (int64_t)n * K + k)) : make_uint4(0, 0, 0, 0);
      }
    }
    for (int i = threadIdx.x; i < MV_ROWS * (MV_KC / 8); i += MV_WARPS * 32) {
      const int r = i / (MV_KC / 8), c = i - r * (MV_KC / 8);
      const int p = rows[r], k = k0 + c * 8;
      xs[r][c] = (p >= 0 && k < K) ? __ldcg(reinterpret_cast<const uint4*>(A + (int64_t)(p / a_div) * lda + k))
                                   : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    if (n0 < N) {
#pragma unroll
      for (int it = 0; it < MV_IT; ++it) {
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r) {
          if (r >= nrows) continue;
          const uint4 xv = xs[r][it * 32 + lane];
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int f = 0; f < MV_FEAT; ++f) {
            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv[f][it]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 a = __bfloat1622float2(xp[j]), b = __bfloat1622float2(wp[j]);
              acc[f][r] = fmaf(a.x, b.x, acc[f][r]);
              acc[f][r] = fmaf(a.y, b.y, acc[f][r]);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  if (n0 >= N) return;
#pragma unroll
  for (int f = 0; f < MV_FEAT; ++f)
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) {
      const float v = warp_sum(acc[f][r]);
      const int p = rows[r];
      if (lane == 0 && p >= 0 && n0 + f < N) moe_st(out + (int64_t)p * N + n0 + f, moe_act(v, act));
    }
}

// xs[i] = x[order[i] / top] for the planned pairs, in the plan's order (rows of K bfloat16, 16 bytes a thread).
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* x, int64_t ldx, int top, const int* order, const int* plan, __nv_bfloat16* xs,
                  int K) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x;
  if (i >= __ldcg(plan + 1)) return;
  const int p = __ldcg(order + i);
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(p / top) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + (int64_t)i * K);
  for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = __ldcg(src + c);
}

// VEC columns a thread (4: H a multiple of 4, float4 loads of y and stores of out).
template <typename TX, int VEC>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* y, const int* idx, const float* wt, const TX* x, int64_t ldx, const void* shared,
                   int shared_dtype, const float* gate, float* out, int T, int H, int top, int n_experts) {
  pdl_wait();
  pdl_trigger();
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (i >= (int64_t)T * H) return;
  const int t = (int)(i / H), col = (int)(i - (int64_t)t * H);
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.0f;
  for (int k = 0; k < top; ++k) {
    const int e = __ldcg(idx + (int64_t)t * top + k);
    if (e < 0) continue;
    const float w = __ldcg(wt + (int64_t)t * top + k);
    float v[VEC];
    if (e >= n_experts) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[j] = moe_ld(x + (int64_t)t * ldx + col + j);
    } else if (VEC == 4) {
      const float4 f = __ldcg(reinterpret_cast<const float4*>(y + ((int64_t)t * top + k) * H + col));
      v[0] = f.x; v[VEC > 1 ? 1 : 0] = f.y; v[VEC > 2 ? 2 : 0] = f.z; v[VEC > 3 ? 3 : 0] = f.w;
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[j] = __ldcg(y + ((int64_t)t * top + k) * H + col + j);
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = fmaf(w, v[j], acc[j]);
  }
  if (shared) {
    const float g = gate ? __ldcg(gate + t) : 1.0f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float s = shared_dtype == DT_F32 ? __ldcg(static_cast<const float*>(shared) + i + j)
                                             : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(shared) + i + j));
      acc[j] = gate ? fmaf(g, s, acc[j]) : acc[j] + s;
    }
  }
  if (VEC == 4) {
    *reinterpret_cast<float4*>(out + i) = make_float4(acc[0], acc[VEC > 1 ? 1 : 0], acc[VEC > 2 ? 2 : 0], acc[VEC > 3 ? 3 : 0]);
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) out[i + j] = acc[j];
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_moe_tile_rows() { return MOE_TM; }

extern "C" int exl3_moe_route(const void* x, int x_dtype, int64_t ldx, const float* wr, const float* corr, int T, int W,
                              int E, int extra, int groups, int keep, int top, float scale, int score_kind, int* idx,
                              float* wt, float* gate_out, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || W < 1 || E < 1 || extra < 0 || extra > 1 || groups < 1 || E % groups != 0 || keep < 1 || keep > groups ||
      top < 1 || top > keep * (E / groups) || (extra && gate_out == nullptr) || score_kind < 0 || score_kind > 3) {
    set_error("moe_route: bad sizes T=%d width=%d outputs=%d groups=%d keep=%d top=%d", T, W, E, groups, keep, top);
    return ERR_BAD_ARGUMENT;
  }
  // few tokens: a block a token with all of its input staged, when that fits
  const int pieces = ceil_div(W, RT_KC);
  const size_t smem_few = ((size_t)pieces * RT_KC + (size_t)(pieces + 1) * (E + extra) + E + 2 * groups) * sizeof(float);
  if (T <= RT_FEW_TOKENS && smem_few <= 160 * 1024 && (x_dtype == DT_F32 || x_dtype == DT_BF16)) {
    void (*few)(const float*, int64_t, const float*, const float*, int, int, int, int, int, int, int, float, int, int*,
                float*, float*) = moe_route_few_kernel<float>;
    void (*few_h)(const __nv_bfloat16*, int64_t, const float*, const float*, int, int, int, int, int, int, int, float,
                  int, int*, float*, float*) = moe_route_few_kernel<__nv_bfloat16>;
    if (smem_few > 48 * 1024) {
      cudaError_t e = x_dtype == DT_F32
                          ? cudaFuncSetAttribute(few, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_few)
                          : cudaFuncSetAttribute(few_h, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_few);
      if (e != cudaSuccess) { set_error("moe_route: shared memory refused: %s", cudaGetErrorString(e)); return (int)e; }
    }
    if (x_dtype == DT_F32)
      launch_pdl(few, dim3(T), dim3(RS_WARPS * 32), smem_few, stream, static_cast<const float*>(x), ldx, wr, corr, T, W, E,
                 extra, groups, keep, top, scale, score_kind, idx, wt, gate_out);
    else
      launch_pdl(few_h, dim3(T), dim3(RS_WARPS * 32), smem_few, stream, static_cast<const __nv_bfloat16*>(x), ldx, wr, corr,
                 T, W, E, extra, groups, keep, top, scale, score_kind, idx, wt, gate_out);
    return launch_status("moe_route");
  }
  const size_t smem = (size_t)RT_TOK * (RT_KC + (E + extra) + E + 2 * groups) * sizeof(float);
  if (smem > 200 * 1024) { set_error("moe_route: %d router outputs are too many", E); return ERR_UNSUPPORTED; }
  void (*kernel)(const float*, int64_t, const float*, const float*, int, int, int, int, int, int, int, float, int, int*,
                 float*, float*) = moe_route_kernel<float>;
  void (*kernel_h)(const __nv_bfloat16*, int64_t, const float*, const float*, int, int, int, int, int, int, int, float,
                   int, int*, float*, float*) = moe_route_kernel<__nv_bfloat16>;
  if (smem > 48 * 1024) {
    cudaError_t e = x_dtype == DT_F32
                        ? cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(kernel_h, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("moe_route: shared memory refused: %s", cudaGetErrorString(e)); return (int)e; }
  }
  const dim3 grid(ceil_div(T, RT_TOK)), threads(RT_WARPS * 32);
  if (x_dtype == DT_F32)
    launch_pdl(kernel, grid, threads, smem, stream, static_cast<const float*>(x), ldx, wr, corr, T, W, E, extra, groups,
               keep, top, scale, score_kind, idx, wt, gate_out);
  else if (x_dtype == DT_BF16)
    launch_pdl(kernel_h, grid, threads, smem, stream, static_cast<const __nv_bfloat16*>(x), ldx, wr, corr, T, W, E, extra,
               groups, keep, top, scale, score_kind, idx, wt, gate_out);
  else { set_error("moe_route: unsupported element type %d", x_dtype); return ERR_UNSUPPORTED; }
  return launch_status("moe_route");
}

extern "C" int exl3_moe_plan(const int* idx, int P, int n_experts, int tile_rows, int* order, int* plan,
                             cudaStream_t stream) {
  if (P == 0) return 0;
  if (P < 0 || n_experts < 1 || n_experts > 4096 || tile_rows < 1) { set_error("moe_plan: bad sizes"); return ERR_BAD_ARGUMENT; }
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), (size_t)3 * n_experts * sizeof(int), stream, idx, P, n_experts,
             tile_rows, order, plan);
  return launch_status("moe_plan");
}

// The most tiles of at most tile_rows rows that a step of P pairs over n_experts experts can have.
extern "C" int exl3_moe_max_tiles(int P, int n_experts, int tile_rows) {
  return tile_rows < 1 ? 0 : min(P, P / tile_rows + n_experts);
}

template <typename TA, typename TW, typename TO>
static int moe_gemm_launch(const void* A, int64_t lda, int a_div, const void* W, const int* order, const int* plan,
                           void* out, int P, int n_experts, int N, int K, int act, cudaStream_t stream) {
  const dim3 grid(exl3_moe_max_tiles(P, n_experts, MOE_TM), ceil_div(N, MOE_TN));
  launch_pdl(moe_gemm_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, static_cast<const TA*>(A), lda, a_div,
             static_cast<const TW*>(W), order, plan, static_cast<TO*>(out), N, K, act);
  return launch_status("moe_gemm");
}

extern "C" int exl3_moe_gemm(const void* A, int a_dtype, int64_t lda, int a_div, const void* W, int w_dtype,
                             const int* order, const int* plan, void* out, int out_dtype, int P, int n_experts, int N,
                             int K, int act, cudaStream_t stream) {
  if (P == 0) return 0;
  if (P < 0 || n_experts < 1 || N < 1 || K < 1 || a_div < 1 || act < 0 || act > 3) {
    set_error("moe_gemm: bad sizes pairs=%d experts=%d N=%d K=%d", P, n_experts, N, K);
    return ERR_BAD_ARGUMENT;
  }
  if (ceil_div(N, MOE_TN) > 65535) { set_error("moe_gemm: grid too large"); return ERR_UNSUPPORTED; }
#define EXL3_MOE(TA, DA, TW, DW, TO, DO)                                                                     \
  if (a_dtype == DA && w_dtype == DW && out_dtype == DO)                                                     \
    return moe_gemm_launch<TA, TW, TO>(A, lda, a_div, W, order, plan, out, P, n_experts, N, K, act, stream);
  EXL3_MOE(float, DT_F32, float, DT_F32, float, DT_F32)
  EXL3_MOE(__nv_bfloat16, DT_BF16, __nv_bfloat16, DT_BF16, __nv_bfloat16, DT_BF16)
  EXL3_MOE(__nv_bfloat16, DT_BF16, __nv_bfloat16, DT_BF16, float, DT_F32)
  EXL3_MOE(float, DT_F32, __nv_bfloat16, DT_BF16, float, DT_F32)
  EXL3_MOE(float, DT_F32, __nv_bfloat16, DT_BF16, __nv_bfloat16, DT_BF16)
#undef EXL3_MOE
  set_error("moe_gemm: unsupported element types %d x %d -> %d", a_dtype, w_dtype, out_dtype);
  return ERR_UNSUPPORTED;
}

extern "C" int exl3_moe_gemv_rows() { return MV_ROWS; }

// The same product as exl3_moe_gemm for a plan of tiles of at most exl3_moe_gemv_rows() rows; bfloat16 A and W with K a
// multiple of 8 and 16-byte aligned rows; out bfloat16 or float32.
extern "C" int exl3_moe_gemv(const void* A, int64_t lda, int a_div, const void* W, const int* order, const int* plan,
                             void* out, int out_dtype, int P, int n_experts, int N, int K, int act, cudaStream_t stream) {
  if (P == 0) return 0;
  if (P < 0 || n_experts < 1 || N < 1 || K < 8 || K % 8 != 0 || lda % 8 != 0 || a_div < 1 || act < 0 || act > 3 ||
      !aligned16(A) || !aligned16(W)) {
    set_error("moe_gemv: bad sizes pairs=%d experts=%d N=%d K=%d (K and the row pitch multiples of 8, 16-byte aligned)", P,
              n_experts, N, K);
    return ERR_BAD_ARGUMENT;
  }
  const dim3 grid(exl3_moe_max_tiles(P, n_experts, MV_ROWS), ceil_div(N, MV_WARPS * MV_FEAT));
  if (grid.y > 65535) { set_error("moe_gemv: grid too large"); return ERR_UNSUPPORTED; }
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(A);
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(W);
  if (out_dtype == DT_BF16)
    launch_pdl(moe_gemv_kernel<__nv_bfloat16>, grid, dim3(MV_WARPS * 32), 0, stream, a, lda, a_div, w, order, plan,
               static_cast<__nv_bfloat16*>(out), N, K, act);
  else if (out_dtype == DT_F32)
    launch_pdl(moe_gemv_kernel<float>, grid, dim3(MV_WARPS * 32), 0, stream, a, lda, a_div, w, order, plan,
               static_cast<float*>(out), N, K, act);
  else { set_error("moe_gemv: unsupported output type %d", out_dtype); return ERR_UNSUPPORTED; }
  return launch_status("moe_gemv");
}

extern "C" int exl3_moe_gather(const void* x, int64_t ldx, int top, const int* order, const int* plan, void* xs, int P,
                               int K, cudaStream_t stream) {
  if (P == 0) return 0;
  if (P < 0 || top < 1 || K < 8 || K % 8 != 0 || ldx % 8 != 0 || !aligned16(x) || !aligned16(xs)) {
    set_error("moe_gather: bad sizes pairs=%d K=%d", P, K);
    return ERR_BAD_ARGUMENT;
  }
  launch_pdl(moe_gather_kernel, dim3(P), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), ldx, top, order, plan,
             static_cast<__nv_bfloat16*>(xs), K);
  return launch_status("moe_gather");
}

extern "C" int exl3_moe_combine(const float* y, const int* idx, const float* wt, const void* x, int x_dtype, int64_t ldx,
                                const void* shared, int shared_dtype, const float* gate, float* out, int T, int H,
                                int top, int n_experts, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || top < 1) { set_error("moe_combine: bad sizes"); return ERR_BAD_ARGUMENT; }
  const bool vec = H % 4 == 0 && (y == nullptr || aligned16(y)) && aligned16(out);
  const int64_t blocks = ((int64_t)T * H / (vec ? 4 : 1) + 255) / 256;
  if (blocks > 0x7fffffffLL) { set_error("moe_combine: too many elements"); return ERR_UNSUPPORTED; }
  if (x_dtype != DT_F32 && x_dtype != DT_BF16) { set_error("moe_combine: unsupported element type %d", x_dtype); return ERR_UNSUPPORTED; }
#define EXL3_COMBINE(TX, VEC)                                                                                        \
  launch_pdl(moe_combine_kernel<TX, VEC>, dim3((unsigned)blocks), dim3(256), 0, stream, y, idx, wt,                  \
             static_cast<const TX*>(x), ldx, shared, shared_dtype, gate, out, T, H, top, n_experts)
  if (x_dtype == DT_F32) { if (vec) EXL3_COMBINE(float, 4); else EXL3_COMBINE(float, 1); }
  else { if (vec) EXL3_COMBINE(__nv_bfloat16, 4); else EXL3_COMBINE(__nv_bfloat16, 1); }
#undef EXL3_COMBINE
  return launch_status("moe_combine");
}

// The activation of experts with a bounded gate: rows of gu hold [gate (I) | up (I)];
//   g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1)
// float32 inside.  Four features a thread where the sizes allow 8- or 16-byte accesses.
namespace exl3 {

template <typename T> __device__ inline void cg_load4(const T* p, float (&v)[4]);
template <> __device__ inline void cg_load4<float>(const float* p, float (&v)[4]) { load_vec_cg(p, v); }
template <> __device__ inline void cg_load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 r = __ldcg(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
  v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
template <typename T> __device__ inline void cg_store4(T* p, const float (&v)[4]);
template <> __device__ inline void cg_store4<float>(float* p, const float (&v)[4]) { store_vec(p, v); }
template <> __device__ inline void cg_store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&lo);
  r.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = r;
}

__device__ inline float clamped_glu_one(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

template <typename TI, typename TO, int V>
__global__ void __launch_bounds__(256)
clamped_glu_kernel(const TI* __restrict__ gu, int64_t ld, TO* __restrict__ out, int T, int I, float limit, float alpha) {
  pdl_wait();
  pdl_trigger();
  const int per_row = I / V;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)T * per_row) return;
  const int64_t t = idx / per_row;
  const int c = (int)(idx - t * per_row) * V;
  if (V == 4) {
    float g[4], u[4], y[4];
    cg_load4<TI>(gu + t * ld + c, g);
    cg_load4<TI>(gu + t * ld + I + c, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) y[e] = clamped_glu_one(g[e], u[e], limit, alpha);
    cg_store4<TO>(out + t * I + c, y);
  } else {
    const float g = Elem<TI>::load(gu + t * ld + c), u = Elem<TI>::load(gu + t * ld + I + c);
    Elem<TO>::store(out + t * I + c, clamped_glu_one(g, u, limit, alpha));
  }
}

template <typename TI, typename TO>
static int clamped_glu_launch(const void* gu, int64_t ld, void* out, int T, int I, float limit, float alpha, bool vec,
                              cudaStream_t stream) {
  const int64_t total = (int64_t)T * (I / (vec ? 4 : 1));
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) { set_error("clamped_glu: too many elements"); return ERR_UNSUPPORTED; }
  if (vec)
    launch_pdl(clamped_glu_kernel<TI, TO, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, static_cast<const TI*>(gu), ld,
               static_cast<TO*>(out), T, I, limit, alpha);
  else
    launch_pdl(clamped_glu_kernel<TI, TO, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, static_cast<const TI*>(gu), ld,
               static_cast<TO*>(out), T, I, limit, alpha);
  return launch_status("clamped_glu");
}

}  // namespace exl3

extern "C" int exl3_clamped_glu(const void* gu, int in_dtype, int64_t ld, void* out, int out_dtype, int T, int I,
                                float limit, float alpha, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || I < 1 || ld < 2 * (int64_t)I || !(limit > 0.0f)) {
    set_error("clamped_glu: bad sizes rows=%d inner=%d pitch=%lld limit=%g", T, I, (long long)ld, (double)limit);
    return ERR_BAD_ARGUMENT;
  }
  const bool vec = I % 4 == 0 && ld % 4 == 0 && aligned16(gu) && aligned16(out);
  if (in_dtype == DT_F32 && out_dtype == DT_F32) return clamped_glu_launch<float, float>(gu, ld, out, T, I, limit, alpha, vec, stream);
  if (in_dtype == DT_F32 && out_dtype == DT_BF16) return clamped_glu_launch<float, __nv_bfloat16>(gu, ld, out, T, I, limit, alpha, vec, stream);
  if (in_dtype == DT_BF16 && out_dtype == DT_BF16) return clamped_glu_launch<__nv_bfloat16, __nv_bfloat16>(gu, ld, out, T, I, limit, alpha, vec, stream);
  if (in_dtype == DT_BF16 && out_dtype == DT_F32) return clamped_glu_launch<__nv_bfloat16, float>(gu, ld, out, T, I, limit, alpha, vec, stream);
  set_error("clamped_glu: unsupported element types %d -> %d", in_dtype, out_dtype);
  return ERR_UNSUPPORTED;
}
