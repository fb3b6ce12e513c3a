// Recurrences whose state is a matrix per head and whose step is not a plain decayed sum, and the short convolution that
// feeds one of them.  The state S [dk, dv] of a (sequence, head) is float32, kept per sequence by the cache, read at a
// row's first token of the step and written at its last, so a prompt cut into steps in any way and token-by-token
// decoding walk the same chain in the same order of arithmetic.
//
// Mode 0, a matrix memory with exponential gates (mLSTM).  Per head, with the gates' pre-activations zi, zf:
//   i = cap tanh(zi / cap),  f = logsigmoid(cap tanh(zf / cap)),  m' = max(f + m, i)        (m starts at 0)
//   S' = exp(f + m - m') S + exp(i - m') k v^T,   n' likewise with k alone
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)                                          (q times q_scale)
// State: S (kept column by column, [dv][dk]), n [dk], m.
//
// Mode 1, the gated delta rule.  Per head, with a decay per key channel g = exp(-exp(A_h) softplus(za + dt_bias)) and
// beta = sigmoid(zb):
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                      (the read sees the write)
// Query and key heads may be shared by several value heads (head h reads q/k head h / (heads / qk_heads)).
//
// Both: a block owns some columns of S of one (row, head) and walks the row's tokens in order; a column lives in the
// registers of L = 4 or 8 neighbouring lanes (a lane holds NR rows in a row, i = NR (lane % L) + r), the two dot products of a token are summed
// inside those lanes; q, k, the decays, the block's values and the tokens' scalars are staged in shared memory a chunk of
// tokens at a time (the gates' exponentials of a chunk side by side, only the running maximum in order), so that a
// token's step reads shared memory only and a chunk's load latency is paid once.
//
// Mode 1 for prompts: a token multiplies the state by (I - beta k k^T) diag(g) and adds beta k v^T, so a piece of tokens
// multiplies the state it finds by a matrix T [dk x dk] and adds what it leaves from a zero state.  The summaries' kernel
// gets T by walking dk more columns that start as the identity with values of zero; a fold (delta_fold_kernel) takes
// S <- T S + B through a row's pieces in order; the outputs' kernel starts every piece from the state before it.
//
// Mode 0 for prompts: between two tokens the state only decays by one number a head (a = exp(f + m - m')) once the
// running maxima are known, so a row is cut into pieces that run side by side.  A first kernel walks the gates of a row
// in order and leaves a, b = exp(i - m') and exp(-m') per token; a second walks every piece but a row's last from a
// zero state and leaves S and n at its end with the piece's whole decay (and keeps a copy of the states the step found);
// a third folds, per element, a row's summaries in order into the states after every piece; a fourth starts every piece
// from the state after the piece before it (a row's first from the copy) and walks it with the outputs; a row's last
// piece writes the states back.  The pieces' borders count from the row's first token
// of the step, so a prompt cut otherwise sums in another order: roundings differ, nothing else.
//
// conv_prep: per channel a causal convolution over time of `taps` taps (the last tap is the current token's), no bias,
// zeros before the sequence's start, then SiLU; the q and k heads are then made unit vectors, x / sqrt(sum x^2 + eps),
// and q is multiplied by q_scale.  The last taps - 1 inputs of every channel are per-sequence state.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int MM_COLS = 32;             // columns a block owns; a column is shared by L = 4 or 8 lanes (a template parameter)
constexpr int MM_CHUNK = 128;           // tokens whose vectors are staged in shared memory at once (at most a block's threads)
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_MIN_CHUNK = 4;       // tokens a warp walks at least
constexpr int CONV_WARPS = 4;
constexpr int CONV_MAX_PER_LANE = 8;    // heads of up to 256 channels

__device__ inline float mm_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}

// Four consecutive elements (the address a multiple of four elements, the base 16-byte aligned).
__device__ inline void mm_load4(const void* p, int dtype, int64_t i, float (&v)[4]) {
  if (dtype == DT_F32) {
    load_vec_cg(static_cast<const float*>(p) + i, v);
  } else {
    const uint2 r = __ldcg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i));
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
  }
}

__device__ inline float mm_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ inline float mm_logsigmoid(float x) { return -mm_softplus(-x); }

struct MatrixMemoryArgs {
  const void* q; const void* k; const void* v; int qkv_dtype;
  int64_t ldq, ldk, ldv;              // row pitches (elements); heads are dense inside a row
  float q_scale;
  // mode 0
  const void* zi; const void* zf; int gate_dtype; int64_t ld_gate; float cap;
  float* n_state; float* m_state;     // [slots, H, dk], [slots, H]
  // mode 1
  const void* zb; int zb_dtype; int64_t ld_zb;        // [T, H]
  const void* za; int za_dtype; int64_t ld_za;        // [T, H * dk]
  const float* a_log; const float* dt_bias;           // [H], [H * dk]
  float* s_state;                     // [slots, H, dv, dk]: a column of S is contiguous
  const int* slot_ids; const int* row_start;
  float* out;                         // [T, H * dv]
  int H, QH, dk, dv;
  int vec;                            // q, k (and za) can be read four elements at a time
  // Mode 0 for rows of many tokens: pieces of piece_len tokens side by side (see below).  pre [T, H, 4] holds every
  // token's a, b, exp(-m'); phase 1 leaves a piece's summary, phase 2 folds the summaries before a piece into its start.
  const float* pre;
  int phase, piece_len, pieces;       // phase 0: a row is one piece and the gates are worked out here
  float* sums;                        // [rows * pieces, H, dv * dk + dk + 1]: S and n at a piece's end from zero, its decay
  float* init;                        // [rows, H, dv * dk + dk]: the states as the step found them
};

// Stages a chunk of up to MM_CHUNK tokens from t0 on into shared memory: q (scaled) and k as [token][dk], for mode 1 the
// decays likewise, the block's columns of v as [token][MM_COLS], and the tokens' scalars as [token][4]: mode 0
// a = exp(f + m - m'), b = exp(i - m'), exp(-m'); mode 1 beta.  Every thread of the block takes part; the running
// maximum m_run (mode 0) is carried by every thread alike.  Ends with a barrier.
template <int MODE>
__device__ inline void mm_stage_chunk(const MatrixMemoryArgs& g, int t0, int n, int h, int qh, int j0, float* sq, float* sk,
                                      float* sg, float* sv, float* sc, float* sgate, float& m_run, int ln) {
  const int dk = g.dk, dv = g.dv;
  if (ln > dk) {                                    // rows beyond the key's features: keys of zero, decays of one
    const int pad = ln - dk;
    for (int e = threadIdx.x; e < n * pad; e += blockDim.x) {
      const int tt = e / pad, i = dk + e - tt * pad;
      sq[tt * ln + i] = 0.0f;
      sk[tt * ln + i] = 0.0f;
      if (MODE == 1) sg[tt * ln + i] = 1.0f;
    }
  }
  if (g.vec) {
    // rows of q, k (and the decays' pre-activations) in 16-byte pieces, four pieces of each in flight a thread
    const int per = dk / 4;                           // pieces of four features in a token's row
    const float ea = MODE == 1 ? expf(__ldg(g.a_log + h)) : 0.0f;
    for (int e0 = threadIdx.x; e0 < n * per; e0 += blockDim.x * 4) {
      float vq[4][4], vk[4][4], va[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * blockDim.x;
        if (e < n * per) {
          const int tt = e / per, i = (e - tt * per) * 4;
          const int64_t t = t0 + tt;
          mm_load4(g.q, g.qkv_dtype, t * g.ldq + (int64_t)qh * dk + i, vq[u]);
          mm_load4(g.k, g.qkv_dtype, t * g.ldk + (int64_t)qh * dk + i, vk[u]);
          if (MODE == 1) mm_load4(g.za, g.za_dtype, t * g.ld_za + (int64_t)h * dk + i, va[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = e0 + u * blockDim.x;
        if (e < n * per) {
          const int tt = e / per, i = (e - tt * per) * 4;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            sq[tt * ln + i + c] = vq[u][c] * g.q_scale;
            sk[tt * ln + i + c] = vk[u][c];
            if (MODE == 1) sg[tt * ln + i + c] = expf(-ea * mm_softplus(va[u][c] + __ldg(g.dt_bias + h * dk + i + c)));
          }
        }
      }
    }
  } else {
    for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
      const int tt = e / dk, i = e - tt * dk;
      const int64_t t = t0 + tt;
      sq[tt * ln + i] = mm_load(g.q, g.qkv_dtype, t * g.ldq + (int64_t)qh * dk + i) * g.q_scale;
      sk[tt * ln + i] = mm_load(g.k, g.qkv_dtype, t * g.ldk + (int64_t)qh * dk + i);
      if (MODE == 1) {
        const float za = mm_load(g.za, g.za_dtype, t * g.ld_za + (int64_t)h * dk + i) + __ldg(g.dt_bias + h * dk + i);
        sg[tt * ln + i] = expf(-expf(__ldg(g.a_log + h)) * mm_softplus(za));
      }
    }
  }
  for (int e = threadIdx.x; e < n * MM_COLS; e += blockDim.x) {
    const int tt = e / MM_COLS, c = e - tt * MM_COLS;
    sv[e] = (j0 + c < dv) ? mm_load(g.v, g.qkv_dtype, (int64_t)(t0 + tt) * g.ldv + (int64_t)h * dv + j0 + c) : 0.0f;
  }
  if (MODE == 1) {
    if (threadIdx.x < n)
      sc[threadIdx.x * 4 + 3] = 1.0f / (1.0f + expf(-mm_load(g.zb, g.zb_dtype, (int64_t)(t0 + threadIdx.x) * g.ld_zb + h)));
    __syncthreads();
    return;
  }
  if (g.pre != nullptr) {                           // the tokens' factors were worked out by mlstm_gates_kernel
    if (threadIdx.x < n) {
      const float4 f4 = __ldcg(reinterpret_cast<const float4*>(g.pre) + (int64_t)(t0 + threadIdx.x) * g.H + h);
      sc[threadIdx.x * 4 + 0] = f4.x;
      sc[threadIdx.x * 4 + 1] = f4.y;
      sc[threadIdx.x * 4 + 2] = f4.z;
    }
    __syncthreads();
    return;
  }
  // mode 0: the gates of the chunk's tokens side by side, then the running maximum in order, then the three factors
  if (threadIdx.x < n) {
    const int64_t t = t0 + threadIdx.x;
    const float zi = mm_load(g.zi, g.gate_dtype, t * g.ld_gate + h), zf = mm_load(g.zf, g.gate_dtype, t * g.ld_gate + h);
    sgate[2 * threadIdx.x] = g.cap * tanhf(zi / g.cap);
    sgate[2 * threadIdx.x + 1] = mm_logsigmoid(g.cap * tanhf(zf / g.cap));
  }
  __syncthreads();
  // every thread walks the maxima itself (a few instructions a token, no exponentials): all hold the same m_run
  float m = m_run;
  float m_before = m, m_after = m;
  for (int tt = 0; tt < n; ++tt) {
    const float mn = fmaxf(sgate[2 * tt + 1] + m, sgate[2 * tt]);
    if (tt == (int)threadIdx.x) { m_before = m; m_after = mn; }
    m = mn;
  }
  m_run = m;
  if (threadIdx.x < n) {
    const float gi = sgate[2 * threadIdx.x], gf = sgate[2 * threadIdx.x + 1];
    sc[threadIdx.x * 4 + 0] = expf(gf + m_before - m_after);
    sc[threadIdx.x * 4 + 1] = expf(gi - m_after);
    sc[threadIdx.x * 4 + 2] = expf(-m_after);
  }
  __syncthreads();
}

// L: lanes that share a column (4 or 8); NR: rows of a column that one lane holds (dk <= L NR).  The state lies in
// memory column by column, [dv][dk], so that the lanes of a column read and write neighbouring addresses.
template <int MODE, int L, int NR>
__global__ void __launch_bounds__(L * MM_COLS) matrix_memory_kernel(MatrixMemoryArgs g, int chunk) {
  extern __shared__ __align__(16) float sm[];        // q, k, (g) [chunk][LN]; v [chunk][MM_COLS]; scalars [chunk][4]; gates [chunk][2]
  constexpr int LN = L * NR;                         // a token's vectors padded to the rows the lanes hold
  const int dk = g.dk, dv = g.dv;
  float* sq = sm;
  float* sk = sq + chunk * LN;
  float* sg = sk + chunk * LN;
  float* sv = sg + (MODE == 1 ? chunk * LN : 0);
  float* sc = sv + chunk * MM_COLS;
  float* sgate = sc + chunk * 4;
  const int phase = g.phase;
  const int row = phase ? blockIdx.x / g.pieces : blockIdx.x, piece = phase ? blockIdx.x - row * g.pieces : 0;
  const int h = blockIdx.y, j0 = blockIdx.z * MM_COLS;
  const int qh = h / (g.H / g.QH);
  const int lane4 = threadIdx.x & (L - 1);          // this lane's place among the lanes of its column
  const int col = threadIdx.x / L;
  const int j = j0 + col;
  // Mode 1, phase 1: dk more columns behind the values' own.  They start as the identity and get values of zero, so
  // they end as the matrix that the piece's tokens multiply a state by (the step is linear in the state).
  const bool t_col = MODE == 1 && phase == 1 && j >= dv && j < dv + dk;
  const bool col_ok = j < dv || t_col;
  pdl_wait();
  pdl_trigger();
  int t0 = __ldcg(g.row_start + row), t1 = __ldcg(g.row_start + row + 1);
  if (t0 >= t1) return;
  const int slot = __ldcg(g.slot_ids + row);
  float* Sp = g.s_state + ((int64_t)slot * g.H + h) * dk * dv;
  float S[NR], nn[NR];
  const int row_end = t1;
  // floats of a piece's summary: mode 0 S, n and the piece's decay; mode 1 S and the dk columns of the piece's matrix
  const int rec = MODE == 0 ? dv * dk + dk + 1 : (dv + dk) * dk;
  float* init = phase ? g.init + ((int64_t)row * g.H + h) * (MODE == 0 ? dv * dk + dk : dv * dk) : nullptr;
  if (phase) {                                       // this block's piece of the row
    t0 += piece * g.piece_len;
    if (t0 >= t1) return;
    t1 = min(t1, t0 + g.piece_len);
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int i = lane4 * NR + r;
    S[r] = 0.0f;
    nn[r] = 0.0f;
    if (phase == 2) {
      // the states at this piece's start: the step's own for a row's first piece, else what the fold left in the
      // summary of the piece before
      const float* from = piece == 0 ? init : g.sums + (((int64_t)row * g.pieces + piece - 1) * g.H + h) * rec;
      if (col_ok && i < dk) S[r] = __ldcg(from + (int64_t)j * dk + i);
      if (MODE == 0 && i < dk) nn[r] = __ldcg(from + dv * dk + i);
    } else if (phase == 0 || piece == 0) {
      if (j < dv && i < dk) S[r] = Sp[(int64_t)j * dk + i];
      if (MODE == 0 && i < dk) nn[r] = g.n_state[((int64_t)slot * g.H + h) * dk + i];
    }
  }
  if (phase == 1) {
    if (piece == 0) {                                // the states as the step found them, for the third kernel
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int i = lane4 * NR + r;
        if (j < dv && i < dk) init[(int64_t)j * dk + i] = S[r];
        if (MODE == 0 && blockIdx.z == 0 && col == 0 && i < dk) init[dv * dk + i] = nn[r];
        S[r] = 0.0f;                                 // a summary starts from nothing
        nn[r] = 0.0f;
      }
    }
    if (t1 >= row_end) return;                       // nobody needs the summary of a row's last piece
    if (t_col) {
#pragma unroll
      for (int r = 0; r < NR; ++r) S[r] = (lane4 * NR + r == j - dv) ? 1.0f : 0.0f;
    }
  }
  float decay = 1.0f;                                // the piece's whole decay (phase 1)
  float m_run = (MODE == 0 && phase == 0) ? g.m_state[(int64_t)slot * g.H + h] : 0.0f;
  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int n = min(chunk, t1 - c0);
    mm_stage_chunk<MODE>(g, c0, n, h, qh, j0, sq, sk, sg, sv, sc, sgate, m_run, LN);
    for (int tt = 0; tt < n; ++tt) {
      // this lane's rows of the token's vectors, 16 bytes at a time (the padding makes every row valid)
      const float4* q4 = reinterpret_cast<const float4*>(sq + tt * LN + lane4 * NR);
      const float4* k4 = reinterpret_cast<const float4*>(sk + tt * LN + lane4 * NR);
      const float vj = sv[tt * MM_COLS + col];
      float o = 0.0f;
      if (MODE == 0) {
        const float a = sc[tt * 4], bw = sc[tt * 4 + 1];
        const float bv = bw * vj;
        decay *= a;
        if (phase == 1) {                              // a summary needs no read-out
#pragma unroll
          for (int r4 = 0; r4 < NR / 4; ++r4) {
            const float4 kk = k4[r4];
            const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              S[r4 * 4 + c] = fmaf(a, S[r4 * 4 + c], kv[c] * bv);
              nn[r4 * 4 + c] = fmaf(a, nn[r4 * 4 + c], bw * kv[c]);
            }
          }
        } else {
          float num = 0.0f, nq = 0.0f;
#pragma unroll
          for (int r4 = 0; r4 < NR / 4; ++r4) {
            const float4 kk = k4[r4], qq = q4[r4];
            const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              S[r4 * 4 + c] = fmaf(a, S[r4 * 4 + c], kv[c] * bv);
              nn[r4 * 4 + c] = fmaf(a, nn[r4 * 4 + c], bw * kv[c]);
              num = fmaf(S[r4 * 4 + c], qv[c], num);
              nq = fmaf(nn[r4 * 4 + c], qv[c], nq);
            }
          }
#pragma unroll
          for (int o2 = 1; o2 < L; o2 <<= 1) {
            num += __shfl_xor_sync(0xffffffffu, num, o2);
            nq += __shfl_xor_sync(0xffffffffu, nq, o2);
          }
          o = __fdividef(num, fmaxf(fabsf(nq), sc[tt * 4 + 2]) + 1e-6f);
        }
      } else {
        const float4* g4 = reinterpret_cast<const float4*>(sg + tt * LN + lane4 * NR);
        float kr[NR];
        float dot = 0.0f;
#pragma unroll
        for (int r4 = 0; r4 < NR / 4; ++r4) {
          const float4 gg = g4[r4], kk = k4[r4];
          const float gv[4] = {gg.x, gg.y, gg.z, gg.w}, kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            kr[r4 * 4 + c] = kv[c];
            S[r4 * 4 + c] *= gv[c];
            dot = fmaf(S[r4 * 4 + c], kv[c], dot);
          }
        }
#pragma unroll
        for (int o2 = 1; o2 < L; o2 <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o2);
        const float u = sc[tt * 4 + 3] * (vj - dot);
        float num = 0.0f;
#pragma unroll
        for (int r4 = 0; r4 < NR / 4; ++r4) {
          const float4 qq = q4[r4];
          const float qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            S[r4 * 4 + c] = fmaf(kr[r4 * 4 + c], u, S[r4 * 4 + c]);
            num = fmaf(S[r4 * 4 + c], qv[c], num);
          }
        }
#pragma unroll
        for (int o2 = 1; o2 < L; o2 <<= 1) num += __shfl_xor_sync(0xffffffffu, num, o2);
        o = num;
      }
      if (col_ok && lane4 == 0 && phase != 1) g.out[(int64_t)(c0 + tt) * g.H * dv + (int64_t)h * dv + j] = o;
    }
    __syncthreads();                                   // the chunk's vectors are free for the next one
  }
  if (phase == 1) {                                  // the piece's summary
    float* sm_c = g.sums + (((int64_t)row * g.pieces + piece) * g.H + h) * rec;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int i = lane4 * NR + r;
      if (col_ok && i < dk) sm_c[(int64_t)j * dk + i] = S[r];
      if (MODE == 0 && blockIdx.z == 0 && col == 0 && i < dk) sm_c[dv * dk + i] = nn[r];
    }
    if (MODE == 0 && blockIdx.z == 0 && threadIdx.x == 0) sm_c[dv * dk + dk] = decay;
    return;
  }
  if (phase == 2 && t1 < row_end) return;            // only a row's last piece holds the row's last state
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int i = lane4 * NR + r;
    if (col_ok && i < dk) Sp[(int64_t)j * dk + i] = S[r];
    // the normaliser and the maximum are the same in every block of a head: the first block's first column writes them
    if (MODE == 0 && blockIdx.z == 0 && col == 0 && i < dk)
      g.n_state[((int64_t)slot * g.H + h) * dk + i] = nn[r];
  }
  if (MODE == 0 && phase == 0 && blockIdx.z == 0 && threadIdx.x == 0) g.m_state[(int64_t)slot * g.H + h] = m_run;
}

// The gates of a row's tokens in order: per (row, head) a block that takes 128 tokens at a time (their caps, logsigmoid
// and exponentials side by side, the running maximum in order) and leaves a, b, exp(-m') per token; the head's maximum
// after the row goes back to the state.
__global__ void __launch_bounds__(128) mlstm_gates_kernel(MatrixMemoryArgs g, float* __restrict__ pre) {
  __shared__ float sgate[256];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, h = blockIdx.y;
  const int t0 = __ldcg(g.row_start + row), t1 = __ldcg(g.row_start + row + 1);
  if (t0 >= t1) return;
  const int slot = __ldcg(g.slot_ids + row);
  float m = g.m_state[(int64_t)slot * g.H + h];
  for (int p0 = t0; p0 < t1; p0 += 128) {
    const int n = min(128, t1 - p0);
    if (threadIdx.x < n) {
      const int64_t t = p0 + threadIdx.x;
      const float zi = mm_load(g.zi, g.gate_dtype, t * g.ld_gate + h), zf = mm_load(g.zf, g.gate_dtype, t * g.ld_gate + h);
      sgate[2 * threadIdx.x] = g.cap * tanhf(zi / g.cap);
      sgate[2 * threadIdx.x + 1] = mm_logsigmoid(g.cap * tanhf(zf / g.cap));
    }
    __syncthreads();
    float m_before = m, m_after = m;
    for (int tt = 0; tt < n; ++tt) {
      const float mn = fmaxf(sgate[2 * tt + 1] + m, sgate[2 * tt]);
      if (tt == (int)threadIdx.x) { m_before = m; m_after = mn; }
      m = mn;
    }
    if (threadIdx.x < n) {
      const float gi = sgate[2 * threadIdx.x], gf = sgate[2 * threadIdx.x + 1];
      reinterpret_cast<float4*>(pre)[(int64_t)(p0 + threadIdx.x) * g.H + h] =
          make_float4(expf(gf + m_before - m_after), expf(gi - m_after), expf(-m_after), 0.0f);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) g.m_state[(int64_t)slot * g.H + h] = m;
}

// Between the two walks: per element of S and n, through a row's pieces in order, s <- A s + (the piece's end from
// zero), left in the piece's summary: the state after that piece, which is the next piece's start.
__global__ void __launch_bounds__(256) mlstm_fold_kernel(MatrixMemoryArgs g) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, h = blockIdx.y;
  const int width = g.dv * g.dk + g.dk, rec = width + 1;
  const int e = blockIdx.z * 256 + threadIdx.x;
  const int n = __ldcg(g.row_start + row + 1) - __ldcg(g.row_start + row);
  const int summaries = (n + g.piece_len - 1) / g.piece_len - 1;        // every piece of the row but its last has one
  if (e >= width || summaries < 1) return;
  float s = __ldcg(g.init + ((int64_t)row * g.H + h) * width + e);
  float* base = g.sums + ((int64_t)row * g.pieces * g.H + h) * rec;
  const int64_t step = (int64_t)g.H * rec;
  for (int c0 = 0; c0 < summaries; c0 += 4) {
    float A[4], v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (c0 + u < summaries) {
        A[u] = __ldcg(base + (c0 + u) * step + width);
        v[u] = __ldcg(base + (c0 + u) * step + e);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (c0 + u < summaries) {
        s = fmaf(A[u], s, v[u]);
        base[(c0 + u) * step + e] = s;
      }
    }
  }
}

// The delta rule's fold: a piece multiplies the state it finds by a matrix T [dk x dk] and adds its own end from zero,
// S <- T S + B.  A block takes four columns of a (row, head)'s state through the row's pieces in order (a column in
// shared memory, a thread an element: dk multiply-adds a piece) and leaves the state after every piece in the piece's
// summary, where the next piece starts.
constexpr int DF_COLS = 4;
__global__ void __launch_bounds__(1024) delta_fold_kernel(MatrixMemoryArgs g) {
  extern __shared__ float scol[];                    // [DF_COLS][dk]
  pdl_wait();
  pdl_trigger();
  const int dk = g.dk, dv = g.dv;
  const int row = blockIdx.x, h = blockIdx.y;
  const int jl = threadIdx.x / dk, i = threadIdx.x - jl * dk;
  const int j = blockIdx.z * DF_COLS + jl;
  const int n = __ldcg(g.row_start + row + 1) - __ldcg(g.row_start + row);
  const int summaries = (n + g.piece_len - 1) / g.piece_len - 1;
  if (summaries < 1) return;
  const bool ok = jl < DF_COLS && j < dv;
  const int rec = (dv + dk) * dk;
  float s = ok ? __ldcg(g.init + ((int64_t)row * g.H + h) * dv * dk + (int64_t)j * dk + i) : 0.0f;
  for (int c = 0; c < summaries; ++c) {
    float* sm_c = g.sums + (((int64_t)row * g.pieces + c) * g.H + h) * rec;
    if (ok) scol[jl * dk + i] = s;
    __syncthreads();
    if (ok) {
      const float* T = sm_c + (int64_t)dv * dk;      // column m of the matrix at T + m dk
      float a0 = __ldcg(sm_c + (int64_t)j * dk + i), a1 = 0.0f;
      int m = 0;
      for (; m + 16 <= dk; m += 16) {                // sixteen of the matrix's elements in flight before the first is used
        float tv[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) tv[u] = __ldcg(T + (int64_t)(m + u) * dk + i);
#pragma unroll
        for (int u = 0; u < 16; u += 2) {
          a0 = fmaf(tv[u], scol[jl * dk + m + u], a0);
          a1 = fmaf(tv[u + 1], scol[jl * dk + m + u + 1], a1);
        }
      }
      for (; m < dk; ++m) a0 = fmaf(__ldcg(T + (int64_t)m * dk + i), scol[jl * dk + m], a0);
      s = a0 + a1;
    }
    __syncthreads();                                 // everyone has read the matrix's rows and the old column
    if (ok) sm_c[(int64_t)j * dk + i] = s;
  }
}

template <int MODE, int L, int NR>
static int mm_launch_nr(const MatrixMemoryArgs& g, dim3 grid, int max_new, cudaStream_t stream) {
  // tokens staged at once: as many as a row brings, up to MM_CHUNK (at most as many as the block has threads) and to
  // what fits 96 KB of shared memory
  const size_t per_token = (size_t)((MODE == 1 ? 3 : 2) * L * NR + MM_COLS + 6) * sizeof(float);
  const int chunk = max(1, min(min(max_new, MM_CHUNK), (int)(96 * 1024 / per_token)));
  const size_t smem = (size_t)chunk * per_token;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(matrix_memory_kernel<MODE, L, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("matrix_memory: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e)); return (int)e; }
  }
  launch_pdl(matrix_memory_kernel<MODE, L, NR>, grid, dim3(L * MM_COLS), smem, stream, g, chunk);
  return launch_status("matrix_memory");
}

template <int MODE>
static int mm_launch(const MatrixMemoryArgs& g, int rows, int max_new, cudaStream_t stream) {
  const dim3 grid(g.phase ? rows * g.pieces : rows, g.H, ceil_div(g.dv + (MODE == 1 && g.phase == 1 ? g.dk : 0), MM_COLS));
  if (g.phase) max_new = g.piece_len;
  // Eight lanes a column from keys of 32 features on: twice the warps of four lanes a column to hide each other's
  // waits, half the rows a lane walks for every token.  (Sixteen lanes a column were measured and lose: what a token
  // costs a warp beyond its rows, the sums across lanes, the division, the store, is then paid by twice the warps, and
  // the kernel is bound by the instructions it issues.)
  if (g.dk < 32) return mm_launch_nr<MODE, 4, 8>(g, grid, max_new, stream);
  if (g.phase && g.dk <= 128) {
    // pieces side by side fill the SMs with blocks: four lanes a column then cost the fewest instructions a column
    const int nr4 = ceil_div(g.dk, 4);
    if (nr4 <= 16) return mm_launch_nr<MODE, 4, 16>(g, grid, max_new, stream);
    return mm_launch_nr<MODE, 4, 32>(g, grid, max_new, stream);
  }
  const int nr = ceil_div(g.dk, 8);
  if (nr <= 4) return mm_launch_nr<MODE, 8, 4>(g, grid, max_new, stream);
  if (nr <= 8) return mm_launch_nr<MODE, 8, 8>(g, grid, max_new, stream);
  if (nr <= 16) return mm_launch_nr<MODE, 8, 16>(g, grid, max_new, stream);
  if (nr <= 32) return mm_launch_nr<MODE, 8, 32>(g, grid, max_new, stream);
  set_error("matrix_memory: keys of %d features are too wide (at most 256)", g.dk);
  return ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------------------------

struct ConvPrepArgs {
  const void* x; int x_dtype; int64_t ldx;           // [T, *]: q heads at off[0], k heads at off[1], v heads at off[2]
  int off[3];
  const float* taps[3];                              // [channels of the section, taps]
  int heads[3], dim[3];                              // heads and channels a head of each section
  int n_taps;
  float eps, q_scale;
  float* state;                                      // [slots, channels, taps - 1], oldest first
  const int* slot_ids; const int* row_start;
  float* out;                                        // [T, channels]: q | k | v
  int channels, chunks, chunk_tokens;
};

__global__ void __launch_bounds__(CONV_WARPS * 32) conv_prep_kernel(ConvPrepArgs g) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int unit = blockIdx.y * CONV_WARPS + warp;
  const int units = g.heads[0] + g.heads[1] + g.heads[2];
  if (unit >= units) return;
  const int sec = unit < g.heads[0] ? 0 : (unit < g.heads[0] + g.heads[1] ? 1 : 2);
  const int head = unit - (sec == 0 ? 0 : (sec == 1 ? g.heads[0] : g.heads[0] + g.heads[1]));
  const int d = g.dim[sec];
  const int c_sec = head * d;                                                // first channel within the section
  const int c_out = (sec == 0 ? 0 : (sec == 1 ? g.heads[0] * g.dim[0] : g.heads[0] * g.dim[0] + g.heads[1] * g.dim[1])) + c_sec;
  const int row = blockIdx.x / g.chunks, chunk = blockIdx.x - row * g.chunks;
  const int t0 = __ldcg(g.row_start + row), t1 = __ldcg(g.row_start + row + 1);
  const int first = t0 + chunk * g.chunk_tokens;
  if (first >= t1) return;
  const int last = min(t1, first + g.chunk_tokens);
  const int nt = g.n_taps;
  const int slot = __ldcg(g.slot_ids + row);
  const float* st = g.state + ((int64_t)slot * g.channels + c_out) * (nt - 1);
  const float* w = g.taps[sec] + (int64_t)c_sec * nt;
  const int64_t xcol = g.off[sec] + c_sec;
  for (int t = first; t < last; ++t) {
    float y[CONV_MAX_PER_LANE];
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < CONV_MAX_PER_LANE; ++e) {
      const int c = e * 32 + lane;
      y[e] = 0.0f;
      if (c < d) {
        float a = 0.0f;
        for (int jj = nt - 1; jj >= 0; --jj) {                                // oldest input first
          const int ts = t - jj;
          const float xv = ts >= t0 ? mm_load(g.x, g.x_dtype, (int64_t)ts * g.ldx + xcol + c)
                                    : __ldcg(st + (int64_t)c * (nt - 1) + (nt - 1) + (ts - t0));
          a = fmaf(__ldg(w + (int64_t)c * nt + (nt - 1 - jj)), xv, a);
        }
        y[e] = a / (1.0f + expf(-a));
        ss = fmaf(y[e], y[e], ss);
      }
    }
    float mul = 1.0f;
    if (sec < 2) {
      ss = warp_sum(ss);
      mul = rsqrtf(ss + g.eps) * (sec == 0 ? g.q_scale : 1.0f);
    }
#pragma unroll
    for (int e = 0; e < CONV_MAX_PER_LANE; ++e) {
      const int c = e * 32 + lane;
      if (c < d) g.out[(int64_t)t * g.channels + c_out + c] = y[e] * mul;
    }
  }
  if (chunk != 0 || nt < 2) return;
  // The row's first chunk is the only reader of the state (a chunk is longer than the taps reach back) and, after
  // its reads, the writer of the new one: the last taps - 1 inputs of the old state followed by the row's tokens.
  __syncwarp();
  const int n_new = t1 - t0;
#pragma unroll
  for (int e = 0; e < CONV_MAX_PER_LANE; ++e) {
    const int c = e * 32 + lane;
    if (c >= d) continue;
    float keep[CONV_MAX_TAPS - 1];
#pragma unroll
    for (int s = 0; s < CONV_MAX_TAPS - 1; ++s) {
      keep[s] = 0.0f;
      if (s < nt - 1) {
        const int i = n_new - (nt - 1) + s;                                   // place among the row's tokens of this step
        keep[s] = i >= 0 ? mm_load(g.x, g.x_dtype, (int64_t)(t0 + i) * g.ldx + xcol + c)
                         : __ldcg(st + (int64_t)c * (nt - 1) + (nt - 1) + i);
      }
    }
    float* sw = g.state + ((int64_t)slot * g.channels + c_out + c) * (nt - 1);
#pragma unroll
    for (int s = 0; s < CONV_MAX_TAPS - 1; ++s)
      if (s < nt - 1) sw[s] = keep[s];
  }
}

}  // namespace exl3

using namespace exl3;

static bool mm_dtype_ok(int d) { return d == DT_F32 || d == DT_BF16; }

// Rows of at least MLSTM_MIN_PIECED tokens run as pieces side by side: pieces of a multiple of 64 tokens, about 64 of
// them over the step's rows.  Returns the bytes of scratch that takes (0: the rows run whole, in order).
constexpr int MLSTM_MIN_PIECED = 256;
static size_t mlstm_pieces(int rows, int T, int heads, int dk, int dv, int max_new, int* piece_len, int* pieces) {
  if (max_new < MLSTM_MIN_PIECED) return 0;
  const int len = 64 * exl3::ceil_div(exl3::ceil_div(T, 64), 64);       // about 64 pieces in all, whole sixty-fours
  *piece_len = len < 64 ? 64 : len;
  *pieces = exl3::ceil_div(max_new, *piece_len);
  const size_t rec = (size_t)dv * dk + dk + 1;
  return ((size_t)T * heads * 4 + (size_t)rows * heads * ((size_t)dv * dk + dk) + (size_t)rows * *pieces * heads * rec) * sizeof(float);
}

// The same for the delta rule, whose pieces' summaries also hold the piece's matrix (dk more columns); keys of up to 256
// features (the fold's block is four columns of dk threads).
static size_t delta_pieces(int rows, int T, int heads, int dk, int dv, int max_new, int* piece_len, int* pieces) {
  if (max_new < MLSTM_MIN_PIECED || dk > 256) return 0;
  // The pieces cost the walk in order two and a half times over (dk more columns for the matrices, the fold, the second
  // walk), so they pay only while the walk in order would leave most of the GPU idle: measured even at 64 blocks in
  // order (16 heads of 128 values: 0.91 against 1.01 ms for 2,048 tokens), behind at 128 (32 heads).
  if ((int64_t)rows * heads * exl3::ceil_div(dv, exl3::MM_COLS) > 64) return 0;
  const int len = 64 * exl3::ceil_div(exl3::ceil_div(T, 64), 64);
  *piece_len = len < 64 ? 64 : len;
  *pieces = exl3::ceil_div(max_new, *piece_len);
  return ((size_t)rows * heads * dv * dk + (size_t)rows * *pieces * heads * ((size_t)dv + dk) * dk) * sizeof(float);
}

extern "C" size_t exl3_delta_scan_scratch_bytes(int rows, int T, int heads, int dk, int dv, int max_new) {
  int a = 0, b = 0;
  return delta_pieces(rows, T, heads, dk, dv, max_new, &a, &b);
}

extern "C" size_t exl3_mlstm_scan_scratch_bytes(int rows, int T, int heads, int dk, int dv, int max_new) {
  int a = 0, b = 0;
  return mlstm_pieces(rows, T, heads, dk, dv, max_new, &a, &b);
}
// whether groups of four elements from p on can be read at once (16 bytes of float32, 8 of bfloat16)
static bool mm_aligned(const void* p, int dtype) { return (reinterpret_cast<uintptr_t>(p) & (dtype == DT_F32 ? 15u : 7u)) == 0; }

extern "C" int exl3_mlstm_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                               int qkv_dtype, const void* zi, const void* zf, int gate_dtype, int64_t ld_gate, float cap,
                               float q_scale, float* s_state, float* n_state, float* m_state, const int* slot_ids,
                               const int* row_start, float* out, int rows, int T, int heads, int dk, int dv,
                               int max_new, float* scratch, size_t scratch_bytes, cudaStream_t stream) {
  if (T == 0 || rows == 0) return 0;
  if (T < 0 || rows < 0 || heads < 1 || dk < 1 || dv < 1 || max_new < 1 || !(cap > 0.0f) || !mm_dtype_ok(qkv_dtype) || !mm_dtype_ok(gate_dtype) ||
      heads > 65535 || dv > 65535 * MM_COLS) {
    set_error("mlstm_scan: bad sizes rows=%d T=%d heads=%d dk=%d dv=%d cap=%g", rows, T, heads, dk, dv, (double)cap);
    return ERR_BAD_ARGUMENT;
  }
  MatrixMemoryArgs g = {};
  g.q = q; g.k = k; g.v = v; g.qkv_dtype = qkv_dtype; g.ldq = ldq; g.ldk = ldk; g.ldv = ldv; g.q_scale = q_scale;
  g.zi = zi; g.zf = zf; g.gate_dtype = gate_dtype; g.ld_gate = ld_gate; g.cap = cap;
  g.s_state = s_state; g.n_state = n_state; g.m_state = m_state; g.slot_ids = slot_ids; g.row_start = row_start;
  g.out = out; g.H = heads; g.QH = heads; g.dk = dk; g.dv = dv;
  g.vec = dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && mm_aligned(q, qkv_dtype) && mm_aligned(k, qkv_dtype);
  int piece_len = 0, pieces = 0;
  const size_t need = mlstm_pieces(rows, T, heads, dk, dv, max_new, &piece_len, &pieces);
  if (need == 0) return mm_launch<0>(g, rows, max_new, stream);
  if (scratch == nullptr || scratch_bytes < need || !aligned16(scratch)) {
    set_error("mlstm_scan: rows of up to %d tokens need %zu bytes of 16-byte aligned scratch, got %zu", max_new, need, scratch_bytes);
    return ERR_SCRATCH;
  }
  float* pre = scratch;
  g.pre = pre;
  g.init = pre + (size_t)T * heads * 4;
  g.sums = g.init + (size_t)rows * heads * ((size_t)dv * dk + dk);
  g.piece_len = piece_len;
  g.pieces = pieces;
  launch_pdl(mlstm_gates_kernel, dim3(rows, heads), dim3(128), 0, stream, g, pre);
  int rc = launch_status("mlstm_gates");
  if (rc) return rc;
  g.phase = 1;
  rc = mm_launch<0>(g, rows, max_new, stream);
  if (rc) return rc;
  launch_pdl(mlstm_fold_kernel, dim3(rows, heads, ceil_div(dv * dk + dk, 256)), dim3(256), 0, stream, g);
  rc = launch_status("mlstm_fold");
  if (rc) return rc;
  g.phase = 2;
  return mm_launch<0>(g, rows, max_new, stream);
}

extern "C" int exl3_delta_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                               int qkv_dtype, const void* zb, int zb_dtype, int64_t ld_zb, const void* za, int za_dtype,
                               int64_t ld_za, const float* a_log, const float* dt_bias, float* s_state,
                               const int* slot_ids, const int* row_start, float* out, int rows, int T, int heads,
                               int qk_heads, int dk, int dv, int max_new, float* scratch, size_t scratch_bytes,
                               cudaStream_t stream) {
  if (T == 0 || rows == 0) return 0;
  if (T < 0 || rows < 0 || max_new < 1 || heads < 1 || qk_heads < 1 || heads % qk_heads != 0 || dk < 1 || dv < 1 || !mm_dtype_ok(qkv_dtype) ||
      !mm_dtype_ok(zb_dtype) || !mm_dtype_ok(za_dtype) || heads > 65535 || dv > 65535 * MM_COLS) {
    set_error("delta_scan: bad sizes rows=%d T=%d heads=%d on %d dk=%d dv=%d", rows, T, heads, qk_heads, dk, dv);
    return ERR_BAD_ARGUMENT;
  }
  MatrixMemoryArgs g = {};
  g.q = q; g.k = k; g.v = v; g.qkv_dtype = qkv_dtype; g.ldq = ldq; g.ldk = ldk; g.ldv = ldv; g.q_scale = 1.0f;
  g.zb = zb; g.zb_dtype = zb_dtype; g.ld_zb = ld_zb; g.za = za; g.za_dtype = za_dtype; g.ld_za = ld_za;
  g.a_log = a_log; g.dt_bias = dt_bias; g.s_state = s_state; g.slot_ids = slot_ids; g.row_start = row_start;
  g.out = out; g.H = heads; g.QH = qk_heads; g.dk = dk; g.dv = dv;
  g.vec = dk % 4 == 0 && ldq % 4 == 0 && ldk % 4 == 0 && ld_za % 4 == 0 && mm_aligned(q, qkv_dtype) &&
          mm_aligned(k, qkv_dtype) && mm_aligned(za, za_dtype);
  int piece_len = 0, pieces = 0;
  const size_t need = delta_pieces(rows, T, heads, dk, dv, max_new, &piece_len, &pieces);
  if (need == 0) return mm_launch<1>(g, rows, max_new, stream);
  if (scratch == nullptr || scratch_bytes < need || !aligned16(scratch)) {
    set_error("delta_scan: rows of up to %d tokens need %zu bytes of 16-byte aligned scratch, got %zu", max_new, need, scratch_bytes);
    return ERR_SCRATCH;
  }
  g.init = scratch;
  g.sums = g.init + (size_t)rows * heads * dv * dk;
  g.piece_len = piece_len;
  g.pieces = pieces;
  g.phase = 1;
  int rc = mm_launch<1>(g, rows, max_new, stream);
  if (rc) return rc;
  launch_pdl(delta_fold_kernel, dim3(rows, heads, ceil_div(dv, DF_COLS)), dim3(DF_COLS * dk), (size_t)DF_COLS * dk * sizeof(float),
             stream, g);
  rc = launch_status("delta_fold");
  if (rc) return rc;
  g.phase = 2;
  return mm_launch<1>(g, rows, max_new, stream);
}

extern "C" int exl3_conv_prep_max_taps() { return CONV_MAX_TAPS; }

extern "C" int exl3_conv_prep(const void* x, int x_dtype, int64_t ldx, int q_off, int k_off, int v_off,
                              const float* q_taps, const float* k_taps, const float* v_taps, int qk_heads, int dk,
                              int v_heads, int dv, int n_taps, float eps, float q_scale, float* state,
                              const int* slot_ids, const int* row_start, float* out, int rows, int T, int max_new,
                              cudaStream_t stream) {
  if (T == 0 || rows == 0) return 0;
  if (T < 0 || rows < 0 || qk_heads < 1 || v_heads < 1 || dk < 1 || dv < 1 || dk > 32 * CONV_MAX_PER_LANE ||
      dv > 32 * CONV_MAX_PER_LANE || n_taps < 1 || n_taps > CONV_MAX_TAPS || max_new < 1 || !mm_dtype_ok(x_dtype)) {
    set_error("conv_prep: bad sizes rows=%d T=%d heads=%d/%d of %d/%d (at most %d) taps=%d (at most %d)", rows, T, qk_heads,
              v_heads, dk, dv, 32 * CONV_MAX_PER_LANE, n_taps, CONV_MAX_TAPS);
    return ERR_BAD_ARGUMENT;
  }
  ConvPrepArgs g = {};
  g.x = x; g.x_dtype = x_dtype; g.ldx = ldx;
  g.off[0] = q_off; g.off[1] = k_off; g.off[2] = v_off;
  g.taps[0] = q_taps; g.taps[1] = k_taps; g.taps[2] = v_taps;
  g.heads[0] = qk_heads; g.heads[1] = qk_heads; g.heads[2] = v_heads;
  g.dim[0] = dk; g.dim[1] = dk; g.dim[2] = dv;
  g.n_taps = n_taps; g.eps = eps; g.q_scale = q_scale; g.state = state; g.slot_ids = slot_ids; g.row_start = row_start;
  g.out = out; g.channels = 2 * qk_heads * dk + v_heads * dv;
  // tokens a warp walks: few, so that many warps hide each other's loads, but at least as many as the taps reach back
  // (then only a row's first chunk reads the kept inputs)
  g.chunk_tokens = max(CONV_MIN_CHUNK, n_taps - 1);
  g.chunks = ceil_div(max_new, g.chunk_tokens);
  const int units = 2 * qk_heads + v_heads;
  const int64_t bx = (int64_t)rows * g.chunks;
  if (bx > 0x7fffffffLL || ceil_div(units, CONV_WARPS) > 65535) { set_error("conv_prep: grid too large"); return ERR_UNSUPPORTED; }
  launch_pdl(conv_prep_kernel, dim3((unsigned)bx, ceil_div(units, CONV_WARPS)), dim3(CONV_WARPS * 32), 0, stream, g);
  return launch_status("conv_prep");
}
