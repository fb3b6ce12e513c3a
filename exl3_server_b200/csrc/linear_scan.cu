// Linear recurrences with a matrix state per head, and what stands around them.
//
// State S [dk, dv] per (sequence, head), float32, kept in the cache's per-sequence state between steps.
//
//   mode 0, a decay per token and key channel and a bonus for the current token:
//       o_t = S^T r_t + (sum_i r_ti u_i k_ti) v_t
//       S  <- diag(w_t) S + k_t v_t^T,        w_t = exp(-exp(wraw_t + w0))
//   mode 1, one decay per head (retention):
//       S  <- decay_h S + k_t v_t^T
//       o_t = S^T r_t
//
// A block owns one (row of the batch, head): thread j keeps column j of S in shared memory and walks the row's tokens
// in order; r, k and the decays of eight tokens at a time are staged in shared memory.  The state is read from and
// written back to the row's slot, so a sequence cut into steps in any way walks the same chain of sums.
//
// Rows that bring many tokens are cut into chunks of LS_CHUNK tokens that run side by side, as the element-wise
// recurrence of recurrent.cu does: over a chunk S_out = diag(A) S_in + B with A the product of the chunk's decays
// and B the chunk's own scan from zero.  A first launch leaves (A, B) per chunk, a second folds the (A, B) of the
// chunks before its own, in order, into its start and walks its chunk.  That changes roundings only.  The row's last
// chunk leaves the new state in the slot while the others may still be starting, so the first launch also copies the
// state of every row that has more than one chunk into the scratch, and the second launch starts from that copy.
//
// Everything but the element types of r, k, v (a projection's output) is float32.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float ls_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ inline float ls_load_act(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
// what the projections' outputs go through before they enter the recurrence: 0 nothing, 1 silu
__device__ inline float ls_in(float x, int act) { return act == 1 ? x / (1.0f + expf(-x)) : x; }
__device__ inline void ls_store(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// ---- token shift ---------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
token_shift_kernel(const void* h, int h_dtype, const void* __restrict__ mu, int mu_dtype, int n_mix, float* prev,
                   const int* __restrict__ tok_seq, const int* __restrict__ row_start,
                   const int* __restrict__ slot_ids, void* out, int out_dtype, int T, int H) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int b = __ldcg(tok_seq + t);
  const int first = __ldcg(row_start + b), end = __ldcg(row_start + b + 1);
  float* st = prev + (int64_t)__ldcg(slot_ids + b) * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float x = ls_load_act(h, h_dtype, (int64_t)t * H + c);
    float before;
    if (t == first) {
      // the same thread reads the entry and then leaves the row's last h of this step in it
      before = __ldcg(st + c);
      st[c] = ls_load_act(h, h_dtype, (int64_t)(end - 1) * H + c);
    } else {
      before = ls_load_act(h, h_dtype, (int64_t)(t - 1) * H + c);
    }
    const float d = before - x;
    for (int s = 0; s < n_mix; ++s)
      ls_store(out, out_dtype, ((int64_t)s * T + t) * H + c, fmaf(d, ls_load(mu, mu_dtype, (int64_t)s * H + c), x));
  }
}

// Eight consecutive values as floats from float32 or bfloat16 storage, through L2; and back.
__device__ inline void ls_load8(const float* p, float (&v)[8]) {
  float a[4], b[4];
  load_vec_cg(p, a);
  load_vec_cg(p + 4, b);
#pragma unroll
  for (int e = 0; e < 4; ++e) { v[e] = a[e]; v[4 + e] = b[e]; }
}
__device__ inline void ls_load8(const __nv_bfloat16* p, float (&v)[8]) { load_vec_cg(p, v); }
__device__ inline void ls_store8(float* p, const float (&v)[8]) {
  const float a[4] = {v[0], v[1], v[2], v[3]}, b[4] = {v[4], v[5], v[6], v[7]};
  store_vec(p, a);
  store_vec(p + 4, b);
}
__device__ inline void ls_store8(__nv_bfloat16* p, const float (&v)[8]) { store_vec(p, v); }

// Token shift with eight features a thread (H a multiple of 8, float32 mu).
template <typename TH, typename TO>
__global__ void __launch_bounds__(256)
token_shift_vec_kernel(const TH* h, const float* __restrict__ mu, int n_mix, float* prev, const int* __restrict__ tok_seq,
                       const int* __restrict__ row_start, const int* __restrict__ slot_ids, TO* out, int T, int H) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int b = __ldcg(tok_seq + t);
  const int first = __ldcg(row_start + b), end = __ldcg(row_start + b + 1);
  float* st = prev + (int64_t)__ldcg(slot_ids + b) * H;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float x[8], before[8];
    ls_load8(h + (int64_t)t * H + c, x);
    if (t == first) {
      float last[8];
      ls_load8(st + c, before);
      ls_load8(h + (int64_t)(end - 1) * H + c, last);
      ls_store8(st + c, last);
    } else {
      ls_load8(h + (int64_t)(t - 1) * H + c, before);
    }
    for (int s = 0; s < n_mix; ++s) {
      float m[8], o[8];
      load_vec(mu + (int64_t)s * H + c, reinterpret_cast<float(&)[4]>(m[0]));
      load_vec(mu + (int64_t)s * H + c + 4, reinterpret_cast<float(&)[4]>(m[4]));
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = fmaf(before[e] - x[e], m[e], x[e]);
      ls_store8(out + ((int64_t)s * T + t) * H + c, o);
    }
  }
}

// ---- the scan ------------------------------------------------------------------------------------------------------

constexpr int LS_STAGE = 8;                      // tokens staged in shared memory at a time
constexpr int LS_CHUNK = 64;                     // tokens of a chunk when a row's tokens run side by side

struct ScanArgs {
  const void* r; int64_t r_ld; const void* k; int64_t k_ld; int rk_dtype;
  const void* v; int64_t v_ld; int v_dtype;
  const void* wraw; int64_t w_ld; int w_dtype;
  const void* w0; const void* u; int wu_dtype;
  const float* decay;
  float* state; const int* slot_ids; const int* row_start;
  float* out; float* ab; float* snap;
  int heads, dk, dv, places;
  int act;                                       // see ls_in
};

// Chunk j of batch row b has a place of its own among floor(T / LS_CHUNK) + B + 1 places.
__device__ inline int ls_place(int t0, int b, int j) { return t0 / LS_CHUNK + b + j; }

// phase 0: a row's tokens of the step, from its state, state written back.
// phase 1: a chunk from zero, (A, B) to scratch (no output; the row's last chunk does nothing).
// phase 2: the chunks before folded into the state, then the chunk; the row's last chunk writes the state.
template <int MODE>
__global__ void linear_scan_kernel(ScanArgs a, int phase) {
  extern __shared__ float ls_sm[];
  const int dk = a.dk, dv = a.dv;
  float* S = ls_sm;                              // [dk][dv]
  float* sr = S + dk * dv;                       // [LS_STAGE][dk]
  float* sk = sr + LS_STAGE * dk;                // [LS_STAGE][dk]
  float* sw = sk + LS_STAGE * dk;                // [LS_STAGE][dk] decays (mode 0)
  float* sb = sw + LS_STAGE * dk;                // [LS_STAGE] bonus factors (mode 0)
  float* sA = sb + LS_STAGE;                     // [dk] product of decays (phase 1)
  pdl_wait();
  pdl_trigger();
  const int hd = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int t0 = __ldcg(a.row_start + b), t1 = __ldcg(a.row_start + b + 1);
  int lo = t0, hi = t1;
  if (phase == 1) {
    lo = t0 + c * LS_CHUNK;
    hi = lo + LS_CHUNK;
    if (hi >= t1) return;                        // the row's last chunk has nobody after it
  } else if (phase == 2) {
    lo = t0 + c * LS_CHUNK;
    hi = min(lo + LS_CHUNK, t1);
    if (lo >= t1) return;
  }
  const int j = threadIdx.x;
  const bool col = j < dv;
  float* st = a.state + ((int64_t)__ldcg(a.slot_ids + b) * a.heads + hd) * dk * dv;
  const int64_t rec = (int64_t)dk + (int64_t)dk * dv;      // floats of one (place, head): A then B
  float* snap = a.snap + ((int64_t)b * a.heads + hd) * dk * dv;
  if (phase == 1) {
    if (col) for (int i = 0; i < dk; ++i) S[i * dv + j] = 0.0f;
    for (int i = j; i < dk; i += blockDim.x) sA[i] = 1.0f;
    if (c == 0 && col) for (int i = 0; i < dk; ++i) snap[i * dv + j] = __ldcg(st + i * dv + j);
  } else {
    // a row of several chunks starts from the copy that the first launch took
    const float* from = (phase == 2 && t1 - t0 > LS_CHUNK) ? snap : st;
    if (col) for (int i = 0; i < dk; ++i) S[i * dv + j] = __ldcg(from + i * dv + j);
    if (phase == 2 && col) {
      for (int p = 0; p < c; ++p) {              // the chunks before this one, in order
        const float* ab = a.ab + ((int64_t)ls_place(t0, b, p) * a.heads + hd) * rec;
        for (int i = 0; i < dk; ++i) S[i * dv + j] = fmaf(__ldcg(ab + i), S[i * dv + j], __ldcg(ab + dk + i * dv + j));
      }
    }
  }
  const float gamma = MODE == 1 ? a.decay[hd] : 0.0f;
  for (int s0 = lo; s0 < hi; s0 += LS_STAGE) {
    const int n = min(LS_STAGE, hi - s0);
    __syncthreads();                             // the stage before has been used
    for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
      const int tt = idx / dk, i = idx - tt * dk;
      const int64_t t = s0 + tt;
      sr[idx] = ls_in(ls_load_act(a.r, a.rk_dtype, t * a.r_ld + (int64_t)hd * dk + i), a.act);
      sk[idx] = ls_in(ls_load_act(a.k, a.rk_dtype, t * a.k_ld + (int64_t)hd * dk + i), a.act);
      if (MODE == 0) {
        const float z = ls_load_act(a.wraw, a.w_dtype, t * a.w_ld + (int64_t)hd * dk + i) +
                        ls_load(a.w0, a.wu_dtype, (int64_t)hd * dk + i);
        sw[idx] = expf(-expf(z));
      }
    }
    __syncthreads();
    if (MODE == 0) {
      // the bonus factor sum_i r_i u_i k_i of each staged token, a warp a token
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
      for (int tt = warp; tt < n; tt += nw) {
        float acc = 0.0f;
        for (int i = lane; i < dk; i += 32)
          acc = fmaf(sr[tt * dk + i] * ls_load(a.u, a.wu_dtype, (int64_t)hd * dk + i), sk[tt * dk + i], acc);
        acc = warp_sum(acc);
        if (lane == 0) sb[tt] = acc;
      }
      if (phase == 1)
        for (int i = threadIdx.x; i < dk; i += blockDim.x) {
          float p = sA[i];
          for (int tt = 0; tt < n; ++tt) p *= sw[tt * dk + i];
          sA[i] = p;
        }
      __syncthreads();
    } else if (phase == 1) {
      for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        float p = sA[i];
        for (int tt = 0; tt < n; ++tt) p *= gamma;
        sA[i] = p;
      }
    }
    if (col) {
      for (int tt = 0; tt < n; ++tt) {
        const int64_t t = s0 + tt;
        const float vj = ls_in(ls_load_act(a.v, a.v_dtype, t * a.v_ld + (int64_t)hd * dv + j), a.act);
        const float* rr = sr + tt * dk;
        const float* kk = sk + tt * dk;
        float acc = 0.0f;
        if (MODE == 0) {
          const float* ww = sw + tt * dk;
#pragma unroll 4
          for (int i = 0; i < dk; ++i) {
            const float s = S[i * dv + j];
            acc = fmaf(rr[i], s, acc);
            S[i * dv + j] = fmaf(ww[i], s, kk[i] * vj);
          }
          acc = fmaf(sb[tt], vj, acc);
        } else {
#pragma unroll 4
          for (int i = 0; i < dk; ++i) {
            const float s = fmaf(gamma, S[i * dv + j], kk[i] * vj);
            S[i * dv + j] = s;
            acc = fmaf(rr[i], s, acc);
          }
        }
        if (phase != 1) a.out[t * ((int64_t)a.heads * dv) + (int64_t)hd * dv + j] = acc;
      }
    }
  }
  if (phase == 1) {
    __syncthreads();
    float* ab = a.ab + ((int64_t)ls_place(t0, b, c) * a.heads + hd) * rec;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) ab[i] = sA[i];
    if (col) for (int i = 0; i < dk; ++i) ab[dk + i * dv + j] = S[i * dv + j];
  } else if (hi == t1 && col) {
    for (int i = 0; i < dk; ++i) st[i * dv + j] = S[i * dv + j];
  }
}

// The same with the state in registers, for key sizes of 16, 32, 64 and 128 and up to 128 values a head.  A column of
// S is cut over LS_Q threads (a quarter of the key channels each), so a token costs a thread DK / 4 steps of its chain
// instead of DK and a block has four times the warps to hide its loads behind; the four partial sums of an output
// meet in shared memory once per stage of eight tokens.  r, k and the decays are read four at a time.  (With the whole
// state in shared memory a token cost a warp five shared-memory instructions per key channel, which bounded the
// kernel: 8,192 tokens of 32 heads of 64 x 64 took 0.94 ms a launch.)
constexpr int LS_Q = 4;
constexpr int LS_MAX_DV = 128;

template <int MODE, int DK, int PHASE>
__global__ void __launch_bounds__(LS_Q * LS_MAX_DV, DK <= 64 ? 2 : 1) linear_scan_reg_kernel(ScanArgs a, int) {
  constexpr int phase = PHASE;                       // 1 (a chunk's summary) needs neither r nor the outputs
  constexpr int DKQ = DK / LS_Q;
  __shared__ __align__(16) float sr[LS_STAGE * DK];
  __shared__ __align__(16) float sk[LS_STAGE * DK];
  __shared__ __align__(16) float sw[MODE == 0 ? LS_STAGE * DK : 4];
  __shared__ float sb[LS_STAGE];
  __shared__ float sA[DK];
  extern __shared__ float ls_acc[];                  // [LS_STAGE][LS_Q][dvr] partial outputs
  const int dv = a.dv;
  const int dvr = blockDim.x / LS_Q;                 // dv rounded up to whole warps
  pdl_wait();
  pdl_trigger();
  const int hd = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int t0 = __ldcg(a.row_start + b), t1 = __ldcg(a.row_start + b + 1);
  int lo = t0, hi = t1;
  if (phase == 1) {
    lo = t0 + c * LS_CHUNK;
    hi = lo + LS_CHUNK;
    if (hi >= t1) return;
  } else if (phase == 2) {
    lo = t0 + c * LS_CHUNK;
    hi = min(lo + LS_CHUNK, t1);
    if (lo >= t1) return;
  }
  const int q = threadIdx.x / dvr, j = threadIdx.x - q * dvr;
  const bool col = j < dv;
  const int i0 = q * DKQ;                            // this thread's key channels: i0 .. i0 + DKQ - 1
  float* st = a.state + ((int64_t)__ldcg(a.slot_ids + b) * a.heads + hd) * DK * dv;
  const int64_t rec = (int64_t)DK + (int64_t)DK * dv;
  float* snap = a.snap + ((int64_t)b * a.heads + hd) * DK * dv;
  float S[DKQ];
  if (phase == 1) {
#pragma unroll
    for (int i = 0; i < DKQ; ++i) S[i] = 0.0f;
    for (int i = threadIdx.x; i < DK; i += blockDim.x) sA[i] = 1.0f;
    if (c == 0 && col) {
#pragma unroll
      for (int i = 0; i < DKQ; ++i) snap[(i0 + i) * dv + j] = __ldcg(st + (i0 + i) * dv + j);
    }
  } else {
    const float* from = (phase == 2 && t1 - t0 > LS_CHUNK) ? snap : st;
#pragma unroll
    for (int i = 0; i < DKQ; ++i) S[i] = col ? __ldcg(from + (i0 + i) * dv + j) : 0.0f;
    if (phase == 2 && col) {
#pragma unroll 2
      for (int p = 0; p < c; ++p) {                  // the chunks before this one, in order
        const float* ab = a.ab + ((int64_t)ls_place(t0, b, p) * a.heads + hd) * rec;
#pragma unroll
        for (int i = 0; i < DKQ; ++i) S[i] = fmaf(__ldcg(ab + i0 + i), S[i], __ldcg(ab + DK + (i0 + i) * dv + j));
      }
    }
  }
  const float gamma = MODE == 1 ? a.decay[hd] : 0.0f;
  // A stage's r, k and decay inputs come into registers a stage ahead, so that their way from memory passes under the
  // stage before's arithmetic instead of standing in front of the barrier (a block has at least 128 threads, so
  // PER values a thread cover a stage).
  constexpr int PER = LS_STAGE * DK / 128;
  float pr[PER], pk[PER], pw[MODE == 0 ? PER : 1];
  auto fetch = [&](int s0) {
    const int n = min(LS_STAGE, hi - s0);
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = threadIdx.x + e * blockDim.x;
      if (idx < n * DK) {
        const int tt = idx / DK, i = idx - tt * DK;
        const int64_t t = s0 + tt;
        if (phase != 1) pr[e] = ls_load_act(a.r, a.rk_dtype, t * a.r_ld + (int64_t)hd * DK + i);
        pk[e] = ls_load_act(a.k, a.rk_dtype, t * a.k_ld + (int64_t)hd * DK + i);
        if (MODE == 0) pw[e] = ls_load_act(a.wraw, a.w_dtype, t * a.w_ld + (int64_t)hd * DK + i);
      }
    }
  };
  fetch(lo);
  for (int s0 = lo; s0 < hi; s0 += LS_STAGE) {
    const int n = min(LS_STAGE, hi - s0);
    __syncthreads();                                 // the stage before has been used, its outputs written
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = threadIdx.x + e * blockDim.x;
      if (idx < n * DK) {
        if (phase != 1) sr[idx] = ls_in(pr[e], a.act);
        sk[idx] = ls_in(pk[e], a.act);
        if (MODE == 0) sw[idx] = expf(-expf(pw[e] + ls_load(a.w0, a.wu_dtype, (int64_t)hd * DK + idx % DK)));
      }
    }
    // the values of the stage's tokens, asked for before the barrier
    float vj[LS_STAGE];
#pragma unroll
    for (int tt = 0; tt < LS_STAGE; ++tt)
      vj[tt] = (col && tt < n) ? ls_in(ls_load_act(a.v, a.v_dtype, (int64_t)(s0 + tt) * a.v_ld + (int64_t)hd * dv + j), a.act) : 0.0f;
    __syncthreads();
    if (s0 + LS_STAGE < hi) fetch(s0 + LS_STAGE);
    if (MODE == 0) {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
      for (int tt = warp; phase != 1 && tt < n; tt += nw) {
        float acc = 0.0f;
        for (int i = lane; i < DK; i += 32)
          acc = fmaf(sr[tt * DK + i] * ls_load(a.u, a.wu_dtype, (int64_t)hd * DK + i), sk[tt * DK + i], acc);
        acc = warp_sum(acc);
        if (lane == 0) sb[tt] = acc;
      }
      if (phase == 1)
        for (int i = threadIdx.x; i < DK; i += blockDim.x) {
          float p = sA[i];
          for (int tt = 0; tt < n; ++tt) p *= sw[tt * DK + i];
          sA[i] = p;
        }
      __syncthreads();
    } else if (phase == 1) {
      for (int i = threadIdx.x; i < DK; i += blockDim.x) {
        float p = sA[i];
        for (int tt = 0; tt < n; ++tt) p *= gamma;
        sA[i] = p;
      }
    }
#pragma unroll
    for (int tt = 0; tt < LS_STAGE; ++tt) {
      if (tt < n) {
        const float4* rr = reinterpret_cast<const float4*>(sr + tt * DK + i0);
        const float4* kk = reinterpret_cast<const float4*>(sk + tt * DK + i0);
        float acc0 = 0.0f, acc1 = 0.0f;
        if (MODE == 0) {
          const float4* ww = reinterpret_cast<const float4*>(sw + tt * DK + i0);
#pragma unroll
          for (int i4 = 0; i4 < DKQ / 4; ++i4) {
            const float4 r4 = rr[i4], k4 = kk[i4], w4 = ww[i4];
            if (phase != 1) {
              acc0 = fmaf(r4.x, S[4 * i4 + 0], acc0); acc1 = fmaf(r4.y, S[4 * i4 + 1], acc1);
              acc0 = fmaf(r4.z, S[4 * i4 + 2], acc0); acc1 = fmaf(r4.w, S[4 * i4 + 3], acc1);
            }
            S[4 * i4 + 0] = fmaf(w4.x, S[4 * i4 + 0], k4.x * vj[tt]);
            S[4 * i4 + 1] = fmaf(w4.y, S[4 * i4 + 1], k4.y * vj[tt]);
            S[4 * i4 + 2] = fmaf(w4.z, S[4 * i4 + 2], k4.z * vj[tt]);
            S[4 * i4 + 3] = fmaf(w4.w, S[4 * i4 + 3], k4.w * vj[tt]);
          }
          if (q == 0) acc0 = fmaf(sb[tt], vj[tt], acc0);          // the bonus, once
        } else {
#pragma unroll
          for (int i4 = 0; i4 < DKQ / 4; ++i4) {
            const float4 r4 = rr[i4], k4 = kk[i4];
            S[4 * i4 + 0] = fmaf(gamma, S[4 * i4 + 0], k4.x * vj[tt]);
            S[4 * i4 + 1] = fmaf(gamma, S[4 * i4 + 1], k4.y * vj[tt]);
            S[4 * i4 + 2] = fmaf(gamma, S[4 * i4 + 2], k4.z * vj[tt]);
            S[4 * i4 + 3] = fmaf(gamma, S[4 * i4 + 3], k4.w * vj[tt]);
            if (phase != 1) {
              acc0 = fmaf(r4.x, S[4 * i4 + 0], acc0); acc1 = fmaf(r4.y, S[4 * i4 + 1], acc1);
              acc0 = fmaf(r4.z, S[4 * i4 + 2], acc0); acc1 = fmaf(r4.w, S[4 * i4 + 3], acc1);
            }
          }
        }
        if (phase != 1) ls_acc[(tt * LS_Q + q) * dvr + j] = acc0 + acc1;
      }
    }
    if (phase != 1) {
      __syncthreads();
      // the four parts of every output of the stage, summed in the order of the key channels
      for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int tt = idx / dv, jj = idx - tt * dv;
        const float* pa = ls_acc + tt * LS_Q * dvr + jj;
        a.out[(int64_t)(s0 + tt) * ((int64_t)a.heads * dv) + (int64_t)hd * dv + jj] =
            ((pa[0] + pa[dvr]) + pa[2 * dvr]) + pa[3 * dvr];
      }
    }
  }
  if (phase == 1) {
    __syncthreads();
    float* ab = a.ab + ((int64_t)ls_place(t0, b, c) * a.heads + hd) * rec;
    for (int i = threadIdx.x; i < DK; i += blockDim.x) ab[i] = sA[i];
    if (col) {
#pragma unroll
      for (int i = 0; i < DKQ; ++i) ab[DK + (i0 + i) * dv + j] = S[i];
    }
  } else if (hi == t1 && col) {
#pragma unroll
    for (int i = 0; i < DKQ; ++i) st[(i0 + i) * dv + j] = S[i];
  }
}

// ---- per-head norm and gate ------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* o, const void* __restrict__ w, int w_dtype, const void* gate, int gate_dtype,
                      int64_t gate_ld, int gate_kind, float eps, void* out, int out_dtype, int n_items, int heads, int dv) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);       // (token, head)
  if (item >= n_items) return;
  const int t = item / heads, hd = item - t * heads;
  const float* src = o + (int64_t)item * dv;
  float ss = 0.0f;
  for (int e = lane; e < dv; e += 32) {
    const float x = __ldcg(src + e);
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int e = lane; e < dv; e += 32) {
    float x = __ldcg(src + e) * inv;
    if (w) x *= ls_load(w, w_dtype, (int64_t)hd * dv + e);
    if (gate) {
      const float g = ls_load_act(gate, gate_dtype, (int64_t)t * gate_ld + (int64_t)hd * dv + e);
      x *= (gate_kind == 1 ? 1.0f : g) / (1.0f + expf(-g));
    }
    ls_store(out, out_dtype, (int64_t)item * dv + e, x);
  }
}

// The same for wide heads (all heads normed together make one of heads * dv values): a block per (token, head), the
// head's values kept in registers between the sum of squares and the output (up to HN_WIDE_PER values a thread; what is
// beyond is read again).
constexpr int HN_WIDE_THREADS = 512, HN_WIDE_PER = 8;

__global__ void __launch_bounds__(HN_WIDE_THREADS)
head_norm_gate_wide_kernel(const float* o, const void* __restrict__ w, int w_dtype, const void* gate, int gate_dtype,
                           int64_t gate_ld, int gate_kind, float eps, void* out, int out_dtype, int heads, int dv) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int item = blockIdx.x;
  const int t = item / heads, hd = item - t * heads;
  const float* src = o + (int64_t)item * dv;
  float x[HN_WIDE_PER];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < HN_WIDE_PER; ++i) {
    const int e = threadIdx.x + i * HN_WIDE_THREADS;
    x[i] = e < dv ? __ldcg(src + e) : 0.0f;
    ss = fmaf(x[i], x[i], ss);
  }
  for (int e = threadIdx.x + HN_WIDE_PER * HN_WIDE_THREADS; e < dv; e += HN_WIDE_THREADS) {
    const float v = __ldcg(src + e);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  auto emit = [&](int e, float v) {
    v *= inv;
    if (w) v *= ls_load(w, w_dtype, (int64_t)hd * dv + e);
    if (gate) {
      const float g = ls_load_act(gate, gate_dtype, (int64_t)t * gate_ld + (int64_t)hd * dv + e);
      v *= (gate_kind == 1 ? 1.0f : g) / (1.0f + expf(-g));
    }
    ls_store(out, out_dtype, (int64_t)item * dv + e, v);
  };
#pragma unroll
  for (int i = 0; i < HN_WIDE_PER; ++i) {
    const int e = threadIdx.x + i * HN_WIDE_THREADS;
    if (e < dv) emit(e, x[i]);
  }
  for (int e = threadIdx.x + HN_WIDE_PER * HN_WIDE_THREADS; e < dv; e += HN_WIDE_THREADS) emit(e, __ldcg(src + e));
}

// The same with four values a lane (dv a multiple of 4, at most 128 a head: one piece a lane), float32 weight.
template <typename TG, typename TO>
__global__ void __launch_bounds__(128)
head_norm_gate_vec_kernel(const float* o, const float* __restrict__ w, const TG* gate, int64_t gate_ld, int gate_kind,
                          float eps, TO* out, int n_items, int heads, int dv) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int t = item / heads, hd = item - t * heads;
  const int e = lane * 4;
  float x[4] = {0.0f, 0.0f, 0.0f, 0.0f}, g[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (e < dv) {
    load_vec_cg(o + (int64_t)item * dv + e, x);
    if (gate) {
#pragma unroll
      for (int i = 0; i < 4; ++i)                                      // through L2: a kernel of this step wrote it
        g[i] = ls_load_act(gate, Elem<TG>::code, (int64_t)t * gate_ld + (int64_t)hd * dv + e + i);
    }
  }
  const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  if (e < dv) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = x[i] * inv;
      if (w) v *= w[(int64_t)hd * dv + e + i];
      if (gate) v *= (gate_kind == 1 ? 1.0f : g[i]) / (1.0f + (sizeof(TO) == 4 ? expf(-g[i]) : __expf(-g[i])));
      Elem<TO>::store(out + (int64_t)item * dv + e + i, v);
    }
  }
}

}  // namespace exl3

using namespace exl3;

static bool ls_chunked(int max_new) { return max_new > 2 * LS_CHUNK; }

extern "C" size_t exl3_linear_scan_scratch_bytes(int B, int T, int heads, int dk, int dv, int max_new) {
  if (!ls_chunked(max_new)) return 0;
  return ((size_t)(T / LS_CHUNK + B + 1) * heads * ((size_t)dk + (size_t)dk * dv) + (size_t)B * heads * dk * dv) *
         sizeof(float);
}

extern "C" int exl3_token_shift(const void* h, int h_dtype, const void* mu, int mu_dtype, int n_mix, float* prev,
                                const int* tok_seq, const int* row_start, const int* slot_ids, void* out,
                                int out_dtype, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || n_mix < 1 || prev == nullptr) {
    set_error("token_shift: bad sizes T=%d H=%d mixes=%d", T, H, n_mix);
    return ERR_BAD_ARGUMENT;
  }
  const bool vec = H % 8 == 0 && mu_dtype == DT_F32 && h_dtype == out_dtype && aligned16(h) && aligned16(mu) &&
                   aligned16(prev) && aligned16(out);
  const dim3 threads(H >= 2048 ? 256 : 128);
  if (vec && h_dtype == DT_BF16)
    launch_pdl(token_shift_vec_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), threads, 0, stream,
               static_cast<const __nv_bfloat16*>(h), static_cast<const float*>(mu), n_mix, prev, tok_seq, row_start,
               slot_ids, static_cast<__nv_bfloat16*>(out), T, H);
  else if (vec && h_dtype == DT_F32)
    launch_pdl(token_shift_vec_kernel<float, float>, dim3(T), threads, 0, stream, static_cast<const float*>(h),
               static_cast<const float*>(mu), n_mix, prev, tok_seq, row_start, slot_ids, static_cast<float*>(out), T, H);
  else
    launch_pdl(token_shift_kernel, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream, h, h_dtype, mu, mu_dtype, n_mix,
               prev, tok_seq, row_start, slot_ids, out, out_dtype, T, H);
  return launch_status("token_shift");
}

extern "C" int exl3_linear_scan(int mode, const void* r, int64_t r_ld, const void* k, int64_t k_ld, int rk_dtype,
                                const void* v, int64_t v_ld, int v_dtype, const void* wraw, int64_t w_ld, int w_dtype,
                                const void* w0, const void* u, int wu_dtype, const float* decay, float* state,
                                const int* slot_ids, const int* row_start, float* out, int B, int T, int heads, int dk,
                                int dv, int max_new, int in_act, float* scratch, size_t scratch_bytes, cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  if (B < 0 || T < 0 || heads < 1 || dk < 1 || dv < 1 || dv > 1024 || B > 65535 || mode < 0 || mode > 1 ||
      (mode == 0 && (wraw == nullptr || w0 == nullptr || u == nullptr)) || (mode == 1 && decay == nullptr) || in_act < 0 || in_act > 1) {
    set_error("linear_scan: bad arguments mode=%d rows=%d tokens=%d heads=%d dk=%d dv=%d", mode, B, T, heads, dk, dv);
    return ERR_BAD_ARGUMENT;
  }
  size_t smem = ((size_t)dk * dv + 3 * (size_t)LS_STAGE * dk + LS_STAGE + dk) * sizeof(float);
  if (smem > 200 * 1024) {
    set_error("linear_scan: a state of %d x %d per head does not fit shared memory", dk, dv);
    return ERR_UNSUPPORTED;
  }
  void (*kernel)(ScanArgs, int) = mode == 0 ? linear_scan_kernel<0> : linear_scan_kernel<1>;
  // key sizes of 16, 32, 64 and 128 with up to 128 values a head: the state in registers
  bool regs = dv <= LS_MAX_DV;
  void (*by_phase[3])(ScanArgs, int) = {kernel, kernel, kernel};
#define EXL3_SCAN(DKV)                                                                                            \
  case DKV:                                                                                                       \
    for (int ph = 0; ph < 3; ++ph)                                                                                \
      by_phase[ph] = mode == 0 ? (ph == 0 ? linear_scan_reg_kernel<0, DKV, 0> : ph == 1 ? linear_scan_reg_kernel<0, DKV, 1> \
                                                                                         : linear_scan_reg_kernel<0, DKV, 2>) \
                               : (ph == 0 ? linear_scan_reg_kernel<1, DKV, 0> : ph == 1 ? linear_scan_reg_kernel<1, DKV, 1> \
                                                                                         : linear_scan_reg_kernel<1, DKV, 2>); \
    break;
  if (regs) {
    switch (dk) {
      EXL3_SCAN(16) EXL3_SCAN(32) EXL3_SCAN(64) EXL3_SCAN(128)
      default: regs = false;
    }
  }
#undef EXL3_SCAN
  const int dvr = (dv + 31) / 32 * 32;
  if (regs) smem = (size_t)LS_STAGE * LS_Q * dvr * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("linear_scan: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return (int)e;
    }
  }
  ScanArgs a;
  a.r = r; a.r_ld = r_ld; a.k = k; a.k_ld = k_ld; a.rk_dtype = rk_dtype; a.v = v; a.v_ld = v_ld; a.v_dtype = v_dtype;
  a.wraw = wraw; a.w_ld = w_ld; a.w_dtype = w_dtype; a.w0 = w0; a.u = u; a.wu_dtype = wu_dtype; a.decay = decay;
  a.state = state; a.slot_ids = slot_ids; a.row_start = row_start; a.out = out; a.ab = scratch;
  a.act = in_act;
  a.heads = heads; a.dk = dk; a.dv = dv; a.places = T / LS_CHUNK + B + 1;
  a.snap = scratch ? scratch + (size_t)a.places * heads * ((size_t)dk + (size_t)dk * dv) : nullptr;
  const int threads = regs ? LS_Q * dvr : dvr;
  if (ls_chunked(max_new)) {
    const int chunks = ceil_div(max_new, LS_CHUNK);
    if (scratch == nullptr || exl3_linear_scan_scratch_bytes(B, T, heads, dk, dv, max_new) > scratch_bytes ||
        chunks > 65535) {
      set_error("linear_scan: scratch of %zu bytes is too small for %d tokens", scratch_bytes, T);
      return ERR_SCRATCH;
    }
    launch_pdl(by_phase[1], dim3(heads, chunks, B), dim3(threads), smem, stream, a, 1);
    int rc = launch_status("linear_scan (chunks)");
    if (rc) return rc;
    launch_pdl(by_phase[2], dim3(heads, chunks, B), dim3(threads), smem, stream, a, 2);
    return launch_status("linear_scan (fold)");
  }
  launch_pdl(by_phase[0], dim3(heads, 1, B), dim3(threads), smem, stream, a, 0);
  return launch_status("linear_scan");
}

extern "C" int exl3_head_norm_gate(const float* o, const void* w, int w_dtype, const void* gate, int gate_dtype,
                                   int64_t gate_ld, int gate_kind, float eps, void* out, int out_dtype, int T, int heads,
                                   int dv, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || heads < 1 || dv < 1 || gate_kind < 0 || gate_kind > 1) { set_error("head_norm_gate: bad sizes"); return ERR_BAD_ARGUMENT; }
  const int items = T * heads;
  const bool vec = dv % 4 == 0 && dv <= 128 && (w == nullptr || w_dtype == DT_F32) && aligned16(o) &&
                   (gate == nullptr || gate_ld % 4 == 0);
  const float* wf = static_cast<const float*>(w);
  const dim3 grid(ceil_div(items, 4)), threads(128);
  if (dv > 256)
    launch_pdl(head_norm_gate_wide_kernel, dim3(items), dim3(HN_WIDE_THREADS), 0, stream, o, w, w_dtype, gate, gate_dtype,
               gate_ld, gate_kind, eps, out, out_dtype, heads, dv);
  else if (vec && gate_dtype == DT_BF16 && out_dtype == DT_BF16)
    launch_pdl(head_norm_gate_vec_kernel<__nv_bfloat16, __nv_bfloat16>, grid, threads, 0, stream, o, wf,
               static_cast<const __nv_bfloat16*>(gate), gate_ld, gate_kind, eps, static_cast<__nv_bfloat16*>(out), items, heads, dv);
  else if (vec && gate_dtype == DT_F32 && out_dtype == DT_BF16)
    launch_pdl(head_norm_gate_vec_kernel<float, __nv_bfloat16>, grid, threads, 0, stream, o, wf,
               static_cast<const float*>(gate), gate_ld, gate_kind, eps, static_cast<__nv_bfloat16*>(out), items, heads, dv);
  else if (vec && gate_dtype == DT_F32 && out_dtype == DT_F32)
    launch_pdl(head_norm_gate_vec_kernel<float, float>, grid, threads, 0, stream, o, wf, static_cast<const float*>(gate),
               gate_ld, gate_kind, eps, static_cast<float*>(out), items, heads, dv);
  else
    launch_pdl(head_norm_gate_kernel, grid, threads, 0, stream, o, w, w_dtype, gate, gate_dtype, gate_ld, gate_kind, eps,
               out, out_dtype, items, heads, dv);
  return launch_status("head_norm_gate");
}
