// Recurrences whose state is a matrix per head and whose step is not a plain decayed sum, and the short convolution that
// feeds one of them.  The state S [dk, dv] of a (sequence, head) is float32, kept per sequence by the cache, read at a
// row's first token of the step and written at its last, so a prompt cut into steps in any way and token-by-token
// decoding walk the same chain in the same order of arithmetic.
//
// Mode 0, a matrix memory with exponential gates (mLSTM).  Per head, with the gates' pre-activations zi, zf:
//   i = cap tanh(zi / cap),  f = logsigmoid(cap tanh(zf / cap)),  m' = max(f + m, i)        (m starts at 0)
//   S' = exp(f + m - m') S + exp(i - m') k v^T,   n' likewise with k alone
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)                                          (q times q_scale)
// State: S, n [dk], m.
//
// Mode 1, the gated delta rule.  Per head, with a decay per key channel g = exp(-exp(A_h) softplus(za + dt_bias)) and
// beta = sigmoid(zb):
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                      (the read sees the write)
// Query and key heads may be shared by several value heads (head h reads q/k head h / (heads / qk_heads)).
//
// Both: a block owns some columns of S of one (row, head) and walks the row's tokens in order; a column lives in the
// registers of four neighbouring lanes (rows i = 4 j + lane % 4), the two dot products of a token are summed inside
// the four lanes; q, k, the decays and the token's scalars are staged in shared memory one token ahead.
//
// conv_prep: per channel a causal convolution over time of `taps` taps (the last tap is the current token's), no bias,
// zeros before the sequence's start, then SiLU; the q and k heads are then made unit vectors, x / sqrt(sum x^2 + eps),
// and q is multiplied by q_scale.  The last taps - 1 inputs of every channel are per-sequence state.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

constexpr int MM_LANES = 4;             // lanes that share a column
constexpr int MM_COLS = 32;             // columns a block owns
constexpr int MM_THREADS = MM_LANES * MM_COLS;
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_CHUNK = 16;          // tokens a warp walks (at least CONV_MAX_TAPS - 1)
constexpr int CONV_WARPS = 4;
constexpr int CONV_MAX_PER_LANE = 8;    // heads of up to 256 channels

__device__ inline float mm_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
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
  float* s_state;                     // [slots, H, dk, dv]
  const int* slot_ids; const int* row_start;
  float* out;                         // [T, H * dv]
  int H, QH, dk, dv;
};

// Stages token t's q, k (and decays) and scalars into buffer `buf`.  sc: [0] a (decay of the state), [1] b (weight of
// the write), [2] exp(-m'), [3] beta.  m_run is thread 0's running maximum (mode 0).
template <int MODE>
__device__ inline void mm_stage(const MatrixMemoryArgs& g, int64_t t, int h, int qh, float* sq, float* sk, float* sg,
                                float* sc, float& m_run) {
  for (int i = threadIdx.x; i < g.dk; i += MM_THREADS) {
    sq[i] = mm_load(g.q, g.qkv_dtype, t * g.ldq + (int64_t)qh * g.dk + i) * g.q_scale;
    sk[i] = mm_load(g.k, g.qkv_dtype, t * g.ldk + (int64_t)qh * g.dk + i);
    if (MODE == 1) {
      const float za = mm_load(g.za, g.za_dtype, t * g.ld_za + (int64_t)h * g.dk + i) + __ldg(g.dt_bias + h * g.dk + i);
      sg[i] = expf(-expf(__ldg(g.a_log + h)) * mm_softplus(za));
    }
  }
  if (threadIdx.x == 0) {
    if (MODE == 0) {
      const float zi = mm_load(g.zi, g.gate_dtype, t * g.ld_gate + h), zf = mm_load(g.zf, g.gate_dtype, t * g.ld_gate + h);
      const float gi = g.cap * tanhf(zi / g.cap);
      const float gf = mm_logsigmoid(g.cap * tanhf(zf / g.cap));
      const float mn = fmaxf(gf + m_run, gi);
      sc[0] = expf(gf + m_run - mn);
      sc[1] = expf(gi - mn);
      sc[2] = expf(-mn);
      sc[4] = mn;
      m_run = mn;
    } else {
      sc[3] = 1.0f / (1.0f + expf(-mm_load(g.zb, g.zb_dtype, t * g.ld_zb + h)));
    }
  }
}

// NR: rows of a column that one lane holds (dk <= 4 NR).
template <int MODE, int NR>
__global__ void __launch_bounds__(MM_THREADS) matrix_memory_kernel(MatrixMemoryArgs g) {
  extern __shared__ float sm[];                      // two buffers of [q | k | g] (dk each) and 8 scalars
  const int dk = g.dk, dv = g.dv;
  const int per = 3 * dk + 8;
  const int row = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * MM_COLS;
  const int qh = h / (g.H / g.QH);
  const int lane4 = threadIdx.x & (MM_LANES - 1);
  const int j = j0 + (threadIdx.x >> 2);
  const bool col_ok = j < dv;
  pdl_wait();
  pdl_trigger();
  const int t0 = __ldcg(g.row_start + row), t1 = __ldcg(g.row_start + row + 1);
  if (t0 >= t1) return;
  const int slot = __ldcg(g.slot_ids + row);
  float* Sp = g.s_state + ((int64_t)slot * g.H + h) * dk * dv;
  float S[NR], nn[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int i = r * MM_LANES + lane4;
    S[r] = (col_ok && i < dk) ? Sp[(int64_t)i * dv + j] : 0.0f;
    nn[r] = 0.0f;
    if (MODE == 0 && i < dk) nn[r] = g.n_state[((int64_t)slot * g.H + h) * dk + i];
  }
  float m_run = MODE == 0 ? g.m_state[(int64_t)slot * g.H + h] : 0.0f;
  mm_stage<MODE>(g, t0, h, qh, sm, sm + dk, sm + 2 * dk, sm + 3 * dk, m_run);
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int b = (t - t0) & 1;
    float* cur = sm + b * per;
    float* nxt = sm + (b ^ 1) * per;
    // the next token's vectors go to the other buffer while this token is worked on
    if (t + 1 < t1) mm_stage<MODE>(g, t + 1, h, qh, nxt, nxt + dk, nxt + 2 * dk, nxt + 3 * dk, m_run);
    const float* sq = cur;
    const float* sk = cur + dk;
    const float* sg = cur + 2 * dk;
    const float* sc = cur + 3 * dk;
    const float vj = col_ok ? mm_load(g.v, g.qkv_dtype, (int64_t)t * g.ldv + (int64_t)h * dv + j) : 0.0f;
    float o;
    if (MODE == 0) {
      const float a = sc[0], bw = sc[1];
      const float bv = bw * vj;
      float num = 0.0f, nq = 0.0f;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int i = r * MM_LANES + lane4;
        const float kk = i < dk ? sk[i] : 0.0f, qq = i < dk ? sq[i] : 0.0f;
        S[r] = fmaf(a, S[r], kk * bv);
        nn[r] = fmaf(a, nn[r], bw * kk);
        num = fmaf(S[r], qq, num);
        nq = fmaf(nn[r], qq, nq);
      }
      num += __shfl_xor_sync(0xffffffffu, num, 1);
      nq += __shfl_xor_sync(0xffffffffu, nq, 1);
      num += __shfl_xor_sync(0xffffffffu, num, 2);
      nq += __shfl_xor_sync(0xffffffffu, nq, 2);
      o = num / (fmaxf(fabsf(nq), sc[2]) + 1e-6f);
    } else {
      float dot = 0.0f;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int i = r * MM_LANES + lane4;
        const float gg = i < dk ? sg[i] : 1.0f, kk = i < dk ? sk[i] : 0.0f;
        S[r] *= gg;
        dot = fmaf(S[r], kk, dot);
      }
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      const float u = sc[3] * (vj - dot);
      float num = 0.0f;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int i = r * MM_LANES + lane4;
        const float kk = i < dk ? sk[i] : 0.0f, qq = i < dk ? sq[i] : 0.0f;
        S[r] = fmaf(kk, u, S[r]);
        num = fmaf(S[r], qq, num);
      }
      num += __shfl_xor_sync(0xffffffffu, num, 1);
      num += __shfl_xor_sync(0xffffffffu, num, 2);
      o = num;
    }
    if (col_ok && lane4 == 0) g.out[(int64_t)t * g.H * dv + (int64_t)h * dv + j] = o;
    __syncthreads();                                   // the next buffer is complete and this one is free
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int i = r * MM_LANES + lane4;
    if (col_ok && i < dk) Sp[(int64_t)i * dv + j] = S[r];
    // the normaliser and the maximum are the same in every block of a head: the first block's first column writes them
    if (MODE == 0 && blockIdx.z == 0 && (threadIdx.x >> 2) == 0 && i < dk)
      g.n_state[((int64_t)slot * g.H + h) * dk + i] = nn[r];
  }
  if (MODE == 0 && blockIdx.z == 0 && threadIdx.x == 0) g.m_state[(int64_t)slot * g.H + h] = m_run;
}

template <int MODE>
static int mm_launch(const MatrixMemoryArgs& g, int rows, cudaStream_t stream) {
  const dim3 grid(rows, g.H, ceil_div(g.dv, MM_COLS));
  const size_t smem = 2 * (size_t)(3 * g.dk + 8) * sizeof(float);
  const int nr = ceil_div(g.dk, MM_LANES);
  if (nr <= 8) launch_pdl(matrix_memory_kernel<MODE, 8>, grid, dim3(MM_THREADS), smem, stream, g);
  else if (nr <= 16) launch_pdl(matrix_memory_kernel<MODE, 16>, grid, dim3(MM_THREADS), smem, stream, g);
  else if (nr <= 32) launch_pdl(matrix_memory_kernel<MODE, 32>, grid, dim3(MM_THREADS), smem, stream, g);
  else if (nr <= 64) launch_pdl(matrix_memory_kernel<MODE, 64>, grid, dim3(MM_THREADS), smem, stream, g);
  else { set_error("matrix_memory: keys of %d features are too wide (at most 256)", g.dk); return ERR_UNSUPPORTED; }
  return launch_status("matrix_memory");
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
  int channels, chunks;
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
  const int first = t0 + chunk * CONV_CHUNK;
  if (first >= t1) return;
  const int last = min(t1, first + CONV_CHUNK);
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

extern "C" int exl3_mlstm_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                               int qkv_dtype, const void* zi, const void* zf, int gate_dtype, int64_t ld_gate, float cap,
                               float q_scale, float* s_state, float* n_state, float* m_state, const int* slot_ids,
                               const int* row_start, float* out, int rows, int T, int heads, int dk, int dv,
                               cudaStream_t stream) {
  if (T == 0 || rows == 0) return 0;
  if (T < 0 || rows < 0 || heads < 1 || dk < 1 || dv < 1 || !(cap > 0.0f) || !mm_dtype_ok(qkv_dtype) || !mm_dtype_ok(gate_dtype) ||
      heads > 65535 || dv > 65535 * MM_COLS) {
    set_error("mlstm_scan: bad sizes rows=%d T=%d heads=%d dk=%d dv=%d cap=%g", rows, T, heads, dk, dv, (double)cap);
    return ERR_BAD_ARGUMENT;
  }
  MatrixMemoryArgs g = {};
  g.q = q; g.k = k; g.v = v; g.qkv_dtype = qkv_dtype; g.ldq = ldq; g.ldk = ldk; g.ldv = ldv; g.q_scale = q_scale;
  g.zi = zi; g.zf = zf; g.gate_dtype = gate_dtype; g.ld_gate = ld_gate; g.cap = cap;
  g.s_state = s_state; g.n_state = n_state; g.m_state = m_state; g.slot_ids = slot_ids; g.row_start = row_start;
  g.out = out; g.H = heads; g.QH = heads; g.dk = dk; g.dv = dv;
  return mm_launch<0>(g, rows, stream);
}

extern "C" int exl3_delta_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                               int qkv_dtype, const void* zb, int zb_dtype, int64_t ld_zb, const void* za, int za_dtype,
                               int64_t ld_za, const float* a_log, const float* dt_bias, float* s_state,
                               const int* slot_ids, const int* row_start, float* out, int rows, int T, int heads,
                               int qk_heads, int dk, int dv, cudaStream_t stream) {
  if (T == 0 || rows == 0) return 0;
  if (T < 0 || rows < 0 || heads < 1 || qk_heads < 1 || heads % qk_heads != 0 || dk < 1 || dv < 1 || !mm_dtype_ok(qkv_dtype) ||
      !mm_dtype_ok(zb_dtype) || !mm_dtype_ok(za_dtype) || heads > 65535 || dv > 65535 * MM_COLS) {
    set_error("delta_scan: bad sizes rows=%d T=%d heads=%d on %d dk=%d dv=%d", rows, T, heads, qk_heads, dk, dv);
    return ERR_BAD_ARGUMENT;
  }
  MatrixMemoryArgs g = {};
  g.q = q; g.k = k; g.v = v; g.qkv_dtype = qkv_dtype; g.ldq = ldq; g.ldk = ldk; g.ldv = ldv; g.q_scale = 1.0f;
  g.zb = zb; g.zb_dtype = zb_dtype; g.ld_zb = ld_zb; g.za = za; g.za_dtype = za_dtype; g.ld_za = ld_za;
  g.a_log = a_log; g.dt_bias = dt_bias; g.s_state = s_state; g.slot_ids = slot_ids; g.row_start = row_start;
  g.out = out; g.H = heads; g.QH = qk_heads; g.dk = dk; g.dv = dv;
  return mm_launch<1>(g, rows, stream);
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
  g.chunks = ceil_div(max_new, CONV_CHUNK);
  const int units = 2 * qk_heads + v_heads;
  const int64_t bx = (int64_t)rows * g.chunks;
  if (bx > 0x7fffffffLL || ceil_div(units, CONV_WARPS) > 65535) { set_error("conv_prep: grid too large"); return ERR_UNSUPPORTED; }
  launch_pdl(conv_prep_kernel, dim3((unsigned)bx, ceil_div(units, CONV_WARPS)), dim3(CONV_WARPS * 32), 0, stream, g);
  return launch_status("conv_prep");
}
