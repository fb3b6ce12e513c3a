// Hyper-connections: a residual of several streams.
//
// Instead of one residual row a token has S of them, x_1 .. x_S (all equal to the embedding at the start).  A sublayer
// reads a weighted sum of the streams and writes to all of them at once:
//
//   read:   u = sum_s a[s] x_s;   r = u / sqrt(mean(u^2) + eps) * w          (the sublayer's input)
//   write:  x'_t = sum_s M[s, t] x_s + b[t] * y     for every t, from the old streams
//
// One kernel does a write (when y is given) and the read that follows it (when a is given), so a layer of two sublayers
// has two element-wise kernels, as a layer with one residual row has.  With S = 1, M = [[1]], a = b = [1] this is the
// ordinary pre-norm residual.  The model's last norm reads with a = 1 (the sum of the streams) and may do so for a list
// of rows only.  The streams going in may be a single row per token (s_in = 1: the embedding's output), which stands for
// S equal streams.  Everything is float32 inside, sums over streams in the order s = 0 .. S - 1.
#include "api.h"
#include "common.cuh"

namespace exl3 {

constexpr int HC_MAX_STREAMS = 16;      // the kernels are built for up to 4, 8 and 16 streams (MS)
constexpr int HC_THREADS = 256;

struct HyperArgs {
  const float* xin; int s_in;        // [T, s_in, W]
  float* xout;                       // [T, S, W] or null (nothing is stored)
  int S;
  const void* y; int y_dtype;        // [T, W] or null
  const float* mix;                  // [S, S] (from, to), with y
  const float* w_out;                // [S], with y
  const float* w_in;                 // [S] or null (no read)
  const void* norm_w; int norm_w_dtype;   // [W] or null
  float eps;
  void* r; int r_dtype;              // [n, W]
  const int* rows; int n;
  int W;
};

__device__ inline float hc_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}

template <int MS>
__global__ void __launch_bounds__(HC_THREADS) hyper_step_kernel(HyperArgs g) {
  extern __shared__ float su[];                      // [W] the read's sum, then 32 floats for the block's reduction
  float* red = su + g.W;
  __shared__ float smix[MS * MS], sout[MS], sin_[MS];
  const int S = g.S;
  if (threadIdx.x < S * S && g.y) smix[threadIdx.x] = __ldg(g.mix + threadIdx.x);
  if (threadIdx.x < S) {
    if (g.y) sout[threadIdx.x] = __ldg(g.w_out + threadIdx.x);
    if (g.w_in) sin_[threadIdx.x] = __ldg(g.w_in + threadIdx.x);
  }
  pdl_wait();
  pdl_trigger();
  __syncthreads();
  const int i = blockIdx.x;
  const int64_t t = g.rows ? __ldcg(g.rows + i) : i;
  const float* xi = g.xin + t * g.s_in * g.W;
  float* xo = g.xout ? g.xout + t * S * g.W : nullptr;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < g.W; c += HC_THREADS) {
    float x[MS];
#pragma unroll
    for (int s = 0; s < MS; ++s)
      if (s < S) x[s] = __ldcg(xi + (g.s_in == 1 ? 0 : (int64_t)s * g.W) + c);
    if (g.y) {
      const float y = hc_load(g.y, g.y_dtype, t * g.W + c);
      float nx[MS];
#pragma unroll
      for (int to = 0; to < MS; ++to) {
        if (to < S) {
          float a = 0.0f;
#pragma unroll
          for (int s = 0; s < MS; ++s)
            if (s < S) a = fmaf(smix[s * S + to], x[s], a);
          nx[to] = fmaf(sout[to], y, a);
        }
      }
#pragma unroll
      for (int s = 0; s < MS; ++s)
        if (s < S) x[s] = nx[s];
    }
    if (xo && (g.y || g.s_in != S)) {
#pragma unroll
      for (int s = 0; s < MS; ++s)
        if (s < S) xo[(int64_t)s * g.W + c] = x[s];
    }
    if (g.w_in) {
      float u = 0.0f;
#pragma unroll
      for (int s = 0; s < MS; ++s)
        if (s < S) u = fmaf(sin_[s], x[s], u);
      su[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!g.w_in) return;
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)g.W + g.eps);
  for (int c = threadIdx.x; c < g.W; c += HC_THREADS) {
    float v = su[c] * inv;                             // su[c] was written by this same thread
    if (g.norm_w) v *= g.norm_w_dtype == DT_F32 ? __ldg(static_cast<const float*>(g.norm_w) + c)
                                                 : __bfloat162float(static_cast<const __nv_bfloat16*>(g.norm_w)[c]);
    if (g.r_dtype == DT_F32) static_cast<float*>(g.r)[(int64_t)i * g.W + c] = v;
    else static_cast<__nv_bfloat16*>(g.r)[(int64_t)i * g.W + c] = __float2bfloat16_rn(v);
  }
}

// The same with four columns a thread (16-byte accesses of the streams): W a multiple of 4, everything aligned.
template <typename TY, typename TR, int MS>
__global__ void __launch_bounds__(HC_THREADS) hyper_step_vec_kernel(HyperArgs g) {
  extern __shared__ float su[];
  float* red = su + g.W;
  __shared__ float smix[MS * MS], sout[MS], sin_[MS];
  const int S = g.S;
  if (threadIdx.x < S * S && g.y) smix[threadIdx.x] = __ldg(g.mix + threadIdx.x);
  if (threadIdx.x < S) {
    if (g.y) sout[threadIdx.x] = __ldg(g.w_out + threadIdx.x);
    if (g.w_in) sin_[threadIdx.x] = __ldg(g.w_in + threadIdx.x);
  }
  pdl_wait();
  pdl_trigger();
  __syncthreads();
  const int i = blockIdx.x;
  const int64_t t = g.rows ? __ldcg(g.rows + i) : i;
  const float* xi = g.xin + t * g.s_in * g.W;
  float* xo = g.xout ? g.xout + t * S * g.W : nullptr;
  const TY* yp = static_cast<const TY*>(g.y);
  float ss = 0.0f;
  for (int c = threadIdx.x * 4; c < g.W; c += HC_THREADS * 4) {
    float x[MS][4];
#pragma unroll
    for (int s = 0; s < MS; ++s)
      if (s < S) load_vec_cg(xi + (g.s_in == 1 ? 0 : (int64_t)s * g.W) + c, x[s]);
    if (g.y) {
      float y[4];
      if (sizeof(TY) == 4) {
        load_vec_cg(reinterpret_cast<const float*>(yp) + t * g.W + c, y);
      } else {
        const uint2 rr = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(yp) + t * g.W + c));
        y[0] = __uint_as_float(rr.x << 16); y[1] = __uint_as_float(rr.x & 0xffff0000u);
        y[2] = __uint_as_float(rr.y << 16); y[3] = __uint_as_float(rr.y & 0xffff0000u);
      }
      float nx[MS][4];
#pragma unroll
      for (int to = 0; to < MS; ++to) {
        if (to < S) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a = 0.0f;
#pragma unroll
            for (int s = 0; s < MS; ++s)
              if (s < S) a = fmaf(smix[s * S + to], x[s][e], a);
            nx[to][e] = fmaf(sout[to], y[e], a);
          }
        }
      }
#pragma unroll
      for (int s = 0; s < MS; ++s)
        if (s < S) {
#pragma unroll
          for (int e = 0; e < 4; ++e) x[s][e] = nx[s][e];
        }
    }
    if (xo && (g.y || g.s_in != S)) {
#pragma unroll
      for (int s = 0; s < MS; ++s)
        if (s < S) store_vec(xo + (int64_t)s * g.W + c, x[s]);
    }
    if (g.w_in) {
      float u[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = 0.0f;
#pragma unroll
        for (int s = 0; s < MS; ++s)
          if (s < S) a = fmaf(sin_[s], x[s][e], a);
        u[e] = a;
        ss = fmaf(a, a, ss);
      }
      store_vec(su + c, u);
    }
  }
  if (!g.w_in) return;
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)g.W + g.eps);
  for (int c = threadIdx.x * 4; c < g.W; c += HC_THREADS * 4) {
    float v[4];
    load_vec(su + c, v);                               // written by this same thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] *= inv;
      if (g.norm_w) v[e] *= g.norm_w_dtype == DT_F32 ? __ldg(static_cast<const float*>(g.norm_w) + c + e)
                                                      : __bfloat162float(static_cast<const __nv_bfloat16*>(g.norm_w)[c + e]);
    }
    TR* rp = static_cast<TR*>(g.r) + (int64_t)i * g.W + c;
    if (sizeof(TR) == 4) {
      store_vec(reinterpret_cast<float*>(rp), v);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
      uint2 rr;
      rr.x = *reinterpret_cast<uint32_t*>(&lo);
      rr.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(rp) = rr;
    }
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_hyper_max_streams() { return HC_MAX_STREAMS; }

extern "C" int exl3_hyper_step(const float* xin, int s_in, float* xout, int S, const void* y, int y_dtype,
                               const float* mix, const float* w_out, const float* w_in, const void* norm_w,
                               int norm_w_dtype, float eps, void* r, int r_dtype, const int* rows, int n_rows, int T,
                               int W, cudaStream_t stream) {
  const int n = rows ? n_rows : T;
  if (n == 0) return 0;
  if (n < 0 || W < 1 || S < 1 || S > HC_MAX_STREAMS || (s_in != 1 && s_in != S) || xin == nullptr ||
      (y != nullptr && (mix == nullptr || w_out == nullptr || xout == nullptr || rows != nullptr)) ||
      (w_in != nullptr && r == nullptr) || (w_in == nullptr && y == nullptr && !(xout != nullptr && s_in != S)) ||
      (s_in != S && xout == nullptr && y != nullptr)) {
    set_error("hyper_step: bad arguments rows=%d width=%d streams=%d (at most %d) streams in=%d", n, W, S, HC_MAX_STREAMS,
              s_in);
    return ERR_BAD_ARGUMENT;
  }
  if ((y && y_dtype != DT_F32 && y_dtype != DT_BF16) || (r && r_dtype != DT_F32 && r_dtype != DT_BF16)) {
    set_error("hyper_step: unsupported element types %d / %d", y_dtype, r_dtype);
    return ERR_UNSUPPORTED;
  }
  HyperArgs g;
  g.xin = xin; g.s_in = s_in; g.xout = xout; g.S = S; g.y = y; g.y_dtype = y_dtype; g.mix = mix; g.w_out = w_out;
  g.w_in = w_in; g.norm_w = norm_w; g.norm_w_dtype = norm_w_dtype; g.eps = eps; g.r = r; g.r_dtype = r_dtype;
  g.rows = rows; g.n = n; g.W = W;
  const size_t smem = ((size_t)W + 32) * sizeof(float);
  if (smem > 200 * 1024) { set_error("hyper_step: rows of %d features are too wide", W); return ERR_UNSUPPORTED; }
  const bool vec = W % 4 == 0 && aligned16(xin) && (xout == nullptr || aligned16(xout)) &&
                   (y == nullptr || (y_dtype == DT_F32 ? aligned16(y) : (reinterpret_cast<uintptr_t>(y) & 7u) == 0)) &&
                   (r == nullptr || (r_dtype == DT_F32 ? aligned16(r) : (reinterpret_cast<uintptr_t>(r) & 7u) == 0));
#define EXL3_HC(KERNEL)                                                                                        \
  do {                                                                                                         \
    if (smem > 48 * 1024) {                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
      if (e != cudaSuccess) { set_error("hyper_step: shared memory refused: %s", cudaGetErrorString(e)); return (int)e; } \
    }                                                                                                          \
    launch_pdl(KERNEL, dim3(n), dim3(HC_THREADS), smem, stream, g);                                            \
  } while (0)
#define EXL3_HC_MS(MS)                                                                                         \
  do {                                                                                                         \
    if (!vec) {                                                                                                \
      EXL3_HC((hyper_step_kernel<MS>));                                                                        \
    } else {                                                                                                   \
      const bool yf = y == nullptr || y_dtype == DT_F32, rf = r == nullptr || r_dtype == DT_F32;               \
      if (yf && rf) EXL3_HC((hyper_step_vec_kernel<float, float, MS>));                                        \
      else if (yf) EXL3_HC((hyper_step_vec_kernel<float, __nv_bfloat16, MS>));                                 \
      else if (rf) EXL3_HC((hyper_step_vec_kernel<__nv_bfloat16, float, MS>));                                 \
      else EXL3_HC((hyper_step_vec_kernel<__nv_bfloat16, __nv_bfloat16, MS>));                                 \
    }                                                                                                          \
  } while (0)
  if (S <= 4) EXL3_HC_MS(4);
  else if (S <= 8) EXL3_HC_MS(8);
  else EXL3_HC_MS(16);
#undef EXL3_HC_MS
#undef EXL3_HC
  return launch_status("hyper_step");
}
