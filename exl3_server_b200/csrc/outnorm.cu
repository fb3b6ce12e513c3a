// Parts of a layer whose norm sits on the sublayer's OUTPUT, and the xIELU activation.
//
//   norm_add:  h += y * rsqrt(mean(y^2) + eps) * w        (the residual sum, float32)
//              x  = h in the activation type                (what the next sublayer's projections read)
//   xielu:     a(z) = softplus(p) z^2 + z / 2                          for z > 0
//                     (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2     for z <= 0
//
// Statistics, the sum and the activation are float32 whatever the element types around them.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float on_load_any(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
// for data that an earlier kernel of the same step wrote: through L2 (see load_vec_cg in common.cuh)
__device__ inline float on_load_act(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline void on_store_any(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

constexpr int NA_THREADS = 256;
constexpr int NA_KEEP = 8;                       // values of y a thread keeps in registers: rows up to 2048 are read once

__global__ void __launch_bounds__(NA_THREADS)
norm_add_kernel(float* h, const void* y, int y_dtype, const void* __restrict__ w, int w_dtype, float eps, void* x,
                int x_dtype, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  if (y == nullptr) {
    if (x) for (int c = threadIdx.x; c < H; c += NA_THREADS) on_store_any(x, x_dtype, base + c, __ldcg(h + base + c));
    return;
  }
  float keep[NA_KEEP];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    keep[p] = c < H ? on_load_act(y, y_dtype, base + c) : 0.0f;
    ss += keep[p] * keep[p];
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS) {
    const float v = on_load_act(y, y_dtype, base + c);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    if (c < H) {
      const float v = __ldcg(h + base + c) + keep[p] * inv * on_load_any(w, w_dtype, c);
      h[base + c] = v;
      if (x) on_store_any(x, x_dtype, base + c, v);
    }
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS) {
    const float v = __ldcg(h + base + c) + on_load_act(y, y_dtype, base + c) * inv * on_load_any(w, w_dtype, c);
    h[base + c] = v;
    if (x) on_store_any(x, x_dtype, base + c, v);
  }
}

// Eight consecutive values as floats, from float32 or bfloat16 storage (p 16-byte aligned for bfloat16, 32 for float32).
__device__ inline void on_load8(const float* p, float (&v)[8], bool through_l2) {
  float a[4], b[4];
  if (through_l2) { load_vec_cg(p, a); load_vec_cg(p + 4, b); } else { load_vec(p, a); load_vec(p + 4, b); }
#pragma unroll
  for (int e = 0; e < 4; ++e) { v[e] = a[e]; v[4 + e] = b[e]; }
}
__device__ inline void on_load8(const __nv_bfloat16* p, float (&v)[8], bool through_l2) {
  if (through_l2) load_vec_cg(p, v); else load_vec(p, v);
}
__device__ inline void on_store8(float* p, const float (&v)[8]) {
  const float a[4] = {v[0], v[1], v[2], v[3]}, b[4] = {v[4], v[5], v[6], v[7]};
  store_vec(p, a);
  store_vec(p + 4, b);
}
__device__ inline void on_store8(__nv_bfloat16* p, const float (&v)[8]) { store_vec(p, v); }

constexpr int NA_VECS = 4;                       // pieces of 8 values per thread: rows up to 8192

// The same for rows of up to NA_THREADS * 8 * NA_VECS values, a multiple of 8: a thread keeps its pieces of y in
// registers and every access is 16 or 32 bytes wide.  TX void: no copy of the residual is written.
template <typename TY, typename TW, typename TX>
__global__ void __launch_bounds__(NA_THREADS)
norm_add_vec_kernel(float* h, const TY* y, const TW* __restrict__ w, float eps, TX* x, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  float keep[NA_VECS][8];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      on_load8(y + base + c, keep[p], true);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += keep[p][e] * keep[p][e];
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      float hv[8], wv[8];
      on_load8(h + base + c, hv, true);
      on_load8(w + c, wv, false);
#pragma unroll
      for (int e = 0; e < 8; ++e) hv[e] += keep[p][e] * inv * wv[e];
      on_store8(h + base + c, hv);
      if (x) on_store8(x + base + c, hv);
    }
  }
}

__device__ inline float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

__global__ void xielu_kernel(const void* z, int z_dtype, const void* __restrict__ pq, int pq_dtype, void* out,
                             int out_dtype, int64_t n) {
  pdl_wait();
  pdl_trigger();
  const float ap = softplus_f(on_load_any(pq, pq_dtype, 0));
  const float an = 0.5f + softplus_f(on_load_any(pq, pq_dtype, 1));
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = on_load_act(z, z_dtype, i);
    const float r = v > 0.0f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
    on_store_any(out, out_dtype, i, r);
  }
}

// exp(v) - 1 - v for v <= 0.  Near zero the two subtractions would cancel: there the series v^2/2 + v^3/6 + ... (to
// v^7, below 1e-8 of the result for |v| < 1/4); elsewhere the plain expression.
template <bool FAST>
__device__ inline float xielu_neg(float v) {
  if (!FAST) return expm1f(v) - v;
  if (v > -0.25f) {
    const float p = fmaf(v, fmaf(v, fmaf(v, fmaf(v, fmaf(v, 1.0f / 5040.0f, 1.0f / 720.0f), 1.0f / 120.0f), 1.0f / 24.0f), 1.0f / 6.0f), 0.5f);
    return v * v * p;
  }
  return __expf(v) - 1.0f - v;
}

template <typename TI, typename TO>
__global__ void xielu_vec_kernel(const TI* z, const void* __restrict__ pq, int pq_dtype, TO* out, int64_t n8) {
  pdl_wait();
  pdl_trigger();
  const float ap = softplus_f(on_load_any(pq, pq_dtype, 0));
  const float an = 0.5f + softplus_f(on_load_any(pq, pq_dtype, 1));
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    float v[8];
    on_load8(z + i * 8, v, true);
#pragma unroll
    // results rounded to 16 bits take the short way to the exponential; float32 results the exact one
    for (int e = 0; e < 8; ++e)
      v[e] = v[e] > 0.0f ? fmaf(ap * v[e], v[e], 0.5f * v[e]) : fmaf(an, xielu_neg<sizeof(TO) == 2>(v[e]), 0.5f * v[e]);
    on_store8(out + i * 8, v);
  }
}

template <typename TY, typename TW>
static void norm_add_vec(float* h, const void* y, const void* w, float eps, void* x, int x_dtype, int T, int H,
                         cudaStream_t stream) {
  if (x == nullptr || x_dtype == DT_F32)
    launch_pdl(norm_add_vec_kernel<TY, TW, float>, dim3(T), dim3(NA_THREADS), 0, stream, h, static_cast<const TY*>(y),
               static_cast<const TW*>(w), eps, static_cast<float*>(x), H);
  else
    launch_pdl(norm_add_vec_kernel<TY, TW, __nv_bfloat16>, dim3(T), dim3(NA_THREADS), 0, stream, h,
               static_cast<const TY*>(y), static_cast<const TW*>(w), eps, static_cast<__nv_bfloat16*>(x), H);
}

// norm_add followed by the next sublayer's input norm over the new residual, in one pass: a thread keeps its
// values of the row in registers between the two (rows up to NA_KEEP * NA_THREADS values; beyond that the rest is
// read again).
__global__ void __launch_bounds__(NA_THREADS)
norm_add_norm_kernel(float* h, const void* y, int y_dtype, const void* __restrict__ w, int w_dtype, float eps,
                     const void* __restrict__ w2, int w2_dtype, float eps2, void* x, int x_dtype, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  float keep[NA_KEEP];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    keep[p] = c < H ? on_load_act(y, y_dtype, base + c) : 0.0f;
    ss += keep[p] * keep[p];
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS) {
    const float v = on_load_act(y, y_dtype, base + c);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  float ss2 = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    if (c < H) {
      const float v = __ldcg(h + base + c) + keep[p] * inv * on_load_any(w, w_dtype, c);
      h[base + c] = v;
      keep[p] = v;
      ss2 += v * v;
    }
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS) {
    const float v = __ldcg(h + base + c) + on_load_act(y, y_dtype, base + c) * inv * on_load_any(w, w_dtype, c);
    h[base + c] = v;
    ss2 += v * v;
  }
  ss2 = block_sum(ss2, red);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)H + eps2);
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    if (c < H) on_store_any(x, x_dtype, base + c, keep[p] * inv2 * on_load_any(w2, w2_dtype, c));
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS)      // the same thread wrote h[c]
    on_store_any(x, x_dtype, base + c, h[base + c] * inv2 * on_load_any(w2, w2_dtype, c));
}

// The same for rows of up to NA_THREADS * 8 * NA_VECS values, a multiple of 8, with float32 weights: a thread keeps its
// pieces of the row in registers through both norms and every access is 16 or 32 bytes wide.
template <typename TY, typename TX>
__global__ void __launch_bounds__(NA_THREADS)
norm_add_norm_vec_kernel(float* h, const TY* y, const float* __restrict__ w, float eps, const float* __restrict__ w2,
                         float eps2, TX* x, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  float keep[NA_VECS][8];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      on_load8(y + base + c, keep[p], true);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += keep[p][e] * keep[p][e];
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  float ss2 = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      float hv[8], wv[8];
      on_load8(h + base + c, hv, true);
      on_load8(w + c, wv, false);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        hv[e] += keep[p][e] * inv * wv[e];
        keep[p][e] = hv[e];
        ss2 += hv[e] * hv[e];
      }
      on_store8(h + base + c, hv);
    }
  }
  ss2 = block_sum(ss2, red);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)H + eps2);
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      float wv[8];
      on_load8(w2 + c, wv, false);
#pragma unroll
      for (int e = 0; e < 8; ++e) keep[p][e] *= inv2 * wv[e];
      on_store8(x + base + c, keep[p]);
    }
  }
}

// The two-output norm and sum with 16-byte accesses (rows as above, float32 weights).
template <typename TA>
__global__ void __launch_bounds__(NA_THREADS)
normed_sum2_vec_kernel(const TA* a, const TA* b, const float* __restrict__ wa, const float* __restrict__ wb, float eps,
                       float coef, float* out, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  float ka[NA_VECS][8], kb[NA_VECS][8];
  float sa = 0.0f, sb = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      on_load8(a + base + c, ka[p], true);
      on_load8(b + base + c, kb[p], true);
#pragma unroll
      for (int e = 0; e < 8; ++e) { sa += ka[p][e] * ka[p][e]; sb += kb[p][e] * kb[p][e]; }
    }
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ia = coef / sqrtf(sa / (float)H + eps), ib = coef / sqrtf(sb / (float)H + eps);
#pragma unroll
  for (int p = 0; p < NA_VECS; ++p) {
    const int c = (p * NA_THREADS + threadIdx.x) * 8;
    if (c < H) {
      float wx[8], wy[8], o[8];
      on_load8(wa + c, wx, false);
      on_load8(wb + c, wy, false);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = ka[p][e] * ia * wx[e] + kb[p][e] * ib * wy[e];
      on_store8(out + base + c, o);
    }
  }
}

// Two sublayer outputs side by side, each normed over the row with its own weight, then averaged:
//   out[t] = coef * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb), float32.
__global__ void __launch_bounds__(NA_THREADS)
normed_sum2_kernel(const void* a, const void* b, int ab_dtype, const void* __restrict__ wa, const void* __restrict__ wb,
                   int w_dtype, float eps, float coef, float* out, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  float sa = 0.0f, sb = 0.0f;
  for (int c = threadIdx.x; c < H; c += NA_THREADS) {
    const float x = on_load_act(a, ab_dtype, base + c), y = on_load_act(b, ab_dtype, base + c);
    sa += x * x;
    sb += y * y;
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ia = 1.0f / sqrtf(sa / (float)H + eps), ib = 1.0f / sqrtf(sb / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += NA_THREADS) {
    const float x = on_load_act(a, ab_dtype, base + c) * ia * on_load_any(wa, w_dtype, c);
    const float y = on_load_act(b, ab_dtype, base + c) * ib * on_load_any(wb, w_dtype, c);
    out[base + c] = coef * (x + y);
  }
}

// Element-wise activations, float32 inside: GELU exact (erf, kind 0) or by the tanh formula (1), tanh (2), and the
// square of relu (3).
__device__ inline float act_apply(float v, int kind) {
  if (kind == 0) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
  if (kind == 1) return 0.5f * v * (1.0f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v)));
  if (kind == 3) { const float r = fmaxf(v, 0.0f); return r * r; }
  return tanhf(v);
}

__global__ void gelu_kernel(const void* z, int z_dtype, void* out, int out_dtype, int64_t n, int kind) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = on_load_act(z, z_dtype, i);
    on_store_any(out, out_dtype, i, act_apply(v, kind));
  }
}

template <typename TI, typename TO>
__global__ void gelu_vec_kernel(const TI* z, TO* out, int64_t n8, int kind) {
  pdl_wait();
  pdl_trigger();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    float v[8];
    on_load8(z + i * 8, v, true);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = act_apply(v[e], kind);
    on_store8(out + i * 8, v);
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_norm_add_norm(float* h, const void* y, int y_dtype, const void* w, int w_dtype, float eps,
                                  const void* w2, int w2_dtype, float eps2, void* x, int x_dtype, int T, int H,
                                  cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || y == nullptr || w == nullptr || w2 == nullptr || x == nullptr) {
    set_error("norm_add_norm: bad arguments T=%d H=%d", T, H);
    return ERR_BAD_ARGUMENT;
  }
  const bool vec = H % 8 == 0 && H <= NA_THREADS * 8 * NA_VECS && w_dtype == DT_F32 && w2_dtype == DT_F32 &&
                   aligned16(h) && aligned16(y) && aligned16(w) && aligned16(w2) && aligned16(x);
  const float* wf = static_cast<const float*>(w);
  const float* w2f = static_cast<const float*>(w2);
  if (vec && y_dtype == DT_BF16 && x_dtype == DT_BF16)
    launch_pdl(norm_add_norm_vec_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(T), dim3(NA_THREADS), 0, stream, h,
               static_cast<const __nv_bfloat16*>(y), wf, eps, w2f, eps2, static_cast<__nv_bfloat16*>(x), H);
  else if (vec && y_dtype == DT_F32 && x_dtype == DT_BF16)
    launch_pdl(norm_add_norm_vec_kernel<float, __nv_bfloat16>, dim3(T), dim3(NA_THREADS), 0, stream, h,
               static_cast<const float*>(y), wf, eps, w2f, eps2, static_cast<__nv_bfloat16*>(x), H);
  else if (vec && y_dtype == DT_F32 && x_dtype == DT_F32)
    launch_pdl(norm_add_norm_vec_kernel<float, float>, dim3(T), dim3(NA_THREADS), 0, stream, h,
               static_cast<const float*>(y), wf, eps, w2f, eps2, static_cast<float*>(x), H);
  else
    launch_pdl(norm_add_norm_kernel, dim3(T), dim3(NA_THREADS), 0, stream, h, y, y_dtype, w, w_dtype, eps, w2, w2_dtype,
               eps2, x, x_dtype, H);
  return launch_status("norm_add_norm");
}

extern "C" int exl3_normed_sum2(const void* a, const void* b, int ab_dtype, const void* wa, const void* wb, int w_dtype,
                                float eps, float coef, float* out, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || a == nullptr || b == nullptr || wa == nullptr || wb == nullptr) {
    set_error("normed_sum2: bad arguments T=%d H=%d", T, H);
    return ERR_BAD_ARGUMENT;
  }
  const bool vec = H % 8 == 0 && H <= NA_THREADS * 8 * NA_VECS && w_dtype == DT_F32 && aligned16(a) && aligned16(b) &&
                   aligned16(wa) && aligned16(wb) && aligned16(out);
  if (vec && ab_dtype == DT_BF16)
    launch_pdl(normed_sum2_vec_kernel<__nv_bfloat16>, dim3(T), dim3(NA_THREADS), 0, stream,
               static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<const float*>(wa),
               static_cast<const float*>(wb), eps, coef, out, H);
  else if (vec && ab_dtype == DT_F32)
    launch_pdl(normed_sum2_vec_kernel<float>, dim3(T), dim3(NA_THREADS), 0, stream, static_cast<const float*>(a),
               static_cast<const float*>(b), static_cast<const float*>(wa), static_cast<const float*>(wb), eps, coef, out, H);
  else
    launch_pdl(normed_sum2_kernel, dim3(T), dim3(NA_THREADS), 0, stream, a, b, ab_dtype, wa, wb, w_dtype, eps, coef, out, H);
  return launch_status("normed_sum2");
}

// out[t] = sa * a[t] + sb * b[t], float32 (two sublayer outputs side by side with a constant each).
__global__ void __launch_bounds__(256)
scaled_sum2_kernel(const void* a, const void* b, int ab_dtype, float sa, float sb, float* out, int64_t n) {
  pdl_wait();
  pdl_trigger();
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 4 <= n && ab_dtype == DT_F32) {
    float x[4], y[4], o[4];
    load_vec_cg(static_cast<const float*>(a) + i, x);
    load_vec_cg(static_cast<const float*>(b) + i, y);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = fmaf(sb, y[e], sa * x[e]);
    store_vec(out + i, o);
    return;
  }
  for (int64_t e = i; e < n && e < i + 4; ++e)
    out[e] = fmaf(sb, on_load_act(b, ab_dtype, e), sa * on_load_act(a, ab_dtype, e));
}

extern "C" int exl3_scaled_sum2(const void* a, const void* b, int ab_dtype, float sa, float sb, float* out, int64_t n,
                                cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0 || a == nullptr || b == nullptr || out == nullptr || (ab_dtype != DT_F32 && ab_dtype != DT_BF16) ||
      !aligned16(a) || !aligned16(b) || !aligned16(out)) {
    set_error("scaled_sum2: bad arguments n=%lld", (long long)n);
    return ERR_BAD_ARGUMENT;
  }
  const int64_t blocks = (n / 4 + 1 + 255) / 256;
  if (blocks > 0x7fffffffLL) { set_error("scaled_sum2: too many elements"); return ERR_UNSUPPORTED; }
  launch_pdl(scaled_sum2_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, ab_dtype, sa, sb, out, n);
  return launch_status("scaled_sum2");
}

extern "C" int exl3_activation(const void* z, int z_dtype, void* out, int out_dtype, int64_t n, int kind, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0 || kind < 0 || kind > 3) { set_error("activation: bad arguments"); return ERR_BAD_ARGUMENT; }
  if (n % 8 == 0 && aligned16(z) && aligned16(out)) {
    const int64_t n8 = n / 8;
    int64_t blocks = (n8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const dim3 g((unsigned)blocks), t(256);
    if (z_dtype == DT_F32 && out_dtype == DT_BF16)
      launch_pdl(gelu_vec_kernel<float, __nv_bfloat16>, g, t, 0, stream, static_cast<const float*>(z), static_cast<__nv_bfloat16*>(out), n8, kind);
    else if (z_dtype == DT_BF16 && out_dtype == DT_BF16)
      launch_pdl(gelu_vec_kernel<__nv_bfloat16, __nv_bfloat16>, g, t, 0, stream, static_cast<const __nv_bfloat16*>(z), static_cast<__nv_bfloat16*>(out), n8, kind);
    else if (z_dtype == DT_F32 && out_dtype == DT_F32)
      launch_pdl(gelu_vec_kernel<float, float>, g, t, 0, stream, static_cast<const float*>(z), static_cast<float*>(out), n8, kind);
    else
      launch_pdl(gelu_vec_kernel<__nv_bfloat16, float>, g, t, 0, stream, static_cast<const __nv_bfloat16*>(z), static_cast<float*>(out), n8, kind);
    return launch_status("activation");
  }
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  launch_pdl(gelu_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, z, z_dtype, out, out_dtype, n, kind);
  return launch_status("activation");
}

extern "C" int exl3_norm_add(float* h, const void* y, int y_dtype, const void* w, int w_dtype, float eps, void* x,
                             int x_dtype, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || (y != nullptr && w == nullptr) || (y == nullptr && x == nullptr)) {
    set_error("norm_add: bad arguments T=%d H=%d", T, H);
    return ERR_BAD_ARGUMENT;
  }
  const bool vec = y != nullptr && H % 8 == 0 && H <= NA_THREADS * 8 * NA_VECS && aligned16(h) && aligned16(y) &&
                   aligned16(w) && aligned16(x);
  if (vec && y_dtype == DT_BF16 && w_dtype == DT_BF16) norm_add_vec<__nv_bfloat16, __nv_bfloat16>(h, y, w, eps, x, x_dtype, T, H, stream);
  else if (vec && y_dtype == DT_F32 && w_dtype == DT_BF16) norm_add_vec<float, __nv_bfloat16>(h, y, w, eps, x, x_dtype, T, H, stream);
  else if (vec && y_dtype == DT_BF16 && w_dtype == DT_F32) norm_add_vec<__nv_bfloat16, float>(h, y, w, eps, x, x_dtype, T, H, stream);
  else if (vec && y_dtype == DT_F32 && w_dtype == DT_F32) norm_add_vec<float, float>(h, y, w, eps, x, x_dtype, T, H, stream);
  else launch_pdl(norm_add_kernel, dim3(T), dim3(NA_THREADS), 0, stream, h, y, y_dtype, w, w_dtype, eps, x, x_dtype, H);
  return launch_status("norm_add");
}

extern "C" int exl3_xielu(const void* z, int z_dtype, const void* pq, int pq_dtype, void* out, int out_dtype,
                          int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0) { set_error("xielu: bad size"); return ERR_BAD_ARGUMENT; }
  if (n % 8 == 0 && aligned16(z) && aligned16(out)) {
    const int64_t n8 = n / 8;
    int64_t blocks = (n8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const dim3 g((unsigned)blocks), t(256);
    if (z_dtype == DT_F32 && out_dtype == DT_BF16)
      launch_pdl(xielu_vec_kernel<float, __nv_bfloat16>, g, t, 0, stream, static_cast<const float*>(z), pq, pq_dtype, static_cast<__nv_bfloat16*>(out), n8);
    else if (z_dtype == DT_BF16 && out_dtype == DT_BF16)
      launch_pdl(xielu_vec_kernel<__nv_bfloat16, __nv_bfloat16>, g, t, 0, stream, static_cast<const __nv_bfloat16*>(z), pq, pq_dtype, static_cast<__nv_bfloat16*>(out), n8);
    else if (z_dtype == DT_F32 && out_dtype == DT_F32)
      launch_pdl(xielu_vec_kernel<float, float>, g, t, 0, stream, static_cast<const float*>(z), pq, pq_dtype, static_cast<float*>(out), n8);
    else
      launch_pdl(xielu_vec_kernel<__nv_bfloat16, float>, g, t, 0, stream, static_cast<const __nv_bfloat16*>(z), pq, pq_dtype, static_cast<float*>(out), n8);
    return launch_status("xielu");
  }
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  launch_pdl(xielu_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, z, z_dtype, pq, pq_dtype, out, out_dtype, n);
  return launch_status("xielu");
}
