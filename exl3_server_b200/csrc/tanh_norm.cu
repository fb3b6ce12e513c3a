// A norm without statistics and the residual step of layers whose sublayers run side by side.
//
//   norm:  y = tanh(alpha * x) * w + b            (alpha one learned number, w and b vectors)
//   step:  h <- h + m * (sa * a + sb * b)         (a, b the outputs of two sublayers that read the same h, each
//                                                  times a vector of its own; b may be absent)
//
// One kernel does the step (when a is given) and up to two norms of the new residual, so a layer whose mixer and
// feed-forward read two norms of the same residual has one element-wise kernel between its projections.  With a
// list of rows and no step it norms only those rows (the positions whose logits are wanted).  Everything is
// float32 inside; a and b are float32 or bfloat16, the outputs either.
#include "api.h"
#include "common.cuh"

namespace exl3 {

struct TanhNormArgs {
  float* h;
  const void* a; const void* b; int a_dtype, b_dtype;
  const float* sa; const float* sb; float m;
  const int* rows;
  const float* w1; const float* b1; const float* alpha1; void* out1;
  const float* w2; const float* b2; const float* alpha2; void* out2;
  int out_dtype;
  int n, H;
};

template <typename T, int V> __device__ inline void tn_load(const T* p, float (&v)[V]);
template <> __device__ inline void tn_load<float, 1>(const float* p, float (&v)[1]) { v[0] = __ldcg(p); }
template <> __device__ inline void tn_load<__nv_bfloat16, 1>(const __nv_bfloat16* p, float (&v)[1]) {
  v[0] = __bfloat162float(__ldcg(p));
}
template <> __device__ inline void tn_load<float, 4>(const float* p, float (&v)[4]) { load_vec_cg(p, v); }
template <> __device__ inline void tn_load<__nv_bfloat16, 4>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 r = __ldcg(reinterpret_cast<const uint2*>(p));
  v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
  v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
template <typename T, int V> __device__ inline void tn_store(T* p, const float (&v)[V]);
template <> __device__ inline void tn_store<float, 1>(float* p, const float (&v)[1]) { p[0] = v[0]; }
template <> __device__ inline void tn_store<__nv_bfloat16, 1>(__nv_bfloat16* p, const float (&v)[1]) {
  p[0] = __float2bfloat16_rn(v[0]);
}
template <> __device__ inline void tn_store<float, 4>(float* p, const float (&v)[4]) { store_vec(p, v); }
template <> __device__ inline void tn_store<__nv_bfloat16, 4>(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&lo);
  r.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = r;
}

template <typename TO, int V>
__global__ void __launch_bounds__(256) tanh_norm_add_kernel(TanhNormArgs g) {
  pdl_wait();
  pdl_trigger();
  const int per_row = g.H / V;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)g.n * per_row) return;
  const int i = (int)(idx / per_row);
  const int c = (int)(idx - (int64_t)i * per_row) * V;
  const int64_t t = g.rows ? __ldcg(g.rows + i) : i;
  float x[V];
  tn_load<float, V>(g.h + t * g.H + c, x);
  if (g.a) {
    float a[V], sa[V];
    if (g.a_dtype == DT_F32) tn_load<float, V>(static_cast<const float*>(g.a) + t * g.H + c, a);
    else tn_load<__nv_bfloat16, V>(static_cast<const __nv_bfloat16*>(g.a) + t * g.H + c, a);
    tn_load<float, V>(g.sa + c, sa);
    float s[V];
#pragma unroll
    for (int e = 0; e < V; ++e) s[e] = sa[e] * a[e];
    if (g.b) {
      float b[V], sb[V];
      if (g.b_dtype == DT_F32) tn_load<float, V>(static_cast<const float*>(g.b) + t * g.H + c, b);
      else tn_load<__nv_bfloat16, V>(static_cast<const __nv_bfloat16*>(g.b) + t * g.H + c, b);
      tn_load<float, V>(g.sb + c, sb);
#pragma unroll
      for (int e = 0; e < V; ++e) s[e] = fmaf(sb[e], b[e], s[e]);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) x[e] = fmaf(g.m, s[e], x[e]);
    tn_store<float, V>(g.h + t * g.H + c, x);
  }
  if (g.out1) {
    const float al = __ldg(g.alpha1);
    float w[V], b[V], y[V];
    tn_load<float, V>(g.w1 + c, w);
    tn_load<float, V>(g.b1 + c, b);
#pragma unroll
    for (int e = 0; e < V; ++e) y[e] = fmaf(tanhf(al * x[e]), w[e], b[e]);
    tn_store<TO, V>(static_cast<TO*>(g.out1) + (int64_t)i * g.H + c, y);
  }
  if (g.out2) {
    const float al = __ldg(g.alpha2);
    float w[V], b[V], y[V];
    tn_load<float, V>(g.w2 + c, w);
    tn_load<float, V>(g.b2 + c, b);
#pragma unroll
    for (int e = 0; e < V; ++e) y[e] = fmaf(tanhf(al * x[e]), w[e], b[e]);
    tn_store<TO, V>(static_cast<TO*>(g.out2) + (int64_t)i * g.H + c, y);
  }
}

template <typename TO>
static int tn_launch(const TanhNormArgs& g, bool vec, cudaStream_t stream) {
  const int V = vec ? 4 : 1;
  const int64_t total = (int64_t)g.n * (g.H / V);
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) { set_error("tanh_norm_add: too many elements"); return ERR_UNSUPPORTED; }
  if (vec) launch_pdl(tanh_norm_add_kernel<TO, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, g);
  else launch_pdl(tanh_norm_add_kernel<TO, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, g);
  return launch_status("tanh_norm_add");
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_tanh_norm_add(float* h, const void* a, int a_dtype, const void* b, int b_dtype, const float* sa, const float* sb,
                                  float m, const int* rows, int n_rows, const float* w1, const float* b1,
                                  const float* alpha1, void* out1, const float* w2, const float* b2,
                                  const float* alpha2, void* out2, int out_dtype, int T, int H, cudaStream_t stream) {
  const int n = rows ? n_rows : T;
  if (n == 0) return 0;
  if (n < 0 || H < 1 || h == nullptr || (a == nullptr && b != nullptr) || (a != nullptr && rows != nullptr) ||
      (a != nullptr && sa == nullptr) || (b != nullptr && sb == nullptr) ||
      (out1 != nullptr && (w1 == nullptr || b1 == nullptr || alpha1 == nullptr)) ||
      (out2 != nullptr && (w2 == nullptr || b2 == nullptr || alpha2 == nullptr))) {
    set_error("tanh_norm_add: bad arguments rows=%d width=%d", n, H);
    return ERR_BAD_ARGUMENT;
  }
  TanhNormArgs g;
  g.h = h; g.a = a; g.b = b; g.a_dtype = a_dtype; g.b_dtype = b_dtype; g.sa = sa; g.sb = sb; g.m = m; g.rows = rows;
  g.w1 = w1; g.b1 = b1; g.alpha1 = alpha1; g.out1 = out1; g.w2 = w2; g.b2 = b2; g.alpha2 = alpha2; g.out2 = out2;
  g.out_dtype = out_dtype; g.n = n; g.H = H;
  const bool al8 = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out1) |
                     reinterpret_cast<uintptr_t>(out2)) & 7u) == 0;
  const bool vec = H % 4 == 0 && aligned16(h) && aligned16(sa) && aligned16(sb) && aligned16(w1) && aligned16(b1) &&
                   aligned16(w2) && aligned16(b2) && al8 &&
                   (a_dtype != DT_F32 || aligned16(a)) && (b_dtype != DT_F32 || aligned16(b)) &&
                   (out_dtype != DT_F32 || (aligned16(out1) && aligned16(out2)));
  if ((a && a_dtype != DT_F32 && a_dtype != DT_BF16) || (b && b_dtype != DT_F32 && b_dtype != DT_BF16)) {
    set_error("tanh_norm_add: unsupported element types %d / %d", a_dtype, b_dtype);
    return ERR_UNSUPPORTED;
  }
  if (out_dtype == DT_F32) return tn_launch<float>(g, vec, stream);
  if (out_dtype == DT_BF16) return tn_launch<__nv_bfloat16>(g, vec, stream);
  set_error("tanh_norm_add: unsupported output type %d", out_dtype);
  return ERR_UNSUPPORTED;
}
