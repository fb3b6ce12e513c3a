// The plain entry point of the weight-streaming projection; the kernel is in gemv_bf16.cuh.
#include "gemv_bf16.cuh"

using namespace exl3;

// epilogue 0: plain; 1: silu(gate) * up over rows interleaved in eights (N even, N % 16 == 0)
extern "C" int exl3_gemv_bf16(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M,
                              int N, int K, int epilogue, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K < 8 || K % 8 != 0) {
    set_error("gemv_bf16: needs 1 <= M <= 16 and K a multiple of 8, got M=%d N=%d K=%d", M, N, K);
    return ERR_BAD_ARGUMENT;
  }
  if (epilogue != 0 && (epilogue != 1 || N % 16 != 0)) {
    set_error("gemv_bf16: the gated epilogue needs N a multiple of 16, got N=%d epilogue=%d", N, epilogue);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w)) { set_error("gemv_bf16: x and w must be 16-byte aligned"); return ERR_ALIGNMENT; }
  const bool f32 = out_dtype == DT_F32;
  if (!f32 && out_dtype != DT_BF16) { set_error("gemv_bf16: unsupported output type %d", out_dtype); return ERR_UNSUPPORTED; }
  int warps, stages;
  const int nt = gemv_shape(M, N, K, warps, stages);
#define EXL3_GEMV(NT, EPI, ST)                                                                  \
  return f32 ? launch<NT, float, EPI, ST>(x, w, bias, y, M, N, K, warps, stream)                \
             : launch<NT, __nv_bfloat16, EPI, ST>(x, w, bias, y, M, N, K, warps, stream)
#define EXL3_GEMV_ST(NT, EPI) { EXL3_GEMV(NT, EPI, gemv_stages(NT)); }   /* the ring's depth follows from NT */
  if (nt == 1) { if (epilogue) { EXL3_GEMV_ST(1, 1) } else { EXL3_GEMV_ST(1, 0) } }
  if (epilogue) { EXL3_GEMV_ST(2, 1) } else { EXL3_GEMV_ST(2, 0) }
#undef EXL3_GEMV_ST
#undef EXL3_GEMV
}

// The plain projection with the xIELU activation on its results (EPI 3 in gemv_bf16.cuh): act_p = softplus(p),
// act_n = 1/2 + softplus(q).
static int gemv_act(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                    float act_p, float act_n, int act_kind, cudaStream_t stream);

extern "C" int exl3_gemv_bf16_act(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M,
                                  int N, int K, float act_p, float act_n, cudaStream_t stream) {
  return gemv_act(x, w, bias, y, out_dtype, M, N, K, act_p, act_n, 0, stream);
}

// The same with GELU on the results: kind 0 exact (erf), 1 by the tanh formula; kind 2: the square of relu.
extern "C" int exl3_gemv_bf16_gelu(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M,
                                   int N, int K, int kind, cudaStream_t stream) {
  if (kind < 0 || kind > 2) { set_error("gemv_bf16_gelu: kind is 0 (erf), 1 (tanh) or 2 (relu squared)"); return ERR_BAD_ARGUMENT; }
  return gemv_act(x, w, bias, y, out_dtype, M, N, K, 0.0f, 0.0f, 1 + kind, stream);
}

static int gemv_act(const void* x, const void* w, const void* bias, void* y, int out_dtype, int M, int N, int K,
                    float act_p, float act_n, int act_kind, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (M < 0 || M > 16 || N < 0 || K < 8 || K % 8 != 0) {
    set_error("gemv_bf16_act: needs 1 <= M <= 16 and K a multiple of 8, got M=%d N=%d K=%d", M, N, K);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(x) || !aligned16(w)) { set_error("gemv_bf16_act: x and w must be 16-byte aligned"); return ERR_ALIGNMENT; }
  const bool f32 = out_dtype == DT_F32;
  if (!f32 && out_dtype != DT_BF16) { set_error("gemv_bf16_act: unsupported output type %d", out_dtype); return ERR_UNSUPPORTED; }
  GemvNorm nrm = {};
  nrm.act_p = act_p;
  nrm.act_n = act_n;
  nrm.act_kind = act_kind;
  int warps, stages;
  const int nt = gemv_shape(M, N, K, warps, stages);
  if (nt == 1)
    return f32 ? launch<1, float, 3, gemv_stages(1)>(x, w, bias, y, M, N, K, warps, stream, nrm)
               : launch<1, __nv_bfloat16, 3, gemv_stages(1)>(x, w, bias, y, M, N, K, warps, stream, nrm);
  return f32 ? launch<2, float, 3, gemv_stages(2)>(x, w, bias, y, M, N, K, warps, stream, nrm)
             : launch<2, __nv_bfloat16, 3, gemv_stages(2)>(x, w, bias, y, M, N, K, warps, stream, nrm);
}
