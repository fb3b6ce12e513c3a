// Attention whose heads hold several maps (softmaxes of their own over the same values), as in differential
// attention: what stands before and after the attention kernels.
//
// A head's query is [map 0 | map 1 | ...], each of d features; a key/value head's key likewise.  The attention
// kernels know nothing of maps: a key row of the cache is the kv head's maps side by side (maps * d features), and
// every map of a query head becomes a query head of its own of maps * d features that is zero outside its map, so
// that q . k is the map's own score.  Query head h, map m is head h * maps + m there; all maps of the query heads of
// a group read the group's one key row and the one value row.
//
//   maps_prep     rotary positions (half-split pairs over the first `rot` features of every map), the widened
//                 queries, keys and values into the paged cache.  A token's sines and cosines are worked out once
//                 per block.
//   diff_combine  o = a_0 - lambda * a_1, divided by its root mean square over the head's values (no weight), times
//                 a constant, times sigmoid(gate[t, head]).
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace exl3 {

__device__ inline float da_ld(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline void da_st(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// feature i of a map of d features, rotated: pairs (i, i + rot / 2) for i < rot / 2
__device__ inline float da_rotated(const void* x, int dtype, int64_t base, int i, int rot, const float* sn,
                                   const float* cs) {
  const float v = da_ld(x, dtype, base + i);
  if (i >= rot) return v;
  const int half = rot >> 1;
  if (i < half) return v * cs[i] - da_ld(x, dtype, base + i + half) * sn[i];
  return v * cs[i - half] + da_ld(x, dtype, base + i - half) * sn[i - half];
}

// A block takes MP_ITEMS outputs of one token: the widened queries first, then the key rows, then the value rows.
constexpr int MP_THREADS = 256, MP_ITEMS = 2048;

__global__ void __launch_bounds__(MP_THREADS)
maps_prep_kernel(const void* x, int x_dtype, int64_t ld, int q_off, int k_off, int v_off, int nh, int nkv, int maps, int d,
                 int dv, int row, int v_row, int rot, const float* __restrict__ f_hi, const float* __restrict__ f_lo,
                 const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride, int page, void* q_out,
                 int q_dtype, void* k_pool, void* v_pool, int pool_dtype) {
  extern __shared__ float sc[];                    // [rot / 2] sines, [rot / 2] cosines
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = __ldcg(tok_pos + t);
  const int half = rot >> 1;
  float* sn = sc;
  float* cs = sc + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) rope_sincos((float)pos, f_hi[i], f_lo[i], sn + i, cs + i);
  __syncthreads();
  const int64_t xb = (int64_t)t * ld;
  const int nq = nh * maps;
  const int n_q = nq * row, n_k = nkv * row, n_v = nkv * v_row;
  const int pg = __ldcg(block_table + (int64_t)__ldcg(tok_seq + t) * bt_stride + pos / page);
  const int slot = pos % page;
  const int first = blockIdx.y * MP_ITEMS;
  const int last = min(first + MP_ITEMS, n_q + n_k + n_v);
  for (int item = first + threadIdx.x; item < last; item += MP_THREADS) {
    if (item < n_q) {
      // queries: head h, map m -> head h * maps + m, features [m * d, m * d + d) of `row`, zero elsewhere
      const int vh = item / row, c = item - vh * row;
      const int m = vh % maps;
      float v = 0.0f;
      if (c >= m * d && c < m * d + d) v = da_rotated(x, x_dtype, xb + q_off + (int64_t)vh * d, c - m * d, rot, sn, cs);
      da_st(q_out, q_dtype, (int64_t)t * n_q + item, v);
    } else if (pg < 0) {
      continue;
    } else if (item < n_q + n_k) {
      const int idx = item - n_q;
      const int g = idx / row, c = idx - g * row;
      float v = 0.0f;
      if (c < maps * d) {
        const int m = c / d;
        v = da_rotated(x, x_dtype, xb + k_off + ((int64_t)g * maps + m) * d, c - m * d, rot, sn, cs);
      }
      da_st(k_pool, pool_dtype, (((int64_t)pg * nkv + g) * page + slot) * row + c, v);
    } else {
      const int idx = item - n_q - n_k;
      const int g = idx / v_row, c = idx - g * v_row;
      const float v = c < dv ? da_ld(x, x_dtype, xb + v_off + (int64_t)g * dv + c) : 0.0f;
      da_st(v_pool, pool_dtype, (((int64_t)pg * nkv + g) * page + slot) * v_row + c, v);
    }
  }
}

// The same for bfloat16 queries and cache (the projection bfloat16 or float32) with every size a multiple of 8 (d,
// rot / 2, dv, the rows, the offsets, the row pitch): a thread takes 8 neighbouring outputs with 16-byte loads and stores.
__device__ inline void mp_ld8(const __nv_bfloat16* p, float (&v)[8]) { load_vec_cg(p, v); }
__device__ inline void mp_ld8(const float* p, float (&v)[8]) {
  float a[4], b[4];
  load_vec_cg(p, a);
  load_vec_cg(p + 4, b);
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[j] = a[j]; v[4 + j] = b[j]; }
}

template <typename TX>
__device__ inline void mp_rot8(const TX* src, int i, int rot, const float* sn, const float* cs, float (&v)[8]) {
  mp_ld8(src + i, v);
  if (i >= rot) return;
  const int half = rot >> 1;
  float o[8];
  if (i < half) {
    mp_ld8(src + i + half, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] * cs[i + j] - o[j] * sn[i + j];
  } else {
    mp_ld8(src + i - half, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] * cs[i - half + j] + o[j] * sn[i - half + j];
  }
}

template <typename TX>
__global__ void __launch_bounds__(MP_THREADS)
maps_prep_vec_kernel(const TX* x, int64_t ld, int q_off, int k_off, int v_off, int nh, int nkv, int maps, int d,
                     int dv, int row, int v_row, int rot, const float* __restrict__ f_hi, const float* __restrict__ f_lo,
                     const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride, int page,
                     __nv_bfloat16* q_out, __nv_bfloat16* k_pool, __nv_bfloat16* v_pool) {
  extern __shared__ float sc[];                    // [rot / 2] sines, [rot / 2] cosines
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int pos = __ldcg(tok_pos + t);
  const int half = rot >> 1;
  float* sn = sc;
  float* cs = sc + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) rope_sincos((float)pos, f_hi[i], f_lo[i], sn + i, cs + i);
  __syncthreads();
  const TX* xt = x + (int64_t)t * ld;
  const int nq = nh * maps;
  const int n_q = nq * row, n_k = nkv * row, n_v = nkv * v_row;
  const int pg = __ldcg(block_table + (int64_t)__ldcg(tok_seq + t) * bt_stride + pos / page);
  const int slot = pos % page;
  const int first = blockIdx.y * MP_ITEMS;
  const int last = min(first + MP_ITEMS, n_q + n_k + n_v);
  for (int item = first + threadIdx.x * 8; item < last; item += MP_THREADS * 8) {
    float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (item < n_q) {
      const int vh = item / row, c = item - vh * row;
      const int m = vh % maps;
      if (c >= m * d && c < m * d + d) mp_rot8(xt + q_off + (int64_t)vh * d, c - m * d, rot, sn, cs, v);
      store_vec(q_out + (int64_t)t * n_q + item, v);
    } else if (pg < 0) {
      continue;
    } else if (item < n_q + n_k) {
      const int idx = item - n_q;
      const int g = idx / row, c = idx - g * row;
      if (c < maps * d) {
        const int m = c / d;
        mp_rot8(xt + k_off + ((int64_t)g * maps + m) * d, c - m * d, rot, sn, cs, v);
      }
      store_vec(k_pool + (((int64_t)pg * nkv + g) * page + slot) * row + c, v);
    } else {
      const int idx = item - n_q - n_k;
      const int g = idx / v_row, c = idx - g * v_row;
      if (c < dv) mp_ld8(xt + v_off + (int64_t)g * dv + c, v);
      store_vec(v_pool + (((int64_t)pg * nkv + g) * page + slot) * v_row + c, v);
    }
  }
}

// a [T, heads * 2, a_row]: the two maps' outputs of every head; a warp per (token, head).
__global__ void __launch_bounds__(128)
diff_combine_kernel(const void* a, int a_dtype, int a_row, const void* gate, int gate_dtype, int64_t gate_ld, float lambda,
                    float eps, float mult, void* out, int out_dtype, int out_row, int n_items, int heads, int dv) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const int t = item / heads, h = item - t * heads;
  const int64_t a1 = (int64_t)item * 2 * a_row, a2 = a1 + a_row;
  float ss = 0.0f;
  for (int e = lane; e < dv; e += 32) {
    const float o = da_ld(a, a_dtype, a1 + e) - lambda * da_ld(a, a_dtype, a2 + e);
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  float f = mult / sqrtf(ss / (float)dv + eps);
  if (gate) f *= 1.0f / (1.0f + expf(-da_ld(gate, gate_dtype, (int64_t)t * gate_ld + h)));
  for (int e = lane; e < out_row; e += 32) {
    float o = 0.0f;
    if (e < dv) o = (da_ld(a, a_dtype, a1 + e) - lambda * da_ld(a, a_dtype, a2 + e)) * f;
    da_st(out, out_dtype, (int64_t)item * out_row + e, o);
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_maps_prep(const void* x, int x_dtype, int64_t ld, int q_off, int k_off, int v_off, int T, int nh,
                              int nkv, int maps, int d, int dv, int row, int v_row, int rot, const float* f_hi,
                              const float* f_lo, const int* tok_pos, const int* tok_seq, const int* block_table,
                              int bt_stride, int page, void* q_out, int q_dtype, void* k_pool, void* v_pool,
                              int pool_dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 1 || nkv < 1 || maps < 1 || d < 1 || dv < 1 || row < maps * d || v_row < dv || rot < 0 || rot > d ||
      (rot & 1) || page < 1 || (rot > 0 && (f_hi == nullptr || f_lo == nullptr)) || k_pool == nullptr ||
      v_pool == nullptr || block_table == nullptr) {
    set_error("maps_prep: bad sizes T=%d heads=%d kv_heads=%d maps=%d d=%d dv=%d rows=%d/%d rot=%d", T, nh, nkv, maps, d,
              dv, row, v_row, rot);
    return ERR_BAD_ARGUMENT;
  }
  const int items = nh * maps * row + nkv * row + nkv * v_row;
  if (ceil_div(items, MP_ITEMS) > 65535) { set_error("maps_prep: rows too wide"); return ERR_UNSUPPORTED; }
  const bool vec = (x_dtype == DT_BF16 || x_dtype == DT_F32) && q_dtype == DT_BF16 && pool_dtype == DT_BF16 && d % 8 == 0 && (rot >> 1) % 8 == 0 &&
                   dv % 8 == 0 && row % 8 == 0 && v_row % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
                   ld % 8 == 0 && aligned16(x) && aligned16(q_out) && aligned16(k_pool) && aligned16(v_pool);
  if (vec && x_dtype == DT_BF16) {
    launch_pdl(maps_prep_vec_kernel<__nv_bfloat16>, dim3(T, ceil_div(items, MP_ITEMS)), dim3(MP_THREADS),
               (size_t)rot * sizeof(float), stream, static_cast<const __nv_bfloat16*>(x), ld, q_off, k_off, v_off, nh, nkv,
               maps, d, dv, row, v_row, rot, f_hi, f_lo, tok_pos, tok_seq, block_table, bt_stride, page,
               static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool));
    return launch_status("maps_prep");
  }
  if (vec) {
    launch_pdl(maps_prep_vec_kernel<float>, dim3(T, ceil_div(items, MP_ITEMS)), dim3(MP_THREADS),
               (size_t)rot * sizeof(float), stream, static_cast<const float*>(x), ld, q_off, k_off, v_off, nh, nkv, maps, d,
               dv, row, v_row, rot, f_hi, f_lo, tok_pos, tok_seq, block_table, bt_stride, page,
               static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool));
    return launch_status("maps_prep");
  }
  launch_pdl(maps_prep_kernel, dim3(T, ceil_div(items, MP_ITEMS)), dim3(MP_THREADS), (size_t)rot * sizeof(float), stream,
             x, x_dtype, ld, q_off, k_off, v_off, nh, nkv, maps, d, dv, row, v_row, rot, f_hi, f_lo, tok_pos, tok_seq,
             block_table, bt_stride, page, q_out, q_dtype, k_pool, v_pool, pool_dtype);
  return launch_status("maps_prep");
}

extern "C" int exl3_diff_combine(const void* a, int a_dtype, int a_row, const void* gate, int gate_dtype, int64_t gate_ld,
                                 float lambda, float eps, float mult, void* out, int out_dtype, int out_row, int T,
                                 int heads, int dv, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || heads < 1 || dv < 1 || a_row < dv || out_row < dv) {
    set_error("diff_combine: bad sizes T=%d heads=%d dv=%d rows=%d/%d", T, heads, dv, a_row, out_row);
    return ERR_BAD_ARGUMENT;
  }
  const int items = T * heads;
  launch_pdl(diff_combine_kernel, dim3(ceil_div(items, 4)), dim3(128), 0, stream, a, a_dtype, a_row, gate, gate_dtype,
             gate_ld, lambda, eps, mult, out, out_dtype, out_row, items, heads, dv);
  return launch_status("diff_combine");
}
