// The experts' projections of a routed feed-forward for many rows (prompts) on the 5th-generation tensor cores: a
// grouped matrix product over the tiles of a plan (see moe.cu),
//   out[i, n] = act(sum_k A[i, k] * W[e(tile of i), n, k]),   bfloat16 operands, float32 accumulation in tensor memory.
//
// A holds one row per planned pair in the plan's order (the pairs of an expert are neighbours), so that a tile's
// rows are one TMA box of 128 rows from the tile's first place on; the rows of the box beyond the tile's own belong
// to the next expert (or to nobody) and are computed with this tile's expert and never stored.  W is the experts'
// matrices stacked, [n_experts * N, K]; a box of 256 rows from row e * N + n0 on may likewise run into the next
// expert's rows, whose columns are never stored.  The number of tiles is read from the plan on the device: a
// step is the same launch whatever the router chose.
//
// Structure (one persistent block per SM, 6 warps), as the dense product's:
//   warp 0    TMA producer: 128 x 64 boxes of A and 256 x 64 boxes of W into a ring of four 128B-swizzled stages
//   warp 1    one thread issues tcgen05.mma (M 128, N 256, K 16); tcgen05.commit frees stages and hands over accumulators
//   warps 2-5 epilogue: thread = row, 32 accumulator columns at a time from tensor memory, the activation, and
//             16-byte stores: in the plan's order (the first projection's output, the second one's input) or to the
//             pair's own place order[i] (float32, for the weighted sum)
// Two accumulators let the epilogue of one tile overlap the products of the next.  Work items are dealt to the blocks in turn
// with the plan's tile fastest: blocks that run together read the same 256 rows of an expert that has several tiles.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel records a code, leaves its loops, waits
// (bounded) for the copies it may have in flight, frees its tensor memory and returns; exl3_moe_tc_status() reads it.
#include "api.h"
#include "tcgen05.cuh"

#include <cuda.h>
#include <math.h>

namespace exl3 {

using namespace tc5;

constexpr int MT_BM = 128, MT_BN = 256, MT_BK = 64, MT_STAGES = 4;
constexpr int MT_THREADS = 192, MT_TMEM_COLS = 512;
constexpr uint32_t MT_STAGE_A = MT_BM * MT_BK * 2, MT_STAGE_B = MT_BN * MT_BK * 2;
constexpr uint32_t MT_SMEM = MT_STAGES * (MT_STAGE_A + MT_STAGE_B) + 1024 /* alignment */ + 256 /* barriers */;
constexpr uint32_t MT_IDESC = idesc_bf16(MT_BM, MT_BN);

static __device__ int g_mt_error = 0;

__device__ inline float mt_act(float v, int act) {
  if (act == 1) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
  if (act == 2) return 0.5f * v * (1.0f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v)));
  if (act == 3) return v / (1.0f + expf(-v));
  return v;
}

__device__ inline void mt_store8(__nv_bfloat16* p, const float (&v)[8]) { store_vec(p, v); }
__device__ inline void mt_store8(float* p, const float (&v)[8]) {
  const float a[4] = {v[0], v[1], v[2], v[3]}, b[4] = {v[4], v[5], v[6], v[7]};
  store_vec(p, a);
  store_vec(p + 4, b);
}

// TO bfloat16: out[i] in the plan's order.  TO float: out[order[i]].
template <typename TO>
__global__ void __launch_bounds__(MT_THREADS, 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, TO* out,
              const int* order, const int* plan, int N, int K, int act) {
  extern __shared__ unsigned char mt_smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(mt_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = base;
  unsigned char* sB = base + MT_STAGES * MT_STAGE_A;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + MT_STAGES * (MT_STAGE_A + MT_STAGE_B));
  uint64_t* full = bars;                       // [STAGES] copies landed
  uint64_t* empty = bars + MT_STAGES;          // [STAGES] the products that read the stage are done
  uint64_t* acc_full = bars + 2 * MT_STAGES;   // [2] accumulator complete
  uint64_t* acc_empty = acc_full + 2;          // [2] accumulator read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < MT_STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc<MT_TMEM_COLS>(tmem_slot);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_m = __ldcg(plan);                            // tiles of the plan
  const int n_n = (N + MT_BN - 1) / MT_BN;
  const int n_items = n_m * n_n, kblocks = (K + MT_BK - 1) / MT_BK;
  bool ok = true;

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------------------------
    uint32_t it = 0;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int mt = item % n_m, nt = item / n_m;
      const int e = __ldcg(plan + 4 + 3 * mt), start = __ldcg(plan + 5 + 3 * mt);
      const int w0 = e * N + nt * MT_BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % MT_STAGES;
        if (!mbar_wait(empty + s, ((it / MT_STAGES) & 1) ^ 1)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(full + s, MT_STAGE_A + MT_STAGE_B);
          tma_load_2d(sA + s * MT_STAGE_A, &map_a, full + s, kb * MT_BK, start);
          tma_load_2d(sB + s * MT_STAGE_B, &map_w, full + s, kb * MT_BK, w0);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) atomicExch(&g_mt_error, 1);
    if (!ok) {                                   // copies still in flight must land before the shared memory goes away
      for (uint32_t back = 1; back <= (uint32_t)MT_STAGES && back <= it; ++back) {
        const uint32_t j = it - back;
        mbar_wait(full + (j % MT_STAGES), (j / MT_STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---- products -----------------------------------------------------------------------------------------------
    uint32_t it = 0, tcount = 0;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++tcount) {
      const uint32_t buf = tcount & 1;
      if (!mbar_wait(acc_empty + buf, ((tcount >> 1) & 1) ^ 1)) { ok = false; break; }
      fence_after();
      const uint32_t d_tmem = tmem_base + buf * MT_BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % MT_STAGES;
        if (!mbar_wait(full + s, (it / MT_STAGES) & 1)) { ok = false; break; }
        fence_after();
        if (lane == 0) {
          const uint64_t da = smem_desc_k128(smem_u32(sA + s * MT_STAGE_A));
          const uint64_t db = smem_desc_k128(smem_u32(sB + s * MT_STAGE_B));
#pragma unroll
          for (int k = 0; k < MT_BK / 16; ++k)           // 32 bytes further along K: start address + 2
            mma_ss(d_tmem, da + 2 * k, db + 2 * k, MT_IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          mma_commit(empty + s);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) mma_commit(acc_full + buf);
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(&g_mt_error, 2);
  } else {
    // ---- epilogue -------------------------------------------------------------------------------------------------
    const int q = warp & 3;                                // the 32 lanes of tensor memory this warp may read
    uint32_t tcount = 0;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++tcount) {
      const int mt = item % n_m, nt = item / n_m;
      const int start = __ldcg(plan + 5 + 3 * mt), nrows = __ldcg(plan + 6 + 3 * mt);
      const int n0 = nt * MT_BN;
      const uint32_t buf = tcount & 1;
      if (!mbar_wait(acc_full + buf, (tcount >> 1) & 1)) { ok = false; break; }
      fence_after();
      const int r = q * 32 + lane;
      const bool row_ok = r < nrows;
      int64_t dst_row = start + r;
      if (sizeof(TO) == 4 && row_ok) dst_row = __ldcg(order + start + r);
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * MT_BN;
#pragma unroll 1
      for (int c = 0; c < MT_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        const int col = n0 + c * 32;
        if (!row_ok || col >= N) continue;
        TO* dst = out + dst_row * N + col;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          if (col + p * 8 + 8 <= N) {
            float o8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o8[j] = mt_act(__uint_as_float(v[p * 8 + j]), act);
            mt_store8(dst + p * 8, o8);
          }
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
    }
    if (!ok && lane == 0) atomicExch(&g_mt_error, 3);
  }

  fence_before();
  __syncthreads();
  fence_after();
  if (warp == 1) tmem_free<MT_TMEM_COLS>(tmem_base);
}

static int mt_sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_moe_tc_rows() { return MT_BM; }

// 0 when no kernel of this file has given up on a wait since the last call; else 1 (copies), 2 (products), 3 (epilogue).
extern "C" int exl3_moe_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_mt_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_mt_error, &z, sizeof(int)); }
  return v;
}

extern "C" int exl3_moe_tc_supported(int N, int K) { return N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0; }

// A bfloat16 [P, K], a row per planned pair in the plan's order (tiles of at most exl3_moe_tc_rows() rows);
// W bfloat16 [n_experts, N, K]; out bfloat16 [P, N] in the plan's order, or float32 [P, N] at the pairs' own places.
extern "C" int exl3_moe_gemm_tc(const void* A, const void* W, const int* order, const int* plan, void* out, int out_dtype,
                                int P, int n_experts, int N, int K, int act, cudaStream_t stream) {
  if (P == 0) return 0;
  if (P < 0 || n_experts < 1 || !exl3_moe_tc_supported(N, K) || act < 0 || act > 3 ||
      (out_dtype != DT_BF16 && out_dtype != DT_F32)) {
    set_error("moe_gemm_tc: needs N and K multiples of 8 and a bfloat16 or float32 output, got pairs=%d experts=%d N=%d "
              "K=%d out=%d", P, n_experts, N, K, out_dtype);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(A) || !aligned16(W) || !aligned16(out)) { set_error("moe_gemm_tc: A, W and out must be 16-byte aligned"); return ERR_ALIGNMENT; }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MT_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(moe_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MT_SMEM);
    if (e != cudaSuccess) { set_error("moe_gemm_tc: cannot get %u bytes of shared memory: %s", MT_SMEM, cudaGetErrorString(e)); return (int)e; }
    configured = true;
  }
  CUtensorMap map_a, map_w;
  int rc = make_map_k64(&map_a, A, P, K, MT_BM, "moe_gemm_tc");
  if (rc) return rc;
  rc = make_map_k64(&map_w, W, (int64_t)n_experts * N, K, MT_BN, "moe_gemm_tc");
  if (rc) return rc;
  const int items = exl3_moe_max_tiles(P, n_experts, MT_BM) * ceil_div(N, MT_BN);
  const int grid = items < mt_sm_count() ? items : mt_sm_count();
  if (out_dtype == DT_BF16)
    moe_tc_kernel<__nv_bfloat16><<<grid, MT_THREADS, MT_SMEM, stream>>>(map_a, map_w, static_cast<__nv_bfloat16*>(out),
                                                                       order, plan, N, K, act);
  else
    moe_tc_kernel<float><<<grid, MT_THREADS, MT_SMEM, stream>>>(map_a, map_w, static_cast<float*>(out), order, plan, N, K,
                                                              act);
  return launch_status("moe_gemm_tc");
}
