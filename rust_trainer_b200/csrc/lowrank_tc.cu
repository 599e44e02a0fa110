// The low-rank side products of a LoRA linear, Hs = X.(sA)^T and Gs = dY.(sB) (reference
// src/linear.rs:84-91,105-117), on tcgen05: out[M x 64] (f16) = X[M x K] . Wt[r x K]^T, r <= 64.
//
// The product is a pure stream over X (2 K bytes per token against 2 r K flops), so what matters
// is how many SMs pull on HBM at once and how few bytes TMA moves per token (an SM takes about
// 75 GB/s through TMA, zero-filled rows included).  The TOKENS are the MMA's N dimension: one CTA
// takes TN = 64 token rows (128 CTAs for 8192 tokens), two producer threads bring [TN x 64] tiles
// of X and [r x 64] tiles of Wt (r rounded up to 8) through a ring of six stages, one thread issues
// tcgen05.mma (M = 128 rank lanes, N = TN tokens, K = 16) into TN TMEM columns.  Only r of the
// MMA's 128 A rows are loaded: the other rows of the operand are whatever follows in shared memory,
// and row i only reaches accumulator lane i.  Two warps read lanes 0..63 (one rank index per
// thread), write zeros from r up, transpose through shared memory, and the tile leaves as one
// contiguous block of [TN][64] f16.  Columns from r up to 63 are exact zeros, which is what the big
// matmul's low-rank chunk expects to find there.
#include "ctx.h"
#include "pdl.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>
#include <stdint.h>

namespace rt {

namespace {

template <int TN, int NS>
struct LrCfg {
  static constexpr uint32_t W_BYTES = 64 * 128, X_BYTES = TN * 128, STAGE = W_BYTES + X_BYTES;
  // the MMA's A descriptor spans 128 rows = 16 KB from a stage's start: the last stage needs that much behind it
  static constexpr uint32_t OFF_OUT = NS * STAGE + (STAGE < 16384 ? 16384 - STAGE : 0);
  static constexpr uint32_t OFF_BAR = OFF_OUT + TN * 128;
  static constexpr uint32_t TOTAL = OFF_BAR + 256 + 1024;
  static_assert(STAGE % 1024 == 0, "stages start on a swizzle atom");
};
enum { SITE_LR_FREE = 491, SITE_LR_FULL, SITE_LR_DONE };

#ifdef RT_B200_QPROF
__device__ unsigned long long g_lr_prof[64];
#define LR_STAMP(i) do { if (blockIdx.x == gridDim.x / 2) g_lr_prof[i] = globaltimer_ns(); } while (0)
#else
#define LR_STAMP(i) do { } while (0)
#endif

template <int TN, int NS>
__global__ void __launch_bounds__(192)
lowrank_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, int M, int K, int r,
                  __half* __restrict__ out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  using Cfg = LrCfg<TN, NS>;
  constexpr int LR_NS = NS, LR_TN = TN;
  constexpr uint32_t LR_STAGE = Cfg::STAGE, LR_W_BYTES = Cfg::W_BYTES, LR_OFF_OUT = Cfg::OFF_OUT, LR_OFF_BAR = Cfg::OFF_BAR;
  uint8_t* sm = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t* bars = (uint64_t*)(sm + LR_OFF_BAR);
  uint64_t* full = bars;            // [NS]
  uint64_t* empty = bars + LR_NS;   // [NS]
  uint64_t* done = bars + 2 * LR_NS;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * LR_NS + 2);
  pdl_launch_dependents();
  if (threadIdx.x == 0) LR_STAMP(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * LR_TN;
  const int nk = (K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < LR_NS; ++i) {
      mbar_init(&full[i], 2);  // the two producer threads
      mbar_init(&empty[i], 1);
    }
    mbar_init(done, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_w);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, LR_TN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  pdl_wait();
  if (threadIdx.x == 0) LR_STAMP(1);

  if (warp == 4 || warp == 3) {
    // two producer threads (one TMA instruction costs its thread about 0.1 us): X tiles and factor tiles
    if (lane == 0) {
      const bool xs = warp == 4;
      for (int kc = 0; kc < nk; ++kc) {
        const int s = kc % LR_NS;
        if (!mbar_wait(&empty[s], (((uint32_t)(kc / LR_NS)) & 1) ^ 1, status, SITE_LR_FREE)) break;
        if (xs) {
          mbar_expect_tx(&full[s], Cfg::X_BYTES);
          tma_load_2d(sm + s * LR_STAGE + LR_W_BYTES, &tm_x, kc * 64, m0, &full[s]);
        } else {
          mbar_expect_tx(&full[s], (uint32_t)((r + 7) & ~7) * 128u);
          tma_load_2d(sm + s * LR_STAGE, &tm_w, kc * 64, 0, &full[s]);
        }
        if (kc == 0 && xs) LR_STAMP(2);
      }
      if (xs) LR_STAMP(3);
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(0, 0, 0, 0, 128, LR_TN);
      const uint32_t s0 = smem_u32(sm);
      bool ok = true;
      for (int kc = 0; kc < nk && ok; ++kc) {
        const int s = kc % LR_NS;
        if (!mbar_wait(&full[s], ((uint32_t)(kc / LR_NS)) & 1, status, SITE_LR_FULL)) { ok = false; break; }
        if (kc < 24) LR_STAMP(8 + kc);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ad = umma_desc_sw128(s0 + s * LR_STAGE + kk * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(s0 + s * LR_STAGE + LR_W_BYTES + kk * 32, 16, 1024);
          umma_f16(tmem_base, ad, bd, idesc, (kc | kk) != 0);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(done);
      LR_STAMP(4);
    }
  } else if (warp < 2) {
    // thread = rank index = TMEM lane; its TN columns are the tile's tokens
    if (mbar_wait(done, 0, status, SITE_LR_DONE)) {
      if (threadIdx.x == 0) LR_STAMP(5);
      tc_fence_after();
      uint32_t v[LR_TN];
#pragma unroll
      for (int c = 0; c < LR_TN; c += 32) tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + c, v + c);
      tmem_ld_wait();
      const bool keep = warp * 32 + lane < r;  // lanes from r up hold products with whatever follows the factor tile
      __half* so = (__half*)(sm + LR_OFF_OUT) + warp * 32 + lane;
#pragma unroll
      for (int t = 0; t < LR_TN; ++t) so[t * 64] = __float2half_rn(keep ? __uint_as_float(v[t]) : 0.f);
    }
  }
  if (*(volatile int*)status != 0) {
    for (int k = 0; k < 1000; ++k) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (*(volatile int*)status == 0) {
    // [TN tokens][64] f16 is one contiguous block of the output
    const int rows = M - m0 < LR_TN ? M - m0 : LR_TN;
    const uint4* src = (const uint4*)(sm + LR_OFF_OUT);
    uint4* dst = (uint4*)(out + (size_t)m0 * 64);
    for (int e = threadIdx.x; e < rows * 8; e += 192) dst[e] = src[e];
  }
  if (threadIdx.x == 0) LR_STAMP(6);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, LR_TN);
  }
}

}  // namespace

constexpr int LR_TN_DEFAULT = 64, LR_NS_DEFAULT = 6;

template <int TN, int NS>
static int lowrank_launch(rt_ctx* c, const __half* X, const __half* Wt, int M, int K, int r, __half* out64) {
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(lowrank_tc_kernel<TN, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LrCfg<TN, NS>::TOTAL) !=
        cudaSuccess)
      return 3;
    attr = true;
  }
  CUtensorMap tx, tw;
  if (tensor_map_f16_2d(c, &tx, X, (uint64_t)M, (uint64_t)K, 64, TN)) return 3;
  if (tensor_map_f16_2d(c, &tw, Wt, (uint64_t)r, (uint64_t)K, 64, (uint32_t)((r + 7) & ~7))) return 3;
  pdl(lowrank_tc_kernel<TN, NS>, (M + TN - 1) / TN, 192, LrCfg<TN, NS>::TOTAL, c->stream)(tx, tw, M, K, r, out64, c->status_dev);
  RT_COUNT_LAUNCH(1);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// 0: launched; 1: shape not supported (the caller has other routes); 3: launch failure
int launch_lowrank_tc(rt_ctx* c, const __half* X, const __half* Wt, int M, int K, int r, __half* out64) {
  if (M <= 0) return 0;
  if (r <= 0 || r > 64 || K % 8 != 0 || ((uintptr_t)X & 15) || ((uintptr_t)Wt & 15) || ((uintptr_t)out64 & 15)) return 1;
  return lowrank_launch<LR_TN_DEFAULT, LR_NS_DEFAULT>(c, X, Wt, M, K, r, out64);
}

#ifdef RT_B200_QPROF
// measurement aid: times `iters` launches of one configuration on fresh buffers and returns the stamps of one CTA
extern "C" int rt_debug_lowrank_bench(rt_ctx* c, int M, int K, int r, int tn, int ns, int iters, float* us_out,
                                      unsigned long long* prof, int nprof) {
  __half *X = nullptr, *W = nullptr, *O = nullptr;
  if (cudaMalloc(&X, (size_t)M * K * 2) || cudaMalloc(&W, (size_t)r * K * 2) || cudaMalloc(&O, (size_t)M * 64 * 2 + 256)) return 2;
  cudaMemset(X, 0, (size_t)M * K * 2);
  cudaMemset(W, 0, (size_t)r * K * 2);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  int rc = 0;
  auto go = [&]() {
    if (tn == 32 && ns == 4) return lowrank_launch<32, 4>(c, X, W, M, K, r, O);
    if (tn == 32 && ns == 6) return lowrank_launch<32, 6>(c, X, W, M, K, r, O);
    if (tn == 32 && ns == 8) return lowrank_launch<32, 8>(c, X, W, M, K, r, O);
    if (tn == 64 && ns == 4) return lowrank_launch<64, 4>(c, X, W, M, K, r, O);
    if (tn == 64 && ns == 6) return lowrank_launch<64, 6>(c, X, W, M, K, r, O);
    if (tn == 64 && ns == 8) return lowrank_launch<64, 8>(c, X, W, M, K, r, O);
    return 1;
  };
  for (int i = 0; i < 3 && !rc; ++i) rc = go();
  cudaEventRecord(e0, c->stream);
  for (int i = 0; i < iters && !rc; ++i) rc = go();
  cudaEventRecord(e1, c->stream);
  cudaStreamSynchronize(c->stream);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  *us_out = ms * 1000.f / iters;
  cudaMemcpyFromSymbol(prof, g_lr_prof, sizeof(unsigned long long) * (nprof < 64 ? nprof : 64));
  cudaFree(X); cudaFree(W); cudaFree(O);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  return rc;
}
#endif

}  // namespace rt
