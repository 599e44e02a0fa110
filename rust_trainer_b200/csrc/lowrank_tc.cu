// The low-rank side products of a LoRA linear, Hs = X.(sA)^T and Gs = dY.(sB) (reference
// src/linear.rs:84-91,105-117), on tcgen05: out[M x 64] (f16) = X[M x K] . Wt[r x K]^T, r <= 64.
//
// The product is a pure stream over X (2 K bytes per token against 2 r K flops): one CTA takes 128
// token rows, TMA brings [128 x 64] tiles of X and [64 x 64] tiles of Wt (rows past r are
// zero-filled by the tensor map) through a ring of six stages, one thread issues
// tcgen05.mma (M = 128 tokens, N = 64, K = 16) into a 64-column TMEM accumulator, and four warps
// write the rows out as f16.  Columns from r up to 63 come out as exact zeros, which is what the
// big matmul's low-rank chunk expects to find there.
#include "ctx.h"
#include "ptx.cuh"
#include <cuda_fp16.h>
#include <stdint.h>

namespace rt {

namespace {

constexpr int LR_NS = 6;
constexpr uint32_t LR_X_BYTES = 128 * 128, LR_W_BYTES = 64 * 128, LR_STAGE = LR_X_BYTES + LR_W_BYTES;
constexpr uint32_t LR_OFF_BAR = LR_NS * LR_STAGE;
constexpr uint32_t LR_TOTAL = LR_OFF_BAR + 256 + 1024;
enum { SITE_LR_FREE = 491, SITE_LR_FULL, SITE_LR_DONE };

__global__ void __launch_bounds__(192, 1)
lowrank_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, int M, int K,
                  __half* __restrict__ out, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t* bars = (uint64_t*)(sm + LR_OFF_BAR);
  uint64_t* full = bars;            // [NS]
  uint64_t* empty = bars + LR_NS;   // [NS]
  uint64_t* done = bars + 2 * LR_NS;
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * LR_NS + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * 128;
  const int nk = (K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < LR_NS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(done, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_w);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      for (int kc = 0; kc < nk; ++kc) {
        const int s = kc % LR_NS;
        if (!mbar_wait(&empty[s], (((uint32_t)(kc / LR_NS)) & 1) ^ 1, status, SITE_LR_FREE)) break;
        mbar_expect_tx(&full[s], LR_STAGE);
        tma_load_2d(sm + s * LR_STAGE, &tm_x, kc * 64, m0, &full[s]);
        tma_load_2d(sm + s * LR_STAGE + LR_X_BYTES, &tm_w, kc * 64, 0, &full[s]);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(0, 0, 0, 0, 128, 64);
      const uint32_t s0 = smem_u32(sm);
      bool ok = true;
      for (int kc = 0; kc < nk && ok; ++kc) {
        const int s = kc % LR_NS;
        if (!mbar_wait(&full[s], ((uint32_t)(kc / LR_NS)) & 1, status, SITE_LR_FULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ad = umma_desc_sw128(s0 + s * LR_STAGE + kk * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(s0 + s * LR_STAGE + LR_X_BYTES + kk * 32, 16, 1024);
          umma_f16(tmem_base, ad, bd, idesc, (kc | kk) != 0);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(done);
    }
  } else {
    // thread = token row = TMEM lane
    const int r = warp * 32 + lane, m = m0 + r;
    if (mbar_wait(done, 0, status, SITE_LR_DONE)) {
      tc_fence_after();
      uint32_t v[64];
      tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16), v);
      tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + 32, v + 32);
      tmem_ld_wait();
      if (m < M) {
        uint4* orow = (uint4*)(out + (size_t)m * 64);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 w;
          __half2 h0 = __floats2half2_rn(__uint_as_float(v[8 * c]), __uint_as_float(v[8 * c + 1]));
          __half2 h1 = __floats2half2_rn(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3]));
          __half2 h2 = __floats2half2_rn(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5]));
          __half2 h3 = __floats2half2_rn(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7]));
          w.x = *(uint32_t*)&h0; w.y = *(uint32_t*)&h1; w.z = *(uint32_t*)&h2; w.w = *(uint32_t*)&h3;
          orow[c] = w;
        }
      }
    }
  }
  if (*(volatile int*)status != 0) {
    for (int k = 0; k < 1000; ++k) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

}  // namespace

// 0: launched; 1: shape not supported (the caller has other routes); 3: launch failure
int launch_lowrank_tc(rt_ctx* c, const __half* X, const __half* Wt, int M, int K, int r, __half* out64) {
  if (M <= 0) return 0;
  if (r <= 0 || r > 64 || K % 8 != 0 || ((uintptr_t)X & 15) || ((uintptr_t)Wt & 15) || ((uintptr_t)out64 & 15)) return 1;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(lowrank_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LR_TOTAL) != cudaSuccess) return 3;
    attr = true;
  }
  CUtensorMap tx, tw;
  if (tensor_map_f16_2d(c, &tx, X, (uint64_t)M, (uint64_t)K, 64, 128)) return 3;
  if (tensor_map_f16_2d(c, &tw, Wt, (uint64_t)r, (uint64_t)K, 64, 64)) return 3;
  lowrank_tc_kernel<<<(M + 127) / 128, 192, LR_TOTAL, c->stream>>>(tx, tw, M, K, out64, c->status_dev);
  RT_COUNT_LAUNCH(1);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace rt
