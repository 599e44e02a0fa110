// LoRA gradients of one linear (or of a stacked group) as token contractions on tcgen05
// (reference src/linear.rs:105-117):
//
//   dB[n, i] = sum_m dY[m, n] * Hs[m, i]      dA[i, k] = sum_m Gs[m, i] * X[m, k]
//
// Both are  part[split][i, c] = sum_{m in split} Small[m, i] * Big[m, c]  with Big = dY or X
// ([M x C], read ONCE: the kernel is a stream over Big) and Small = Hs or Gs ([M x 64]).  One CTA
// takes 128 columns of Big and a FIXED range of tokens; the tokens are the MMA's K dimension, so
// both operands are read MN-major straight from their row-major tiles:
//   A = Big tile   [64 tokens][128 columns]  (two swizzled panels of 64 columns, TMA)
//   B = Small tile [64 tokens][64]           (TMA, then scaled in place, see below)
//   D[column (lane), i] in 64 TMEM columns.
// Warps: 0-3 scale the Small tiles and run the epilogue, 4, 6, 7 are TMA producers, 5 issues the MMAs.
// dY arrives row-normalised with one factor per token.  The factors go onto the Small rows
// relative to the split's largest factor (rounded up to a power of two, so what a row rounds to
// does not depend on its split mates), and the largest factor multiplies the split's sums.
// Partial sums of the splits are added in order by the reduce kernels of lora_kernels.cu:
// deterministic, no atomics.
#include "ctx.h"
#include "ops.h"
#include "pdl.cuh"
#include "ptx.cuh"
#include "rt_internal.h"
#include <cuda_fp16.h>
#include <stdint.h>

namespace rt {

namespace {

constexpr int LG_NS = 4;
constexpr uint32_t LG_Q_BYTES = 2 * 64 * 128, LG_P_BYTES = 64 * 128, LG_STAGE = LG_Q_BYTES + LG_P_BYTES;
constexpr uint32_t LG_OFF_SCALE = LG_NS * LG_STAGE;         // factors of this split's tokens / largest
constexpr int LG_MAX_TPS = 1024;
constexpr uint32_t LG_OFF_BAR = LG_OFF_SCALE + LG_MAX_TPS * 4;
constexpr uint32_t LG_TOTAL = LG_OFF_BAR + 256 + 1024;
enum { SITE_LG_FREE = 495, SITE_LG_FULL, SITE_LG_READY, SITE_LG_DONE };

struct LoraGradTcArgs {
  const float* pscale;  // [M] or null
  int M, N, K, r, nbB, tps;
  float* partB;  // [splits][r x N]
  float* partA;  // [splits][r x K]
};

__global__ void __launch_bounds__(256, 2)
lora_grads_tc_kernel(const __grid_constant__ CUtensorMap tm_pb, const __grid_constant__ CUtensorMap tm_qb,
                     const __grid_constant__ CUtensorMap tm_pa, const __grid_constant__ CUtensorMap tm_qa,
                     const LoraGradTcArgs g, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  float* s_scale = (float*)(sm + LG_OFF_SCALE);
  uint64_t* bars = (uint64_t*)(sm + LG_OFF_BAR);
  uint64_t* full = bars;               // [NS] TMA landed
  uint64_t* ready = bars + LG_NS;      // [NS] Small tile scaled
  uint64_t* empty = bars + 2 * LG_NS;  // [NS] MMAs retired
  uint64_t* done = bars + 3 * LG_NS;
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * LG_NS + 2);
  __shared__ float s_red[4];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool isB = (int)blockIdx.x < g.nbB;
  const CUtensorMap* tm_p = isB ? &tm_pb : &tm_pa;
  const CUtensorMap* tm_q = isB ? &tm_qb : &tm_qa;
  const int C = isB ? g.N : g.K;
  const int j0 = (isB ? (int)blockIdx.x : (int)blockIdx.x - g.nbB) * 128;
  const int m_begin = blockIdx.y * g.tps, m_end = min(g.M, m_begin + g.tps);
  const int nchunks = (m_end - m_begin + 63) / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < LG_NS; ++i) {
      mbar_init(&full[i], 3);  // three producer threads
      mbar_init(&ready[i], 4);
      mbar_init(&empty[i], 1);
    }
    mbar_init(done, 1);
    mbar_fence_init();
    prefetch_tmap(tm_p);
    prefetch_tmap(tm_q);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  pdl_wait();

  if (warp == 4 || warp >= 6) {
    // three producer threads, one TMA instruction per stage each (an instruction costs its thread about 0.1 us)
    if (lane == 0) {
      const int which = warp == 4 ? 0 : warp - 5;  // 0, 1: the two 64-column panels of Big; 2: the Small tile
      for (int ch = 0; ch < nchunks; ++ch) {
        const int s = ch % LG_NS;
        if (!mbar_wait(&empty[s], (((uint32_t)(ch / LG_NS)) & 1) ^ 1, status, SITE_LG_FREE)) break;
        const int mrow = m_begin + ch * 64;
        mbar_expect_tx(&full[s], 8192);
        if (which == 2) tma_load_2d(sm + s * LG_STAGE + LG_Q_BYTES, tm_p, 0, mrow, &full[s]);
        else tma_load_2d(sm + s * LG_STAGE + which * 8192, tm_q, j0 + which * 64, mrow, &full[s]);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(0, 0, 1, 1, 128, 64);
      const uint32_t s0 = smem_u32(sm);
      bool ok = true;
      for (int ch = 0; ch < nchunks && ok; ++ch) {
        const int s = ch % LG_NS;
        if (!mbar_wait(&ready[s], ((uint32_t)(ch / LG_NS)) & 1, status, SITE_LG_READY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ad = umma_desc_sw128(s0 + s * LG_STAGE + kk * 2048, 8192, 1024);
          const uint64_t bd = umma_desc_sw128(s0 + s * LG_STAGE + LG_Q_BYTES + kk * 2048, 8192, 1024);
          umma_f16(tmem_base, ad, bd, idesc, (ch | kk) != 0);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(done);
    }
  } else {
    // ---- 128 threads: factors of the split, Small tiles scaled in place, then the epilogue
    const int tid = threadIdx.x;
    // out_mul: what the split's sums are multiplied by at the end (the split's largest factor)
    float out_mul = 1.0f;
    if (g.pscale) {
      // Largest factor of the split (factors are >= 0), rounded up to a power of two so that
      // dividing by it changes no mantissa.  (Lifting the rows further, to the top of f16's range by
      // the largest magnitude of the split's Small rows, was tried: it needs a pass over those
      // rows before the first tile can be scaled, 6 us of a 22 us launch, and changed no digit of
      // the shards-against-whole-batch check once the attention backward weighed rows per sequence.)
      float v = 0.f;
      for (int m = m_begin + tid; m < m_end; m += 128) v = fmaxf(v, g.pscale[m]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) s_red[warp] = v;
      named_barrier_sync(1, 128);
      float lmax = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
      lmax = __int_as_float((__float_as_int(lmax) + 0x007FFFFF) & 0x7F800000);
      const float inv = lmax > 0.f ? 1.0f / lmax : 0.f;
      out_mul = lmax;
      for (int m = tid; m < nchunks * 64; m += 128) s_scale[m] = (m_begin + m < m_end) ? g.pscale[m_begin + m] * inv : 0.f;
      named_barrier_sync(1, 128);
    }
    bool ok = true;
    for (int ch = 0; ch < nchunks && ok; ++ch) {
      const int s = ch % LG_NS;
      if (!mbar_wait(&full[s], ((uint32_t)(ch / LG_NS)) & 1, status, SITE_LG_FULL)) { ok = false; break; }
      if (g.pscale) {
        uint8_t* pt = sm + s * LG_STAGE + LG_Q_BYTES;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int e = tid + k * 128;  // 16-byte unit; its token row is e / 8 whatever the swizzle
          const float f = s_scale[ch * 64 + (e >> 3)];
          uint4* ptr = (uint4*)(pt + e * 16);
          uint4 v = *ptr;
          __half2* h2 = (__half2*)&v;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 x = __half22float2(h2[q]);
            h2[q] = __floats2half2_rn(x.x * f, x.y * f);
          }
          *ptr = v;
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ready[s]);
    }
    if (ok && mbar_wait(done, 0, status, SITE_LG_DONE)) {
      tc_fence_after();
      uint32_t v[64];
      tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16), v);
      if (g.r > 32) tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + 32, v + 32);
      tmem_ld_wait();
      const int j = j0 + warp * 32 + lane;
      if (j < C) {
        float* dst = (isB ? g.partB : g.partA) + (size_t)blockIdx.y * g.r * C + j;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < g.r) dst[(size_t)i * C] = __uint_as_float(v[i]) * out_mul;
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

// Tokens per split of the tcgen05 contraction: fixed by the token count's range only.
int lora_grads_tc_tokens_per_split(int M) { return M >= 4096 ? 1024 : M >= 1024 ? 256 : M >= 512 ? 128 : 64; }

// Launches the product kernel only (the caller adds the splits).  partB / partA: [splits][r x N] / [splits][r x K]
// with splits = ceil(M / lora_grads_tc_tokens_per_split(M)).  0: launched; 1: shape not covered; 3: launch failure.
int launch_lora_grads_tc(rt_ctx* c, const __half* hs, const __half* dy16, int ld_dy, const __half* gs, const __half* x16,
                         const float* dscale, int M, int N, int K, int r, float* partB, float* partA) {
  if (M <= 0) return 0;
  if (r <= 0 || r > 64 || N % 8 != 0 || K % 8 != 0 || ld_dy % 8 != 0) return 1;
  if (((uintptr_t)hs | (uintptr_t)dy16 | (uintptr_t)gs | (uintptr_t)x16) & 15) return 1;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(lora_grads_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LG_TOTAL) != cudaSuccess) return 3;
    attr = true;
  }
  CUtensorMap tpb, tqb, tpa, tqa;
  if (tensor_map_f16_2d_ld(c, &tpb, hs, (uint64_t)M, 64, 64, 64, 64)) return 3;
  if (tensor_map_f16_2d_ld(c, &tqb, dy16, (uint64_t)M, (uint64_t)N, (uint64_t)ld_dy, 64, 64)) return 3;
  if (tensor_map_f16_2d_ld(c, &tpa, gs, (uint64_t)M, 64, 64, 64, 64)) return 3;
  if (tensor_map_f16_2d_ld(c, &tqa, x16, (uint64_t)M, (uint64_t)K, (uint64_t)K, 64, 64)) return 3;
  LoraGradTcArgs g;
  g.pscale = dscale;
  g.M = M; g.N = N; g.K = K; g.r = r;
  g.nbB = (N + 127) / 128;
  g.tps = lora_grads_tc_tokens_per_split(M);
  g.partB = partB;
  g.partA = partA;
  const int splits = (M + g.tps - 1) / g.tps;
  dim3 grid(g.nbB + (K + 127) / 128, splits);
  pdl(lora_grads_tc_kernel, grid, 256, LG_TOTAL, c->stream)(tpb, tqb, tpa, tqa, g, c->status_dev);
  RT_COUNT_LAUNCH(1);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace rt
