// Causal grouped-query attention on the fifth-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   forward  (reference src/attention.rs:187-230): P = softmax(mask(q.k^T / sqrt(hd))), O = P.V
//
// One CTA owns 128 query rows of one head; a thread of the four softmax warps owns ONE row, which
// is one TMEM lane, so the row maximum and the row sum need no shuffles.  Per key tile of 64:
//   S = Q.K^T   tcgen05.mma, A = Q [128 x hd] and B = K [64 x hd] both K-major in shared memory
//               (TMA, 128-byte swizzle), D = S in TMEM (two buffers of 64 columns)
//   softmax     tcgen05.ld of the thread's row, mask, running maximum, p = 2^(s - m), P to shared
//               memory in f16 as the next product's A operand
//   O += P.V    tcgen05.mma, B = V [64 x hd] read MN-major from the tile TMA brought, D = O in TMEM
// The running maximum moves only when a row's new maximum exceeds it by more than 2^8 (p stays
// below 256, exact in f16's range); only then is O rescaled in TMEM (tcgen05.ld / st), which after
// the first tiles of a row almost never happens.  K and V tiles are double buffered; QK(n+1) is
// issued before the softmax of tile n, so the tensor core works under the exponentials.  Two CTAs
// fit an SM (112 KB of shared memory, 256 TMEM columns each) and cover each other's prologue.
//
// A batch is a concatenation of independent sequences: row i sees keys j with
// seq_start[i] <= j <= i and, when a gap array is given, j outside [gap[i].x, gap[i].y) (the
// reference's `allowed` rule for packed shared-prompt groups, src/ops.rs:156-164).
// Every wait is bounded and reports through the ctx status word.
#include "ctx.h"
#include "pdl.cuh"
#include "ptx.cuh"
#include <cuda_fp16.h>
#include <stdint.h>

namespace rt {

namespace {

constexpr int BM = 128;  // query rows per CTA (TMEM lanes)
constexpr int BN = 64;   // keys per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units the stale maximum may lag behind

// wait sites reported with RT_ERR_DEVICE_WAIT_TIMEOUT
enum { SITE_Q = 401, SITE_KFREE, SITE_VFREE, SITE_KFULL, SITE_SFREE, SITE_PFULL, SITE_VFULL, SITE_SFULL, SITE_PVDONE, SITE_END };

template <int HD>
struct FwdLayout {
  static constexpr int PAN = HD / 64;                    // 64-column panels per row
  static constexpr uint32_t Q_PANEL = BM * 128;          // bytes: [128 rows][64 f16]
  static constexpr uint32_t KV_PANEL = BN * 128;         // bytes: [64 rows][64 f16]
  static constexpr uint32_t Q_BYTES = PAN * Q_PANEL, KV_BYTES = PAN * KV_PANEL, P_BYTES = BM * 128;
  static constexpr uint32_t OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_P + P_BYTES;
  // Two CTAs must fit an SM's 228 KB (each also pays 1 KB of system shared memory), so the slack for
  // rounding the base up to a 1 KB boundary is 768 bytes: enough for any base that is 256-byte
  // aligned (the kernel checks, and reports a status instead of running, if it ever is not).
  static constexpr uint32_t USED = OFF_BAR + 256;
  static constexpr uint32_t TOTAL = USED + 768;
  static constexpr uint32_t TMEM_COLS = 256;               // S[2] (64 each) + O (hd <= 128)
  static constexpr uint32_t COL_S = 0, COL_O = 2 * BN;
};

// Timeline stamps of one CTA's first softmax thread, measurement builds only (-DRT_B200_QPROF).
#ifdef RT_B200_QPROF
__device__ unsigned long long g_attn_prof[512];
#define AT_STAMP(slot)                                                                     \
  do {                                                                                     \
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && (slot) < 512) g_attn_prof[(slot)] = globaltimer_ns(); \
  } while (0)
#ifndef RT_B200_ATTN_PROF_KERNEL
#define RT_B200_ATTN_PROF_KERNEL 0  // 0: forward, 1: dK/dV, 2: dQ
#endif
#else
#define AT_STAMP(slot) do { } while (0)
#define RT_B200_ATTN_PROF_KERNEL -1
#endif
#define AT_STAMP_F(slot) do { if (RT_B200_ATTN_PROF_KERNEL == 0) AT_STAMP(slot); } while (0)
#define AT_STAMP_K(slot) do { if (RT_B200_ATTN_PROF_KERNEL == 1) AT_STAMP(slot); } while (0)
#define AT_STAMP_Q(slot) do { if (RT_B200_ATTN_PROF_KERNEL == 2) AT_STAMP(slot); } while (0)

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *(uint32_t*)&h;
}

template <int HD>
__global__ void __launch_bounds__(192, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   const int* __restrict__ seq_start, const int2* __restrict__ gap, int M, int nh, int nkv, float scale,
                   float* __restrict__ lse, int* status) {
  using L = FwdLayout<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;  // 128-byte-swizzled tiles start on 1 KB boundaries
  pdl_launch_dependents();
  if (pad + L::USED > L::TOTAL) {
    pdl_wait();
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_CUDA);
    return;
  }
  uint8_t* sm = smem_raw + pad;
  uint64_t* bars = (uint64_t*)(sm + L::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* v_full = bars + 3;   // [2]
  uint64_t* k_free = bars + 5;   // [2]
  uint64_t* v_free = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* s_free = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* pv_done = bars + 14;
  uint32_t* tmem_slot = (uint32_t*)(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last query tiles of a sequence see the most keys: start them first
  const int m0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM, h = blockIdx.y, g = h / (nh / nkv);
  const int kbeg = seq_start[m0];
  const int kend = min(m0 + BM, M);
  const int ntiles = (kend - kbeg + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_free[i], 1);
      mbar_init(&v_free[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);   // one arrival per softmax warp
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_o);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  pdl_wait();  // seq_start, read above, is an input of the whole pass, not a predecessor's output

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, L::Q_BYTES);
      for (int p = 0; p < L::PAN; ++p) tma_load_2d(sm + L::OFF_Q + p * L::Q_PANEL, &tm_q, h * HD + p * 64, m0, q_full);
      for (int n = 0; n < ntiles; ++n) {
        const int b = n & 1;
        const uint32_t free_parity = ((n >> 1) & 1) ^ 1;  // the first use of a buffer finds it free
        const int n0 = kbeg + n * BN;
        if (!mbar_wait(&k_free[b], free_parity, status, SITE_KFREE)) break;
        mbar_expect_tx(&k_full[b], L::KV_BYTES);
        for (int p = 0; p < L::PAN; ++p)
          tma_load_2d(sm + L::OFF_K + b * L::KV_BYTES + p * L::KV_PANEL, &tm_k, g * HD + p * 64, n0, &k_full[b]);
        if (!mbar_wait(&v_free[b], free_parity, status, SITE_VFREE)) break;
        mbar_expect_tx(&v_full[b], L::KV_BYTES);
        for (int p = 0; p < L::PAN; ++p)
          tma_load_2d(sm + L::OFF_V + b * L::KV_BYTES + p * L::KV_PANEL, &tm_v, g * HD + p * 64, n0, &v_full[b]);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issue (one thread)
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(0, 0, 0, 0, BM, BN);   // S: A, B K-major, N = 64 keys
      const uint32_t idesc_o = umma_idesc(0, 0, 0, 1, BM, HD);   // O: A K-major (P), B MN-major (V), N = hd
      const uint32_t sQ = smem_u32(sm + L::OFF_Q), sK = smem_u32(sm + L::OFF_K), sV = smem_u32(sm + L::OFF_V), sP = smem_u32(sm + L::OFF_P);
      bool ok = mbar_wait(q_full, 0, status, SITE_Q);
      auto issue_qk = [&](int n) -> bool {
        const int b = n & 1;
        const uint32_t u = (uint32_t)(n >> 1) & 1;
        if (!mbar_wait(&k_full[b], u, status, SITE_KFULL)) return false;
        if (!mbar_wait(&s_free[b], u ^ 1, status, SITE_SFREE)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sQ + (kk >> 2) * L::Q_PANEL + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sK + b * L::KV_BYTES + (kk >> 2) * L::KV_PANEL + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + L::COL_S + b * BN, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(&s_full[b]);
        umma_commit(&k_free[b]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int n = 0; n < ntiles && ok; ++n) {
        if (n + 1 < ntiles && !issue_qk(n + 1)) { ok = false; break; }
        const int b = n & 1;
        if (!mbar_wait(p_full, (uint32_t)n & 1, status, SITE_PFULL)) { ok = false; break; }
        if (!mbar_wait(&v_full[b], (uint32_t)(n >> 1) & 1, status, SITE_VFULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sP + kk * 32, 16, 1024);
          // V tile: rows are keys (the contraction), 64-column panels L::KV_PANEL bytes apart are hd (N)
          const uint64_t bd = umma_desc_sw128(sV + b * L::KV_BYTES + kk * 2048, L::KV_PANEL, 1024);
          umma_f16(tmem_base + L::COL_O, ad, bd, idesc_o, (n | kk) != 0);
        }
        umma_commit(pv_done);
        umma_commit(&v_free[b]);
      }
      // the last arrivals of the tensor core on this CTA's barriers land before the CTA leaves
      if (ok) mbar_wait(&v_free[(ntiles - 1) & 1], (uint32_t)((ntiles - 1) >> 1) & 1, status, SITE_END);
    }
  } else {
    // ------------------------------------------------------------ softmax: thread = query row = TMEM lane
    const int r = warp * 32 + lane;
    const int i = m0 + r;
    const int ss_i = i < M ? seq_start[i] : 0x7fffffff;
    const int2 gp = (gap && i < M) ? gap[i] : make_int2(0, 0);
    const int ss_last = seq_start[kend - 1];  // the largest first-key index among the tile's rows
    const float sl2 = scale * LOG2E;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    AT_STAMP_F(0);
    for (int n = 0; n < ntiles; ++n) {
      const int b = n & 1;
      const int n0 = kbeg + n * BN;
      if (!mbar_wait(&s_full[b], (uint32_t)(n >> 1) & 1, status, SITE_SFULL)) { ok = false; break; }
      AT_STAMP_F(1 + 6 * n);
      tc_fence_after();
      uint32_t v[BN];
      tmem_ld32(lane_addr + L::COL_S + b * BN, v);
      tmem_ld32(lane_addr + L::COL_S + b * BN + 32, v + 32);
      tmem_ld_wait();
      AT_STAMP_F(2 + 6 * n);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[b]);
      // a tile wholly below the diagonal of every row, inside every row's sequence, needs no mask
      const bool need_mask = (n0 + BN - 1 > m0) || (n0 < ss_last);
      // four interleaved chains for the maximum and for the sum: a thread is alone on its row, so the
      // instruction-level parallelism has to come from inside the row
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask || gap != nullptr) {
        // valid keys of this row inside the tile: columns [c_lo, c_hi], minus the hidden range
        const int c_lo = ss_i - n0, c_hi = i - n0;
        const int g_lo = gp.x - n0, g_hi = gp.y - n0;
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const bool valid = c >= c_lo && c <= c_hi && (c < g_lo || c >= g_hi);
          const float s = valid ? __uint_as_float(v[c]) * sl2 : -INFINITY;
          v[c] = __float_as_uint(s);
          mx4[c & 3] = fmaxf(mx4[c & 3], s);
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const float s = __uint_as_float(v[c]) * sl2;
          v[c] = __float_as_uint(s);
          mx4[c & 3] = fmaxf(mx4[c & 3], s);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const bool grow = mx > m_used + RESCALE_THRESHOLD;  // also the first tile that shows the row a key
      const float m_new = grow ? mx : m_used;
      const float corr = grow ? ex2_approx(m_used - m_new) : 1.0f;  // 0 when the row had seen nothing
      const float mref = m_new == -INFINITY ? 0.f : m_new;
      l_run *= corr;
      uint32_t ph[BN / 2];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BN; c += 2) {
        const float p0 = ex2_approx(__uint_as_float(v[c]) - mref), p1 = ex2_approx(__uint_as_float(v[c + 1]) - mref);
        sum4[(c >> 1) & 3] += p0 + p1;
        ph[c >> 1] = pack_h2(p0, p1);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l_run += sum;
      m_used = m_new;
      // P's buffer is free, and O is at rest, once the previous tile's P.V has completed
      AT_STAMP_F(3 + 6 * n);
      if (n > 0) {
        if (!mbar_wait(pv_done, (uint32_t)(n - 1) & 1, status, SITE_PVDONE)) { ok = false; break; }
        AT_STAMP_F(4 + 6 * n);
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow && corr != 1.0f)) {
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t t[32];
            tmem_ld32(lane_addr + L::COL_O + c * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; ++k) t[k] = __float_as_uint(__uint_as_float(t[k]) * corr);
            tmem_st32(lane_addr + L::COL_O + c * 32, t);
          }
          tmem_st_wait();
        }
      }
      // row r of P: eight 16-byte chunks, chunk c at (c ^ (r & 7)) as the 128-byte swizzle places it
      uint8_t* prow = sm + L::OFF_P + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *(uint4*)(prow + ((c ^ (r & 7)) << 4)) = make_uint4(ph[4 * c], ph[4 * c + 1], ph[4 * c + 2], ph[4 * c + 3]);
      AT_STAMP_F(5 + 6 * n);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      AT_STAMP_F(6 + 6 * n);
    }
    AT_STAMP_F(500);
    if (ok && mbar_wait(pv_done, (uint32_t)(ntiles - 1) & 1, status, SITE_PVDONE)) {
      // O / l as f16 into Q's shared memory (every product that read Q has completed), in the
      // layout of a swizzled TMA box, then one bulk store per 64-column panel: rows past the end of
      // the batch are clipped by the tensor map
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t t[32];
        tmem_ld32(lane_addr + L::COL_O + c * 32, t);
        tmem_ld_wait();
        uint8_t* orow = sm + L::OFF_Q + (c >> 1) * L::Q_PANEL + r * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint4 w;
          w.x = pack_h2(__uint_as_float(t[8 * k]) * inv, __uint_as_float(t[8 * k + 1]) * inv);
          w.y = pack_h2(__uint_as_float(t[8 * k + 2]) * inv, __uint_as_float(t[8 * k + 3]) * inv);
          w.z = pack_h2(__uint_as_float(t[8 * k + 4]) * inv, __uint_as_float(t[8 * k + 5]) * inv);
          w.w = pack_h2(__uint_as_float(t[8 * k + 6]) * inv, __uint_as_float(t[8 * k + 7]) * inv);
          const int chunk = (c & 1) * 4 + k;
          *(uint4*)(orow + ((chunk ^ (r & 7)) << 4)) = w;
        }
      }
      if (i < M) lse[(size_t)h * M + i] = m_used / LOG2E + logf(l_run);
      fence_proxy_async_smem();
      named_barrier_sync(1, 128);  // the four softmax warps only
      if (threadIdx.x == 0) {
        for (int p = 0; p < L::PAN; ++p) tma_store_2d(&tm_o, h * HD + p * 64, m0, sm + L::OFF_Q + p * L::Q_PANEL);
        bulk_commit_group();
        bulk_wait_group_read<0>();  // shared memory may go once the store has read it
      }
      AT_STAMP_F(501);
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*(volatile int*)status != 0) {
    // a wait gave up somewhere: give copies already in flight time to land before shared memory goes away
    for (int k = 0; k < 1000; ++k) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <int HD>
int fwd_tc_impl(rt_ctx* c, const __half* q, const __half* k, const __half* v, const int* seq_start, const int2* gap, int M,
                int nh, int nkv, __half* o, float* lse) {
  using L = FwdLayout<HD>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::TOTAL) != cudaSuccess) return 3;
    attr = true;
  }
  CUtensorMap tq, tk, tv, to;
  if (tensor_map_f16_2d(c, &tq, q, (uint64_t)M, (uint64_t)nh * HD, 64, BM)) return 3;
  if (tensor_map_f16_2d(c, &to, o, (uint64_t)M, (uint64_t)nh * HD, 64, BM)) return 3;
  if (tensor_map_f16_2d(c, &tk, k, (uint64_t)M, (uint64_t)nkv * HD, 64, BN)) return 3;
  if (tensor_map_f16_2d(c, &tv, v, (uint64_t)M, (uint64_t)nkv * HD, 64, BN)) return 3;
  dim3 grid((M + BM - 1) / BM, nh);
  pdl(attn_fwd_tc_kernel<HD>, grid, 192, L::TOTAL, c->stream)(tq, tk, tv, to, seq_start, gap, M, nh, nkv, 1.0f / sqrtf((float)HD),
                                                            lse, c->status_dev);
  RT_COUNT_LAUNCH(1);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}


// ==================================================================== backward
//   (reference src/attention.rs:272-328)  dV = P^T.dO, dP = dO.V^T, dS = P*(dP - rowsum(P*dP))/sqrt(hd),
//   dQ = dS.K, dK = dS^T.Q, the K/V gradients summed over the query heads that share a KV head.
// Two kernels, so that every output element has exactly one writer (no float atomics: the same
// bits every run).  P is recomputed from the forward's log-sum-exp.  dO arrives as f16 rows
// divided by a per-row factor; a query row enters the sums over queries with weight
// factor / top (top = a power of two >= the largest factor, so the weights change no mantissa),
// and dQ rows get their own factor back.

// ------------------------------------------------------------------ dK, dV: one CTA per (128 keys, KV head)
// Thread = key row = TMEM lane.  K and V stay in shared memory; the (query head of the group) x
// (query tiles of 64 rows that can see these keys) work list streams through double buffers.
// Per item: S^T = K.Q^T and dP^T = V.dO^T into TMEM (two buffers each), the threads turn them
// into P^T and dS^T (f16, shared memory), then dV += P^T.dO and dK += dS^T.Q with Q and dO read
// MN-major from the same tiles.  TMEM: 2 x 64 + 2 x 64 + hd + hd columns (512 for hd = 128).
// P (<= 1, times a row weight <= 1) and dS are handed to the tensor cores in f16, whose normal
// range ends at 6e-5: attention probabilities of long rows and the gradients of lightly weighted
// rows live below that.  They are therefore stored times a power of two (exact), which the f32
// results are divided by again: 2^14 keeps P.w <= 16384, 2^10 keeps dS inside f16 for |dP - delta|
// up to ~700.
constexpr float P_BOOST = 16384.0f, DS_BOOST = 1024.0f;
constexpr int BQ = 64;  // query rows per work item
constexpr int BWD_THREADS = 320, BWD_TMA_WARP = 8, BWD_MMA_WARP = 9;  // warps 0-7 compute
enum { SITE_B_KV = 451, SITE_B_QFREE, SITE_B_QFULL, SITE_B_STFREE, SITE_B_PFULL, SITE_B_SFULL, SITE_B_PDDONE, SITE_B_END };

template <int HD>
struct DkvLayout {
  static constexpr int PAN = HD / 64;
  static constexpr uint32_t KV_PANEL = 128 * 128, Q_PANEL = BQ * 128;
  static constexpr uint32_t KV_BYTES = PAN * KV_PANEL, Q_BYTES = PAN * Q_PANEL, P_BYTES = 128 * 128;
  // Q, dO and the per-query vectors go through a ring of NS items: a slot is released by the item's
  // last product, so with three slots the fetch of item n+2 runs under all of item n+1
  static constexpr int NS = 3;
  static constexpr uint32_t OFF_K = 0, OFF_V = KV_BYTES, OFF_Q = 2 * KV_BYTES, OFF_DO = OFF_Q + NS * Q_BYTES;
  static constexpr uint32_t OFF_PT = OFF_DO + NS * Q_BYTES, OFF_DST = OFF_PT + P_BYTES, OFF_AUX = OFF_DST + P_BYTES;
  static constexpr uint32_t AUX_BYTES = 6 * BQ * 4;  // lse, delta, weight, seq_start, gap.x, gap.y per query row
  static constexpr uint32_t OFF_BAR = OFF_AUX + NS * AUX_BYTES;
  static constexpr uint32_t USED = OFF_BAR + 256, TOTAL = USED + 1024;
  static constexpr uint32_t COL_ST = 0, COL_DPT = 2 * BQ, COL_DV = 4 * BQ, COL_DK = 4 * BQ + HD;
  static constexpr uint32_t TMEM_COLS = 512;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                        const float* __restrict__ do_scale, const float* __restrict__ row_scale,
                        const float* __restrict__ lse, const float* __restrict__ delta, const int* __restrict__ seq_start,
                        const int2* __restrict__ gap, int M, int nh, int nkv, float scale, float* __restrict__ dk,
                        float* __restrict__ dv, int* status) {
  using L = DkvLayout<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  pdl_launch_dependents();
  uint64_t* bars = (uint64_t*)(sm + L::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;    // [NS] Q, dO and the per-query vectors of an item
  uint64_t* q_free = bars + 4;    // [NS]
  uint64_t* s_full = bars + 7;    // [2]  S^T and dP^T of an item are in TMEM
  uint64_t* st_free = bars + 9;   // [2]  ... and have been read
  uint64_t* p_full = bars + 11;   //      P^T and dS^T are in shared memory
  uint64_t* pd_done = bars + 12;  //      the item's dV, dK products have completed
  uint32_t* tmem_slot = (uint32_t*)(bars + 14);
  constexpr int NS = L::NS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128, g = blockIdx.y, group = nh / nkv;
  // queries that can see these keys: [n0, end of the sequence holding the tile's last key)
  const int last_key = min(n0 + 128, M) - 1;
  int qend;
  {
    const int ss_last = seq_start[last_key];
    int e = last_key + 1;
    while (e + 128 <= M && seq_start[e + 127] == ss_last) e += 128;
    while (e < M && seq_start[e] == ss_last) ++e;
    qend = e;
  }
  const int nqt = (qend - n0 + BQ - 1) / BQ;
  const int n_items = group * nqt;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&q_full[i], 2);  // the expect-tx arrival + the producer warp's arrival after the vectors
      mbar_init(&q_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&st_free[i], 8);  // one arrival per compute warp
    }
    mbar_init(p_full, 8);
    mbar_init(pd_done, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_do);
  }
  if (warp == BWD_MMA_WARP) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  pdl_wait();

  if (warp == BWD_TMA_WARP) {
    // ------------------------------------------------------------ producer: TMA + the per-query vectors
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * L::KV_BYTES);
      for (int p = 0; p < L::PAN; ++p) {
        tma_load_2d(sm + L::OFF_K + p * L::KV_PANEL, &tm_k, g * HD + p * 64, n0, kv_full);
        tma_load_2d(sm + L::OFF_V + p * L::KV_PANEL, &tm_v, g * HD + p * 64, n0, kv_full);
      }
    }
    for (int it = 0; it < n_items; ++it) {
      const int b = it % NS;
      const int h = g * group + it / nqt, m0 = n0 + (it % nqt) * BQ;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(&q_free[b], (((uint32_t)(it / NS)) & 1) ^ 1, status, SITE_B_QFREE);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&q_full[b], 2 * L::Q_BYTES);
        for (int p = 0; p < L::PAN; ++p) {
          tma_load_2d(sm + L::OFF_Q + b * L::Q_BYTES + p * L::Q_PANEL, &tm_q, h * HD + p * 64, m0, &q_full[b]);
          tma_load_2d(sm + L::OFF_DO + b * L::Q_BYTES + p * L::Q_PANEL, &tm_do, h * HD + p * 64, m0, &q_full[b]);
        }
      }
      float* aux = (float*)(sm + L::OFF_AUX + b * L::AUX_BYTES);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int il = lane + 32 * k, m = m0 + il;
        const bool in = m < M;
        aux[il] = in ? lse[(size_t)h * M + m] * LOG2E : 0.f;
        aux[BQ + il] = in ? delta[(size_t)h * M + m] : 0.f;
        // with per-row factors do_scale[m] is the largest factor (a power of two) of m's own sequence
        // and do_scale[M + m] the row's weight against it
        aux[2 * BQ + il] = in ? (row_scale ? do_scale[M + m] : 1.0f) * P_BOOST : 0.f;
        ((int*)aux)[3 * BQ + il] = in ? seq_start[m] : 0x7fffffff;
        const int2 gp = (gap && in) ? gap[m] : make_int2(0, 0);
        ((int*)aux)[4 * BQ + il] = gp.x;
        ((int*)aux)[5 * BQ + il] = gp.y;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[b]);  // (release: the warp's vectors are visible to whoever passes the barrier)
    }
  } else if (warp == BWD_MMA_WARP) {
    // ------------------------------------------------------------ MMA issue (one thread)
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(0, 0, 0, 0, 128, BQ);
      const uint32_t idesc_g = umma_idesc(0, 0, 0, 1, 128, HD);
      const uint32_t sK = smem_u32(sm + L::OFF_K), sV = smem_u32(sm + L::OFF_V), sQ = smem_u32(sm + L::OFF_Q);
      const uint32_t sDO = smem_u32(sm + L::OFF_DO), sPt = smem_u32(sm + L::OFF_PT), sDSt = smem_u32(sm + L::OFF_DST);
      bool ok = n_items == 0 || mbar_wait(kv_full, 0, status, SITE_B_KV);
      auto issue_s = [&](int it) -> bool {
        const int b = it & 1, rb = it % NS;  // TMEM buffer, ring slot
        const uint32_t u = ((uint32_t)it >> 1) & 1;
        if (!mbar_wait(&q_full[rb], (uint32_t)(it / NS) & 1, status, SITE_B_QFULL)) return false;
        if (!mbar_wait(&st_free[b], u ^ 1, status, SITE_B_STFREE)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sK + (kk >> 2) * L::KV_PANEL + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sQ + rb * L::Q_BYTES + (kk >> 2) * L::Q_PANEL + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + L::COL_ST + b * BQ, ad, bd, idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sV + (kk >> 2) * L::KV_PANEL + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sDO + rb * L::Q_BYTES + (kk >> 2) * L::Q_PANEL + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + L::COL_DPT + b * BQ, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(&s_full[b]);
        return true;
      };
      if (ok && n_items > 0) ok = issue_s(0);
      for (int it = 0; it < n_items && ok; ++it) {
        if (it + 1 < n_items && !issue_s(it + 1)) { ok = false; break; }
        const int b = it % NS;
        if (!mbar_wait(p_full, (uint32_t)it & 1, status, SITE_B_PFULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          // dO / Q tiles: rows are queries (the contraction), 64-column panels Q_PANEL bytes apart are hd (N)
          const uint64_t ap = umma_desc_sw128(sPt + kk * 32, 16, 1024);
          const uint64_t bo = umma_desc_sw128(sDO + b * L::Q_BYTES + kk * 2048, L::Q_PANEL, 1024);
          umma_f16(tmem_base + L::COL_DV, ap, bo, idesc_g, (it | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sDSt + kk * 32, 16, 1024);
          const uint64_t bq = umma_desc_sw128(sQ + b * L::Q_BYTES + kk * 2048, L::Q_PANEL, 1024);
          umma_f16(tmem_base + L::COL_DK, ad, bq, idesc_g, (it | kk) != 0);
        }
        umma_commit(pd_done);
        umma_commit(&q_free[b]);
      }
      if (ok && n_items > 0) mbar_wait(&q_free[(n_items - 1) % NS], (uint32_t)((n_items - 1) / NS) & 1, status, SITE_B_END);
    }
  } else {
    // ------------------------------------------------------------ eight warps: key row = TMEM lane, two threads per row
    // warps w and w + 4 read TMEM lane quarter w (a warp reaches the quarter warp % 4 only) and
    // take 32 of an item's 64 query columns each: two warps per scheduler hide each other's latencies
    const int quarter = warp & 3, hf = warp >> 2;
    const int r = quarter * 32 + lane;
    const int j = n0 + r;
    const float sl2 = scale * LOG2E;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    AT_STAMP_K(0);
    for (int it = 0; it < n_items; ++it) {
      const int b = it & 1;
      const int m0 = n0 + (it % nqt) * BQ;
      if (!mbar_wait(&s_full[b], ((uint32_t)it >> 1) & 1, status, SITE_B_SFULL)) { ok = false; break; }
      AT_STAMP_K(1 + 6 * it);
      // (completed long ago; passing it orders the producer lanes' per-query vectors before the reads below)
      if (!mbar_wait(&q_full[it % NS], (uint32_t)(it / NS) & 1, status, SITE_B_QFULL)) { ok = false; break; }
      tc_fence_after();
      const float* aux = (const float*)(sm + L::OFF_AUX + (it % NS) * L::AUX_BYTES);
      const int* auxi = (const int*)aux;
      // element (key row j, query column i): P^T (weighted) and dS^T
      uint32_t ph[16], dh[16];  // this thread's 32 columns
      // a tile whose queries all lie past these keys, inside one sequence, without hidden ranges, needs no mask
      const bool need_mask = (m0 < n0 + 127) || auxi[3 * BQ + BQ - 1] > n0;  // (rows past the batch carry INT_MAX)
      // 32 query columns at a time (fewer live registers), the per-query vectors fetched four at a
      // time with 128-bit shared loads ahead of their use: a thread is alone on its scheduler most
      // of the time, so one 32-bit shared load per use would put its latency on every element
      {
        uint32_t st[32], dp[32];
        tmem_ld32(lane_addr + L::COL_ST + b * BQ + hf * 32, st);
        tmem_ld32(lane_addr + L::COL_DPT + b * BQ + hf * 32, dp);
        tmem_ld_wait();
        AT_STAMP_K(2 + 6 * it);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&st_free[b]);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const int il0 = hf * 32 + c4 * 4;
          const float4 ls = *(const float4*)(aux + il0), de = *(const float4*)(aux + BQ + il0), wt = *(const float4*)(aux + 2 * BQ + il0);
          const float lsv[4] = {ls.x, ls.y, ls.z, ls.w}, dev[4] = {de.x, de.y, de.z, de.w}, wtv[4] = {wt.x, wt.y, wt.z, wt.w};
          float pv[4], dsv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            pv[e] = ex2_approx(__uint_as_float(st[c4 * 4 + e]) * sl2 - lsv[e]) * wtv[e];
          if (need_mask) {
            const int4 sq = *(const int4*)(auxi + 3 * BQ + il0);
            const int sqv[4] = {sq.x, sq.y, sq.z, sq.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) pv[e] = (j <= m0 + il0 + e && j >= sqv[e]) ? pv[e] : 0.f;
          }
          if (gap != nullptr) {
            const int4 ga = *(const int4*)(auxi + 4 * BQ + il0), gb = *(const int4*)(auxi + 5 * BQ + il0);
            const int gav[4] = {ga.x, ga.y, ga.z, ga.w}, gbv[4] = {gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) pv[e] = (j < gav[e] || j >= gbv[e]) ? pv[e] : 0.f;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) dsv[e] = pv[e] * (__uint_as_float(dp[c4 * 4 + e]) - dev[e]) * (scale * (DS_BOOST / P_BOOST));
          ph[2 * c4] = pack_h2(pv[0], pv[1]);
          ph[2 * c4 + 1] = pack_h2(pv[2], pv[3]);
          dh[2 * c4] = pack_h2(dsv[0], dsv[1]);
          dh[2 * c4 + 1] = pack_h2(dsv[2], dsv[3]);
        }
      }
      AT_STAMP_K(3 + 6 * it);
      if (it > 0) {
        if (!mbar_wait(pd_done, (uint32_t)(it - 1) & 1, status, SITE_B_PDDONE)) { ok = false; break; }
      }
      AT_STAMP_K(4 + 6 * it);
      uint8_t* prow = sm + L::OFF_PT + r * 128;
      uint8_t* drow = sm + L::OFF_DST + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // this thread's four 16-byte chunks of the row
        const int ch = hf * 4 + c;
        *(uint4*)(prow + ((ch ^ (r & 7)) << 4)) = make_uint4(ph[4 * c], ph[4 * c + 1], ph[4 * c + 2], ph[4 * c + 3]);
        *(uint4*)(drow + ((ch ^ (r & 7)) << 4)) = make_uint4(dh[4 * c], dh[4 * c + 1], dh[4 * c + 2], dh[4 * c + 3]);
      }
      AT_STAMP_K(5 + 6 * it);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      AT_STAMP_K(6 + 6 * it);
    }
    AT_STAMP_K(500);
    // write this key row's gradients (zeros when no query sees these keys)
    // a key row only ever meets queries of its own sequence, so its sums are in units of that sequence's largest factor
    const float top_j = row_scale ? do_scale[j < M ? j : M - 1] : do_scale[0];
    const float sc_v = top_j * (1.0f / P_BOOST), sc_k = top_j * (1.0f / DS_BOOST);
    if (n_items > 0 && ok) ok = mbar_wait(pd_done, (uint32_t)(n_items - 1) & 1, status, SITE_B_PDDONE);
    if (ok) {
      tc_fence_after();
      float* dkrow = dk + ((size_t)j * nkv + g) * HD;
      float* dvrow = dv + ((size_t)j * nkv + g) * HD;
#pragma unroll
      for (int cc = 0; cc < HD / 64; ++cc) {  // each of the row's two threads writes half of its columns
        const int c = hf * (HD / 64) + cc;
        uint32_t a[32], bb[32];
        if (n_items > 0) {
          tmem_ld32(lane_addr + L::COL_DK + c * 32, a);
          tmem_ld32(lane_addr + L::COL_DV + c * 32, bb);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) a[k] = bb[k] = 0u;
        }
        if (j < M) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            *(float4*)(dkrow + c * 32 + 4 * k) = make_float4(__uint_as_float(a[4 * k]) * sc_k, __uint_as_float(a[4 * k + 1]) * sc_k,
                                                             __uint_as_float(a[4 * k + 2]) * sc_k, __uint_as_float(a[4 * k + 3]) * sc_k);
            *(float4*)(dvrow + c * 32 + 4 * k) = make_float4(__uint_as_float(bb[4 * k]) * sc_v, __uint_as_float(bb[4 * k + 1]) * sc_v,
                                                             __uint_as_float(bb[4 * k + 2]) * sc_v, __uint_as_float(bb[4 * k + 3]) * sc_v);
          }
        }
      }
    }
  }

  if (*(volatile int*)status != 0) {
    for (int k = 0; k < 1000; ++k) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BWD_MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ dQ: one CTA per (128 query rows, head)
// Thread = query row = TMEM lane.  Q and dO stay in shared memory; per key tile of 64:
// S = Q.K^T and dP = dO.V^T into TMEM, dS = P*(dP - delta)*scale to shared memory in f16, then
// dQ += dS.K with K read MN-major from the tile that just served Q.K^T.  K and V tiles go through
// a ring of three slots (a K slot is released by the tile's dQ product, so the fetch of tile n+2
// runs under all of tile n+1); S and dP have two TMEM buffers each and are issued one tile ahead.
enum { SITE_Q_QDO = 471, SITE_Q_KFREE, SITE_Q_VFREE, SITE_Q_KFULL, SITE_Q_VFULL, SITE_Q_SFREE, SITE_Q_DSFULL, SITE_Q_SFULL, SITE_Q_DQDONE, SITE_Q_END };

template <int HD>
struct DqLayout {
  static constexpr int PAN = HD / 64;
  static constexpr uint32_t Q_PANEL = BM * 128, KV_PANEL = BN * 128;
  static constexpr uint32_t Q_BYTES = PAN * Q_PANEL, KV_BYTES = PAN * KV_PANEL, DS_BYTES = BM * 128;
  static constexpr int NS = 3;
  static constexpr uint32_t OFF_Q = 0, OFF_DO = Q_BYTES, OFF_K = 2 * Q_BYTES, OFF_V = OFF_K + NS * KV_BYTES, OFF_DS = OFF_V + NS * KV_BYTES;
  static constexpr uint32_t OFF_BAR = OFF_DS + DS_BYTES;
  static constexpr uint32_t USED = OFF_BAR + 256, TOTAL = USED + 1024;
  static constexpr uint32_t COL_S = 0, COL_DP = 2 * BN, COL_DQ = 4 * BN, TMEM_COLS = 512;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const float* __restrict__ do_scale, const float* __restrict__ row_scale, const float* __restrict__ lse,
                      const float* __restrict__ delta, const int* __restrict__ seq_start, const int2* __restrict__ gap, int M,
                      int nh, int nkv, float scale, float* __restrict__ dq, int* status) {
  using L = DqLayout<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  pdl_launch_dependents();
  uint64_t* bars = (uint64_t*)(sm + L::OFF_BAR);
  constexpr int NS = L::NS;
  uint64_t* qdo_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [NS]
  uint64_t* v_full = bars + 4;    // [NS]
  uint64_t* k_free = bars + 7;    // [NS]
  uint64_t* v_free = bars + 10;   // [NS]
  uint64_t* s_full = bars + 13;   // [2]
  uint64_t* s_free = bars + 15;   // [2]
  uint64_t* ds_full = bars + 17;
  uint64_t* dq_done = bars + 18;
  uint32_t* tmem_slot = (uint32_t*)(bars + 20);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last query tiles of a sequence see the most keys: start them first
  const int m0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM, h = blockIdx.y, g = h / (nh / nkv);
  const int kbeg = seq_start[m0];
  const int kend = min(m0 + BM, M);
  const int ntiles = (kend - kbeg + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_free[i], 1);
      mbar_init(&v_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 8);
    }
    mbar_init(ds_full, 8);
    mbar_init(dq_done, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  if (warp == BWD_MMA_WARP) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  AT_STAMP_Q(510);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;
  pdl_wait();
  AT_STAMP_Q(511);

  if (warp == BWD_TMA_WARP) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 2 * L::Q_BYTES);
      for (int p = 0; p < L::PAN; ++p) {
        tma_load_2d(sm + L::OFF_Q + p * L::Q_PANEL, &tm_q, h * HD + p * 64, m0, qdo_full);
        tma_load_2d(sm + L::OFF_DO + p * L::Q_PANEL, &tm_do, h * HD + p * 64, m0, qdo_full);
      }
      for (int n = 0; n < ntiles; ++n) {
        const int rb = n % NS;
        const uint32_t free_parity = ((uint32_t)(n / NS) & 1) ^ 1;
        const int n0 = kbeg + n * BN;
        if (!mbar_wait(&v_free[rb], free_parity, status, SITE_Q_VFREE)) break;
        mbar_expect_tx(&v_full[rb], L::KV_BYTES);
        for (int p = 0; p < L::PAN; ++p)
          tma_load_2d(sm + L::OFF_V + rb * L::KV_BYTES + p * L::KV_PANEL, &tm_v, g * HD + p * 64, n0, &v_full[rb]);
        if (!mbar_wait(&k_free[rb], free_parity, status, SITE_Q_KFREE)) break;
        mbar_expect_tx(&k_full[rb], L::KV_BYTES);
        for (int p = 0; p < L::PAN; ++p)
          tma_load_2d(sm + L::OFF_K + rb * L::KV_BYTES + p * L::KV_PANEL, &tm_k, g * HD + p * 64, n0, &k_full[rb]);
      }
    }
  } else if (warp == BWD_MMA_WARP) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(0, 0, 0, 0, BM, BN);
      const uint32_t idesc_g = umma_idesc(0, 0, 0, 1, BM, HD);
      const uint32_t sQ = smem_u32(sm + L::OFF_Q), sDO = smem_u32(sm + L::OFF_DO), sK = smem_u32(sm + L::OFF_K);
      const uint32_t sV = smem_u32(sm + L::OFF_V), sDS = smem_u32(sm + L::OFF_DS);
      bool ok = mbar_wait(qdo_full, 0, status, SITE_Q_QDO);
      auto issue_s = [&](int n) -> bool {
        const int b = n & 1, rb = n % NS;  // TMEM buffer, ring slot
        const uint32_t rph = (uint32_t)(n / NS) & 1;
        if (!mbar_wait(&k_full[rb], rph, status, SITE_Q_KFULL) || !mbar_wait(&v_full[rb], rph, status, SITE_Q_VFULL) ||
            !mbar_wait(&s_free[b], (((uint32_t)n >> 1) & 1) ^ 1, status, SITE_Q_SFREE))
          return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sDO + (kk >> 2) * L::Q_PANEL + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sV + rb * L::KV_BYTES + (kk >> 2) * L::KV_PANEL + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + L::COL_DP + b * BN, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(&v_free[rb]);  // V served dP only
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sQ + (kk >> 2) * L::Q_PANEL + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sK + rb * L::KV_BYTES + (kk >> 2) * L::KV_PANEL + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + L::COL_S + b * BN, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(&s_full[b]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int n = 0; n < ntiles && ok; ++n) {
        if (n + 1 < ntiles && !issue_s(n + 1)) { ok = false; break; }
        const int rb = n % NS;
        if (!mbar_wait(ds_full, (uint32_t)n & 1, status, SITE_Q_DSFULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t ad = umma_desc_sw128(sDS + kk * 32, 16, 1024);
          const uint64_t bd = umma_desc_sw128(sK + rb * L::KV_BYTES + kk * 2048, L::KV_PANEL, 1024);  // K tile read MN-major: rows are keys
          umma_f16(tmem_base + L::COL_DQ, ad, bd, idesc_g, (n | kk) != 0);
        }
        umma_commit(dq_done);
        umma_commit(&k_free[rb]);
      }
      if (ok) mbar_wait(&k_free[(ntiles - 1) % NS], (uint32_t)((ntiles - 1) / NS) & 1, status, SITE_Q_END);
    }
  } else {
    // eight warps: warps w and w + 4 share TMEM lane quarter w and take 32 of a tile's 64 key columns each
    const int quarter = warp & 3, hf = warp >> 2;
    const int r = quarter * 32 + lane;
    const int i = m0 + r;
    const int ss_i = i < M ? seq_start[i] : 0x7fffffff;
    const int2 gp = (gap && i < M) ? gap[i] : make_int2(0, 0);
    const int ss_last = seq_start[kend - 1];
    const float l2 = i < M ? lse[(size_t)h * M + i] * LOG2E : 0.f;
    const float dl = i < M ? delta[(size_t)h * M + i] : 0.f;
    const float sl2 = scale * LOG2E;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    AT_STAMP_Q(0);
    for (int n = 0; n < ntiles; ++n) {
      const int b = n & 1;
      const int n0 = kbeg + n * BN;
      if (!mbar_wait(&s_full[b], ((uint32_t)n >> 1) & 1, status, SITE_Q_SFULL)) { ok = false; break; }
      AT_STAMP_Q(1 + 6 * n);
      tc_fence_after();
      const bool need_mask = (n0 + BN - 1 > m0) || (n0 < ss_last);
      const int c_lo = ss_i - n0, c_hi = i - n0, g_lo = gp.x - n0, g_hi = gp.y - n0;
      uint32_t dh[16];  // this thread's 32 columns
      {
        uint32_t sv[32], dp[32];
        tmem_ld32(lane_addr + L::COL_S + b * BN + hf * 32, sv);
        tmem_ld32(lane_addr + L::COL_DP + b * BN + hf * 32, dp);
        tmem_ld_wait();
        AT_STAMP_Q(2 + 6 * n);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[b]);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float dsv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int cc = hf * 32 + c + e;
            float p = ex2_approx(__uint_as_float(sv[c + e]) * sl2 - l2);
            if (need_mask) p = (cc >= c_lo && cc <= c_hi) ? p : 0.f;
            if (gap != nullptr) p = (cc < g_lo || cc >= g_hi) ? p : 0.f;
            dsv[e] = p * (__uint_as_float(dp[c + e]) - dl) * (scale * DS_BOOST);
          }
          dh[c >> 1] = pack_h2(dsv[0], dsv[1]);
        }
      }
      AT_STAMP_Q(3 + 6 * n);
      if (n > 0) {
        if (!mbar_wait(dq_done, (uint32_t)(n - 1) & 1, status, SITE_Q_DQDONE)) { ok = false; break; }
      }
      AT_STAMP_Q(4 + 6 * n);
      uint8_t* drow = sm + L::OFF_DS + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int ch = hf * 4 + c;
        *(uint4*)(drow + ((ch ^ (r & 7)) << 4)) = make_uint4(dh[4 * c], dh[4 * c + 1], dh[4 * c + 2], dh[4 * c + 3]);
      }
      AT_STAMP_Q(5 + 6 * n);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      AT_STAMP_Q(6 + 6 * n);
    }
    AT_STAMP_Q(500);
    if (ok && mbar_wait(dq_done, (uint32_t)(ntiles - 1) & 1, status, SITE_Q_DQDONE)) {
      tc_fence_after();
      // a query row's gradient carries only that row's factor
      const float sc = (row_scale ? (i < M ? row_scale[i] : 0.f) : do_scale[0]) * (1.0f / DS_BOOST);
      float* qrow = dq + ((size_t)i * nh + h) * HD;
#pragma unroll
      for (int cc = 0; cc < HD / 64; ++cc) {
        const int c = hf * (HD / 64) + cc;
        uint32_t a[32];
        tmem_ld32(lane_addr + L::COL_DQ + c * 32, a);
        tmem_ld_wait();
        if (i < M) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            *(float4*)(qrow + c * 32 + 4 * k) = make_float4(__uint_as_float(a[4 * k]) * sc, __uint_as_float(a[4 * k + 1]) * sc,
                                                            __uint_as_float(a[4 * k + 2]) * sc, __uint_as_float(a[4 * k + 3]) * sc);
        }
      }
      AT_STAMP_Q(501);
    }
  }

  if (*(volatile int*)status != 0) {
    for (int k = 0; k < 1000; ++k) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BWD_MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

// delta[h, m] = sum_d O * dO (the row sum of P * dP, src/attention.rs:282-287).  A pure stream:
// HD / 8 lanes share a row with one 16-byte load of each operand per lane, four rows per lane
// group in flight.
template <int HD>
__global__ void attn_delta_tc_kernel(const __half* __restrict__ o, const __half* __restrict__ dO, int M, int nh,
                                     float* __restrict__ delta) {
  pdl_entry();
  constexpr int LPR = HD / 8, RPW = 32 / LPR, UN = 4;
  const int lane = threadIdx.x & 31, sub = lane % LPR, grp = lane / LPR;
  const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long total = (long long)M * nh, row0 = wg * (UN * RPW) + grp;
  uint4 av[UN], bv[UN];
#pragma unroll
  for (int u = 0; u < UN; ++u) {
    const long long r = row0 + u * RPW;
    if (r < total) {
      av[u] = *(const uint4*)(o + r * HD + sub * 8);
      bv[u] = *(const uint4*)(dO + r * HD + sub * 8);
    } else {
      av[u] = bv[u] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
#pragma unroll
  for (int u = 0; u < UN; ++u) {
    const __half2* a2 = (const __half2*)&av[u];
    const __half2* b2 = (const __half2*)&bv[u];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = __half22float2(a2[k]), y = __half22float2(b2[k]);
      s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    const long long r = row0 + u * RPW;
    if (sub == 0 && r < total) delta[(size_t)(r % nh) * M + (size_t)(r / nh)] = s;
  }
}

template <int HD>
int bwd_tc_impl(rt_ctx* c, const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO,
                const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int2* gap, int M,
                int nh, int nkv, float* delta, float* dq, float* dk, float* dv) {
  using LK = DkvLayout<HD>;
  using LQ = DqLayout<HD>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_dkdv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LK::TOTAL) != cudaSuccess) return 3;
    if (cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LQ::TOTAL) != cudaSuccess) return 3;
    attr = true;
  }
  CUtensorMap tq128, tdo128, tk64, tv64, tk128, tv128, tq64, tdo64;
  if (tensor_map_f16_2d(c, &tq128, q, (uint64_t)M, (uint64_t)nh * HD, 64, 128)) return 3;
  if (tensor_map_f16_2d(c, &tdo128, dO, (uint64_t)M, (uint64_t)nh * HD, 64, 128)) return 3;
  if (tensor_map_f16_2d(c, &tq64, q, (uint64_t)M, (uint64_t)nh * HD, 64, 64)) return 3;
  if (tensor_map_f16_2d(c, &tdo64, dO, (uint64_t)M, (uint64_t)nh * HD, 64, 64)) return 3;
  if (tensor_map_f16_2d(c, &tk128, k, (uint64_t)M, (uint64_t)nkv * HD, 64, 128)) return 3;
  if (tensor_map_f16_2d(c, &tv128, v, (uint64_t)M, (uint64_t)nkv * HD, 64, 128)) return 3;
  if (tensor_map_f16_2d(c, &tk64, k, (uint64_t)M, (uint64_t)nkv * HD, 64, 64)) return 3;
  if (tensor_map_f16_2d(c, &tv64, v, (uint64_t)M, (uint64_t)nkv * HD, 64, 64)) return 3;
  const float scale = 1.0f / sqrtf((float)HD);
  cudaStream_t st = c->stream;
  // one warp takes 4 passes of 32 / (HD / 8) rows
  const long long delta_warps = ((long long)M * nh + (4 * 32 / (HD / 8)) - 1) / (4 * 32 / (HD / 8));
  pdl(attn_delta_tc_kernel<HD>, (unsigned)((delta_warps * 32 + 255) / 256), 256, 0, st)(o, dO, M, nh, delta);
  dim3 gkv((M + 127) / 128, nkv), gq((M + BM - 1) / BM, nh);
  pdl(attn_bwd_dkdv_tc_kernel<HD>, gkv, BWD_THREADS, LK::TOTAL, st)(tk128, tv128, tq64, tdo64, do_scale, row_scale, lse, delta, seq_start, gap,
                                                          M, nh, nkv, scale, dk, dv, c->status_dev);
  pdl(attn_bwd_dq_tc_kernel<HD>, gq, BWD_THREADS, LQ::TOTAL, st)(tq128, tdo128, tk64, tv64, do_scale, row_scale, lse, delta, seq_start, gap, M,
                                                       nh, nkv, scale, dq, c->status_dev);
  RT_COUNT_LAUNCH(3);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace

int launch_attn_fwd_tc(rt_ctx* c, const __half* q, const __half* k, const __half* v, const int* seq_start, const int* gap, int M,
                       int nh, int nkv, int hd, __half* o, float* lse) {
  if (M <= 0) return 0;
  if (hd == 128) return fwd_tc_impl<128>(c, q, k, v, seq_start, (const int2*)gap, M, nh, nkv, o, lse);
  if (hd == 64) return fwd_tc_impl<64>(c, q, k, v, seq_start, (const int2*)gap, M, nh, nkv, o, lse);
  return 1;
}

#ifdef RT_B200_QPROF
extern "C" int rt_debug_attn_prof(unsigned long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_attn_prof, sizeof(unsigned long long) * (n < 512 ? n : 512));
}
#endif

int launch_attn_bwd_tc(rt_ctx* c, const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO16,
                       const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int* gap,
                       int M, int nh, int nkv, int hd, float* delta, float* dq, float* dk, float* dv) {
  if (M <= 0) return 0;
  if (hd == 128) return bwd_tc_impl<128>(c, q, k, v, o, dO16, do_scale, row_scale, lse, seq_start, (const int2*)gap, M, nh, nkv, delta, dq, dk, dv);
  if (hd == 64) return bwd_tc_impl<64>(c, q, k, v, o, dO16, do_scale, row_scale, lse, seq_start, (const int2*)gap, M, nh, nkv, delta, dq, dk, dv);
  return 1;
}

}  // namespace rt
