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
  static constexpr uint32_t TOTAL = OFF_BAR + 256 + 1024;  // barriers, alignment slack
  static constexpr uint32_t TMEM_COLS = 256;               // S[2] (64 each) + O (hd <= 128)
  static constexpr uint32_t COL_S = 0, COL_O = 2 * BN;
};

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *(uint32_t*)&h;
}

template <int HD>
__global__ void __launch_bounds__(192, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const int* __restrict__ seq_start,
                   const int2* __restrict__ gap, int M, int nh, int nkv, float scale, __half* __restrict__ o,
                   float* __restrict__ lse, int* status) {
  using L = FwdLayout<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + 1023u) & ~1023u) - raw);  // 128-byte-swizzled tiles start on 1 KB boundaries
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
  const int m0 = blockIdx.x * BM, h = blockIdx.y, g = h / (nh / nkv);
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
      mbar_init(&s_free[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    mbar_fence_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *(volatile uint32_t*)tmem_slot;

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
    for (int n = 0; n < ntiles; ++n) {
      const int b = n & 1;
      const int n0 = kbeg + n * BN;
      if (!mbar_wait(&s_full[b], (uint32_t)(n >> 1) & 1, status, SITE_SFULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[BN];
      tmem_ld32(lane_addr + L::COL_S + b * BN, v);
      tmem_ld32(lane_addr + L::COL_S + b * BN + 32, v + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_free[b]);
      // a tile wholly below the diagonal of every row, inside every row's sequence, needs no mask
      const bool need_mask = (n0 + BN - 1 > m0) || (n0 < ss_last) || gap != nullptr;
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const int j = n0 + c;
          const bool valid = j <= i && j >= ss_i && (j < gp.x || j >= gp.y);
          const float s = valid ? __uint_as_float(v[c]) * sl2 : -INFINITY;
          v[c] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const float s = __uint_as_float(v[c]) * sl2;
          v[c] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      }
      const bool grow = mx > m_used + RESCALE_THRESHOLD;  // also the first tile that shows the row a key
      const float m_new = grow ? mx : m_used;
      const float corr = grow ? ex2_approx(m_used - m_new) : 1.0f;  // 0 when the row had seen nothing
      const float mref = m_new == -INFINITY ? 0.f : m_new;
      l_run *= corr;
      uint32_t ph[BN / 2];
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < BN; c += 2) {
        const float p0 = ex2_approx(__uint_as_float(v[c]) - mref), p1 = ex2_approx(__uint_as_float(v[c + 1]) - mref);
        sum += p0 + p1;
        ph[c >> 1] = pack_h2(p0, p1);
      }
      l_run += sum;
      m_used = m_new;
      // P's buffer is free, and O is at rest, once the previous tile's P.V has completed
      if (n > 0) {
        if (!mbar_wait(pv_done, (uint32_t)(n - 1) & 1, status, SITE_PVDONE)) { ok = false; break; }
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
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok && mbar_wait(pv_done, (uint32_t)(ntiles - 1) & 1, status, SITE_PVDONE)) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      __half* orow = o + ((size_t)i * nh + h) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t t[32];
        tmem_ld32(lane_addr + L::COL_O + c * 32, t);
        tmem_ld_wait();
        if (i < M) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 w;
            w.x = pack_h2(__uint_as_float(t[8 * k]) * inv, __uint_as_float(t[8 * k + 1]) * inv);
            w.y = pack_h2(__uint_as_float(t[8 * k + 2]) * inv, __uint_as_float(t[8 * k + 3]) * inv);
            w.z = pack_h2(__uint_as_float(t[8 * k + 4]) * inv, __uint_as_float(t[8 * k + 5]) * inv);
            w.w = pack_h2(__uint_as_float(t[8 * k + 6]) * inv, __uint_as_float(t[8 * k + 7]) * inv);
            *(uint4*)(orow + c * 32 + k * 8) = w;
          }
        }
      }
      if (i < M) lse[(size_t)h * M + i] = m_used / LOG2E + logf(l_run);
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
  CUtensorMap tq, tk, tv;
  if (tensor_map_f16_2d(c, &tq, q, (uint64_t)M, (uint64_t)nh * HD, 64, BM)) return 3;
  if (tensor_map_f16_2d(c, &tk, k, (uint64_t)M, (uint64_t)nkv * HD, 64, BN)) return 3;
  if (tensor_map_f16_2d(c, &tv, v, (uint64_t)M, (uint64_t)nkv * HD, 64, BN)) return 3;
  dim3 grid((M + BM - 1) / BM, nh);
  attn_fwd_tc_kernel<HD><<<grid, 192, L::TOTAL, c->stream>>>(tq, tk, tv, seq_start, gap, M, nh, nkv, 1.0f / sqrtf((float)HD), o,
                                                            lse, c->status_dev);
  RT_COUNT_LAUNCH(1);
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

}  // namespace rt
