// Causal grouped-query attention, forward and backward, flash style: the [T x T] probability
// matrix the reference stores (src/attention.rs:138,232) is never materialised; the forward
// keeps one log-sum-exp per (head, row) and the backward recomputes P from it.
//
//   forward  (reference src/attention.rs:187-230): P = softmax(mask(q.k^T / sqrt(hd))), O = P.V
//   backward (reference src/attention.rs:272-328): dV = P^T.dO, dP = dO.V^T,
//            dS = P*(dP - rowsum(P*dP))/sqrt(hd), dQ = dS.K, dK = dS^T.Q, summed over the
//            query heads that share a KV head
//
// A batch is a concatenation of independent sequences; row i attends to keys j with
// seq_start[i] <= j <= i and, when a gap array is given, j outside [gap[i].x, gap[i].y) (the other
// examples' own tokens of a shared-prompt group), which is the reference's `allowed` rule (src/ops.rs:156-164) for
// unpacked sequences.  K and V arrive already rounded to f16, as the reference's f16 KV view
// has them (src/attention.rs:180-185); Q, P and dS are rounded to f16 for the tensor cores,
// all sums are f32.  The backward is two kernels (dK/dV per key tile, dQ per query tile) so
// that every output element is written by exactly one thread: no float atomics, same result
// every run.
#include "ops.h"
#include "rt_internal.h"
#include <cuda_fp16.h>
#include <stdint.h>

namespace rt {

namespace {

constexpr int BT = 64;  // tile rows (queries or keys)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Tile of BT rows x HD halves, 16-byte chunks XOR-swizzled by row so ldmatrix is conflict free.
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // size 0: nothing is read, the 16 bytes are zero filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// all but the most recent group have landed
__device__ __forceinline__ void cp_async_wait_prev() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// rows [row0, row0+BT) of a [M x heads x HD] tensor, one head, into a swizzled tile
template <int HD>
__device__ __forceinline__ void load_tile(uint32_t sbase, const __half* g, int row0, int M, int heads, int head) {
  constexpr int CH = HD / 8;
  for (int e = threadIdx.x; e < BT * CH; e += blockDim.x) {
    const int r = e / CH, c = e % CH;
    const int m = row0 + r;
    const bool ok = m < M;
    const __half* src = g + ((size_t)(ok ? m : 0) * heads + head) * HD + c * 8;
    cp_async16(sbase + tile_off<HD>(r, c), src, ok);
  }
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *(uint32_t*)&h;
}

// A fragment: rows [r0, r0+16) x k-slice kk (16 wide) of a row-major tile
template <int HD>
__device__ __forceinline__ void frag_a(uint32_t sbase, int r0, int kk, uint32_t* a) {
  const int lane = threadIdx.x & 31, mat = lane >> 3, rr = lane & 7;
  ldsm_x4(sbase + tile_off<HD>(r0 + (mat & 1) * 8 + rr, kk * 2 + (mat >> 1)), a);
}
// B fragments for two n-tiles (16 tile rows starting at n0 act as n) x k-slice kk: tile rows are n, columns k
template <int HD>
__device__ __forceinline__ void frag_b_nk(uint32_t sbase, int n0, int kk, uint32_t* b) {
  const int lane = threadIdx.x & 31, mat = lane >> 3, rr = lane & 7;
  ldsm_x4(sbase + tile_off<HD>(n0 + (mat >> 1) * 8 + rr, kk * 2 + (mat & 1)), b);
}
// B fragments for two n-tiles (column chunks nc, nc+1) x 16 tile rows starting at k0: tile rows are k, columns n
template <int HD>
__device__ __forceinline__ void frag_b_kn(uint32_t sbase, int k0, int nc, uint32_t* b) {
  const int lane = threadIdx.x & 31, mat = lane >> 3, rr = lane & 7;
  ldsm_x4_trans(sbase + tile_off<HD>(k0 + (mat & 1) * 8 + rr, nc + (mat >> 1)), b);
}

constexpr float LOG2E = 1.4426950408889634f;

// ------------------------------------------------------------------ forward
// K and V are single-buffered (48 KB per CTA with Q, so three CTAs fit an SM): V(n) is fetched
// while Q.K(n)^T runs, K(n+1) while the softmax and P.V(n) run.
template <int HD>
__global__ void __launch_bounds__(128, HD == 128 ? 3 : 4)
attn_fwd_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                const int* __restrict__ seq_start, const int2* __restrict__ gap, int M, int nh, int nkv, float scale,
                __half* __restrict__ o, float* __restrict__ lse) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_addr(smem), sK = sQ + BT * HD * 2, sV = sK + BT * HD * 2;
  const int m0 = blockIdx.x * BT, h = blockIdx.y, g = h / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const float sl2 = scale * LOG2E;

  const int kbeg = (seq_start[m0] / BT) * BT;
  const int kend = min(m0 + BT, M);
  load_tile<HD>(sQ, q, m0, M, nh, h);
  load_tile<HD>(sK, k, kbeg, M, nkv, g);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) frag_a<HD>(sQ, warp * 16, kk, qf[kk]);

  const int i0 = m0 + warp * 16 + gq, i1 = i0 + 8;
  const int ss0 = i0 < M ? seq_start[i0] : 0x7fffffff, ss1 = i1 < M ? seq_start[i1] : 0x7fffffff;
  // keys in [gap.x, gap.y) are hidden from the row (other examples' tokens of a packed group)
  const int2 gp0 = (gap && i0 < M) ? gap[i0] : make_int2(0, 0), gp1 = (gap && i1 < M) ? gap[i1] : make_int2(0, 0);
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float oacc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

  for (int n0 = kbeg; n0 < kend; n0 += BT) {
    // K(n) is in shared memory and every warp is past P.V(n-1): V(n) may overwrite the V buffer
    load_tile<HD>(sV, v, n0, M, nkv, g);
    cp_async_commit();

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        frag_b_nk<HD>(sK, np * 16, kk, b);
        mma16816(s[2 * np], qf[kk], b);
        mma16816(s[2 * np + 1], qf[kk], b + 2);
      }
    }
    cp_async_wait_all();
    __syncthreads();  // V(n) has landed; every warp is done with K(n)
    if (n0 + BT < kend) load_tile<HD>(sK, k, n0 + BT, M, nkv, g);
    cp_async_commit();
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = n0 + nt * 8 + 2 * tq + (e & 1);
        const int i = (e < 2) ? i0 : i1, ss = (e < 2) ? ss0 : ss1;
        const int2 gp = (e < 2) ? gp0 : gp1;
        const bool ok = j <= i && j >= ss && (j < gp.x || j >= gp.y);
        const float val = ok ? s[nt][e] * sl2 : -INFINITY;
        s[nt][e] = val;
        mx[e >> 1] = fmaxf(mx[e >> 1], val);
      }
    }
    float corr[2], mref[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mn = fmaxf(m_run[r], mx[r]);
      mref[r] = mn == -INFINITY ? 0.f : mn;
      corr[r] = exp2f(m_run[r] - mref[r]);  // m_run = -inf gives 0
      m_run[r] = mn;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[nt][e] - mref[e >> 1]);
        s[nt][e] = p;
        l_run[e >> 1] += p;
      }
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      oacc[i][0] *= corr[0]; oacc[i][1] *= corr[0];
      oacc[i][2] *= corr[1]; oacc[i][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4] = {pack_h2(s[2 * kk][0], s[2 * kk][1]), pack_h2(s[2 * kk][2], s[2 * kk][3]),
                       pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        uint32_t b[4];
        frag_b_kn<HD>(sV, kk * 16, 2 * np, b);
        mma16816(oacc[2 * np], a, b);
        mma16816(oacc[2 * np + 1], a, b + 2);
      }
    }
    cp_async_wait_all();
    __syncthreads();  // K(n+1) has landed; every warp is done with V(n)
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv0 = 1.f / l_run[0], inv1 = 1.f / l_run[1];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int c = nt * 8 + 2 * tq;
    if (i0 < M) *(__half2*)(o + ((size_t)i0 * nh + h) * HD + c) = __floats2half2_rn(oacc[nt][0] * inv0, oacc[nt][1] * inv0);
    if (i1 < M) *(__half2*)(o + ((size_t)i1 * nh + h) * HD + c) = __floats2half2_rn(oacc[nt][2] * inv1, oacc[nt][3] * inv1);
  }
  if (tq == 0) {
    if (i0 < M) lse[(size_t)h * M + i0] = m_run[0] / LOG2E + logf(l_run[0]);
    if (i1 < M) lse[(size_t)h * M + i1] = m_run[1] / LOG2E + logf(l_run[1]);
  }
}

// ------------------------------------------------------------------ delta[h, m] = sum_d O * dO
template <int HD>
__global__ void attn_delta_kernel(const __half* __restrict__ o, const __half* __restrict__ dO, int M, int nh,
                                  float* __restrict__ delta) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= M * nh) return;
  const int m = warp / nh, h = warp % nh;
  const __half* a = o + ((size_t)m * nh + h) * HD;
  const __half* b = dO + ((size_t)m * nh + h) * HD;
  float s = 0.f;
  for (int i = lane * 2; i < HD; i += 64) {
    float2 x = __half22float2(*(const __half2*)(a + i)), y = __half22float2(*(const __half2*)(b + i));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[(size_t)h * M + m] = s;
}

// ------------------------------------------------------------------ backward: dK, dV per key tile
template <int HD>
__global__ void __launch_bounds__(128)
attn_bwd_dkdv_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                     const __half* __restrict__ dO, const float* __restrict__ do_scale,
                     const float* __restrict__ row_scale,
                     const float* __restrict__ lse, const float* __restrict__ delta,
                     const int* __restrict__ seq_start, const int2* __restrict__ gap, int M, int nh, int nkv, float scale,
                     float* __restrict__ dk, float* __restrict__ dv) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sK = smem_addr(smem), sV = sK + BT * HD * 2, sQdO = sV + BT * HD * 2;  // then two (Q, dO) buffers
  float* sAux = (float*)(smem + 6 * BT * HD * 2);  // two buffers of (lse, delta, seq_start, weight, gap) per query row
  // dO row i stands for row_scale[i] * dO[i] (do_scale[0] = the largest factor): a query row
  // enters the sums over queries with weight row_scale[i] / do_scale[0] <= 1
  const float inv_top = row_scale ? 1.0f / fmaxf(do_scale[0], 1e-38f) : 1.0f;
  const int n0 = blockIdx.x * BT, g = blockIdx.y, group = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const float sl2 = scale * LOG2E;

  load_tile<HD>(sK, k, n0, M, nkv, g);
  load_tile<HD>(sV, v, n0, M, nkv, g);

  float dkacc[HD / 8][4], dvacc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    dkacc[i][0] = dkacc[i][1] = dkacc[i][2] = dkacc[i][3] = 0.f;
    dvacc[i][0] = dvacc[i][1] = dvacc[i][2] = dvacc[i][3] = 0.f;
  }
  const int j0 = n0 + warp * 16 + gq, j1 = j0 + 8;  // this thread's two key rows
  // Queries that can see these keys lie in [n0, end of the sequence holding the tile's last key).
  const int last_key = min(n0 + BT, M) - 1;
  int qend = last_key + 1;
  {
    const int ss_last = seq_start[last_key];
    // the sequence of last_key ends where seq_start changes; walk forward in tile-sized strides then finish linearly
    int e = last_key + 1;
    while (e + BT <= M && seq_start[e + BT - 1] == ss_last) e += BT;
    while (e < M && seq_start[e] == ss_last) ++e;
    qend = e;
  }
  // work list: (query head of the group) x (query tiles that can see these keys); tile idx+1 is
  // prefetched while tile idx is used
  const int nqt = qend > n0 ? (qend - n0 + BT - 1) / BT : 0;
  const int n_work = group * nqt;
  auto prefetch = [&](int idx, int buf) {
    const int h = g * group + idx / nqt, m0 = n0 + (idx % nqt) * BT;
    load_tile<HD>(sQdO + buf * 2 * BT * HD * 2, q, m0, M, nh, h);
    load_tile<HD>(sQdO + buf * 2 * BT * HD * 2 + BT * HD * 2, dO, m0, M, nh, h);
    if (threadIdx.x < BT) {
      const int m = m0 + threadIdx.x;
      float* aux = sAux + buf * 6 * BT;
      aux[threadIdx.x] = m < M ? lse[(size_t)h * M + m] * LOG2E : 0.f;
      aux[BT + threadIdx.x] = m < M ? delta[(size_t)h * M + m] : 0.f;
      ((int*)aux)[2 * BT + threadIdx.x] = m < M ? seq_start[m] : 0x7fffffff;
      aux[3 * BT + threadIdx.x] = (row_scale && m < M) ? row_scale[m] * inv_top : 1.0f;
      const int2 gp = (gap && m < M) ? gap[m] : make_int2(0, 0);
      ((int*)aux)[4 * BT + threadIdx.x] = gp.x;
      ((int*)aux)[5 * BT + threadIdx.x] = gp.y;
    }
  };
  if (n_work > 0) prefetch(0, 0);
  cp_async_commit();
  for (int idx = 0; idx < n_work; ++idx) {
    {
      const int m0 = n0 + (idx % nqt) * BT;
      const int buf = idx & 1;
      const uint32_t sQ = sQdO + buf * 2 * BT * HD * 2, sdO = sQ + BT * HD * 2;
      const float* sLse = sAux + buf * 6 * BT;
      const float* sDel = sLse + BT;
      const int* sSS = (const int*)(sLse + 2 * BT);
      const float* sWt = sLse + 3 * BT;
      const int* sGlo = (const int*)(sLse + 4 * BT);
      const int* sGhi = (const int*)(sLse + 5 * BT);
      if (idx + 1 < n_work) prefetch(idx + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait_prev();
      __syncthreads();
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        const int qb = half * 32;
        float st[4][4], dp[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
          dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          uint32_t ak[4], av[4];
          frag_a<HD>(sK, warp * 16, kk, ak);
          frag_a<HD>(sV, warp * 16, kk, av);
#pragma unroll
          for (int np = 0; np < 2; ++np) {
            uint32_t b[4];
            frag_b_nk<HD>(sQ, qb + np * 16, kk, b);
            mma16816(st[2 * np], ak, b);
            mma16816(st[2 * np + 1], ak, b + 2);
            frag_b_nk<HD>(sdO, qb + np * 16, kk, b);
            mma16816(dp[2 * np], av, b);
            mma16816(dp[2 * np + 1], av, b + 2);
          }
        }
        // element (key row j, query column i): P^T and dS^T
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int il = qb + nt * 8 + 2 * tq + (e & 1);
            const int i = m0 + il;
            const int j = (e < 2) ? j0 : j1;
            const bool ok = i < M && j <= i && j >= sSS[il] && (j < sGlo[il] || j >= sGhi[il]);
            const float p = ok ? exp2f(st[nt][e] * sl2 - sLse[il]) * sWt[il] : 0.f;
            st[nt][e] = p;
            dp[nt][e] = p * (dp[nt][e] - sDel[il]) * scale;
          }
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          uint32_t ap[4] = {pack_h2(st[2 * kk][0], st[2 * kk][1]), pack_h2(st[2 * kk][2], st[2 * kk][3]),
                            pack_h2(st[2 * kk + 1][0], st[2 * kk + 1][1]), pack_h2(st[2 * kk + 1][2], st[2 * kk + 1][3])};
          uint32_t ad[4] = {pack_h2(dp[2 * kk][0], dp[2 * kk][1]), pack_h2(dp[2 * kk][2], dp[2 * kk][3]),
                            pack_h2(dp[2 * kk + 1][0], dp[2 * kk + 1][1]), pack_h2(dp[2 * kk + 1][2], dp[2 * kk + 1][3])};
#pragma unroll
          for (int np = 0; np < HD / 16; ++np) {
            uint32_t b[4];
            frag_b_kn<HD>(sdO, qb + kk * 16, 2 * np, b);
            mma16816(dvacc[2 * np], ap, b);
            mma16816(dvacc[2 * np + 1], ap, b + 2);
            frag_b_kn<HD>(sQ, qb + kk * 16, 2 * np, b);
            mma16816(dkacc[2 * np], ad, b);
            mma16816(dkacc[2 * np + 1], ad, b + 2);
          }
        }
      }
      __syncthreads();  // done with this (Q, dO) buffer before the next prefetch reuses it
    }
  }
  const float sc = do_scale[0];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int c = nt * 8 + 2 * tq;
    if (j0 < M) {
      *(float2*)(dk + ((size_t)j0 * nkv + g) * HD + c) = make_float2(dkacc[nt][0] * sc, dkacc[nt][1] * sc);
      *(float2*)(dv + ((size_t)j0 * nkv + g) * HD + c) = make_float2(dvacc[nt][0] * sc, dvacc[nt][1] * sc);
    }
    if (j1 < M) {
      *(float2*)(dk + ((size_t)j1 * nkv + g) * HD + c) = make_float2(dkacc[nt][2] * sc, dkacc[nt][3] * sc);
      *(float2*)(dv + ((size_t)j1 * nkv + g) * HD + c) = make_float2(dvacc[nt][2] * sc, dvacc[nt][3] * sc);
    }
  }
}

// ------------------------------------------------------------------ backward: dQ per query tile
template <int HD>
__global__ void __launch_bounds__(128)
attn_bwd_dq_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                   const __half* __restrict__ dO, const float* __restrict__ do_scale, const float* __restrict__ row_scale,
                   const float* __restrict__ lse,
                   const float* __restrict__ delta, const int* __restrict__ seq_start, const int2* __restrict__ gap, int M,
                   int nh, int nkv, float scale, float* __restrict__ dq) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_addr(smem), sdO = sQ + BT * HD * 2, sKV = sdO + BT * HD * 2;  // then two (K, V) buffers
  const int m0 = blockIdx.x * BT, h = blockIdx.y, g = h / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const float sl2 = scale * LOG2E;
  load_tile<HD>(sQ, q, m0, M, nh, h);
  load_tile<HD>(sdO, dO, m0, M, nh, h);
  const int i0 = m0 + warp * 16 + gq, i1 = i0 + 8;
  const int ss0 = i0 < M ? seq_start[i0] : 0x7fffffff, ss1 = i1 < M ? seq_start[i1] : 0x7fffffff;
  const int2 gp0 = (gap && i0 < M) ? gap[i0] : make_int2(0, 0), gp1 = (gap && i1 < M) ? gap[i1] : make_int2(0, 0);
  const float l0 = i0 < M ? lse[(size_t)h * M + i0] * LOG2E : 0.f, l1 = i1 < M ? lse[(size_t)h * M + i1] * LOG2E : 0.f;
  const float d0 = i0 < M ? delta[(size_t)h * M + i0] : 0.f, d1 = i1 < M ? delta[(size_t)h * M + i1] : 0.f;
  float acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const int kbeg = (seq_start[m0] / BT) * BT;
  const int kend = min(m0 + BT, M);
  load_tile<HD>(sKV, k, kbeg, M, nkv, g);
  load_tile<HD>(sKV + BT * HD * 2, v, kbeg, M, nkv, g);
  cp_async_commit();
  int it = 0;
  for (int n0 = kbeg; n0 < kend; n0 += BT, ++it) {
    const uint32_t sK = sKV + (it & 1) * 2 * BT * HD * 2, sV = sK + BT * HD * 2;
    if (n0 + BT < kend) {
      const uint32_t nK = sKV + ((it & 1) ^ 1) * 2 * BT * HD * 2;
      load_tile<HD>(nK, k, n0 + BT, M, nkv, g);
      load_tile<HD>(nK + BT * HD * 2, v, n0 + BT, M, nkv, g);
    }
    cp_async_commit();
    cp_async_wait_prev();
    __syncthreads();
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      const int kb = half * 32;
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t aq[4], ad[4];
        frag_a<HD>(sQ, warp * 16, kk, aq);
        frag_a<HD>(sdO, warp * 16, kk, ad);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          frag_b_nk<HD>(sK, kb + np * 16, kk, b);
          mma16816(s[2 * np], aq, b);
          mma16816(s[2 * np + 1], aq, b + 2);
          frag_b_nk<HD>(sV, kb + np * 16, kk, b);
          mma16816(dp[2 * np], ad, b);
          mma16816(dp[2 * np + 1], ad, b + 2);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = n0 + kb + nt * 8 + 2 * tq + (e & 1);
          const int i = (e < 2) ? i0 : i1, ss = (e < 2) ? ss0 : ss1;
          const int2 gp = (e < 2) ? gp0 : gp1;
          const bool ok = i < M && j <= i && j >= ss && (j < gp.x || j >= gp.y);
          const float p = ok ? exp2f(s[nt][e] * sl2 - ((e < 2) ? l0 : l1)) : 0.f;
          dp[nt][e] = p * (dp[nt][e] - ((e < 2) ? d0 : d1)) * scale;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t a[4] = {pack_h2(dp[2 * kk][0], dp[2 * kk][1]), pack_h2(dp[2 * kk][2], dp[2 * kk][3]),
                         pack_h2(dp[2 * kk + 1][0], dp[2 * kk + 1][1]), pack_h2(dp[2 * kk + 1][2], dp[2 * kk + 1][3])};
#pragma unroll
        for (int np = 0; np < HD / 16; ++np) {
          uint32_t b[4];
          frag_b_kn<HD>(sK, kb + kk * 16, 2 * np, b);
          mma16816(acc[2 * np], a, b);
          mma16816(acc[2 * np + 1], a, b + 2);
        }
      }
    }
    __syncthreads();
  }
  // a query row's gradient carries only that row's factor
  const float sc0 = row_scale ? (i0 < M ? row_scale[i0] : 0.f) : do_scale[0];
  const float sc1 = row_scale ? (i1 < M ? row_scale[i1] : 0.f) : do_scale[0];
#pragma unroll
  for (int nt = 0; nt < HD / 8; ++nt) {
    const int c = nt * 8 + 2 * tq;
    if (i0 < M) *(float2*)(dq + ((size_t)i0 * nh + h) * HD + c) = make_float2(acc[nt][0] * sc0, acc[nt][1] * sc0);
    if (i1 < M) *(float2*)(dq + ((size_t)i1 * nh + h) * HD + c) = make_float2(acc[nt][2] * sc1, acc[nt][3] * sc1);
  }
}

template <int HD>
int fwd_impl(const __half* q, const __half* k, const __half* v, const int* seq_start, const int2* gap, int M, int nh, int nkv,
             __half* o, float* lse, cudaStream_t st) {
  const size_t smem = 3 * BT * HD * 2;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 3;
    attr = true;
  }
  dim3 grid((M + BT - 1) / BT, nh);
  { attn_fwd_kernel<HD><<<grid, 128, smem, st>>>(q, k, v, seq_start, gap, M, nh, nkv, 1.0f / sqrtf((float)HD), o, lse); RT_COUNT_LAUNCH(1); }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

template <int HD>
int bwd_impl(const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO,
             const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int2* gap, int M,
             int nh, int nkv, float* delta, float* dq, float* dk, float* dv, cudaStream_t st) {
  const size_t smem_kv = 6 * BT * HD * 2 + 2 * 6 * BT * 4, smem_q = 6 * BT * HD * 2;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_dkdv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv) != cudaSuccess) return 3;
    if (cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q) != cudaSuccess) return 3;
    attr = true;
  }
  const float scale = 1.0f / sqrtf((float)HD);
  const int warps = M * nh;
  { attn_delta_kernel<HD><<<(warps * 32 + 255) / 256, 256, 0, st>>>(o, dO, M, nh, delta); RT_COUNT_LAUNCH(1); }
  dim3 gkv((M + BT - 1) / BT, nkv), gq((M + BT - 1) / BT, nh);
  { attn_bwd_dkdv_kernel<HD><<<gkv, 128, smem_kv, st>>>(q, k, v, dO, do_scale, row_scale, lse, delta, seq_start, gap, M, nh, nkv, scale, dk, dv); RT_COUNT_LAUNCH(1); }
  { attn_bwd_dq_kernel<HD><<<gq, 128, smem_q, st>>>(q, k, v, dO, do_scale, row_scale, lse, delta, seq_start, gap, M, nh, nkv, scale, dq); RT_COUNT_LAUNCH(1); }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace

int launch_attn_fwd(const __half* q, const __half* k, const __half* v, const int* seq_start, const int* gap, int M, int nh,
                    int nkv, int hd, __half* o, float* lse, cudaStream_t st) {
  if (M <= 0) return 0;
  if (hd == 128) return fwd_impl<128>(q, k, v, seq_start, (const int2*)gap, M, nh, nkv, o, lse, st);
  if (hd == 64) return fwd_impl<64>(q, k, v, seq_start, (const int2*)gap, M, nh, nkv, o, lse, st);
  return 1;  // unsupported head size
}

int launch_attn_bwd(const __half* q, const __half* k, const __half* v, const __half* o, const __half* dO16,
                    const float* do_scale, const float* row_scale, const float* lse, const int* seq_start, const int* gap,
                    int M, int nh, int nkv, int hd, float* delta, float* dq, float* dk, float* dv, cudaStream_t st) {
  if (M <= 0) return 0;
  if (hd == 128) return bwd_impl<128>(q, k, v, o, dO16, do_scale, row_scale, lse, seq_start, (const int2*)gap, M, nh, nkv, delta, dq, dk, dv, st);
  if (hd == 64) return bwd_impl<64>(q, k, v, o, dO16, do_scale, row_scale, lse, seq_start, (const int2*)gap, M, nh, nkv, delta, dq, dk, dv, st);
  return 1;
}

}  // namespace rt
