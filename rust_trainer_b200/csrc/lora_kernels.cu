// The low-rank side products of a LoRA linear (reference src/linear.rs:84-91,105-117), which
// are memory bound (rank <= 64 against thousands of tokens and features), as small
// warp-level tensor-core kernels:
//
//   tok_contract : part[split][r x C] = sum_{m in split} P[m, i] * Q[m, j]
//                  (dA = Gs^T.X, dB = dY^T.Hs), summed over splits in order by a second kernel
//
// Operands are f16, accumulation f32.  Tiles are 64 halves wide (128-byte rows) with the
// 16-byte chunks XOR-swizzled by row, loaded with cp.async and double buffered.
#include "ops.h"
#include "pdl.cuh"
#include "rt_internal.h"
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdlib.h>

namespace rt {
namespace {

__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t toff(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }
__device__ __forceinline__ void cpa16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// rows [row0, row0+64) x columns [col0, col0+64) of a row-major [rows x ld] f16 matrix -> swizzled 64x64 tile
__device__ __forceinline__ void load64x64(uint32_t sbase, const __half* g, int row0, int rows, int col0, int cols, int ld,
                                          int row_limit = 64) {
  for (int e = threadIdx.x; e < 64 * 8; e += blockDim.x) {
    const int r = e >> 3, c = e & 7;
    const int gr = row0 + r, gc = col0 + c * 8;
    const bool ok = r < row_limit && gr < rows && gc < cols;
    cpa16(sbase + toff(r, c), g + (size_t)(ok ? gr : 0) * ld + (ok ? gc : 0), ok);
  }
}

// ------------------------------------------------------------------ part[split] = P^T . Q over a token range
template <int R16>
__global__ void __launch_bounds__(128)
tok_contract_kernel(const __half* __restrict__ P, const __half* __restrict__ Q, const float* __restrict__ pscale,
                    const float* __restrict__ smax, int M, int C, int r, int tokens_per_split, float* __restrict__ part) {
  constexpr int NST = 3, SB = 8192 + 16384;  // per stage: P chunk, two Q panels
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s0 = saddr(smem);
  const int j0 = blockIdx.x * 128;
  const int m_begin = blockIdx.y * tokens_per_split, m_end = min(M, m_begin + tokens_per_split);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int mat = lane >> 3, rr = lane & 7;
  const int panel = warp >> 1, cbase = (warp & 1) * 4;  // this warp's 32 columns: panel, first 16-byte chunk
  float acc[R16][4][4];
#pragma unroll
  for (int a = 0; a < R16; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;
  const int nchunks = (m_end - m_begin + 63) / 64;
  auto load = [&](int ch, int buf) {
    const int mrow = m_begin + ch * 64;
    load64x64(s0 + buf * SB, P, mrow, m_end, 0, 64, 64);
    load64x64(s0 + buf * SB + 8192, Q, mrow, m_end, j0, C, C);
    load64x64(s0 + buf * SB + 16384, Q, mrow, m_end, j0 + 64, C, C);
  };
  for (int i = 0; i < NST - 1; ++i) {
    if (i < nchunks) load(i, i);
    cpa_commit();
  }
  for (int ch = 0; ch < nchunks; ++ch) {
    const int b = ch % NST;
    if (ch + NST - 1 < nchunks) load(ch + NST - 1, (ch + NST - 1) % NST);
    cpa_commit();
    cpa_wait<NST - 1>();
    __syncthreads();
    const uint32_t sP = s0 + b * SB;
    if (pscale) {
      // rows of P times scale[m] / max(scale): the per-token factors of dY, normalised so f16 holds them
      const float inv = 1.0f / smax[0];
      for (int e = threadIdx.x; e < 64 * 8; e += blockDim.x) {
        const int row = e >> 3, c = e & 7, mrow = m_begin + ch * 64 + row;
        const float f = mrow < m_end ? pscale[mrow] * inv : 0.f;
        uint4* ptr = (uint4*)(smem + b * SB + toff(row, c));
        uint4 v = *ptr;
        __half2* h2 = (__half2*)&v;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = __half22float2(h2[k]);
          h2[k] = __floats2half2_rn(x.x * f, x.y * f);
        }
        *ptr = v;
      }
      __syncthreads();
    }
    const uint32_t q = sP + 8192 + panel * 8192;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t bf[2][4];
#pragma unroll
      for (int np = 0; np < 2; ++np) ldsm4t(q + toff(kk * 16 + (mat & 1) * 8 + rr, cbase + 2 * np + (mat >> 1)), bf[np]);
#pragma unroll
      for (int mi = 0; mi < R16; ++mi) {
        uint32_t a[4];  // A = P^T: rows i, k = tokens; P is stored [token][i]
        ldsm4t(sP + toff(kk * 16 + (mat >> 1) * 8 + rr, mi * 2 + (mat & 1)), a);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          mma(acc[mi][2 * np], a, bf[np]);
          mma(acc[mi][2 * np + 1], a, bf[np] + 2);
        }
      }
    }
    __syncthreads();
  }
  float* dst = part + (size_t)blockIdx.y * r * C;
#pragma unroll
  for (int mi = 0; mi < R16; ++mi)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int j = j0 + warp * 32 + nt * 8 + 2 * tq;
      const int i0 = mi * 16 + gq, i1 = i0 + 8;
      if (j < C) {
        if (i0 < r) { dst[(size_t)i0 * C + j] = acc[mi][nt][0]; if (j + 1 < C) dst[(size_t)i0 * C + j + 1] = acc[mi][nt][1]; }
        if (i1 < r) { dst[(size_t)i1 * C + j] = acc[mi][nt][2]; if (j + 1 < C) dst[(size_t)i1 * C + j + 1] = acc[mi][nt][3]; }
      }
    }
}

// out[i*so_i + j*so_j] += alpha * sum_s part[s][i, j]   (splits added in order: deterministic)
__global__ void tok_reduce_kernel(const float* __restrict__ part, int splits, int C, int r, size_t so_i, size_t so_j,
                                  const float* __restrict__ alpha_dev, float* __restrict__ out) {
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (size_t)r * C) return;
  const int i = (int)(e / C), j = (int)(e % C);
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(size_t)k * r * C + e];
  if (alpha_dev) s *= alpha_dev[0];
  out[i * so_i + j * so_j] += s;
}

// ------------------------------------------------------------------ both LoRA gradients of one linear in one launch
// Blocks [0, nbB) of grid.x work on dB (P = Hs, Q = dY, C = N), the rest on dA (P = Gs, Q = X,
// C = K); grid.y is the token split.  The per-token factors of dY are applied to the rows of the
// skinny operand relative to the LARGEST FACTOR OF THE SPLIT (found by the block itself), and
// that maximum multiplies the split's partial sums, so no pass over all factors comes first.
struct LoraGroupMember { float *gb, *ga; int row_off, rows, rank_off, r; };
struct LoraGroupTable { int n; LoraGroupMember m[3]; };
struct LoraGradArgs {
  const __half *Pb, *Qb, *Pa, *Qa;  // Hs, dY, Gs, X
  const float* pscale;              // per-token factors of dY, or null
  int M, N, K, r, nbB, tokens_per_split;
  int ldb;                          // row pitch of dY (>= N: dY may be a column slice of a wider matrix)
  float *partB, *partA;             // [splits][r x N], [splits][r x K]
};

template <int R16>
__global__ void __launch_bounds__(128) lora_grads_kernel(const LoraGradArgs g) {
  constexpr int NST = 3, SB = 8192 + 16384;  // per stage: P chunk, two Q panels
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s_red[4];
  const uint32_t s0 = saddr(smem);
  const bool isB = (int)blockIdx.x < g.nbB;
  const __half* P = isB ? g.Pb : g.Pa;
  const __half* Q = isB ? g.Qb : g.Qa;
  const int C = isB ? g.N : g.K;
  const int ldq = isB ? g.ldb : g.K;
  const int j0 = (isB ? (int)blockIdx.x : (int)blockIdx.x - g.nbB) * 128;
  const int m_begin = blockIdx.y * g.tokens_per_split, m_end = min(g.M, m_begin + g.tokens_per_split);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int mat = lane >> 3, rr = lane & 7;
  const int panel = warp >> 1, cbase = (warp & 1) * 4;
  float acc[R16][4][4];
#pragma unroll
  for (int a = 0; a < R16; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;
  const int nchunks = (m_end - m_begin + 63) / 64;
  auto load = [&](int ch, int buf) {
    const int mrow = m_begin + ch * 64;
    load64x64(s0 + buf * SB, P, mrow, m_end, 0, 64, 64);
    load64x64(s0 + buf * SB + 8192, Q, mrow, m_end, j0, C, ldq);
    load64x64(s0 + buf * SB + 16384, Q, mrow, m_end, j0 + 64, C, ldq);
  };
  for (int i = 0; i < NST - 1; ++i) {
    if (i < nchunks) load(i, i);
    cpa_commit();
  }
  // largest factor of this split (factors are >= 0), while the first tiles are in flight
  float lmax = 1.0f, inv = 1.0f;
  if (g.pscale) {
    float v = 0.f;
    for (int m = m_begin + threadIdx.x; m < m_end; m += 128) v = fmaxf(v, g.pscale[m]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    lmax = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    // up to a power of two: the f16 roundings below then do not depend on which tokens share the split
    lmax = __int_as_float((__float_as_int(lmax) + 0x007FFFFF) & 0x7F800000);
    inv = lmax > 0.f ? 1.0f / lmax : 0.f;
  }
  for (int ch = 0; ch < nchunks; ++ch) {
    const int b = ch % NST;
    if (ch + NST - 1 < nchunks) load(ch + NST - 1, (ch + NST - 1) % NST);
    cpa_commit();
    cpa_wait<NST - 1>();
    __syncthreads();
    const uint32_t sP = s0 + b * SB;
    if (g.pscale) {
      for (int e = threadIdx.x; e < 64 * 8; e += blockDim.x) {
        const int row = e >> 3, c = e & 7, mrow = m_begin + ch * 64 + row;
        const float f = mrow < m_end ? g.pscale[mrow] * inv : 0.f;
        uint4* ptr = (uint4*)(smem + b * SB + toff(row, c));
        uint4 v = *ptr;
        __half2* h2 = (__half2*)&v;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = __half22float2(h2[k]);
          h2[k] = __floats2half2_rn(x.x * f, x.y * f);
        }
        *ptr = v;
      }
      __syncthreads();
    }
    const uint32_t q = sP + 8192 + panel * 8192;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t bf[2][4];
#pragma unroll
      for (int np = 0; np < 2; ++np) ldsm4t(q + toff(kk * 16 + (mat & 1) * 8 + rr, cbase + 2 * np + (mat >> 1)), bf[np]);
#pragma unroll
      for (int mi = 0; mi < R16; ++mi) {
        uint32_t a[4];  // A = P^T: rows i, k = tokens; P is stored [token][i]
        ldsm4t(sP + toff(kk * 16 + (mat >> 1) * 8 + rr, mi * 2 + (mat & 1)), a);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          mma(acc[mi][2 * np], a, bf[np]);
          mma(acc[mi][2 * np + 1], a, bf[np] + 2);
        }
      }
    }
    __syncthreads();
  }
  float* dst = (isB ? g.partB : g.partA) + (size_t)blockIdx.y * g.r * C;
#pragma unroll
  for (int mi = 0; mi < R16; ++mi)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int j = j0 + warp * 32 + nt * 8 + 2 * tq;
      const int i0 = mi * 16 + gq, i1 = i0 + 8;
      if (j < C) {  // C is a multiple of 8, so j + 1 < C too
        if (i0 < g.r) *(float2*)(dst + (size_t)i0 * C + j) = make_float2(acc[mi][nt][0] * lmax, acc[mi][nt][1] * lmax);
        if (i1 < g.r) *(float2*)(dst + (size_t)i1 * C + j) = make_float2(acc[mi][nt][2] * lmax, acc[mi][nt][3] * lmax);
      }
    }
}

// gb[n*r + i] += sum_s partB[s][i, n] ; ga[i*K + k] += sum_s partA[s][i, k]   (splits in order: deterministic)
__global__ void lora_grads_reduce_kernel(const float* __restrict__ partB, const float* __restrict__ partA, int splits, int N,
                                         int K, int r, float* __restrict__ gb, float* __restrict__ ga) {
  pdl_entry();
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nB = (size_t)r * N, nA = (size_t)r * K;
  if (e < nB) {
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partB[(size_t)k * nB + e];
    const int i = (int)(e / N), n = (int)(e % N);
    gb[(size_t)n * r + i] += s;
  } else if (e < nB + nA) {
    const size_t f = e - nB;
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partA[(size_t)k * nA + f];
    ga[f] += s;
  }
}

// The same for a group of linears that share X: partB is [splits][R x N_total] with the members'
// diagonal blocks wanted (member j: rows rank_off..+r of the rank axis, columns row_off..+rows),
// partA is [splits][R x K] with member j owning rows rank_off..+r.
__global__ void lora_grads_group_reduce_kernel(const float* __restrict__ partB, const float* __restrict__ partA, int splits,
                                               int NT, int K, int R, const LoraGroupTable t) {
  pdl_entry();
  size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nB = (size_t)R * NT, nA = (size_t)R * K;
  for (int j = 0; j < t.n; ++j) {
    const LoraGroupMember& mb = t.m[j];
    const size_t cb = (size_t)mb.r * mb.rows, ca = (size_t)mb.r * K;
    if (e < cb) {
      const int i = (int)(e / mb.rows), n = (int)(e % mb.rows);
      const size_t src = (size_t)(mb.rank_off + i) * NT + mb.row_off + n;
      float s = 0.f;
      for (int k = 0; k < splits; ++k) s += partB[(size_t)k * nB + src];
      mb.gb[(size_t)n * mb.r + i] += s;
      return;
    }
    e -= cb;
    if (e < ca) {
      const size_t src = (size_t)mb.rank_off * K + e;
      float s = 0.f;
      for (int k = 0; k < splits; ++k) s += partA[(size_t)k * nA + src];
      mb.ga[e] += s;
      return;
    }
    e -= ca;
  }
}

}  // namespace

static void tok_plan(int M, int* tokens_per_split, int* splits) {
  int tps = 256;
  if (M < 1024) tps = 128;
  if (M < 512) tps = 64;
  *tokens_per_split = tps;
  *splits = (M + tps - 1) / tps;
}
size_t tok_contract_workspace_floats(int M, int C, int r) {
  int tps, splits;
  tok_plan(M, &tps, &splits);
  return (size_t)splits * r * C;
}
int launch_tok_contract(const __half* P, const __half* Q, const float* pscale, int M, int C, int r, size_t so_i, size_t so_j,
                        const float* alpha_dev, float* out, float* workspace, cudaStream_t st) {
  if (M <= 0) return 0;
  if (r <= 0 || r > 64 || C % 8 != 0) return 1;
  int tps, splits;
  tok_plan(M, &tps, &splits);
  dim3 grid((C + 127) / 128, splits);
  constexpr int TOK_SMEM = 3 * (8192 + 16384);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(tok_contract_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    cudaFuncSetAttribute(tok_contract_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    cudaFuncSetAttribute(tok_contract_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    attr = true;
  }
  if (r <= 16) tok_contract_kernel<1><<<grid, 128, TOK_SMEM, st>>>(P, Q, pscale, alpha_dev, M, C, r, tps, workspace);
  else if (r <= 32) tok_contract_kernel<2><<<grid, 128, TOK_SMEM, st>>>(P, Q, pscale, alpha_dev, M, C, r, tps, workspace);
  else tok_contract_kernel<4><<<grid, 128, TOK_SMEM, st>>>(P, Q, pscale, alpha_dev, M, C, r, tps, workspace);
  const size_t n = (size_t)r * C;
  tok_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(workspace, splits, C, r, so_i, so_j, alpha_dev, out);
  RT_COUNT_LAUNCH(2);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

size_t lora_grads_workspace_floats(int M, int N, int K, int r) {
  int tps, splits;
  tok_plan(M, &tps, &splits);
  return (size_t)splits * r * ((size_t)N + (size_t)K);
}

// dB and dA of one linear: two launches in all.  Returns 1 for shapes these kernels do not cover.
// hs / gs are [M x 64] matrices; a pointer into such a matrix at a column offset (a multiple of 8)
// selects the r columns from there on, and then the 64-wide row reads run past the last row's end
// by that offset: the caller keeps that much slack behind the matrix.  dy16 has row pitch ld_dy.
int launch_lora_grads(rt_ctx* c, const __half* hs, const __half* dy16, int ld_dy, const __half* gs, const __half* x16,
                      const float* dscale, int M, int N, int K, int r, float* gb, float* ga, float* workspace, cudaStream_t st) {
  if (M <= 0) return 0;
  if (ld_dy <= 0) ld_dy = N;
  if (r <= 0 || r > 64 || N % 8 != 0 || K % 8 != 0 || ld_dy % 8 != 0) return 1;
  int tps, splits;
  {  // the tcgen05 kernel takes every shape whose pointers are 16-byte aligned
    const int tps_tc = lora_grads_tc_tokens_per_split(M), splits_tc = (M + tps_tc - 1) / tps_tc;
    float* pB = workspace;
    float* pA = workspace + (size_t)splits_tc * r * N;
    const int rc = launch_lora_grads_tc(c, hs, dy16, ld_dy, gs, x16, dscale, M, N, K, r, pB, pA);
    if (rc == 3) return 3;
    if (rc == 0) {
      const size_t n = (size_t)r * ((size_t)N + (size_t)K);
      pdl(lora_grads_reduce_kernel, (unsigned)((n + 255) / 256), 256, 0, st)(pB, pA, splits_tc, N, K, r, gb, ga);
      RT_COUNT_LAUNCH(1);
      return cudaGetLastError() == cudaSuccess ? 0 : 3;
    }
  }
  tok_plan(M, &tps, &splits);
  LoraGradArgs g;
  g.Pb = hs; g.Qb = dy16; g.Pa = gs; g.Qa = x16;
  g.pscale = dscale;
  g.M = M; g.N = N; g.K = K; g.r = r;
  g.nbB = (N + 127) / 128;
  g.ldb = ld_dy;
  g.tokens_per_split = tps;
  g.partB = workspace;
  g.partA = workspace + (size_t)splits * r * N;
  dim3 grid(g.nbB + (K + 127) / 128, splits);
  constexpr int TOK_SMEM = 3 * (8192 + 16384);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(lora_grads_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    cudaFuncSetAttribute(lora_grads_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    cudaFuncSetAttribute(lora_grads_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    attr = true;
  }
  if (r <= 16) lora_grads_kernel<1><<<grid, 128, TOK_SMEM, st>>>(g);
  else if (r <= 32) lora_grads_kernel<2><<<grid, 128, TOK_SMEM, st>>>(g);
  else lora_grads_kernel<4><<<grid, 128, TOK_SMEM, st>>>(g);
  const size_t n = (size_t)r * ((size_t)N + (size_t)K);
  pdl(lora_grads_reduce_kernel, (unsigned)((n + 255) / 256), 256, 0, st)(g.partB, g.partA, splits, N, K, r, gb, ga);
  RT_COUNT_LAUNCH(2);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// dA and dB of every member of a stacked group in one product launch and one reduce launch.
// gb/ga/row_off/rows/rank_off/rank: per member (n <= 3).  Workspace: lora_grads_workspace_floats(M, NT, K, R).
int launch_lora_grads_group(rt_ctx* c, const __half* hs, const __half* dy16, const __half* gs, const __half* x16,
                            const float* dscale, int M, int NT, int K, int R, int n, float* const* gb, float* const* ga,
                            const int* row_off, const int* rows, const int* rank_off, const int* rank, float* workspace,
                            cudaStream_t st) {
  if (M <= 0 || n <= 0) return 0;
  if (n > 3 || R <= 0 || R > 64 || NT % 8 != 0 || K % 8 != 0) return 1;
  int tps, splits;
  {
    const int tps_tc = lora_grads_tc_tokens_per_split(M), splits_tc = (M + tps_tc - 1) / tps_tc;
    float* pB = workspace;
    float* pA = workspace + (size_t)splits_tc * R * NT;
    const int rc = launch_lora_grads_tc(c, hs, dy16, NT, gs, x16, dscale, M, NT, K, R, pB, pA);
    if (rc == 3) return 3;
    if (rc == 0) {
      LoraGroupTable t;
      t.n = n;
      size_t total = 0;
      for (int j = 0; j < n; ++j) {
        t.m[j] = LoraGroupMember{gb[j], ga[j], row_off[j], rows[j], rank_off[j], rank[j]};
        total += (size_t)rank[j] * ((size_t)rows[j] + (size_t)K);
      }
      pdl(lora_grads_group_reduce_kernel, (unsigned)((total + 255) / 256), 256, 0, st)(pB, pA, splits_tc, NT, K, R, t);
      RT_COUNT_LAUNCH(1);
      return cudaGetLastError() == cudaSuccess ? 0 : 3;
    }
  }
  tok_plan(M, &tps, &splits);
  LoraGradArgs g;
  g.Pb = hs; g.Qb = dy16; g.Pa = gs; g.Qa = x16;
  g.pscale = dscale;
  g.M = M; g.N = NT; g.K = K; g.r = R;
  g.nbB = (NT + 127) / 128;
  g.ldb = NT;
  g.tokens_per_split = tps;
  g.partB = workspace;
  g.partA = workspace + (size_t)splits * R * NT;
  dim3 grid(g.nbB + (K + 127) / 128, splits);
  constexpr int TOK_SMEM = 3 * (8192 + 16384);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(lora_grads_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    cudaFuncSetAttribute(lora_grads_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    cudaFuncSetAttribute(lora_grads_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, TOK_SMEM);
    attr = true;
  }
  if (R <= 16) lora_grads_kernel<1><<<grid, 128, TOK_SMEM, st>>>(g);
  else if (R <= 32) lora_grads_kernel<2><<<grid, 128, TOK_SMEM, st>>>(g);
  else lora_grads_kernel<4><<<grid, 128, TOK_SMEM, st>>>(g);
  LoraGroupTable t;
  t.n = n;
  size_t total = 0;
  for (int j = 0; j < n; ++j) {
    t.m[j] = LoraGroupMember{gb[j], ga[j], row_off[j], rows[j], rank_off[j], rank[j]};
    total += (size_t)rank[j] * ((size_t)rows[j] + (size_t)K);
  }
  pdl(lora_grads_group_reduce_kernel, (unsigned)((total + 255) / 256), 256, 0, st)(g.partB, g.partA, splits, NT, K, R, t);
  RT_COUNT_LAUNCH(2);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace rt
