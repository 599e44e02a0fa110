// The low-rank side products of a LoRA linear (reference src/linear.rs:84-91,105-117), which
// are memory bound (rank <= 64 against thousands of tokens and features), as small
// warp-level tensor-core kernels:
//
//   skinny_nt : Hs[M x 64] = X[M x K] . Wt[r x K]^T      (Hs = X.(sA)^T, Gs = dY.(sB))
//   tok_contract : part[split][r x C] = sum_{m in split} P[m, i] * Q[m, j]
//                  (dA = Gs^T.X, dB = dY^T.Hs), summed over splits in order by a second kernel
//
// Operands are f16, accumulation f32.  Tiles are 64 halves wide (128-byte rows) with the
// 16-byte chunks XOR-swizzled by row, loaded with cp.async and double buffered.
#include "ops.h"
#include "rt_internal.h"
#include <cuda_fp16.h>
#include <stdint.h>

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

// ------------------------------------------------------------------ Hs = X . Wt^T
template <int R16>
__global__ void __launch_bounds__(128)
skinny_nt_kernel(const __half* __restrict__ X, const __half* __restrict__ Wt, int M, int K, int r, __half* __restrict__ out) {
  __shared__ __align__(128) uint8_t smem[2 * 8192 + 2 * 8192];
  const uint32_t sX = saddr(smem), sW = sX + 2 * 8192;
  const int m0 = blockIdx.x * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int mat = lane >> 3, rr = lane & 7;
  float acc[2 * R16][4];
#pragma unroll
  for (int i = 0; i < 2 * R16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const int nk = (K + 63) / 64;
  load64x64(sX, X, m0, M, 0, K, K);
  load64x64(sW, Wt, 0, r, 0, K, K, 16 * R16);
  cpa_commit();
  for (int kc = 0; kc < nk; ++kc) {
    const int b = kc & 1;
    if (kc + 1 < nk) {
      load64x64(sX + (b ^ 1) * 8192, X, m0, M, (kc + 1) * 64, K, K);
      load64x64(sW + (b ^ 1) * 8192, Wt, 0, r, (kc + 1) * 64, K, K, 16 * R16);
    }
    cpa_commit();
    cpa_wait<1>();
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      ldsm4(sX + b * 8192 + toff(warp * 16 + (mat & 1) * 8 + rr, kk * 2 + (mat >> 1)), a);
#pragma unroll
      for (int np = 0; np < R16; ++np) {
        uint32_t bf[4];
        ldsm4(sW + b * 8192 + toff(np * 16 + (mat >> 1) * 8 + rr, kk * 2 + (mat & 1)), bf);
        mma(acc[2 * np], a, bf);
        mma(acc[2 * np + 1], a, bf + 2);
      }
    }
    __syncthreads();
  }
  const int i0 = m0 + warp * 16 + gq, i1 = i0 + 8;
#pragma unroll
  for (int nt = 0; nt < 2 * R16; ++nt) {
    const int c = nt * 8 + 2 * tq;
    if (c < r) {  // r is even (a multiple of 2 is enough for the paired store; ranks are)
      if (i0 < M) *(__half2*)(out + (size_t)i0 * 64 + c) = __floats2half2_rn(acc[nt][0], acc[nt][1]);
      if (i1 < M) *(__half2*)(out + (size_t)i1 * 64 + c) = __floats2half2_rn(acc[nt][2], acc[nt][3]);
    }
  }
}

// ------------------------------------------------------------------ part[split] = P^T . Q over a token range
template <int R16>
__global__ void __launch_bounds__(128)
tok_contract_kernel(const __half* __restrict__ P, const __half* __restrict__ Q, int M, int C, int r, int tokens_per_split,
                    float* __restrict__ part) {
  __shared__ __align__(128) uint8_t smem[2 * 8192 + 2 * 16384];
  const uint32_t sP = saddr(smem), sQ = sP + 2 * 8192;
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
    load64x64(sP + buf * 8192, P, mrow, m_end, 0, 64, 64);
    load64x64(sQ + buf * 16384, Q, mrow, m_end, j0, C, C);
    load64x64(sQ + buf * 16384 + 8192, Q, mrow, m_end, j0 + 64, C, C);
  };
  if (nchunks > 0) load(0, 0);
  cpa_commit();
  for (int ch = 0; ch < nchunks; ++ch) {
    const int b = ch & 1;
    if (ch + 1 < nchunks) load(ch + 1, b ^ 1);
    cpa_commit();
    cpa_wait<1>();
    __syncthreads();
    const uint32_t q = sQ + b * 16384 + panel * 8192;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t bf[2][4];
#pragma unroll
      for (int np = 0; np < 2; ++np) ldsm4t(q + toff(kk * 16 + (mat & 1) * 8 + rr, cbase + 2 * np + (mat >> 1)), bf[np]);
#pragma unroll
      for (int mi = 0; mi < R16; ++mi) {
        uint32_t a[4];  // A = P^T: rows i, k = tokens; P is stored [token][i]
        ldsm4t(sP + b * 8192 + toff(kk * 16 + (mat >> 1) * 8 + rr, mi * 2 + (mat & 1)), a);
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

}  // namespace

int launch_skinny_nt(const __half* X, const __half* Wt, int M, int K, int r, __half* out, cudaStream_t st) {
  if (M <= 0) return 0;
  if (r <= 0 || r > 64 || (r & 1) || K % 8 != 0) return 1;
  const int grid = (M + 63) / 64;
  if (r <= 16) skinny_nt_kernel<1><<<grid, 128, 0, st>>>(X, Wt, M, K, r, out);
  else if (r <= 32) skinny_nt_kernel<2><<<grid, 128, 0, st>>>(X, Wt, M, K, r, out);
  else skinny_nt_kernel<4><<<grid, 128, 0, st>>>(X, Wt, M, K, r, out);
  RT_COUNT_LAUNCH(1);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

static void tok_plan(int M, int* tokens_per_split, int* splits) {
  int tps = 512;
  if (M < 2048) tps = 256;
  if (M < 512) tps = 64;
  *tokens_per_split = tps;
  *splits = (M + tps - 1) / tps;
}
size_t tok_contract_workspace_floats(int M, int C, int r) {
  int tps, splits;
  tok_plan(M, &tps, &splits);
  return (size_t)splits * r * C;
}
int launch_tok_contract(const __half* P, const __half* Q, int M, int C, int r, size_t so_i, size_t so_j,
                        const float* alpha_dev, float* out, float* workspace, cudaStream_t st) {
  if (M <= 0) return 0;
  if (r <= 0 || r > 64 || C % 8 != 0) return 1;
  int tps, splits;
  tok_plan(M, &tps, &splits);
  dim3 grid((C + 127) / 128, splits);
  if (r <= 16) tok_contract_kernel<1><<<grid, 128, 0, st>>>(P, Q, M, C, r, tps, workspace);
  else if (r <= 32) tok_contract_kernel<2><<<grid, 128, 0, st>>>(P, Q, M, C, r, tps, workspace);
  else tok_contract_kernel<4><<<grid, 128, 0, st>>>(P, Q, M, C, r, tps, workspace);
  const size_t n = (size_t)r * C;
  tok_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(workspace, splits, C, r, so_i, so_j, alpha_dev, out);
  RT_COUNT_LAUNCH(2);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace rt
