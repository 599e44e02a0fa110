// Internal declarations shared by the .cu/.cpp files of the library (not part of the C ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/rt_b200.h"  // status codes and public types

#include <atomic>

namespace rt {

struct QWeight;

// Kernels launched by this library in this process (every launcher adds its own).
extern std::atomic<unsigned long long> g_launch_count;
#ifdef RT_B200_SITEPROF
void prof_mark(const char* file, int line);  // site_prof.cu
#define RT_COUNT_LAUNCH(n) (rt::g_launch_count.fetch_add((n), std::memory_order_relaxed), rt::prof_mark(__FILE__, __LINE__))
#else
#define RT_COUNT_LAUNCH(n) (rt::g_launch_count.fetch_add((n), std::memory_order_relaxed))
#endif

// ---- repack.cu
void launch_repack(const uint8_t* raw_dev, const QWeight& w, cudaStream_t st);
void launch_gather_rows(const QWeight& w, const int* ids_dev, int n, float* out, int* status, cudaStream_t st);

// ---- qgemm.cu
enum { QG_FWD = 0, QG_BWD = 1 };
enum { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2 };  // same values as RT_DT_* in the public header

// Extra contraction chunk of rank r <= 64 appended after the frozen weight's own chunks:
//   forward : Y += Hs[M x 64] . Bp[N x 64]^T      (Hs = s.X.A^T, zero beyond column r)
//   backward: dX += Gs[M x 64] . A[r x K]          (Gs = s.dY.B,  zero beyond column r)
// Both operands have the 16-bit type of the call's activations.
struct LoraSide {
  const void* act = nullptr;  // Hs / Gs, [M x 64]
  const void* w = nullptr;    // forward: Bp [N x 64]; backward: A [r x K]
  int rank = 0;
};

struct QGemmArgs {
  int dir = QG_FWD;
  const void* act = nullptr;           // forward: X [M x K]; backward: dY [M x N]; f16 or bf16
  int act_f16 = 0;                     // 1: activations are f16, 0: bf16
  int M = 0;
  void* out = nullptr;                 // forward: Y [M x N]; backward: dX [M x K]
  int out_dtype = OUT_F32;
  int accumulate = 0;                  // out += result (f32 only)
  int ld_out = 0;                      // row pitch of out in elements (0: the output width)
  const float* bias = nullptr;         // forward only, per output feature
  const float* row_scale = nullptr;    // optional per-token factor on the result (before bias)
  LoraSide lora;
  // token-contraction mode (LoRA gradients): out[i*out_s_tok + j*out_s_row] (+)= alpha * sum_m P[m,i] * Q[m,j]
  // with Q = the dense 16-bit `w` [tokens x C], P = act [tokens x 64], M = rank (i < M), dir = QG_BWD
  int tok_mode = 0;
  size_t out_s_tok = 0, out_s_row = 1;
  const float* alpha_dev = nullptr;    // optional device scalar factor (split-K / token mode only)
  // split-K partials go to this caller-provided buffer instead of ctx scratch (and nothing is
  // cached or allocated on the way); a launch that needs more fails with RT_ERR_TOO_LARGE
  float* fixed_part = nullptr;
  size_t fixed_part_floats = 0;
  int aux = 0;                         // 1: a skinny LoRA helper product (kept apart in the profile)
};

int qgemm_launch(rt_ctx* ctx, const QWeight& w, const QGemmArgs& a);
// The product with a frozen weight of any storage: one qgemm launch, or, for f32 weights held as
// a two-term f16 split, the high term followed by the low term accumulated into an f32 result
// (a 16-bit result cannot resolve the low term and skips it).
int frozen_matmul_launch(rt_ctx* ctx, const QWeight& w, const QGemmArgs& a);
// Tiled TMA descriptor of a row-major f16 matrix [rows x cols], box = box_cols x box_rows elements,
// 128-byte swizzle (box_cols = 64); cached per ctx by (base, shape, box).
int tensor_map_f16_2d(rt_ctx* ctx, CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                      uint32_t box_rows);
// The same with a row pitch of `ld` elements (a column slice of a wider matrix).
int tensor_map_f16_2d_ld(rt_ctx* ctx, CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_cols, uint32_t box_rows);
size_t qgemm_smem_bytes();
int qgemm_init();  // resolves the driver entry point for tensor-map encoding; sets smem attributes

}  // namespace rt
