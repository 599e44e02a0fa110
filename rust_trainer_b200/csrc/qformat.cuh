// Device-side storage of a frozen ggml weight matrix.
//
// Quantised formats (Q4_0, Q8_0, Q4_K, Q6_K) are re-tiled ONCE at upload, bit for bit, from
// ggml's row-of-blocks order into "bricks" of 64 rows x 64 columns.  A brick holds the same
// codes and scales as the ggml blocks it covers (no dequantised copy is ever stored); only
// their order changes, so that (a) a brick is one contiguous, 16-byte aligned bulk copy and
// (b) one thread owns one (row, 32-column) unit and reads it with 128-bit shared loads.
// The forward GEMM (contract over columns) fetches the two bricks that are row neighbours,
// the backward GEMM (contract over rows) the two that are column neighbours: one layout
// serves W.x and W^T.dy.
//
// Unit t of a brick = (row t>>1, column half t&1), 32 codes.  Within a unit, codes are kept
// in four 32-bit words of eight 4-bit fields; field p holds element 2p, field p+4 element
// 2p+1 of that word's eight consecutive columns, so `(w >> 4p) & 0x000F000F` yields the
// pair (2p, 2p+1) in the two halves of a 32-bit register.
//
//   Q4_0 : [128 x 16 B codes][128 x f16 d]                                   2304 B
//   Q8_0 : [128 x 32 B codes+128][128 x f16 d]                               4352 B
//   Q4_K : [128 x 16 B codes][64 x (f16 d, f16 dmin)][128 x (u8 sc, u8 m)]   2560 B
//   Q6_K : [128 x 16 B low4][128 x 8 B high2][128 x 2 x i8 sc][64 x f16 d]   3456 B
//
// F16 and BF16 matrices stay exactly as they are (row-major) and are read by tiled TMA.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace rt {

// ggml type ids (the values GGUF files carry).
enum : int { GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q8_0 = 8, GGML_Q4_K = 12, GGML_Q6_K = 14, GGML_BF16 = 30 };

__host__ __device__ inline bool fmt_is_16bit(int fmt) { return fmt == GGML_F16 || fmt == GGML_BF16; }
__host__ __device__ inline int fmt_block_elems(int fmt) {
  switch (fmt) {
    case GGML_Q4_0: case GGML_Q8_0: return 32;
    case GGML_Q4_K: case GGML_Q6_K: return 256;
    default: return 1;
  }
}
__host__ __device__ inline int fmt_block_bytes(int fmt) {
  switch (fmt) {
    case GGML_Q4_0: return 18;
    case GGML_Q8_0: return 34;
    case GGML_Q4_K: return 144;
    case GGML_Q6_K: return 210;
    case GGML_F16: case GGML_BF16: return 2;
    default: return 0;
  }
}
__host__ __device__ inline int fmt_brick_bytes(int fmt) {
  switch (fmt) {
    case GGML_Q4_0: return 2304;
    case GGML_Q8_0: return 4352;
    case GGML_Q4_K: return 2560;
    case GGML_Q6_K: return 3456;
    default: return 0;
  }
}

struct QWeight {
  int fmt = 0;
  int rows = 0, cols = 0;        // [out x in]
  int nbr = 0, nbk = 0;          // brick grid (each padded to an even count)
  uint8_t* bricks = nullptr;     // quantised formats
  void* dense16 = nullptr;       // F16 / BF16: row-major [rows x cols]
  // f32 weights (the reference's FrozenWeight::F32, src/frozen.rs:33-38): the exact values for
  // row(), and their two-term f16 split W = hi + lo for the tensor cores (hi in dense16 with
  // fmt = F16, lo = f16(W - hi) here: 17 to 22 significant bits together)
  const float* f32 = nullptr;
  void* dense16_lo = nullptr;
  size_t ggml_nbytes = 0;        // size of the original ggml tensor
  size_t dev_nbytes = 0;
};

// Exact (f32) value of element (r, k) from the brick store; mirrors ggml's dequantisation
// arithmetic operation for operation so rows come out bit-identical to a CPU dequantise.
__device__ inline float brick_value(const QWeight& w, int r, int k) {
  if (w.f32) return w.f32[(size_t)r * w.cols + k];
  if (w.fmt == GGML_F16) return __half2float(((const __half*)w.dense16)[(size_t)r * w.cols + k]);
  if (w.fmt == GGML_BF16) return __bfloat162float(((const __nv_bfloat16*)w.dense16)[(size_t)r * w.cols + k]);
  const uint8_t* b = w.bricks + ((size_t)(r >> 6) * w.nbk + (k >> 6)) * fmt_brick_bytes(w.fmt);
  int rr = r & 63, kk = k & 63;
  int t = rr * 2 + (kk >> 5);
  int e = kk & 31;                // element in unit
  int word = e >> 3, p = (e & 7) >> 1, hi = e & 1;
  int field = p + 4 * hi;
  switch (w.fmt) {
    case GGML_Q4_0: {
      uint32_t u = ((const uint32_t*)(b + t * 16))[word];
      int q = (u >> (4 * field)) & 15;
      float d = __half2float(((const __half*)(b + 2048))[t]);
      return __fmul_rn((float)(q - 8), d);
    }
    case GGML_Q8_0: {
      int q = (int)b[t * 32 + e] - 128;
      float d = __half2float(((const __half*)(b + 4096))[t]);
      return __fmul_rn((float)q, d);
    }
    case GGML_Q4_K: {
      uint32_t u = ((const uint32_t*)(b + t * 16))[word];
      int q = (u >> (4 * field)) & 15;
      const __half* dd = (const __half*)(b + 2048) + rr * 2;
      float d = __half2float(dd[0]), dmin = __half2float(dd[1]);
      float sc = (float)b[2304 + t * 2], m = (float)b[2304 + t * 2 + 1];
      return __fsub_rn(__fmul_rn(__fmul_rn(d, sc), (float)q), __fmul_rn(dmin, m));
    }
    case GGML_Q6_K: {
      uint32_t lo = ((const uint32_t*)(b + t * 16))[word];
      uint32_t hw = ((const uint32_t*)(b + 2048 + t * 8))[word >> 1];
      if (word & 1) hw = __funnelshift_r(hw, hw, 8);
      int q = ((lo >> (4 * field)) & 15) | (((hw >> (2 * p + 16 * hi)) & 0x30));
      float d = __half2float(((const __half*)(b + 3328))[rr]);
      float sc = (float)((const int8_t*)(b + 3072))[t * 2 + (e >> 4)];
      return __fmul_rn(__fmul_rn(d, sc), (float)(q - 32));
    }
  }
  return 0.f;
}

}  // namespace rt
