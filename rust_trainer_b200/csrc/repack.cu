// Upload-time re-tiling of ggml blocks into 64x64 bricks (see qformat.cuh), exact row
// dequantisation (FrozenMatmul::row, reference src/rie.rs:122-124) and the embedding gather
// built on it (Model::embed_tokens, reference src/model.rs:446-454).
#include "qformat.cuh"
#include "rt_internal.h"

namespace rt {

__device__ inline float f16_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// One thread per (row, 32-column) unit of the PADDED brick grid.
__global__ void repack_kernel(const uint8_t* __restrict__ raw, QWeight w) {
  const int units_per_row = w.nbk * 2;
  size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total = (size_t)w.nbr * 64 * units_per_row;
  if (gid >= total) return;
  int r = (int)(gid / units_per_row);
  int ku = (int)(gid % units_per_row);  // 32-column unit index along the row
  int k0 = ku * 32;
  const int bb = fmt_brick_bytes(w.fmt);
  uint8_t* b = w.bricks + ((size_t)(r >> 6) * w.nbk + (ku >> 1)) * bb;
  const int t = (r & 63) * 2 + (ku & 1);
  const bool inside = r < w.rows && k0 < w.cols;

  uint8_t code[32];
  for (int i = 0; i < 32; ++i) code[i] = 0;

  if (w.fmt == GGML_Q4_0) {
    uint16_t d = 0;
    if (inside) {
      const uint8_t* blk = raw + ((size_t)r * (w.cols / 32) + ku) * 18;
      d = blk[0] | (blk[1] << 8);
      for (int i = 0; i < 16; ++i) { code[i] = blk[2 + i] & 15; code[i + 16] = blk[2 + i] >> 4; }
    } else {
      for (int i = 0; i < 32; ++i) code[i] = 8;  // (8 - 8) * d = 0
    }
    uint32_t* dst = (uint32_t*)(b + t * 16);
    for (int wd = 0; wd < 4; ++wd) {
      uint32_t u = 0;
      for (int p = 0; p < 4; ++p) u |= (uint32_t)code[wd * 8 + 2 * p] << (4 * p) | (uint32_t)code[wd * 8 + 2 * p + 1] << (16 + 4 * p);
      dst[wd] = u;
    }
    ((uint16_t*)(b + 2048))[t] = d;
  } else if (w.fmt == GGML_Q8_0) {
    uint16_t d = 0;
    uint8_t* dst = b + t * 32;
    if (inside) {
      const uint8_t* blk = raw + ((size_t)r * (w.cols / 32) + ku) * 34;
      d = blk[0] | (blk[1] << 8);
      for (int i = 0; i < 32; ++i) dst[i] = blk[2 + i] ^ 0x80;  // int8 -> offset-128 unsigned
    } else {
      for (int i = 0; i < 32; ++i) dst[i] = 0x80;
    }
    ((uint16_t*)(b + 4096))[t] = d;
  } else if (w.fmt == GGML_Q4_K) {
    uint16_t d = 0, dmin = 0;
    uint8_t sc = 0, mn = 0;
    if (inside) {
      const uint8_t* blk = raw + ((size_t)r * (w.cols / 256) + (k0 >> 8)) * 144;
      d = blk[0] | (blk[1] << 8);
      dmin = blk[2] | (blk[3] << 8);
      const uint8_t* scales = blk + 4;
      const uint8_t* qs = blk + 16;
      int j = (k0 & 255) >> 5;  // sub-block 0..7
      if (j < 4) { sc = scales[j] & 63; mn = scales[j + 4] & 63; }
      else { sc = (scales[j + 4] & 0xF) | ((scales[j - 4] >> 6) << 4); mn = (scales[j + 4] >> 4) | ((scales[j] >> 6) << 4); }
      const uint8_t* q = qs + (j >> 1) * 32;
      for (int i = 0; i < 32; ++i) code[i] = (j & 1) ? (q[i] >> 4) : (q[i] & 15);
    }
    uint32_t* dst = (uint32_t*)(b + t * 16);
    for (int wd = 0; wd < 4; ++wd) {
      uint32_t u = 0;
      for (int p = 0; p < 4; ++p) u |= (uint32_t)code[wd * 8 + 2 * p] << (4 * p) | (uint32_t)code[wd * 8 + 2 * p + 1] << (16 + 4 * p);
      dst[wd] = u;
    }
    {  // both units of a brick row lie in one super-block and write the same (d, dmin)
      uint16_t* dd = (uint16_t*)(b + 2048) + (r & 63) * 2;
      dd[0] = d;
      dd[1] = dmin;
    }
    b[2304 + t * 2] = sc;
    b[2304 + t * 2 + 1] = mn;
  } else if (w.fmt == GGML_Q6_K) {
    uint16_t d = 0;
    int8_t s0 = 0, s1 = 0;
    for (int i = 0; i < 32; ++i) code[i] = 32;
    if (inside) {
      const uint8_t* blk = raw + ((size_t)r * (w.cols / 256) + (k0 >> 8)) * 210;
      const uint8_t* ql = blk;
      const uint8_t* qh = blk + 128;
      const int8_t* scs = (const int8_t*)(blk + 192);
      d = blk[208] | (blk[209] << 8);
      int e0 = k0 & 255;          // first element of this unit inside the super-block
      int half = e0 >> 7;         // which 128-element half
      int quarter = (e0 & 127) >> 5;  // 0..3: y[l], y[l+32], y[l+64], y[l+96]
      const uint8_t* qlh = ql + half * 64;
      const uint8_t* qhh = qh + half * 32;
      for (int l = 0; l < 32; ++l) {
        int lo = (quarter & 1) ? qlh[l + 32] : qlh[l];
        lo = (quarter & 2) ? (lo >> 4) : (lo & 15);
        int hi = (qhh[l] >> (2 * quarter)) & 3;
        code[l] = lo | (hi << 4);
      }
      s0 = scs[half * 8 + quarter * 2];
      s1 = scs[half * 8 + quarter * 2 + 1];
    }
    uint32_t* dlo = (uint32_t*)(b + t * 16);
    uint32_t* dhi = (uint32_t*)(b + 2048 + t * 8);
    uint32_t H[2] = {0, 0};
    for (int wd = 0; wd < 4; ++wd) {
      uint32_t u = 0;
      for (int p = 0; p < 4; ++p) {
        for (int hi = 0; hi < 2; ++hi) {
          int c = code[wd * 8 + 2 * p + hi];
          u |= (uint32_t)(c & 15) << (4 * p + 16 * hi);
          int pos = 4 + 2 * p + 16 * hi;
          if (wd & 1) pos = (pos + 8) & 31;
          H[wd >> 1] |= (uint32_t)(c >> 4) << pos;
        }
      }
      dlo[wd] = u;
    }
    dhi[0] = H[0];
    dhi[1] = H[1];
    ((int8_t*)(b + 3072))[t * 2] = s0;
    ((int8_t*)(b + 3072))[t * 2 + 1] = s1;
    ((uint16_t*)(b + 3328))[r & 63] = d;  // same value from both units of the brick row
  }
}

void launch_repack(const uint8_t* raw_dev, const QWeight& w, cudaStream_t st) {
  size_t total = (size_t)w.nbr * 64 * w.nbk * 2;
  int threads = 128;
  size_t blocks = (total + threads - 1) / threads;
  { repack_kernel<<<(unsigned)blocks, threads, 0, st>>>(raw_dev, w); RT_COUNT_LAUNCH(1); }
}

// out[i, :] = dequantised row ids[i]  (f32, and optionally a bf16 copy)
__global__ void gather_rows_kernel(QWeight w, const int* __restrict__ ids, int n, float* __restrict__ out,
                                   int* status) {
  int i = blockIdx.x;
  if (i >= n) return;
  int r = ids ? ids[i] : i;
  if (r < 0 || r >= w.rows) {
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_BAD_INDEX);
    return;
  }
  for (int k = threadIdx.x; k < w.cols; k += blockDim.x) out[(size_t)i * w.cols + k] = brick_value(w, r, k);
}

void launch_gather_rows(const QWeight& w, const int* ids_dev, int n, float* out, int* status, cudaStream_t st) {
  if (n <= 0) return;
  { gather_rows_kernel<<<n, 256, 0, st>>>(w, ids_dev, n, out, status); RT_COUNT_LAUNCH(1); }
}

}  // namespace rt
