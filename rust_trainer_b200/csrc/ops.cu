// Memory-bound device ops around the frozen matmuls: RMSNorm, QK-norm + RoPE, SwiGLU,
// cross-entropy, row gathers, LoRA gradient reductions, AdamW.  One CTA per token row unless
// noted.  Every kernel that produces the 16-bit input of a backward matmul writes the row
// divided by its largest magnitude plus that magnitude as a per-row scale: f16 then keeps 11
// significant bits whatever the size of the gradients, and the matmul's epilogue multiplies
// the scale back in (the matmul is linear in each token row).
#include "ctx.h"
#include "ops.h"
#include "pdl.cuh"

namespace rt {

// ------------------------------------------------------------------ reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Block-wide reductions (blockDim.x <= 1024); result broadcast to every thread.
__device__ float block_sum(float v) {
  __shared__ float sh[33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < (int)((blockDim.x + 31) >> 5) ? sh[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) sh[32] = t;
  }
  __syncthreads();
  return sh[32];
}
__device__ float block_max(float v) {
  __shared__ float sh[33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < (int)((blockDim.x + 31) >> 5) ? sh[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) sh[32] = t;
  }
  __syncthreads();
  return sh[32];
}
__device__ double block_sum_d(double v) {
  __shared__ double sh[33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum_d(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  if (w == 0) {
    double t = lane < (int)((blockDim.x + 31) >> 5) ? sh[lane] : 0.0;
    t = warp_sum_d(t);
    if (lane == 0) sh[32] = t;
  }
  __syncthreads();
  return sh[32];
}

// ------------------------------------------------------------------ conversions
template <bool F16>
__global__ void f32_to_16_kernel(const float* __restrict__ in, uint16_t* __restrict__ out, size_t n) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 v = *(const float4*)(in + i);
    uint32_t a, b;
    if (F16) {
      __half2 x = __floats2half2_rn(v.x, v.y), y = __floats2half2_rn(v.z, v.w);
      a = *(uint32_t*)&x; b = *(uint32_t*)&y;
    } else {
      __nv_bfloat162 x = __floats2bfloat162_rn(v.x, v.y), y = __floats2bfloat162_rn(v.z, v.w);
      a = *(uint32_t*)&x; b = *(uint32_t*)&y;
    }
    *(uint2*)(out + i) = make_uint2(a, b);
  } else {
    for (; i < n; ++i) {
      if (F16) { __half h = __float2half_rn(in[i]); out[i] = *(uint16_t*)&h; }
      else { __nv_bfloat16 h = __float2bfloat16_rn(in[i]); out[i] = *(uint16_t*)&h; }
    }
  }
}
void launch_f32_to_16(const float* in, void* out, size_t n, bool to_f16, cudaStream_t st) {
  if (n == 0) return;
  size_t threads = (n + 3) / 4;
  unsigned blocks = (unsigned)((threads + 255) / 256);
  if (to_f16) { f32_to_16_kernel<true><<<blocks, 256, 0, st>>>(in, (uint16_t*)out, n); RT_COUNT_LAUNCH(1); }
  else { f32_to_16_kernel<false><<<blocks, 256, 0, st>>>(in, (uint16_t*)out, n); RT_COUNT_LAUNCH(1); }
}

__global__ void split_f32_hi_lo_kernel(const float* __restrict__ w, size_t n, __half* __restrict__ hi, __half* __restrict__ lo) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = w[i];
  const __half h = __float2half_rn(v);
  hi[i] = h;
  lo[i] = __float2half_rn(v - __half2float(h));
}
void launch_split_f32_hi_lo(const float* w, size_t n, __half* hi, __half* lo, cudaStream_t st) {
  if (n == 0) return;
  split_f32_hi_lo_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w, n, hi, lo);
  RT_COUNT_LAUNCH(1);
}

// Row-normalised f16 copy: y16[r,:] = x[r,:] / amax_r, scale[r] = amax_r (1 if the row is zero).
__global__ void normalize_rows_kernel(const float* __restrict__ x, int d, __half* __restrict__ y16,
                                      float* __restrict__ scale) {
  pdl_entry();
  const size_t r = blockIdx.x;
  const float* xr = x + r * d;
  float m = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) m = fmaxf(m, fabsf(xr[i]));
  m = block_max(m);
  const float s = m > 0.f ? m : 1.f, inv = 1.f / s;
  for (int i = threadIdx.x; i < d; i += blockDim.x) y16[r * d + i] = __float2half_rn(xr[i] * inv);
  // an all-zero row reports the factor 0, not 1: consumers that weigh rows by factor / largest
  // factor (attention backward, the token contractions) must not see a 1 that towers over the
  // real rows' small factors and pushes their f16 products into the subnormals
  if (threadIdx.x == 0) scale[r] = m;
}
void launch_normalize_rows(const float* x, int rows, int d, __half* y16, float* scale, cudaStream_t st) {
  if (rows > 0) { pdl(normalize_rows_kernel, rows, 256, 0, st)(x, d, y16, scale); RT_COUNT_LAUNCH(1); }
}

// ------------------------------------------------------------------ RMSNorm (reference src/ops.rs:8-56)
// y16 = x * ir * w  with ir = 1/sqrt(mean(x^2) + eps)
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w, int d, float eps,
                                   __half* __restrict__ y16) {
  const size_t r = blockIdx.x;
  const float* xr = x + r * d;
  float ss = 0.f;
  if ((d & 3) == 0) {
    const float4* x4 = (const float4*)xr;
    const float4* w4 = (const float4*)w;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
      const float4 v = x4[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss);
    const float ir = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
      const float4 v = x4[i], g = w4[i];
      __half2 a = __floats2half2_rn(v.x * ir * g.x, v.y * ir * g.y), b = __floats2half2_rn(v.z * ir * g.z, v.w * ir * g.w);
      *(uint2*)(y16 + r * d + 4 * i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
    return;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss);
  const float ir = 1.0f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) y16[r * d + i] = __float2half_rn(xr[i] * ir * w[i]);
}
// Warp-per-row versions for rows of up to 1024 floats (a multiple of 128): the row lives in
// registers, the reductions are warp shuffles, and eight rows per CTA keep far more bytes in
// flight per SM than one small CTA per row.
template <int NV>  // float4s per lane: d = 128 * NV
__global__ void __launch_bounds__(256)
rmsnorm_fwd_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, int rows, float eps,
                        __half* __restrict__ y16) {
  pdl_entry();
  constexpr int D = 128 * NV;
  const int lane = threadIdx.x & 31;
  const size_t r = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= (size_t)rows) return;
  const float4* x4 = (const float4*)(x + r * D);
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    v[k] = x4[lane + 32 * k];
    ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  ss = warp_sum(ss);
  const float ir = 1.0f / sqrtf(ss / (float)D + eps);
  const float4* w4 = (const float4*)w;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const float4 g = w4[lane + 32 * k];
    __half2 a = __floats2half2_rn(v[k].x * ir * g.x, v[k].y * ir * g.y), b = __floats2half2_rn(v[k].z * ir * g.z, v[k].w * ir * g.w);
    *(uint2*)(y16 + r * D + 4 * (lane + 32 * k)) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
  }
}
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ dn,
                        const float* dres, int rows, float eps, float* out, __half* __restrict__ out16,
                        float* __restrict__ scale) {
  pdl_entry();
  constexpr int D = 128 * NV;
  const int lane = threadIdx.x & 31;
  const size_t r = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= (size_t)rows) return;
  const float4 *x4 = (const float4*)(x + r * D), *d4 = (const float4*)(dn + r * D), *w4 = (const float4*)w;
  float4 xv[NV], gv[NV], rv[NV];
  float ss = 0.f, gx = 0.f;
  // every load of the row is issued before the first reduction: one round of memory latency, not two
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    xv[k] = x4[lane + 32 * k];
    gv[k] = d4[lane + 32 * k];
    rv[k] = dres ? ((const float4*)(dres + r * D))[lane + 32 * k] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const float4 wv = w4[lane + 32 * k];
    gv[k] = make_float4(gv[k].x * wv.x, gv[k].y * wv.y, gv[k].z * wv.z, gv[k].w * wv.w);
    ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
    gx += gv[k].x * xv[k].x + gv[k].y * xv[k].y + gv[k].z * xv[k].z + gv[k].w * xv[k].w;
  }
  ss = warp_sum(ss);
  gx = warp_sum(gx);
  const float ir = 1.0f / sqrtf(ss / (float)D + eps);
  const float c = gx * ir * ir * ir / (float)D;
  float m = 0.f;
  float4* o4 = (float4*)(out + r * D);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float4 v = make_float4(gv[k].x * ir - xv[k].x * c, gv[k].y * ir - xv[k].y * c, gv[k].z * ir - xv[k].z * c,
                           gv[k].w * ir - xv[k].w * c);
    v.x += rv[k].x; v.y += rv[k].y; v.z += rv[k].z; v.w += rv[k].w;
    o4[lane + 32 * k] = v;
    gv[k] = v;
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  if (out16) {
    m = warp_max(m);
    const float sc = m > 0.f ? m : 1.f, inv = 1.f / sc;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      __half2 a = __floats2half2_rn(gv[k].x * inv, gv[k].y * inv), b = __floats2half2_rn(gv[k].z * inv, gv[k].w * inv);
      *(uint2*)(out16 + r * D + 4 * (lane + 32 * k)) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
    if (lane == 0) scale[r] = m;
  }
}
void launch_rmsnorm_fwd(const float* x, const float* w, int rows, int d, float eps, __half* y16, cudaStream_t st) {
  if (rows <= 0) return;
  const int nv = d / 128, grid = (rows + 7) / 8;
  const bool warp_ok = d % 128 == 0 && nv >= 1 && nv <= 8 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
  if (warp_ok) {
    switch (nv) {
      case 1: pdl(rmsnorm_fwd_warp_kernel<1>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      case 2: pdl(rmsnorm_fwd_warp_kernel<2>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      case 3: pdl(rmsnorm_fwd_warp_kernel<3>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      case 4: pdl(rmsnorm_fwd_warp_kernel<4>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      case 5: pdl(rmsnorm_fwd_warp_kernel<5>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      case 6: pdl(rmsnorm_fwd_warp_kernel<6>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      case 7: pdl(rmsnorm_fwd_warp_kernel<7>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
      default: pdl(rmsnorm_fwd_warp_kernel<8>, grid, 256, 0, st)(x, w, rows, eps, y16); break;
    }
  } else {
    rmsnorm_fwd_kernel<<<rows, 256, 0, st>>>(x, w, d, eps, y16);
  }
  RT_COUNT_LAUNCH(1);
}

// dx = g*ir - x*c, g = dn*w, c = dot(g,x)*ir^3/d;  out = (dres ? dres : 0) + dx.
// Optionally also the row-normalised f16 copy of `out` and its scale.
__global__ void rmsnorm_bwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   const float* __restrict__ dn, const float* dres, int d, float eps, float* out,
                                   __half* __restrict__ out16, float* __restrict__ scale) {
  const size_t r = blockIdx.x;
  const float* xr = x + r * d;
  const float* dnr = dn + r * d;
  float ss = 0.f, gx = 0.f, m = 0.f;
  if ((d & 3) == 0) {
    const float4 *x4 = (const float4*)xr, *d4 = (const float4*)dnr, *w4 = (const float4*)w;
    const float4* r4 = dres ? (const float4*)(dres + r * d) : nullptr;
    float4* o4 = (float4*)(out + r * d);
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
      const float4 xv = x4[i], dv = d4[i], wv = w4[i];
      ss += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
      gx += dv.x * wv.x * xv.x + dv.y * wv.y * xv.y + dv.z * wv.z * xv.z + dv.w * wv.w * xv.w;
    }
    ss = block_sum(ss);
    gx = block_sum(gx);
    const float ir = 1.0f / sqrtf(ss / (float)d + eps);
    const float c = gx * ir * ir * ir / (float)d;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
      const float4 xv = x4[i], dv = d4[i], wv = w4[i];
      float4 v = make_float4(dv.x * wv.x * ir - xv.x * c, dv.y * wv.y * ir - xv.y * c, dv.z * wv.z * ir - xv.z * c,
                             dv.w * wv.w * ir - xv.w * c);
      if (r4) { const float4 q = r4[i]; v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w; }
      o4[i] = v;
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    if (out16) {
      m = block_max(m);
      const float sc = m > 0.f ? m : 1.f, inv = 1.f / sc;
      for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        const float4 v = o4[i];  // this thread's own stores
        __half2 a = __floats2half2_rn(v.x * inv, v.y * inv), b = __floats2half2_rn(v.z * inv, v.w * inv);
        *(uint2*)(out16 + r * d + 4 * i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      }
      if (threadIdx.x == 0) scale[r] = m;
    }
    return;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float xv = xr[i];
    ss += xv * xv;
    gx += dnr[i] * w[i] * xv;
  }
  ss = block_sum(ss);
  gx = block_sum(gx);
  const float ir = 1.0f / sqrtf(ss / (float)d + eps);
  const float c = gx * ir * ir * ir / (float)d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = dnr[i] * w[i] * ir - xr[i] * c;
    if (dres) v += dres[r * d + i];
    out[r * d + i] = v;
    m = fmaxf(m, fabsf(v));
  }
  if (out16) {
    m = block_max(m);  // includes a __syncthreads: this thread's stores above are its own re-reads below
    const float sc = m > 0.f ? m : 1.f, inv = 1.f / sc;
    for (int i = threadIdx.x; i < d; i += blockDim.x) out16[r * d + i] = __float2half_rn(out[r * d + i] * inv);
    if (threadIdx.x == 0) scale[r] = m;
  }
}
void launch_rmsnorm_bwd(const float* x, const float* w, const float* dn, const float* dres, int rows, int d, float eps,
                        float* out, __half* out16, float* scale, cudaStream_t st) {
  if (rows <= 0) return;
  const int nv = d / 128, grid = (rows + 7) / 8;
  const bool warp_ok = d % 128 == 0 && nv >= 1 && nv <= 8 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
                       ((uintptr_t)dn & 15) == 0 && ((uintptr_t)out & 15) == 0 && (!dres || ((uintptr_t)dres & 15) == 0);
  if (warp_ok) {
#define RT_RMSB(N) pdl(rmsnorm_bwd_warp_kernel<N>, grid, 256, 0, st)(x, w, dn, dres, rows, eps, out, out16, scale)
    switch (nv) {
      case 1: RT_RMSB(1); break;
      case 2: RT_RMSB(2); break;
      case 3: RT_RMSB(3); break;
      case 4: RT_RMSB(4); break;
      case 5: RT_RMSB(5); break;
      case 6: RT_RMSB(6); break;
      case 7: RT_RMSB(7); break;
      default: RT_RMSB(8); break;
    }
#undef RT_RMSB
  } else {
    rmsnorm_bwd_kernel<<<rows, 256, 0, st>>>(x, w, dn, dres, d, eps, out, out16, scale);
  }
  RT_COUNT_LAUNCH(1);
}

// ------------------------------------------------------------------ RoPE tables (reference src/ops.rs:118-154)
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int half, int max_pos, float* __restrict__ cs,
                                  float* __restrict__ sn) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= max_pos * half) return;
  int p = i / half, f = i % half;
  float a = (float)p * inv_freq[f];
  cs[i] = cosf(a);
  sn[i] = sinf(a);
}
void launch_rope_table(const float* inv_freq, int half, int max_pos, float* cs, float* sn, cudaStream_t st) {
  int n = max_pos * half;
  if (n > 0) { rope_table_kernel<<<(n + 255) / 256, 256, 0, st>>>(inv_freq, half, max_pos, cs, sn); RT_COUNT_LAUNCH(1); }
}

// ------------------------------------------------------------------ QK-norm + RoPE + f16 rounding
// (reference src/attention.rs:170-185).  One CTA per token, one warp per head in turn.
// Heads 0..nh-1 are q, nh..nh+nkv-1 are k, then nkv heads of v (copied and rounded only).
__global__ void qk_rope_fwd_kernel(const float* __restrict__ q_raw, const float* __restrict__ k_raw,
                                   const float* __restrict__ v_raw, const float* __restrict__ qw,
                                   const float* __restrict__ kw, const int* __restrict__ pos,
                                   const float* __restrict__ cs, const float* __restrict__ sn, int nh, int nkv, int hd,
                                   int rot, int neox, float eps, __half* __restrict__ q16, __half* __restrict__ k16,
                                   __half* __restrict__ v16) {
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int half = rot / 2;
  const int p = pos[m];
  const float* csr = cs + (size_t)p * half;
  const float* snr = sn + (size_t)p * half;
  for (int h = warp; h < nh + 2 * nkv; h += nwarps) {
    if (h >= nh + nkv) {
      const int hv = h - nh - nkv;
      const float* src = v_raw + (m * nkv + hv) * hd;
      __half* dst = v16 + (m * nkv + hv) * hd;
      for (int i = lane * 4; i < hd; i += 128) {
        const float4 v = *(const float4*)(src + i);
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        *(uint2*)(dst + i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      }
      continue;
    }
    const bool is_q = h < nh;
    const float* src = is_q ? q_raw + (m * nh + h) * hd : k_raw + (m * nkv + (h - nh)) * hd;
    const float* nw = is_q ? qw : kw;
    __half* dst = is_q ? q16 + (m * nh + h) * hd : k16 + (m * nkv + (h - nh)) * hd;
    float ir = 1.f;
    if (nw) {
      float ss = 0.f;
      for (int i = lane * 4; i < hd; i += 128) {
        const float4 v = *(const float4*)(src + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      ir = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    // two rotation pairs per lane and round; elements beyond rot pass through
    for (int i = lane * 2; i < half; i += 64) {
      const float2 c = *(const float2*)(csr + i), s = *(const float2*)(snr + i);
      if (neox) {
        float2 x1 = *(const float2*)(src + i), x2 = *(const float2*)(src + i + half);
        if (nw) {
          const float2 w1 = *(const float2*)(nw + i), w2 = *(const float2*)(nw + i + half);
          x1.x *= ir * w1.x; x1.y *= ir * w1.y; x2.x *= ir * w2.x; x2.y *= ir * w2.y;
        }
        *(__half2*)(dst + i) = __floats2half2_rn(x1.x * c.x - x2.x * s.x, x1.y * c.y - x2.y * s.y);
        *(__half2*)(dst + i + half) = __floats2half2_rn(x2.x * c.x + x1.x * s.x, x2.y * c.y + x1.y * s.y);
      } else {
        float4 x = *(const float4*)(src + 2 * i);  // pairs (2i, 2i+1), (2i+2, 2i+3)
        if (nw) {
          const float4 w4 = *(const float4*)(nw + 2 * i);
          x.x *= ir * w4.x; x.y *= ir * w4.y; x.z *= ir * w4.z; x.w *= ir * w4.w;
        }
        __half2 a = __floats2half2_rn(x.x * c.x - x.y * s.x, x.y * c.x + x.x * s.x);
        __half2 b = __floats2half2_rn(x.z * c.y - x.w * s.y, x.w * c.y + x.z * s.y);
        *(uint2*)(dst + 2 * i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
      }
    }
    for (int i = rot + lane; i < hd; i += 32) {
      float x = src[i];
      if (nw) x = x * (ir * nw[i]);
      dst[i] = __float2half_rn(x);
    }
  }
}

// Register-resident versions of the two kernels above for the usual shapes (head size 64 or
// 128, at most 8 heads per warp): a warp holds a whole head, EPL consecutive elements per lane,
// so every global load of a token's heads is issued before any of them is used, the rotation
// partner comes from a lane shuffle, and nothing is staged in shared memory.
template <int EPL>
struct RopeLane {
  // what lane `lane` needs to rotate its EPL elements of one head
  float c[EPL], s[EPL];  // cos, and sin signed for the FORWARD rotation (0 / 1 beyond rot)
  int src_lane;          // neox: the lane holding the partner elements; interleaved: unused
  bool rotates;
};
template <int EPL>
__device__ __forceinline__ RopeLane<EPL> rope_lane(int lane, const float* csr, const float* snr, int half, int rot, int neox) {
  RopeLane<EPL> r;
  const int e0 = lane * EPL;
  r.rotates = e0 < rot;
  r.src_lane = lane;
#pragma unroll
  for (int k = 0; k < EPL; ++k) { r.c[k] = 1.f; r.s[k] = 0.f; }
  if (!r.rotates) return r;
  if (neox) {
    const bool first = e0 < half;
    r.src_lane = first ? lane + half / EPL : lane - half / EPL;
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      const int i = first ? e0 + k : e0 + k - half;
      r.c[k] = csr[i];
      r.s[k] = first ? -snr[i] : snr[i];
    }
  } else {
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      const int i = (e0 + k) >> 1;
      r.c[k] = csr[i];
      r.s[k] = (k & 1) ? snr[i] : -snr[i];
    }
  }
  return r;
}
// out = own*c + partner*s*dir  (dir = +1 forward, -1 inverse)
template <int EPL>
__device__ __forceinline__ void rope_apply(const RopeLane<EPL>& r, int neox, float dir, const float* x, float* out) {
  float partner[EPL];
  if (neox) {
#pragma unroll
    for (int k = 0; k < EPL; ++k) partner[k] = __shfl_sync(0xffffffffu, x[k], r.src_lane);
  } else {
#pragma unroll
    for (int k = 0; k < EPL; ++k) partner[k] = x[k ^ 1];
  }
#pragma unroll
  for (int k = 0; k < EPL; ++k) out[k] = x[k] * r.c[k] + partner[k] * (r.s[k] * dir);
}
template <int EPL>
__device__ __forceinline__ void load_epl(const float* p, float* v) {
  if (EPL == 4) { const float4 t = *(const float4*)p; v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  else { const float2 t = *(const float2*)p; v[0] = t.x; v[1] = t.y; }
}
template <int EPL>
__device__ __forceinline__ void store_epl_h(__half* p, const float* v) {
  if (EPL == 4) {
    __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    *(uint2*)p = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
  } else {
    *(__half2*)p = __floats2half2_rn(v[0], v[1]);
  }
}

template <int EPL, int HPW>
__global__ void __launch_bounds__(256)
qk_rope_fwd_reg_kernel(const float* __restrict__ q_raw, const float* __restrict__ k_raw, const float* __restrict__ v_raw,
                       size_t pq, size_t pk, size_t pv,  // row pitches of the three inputs, in elements
                       const float* __restrict__ qw, const float* __restrict__ kw, const int* __restrict__ pos,
                       const float* __restrict__ cs, const float* __restrict__ sn, int nh, int nkv, int rot, int neox,
                       float eps, __half* __restrict__ q16, __half* __restrict__ k16, __half* __restrict__ v16) {
  pdl_entry();
  constexpr int HD = 32 * EPL;
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = rot / 2, nheads = nh + 2 * nkv;
  // the rows first: the position -> cos/sin table chain is two dependent loads, which then run under them
  float x[HPW][EPL];
#pragma unroll
  for (int t = 0; t < HPW; ++t) {
    const int h = warp + t * 8;
    if (h < nheads) {
      const float* src = h < nh ? q_raw + m * pq + h * HD : (h < nh + nkv ? k_raw + m * pk + (h - nh) * HD
                                                                         : v_raw + m * pv + (h - nh - nkv) * HD);
      load_epl<EPL>(src + lane * EPL, x[t]);
    }
  }
  const int p = pos[m];
  const RopeLane<EPL> rl = rope_lane<EPL>(lane, cs + (size_t)p * half, sn + (size_t)p * half, half, rot, neox);
#pragma unroll
  for (int t = 0; t < HPW; ++t) {
    const int h = warp + t * 8;
    if (h >= nheads) continue;  // uniform in the warp
    if (h >= nh + nkv) {
      store_epl_h<EPL>(v16 + (m * nkv + (h - nh - nkv)) * HD + lane * EPL, x[t]);
      continue;
    }
    const bool is_q = h < nh;
    const float* nw = is_q ? qw : kw;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) ss += x[t][k] * x[t][k];
      ss = warp_sum(ss);
      const float ir = 1.0f / sqrtf(ss / (float)HD + eps);
      float w[EPL];
      load_epl<EPL>(nw + lane * EPL, w);
#pragma unroll
      for (int k = 0; k < EPL; ++k) x[t][k] *= ir * w[k];
    }
    float o[EPL];
    rope_apply<EPL>(rl, neox, 1.f, x[t], o);
    __half* dst = is_q ? q16 + (m * nh + h) * HD : k16 + (m * nkv + (h - nh)) * HD;
    store_epl_h<EPL>(dst + lane * EPL, o);
  }
}

// The same for the common geometry with nothing left to decide per head: full rotation
// (rot == head_dim), query and KV head counts that are multiples of the CTA's eight warps (warp w
// owns query heads w, w + 8, .. and KV heads w, w + 8, ..), both norms present or both absent.  The
// general kernel above spends more issue slots on choosing pointers and on uniform branches than on
// arithmetic; it is bound by instruction issue, not by bytes.
template <int EPL, int QPW, int KPW, bool NEOX, bool NORM>
__global__ void __launch_bounds__(256)
qk_rope_fwd_fast_kernel(const float* __restrict__ q_raw, const float* __restrict__ k_raw, const float* __restrict__ v_raw,
                        size_t pq, size_t pk, size_t pv, const float* __restrict__ qw, const float* __restrict__ kw,
                        const int* __restrict__ pos, const float* __restrict__ cs, const float* __restrict__ sn, float eps,
                        __half* __restrict__ q16, __half* __restrict__ k16, __half* __restrict__ v16) {
  pdl_entry();
  constexpr int HD = 32 * EPL, HALF = HD / 2, NH = 8 * QPW, NKV = 8 * KPW;
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = lane * EPL;
  const float* qs = q_raw + m * pq + warp * HD + e0;
  const float* ks = k_raw + m * pk + warp * HD + e0;
  const float* vs = v_raw + m * pv + warp * HD + e0;
  float xq[QPW][EPL], xk[KPW][EPL], xv[KPW][EPL];
#pragma unroll
  for (int t = 0; t < QPW; ++t) load_epl<EPL>(qs + t * 8 * HD, xq[t]);
#pragma unroll
  for (int t = 0; t < KPW; ++t) load_epl<EPL>(ks + t * 8 * HD, xk[t]);
#pragma unroll
  for (int t = 0; t < KPW; ++t) load_epl<EPL>(vs + t * 8 * HD, xv[t]);
  float wq[EPL], wk[EPL];
  if (NORM) {
    load_epl<EPL>(qw + e0, wq);
    load_epl<EPL>(kw + e0, wk);
  }
  // the position -> cos/sin chain (two dependent loads) runs under the row loads
  const int p = pos[m];
  const float* csr = cs + (size_t)p * HALF;
  const float* snr = sn + (size_t)p * HALF;
  float c[EPL], sg[EPL];
  if (NEOX) {
    const bool first = e0 < HALF;
    float sv_[EPL];
    load_epl<EPL>(csr + (first ? e0 : e0 - HALF), c);
    load_epl<EPL>(snr + (first ? e0 : e0 - HALF), sv_);
#pragma unroll
    for (int k = 0; k < EPL; ++k) sg[k] = first ? -sv_[k] : sv_[k];
  } else {
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      c[k] = csr[(e0 + k) >> 1];
      const float t = snr[(e0 + k) >> 1];
      sg[k] = (k & 1) ? t : -t;
    }
  }
  auto finish = [&](float* x, const float* w, __half* dst) {
    if (NORM) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) ss += x[k] * x[k];
      ss = warp_sum(ss);
      const float ir = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
      for (int k = 0; k < EPL; ++k) x[k] *= ir * w[k];
    }
    float o[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      const float partner = NEOX ? __shfl_xor_sync(0xffffffffu, x[k], 16) : x[k ^ 1];
      o[k] = x[k] * c[k] + partner * sg[k];
    }
    store_epl_h<EPL>(dst, o);
  };
#pragma unroll
  for (int t = 0; t < QPW; ++t) finish(xq[t], wq, q16 + (m * NH + warp + 8 * t) * HD + e0);
#pragma unroll
  for (int t = 0; t < KPW; ++t) finish(xk[t], wk, k16 + (m * NKV + warp + 8 * t) * HD + e0);
#pragma unroll
  for (int t = 0; t < KPW; ++t) store_epl_h<EPL>(v16 + (m * NKV + warp + 8 * t) * HD + e0, xv[t]);
}

template <int EPL, int HPW>
__global__ void __launch_bounds__(256, 4)
qk_rope_bwd_reg_kernel(const float* __restrict__ dq, const float* __restrict__ dk, const float* __restrict__ dv,
                       const float* __restrict__ q_raw, const float* __restrict__ k_raw, size_t pq, size_t pk,
                       size_t oq, size_t ok, size_t ov, int common,  // output row pitches; one scale for all three
                       const float* __restrict__ qw,
                       const float* __restrict__ kw, const int* __restrict__ pos, const float* __restrict__ cs,
                       const float* __restrict__ sn, int nh, int nkv, int rot, int neox, float eps,
                       __half* __restrict__ dq16, __half* __restrict__ dk16, __half* __restrict__ dv16,
                       float* __restrict__ sq, float* __restrict__ sk, float* __restrict__ sv) {
  pdl_entry();
  constexpr int HD = 32 * EPL;
  __shared__ float wmax[3][8];
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = rot / 2, nheads = nh + 2 * nkv;
  float g[HPW][EPL], xr[HPW][EPL];
#pragma unroll
  for (int t = 0; t < HPW; ++t) {
    const int h = warp + t * 8;
    if (h < nheads) {
      const float* src = h < nh ? dq + (m * nh + h) * HD : (h < nh + nkv ? dk + (m * nkv + (h - nh)) * HD
                                                                        : dv + (m * nkv + (h - nh - nkv)) * HD);
      load_epl<EPL>(src + lane * EPL, g[t]);
      const float* nw = h < nh ? qw : (h < nh + nkv ? kw : nullptr);
      if (nw) load_epl<EPL>((h < nh ? q_raw + m * pq + h * HD : k_raw + m * pk + (h - nh) * HD) + lane * EPL, xr[t]);
    }
  }
  // after the rows: the position -> cos/sin table chain (two dependent loads) runs under them
  const int p = pos[m];
  const RopeLane<EPL> rl = rope_lane<EPL>(lane, cs + (size_t)p * half, sn + (size_t)p * half, half, rot, neox);
  float mx[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int t = 0; t < HPW; ++t) {
    const int h = warp + t * 8;
    if (h >= nheads) continue;
    const int kind = h < nh ? 0 : (h < nh + nkv ? 1 : 2);
    if (kind < 2) {
      float o[EPL];
      rope_apply<EPL>(rl, neox, -1.f, g[t], o);  // inverse rotation
      const float* nw = kind == 0 ? qw : kw;
      if (nw) {
        float w[EPL];
        load_epl<EPL>(nw + lane * EPL, w);
        float ss = 0.f, gx = 0.f;
#pragma unroll
        for (int k = 0; k < EPL; ++k) { ss += xr[t][k] * xr[t][k]; gx += o[k] * w[k] * xr[t][k]; }
        ss = warp_sum(ss);
        gx = warp_sum(gx);
        const float ir = 1.0f / sqrtf(ss / (float)HD + eps);
        const float c = gx * ir * ir * ir / (float)HD;
#pragma unroll
        for (int k = 0; k < EPL; ++k) o[k] = o[k] * w[k] * ir - xr[t][k] * c;
      }
#pragma unroll
      for (int k = 0; k < EPL; ++k) g[t][k] = o[k];
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k) mx[kind] = fmaxf(mx[kind], fabsf(g[t][k]));
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float v = warp_max(mx[k]);
    if (lane == 0) wmax[k][warp] = v;
  }
  __syncthreads();
  float s3[3], inv[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) v = fmaxf(v, wmax[k][w]);
    s3[k] = v;
  }
  if (common) s3[0] = s3[1] = s3[2] = fmaxf(s3[0], fmaxf(s3[1], s3[2]));
#pragma unroll
  if (threadIdx.x == 0) { sq[m] = s3[0]; sk[m] = s3[1]; sv[m] = s3[2]; }  // 0 for an all-zero row
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    s3[k] = s3[k] > 0.f ? s3[k] : 1.f;
    inv[k] = 1.f / s3[k];
  }
#pragma unroll
  for (int t = 0; t < HPW; ++t) {
    const int h = warp + t * 8;
    if (h >= nheads) continue;
    const int kind = h < nh ? 0 : (h < nh + nkv ? 1 : 2);
    float o[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) o[k] = g[t][k] * inv[kind];
    __half* dst = kind == 0 ? dq16 + m * oq + h * HD : (kind == 1 ? dk16 + m * ok + (h - nh) * HD
                                                                   : dv16 + m * ov + (h - nh - nkv) * HD);
    store_epl_h<EPL>(dst + lane * EPL, o);
  }
}

// Backward for the same common geometry as qk_rope_fwd_fast_kernel (full rotation, head counts
// that are multiples of eight, both norms or none): no per-head decisions left.
template <int EPL, int QPW, int KPW, bool NEOX, bool NORM>
__global__ void __launch_bounds__(256, (QPW + 2 * KPW <= 4) ? 4 : ((QPW + 2 * KPW <= 6) ? 3 : 2))
qk_rope_bwd_fast_kernel(const float* __restrict__ dq, const float* __restrict__ dk, const float* __restrict__ dv,
                        const float* __restrict__ q_raw, const float* __restrict__ k_raw, size_t pq, size_t pk, size_t oq,
                        size_t ok, size_t ov, int common, const float* __restrict__ qw, const float* __restrict__ kw,
                        const int* __restrict__ pos, const float* __restrict__ cs, const float* __restrict__ sn, float eps,
                        __half* __restrict__ dq16, __half* __restrict__ dk16, __half* __restrict__ dv16,
                        float* __restrict__ sq, float* __restrict__ sk, float* __restrict__ sv) {
  pdl_entry();
  constexpr int HD = 32 * EPL, HALF = HD / 2, NH = 8 * QPW, NKV = 8 * KPW;
  __shared__ float wmax[3][8];
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = lane * EPL;
  float gq[QPW][EPL], gk[KPW][EPL], gv[KPW][EPL], xq[QPW][EPL], xk[KPW][EPL];
#pragma unroll
  for (int t = 0; t < QPW; ++t) {
    load_epl<EPL>(dq + (m * NH + warp + 8 * t) * HD + e0, gq[t]);
    if (NORM) load_epl<EPL>(q_raw + m * pq + (warp + 8 * t) * HD + e0, xq[t]);
  }
#pragma unroll
  for (int t = 0; t < KPW; ++t) {
    load_epl<EPL>(dk + (m * NKV + warp + 8 * t) * HD + e0, gk[t]);
    load_epl<EPL>(dv + (m * NKV + warp + 8 * t) * HD + e0, gv[t]);
    if (NORM) load_epl<EPL>(k_raw + m * pk + (warp + 8 * t) * HD + e0, xk[t]);
  }
  float wq[EPL], wk[EPL];
  if (NORM) {
    load_epl<EPL>(qw + e0, wq);
    load_epl<EPL>(kw + e0, wk);
  }
  const int p = pos[m];
  const float* csr = cs + (size_t)p * HALF;
  const float* snr = sn + (size_t)p * HALF;
  float c[EPL], sg[EPL];  // sin signed for the FORWARD rotation; the inverse subtracts
  if (NEOX) {
    const bool first = e0 < HALF;
    float sv_[EPL];
    load_epl<EPL>(csr + (first ? e0 : e0 - HALF), c);
    load_epl<EPL>(snr + (first ? e0 : e0 - HALF), sv_);
#pragma unroll
    for (int k = 0; k < EPL; ++k) sg[k] = first ? -sv_[k] : sv_[k];
  } else {
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      c[k] = csr[(e0 + k) >> 1];
      const float t = snr[(e0 + k) >> 1];
      sg[k] = (k & 1) ? t : -t;
    }
  }
  auto back = [&](float* g, const float* xr, const float* w) -> float {
    float o[EPL];
#pragma unroll
    for (int k = 0; k < EPL; ++k) {
      const float partner = NEOX ? __shfl_xor_sync(0xffffffffu, g[k], 16) : g[k ^ 1];
      o[k] = g[k] * c[k] + partner * (sg[k] * -1.f);
    }
    if (NORM) {
      float ss = 0.f, gx = 0.f;
#pragma unroll
      for (int k = 0; k < EPL; ++k) { ss += xr[k] * xr[k]; gx += o[k] * w[k] * xr[k]; }
      ss = warp_sum(ss);
      gx = warp_sum(gx);
      const float ir = 1.0f / sqrtf(ss / (float)HD + eps);
      const float cc = gx * ir * ir * ir / (float)HD;
#pragma unroll
      for (int k = 0; k < EPL; ++k) o[k] = o[k] * w[k] * ir - xr[k] * cc;
    }
    float mx = 0.f;
#pragma unroll
    for (int k = 0; k < EPL; ++k) { g[k] = o[k]; mx = fmaxf(mx, fabsf(o[k])); }
    return mx;
  };
  float mx[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int t = 0; t < QPW; ++t) mx[0] = fmaxf(mx[0], back(gq[t], xq[t], wq));
#pragma unroll
  for (int t = 0; t < KPW; ++t) mx[1] = fmaxf(mx[1], back(gk[t], xk[t], wk));
#pragma unroll
  for (int t = 0; t < KPW; ++t)
#pragma unroll
    for (int k = 0; k < EPL; ++k) mx[2] = fmaxf(mx[2], fabsf(gv[t][k]));
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float v = warp_max(mx[k]);
    if (lane == 0) wmax[k][warp] = v;
  }
  __syncthreads();
  float s3[3], inv[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) v = fmaxf(v, wmax[k][w]);
    s3[k] = v;
  }
  if (common) s3[0] = s3[1] = s3[2] = fmaxf(s3[0], fmaxf(s3[1], s3[2]));
  if (threadIdx.x == 0) { sq[m] = s3[0]; sk[m] = s3[1]; sv[m] = s3[2]; }  // 0 for an all-zero row
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    s3[k] = s3[k] > 0.f ? s3[k] : 1.f;
    inv[k] = 1.f / s3[k];
  }
  float o[EPL];
#pragma unroll
  for (int t = 0; t < QPW; ++t) {
#pragma unroll
    for (int k = 0; k < EPL; ++k) o[k] = gq[t][k] * inv[0];
    store_epl_h<EPL>(dq16 + m * oq + (warp + 8 * t) * HD + e0, o);
  }
#pragma unroll
  for (int t = 0; t < KPW; ++t) {
#pragma unroll
    for (int k = 0; k < EPL; ++k) o[k] = gk[t][k] * inv[1];
    store_epl_h<EPL>(dk16 + m * ok + (warp + 8 * t) * HD + e0, o);
#pragma unroll
    for (int k = 0; k < EPL; ++k) o[k] = gv[t][k] * inv[2];
    store_epl_h<EPL>(dv16 + m * ov + (warp + 8 * t) * HD + e0, o);
  }
}

// the shapes the register-resident kernels cover
static bool rope_reg_ok(int nh, int nkv, int hd, int rot, int neox, int* epl, int* hpw) {
  if (hd != 64 && hd != 128) return false;
  const int e = hd / 32, half = rot / 2;
  if (rot <= 0 || rot > hd || (rot & 1) || rot % e != 0) return false;
  if (neox && half % e != 0) return false;
  const int heads = nh + 2 * nkv;
  const int per = (heads + 7) / 8;
  if (per > 8) return false;
  *epl = e;
  *hpw = per <= 4 ? 4 : (per <= 6 ? 6 : 8);
  return true;
}
bool qk_rope_takes_pitches(int nh, int nkv, int hd, int rot, int neox) {
  int e, h;
  return rope_reg_ok(nh, nkv, hd, rot, neox, &e, &h);
}
void launch_qk_rope_fwd(const float* q_raw, const float* k_raw, const float* v_raw, size_t raw_pitch, const float* qw,
                        const float* kw, const int* pos, const float* cs, const float* sn, int M, int nh, int nkv, int hd,
                        int rot, int neox, float eps, __half* q16, __half* k16, __half* v16, cudaStream_t st) {
  if (M <= 0) return;
  int epl = 0, hpw = 0;
  // raw_pitch = 0: three separate row-major matrices; else one row pitch for all three (slices of one matrix)
  const size_t pq = raw_pitch ? raw_pitch : (size_t)nh * hd, pk = raw_pitch ? raw_pitch : (size_t)nkv * hd, pv = pk;
  if (hd == 128 && rot == hd && (qw != nullptr) == (kw != nullptr) && nh % 8 == 0 && nkv % 8 == 0) {
    const int qpw = nh / 8, kpw = nkv / 8;
#define RT_ROPE_FAST(Q, K)                                                                                                        \
  if (qpw == Q && kpw == K) {                                                                                                     \
    if (neox) {                                                                                                                   \
      if (qw) pdl(qk_rope_fwd_fast_kernel<4, Q, K, true, true>, M, 256, 0, st)(q_raw, k_raw, v_raw, pq, pk, pv, qw, kw, pos, cs, sn, eps, q16, k16, v16);   \
      else pdl(qk_rope_fwd_fast_kernel<4, Q, K, true, false>, M, 256, 0, st)(q_raw, k_raw, v_raw, pq, pk, pv, qw, kw, pos, cs, sn, eps, q16, k16, v16);     \
    } else {                                                                                                                      \
      if (qw) pdl(qk_rope_fwd_fast_kernel<4, Q, K, false, true>, M, 256, 0, st)(q_raw, k_raw, v_raw, pq, pk, pv, qw, kw, pos, cs, sn, eps, q16, k16, v16);  \
      else pdl(qk_rope_fwd_fast_kernel<4, Q, K, false, false>, M, 256, 0, st)(q_raw, k_raw, v_raw, pq, pk, pv, qw, kw, pos, cs, sn, eps, q16, k16, v16);    \
    }                                                                                                                             \
    RT_COUNT_LAUNCH(1);                                                                                                           \
    return;                                                                                                                       \
  }
    RT_ROPE_FAST(2, 1)
    RT_ROPE_FAST(3, 1)
    RT_ROPE_FAST(4, 1)
    RT_ROPE_FAST(4, 2)
    RT_ROPE_FAST(1, 1)
#undef RT_ROPE_FAST
  }
  if (rope_reg_ok(nh, nkv, hd, rot, neox, &epl, &hpw)) {
#define RT_ROPE_FWD(E, H) pdl(qk_rope_fwd_reg_kernel<E, H>, M, 256, 0, st)(q_raw, k_raw, v_raw, pq, pk, pv, qw, kw, pos, cs, sn, nh, nkv, rot, neox, eps, q16, k16, v16)
    if (epl == 4) { if (hpw == 4) RT_ROPE_FWD(4, 4); else if (hpw == 6) RT_ROPE_FWD(4, 6); else RT_ROPE_FWD(4, 8); }
    else { if (hpw == 4) RT_ROPE_FWD(2, 4); else if (hpw == 6) RT_ROPE_FWD(2, 6); else RT_ROPE_FWD(2, 8); }
#undef RT_ROPE_FWD
  } else {
    qk_rope_fwd_kernel<<<M, 256, 0, st>>>(q_raw, k_raw, v_raw, qw, kw, pos, cs, sn, nh, nkv, hd, rot, neox, eps, q16, k16, v16);
  }
  RT_COUNT_LAUNCH(1);
}

// Backward of the above (reference src/attention.rs:331-341): inverse rotation, then the
// QK-norm backward with the norm's input recomputed from q_raw/k_raw; dv passes through.
// Outputs are the three row-normalised f16 matrices (+ per-token scales) the q/k/v
// backward matmuls consume.  Dynamic shared memory: (nh + 2*nkv) * hd floats.
__global__ void qk_rope_bwd_kernel(const float* __restrict__ dq, const float* __restrict__ dk,
                                   const float* __restrict__ dv, const float* __restrict__ q_raw,
                                   const float* __restrict__ k_raw, const float* __restrict__ qw,
                                   const float* __restrict__ kw, const int* __restrict__ pos,
                                   const float* __restrict__ cs, const float* __restrict__ sn, int nh, int nkv, int hd,
                                   int rot, int neox, float eps, __half* __restrict__ dq16, __half* __restrict__ dk16,
                                   __half* __restrict__ dv16, float* __restrict__ sq, float* __restrict__ sk,
                                   float* __restrict__ sv) {
  extern __shared__ __align__(16) float buf[];  // [q heads | k heads | v heads] of this token, f32 results
  __shared__ float wmax[3][32];
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int half = rot / 2;
  const int p = pos[m];
  const float* csr = cs + (size_t)p * half;
  const float* snr = sn + (size_t)p * half;
  float mx[3] = {0.f, 0.f, 0.f};
  for (int h = warp; h < nh + 2 * nkv; h += nwarps) {
    float* out = buf + (size_t)h * hd;
    if (h >= nh + nkv) {
      const float* src = dv + (m * nkv + (h - nh - nkv)) * hd;
      for (int i = lane * 4; i < hd; i += 128) {
        const float4 v = *(const float4*)(src + i);
        *(float4*)(out + i) = v;
        mx[2] = fmaxf(mx[2], fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      }
      continue;
    }
    const bool is_q = h < nh;
    const float* g = is_q ? dq + (m * nh + h) * hd : dk + (m * nkv + (h - nh)) * hd;
    const float* xr = is_q ? q_raw + (m * nh + h) * hd : k_raw + (m * nkv + (h - nh)) * hd;
    const float* nw = is_q ? qw : kw;
    // inverse rotation (sin negated) into shared memory
    for (int i = lane * 2; i < half; i += 64) {
      const float2 c = *(const float2*)(csr + i), s = *(const float2*)(snr + i);
      if (neox) {
        const float2 x1 = *(const float2*)(g + i), x2 = *(const float2*)(g + i + half);
        *(float2*)(out + i) = make_float2(x1.x * c.x + x2.x * s.x, x1.y * c.y + x2.y * s.y);
        *(float2*)(out + i + half) = make_float2(x2.x * c.x - x1.x * s.x, x2.y * c.y - x1.y * s.y);
      } else {
        const float4 x = *(const float4*)(g + 2 * i);
        *(float4*)(out + 2 * i) = make_float4(x.x * c.x + x.y * s.x, x.y * c.x - x.x * s.x, x.z * c.y + x.w * s.y,
                                              x.w * c.y - x.z * s.y);
      }
    }
    for (int i = rot + lane; i < hd; i += 32) out[i] = g[i];
    __syncwarp();
    float mm = 0.f;
    if (nw) {
      float ss = 0.f, gx = 0.f;
      for (int i = lane * 4; i < hd; i += 128) {
        const float4 xv = *(const float4*)(xr + i), ov = *(const float4*)(out + i), wv = *(const float4*)(nw + i);
        ss += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
        gx += ov.x * wv.x * xv.x + ov.y * wv.y * xv.y + ov.z * wv.z * xv.z + ov.w * wv.w * xv.w;
      }
      ss = warp_sum(ss);
      gx = warp_sum(gx);
      const float ir = 1.0f / sqrtf(ss / (float)hd + eps);
      const float c = gx * ir * ir * ir / (float)hd;
      for (int i = lane * 4; i < hd; i += 128) {
        const float4 xv = *(const float4*)(xr + i), ov = *(const float4*)(out + i), wv = *(const float4*)(nw + i);
        const float4 v = make_float4(ov.x * wv.x * ir - xv.x * c, ov.y * wv.y * ir - xv.y * c, ov.z * wv.z * ir - xv.z * c,
                                     ov.w * wv.w * ir - xv.w * c);
        *(float4*)(out + i) = v;
        mm = fmaxf(mm, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      }
    } else {
      for (int i = lane * 4; i < hd; i += 128) {
        const float4 v = *(const float4*)(out + i);
        mm = fmaxf(mm, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      }
    }
    mx[is_q ? 0 : 1] = fmaxf(mx[is_q ? 0 : 1], mm);
  }
  for (int k = 0; k < 3; ++k) {
    float v = warp_max(mx[k]);
    if (lane == 0) wmax[k][warp] = v;
  }
  __syncthreads();
  float s3[3];
  for (int k = 0; k < 3; ++k) {
    float v = 0.f;
    for (int w = 0; w < nwarps; ++w) v = fmaxf(v, wmax[k][w]);
    s3[k] = v;
  }
  if (threadIdx.x == 0) { sq[m] = s3[0]; sk[m] = s3[1]; sv[m] = s3[2]; }  // 0 for an all-zero row
  for (int k = 0; k < 3; ++k) s3[k] = s3[k] > 0.f ? s3[k] : 1.f;
  const int nq = nh * hd, nk = nkv * hd;
  const float i0 = 1.f / s3[0], i1 = 1.f / s3[1], i2 = 1.f / s3[2];
  for (int i = threadIdx.x * 4; i < nq + 2 * nk; i += blockDim.x * 4) {  // nq, nk are multiples of 4
    const float4 v = *(const float4*)(buf + i);
    const float inv = i < nq ? i0 : (i < nq + nk ? i1 : i2);
    __half* dst = i < nq ? dq16 + m * nq + i : (i < nq + nk ? dk16 + m * nk + (i - nq) : dv16 + m * nk + (i - nq - nk));
    __half2 a = __floats2half2_rn(v.x * inv, v.y * inv), b = __floats2half2_rn(v.z * inv, v.w * inv);
    *(uint2*)dst = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
  }
}
void launch_qk_rope_bwd(const float* dq, const float* dk, const float* dv, const float* q_raw, const float* k_raw,
                        size_t raw_pitch, const float* qw, const float* kw, const int* pos, const float* cs, const float* sn,
                        int M, int nh, int nkv, int hd, int rot, int neox, float eps, __half* dq16, __half* dk16,
                        __half* dv16, size_t out_pitch, float* sq, float* sk, float* sv, cudaStream_t st) {
  if (M <= 0) return;
  int epl = 0, hpw = 0;
  // out_pitch != 0: the three outputs are slices of one matrix and share ONE scale per token
  const size_t pq = raw_pitch ? raw_pitch : (size_t)nh * hd, pk = raw_pitch ? raw_pitch : (size_t)nkv * hd;
  const size_t oq = out_pitch ? out_pitch : (size_t)nh * hd, ok = out_pitch ? out_pitch : (size_t)nkv * hd, ov = ok;
  const int common = out_pitch ? 1 : 0;
  if (hd == 128 && rot == hd && (qw != nullptr) == (kw != nullptr) && nh % 8 == 0 && nkv % 8 == 0) {
    const int qpw = nh / 8, kpw = nkv / 8;
#define RT_ROPE_BFAST_ARGS (dq, dk, dv, q_raw, k_raw, pq, pk, oq, ok, ov, common, qw, kw, pos, cs, sn, eps, dq16, dk16, dv16, sq, sk, sv)
#define RT_ROPE_BFAST(Q, K)                                                                            \
  if (qpw == Q && kpw == K) {                                                                          \
    if (neox) {                                                                                        \
      if (qw) pdl(qk_rope_bwd_fast_kernel<4, Q, K, true, true>, M, 256, 0, st) RT_ROPE_BFAST_ARGS;     \
      else pdl(qk_rope_bwd_fast_kernel<4, Q, K, true, false>, M, 256, 0, st) RT_ROPE_BFAST_ARGS;       \
    } else {                                                                                           \
      if (qw) pdl(qk_rope_bwd_fast_kernel<4, Q, K, false, true>, M, 256, 0, st) RT_ROPE_BFAST_ARGS;    \
      else pdl(qk_rope_bwd_fast_kernel<4, Q, K, false, false>, M, 256, 0, st) RT_ROPE_BFAST_ARGS;      \
    }                                                                                                  \
    RT_COUNT_LAUNCH(1);                                                                                \
    return;                                                                                            \
  }
    RT_ROPE_BFAST(2, 1)
    RT_ROPE_BFAST(3, 1)
    RT_ROPE_BFAST(4, 1)
    RT_ROPE_BFAST(4, 2)
    RT_ROPE_BFAST(1, 1)
#undef RT_ROPE_BFAST
#undef RT_ROPE_BFAST_ARGS
  }
  if (rope_reg_ok(nh, nkv, hd, rot, neox, &epl, &hpw)) {
#define RT_ROPE_BWD(E, H) pdl(qk_rope_bwd_reg_kernel<E, H>, M, 256, 0, st)(dq, dk, dv, q_raw, k_raw, pq, pk, oq, ok, ov, common, qw, kw, pos, cs, sn, nh, nkv, rot, neox, eps, dq16, dk16, dv16, sq, sk, sv)
    if (epl == 4) { if (hpw == 4) RT_ROPE_BWD(4, 4); else if (hpw == 6) RT_ROPE_BWD(4, 6); else RT_ROPE_BWD(4, 8); }
    else { if (hpw == 4) RT_ROPE_BWD(2, 4); else if (hpw == 6) RT_ROPE_BWD(2, 6); else RT_ROPE_BWD(2, 8); }
#undef RT_ROPE_BWD
  } else {
    size_t smem = (size_t)(nh + 2 * nkv) * hd * sizeof(float);
    qk_rope_bwd_kernel<<<M, 256, smem, st>>>(dq, dk, dv, q_raw, k_raw, qw, kw, pos, cs, sn, nh, nkv, hd, rot, neox, eps,
                                             dq16, dk16, dv16, sq, sk, sv);
  }
  RT_COUNT_LAUNCH(1);
}

// ------------------------------------------------------------------ SwiGLU (reference src/model.rs:113-134, src/tensor.rs:122-143)
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) {
  if (x >= 0.f) return 1.0f / (1.0f + expf(-x));
  float e = expf(x);
  return e / (1.0f + e);
}
// true when one of the eight f16 values is inf or NaN: the product left f16's range (the reference
// computes it in f32); the host gets RT_ERR_NONFINITE instead of a NaN loss
__device__ __forceinline__ bool any_nonfinite_f16x8(const uint4& o) {
  const uint32_t w[4] = {o.x, o.y, o.z, o.w};
  bool bad = false;
#pragma unroll
  for (int k = 0; k < 4; ++k) bad |= ((w[k] & 0x7C00u) == 0x7C00u) | ((w[k] & 0x7C000000u) == 0x7C000000u);
  return bad;
}
__global__ void swiglu_fwd_kernel(const __half* __restrict__ g, const __half* __restrict__ u, __half* __restrict__ h,
                                  size_t n, int* status) {
  pdl_entry();
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i + 7 < n) {
    const uint4 gv = *(const uint4*)(g + i), uv = *(const uint4*)(u + i);
    const __half2* g2 = (const __half2*)&gv;
    const __half2* u2 = (const __half2*)&uv;
    uint4 o;
    __half2* o2 = (__half2*)&o;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __half22float2(g2[k]), b = __half22float2(u2[k]);
      o2[k] = __floats2half2_rn(__fdividef(a.x, 1.0f + __expf(-a.x)) * b.x, __fdividef(a.y, 1.0f + __expf(-a.y)) * b.y);
    }
    *(uint4*)(h + i) = o;
    if (status && any_nonfinite_f16x8(o)) atomicCAS(status, 0, RT_ERR_NONFINITE);
  } else {
    for (; i < n; ++i) {
      const __half v = __float2half_rn(silu_f(__half2float(g[i])) * __half2float(u[i]));
      h[i] = v;
      if (status && (__hisinf(v) || __hisnan(v))) atomicCAS(status, 0, RT_ERR_NONFINITE);
    }
  }
}
// gate and up as column slices of one [rows x pitch] matrix (ff a multiple of 8)
__global__ void swiglu_fwd_pitched_kernel(const __half* __restrict__ g, const __half* __restrict__ u, size_t pitch, int ff,
                                          size_t n, __half* __restrict__ h, int* status) {
  pdl_entry();
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const size_t r = i / ff, c = i % ff;
  const uint4 gv = *(const uint4*)(g + r * pitch + c), uv = *(const uint4*)(u + r * pitch + c);
  const __half2* g2 = (const __half2*)&gv;
  const __half2* u2 = (const __half2*)&uv;
  uint4 o;
  __half2* o2 = (__half2*)&o;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 a = __half22float2(g2[k]), b = __half22float2(u2[k]);
    o2[k] = __floats2half2_rn(__fdividef(a.x, 1.0f + __expf(-a.x)) * b.x, __fdividef(a.y, 1.0f + __expf(-a.y)) * b.y);
  }
  *(uint4*)(h + i) = o;
  if (status && any_nonfinite_f16x8(o)) atomicCAS(status, 0, RT_ERR_NONFINITE);
}
void launch_swiglu_fwd(const __half* g, const __half* u, size_t in_pitch, int rows, int ff, __half* h, int* status,
                       cudaStream_t st) {
  const size_t n = (size_t)rows * ff;
  if (n == 0) return;
  size_t threads = (n + 7) / 8;
  if (in_pitch && in_pitch != (size_t)ff && (ff & 7) == 0)
    pdl(swiglu_fwd_pitched_kernel, (unsigned)((threads + 255) / 256), 256, 0, st)(g, u, in_pitch, ff, n, h, status);
  else
    pdl(swiglu_fwd_kernel, (unsigned)((threads + 255) / 256), 256, 0, st)(g, u, h, n, status);
  RT_COUNT_LAUNCH(1);
}
// dg = dh*u*silu'(g), du = dh*silu(g); both written row-normalised in f16 with per-row scales.
// The kernel is bound by the exp/divide per element, so sigma is computed once per element with
// the fast intrinsics (2 ulp, far inside the f16 rounding that follows) and the products are
// kept in registers between the max pass and the write pass.
__device__ __forceinline__ void load8f(const float* p, float* d) {
  const float4 d0 = *(const float4*)p, d1 = *(const float4*)(p + 4);
  d[0] = d0.x; d[1] = d0.y; d[2] = d0.z; d[3] = d0.w; d[4] = d1.x; d[5] = d1.y; d[6] = d1.z; d[7] = d1.w;
}
__device__ __forceinline__ void load8f(const __half* p, float* d) {
  const uint4 v = *(const uint4*)p;
  const __half2* h = (const __half2*)&v;
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); d[2 * k] = f.x; d[2 * k + 1] = f.y; }
}
__device__ __forceinline__ float ld1f(const float* p) { return *p; }
__device__ __forceinline__ float ld1f(const __half* p) { return __half2float(*p); }
template <typename DT>
__device__ __forceinline__ void swiglu_grad8(const DT* dh, const __half* g, const __half* u, float* dg, float* du) {
  float d[8];
  load8f(dh, d);
  const uint4 gv = *(const uint4*)g, uv = *(const uint4*)u;
  const __half2* g2 = (const __half2*)&gv;
  const __half2* u2 = (const __half2*)&uv;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 a = __half22float2(g2[k]), b = __half22float2(u2[k]);
    const float s0 = __fdividef(1.0f, 1.0f + __expf(-a.x)), s1 = __fdividef(1.0f, 1.0f + __expf(-a.y));
    dg[2 * k] = d[2 * k] * b.x * (s0 * (1.0f + a.x * (1.0f - s0)));
    dg[2 * k + 1] = d[2 * k + 1] * b.y * (s1 * (1.0f + a.y * (1.0f - s1)));
    du[2 * k] = d[2 * k] * (a.x * s0);
    du[2 * k + 1] = d[2 * k + 1] * (a.y * s1);
  }
}
// dh is f32, or f16 rows that still lack their per-row factor in_scale[r] (which then only
// multiplies the two output scales).
template <int NCH, typename DT>  // 8-element chunks cached per thread: ff <= NCH * 8 * blockDim.x, ff % 8 == 0
__global__ void swiglu_bwd_cached_kernel(const DT* __restrict__ dh, const float* __restrict__ in_scale,
                                         const __half* __restrict__ g,
                                         const __half* __restrict__ u, size_t gp, int ff, __half* __restrict__ dg16,
                                         __half* __restrict__ du16, size_t op, int common, float* __restrict__ sg,
                                         float* __restrict__ su) {
  pdl_entry();
  const size_t r = blockIdx.x;
  float a[NCH][8], b[NCH][8];
  float mg = 0.f, mu = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    if (i < ff) {
      swiglu_grad8(dh + r * ff + i, g + r * gp + i, u + r * gp + i, a[c], b[c]);
#pragma unroll
      for (int k = 0; k < 8; ++k) { mg = fmaxf(mg, fabsf(a[c][k])); mu = fmaxf(mu, fabsf(b[c][k])); }
    }
  }
  {  // both row maxima through one barrier (magnitudes: 0 is the identity)
    __shared__ float shg[32], shu[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (int)(blockDim.x >> 5);
    mg = warp_max(mg);
    mu = warp_max(mu);
    if (lane == 0) { shg[w] = mg; shu[w] = mu; }
    __syncthreads();
    mg = mu = 0.f;
    for (int k = 0; k < nw; ++k) { mg = fmaxf(mg, shg[k]); mu = fmaxf(mu, shu[k]); }
  }
  if (common) mg = mu = fmaxf(mg, mu);  // gate and up gradients form ONE matrix with one scale per row
  const float s_g = mg > 0.f ? mg : 1.f, s_u = mu > 0.f ? mu : 1.f;
  const float ig = 1.f / s_g, iu = 1.f / s_u;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 8;
    if (i < ff) {
      uint4 oa, ob;
      __half2* pa = (__half2*)&oa;
      __half2* pb = (__half2*)&ob;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        pa[k] = __floats2half2_rn(a[c][2 * k] * ig, a[c][2 * k + 1] * ig);
        pb[k] = __floats2half2_rn(b[c][2 * k] * iu, b[c][2 * k + 1] * iu);
      }
      *(uint4*)(dg16 + r * op + i) = oa;
      *(uint4*)(du16 + r * op + i) = ob;
    }
  }
  if (threadIdx.x == 0) {
    const float f = in_scale ? in_scale[r] : 1.0f;
    sg[r] = mg * f;  // 0 for an all-zero row
    su[r] = mu * f;
  }
}
// general row length: scalar, recomputed in the second pass
template <typename DT>
__global__ void swiglu_bwd_kernel(const DT* __restrict__ dh, const float* __restrict__ in_scale, const __half* __restrict__ g,
                                  const __half* __restrict__ u, size_t gp, int ff, __half* __restrict__ dg16,
                                  __half* __restrict__ du16, size_t op, int common, float* __restrict__ sg,
                                  float* __restrict__ su) {
  const size_t r = blockIdx.x;
  const DT* dhr = dh + r * ff;
  const __half* gr = g + r * gp;
  const __half* ur = u + r * gp;
  float mg = 0.f, mu = 0.f;
  for (int i = threadIdx.x; i < ff; i += blockDim.x) {
    const float gv = __half2float(gr[i]), uv = __half2float(ur[i]), d = ld1f(dhr + i);
    const float s = sigmoid_f(gv);
    mg = fmaxf(mg, fabsf(d * uv * (s * (1.0f + gv * (1.0f - s)))));
    mu = fmaxf(mu, fabsf(d * silu_f(gv)));
  }
  mg = block_max(mg);
  mu = block_max(mu);
  if (common) mg = mu = fmaxf(mg, mu);
  const float s_g = mg > 0.f ? mg : 1.f, s_u = mu > 0.f ? mu : 1.f;
  const float ig = 1.f / s_g, iu = 1.f / s_u;
  for (int i = threadIdx.x; i < ff; i += blockDim.x) {
    const float gv = __half2float(gr[i]), uv = __half2float(ur[i]), d = ld1f(dhr + i);
    const float s = sigmoid_f(gv);
    dg16[r * op + i] = __float2half_rn(d * uv * (s * (1.0f + gv * (1.0f - s))) * ig);
    du16[r * op + i] = __float2half_rn(d * silu_f(gv) * iu);
  }
  if (threadIdx.x == 0) {
    const float f = in_scale ? in_scale[r] : 1.0f;
    sg[r] = mg * f;  // 0 for an all-zero row
    su[r] = mu * f;
  }
}
template <typename DT>
static void launch_swiglu_bwd_t(const DT* dh, const float* in_scale, const __half* g, const __half* u, size_t gp, int rows,
                                int ff, __half* dg16, __half* du16, size_t op, int common, float* sg, float* su,
                                cudaStream_t st) {
  // rows that fill three chunks of 128 threads exactly (3072) leave no thread idle that way
  if ((ff & 7) == 0 && ff > 2 * 8 * 128 && ff <= 3 * 8 * 128) pdl(swiglu_bwd_cached_kernel<3, DT>, rows, 128, 0, st)(dh, in_scale, g, u, gp, ff, dg16, du16, op, common, sg, su);
  else if ((ff & 7) == 0 && ff <= 2 * 8 * 256) pdl(swiglu_bwd_cached_kernel<2, DT>, rows, 256, 0, st)(dh, in_scale, g, u, gp, ff, dg16, du16, op, common, sg, su);
  else if ((ff & 7) == 0 && ff <= 3 * 8 * 512) pdl(swiglu_bwd_cached_kernel<3, DT>, rows, 512, 0, st)(dh, in_scale, g, u, gp, ff, dg16, du16, op, common, sg, su);
  else swiglu_bwd_kernel<DT><<<rows, 256, 0, st>>>(dh, in_scale, g, u, gp, ff, dg16, du16, op, common, sg, su);
  RT_COUNT_LAUNCH(1);
}
void launch_swiglu_bwd(const void* dh, int dh_f16, const float* in_scale, const __half* g, const __half* u, size_t in_pitch,
                       int rows, int ff, __half* dg16, __half* du16, size_t out_pitch, float* sg, float* su, cudaStream_t st) {
  if (rows <= 0) return;
  // in_pitch / out_pitch = 0: separate row-major matrices; else gate|up (dg|du) are slices of one
  // matrix with that row pitch, and with out_pitch the two outputs share one scale per row
  const size_t gp = in_pitch ? in_pitch : (size_t)ff, op = out_pitch ? out_pitch : (size_t)ff;
  const int common = out_pitch ? 1 : 0;
  if (dh_f16) launch_swiglu_bwd_t((const __half*)dh, in_scale, g, u, gp, rows, ff, dg16, du16, op, common, sg, su, st);
  else launch_swiglu_bwd_t((const float*)dh, in_scale, g, u, gp, rows, ff, dg16, du16, op, common, sg, su, st);
}

// ------------------------------------------------------------------ row gather / scatter
__global__ void gather_f32_rows_kernel(const float* __restrict__ x, const int* __restrict__ idx, int d,
                                       float* __restrict__ out) {
  pdl_entry();
  const size_t r = blockIdx.x;
  const float* src = x + (size_t)idx[r] * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) out[r * d + i] = src[i];
}
void launch_gather_f32_rows(const float* x, const int* idx, int rows, int d, float* out, cudaStream_t st) {
  if (rows > 0) { pdl(gather_f32_rows_kernel, rows, 256, 0, st)(x, idx, d, out); RT_COUNT_LAUNCH(1); }
}
// dx[idx[r], :] += src[r, :]   (atomic: two targets may name the same position)
__global__ void scatter_add_rows_kernel(const float* __restrict__ src, const int* __restrict__ idx, int d,
                                        float* __restrict__ dx) {
  pdl_entry();
  const size_t r = blockIdx.x;
  float* dst = dx + (size_t)idx[r] * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(dst + i, src[r * d + i]);
}
void launch_scatter_add_rows(const float* src, const int* idx, int rows, int d, float* dx, cudaStream_t st) {
  if (rows > 0) { pdl(scatter_add_rows_kernel, rows, 256, 0, st)(src, idx, d, dx); RT_COUNT_LAUNCH(1); }
}

// ------------------------------------------------------------------ cross-entropy over one row of logits
// (reference src/model.rs:579-596, src/ops.rs:238-247): lse with an f64 normaliser, logp of
// the target, hit = no logit above the target's, and d16 = p - onehot in f16 with the row scale
// w (so dlogits = w*(p - onehot) exactly as the reference forms it).
// The greedy token of a row: the LAST index holding the maximum, which is what the reference's
// Iterator::max_by(total_cmp) returns on ties (src/eval.rs:167).  One more read of the row.
__device__ void ce_row_argmax(const float* __restrict__ row, int v, float m, int* __restrict__ out) {
  __shared__ int s_arg[32];
  int best = -1;
  for (int i = threadIdx.x; i < v; i += blockDim.x)
    if (row[i] == m) best = i;  // i grows: the thread keeps its last
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, off));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_arg[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x + 31) / 32 ? s_arg[threadIdx.x] : -1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, off));
    if (threadIdx.x == 0) *out = best;
  }
}

__global__ void ce_row_kernel(const float* __restrict__ logits, int v, const int* __restrict__ target,
                              const float* __restrict__ weight, float* __restrict__ logp, int* __restrict__ hits,
                              __half* __restrict__ d16, float* __restrict__ scale, int* __restrict__ argmax, int* status) {
  pdl_entry();
  const size_t r = blockIdx.x;
  const float* row = logits + r * v;
  const int tgt = target[r];
  if (tgt < 0 || tgt >= v) {
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_BAD_INDEX);
    return;
  }
  float m = -INFINITY;
  for (int i = threadIdx.x; i < v; i += blockDim.x) m = fmaxf(m, row[i]);
  m = block_max(m);
  double s = 0.0;
  for (int i = threadIdx.x; i < v; i += blockDim.x) s += (double)expf(row[i] - m);
  s = block_sum_d(s);
  const float tl = row[tgt];
  if (threadIdx.x == 0) {
    logp[r] = tl - (m + (float)log(s));
    if (tl >= m) atomicAdd(hits, 1);
    if (scale) scale[r] = weight[r];
  }
  if (argmax) ce_row_argmax(row, v, m, argmax + r);
  if (d16) {
    const float inv = (float)(1.0 / s);
    for (int i = threadIdx.x; i < v; i += blockDim.x) {
      float p = expf(row[i] - m) * inv;
      if (i == tgt) p -= 1.0f;
      d16[r * v + i] = __float2half_rn(p);
    }
  }
}
// The same for rows whose length is a multiple of 4: 128-bit loads, and the maximum and the sum
// found in ONE pass (each thread keeps a running maximum and rescales its partial sum when the
// maximum moves; the partial sums meet in f64), so the logits are read twice instead of three
// times.
__global__ void __launch_bounds__(1024)
ce_row_vec_kernel(const float* __restrict__ logits, int v, const int* __restrict__ target,
                  const float* __restrict__ weight, float* __restrict__ logp, int* __restrict__ hits,
                  __half* __restrict__ d16, float* __restrict__ scale, int* __restrict__ argmax, int* status) {
  pdl_entry();
  const size_t r = blockIdx.x;
  const float4* row4 = (const float4*)(logits + r * v);
  const int n4 = v >> 2;
  const int tgt = target[r];
  if (tgt < 0 || tgt >= v) {
    if (threadIdx.x == 0) atomicCAS(status, 0, RT_ERR_BAD_INDEX);
    return;
  }
  float mt = -INFINITY, st = 0.f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 x = row4[i];
    const float cm = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
    if (cm > mt) { st *= expf(mt - cm); mt = cm; }  // expf(-inf) = 0 on the first chunk
    st += expf(x.x - mt) + expf(x.y - mt) + expf(x.z - mt) + expf(x.w - mt);
  }
  const float m = block_max(mt);
  const double s = block_sum_d(mt > -INFINITY ? (double)st * (double)expf(mt - m) : 0.0);
  const float tl = logits[r * v + tgt];
  if (threadIdx.x == 0) {
    logp[r] = tl - (m + (float)log(s));
    if (tl >= m) atomicAdd(hits, 1);
    if (scale) scale[r] = weight[r];
  }
  if (argmax) ce_row_argmax(logits + r * v, v, m, argmax + r);
  if (d16) {
    const float inv = (float)(1.0 / s);
    uint2* out = (uint2*)(d16 + r * v);
    const int t4 = tgt >> 2, tk = tgt & 3;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 x = row4[i];
      float p0 = expf(x.x - m) * inv, p1 = expf(x.y - m) * inv, p2 = expf(x.z - m) * inv, p3 = expf(x.w - m) * inv;
      if (i == t4) {
        if (tk == 0) p0 -= 1.0f; else if (tk == 1) p1 -= 1.0f; else if (tk == 2) p2 -= 1.0f; else p3 -= 1.0f;
      }
      const __half2 a = __floats2half2_rn(p0, p1), b = __floats2half2_rn(p2, p3);
      out[i] = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
    }
  }
}
void launch_ce_rows(const float* logits, int rows, int v, const int* target, const float* weight, float* logp, int* hits,
                    __half* d16, float* scale, int* argmax, int* status, cudaStream_t st) {
  if (rows <= 0) return;
  if ((v & 3) == 0 && ((uintptr_t)logits & 15) == 0 && (d16 == nullptr || ((uintptr_t)d16 & 7) == 0))
    pdl(ce_row_vec_kernel, rows, 1024, 0, st)(logits, v, target, weight, logp, hits, d16, scale, argmax, status);
  else
    pdl(ce_row_kernel, rows, 1024, 0, st)(logits, v, target, weight, logp, hits, d16, scale, argmax, status);
  RT_COUNT_LAUNCH(1);
}

// ------------------------------------------------------------------ LoRA shadows and gradients
// 16-bit operand copies of one adapter, rebuilt after every parameter update:
//   a_s  [r x K]  f16 = s*A      (weight of Hs = X.(sA)^T)
//   a_h  [r x K]  f16 = A        (extra rows of the backward matmul: dX += Gs.A)
//   bp   [N x 64] f16 = B, zero padded (extra columns of the forward matmul: Y += Hs.B^T)
//   bt_s [r x N]  f16 = s*B^T    (weight of Gs = dY.(sB))
__global__ void lora_refresh_kernel(const float* __restrict__ a, const float* __restrict__ b, int r, int K, int N,
                                    float s, __half* a_s, __half* a_h, __half* bp, __half* bt_s) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t na = (size_t)r * K, nb = (size_t)N * 64;
  if (i < na) {
    a_s[i] = __float2half_rn(a[i] * s);
    a_h[i] = __float2half_rn(a[i]);
  }
  if (i < nb) {
    const int n = (int)(i / 64), j = (int)(i % 64);
    const float v = j < r ? b[(size_t)n * r + j] : 0.f;
    bp[i] = __float2half_rn(v);
    if (j < r) bt_s[(size_t)j * N + n] = __float2half_rn(v * s);
  }
}
// The same copies of one adapter written into the stacked operands of a group of linears that
// share their input (q|k|v, gate|up): a_s / a_h are this adapter's rows of [R x K]; bp points at
// (this linear's first row, this adapter's first column) of [N_total x 64]; bt_s at (this
// adapter's first row, this linear's first column) of [R x N_total], row pitch ldb.
__global__ void lora_refresh_group_kernel(const float* __restrict__ a, const float* __restrict__ b, int r, int K, int N,
                                          float s, __half* a_s, __half* a_h, __half* bp, __half* bt_s, size_t ldb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t na = (size_t)r * K, nb = (size_t)N * r;
  if (i < na) {
    a_s[i] = __float2half_rn(a[i] * s);
    a_h[i] = __float2half_rn(a[i]);
  }
  if (i < nb) {
    const int n = (int)(i / r), j = (int)(i % r);
    const float v = b[i];
    bp[(size_t)n * 64 + j] = __float2half_rn(v);
    bt_s[(size_t)j * ldb + n] = __float2half_rn(v * s);
  }
}
// Every stale adapter of a model in one launch: a block finds its row of the table by bisection
// on first_block, then does what the two kernels above do for one adapter.
__global__ void lora_refresh_table_kernel(const LoraRefreshJob* __restrict__ jobs, int n_jobs) {
  __shared__ int s_job;
  if (threadIdx.x == 0) {
    int lo = 0, hi = n_jobs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (jobs[mid].first_block <= blockIdx.x) lo = mid;
      else hi = mid - 1;
    }
    s_job = lo;
  }
  __syncthreads();
  const LoraRefreshJob j = jobs[s_job];
  const size_t i = (size_t)(blockIdx.x - j.first_block) * blockDim.x + threadIdx.x;
  const size_t na = (size_t)j.r * j.K;
  if (i < na) {
    const float v = j.a[i];
    j.a_s[i] = __float2half_rn(v * j.s);
    j.a_h[i] = __float2half_rn(v);
  }
  if (j.pad64) {
    if (i < (size_t)j.N * 64) {
      const int n = (int)(i / 64), c = (int)(i % 64);
      const float v = c < j.r ? j.b[(size_t)n * j.r + c] : 0.f;
      j.bp[i] = __float2half_rn(v);
      if (c < j.r) j.bt_s[(size_t)c * j.ldb + n] = __float2half_rn(v * j.s);
    }
  } else if (i < (size_t)j.N * j.r) {
    const int n = (int)(i / j.r), c = (int)(i % j.r);
    const float v = j.b[i];
    j.bp[(size_t)n * 64 + c] = __float2half_rn(v);
    j.bt_s[(size_t)c * j.ldb + n] = __float2half_rn(v * j.s);
  }
}
void launch_lora_refresh_table(const LoraRefreshJob* jobs_dev, int n_jobs, unsigned total_blocks, cudaStream_t st) {
  if (n_jobs <= 0 || total_blocks == 0) return;
  { lora_refresh_table_kernel<<<total_blocks, 256, 0, st>>>(jobs_dev, n_jobs); RT_COUNT_LAUNCH(1); }
}
void launch_lora_refresh_group(const float* a, const float* b, int r, int K, int N, float s, __half* a_s, __half* a_h,
                               __half* bp, __half* bt_s, size_t ldb, cudaStream_t st) {
  size_t n = (size_t)r * K > (size_t)N * r ? (size_t)r * K : (size_t)N * r;
  { lora_refresh_group_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a, b, r, K, N, s, a_s, a_h, bp, bt_s, ldb); RT_COUNT_LAUNCH(1); }
}
void launch_lora_refresh(const float* a, const float* b, int r, int K, int N, float s, __half* a_s, __half* a_h,
                         __half* bp, __half* bt_s, cudaStream_t st) {
  size_t n = (size_t)r * K > (size_t)N * 64 ? (size_t)r * K : (size_t)N * 64;
  { lora_refresh_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a, b, r, K, N, s, a_s, a_h, bp, bt_s); RT_COUNT_LAUNCH(1); }
}

// Token-contraction for the LoRA gradients (reference src/linear.rs:108-116):
//   part[split][i, j] = sum_{m in split} pscale[m] * P[m, i] * qscale[m] * Q[m, j],  i < r, j < C
// P is [M x 64] f16, Q is [M x C] f16.  A second kernel adds the splits, in order, into
// out[i*so_i + j*so_j] (deterministic: no float atomics).
//   dA: P = Gs (unit rows, pscale = row scale of dY), Q = X        -> ga[r x K]: so_i = K, so_j = 1
//   dB: P = Hs,                       Q = dY (qscale = its scale)  -> gb[N x r]: so_i = 1, so_j = r
constexpr int LG_TOK = 32;
__global__ void __launch_bounds__(256)
lora_grad_partial_kernel(const __half* __restrict__ P, const __half* __restrict__ Q, const float* __restrict__ pscale,
                         const float* __restrict__ qscale, int M, int C, int r, int tokens_per_split,
                         float* __restrict__ part) {
  __shared__ float sP[LG_TOK][65];
  __shared__ float sQ[LG_TOK][64];
  const int j0 = blockIdx.x * 64;
  const int m_begin = blockIdx.y * tokens_per_split;
  const int m_end = min(M, m_begin + tokens_per_split);
  const int tj = threadIdx.x & 63, ti = threadIdx.x >> 6;  // column, row group (4 groups)
  float acc[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) acc[k] = 0.f;
  const int rows_per = (r + 3) / 4;  // <= 16
  for (int m0 = m_begin; m0 < m_end; m0 += LG_TOK) {
    __syncthreads();
    for (int e = threadIdx.x; e < LG_TOK * 64; e += 256) {
      const int mm = e >> 6, c = e & 63, m = m0 + mm;
      float pv = 0.f, qv = 0.f;
      if (m < m_end) {
        const float sc = (pscale ? pscale[m] : 1.f) * (qscale ? qscale[m] : 1.f);
        if (c < r) pv = __half2float(P[(size_t)m * 64 + c]) * sc;
        if (j0 + c < C) qv = __half2float(Q[(size_t)m * C + j0 + c]);
      }
      sP[mm][c] = pv;
      sQ[mm][c] = qv;
    }
    __syncthreads();
#pragma unroll 4
    for (int mm = 0; mm < LG_TOK; ++mm) {
      const float q = sQ[mm][tj];
#pragma unroll
      for (int k = 0; k < 16; ++k)
        if (k < rows_per) acc[k] += sP[mm][ti + 4 * k] * q;
    }
  }
  float* dst = part + (size_t)blockIdx.y * r * C;
  for (int k = 0; k < rows_per; ++k) {
    const int i = ti + 4 * k;
    if (i < r && j0 + tj < C) dst[(size_t)i * C + j0 + tj] = acc[k];
  }
}
__global__ void lora_grad_reduce_kernel(const float* __restrict__ part, int splits, int C, int r, size_t so_i,
                                        size_t so_j, float* __restrict__ out) {
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (size_t)r * C) return;
  const int i = (int)(e / C), j = (int)(e % C);
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(size_t)k * r * C + e];
  out[i * so_i + j * so_j] += s;
}
size_t lora_grad_workspace_floats(int M, int C, int r) {
  int splits = (M + 511) / 512;
  if (splits < 1) splits = 1;
  return (size_t)splits * r * C;
}
void launch_lora_grad(const __half* P, const __half* Q, const float* pscale, const float* qscale, int M, int C, int r,
                      size_t so_i, size_t so_j, float* out, float* workspace, cudaStream_t st) {
  if (M <= 0 || r <= 0) return;
  int splits = (M + 511) / 512;
  if (splits < 1) splits = 1;
  const int tps = ((M + splits - 1) / splits + LG_TOK - 1) / LG_TOK * LG_TOK;
  splits = (M + tps - 1) / tps;
  dim3 grid((C + 63) / 64, splits);
  { lora_grad_partial_kernel<<<grid, 256, 0, st>>>(P, Q, pscale, qscale, M, C, r, tps, workspace); RT_COUNT_LAUNCH(1); }
  const size_t n = (size_t)r * C;
  { lora_grad_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(workspace, splits, C, r, so_i, so_j, out); RT_COUNT_LAUNCH(1); }
}

// Largest per-token scale of a backward input, and a [M x 64] low-rank operand with each row
// multiplied by scale[m] / max: the token contractions dA, dB need ONE common scale, so the
// per-row factors move onto the skinny operand and the common factor onto the result.
__global__ void rowscale_max_kernel(const float* __restrict__ sc, int M, float* __restrict__ out) {
  pdl_entry();
  float m = 0.f;
  for (int i = threadIdx.x; i < M; i += blockDim.x) m = fmaxf(m, sc[i]);
  m = block_max(m);
  // rounded up to a power of two: dividing by it changes no mantissa, so what a row rounds to in
  // f16 does not depend on which other rows share the batch (N ranks on shards of a batch then
  // reproduce one rank on the whole of it up to the order of f32 sums)
  if (threadIdx.x == 0) out[0] = m > 0.f ? __int_as_float((__float_as_int(m) + 0x007FFFFF) & 0x7F800000) : 1.f;
}
__global__ void scale_lowrank_rows_kernel(const __half* __restrict__ in, const float* __restrict__ sc,
                                          const float* __restrict__ smax, int M, __half* __restrict__ out) {
  const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (e >= (size_t)M * 64) return;
  const float f = sc[e >> 6] / smax[0];
  float2 v = __half22float2(*(const __half2*)(in + e));
  *(__half2*)(out + e) = __floats2half2_rn(v.x * f, v.y * f);
}
// The same per SEQUENCE: out[m] = largest scale among the tokens of m's sequence (seq_start[m] =
// first token of it), rounded up to a power of two; 1 where the whole sequence is zero; and
// out[M + m] = sc[m] / out[m], the weight of row m among its sequence's rows.  A sequence's
// backward then never sees a number that depends on its batch mates.  One block:
// the slot of a sequence is out[first token]; converting a slot is idempotent, so a reader may
// meet it before or after its own token converted it.
__global__ void rowscale_seqmax_kernel(const float* __restrict__ sc, const int* __restrict__ seq_start, int M,
                                       float* __restrict__ out) {
  pdl_entry();
  for (int i = threadIdx.x; i < M; i += blockDim.x) out[i] = 0.f;
  __syncthreads();
  for (int i = threadIdx.x; i < M; i += blockDim.x) atomicMax((int*)out + seq_start[i], __float_as_int(fmaxf(sc[i], 0.f)));
  __syncthreads();
  for (int i = threadIdx.x; i < M; i += blockDim.x) {
    const float m = out[seq_start[i]];
    const float top = m > 0.f ? __int_as_float((__float_as_int(m) + 0x007FFFFF) & 0x7F800000) : 1.f;
    out[i] = top;
    out[M + i] = fmaxf(sc[i], 0.f) / top;
  }
}
void launch_rowscale_seqmax(const float* sc, const int* seq_start, int M, float* out, cudaStream_t st) {
  if (M > 0) { pdl(rowscale_seqmax_kernel, 1, 1024, 0, st)(sc, seq_start, M, out); RT_COUNT_LAUNCH(1); }
}
void launch_rowscale_max(const float* sc, int M, float* out, cudaStream_t st) {
  if (M > 0) { pdl(rowscale_max_kernel, 1, 1024, 0, st)(sc, M, out); RT_COUNT_LAUNCH(1); }
}
void launch_scale_lowrank_rows(const __half* in, const float* sc, const float* smax, int M, __half* out, cudaStream_t st) {
  if (M <= 0) return;
  const size_t threads = (size_t)M * 32;
  { scale_lowrank_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(in, sc, smax, M, out); RT_COUNT_LAUNCH(1); }
}

// ------------------------------------------------------------------ optimiser (reference src/optim.rs:48-90)
// Sum of squares in f64: fixed-size blocks write partials, one block adds them in order.
__global__ void sumsq_partial_kernel(const float* __restrict__ g, size_t n, double* __restrict__ part) {
  double s = 0.0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    double v = (double)g[i];
    s += v * v;
  }
  s = block_sum_d(s);
  if (threadIdx.x == 0) part[blockIdx.x] = s;
}
__global__ void sumsq_final_kernel(const double* __restrict__ part, int n, double* __restrict__ out) {
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += part[i];
  s = block_sum_d(s);
  if (threadIdx.x == 0) out[0] = s;
}
void launch_sumsq(const float* g, size_t n, double* part /* >= 1024 */, double* out, cudaStream_t st) {
  int blocks = (int)((n + 255) / 256);
  if (blocks > 1024) blocks = 1024;
  if (blocks < 1) blocks = 1;
  { sumsq_partial_kernel<<<blocks, 256, 0, st>>>(g, n, part); RT_COUNT_LAUNCH(1); }
  { sumsq_final_kernel<<<1, 256, 0, st>>>(part, blocks, out); RT_COUNT_LAUNCH(1); }
}
// clip (scale read from the device-side norm) fused with the AdamW update.
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                             size_t n, const double* __restrict__ sumsq, float max_norm, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2, float* __restrict__ norm_out) {
  const float norm = (float)sqrt(sumsq[0]);
  float clip = 1.0f;
  if (max_norm > 0.f && norm > max_norm) clip = max_norm / (norm + 1e-6f);
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0 && norm_out) norm_out[0] = norm;
  if (i >= n) return;
  const float gi = clip != 1.0f ? g[i] * clip : g[i];
  g[i] = gi;
  const float mi = beta1 * m[i] + (1.0f - beta1) * gi;
  const float vi = beta2 * v[i] + (1.0f - beta2) * gi * gi;
  m[i] = mi;
  v[i] = vi;
  const float mh = mi / bc1, vh = vi / bc2;
  p[i] -= lr * (mh / (sqrtf(vh) + eps) + wd * p[i]);
}
void launch_adamw(float* p, float* g, float* m, float* v, size_t n, const double* sumsq, float max_norm, float lr,
                  float beta1, float beta2, float eps, float wd, float bc1, float bc2, float* norm_out,
                  cudaStream_t st) {
  if (n == 0) return;
  { adamw_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p, g, m, v, n, sumsq, max_norm, lr, beta1, beta2, eps, wd,
                                                             bc1, bc2, norm_out); RT_COUNT_LAUNCH(1); }
}

// ------------------------------------------------------------------ misc
__global__ void absmax_kernel(const float* __restrict__ x, size_t n, float* __restrict__ out) {
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(x[i]));
  m = block_max(m);
  if (threadIdx.x == 0) atomicMax((int*)out, __float_as_int(m));  // non-negative floats order like ints
}
// y16 = x / max(amax, tiny); inv/scale read on device
__global__ void scale_to_f16_kernel(const float* __restrict__ x, size_t n, const float* __restrict__ amax,
                                    __half* __restrict__ y) {
  const float a = amax[0];
  const float inv = a > 0.f ? 1.f / a : 1.f;
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i + 1 < n) {
    float2 v = *(const float2*)(x + i);
    *(__half2*)(y + i) = __floats2half2_rn(v.x * inv, v.y * inv);
  } else if (i < n) y[i] = __float2half_rn(x[i] * inv);
}
void launch_global_normalize(const float* x, size_t n, float* amax_dev, __half* y16, cudaStream_t st) {
  if (n == 0) return;
  cudaMemsetAsync(amax_dev, 0, sizeof(float), st);
  int blocks = (int)((n + 255) / 256);
  if (blocks > 1184) blocks = 1184;
  { absmax_kernel<<<blocks, 256, 0, st>>>(x, n, amax_dev); RT_COUNT_LAUNCH(1); }
  size_t threads = (n + 1) / 2;
  { scale_to_f16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(x, n, amax_dev, y16); RT_COUNT_LAUNCH(1); }
}

}  // namespace rt
