// Small memory-bound device ops around the frozen matmuls.
#include "ctx.h"

namespace rt {

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 v = *(const float4*)(in + i);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *(uint2*)(out + i) = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
  } else {
    for (; i < n; ++i) out[i] = __float2bfloat16_rn(in[i]);
  }
}

void launch_f32_to_bf16(const float* in, __nv_bfloat16* out, size_t n, cudaStream_t st) {
  if (n == 0) return;
  size_t threads = (n + 3) / 4;
  f32_to_bf16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(in, out, n);
}

}  // namespace rt
