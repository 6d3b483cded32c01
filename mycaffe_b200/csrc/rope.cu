// Rotary positional embedding on a (B,T,H,D) tensor, forward and backward, one launch each.
// Same arithmetic as the reference's RopeDataGpu<T>::Forward/Backward
// (CudaDnnDLL/Cuda Files/rope.cu:724-864), which runs it as three launches (split into
// real/imaginary scratch buffers, rotate, interleave back) with a device synchronise after
// each: pair p = (x[2p], x[2p+1]), position = (p % (T*H*D/2)) / (H*D/2), frequency = p % (D/2).
// Also the small dtype conversion kernels used at the handle boundary.
#include "common.cuh"
#include "kernels.h"

namespace {

__global__ void rope_kernel(const float2* __restrict__ x, float2* __restrict__ y, int64_t npairs, int64_t tfull,
                            int full, int half, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            int backward) {
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < npairs; p += (int64_t)gridDim.x * blockDim.x) {
    const int64_t base = p % tfull;
    const int64_t idx = (base / full) * half + base % half;
    const float c = __ldg(cos_t + idx), s = __ldg(sin_t + idx);
    const float2 v = x[p];
    float2 o;
    if (!backward) { o.x = v.x * c - v.y * s; o.y = v.x * s + v.y * c; }
    else           { o.x = v.x * c + v.y * s; o.y = -v.x * s + v.y * c; }
    y[p] = o;
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16_rn(x[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = __bfloat162float(x[i]);
}

int grid_for(int64_t n) {
  int64_t b = (n + 255) / 256;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

int mca_rope_f32(const float* x, float* y, int64_t n, int T, int H, int D, const float* cos_table,
                 const float* sin_table, int freq_offset, int backward, void* stream) {
  if (!x || !y || !cos_table || !sin_table) return ERROR_PARAM_NULL;
  if (n <= 0 || (n & 1) || T <= 0 || H <= 0 || D <= 0 || (D & 1)) return ERROR_PARAM_OUT_OF_RANGE;
  const int half = D / 2;
  const int off = freq_offset > 0 ? freq_offset : 0;  // rope.cu:812-818
  rope_kernel<<<grid_for(n / 2), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const float2*>(x), reinterpret_cast<float2*>(y), n / 2, (int64_t)T * half * H, half * H, half,
      cos_table + off, sin_table + off, backward);
  return mca_launch_status();
}

int mca_convert_f32_to_bf16(const float* x, void* y, int64_t n, void* stream) {
  if (!x || !y) return ERROR_PARAM_NULL;
  if (n <= 0) return 0;
  f32_to_bf16_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(x, (__nv_bfloat16*)y, n);
  return mca_launch_status();
}

int mca_convert_bf16_to_f32(const void* x, float* y, int64_t n, void* stream) {
  if (!x || !y) return ERROR_PARAM_NULL;
  if (n <= 0) return 0;
  bf16_to_f32_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, y, n);
  return mca_launch_status();
}
