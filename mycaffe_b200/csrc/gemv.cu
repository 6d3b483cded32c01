// Weight-streaming projections of the llama2 decode attention block, fused with what surrounds them:
//   * RMSNorm + Wq/Wk/Wv:  q,k,v = W · (w_rms ∘ x / sqrt(mean(x²) + eps))
//   * Wo + residual:       x += Wo · attn
// Replaces, for one new token, Primitives::rmsnorm (a square kernel, a thrust::reduce with a
// device-to-host round trip and a scale kernel; CudaExtension.llm32.llama2/Files/
// primitives.cu:281-303) followed by three cublasSgemv calls (primitives.cu:322-340;
// llama2_gpu.cpp:56-61), and the Wo cublasSgemv plus the residual add kernel
// (llama2_gpu.cpp:78-81).  The arithmetic follows the CPU twin (rmsnorm llama2_cpu.cpp:189-202,
// matmul :224-237): o[j] = w[j] * (s * x[j]) with s = 1/sqrt(sum(x²)/n + eps).
//
// These are GEMVs: the weights (dim x dim floats, 67 MB at dim 4096) are read exactly once and
// nothing else matters, so the kernel is bound by HBM bandwidth.  Every CTA first builds the
// normalised activation in shared memory (it is 16 KB per sequence and comes from L2), then
// its warps walk their rows of the stacked [Wq; Wk; Wv] matrix with 128-bit loads, 512
// contiguous bytes per warp instruction, and reduce with shuffles.  Up to 8 sequences share one
// pass over the weights; larger batches take several passes.
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;
constexpr int GV_BMAX = 8;   // sequences per pass over the weights

template <typename WT> struct WLoad;
template <> struct WLoad<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void load(const float* p, float (&w)[4]) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
  }
};
template <> struct WLoad<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&w)[8]) {
    const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p));
    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { w[2 * i] = __uint_as_float(u[i] << 16); w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
};

struct GemvParams {
  const float* x;        // (B, n) input activations
  const float* norm_w;   // (n) RMSNorm weights or null (no normalisation)
  const void* w[3];      // up to three stacked matrices, each (rows[i], n) row-major
  float* out[3];         // (B, rows[i]) each
  int rows[3];
  int n_mats, B, n, accumulate;  // accumulate: out += result (residual connection)
  float eps;
};

template <typename WT, int NB>
__global__ void __launch_bounds__(GV_THREADS) gemv_fused_kernel(const GemvParams p, int b0) {
  extern __shared__ __align__(16) float xs[];  // [NB][n] normalised activations
  __shared__ float red[GV_WARPS][NB];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = p.n;
  // ---- phase 1: activations of this pass's sequences -> shared memory, RMS-normalised
  float ss[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) ss[b] = 0.f;
  for (int k = tid * 4; k < n; k += GV_THREADS * 4) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const float4 v = *reinterpret_cast<const float4*>(p.x + (int64_t)(b0 + b) * n + k);
      *reinterpret_cast<float4*>(xs + b * n + k) = v;
      ss[b] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  if (p.norm_w != nullptr) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[b] += __shfl_xor_sync(0xffffffffu, ss[b], o);
      if (lane == 0) red[warp][b] = ss[b];
    }
    __syncthreads();
    float scale[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < GV_WARPS; ++w) t += red[w][b];
      t = t / (float)n + p.eps;
      scale[b] = 1.0f / sqrtf(t);
    }
    for (int k = tid * 4; k < n; k += GV_THREADS * 4) {
      const float4 g = *reinterpret_cast<const float4*>(p.norm_w + k);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float4 v = *reinterpret_cast<float4*>(xs + b * n + k);
        v.x = g.x * (scale[b] * v.x); v.y = g.y * (scale[b] * v.y); v.z = g.z * (scale[b] * v.z); v.w = g.w * (scale[b] * v.w);
        *reinterpret_cast<float4*>(xs + b * n + k) = v;
      }
    }
  }
  __syncthreads();
  // ---- phase 2: rows of the stacked matrices, one row per warp at a time
  const int total_rows = p.rows[0] + (p.n_mats > 1 ? p.rows[1] : 0) + (p.n_mats > 2 ? p.rows[2] : 0);
  constexpr int VEC = WLoad<WT>::VEC;
  for (int r = blockIdx.x * GV_WARPS + warp; r < total_rows; r += gridDim.x * GV_WARPS) {
    int m = 0, rr = r;
    if (rr >= p.rows[0]) { rr -= p.rows[0]; m = 1; if (rr >= p.rows[1]) { rr -= p.rows[1]; m = 2; } }
    const WT* wrow = reinterpret_cast<const WT*>(p.w[m]) + (int64_t)rr * n;
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[b] = 0.f;
#pragma unroll(NB <= 2 ? 8 : 4)
    for (int k = lane * VEC; k < n; k += 32 * VEC) {
      float w[VEC];
      WLoad<WT>::load(wrow + k, w);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float* xv = xs + b * n + k;
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
          const float4 t = *reinterpret_cast<const float4*>(xv + i);
          acc[b] = fmaf(w[i], t.x, acc[b]); acc[b] = fmaf(w[i + 1], t.y, acc[b]);
          acc[b] = fmaf(w[i + 2], t.z, acc[b]); acc[b] = fmaf(w[i + 3], t.w, acc[b]);
        }
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[b] += __shfl_xor_sync(0xffffffffu, acc[b], o);
    }
    if (lane == 0) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float* dst = p.out[m] + (int64_t)(b0 + b) * p.rows[m] + rr;
        *dst = p.accumulate ? (*dst + acc[b]) : acc[b];
      }
    }
  }
}

template <typename WT, int NB>
int launch_pass(const GemvParams& p, int b0, cudaStream_t st) {
  const size_t smem = sizeof(float) * (size_t)NB * p.n;
  if (smem > 200 * 1024) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  MCA_CUDA_TRY(cudaFuncSetAttribute(gemv_fused_kernel<WT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int total_rows = p.rows[0] + (p.n_mats > 1 ? p.rows[1] : 0) + (p.n_mats > 2 ? p.rows[2] : 0);
  int grid = 148 * (smem > 100 * 1024 ? 1 : smem > 40 * 1024 ? 2 : 4);
  if (grid * GV_WARPS > total_rows) grid = mca_ceil_div(total_rows, GV_WARPS);
  gemv_fused_kernel<WT, NB><<<grid, GV_THREADS, smem, st>>>(p, b0);
  return mca_launch_status();
}

template <typename WT>
int run_gemv(const GemvParams& p, cudaStream_t st) {
  int e = 0;
  for (int b0 = 0; b0 < p.B && !e;) {
    const int left = p.B - b0;
    if (left >= 8 && (size_t)8 * p.n * 4 <= 200 * 1024) { e = launch_pass<WT, 8>(p, b0, st); b0 += 8; }
    else if (left >= 4) { e = launch_pass<WT, 4>(p, b0, st); b0 += 4; }
    else if (left >= 2) { e = launch_pass<WT, 2>(p, b0, st); b0 += 2; }
    else { e = launch_pass<WT, 1>(p, b0, st); b0 += 1; }
  }
  return e;
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int mca_decode_qkv_rmsnorm(const float* x, const float* rms_weight, float eps, const void* wq, const void* wk,
                           const void* wv, int weights_bf16, int B, int dim, int kv_dim, float* q_out, float* k_out,
                           float* v_out, void* stream) {
  if (!x || !rms_weight || !wq || !wk || !wv || !q_out || !k_out || !v_out) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || kv_dim <= 0 || dim % 256 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x) || !al16(rms_weight) || !al16(wq) || !al16(wk) || !al16(wv)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.x = x; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 3;
  p.w[0] = wq; p.w[1] = wk; p.w[2] = wv;
  p.out[0] = q_out; p.out[1] = k_out; p.out[2] = v_out;
  p.rows[0] = dim; p.rows[1] = kv_dim; p.rows[2] = kv_dim;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_out_proj(const float* attn, const void* wo, int weights_bf16, int B, int dim, float* x_inout,
                        void* stream) {
  if (!attn || !wo || !x_inout) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || dim % 256 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(attn) || !al16(wo)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.x = attn; p.norm_w = nullptr; p.eps = 0.f; p.n = dim; p.B = B; p.accumulate = 1; p.n_mats = 1;
  p.w[0] = wo; p.w[1] = p.w[2] = nullptr;
  p.out[0] = x_inout; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = dim; p.rows[1] = p.rows[2] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}
