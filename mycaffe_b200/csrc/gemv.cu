// Weight-streaming projections of the llama2 decode attention block, fused with what surrounds them:
//   * RMSNorm + Wq/Wk/Wv:  q,k,v = W · (w_rms ∘ x / sqrt(mean(x²) + eps))
//   * Wo + residual:       x += Wo · attn
//   * RMSNorm + W1/W3 + SwiGLU:  h = silu(W1 · xn) ∘ (W3 · xn)   (llama2_gpu.cpp:84-91, llama2_cpu.cpp:352-368)
//   * W2 + residual:       x += W2 · h                           (llama2_gpu.cpp:94-97)
//   * final RMSNorm + classifier: logits = Wcls · xn             (llama2_gpu.cpp:101-105)
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
// contiguous bytes per warp instruction, and reduce with shuffles.  Every warp owns the same number
// of consecutive rows and requests its first weight vectors before the activations are staged, so
// HBM is busy from the first cycle.  Up to 8 sequences share one pass over the weights (then two
// rows at a time per warp share the activation reads); larger batches take several passes.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int GV_BMAX = 8;   // sequences per pass over the weights

template <typename WT> struct WLoad;
template <> struct WLoad<float> {
  static constexpr int VEC = 4;
  using Raw = float4;
  static __device__ __forceinline__ Raw raw(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ void unpack(const Raw& t, float (&w)[4]) { w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w; }
};
template <> struct WLoad<__nv_bfloat16> {
  static constexpr int VEC = 8;
  using Raw = uint4;
  static __device__ __forceinline__ Raw raw(const __nv_bfloat16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ void unpack(const Raw& t, float (&w)[8]) {
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
  int swiglu;                    // out[0][r] = silu(w[0] row r . x) * (w[1] row r . x); rows[1] == rows[0]
  int rows_per_warp;             // consecutive rows owned by one warp (a multiple of R)
  float eps;
};

// NB sequences per pass, R rows at a time per warp (they share the activation reads from shared
// memory), THREADS per CTA.  A warp owns rows_per_warp consecutive rows of the stacked matrix, so
// that all warps of the grid have the same amount of weight bytes to stream.
// GLU: the two "rows at a time" are row r of w[0] and row r of w[1], combined by SwiGLU (R must be 2).
template <typename WT, int NB, int R, int THREADS, bool GLU>
__global__ void __launch_bounds__(THREADS) gemv_fused_kernel(const GemvParams p, int b0) {
  static_assert(!GLU || R == 2, "the gated form pairs one row of each matrix");
  constexpr int STEP = GLU ? 1 : R;   // output rows finished per iteration
  constexpr int WARPS = THREADS / 32;
  constexpr int VEC = WLoad<WT>::VEC;
  constexpr int PRE = NB <= 2 ? 8 : 2;         // weight vectors per row requested before the activations are staged
  extern __shared__ __align__(16) float xs[];  // [NB][n] normalised activations
  __shared__ float red[WARPS][NB];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = p.n;
  const int total_rows = GLU ? p.rows[0] : p.rows[0] + (p.n_mats > 1 ? p.rows[1] : 0) + (p.n_mats > 2 ? p.rows[2] : 0);
  const int row_lo = (blockIdx.x * WARPS + warp) * p.rows_per_warp;
  const int row_hi = min(row_lo + p.rows_per_warp, total_rows);
  // operand q of the iteration that starts at output row r: which matrix, which of its rows
  auto row_ptr = [&](int r, int q, int& m, int& rr) -> const WT* {
    if (GLU) {
      m = q; rr = min(r, total_rows - 1);
    } else {
      m = 0; rr = min(r + q, total_rows - 1);
      if (rr >= p.rows[0]) { rr -= p.rows[0]; m = 1; if (rr >= p.rows[1]) { rr -= p.rows[1]; m = 2; } }
    }
    const void* base = m == 0 ? p.w[0] : (m == 1 ? p.w[1] : p.w[2]);  // no dynamic indexing of the parameter block
    return reinterpret_cast<const WT*>(base) + (int64_t)rr * n;
  };
  // ---- the first weight vectors of this warp's first rows leave for HBM before anything else
  typename WLoad<WT>::Raw pre[R][PRE];
  {
#pragma unroll
    for (int q = 0; q < R; ++q) {
      int m, rr;
      const WT* wrow = row_ptr(row_lo, q, m, rr);
#pragma unroll
      for (int u = 0; u < PRE; ++u) {
        const int k = (lane + 32 * u) * VEC;
        pre[q][u] = WLoad<WT>::raw(wrow + (k < n ? k : 0));
      }
    }
  }
  // ---- phase 1: activations of this pass's sequences -> shared memory, RMS-normalised
  float ss[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) ss[b] = 0.f;
  for (int k = tid * 4; k < n; k += THREADS * 4) {
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
      for (int w = 0; w < WARPS; ++w) t += red[w][b];
      t = t / (float)n + p.eps;
      scale[b] = 1.0f / sqrtf(t);
    }
    for (int k = tid * 4; k < n; k += THREADS * 4) {
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
  // ---- phase 2: this warp's rows, R at a time
  for (int r = row_lo; r < row_hi; r += STEP) {
    const WT* wrow[R];
    int mat[R], rin[R];
#pragma unroll
    for (int q = 0; q < R; ++q) wrow[q] = row_ptr(r, q, mat[q], rin[q]);
    float acc[R][NB];
#pragma unroll
    for (int q = 0; q < R; ++q)
#pragma unroll
      for (int b = 0; b < NB; ++b) acc[q][b] = 0.f;
    auto fma_vec = [&](const typename WLoad<WT>::Raw& raw, int q, int k) {
      float w[VEC];
      WLoad<WT>::unpack(raw, w);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float* xv = xs + b * n + k;
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
          const float4 t = *reinterpret_cast<const float4*>(xv + i);
          acc[q][b] = fmaf(w[i], t.x, acc[q][b]); acc[q][b] = fmaf(w[i + 1], t.y, acc[q][b]);
          acc[q][b] = fmaf(w[i + 2], t.z, acc[q][b]); acc[q][b] = fmaf(w[i + 3], t.w, acc[q][b]);
        }
      }
    };
    int k_start = lane * VEC;
    if (r == row_lo) {  // the vectors requested before phase 1
#pragma unroll
      for (int u = 0; u < PRE; ++u) {
        const int k = (lane + 32 * u) * VEC;
        if (k < n) {
#pragma unroll
          for (int q = 0; q < R; ++q) fma_vec(pre[q][u], q, k);
        }
      }
      k_start = (lane + 32 * PRE) * VEC;
    }
#pragma unroll(NB <= 2 ? 8 : 2)
    for (int k = k_start; k < n; k += 32 * VEC) {
      typename WLoad<WT>::Raw raw[R];
#pragma unroll
      for (int q = 0; q < R; ++q) raw[q] = WLoad<WT>::raw(wrow[q] + k);
#pragma unroll
      for (int q = 0; q < R; ++q) fma_vec(raw[q], q, k);
    }
#pragma unroll
    for (int q = 0; q < R; ++q)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[q][b] += __shfl_xor_sync(0xffffffffu, acc[q][b], o);
      }
    if (GLU) {
      if (lane == 0) {
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          // val = hb * (1 / (1 + exp(-hb))) * hb2, llama2_cpu.cpp:359-367
          float val = acc[0][b];
          val *= (1.0f / (1.0f + expf(-val)));
          val *= acc[R - 1][b];
          p.out[0][(int64_t)(b0 + b) * p.rows[0] + r] = val;
        }
      }
    } else if (lane == 0) {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        if (r + q >= row_hi) continue;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float* ob = mat[q] == 0 ? p.out[0] : (mat[q] == 1 ? p.out[1] : p.out[2]);
          const int orows = mat[q] == 0 ? p.rows[0] : (mat[q] == 1 ? p.rows[1] : p.rows[2]);
          float* dst = ob + (int64_t)(b0 + b) * orows + rin[q];
          *dst = p.accumulate ? (*dst + acc[q][b]) : acc[q][b];
        }
      }
    }
  }
}

template <typename WT, int NB, int R, int THREADS, bool GLU = false>
int launch_pass(GemvParams p, int b0, cudaStream_t st) {
  constexpr int STEP = GLU ? 1 : R;
  constexpr int WARPS = THREADS / 32;
  const size_t smem = sizeof(float) * (size_t)NB * p.n;
  if (smem > 200 * 1024) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  MCA_CUDA_TRY(cudaFuncSetAttribute(gemv_fused_kernel<WT, NB, R, THREADS, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int total_rows = GLU ? p.rows[0] : p.rows[0] + (p.n_mats > 1 ? p.rows[1] : 0) + (p.n_mats > 2 ? p.rows[2] : 0);
  // as many warps as fit on the 148 SMs at once, every one of them with the same number of rows
  int ctas_per_sm = 1, dev = 0, sms = 148;
  MCA_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, gemv_fused_kernel<WT, NB, R, THREADS, GLU>, THREADS, smem));
  MCA_CUDA_TRY(cudaGetDevice(&dev));
  MCA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int max_warps = sms * std::max(1, ctas_per_sm) * WARPS;
  int rpw = mca_ceil_div(total_rows, max_warps);
  rpw = mca_ceil_div(rpw, STEP) * STEP;
  p.rows_per_warp = rpw;
  const int grid = mca_ceil_div(total_rows, rpw * WARPS);
  gemv_fused_kernel<WT, NB, R, THREADS, GLU><<<grid, THREADS, smem, st>>>(p, b0);
  return mca_launch_status();
}

template <typename WT>
int run_gemv(const GemvParams& p, cudaStream_t st) {
  int e = 0;
  if (p.swiglu) {
    for (int b0 = 0; b0 < p.B && !e;) {
      const int left = p.B - b0;
      if (left >= 8 && (size_t)8 * p.n * 4 <= 200 * 1024) { e = launch_pass<WT, 8, 2, 512, true>(p, b0, st); b0 += 8; }
      else if (left >= 4 && (size_t)4 * p.n * 4 <= 200 * 1024) { e = launch_pass<WT, 4, 2, 512, true>(p, b0, st); b0 += 4; }
      else if (left >= 2) { e = launch_pass<WT, 2, 2, 256, true>(p, b0, st); b0 += 2; }
      else { e = launch_pass<WT, 1, 2, 256, true>(p, b0, st); b0 += 1; }
    }
    return e;
  }
  // two rows at a time need the stacked matrices to start on even rows
  const bool even = (p.rows[0] % 2 == 0) && (p.rows[1] % 2 == 0);
  for (int b0 = 0; b0 < p.B && !e;) {
    const int left = p.B - b0;
    if (left >= 8 && even && (size_t)8 * p.n * 4 <= 200 * 1024) { e = launch_pass<WT, 8, 2, 512>(p, b0, st); b0 += 8; }
    else if (left >= 4 && even && (size_t)4 * p.n * 4 <= 100 * 1024) { e = launch_pass<WT, 4, 2, 512>(p, b0, st); b0 += 4; }
    else if (left >= 4 && (size_t)4 * p.n * 4 <= 200 * 1024) { e = launch_pass<WT, 4, 1, 256>(p, b0, st); b0 += 4; }
    else if (left >= 2) { e = launch_pass<WT, 2, 1, 256>(p, b0, st); b0 += 2; }
    else { e = launch_pass<WT, 1, 1, 256>(p, b0, st); b0 += 1; }
  }
  return e;
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int mca_decode_qkv_rmsnorm(const float* x, const float* rms_weight, float eps, const void* wq, const void* wk,
                           const void* wv, int weights_bf16, int B, int dim, int kv_dim, float* q_out, float* k_out,
                           float* v_out, void* stream) {
  if (!x || !rms_weight || !wq || !wk || !wv || !q_out || !k_out || !v_out) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || kv_dim <= 0 || dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x) || !al16(rms_weight) || !al16(wq) || !al16(wk) || !al16(wv)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.swiglu = 0;
  p.x = x; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 3;
  p.w[0] = wq; p.w[1] = wk; p.w[2] = wv;
  p.out[0] = q_out; p.out[1] = k_out; p.out[2] = v_out;
  p.rows[0] = dim; p.rows[1] = kv_dim; p.rows[2] = kv_dim;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_out_proj(const float* attn, const void* wo, int weights_bf16, int B, int dim, float* x_inout,
                        void* stream) {
  if (!attn || !wo || !x_inout) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(attn) || !al16(wo)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.swiglu = 0;
  p.x = attn; p.norm_w = nullptr; p.eps = 0.f; p.n = dim; p.B = B; p.accumulate = 1; p.n_mats = 1;
  p.w[0] = wo; p.w[1] = p.w[2] = nullptr;
  p.out[0] = x_inout; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = dim; p.rows[1] = p.rows[2] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_ffn(const float* rms_weight, float eps, const void* w1, const void* w2, const void* w3, int weights_bf16,
                   int B, int dim, int hidden_dim, float* hidden_scratch, float* x_inout, void* stream) {
  if (!rms_weight || !w1 || !w2 || !w3 || !hidden_scratch || !x_inout) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || hidden_dim <= 0 || dim % 8 != 0 || hidden_dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x_inout) || !al16(rms_weight) || !al16(w1) || !al16(w2) || !al16(w3) || !al16(hidden_scratch))
    return ERROR_PARAM_OUT_OF_RANGE;
  if ((size_t)hidden_dim * 4 > 200 * 1024 || (size_t)dim * 4 > 200 * 1024) return ERROR_ATTN_UNSUPPORTED_SHAPE;
  GemvParams p;
  // h = silu(W1 xn) * (W3 xn)
  p.swiglu = 1;
  p.x = x_inout; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 2;
  p.w[0] = w1; p.w[1] = w3; p.w[2] = nullptr;
  p.out[0] = hidden_scratch; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = hidden_dim; p.rows[1] = hidden_dim; p.rows[2] = 0;
  int e = weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
  if (e) return e;
  // x += W2 h
  p.swiglu = 0;
  p.x = hidden_scratch; p.norm_w = nullptr; p.eps = 0.f; p.n = hidden_dim; p.accumulate = 1; p.n_mats = 1;
  p.w[0] = w2; p.w[1] = nullptr;
  p.out[0] = x_inout;
  p.rows[0] = dim; p.rows[1] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}

int mca_decode_logits(const float* x, const float* rms_weight, float eps, const void* wcls, int weights_bf16, int B,
                      int dim, int vocab_size, float* logits, void* stream) {
  if (!x || !rms_weight || !wcls || !logits) return ERROR_PARAM_NULL;
  if (B <= 0 || dim <= 0 || vocab_size <= 0 || dim % 8 != 0) return ERROR_PARAM_OUT_OF_RANGE;
  if (!al16(x) || !al16(rms_weight) || !al16(wcls)) return ERROR_PARAM_OUT_OF_RANGE;
  GemvParams p;
  p.swiglu = 0;
  p.x = x; p.norm_w = rms_weight; p.eps = eps; p.n = dim; p.B = B; p.accumulate = 0; p.n_mats = 1;
  p.w[0] = wcls; p.w[1] = p.w[2] = nullptr;
  p.out[0] = logits; p.out[1] = p.out[2] = nullptr;
  p.rows[0] = vocab_size; p.rows[1] = p.rows[2] = 0;
  return weights_bf16 ? run_gemv<__nv_bfloat16>(p, (cudaStream_t)stream) : run_gemv<float>(p, (cudaStream_t)stream);
}
